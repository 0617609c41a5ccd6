"""Loads ``libimnewton.so``.  There is no fallback: if the library is missing or
lacks a symbol the import of the caller fails with the reason."""

from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import abi

_PATH = Path(__file__).resolve().parent / "libimnewton.so"
_LIB: C.CDLL | None = None


class ImnError(RuntimeError):
    """A C-ABI call returned a negative status."""


def path() -> Path:
    return _PATH


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        if not _PATH.exists():
            raise ImnError(
                f"{_PATH} is not built; run `python -m instantmimic_b200.build` "
                "(nvcc, sm_100a).  This package has no CPU or PyTorch fallback."
            )
        L = abi.bind(C.CDLL(str(_PATH)))
        if L.imn_abi_version() != abi.IMN_ABI_VERSION:
            raise ImnError("libimnewton.so was built from a different imnewton.h")
        _LIB = L
    return _LIB


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().imn_last_error().decode(errors="replace")
        raise ImnError(f"{what} failed ({rc}): {msg}")


def current_stream_handle(stream=None) -> int:
    """cudaStream_t of ``stream`` (torch stream, int, or None = torch's current)."""
    if stream is None:
        import torch

        return int(torch.cuda.current_stream().cuda_stream)
    if isinstance(stream, int):
        return stream
    return int(stream.cuda_stream)


_NVTX = None


def nvtx(name: str):
    """NVTX range around a C-ABI call when profiling is asked for (environment variable
    ``IMN_NVTX=1``); otherwise a no-op context.  The reference wraps the same stages in
    upstream's ``event_scope`` and names its kernels for profilers
    (src/instantmimic/utils/mjw_step_optimized.py:2683, utils/warp_kernels.py:11-14)."""
    global _NVTX
    if _NVTX is None:
        import contextlib
        import os

        if os.environ.get("IMN_NVTX", "0") not in ("", "0"):
            import torch

            _NVTX = torch.cuda.nvtx.range
        else:
            _NVTX = lambda name: contextlib.nullcontext()  # noqa: E731
    return _NVTX(name)
