"""ctypes front end of the CPU oracle (``oracle/liboracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke`` and
by the CPU-baseline / reference legs of ``bench.py``.  The product package never
imports it.  Entry points take the same structs as the CUDA library, filled with
host addresses.
"""

from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path
from typing import Any

from instantmimic_b200 import abi, binding

_HERE = Path(__file__).resolve().parent
_LIB: C.CDLL | None = None


def build(force: bool = False) -> Path:
    """Compile the oracle with its Makefile; returns the library path."""
    lib = _HERE / "liboracle.so"
    srcs = list(_HERE.glob("*.c")) + list(_HERE.glob("*.h")) + [_HERE.parent / "include" / "imnewton.h"]
    stale = not lib.exists() or any(s.stat().st_mtime > lib.stat().st_mtime for s in srcs)
    if force or stale:
        env = dict(os.environ)
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True, env=env,
                       stdout=subprocess.DEVNULL)
    return lib


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = build()
        L = C.CDLL(str(path))
        MP, DP, CP = C.POINTER(abi.ImnModel), C.POINTER(abi.ImnData), C.POINTER(abi.ImnCtx)
        L.oracle_solve.restype = C.c_int
        L.oracle_solve.argtypes = [MP, DP, CP, C.c_int]
        L.oracle_rowless_handoff.restype = C.c_int
        L.oracle_rowless_handoff.argtypes = [MP, DP]
        L.oracle_mul_m.restype = C.c_int
        L.oracle_mul_m.argtypes = [MP, abi.P, abi.I64, abi.P, abi.I64, abi.P, abi.I64, C.c_int]
        _LIB = L
    return _LIB


def solve(m: Any, d: Any, ctx: Any = None, nsolving: Any = None, threads: int = 0,
          sparse_plan_struct=None) -> None:
    """Newton solve of every world of host containers ``m``, ``d`` (in place)."""
    ms = binding.model_struct(m)
    ds = binding.data_struct(m, d)
    cs = binding.ctx_struct(ds, ctx, nsolving, sparse_plan_struct)
    rc = lib().oracle_solve(C.byref(ms), C.byref(ds), C.byref(cs), int(threads))
    if rc != 0:
        raise RuntimeError(f"oracle_solve failed: {rc}")


def rowless_handoff(m: Any, d: Any) -> None:
    ms = binding.model_struct(m)
    ds = binding.data_struct(m, d)
    lib().oracle_rowless_handoff(C.byref(ms), C.byref(ds))


def mul_m(m: Any, M, v, out) -> None:
    ms = binding.model_struct(m)
    lib().oracle_mul_m(C.byref(ms), M.ctypes.data, M.strides[0] // 4, v.ctypes.data,
                       v.strides[0] // 4, out.ctypes.data, out.strides[0] // 4, M.shape[0])
