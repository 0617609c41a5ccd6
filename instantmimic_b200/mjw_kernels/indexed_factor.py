"""Blocked dense Cholesky of M with direct inertia indexing.

Host side of the reference's
``src/instantmimic/utils/mjw_kernels/indexed_factor.py`` (kernels :176-214,
:217-391, :394-493) and of the scratch that feeds it,
``create_blocked_dense_factor_solve_scratch`` / ``_blocked_dense_factor_solve``
(src/instantmimic/utils/mjw_step_optimized.py:893-993).  The kernels are
``blocked_dense_kernel`` in ``csrc/imn_msolve.cu`` behind
``imn_blocked_dense_factor_solve``.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any

import numpy as np

from .. import _lib, abi
from ..arrays import addr, elem_strides, is_contiguous, to_host

# Small blocked tiles avoid the long dependency chain of a full-matrix tile
# (mjw_step_optimized.py:868-872).
BLOCK_SIZE = 16
BLOCK_DIM = 64
MIN_NV = 32


@dataclass
class BlockedDenseFactorSolveScratch:
    nv: int
    pad: int
    block_size: int
    block_dim: int
    U: Any  # (nworld, pad, pad) factor workspace
    indices: Any  # (pad * pad,) block-major gather table; nM addresses the zero slot
    identity: Any  # (256,) ones on the padded diagonal of the last block
    struct: abi.ImnBlockedPlan


def _round_up(value: int, multiple: int) -> int:
    return ((value + multiple - 1) // multiple) * multiple


def dense_index_table(m: Any) -> np.ndarray:
    """(nv, nv) table of M's CSR entry for every dense position (nM where the
    matrix is structurally zero): upstream's ``M_tiles[0].elemid`` for a model whose
    inertia matrix is one dense tile."""
    rowadr, rownnz, colind = (to_host(getattr(m, n)) for n in ("M_rowadr", "M_rownnz", "M_colind"))
    nv, nM = int(m.nv), int(colind.shape[0])
    table = np.full((nv, nv), nM, np.int32)
    for k in range(nv):
        for q in range(int(rownnz[k])):
            e = int(rowadr[k]) + q
            c = int(colind[e])
            table[k, c] = table[c, k] = e
    return table


def block_major_layout(table: np.ndarray, pad: int, zero_index: int) -> np.ndarray:
    """Pad the (nv, nv) index table with ``zero_index`` and reorder it as
    (nblk, nblk, 16, 16) blocks (mjw_step_optimized.py:932-941)."""
    nv = table.shape[0]
    nblk = pad // BLOCK_SIZE
    padded = np.full((pad, pad), zero_index, np.int32)
    padded[:nv, :nv] = table
    return padded.reshape(nblk, BLOCK_SIZE, nblk, BLOCK_SIZE).transpose(0, 2, 1, 3).copy().reshape(-1)


def pad_identity(nv: int, pad: int) -> np.ndarray:
    nblk = pad // BLOCK_SIZE
    ident = np.zeros((BLOCK_SIZE, BLOCK_SIZE), np.float32)
    for i in range(BLOCK_SIZE):
        if (nblk - 1) * BLOCK_SIZE + i >= nv:
            ident[i, i] = 1.0
    return ident.reshape(-1)


def create_blocked_dense_factor_solve_scratch(
    m: Any, d: Any, device: Any = "cuda", *, minimum_nv: int = MIN_NV
) -> BlockedDenseFactorSolveScratch | None:
    """Blocked factor+solve buffers when the model qualifies, else ``None``: small
    models use the single-tile path, and models without M have nothing to factor."""
    import torch

    nv = getattr(m, "nv", 0)
    if not isinstance(nv, int) or nv < minimum_nv:
        return None
    nworld = getattr(d, "nworld", 0)
    if not isinstance(nworld, int) or nworld <= 0 or getattr(d, "M", None) is None:
        return None
    pad = _round_up(nv, BLOCK_SIZE)
    nM = int(d.M.shape[1])
    layout = block_major_layout(dense_index_table(m), pad, nM)
    indices = torch.from_numpy(layout).to(device)
    identity = torch.from_numpy(pad_identity(nv, pad)).to(device)
    U = torch.zeros((nworld, pad, pad), dtype=torch.float32, device=device)
    st = abi.ImnBlockedPlan()
    st.nv, st.pad, st.nM = nv, pad, nM
    st.indices, st.identity = addr(indices), addr(identity)
    return BlockedDenseFactorSolveScratch(
        nv=nv, pad=pad, block_size=BLOCK_SIZE, block_dim=BLOCK_DIM, U=U, indices=indices,
        identity=identity, struct=st,
    )


def _launch(scratch, M, y, U, x, active, nworld, rhs_count, mode, stream):
    for name, a in (("y", y), ("x", x), ("U", U)):
        if not is_contiguous(a):
            raise ValueError(f"blocked dense factor/solve needs a contiguous {name}")
    with _lib.nvtx("imn_blocked_dense_factor_solve"):
        rc = _launch_call(scratch, M, y, U, x, active, nworld, rhs_count, mode, stream)
    _lib.check(rc, "imn_blocked_dense_factor_solve")


def _launch_call(scratch, M, y, U, x, active, nworld, rhs_count, mode, stream):
    return _lib.lib().imn_blocked_dense_factor_solve(
        C.byref(scratch.struct),
        addr(M) if M is not None else None,
        elem_strides(M)[0] if M is not None else 0,
        addr(y), addr(U), addr(x), addr(active), int(nworld), int(rhs_count), int(mode),
        _lib.current_stream_handle(stream),
    )


def blocked_dense_factor_solve(
    d: Any, M: Any, x: Any, y: Any, scratch: BlockedDenseFactorSolveScratch, *,
    factor_workspace: Any = None, stream=None,
) -> None:
    """x = M^-1 y; the upper factor stays in ``scratch.U`` (or ``factor_workspace``)
    (mjw_step_optimized.py:958-993, kernel indexed_factor.py:176-214)."""
    U = scratch.U if factor_workspace is None else factor_workspace
    _launch(scratch, M, y, U, x, None, d.nworld, 1, 0, stream)


def factor_multi_solve(scratch, M, y, active, U, x, rhs_count: int, stream=None) -> None:
    """Factor and solve ``rhs_count`` right-hand sides; worlds whose ``active`` flag
    is 0 are left untouched (indexed_factor.py:217-391).  y, x: (nworld, nv, rhs)."""
    _launch(scratch, M, y, U, x, active, y.shape[0], rhs_count, 0, stream)


def multi_solve(scratch, U, y, active, x, rhs_count: int, stream=None) -> None:
    """Solve with an already computed upper factor (indexed_factor.py:394-493)."""
    _launch(scratch, None, y, U, x, active, y.shape[0], rhs_count, 1, stream)
