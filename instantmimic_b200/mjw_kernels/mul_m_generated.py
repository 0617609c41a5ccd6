"""``M v`` as generated straight-line code.

The reference calls upstream ``support.mul_m`` (mjw_step_optimized.py:2252-2255), a
kernel that walks the model's ``M_mulm_*`` tables at run time.  For batches that fill
the GPU this module turns those tables into a program for the same generator that
compiles the tree L'DL plans (``imn_mul_m_compile``): lane = world, 32 worlds per block,
the block's tile of M and v staged in shared memory by two bulk copies, every warp
keeps the entries of v its rows need in registers and reads each stored entry of M once.
Nothing is looked up at run time, so a multiply-add costs one shared-memory read instead
of three.  The sums are formed in table order, one fmaf per stored entry starting from
zero, exactly as ``imn_mul_m`` forms them: the results are bit-identical.

Falls back to nothing: callers that do not hold a ``GeneratedMulM`` use ``imn_mul_m``
(NVRTC not installed, a model whose tile does not fit, small batches).
"""

from __future__ import annotations

import ctypes as C
from typing import Any

import numpy as np

from .. import _lib
from ..arrays import addr, elem_strides, to_host
from .tree_ldl import OP_LOAD_M, OP_LOAD_Y, OP_STORE_X, OP_ZERO, GeneratedKernel

OP_MULADD = 11  # dst = fmaf(a, b, dst)
WARPS = 4


def mul_m_program(rowadr, col, madr, nv: int, warps: int = WARPS):
    """(prog, ptr, nslot) of ``out = M v`` for the symmetric-row tables of a model.

    Rows are dealt to the warps by stored entries: a row belongs to the warp its first
    entry falls to when the entry list is cut into ``warps`` near-equal runs.  Streams
    0..warps-1 (before the block barriers) load the needed entries of v, streams
    warps+1..2*warps (after them) compute and store the rows; the trunk stream is empty.
    """
    rowadr = np.asarray(rowadr, dtype=np.int64)
    col = np.asarray(col, dtype=np.int64)
    madr = np.asarray(madr, dtype=np.int64)
    nnz = int(rowadr[nv])
    load: list[list[tuple]] = [[] for _ in range(warps)]
    work: list[list[tuple]] = [[] for _ in range(warps)]
    nslot = 0
    for w in range(warps):
        lo, hi = nnz * w // warps, nnz * (w + 1) // warps
        rows = [i for i in range(nv) if lo <= rowadr[i] < hi and rowadr[i + 1] > rowadr[i]]
        vslot: dict[int, int] = {}
        for i in rows:
            for k in range(int(rowadr[i]), int(rowadr[i + 1])):
                c = int(col[k])
                if c not in vslot:
                    vslot[c] = nslot
                    load[w].append((OP_LOAD_Y, nslot, c, 0, 0))
                    nslot += 1
        for i in rows:
            acc = nslot
            nslot += 1
            work[w].append((OP_ZERO, acc, 0, 0, 0))
            for k in range(int(rowadr[i]), int(rowadr[i + 1])):
                t = nslot
                nslot += 1
                work[w].append((OP_LOAD_M, t, int(madr[k]), 0, 0))
                work[w].append((OP_MULADD, acc, t, vslot[int(col[k])], 0))
            work[w].append((OP_STORE_X, i, acc, 0, 0))
    # rows without a stored entry (cannot happen for a mass matrix) would stay unwritten
    if sum(sum(1 for ins in s if ins[0] == OP_STORE_X) for s in work) != nv:
        raise ValueError("mul_m_program: a row of the symmetric tables is empty")
    if nslot > 1 << 16:
        raise ValueError("mul_m_program: more than 65536 values")
    streams = load + [[]] + work
    words, ptr = [], [0]
    for s in streams:
        for op, dst, a, b, c in s:
            words.append((op, dst, a | (b << 16), c))
        ptr.append(len(words))
    prog = np.asarray(words, dtype=np.int32).reshape(-1, 4)
    return prog, np.asarray(ptr, dtype=np.int32), nslot


class GeneratedMulM(GeneratedKernel):
    """Owner of the compiled ``M v`` kernel of one model."""

    def __init__(self, prog: np.ndarray, ptr: np.ndarray, nv: int, nM: int, nslot: int, warps: int = WARPS):
        prog = np.ascontiguousarray(prog, dtype=np.int32)
        ptr = np.ascontiguousarray(ptr, dtype=np.int32)
        handle = C.c_void_p()
        rc = _lib.lib().imn_mul_m_compile(prog.ctypes.data, ptr.ctypes.data, nv, nM, warps, nslot, C.byref(handle))
        _lib.check(rc, "imn_mul_m_compile")
        self.handle = handle
        self.nv, self.nM = nv, nM
        self.staged = "tileM" in self.info()["source"]


def compile_mul_m(m: Any) -> GeneratedMulM | None:
    """The generated kernel of a model, or None when it would not beat ``imn_mul_m``: NVRTC
    is not installed, or the 32-world tile is not staged in shared memory (too large, or a
    lane stride nM that piles the lanes onto a few banks)."""
    nv, nM = int(m.nv), int(m.M_colind.shape[0])
    prog, ptr, nslot = mul_m_program(to_host(m.M_mulm_rowadr), to_host(m.M_mulm_col), to_host(m.M_mulm_madr), nv)
    try:
        kernel = GeneratedMulM(prog, ptr, nv, nM, nslot)
    except _lib.ImnError as err:
        if "NVRTC" in str(err) and "could not be loaded" in str(err):
            return None
        raise
    return kernel if kernel.staged else None


def mul_m(kernel: GeneratedMulM, M: Any, res: Any, vec: Any, stream=None) -> None:
    """res = M vec per world through the generated kernel (res must not alias vec)."""
    for array in (M, res, vec):
        if elem_strides(array)[1] != 1:
            raise ValueError("mul_m needs rows of contiguous floats")
    if addr(res) == addr(vec):
        raise ValueError("mul_m: res must not alias vec")
    rc = _lib.lib().imn_tree_ldl_compiled_solve(
        kernel.handle, addr(M), elem_strides(M)[0], addr(vec), elem_strides(vec)[0], addr(res),
        elem_strides(res)[0], int(M.shape[0]), _lib.current_stream_handle(stream),
    )
    _lib.check(rc, "imn_tree_ldl_compiled_solve")
