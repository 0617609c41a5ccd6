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


def implicit_matrix(m: Any, d: Any, velocity_gain=None):
    """A = M - h qDeriv of host containers; returns (nworld, nM)."""
    import numpy as np

    ps = binding.implicit_struct(m, d, velocity_gain)
    out = np.zeros((d.nworld, m.M_colind.shape[0]), np.float32)
    fn = lib().oracle_implicit_matrix
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(abi.ImnImplicit), abi.P, abi.I64, abi.P, abi.I64, C.c_int]
    fn(C.byref(ps), d.M.ctypes.data, d.M.strides[0] // 4, out.ctypes.data, out.shape[1], d.nworld)
    return out


def advance(m: Any, d: Any, qacc) -> None:
    """qvel, qpos, time of host Data advanced in place."""
    ps = binding.advance_struct(m, d)
    fn = lib().oracle_advance
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(abi.ImnAdvance), abi.P, abi.I64, C.c_int]
    fn(C.byref(ps), qacc.ctypes.data, qacc.strides[0] // 4, d.nworld)


def ball_limit_rows(tables: dict, njoint: int, m: Any, d: Any, overflow, singular) -> None:
    """Append the directional ball-limit rows to host ``Data`` in place."""
    from instantmimic_b200.mjw_kernels import ball_limits

    ps = ball_limits.rows_struct(tables, njoint, m, d, overflow, singular)
    fn = lib().oracle_ball_limit_rows
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(abi.ImnBallLimits), C.c_int]
    fn(C.byref(ps), d.nworld)


def _tree_call(name: str, argtypes):
    fn = getattr(lib(), name)
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(abi.ImnBodyTree)] + argtypes
    return fn


def body_tree_accumulate(m: Any, scratch: Any, values, components: int, skip_root_parent: bool) -> None:
    """values[:, parent] += values[:, body] in depth order, in place; values (W, nbody, C) host."""
    from instantmimic_b200.arrays import addr, shape
    from instantmimic_b200.mjw_kernels import tree_fusion

    t = tree_fusion.tree_struct(m, scratch)
    fn = _tree_call("oracle_body_tree_accumulate", [abi.P, abi.I64, C.c_int, C.c_int, C.c_int])
    dims = shape(values)
    fn(C.byref(t), addr(values), dims[1] * int(components), int(components), int(bool(skip_root_parent)), dims[0])


def crb(m: Any, d: Any, scratch: Any) -> None:
    """d.crb and d.M of host containers."""
    from instantmimic_b200.arrays import addr, elem_strides
    from instantmimic_b200.mjw_kernels import tree_fusion

    t = tree_fusion.tree_struct(m, scratch, dofs=True, inertia=True)
    fn = _tree_call("oracle_crb", [abi.P, abi.P, abi.P, abi.P, abi.I64, C.c_int])
    fn(C.byref(t), addr(d.cinert), addr(d.cdof), addr(d.crb), addr(d.M), elem_strides(d.M)[0], d.nworld)


def rne(m: Any, d: Any, scratch: Any) -> None:
    """d.cacc, d.cfrc_int, d.qfrc_bias of host containers."""
    from instantmimic_b200.arrays import addr, elem_strides
    from instantmimic_b200.mjw_kernels import tree_fusion

    t = tree_fusion.tree_struct(m, scratch, dofs=True, gravity=True)
    fn = _tree_call("oracle_rne", [abi.P] * 5 + [abi.I64, abi.P, abi.P, abi.P, abi.I64, C.c_int])
    fn(C.byref(t), addr(d.cinert), addr(d.cvel), addr(d.cdof), addr(d.cdof_dot), addr(d.qvel), elem_strides(d.qvel)[0],
       addr(d.cacc), addr(d.cfrc_int), addr(d.qfrc_bias), elem_strides(d.qfrc_bias)[0], d.nworld)


def com_vel(m: Any, d: Any, scratch: Any) -> None:
    """d.cvel and d.cdof_dot of host containers."""
    from instantmimic_b200.arrays import addr, elem_strides
    from instantmimic_b200.mjw_kernels import tree_fusion

    t = tree_fusion.tree_struct(m, scratch, dofs=True, joints=True)
    fn = _tree_call("oracle_com_vel", [abi.P, abi.I64, abi.P, abi.P, abi.P, C.c_int])
    fn(C.byref(t), addr(d.qvel), elem_strides(d.qvel)[0], addr(d.cdof), addr(d.cvel), addr(d.cdof_dot), d.nworld)


def sparse_stage(plan_struct, stage: int, x: dict, grad, U, nv: int):
    """One stage of the fused sparse path on host arrays (oracle_sparse_stage): 3 initial
    assembly + factor + solve, 0 update with flipped rows + refactor + solve, 1 solve with
    the factor stored in U.  ``x`` holds J, D, state, nefc, M, ids, count, uni; U is
    updated in place.  Returns (search, search_dot, decrement)."""
    import numpy as np

    W = U.shape[0]
    search = np.zeros((W, nv), np.float32)
    sd, dec = np.zeros(W, np.float32), np.zeros(W, np.float32)
    fn = lib().oracle_sparse_stage
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(abi.ImnSparsePlan), C.c_int, abi.P, C.c_int, abi.P, abi.P, abi.P, abi.P, C.c_int, abi.P,
                   abi.P, abi.P, abi.P, abi.I64, abi.P, abi.P, abi.P, abi.P, C.c_int]
    c = lambda a: np.ascontiguousarray(a).ctypes.data  # noqa: E731
    keep = {k: np.ascontiguousarray(v) for k, v in x.items()}
    grad = np.ascontiguousarray(grad, np.float32)
    fn(C.byref(plan_struct), int(stage), c(keep["J"]), keep["J"].shape[1], c(keep["D"]), c(keep["state"]),
       c(keep["nefc"]), c(keep["M"]), keep["M"].shape[1], c(keep["ids"]), c(keep["count"]), c(keep["uni"]),
       grad.ctypes.data, grad.shape[1], U.ctypes.data, search.ctypes.data, sd.ctypes.data, dec.ctypes.data, W)
    return search, sd, dec


def sparse_factor_nonfused(plan_struct, grad, h, U, nv: int, quad_changed=None, skip_unchanged: bool = False):
    """The non-fused factor / solve on host arrays; U updated in place."""
    import numpy as np

    W = U.shape[0]
    search = np.zeros((W, nv), np.float32)
    sd, dec = np.zeros(W, np.float32), np.zeros(W, np.float32)
    grad, h = np.ascontiguousarray(grad, np.float32), np.ascontiguousarray(h, np.float32)
    qc = None if quad_changed is None else np.ascontiguousarray(quad_changed, np.int32)
    fn = lib().oracle_sparse_factor_nonfused
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(abi.ImnSparsePlan)] + [abi.P] * 2 + [abi.I64] + [abi.P] * 5 + [abi.I64, abi.P, abi.P,
                                                                                          C.c_int, C.c_int, C.c_int]
    fn(C.byref(plan_struct), None, grad.ctypes.data, grad.shape[1], h.ctypes.data,
       None if qc is None else qc.ctypes.data, None, U.ctypes.data, search.ctypes.data, nv, sd.ctypes.data,
       dec.ctypes.data, W, int(bool(skip_unchanged)), 0)
    return search, sd, dec


def _i32(a):
    import numpy as np

    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


def tree_ldl_solve(structure, plan, M, y):
    """x = M^-1 y by the serial form of the tree L'DL plan; M (W, nM), y (W, nv) host."""
    import numpy as np

    rowadr, rownnz, colind = (_i32(a) for a in structure)
    nodes = _i32([k for g in plan.groups for k in g])
    ptr = _i32(np.cumsum([0] + [len(g) for g in plan.groups]))
    trunk = _i32(plan.trunk)
    M = np.ascontiguousarray(M, np.float32)
    y = np.ascontiguousarray(y, np.float32)
    x = np.zeros_like(y)
    fn = lib().oracle_tree_ldl_solve
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.c_int, abi.P, abi.P, abi.P, C.c_int, abi.P, abi.P, C.c_int, abi.P,
                   abi.P, abi.I64, abi.P, abi.I64, abi.P, abi.I64, C.c_int]
    fn(rowadr.size, colind.size, rowadr.ctypes.data, rownnz.ctypes.data, colind.ctypes.data,
       len(plan.groups), ptr.ctypes.data, nodes.ctypes.data, trunk.size, trunk.ctypes.data,
       M.ctypes.data, M.shape[1], y.ctypes.data, y.shape[1], x.ctypes.data, x.shape[1], M.shape[0])
    return x


def blocked_dense_factor_solve(nv, pad, indices, identity, M, y, U=None, active=None, mode=0):
    """Blocked dense Cholesky factor + solve; y (W, nv, rhs).  Returns (x, U)."""
    import numpy as np

    y = np.ascontiguousarray(y, np.float32)
    W, _, rhs = y.shape
    indices, identity = _i32(indices), np.ascontiguousarray(identity, np.float32)
    U = np.zeros((W, pad, pad), np.float32) if U is None else np.ascontiguousarray(U, np.float32)
    x = np.zeros_like(y)
    fn = lib().oracle_blocked_dense_factor_solve
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.c_int, C.c_int, abi.P, abi.P, abi.P, abi.I64, abi.P, abi.P, abi.P, abi.P,
                   C.c_int, C.c_int, C.c_int]
    Mp, nM, ld = (None, 0, 0)
    if M is not None:
        M = np.ascontiguousarray(M, np.float32)
        Mp, nM, ld = M.ctypes.data, M.shape[1], M.shape[1]
    act = _i32(active) if active is not None else None
    fn(nv, pad, nM, indices.ctypes.data, identity.ctypes.data, Mp, ld, y.ctypes.data, U.ctypes.data,
       x.ctypes.data, act.ctypes.data if act is not None else None, W, rhs, mode)
    return x, U
