"""Fused per-world Newton iteration: eligibility, launch geometry and the launch.

Mirrors the interface of the reference's
``src/instantmimic/utils/mjw_kernels/newton_fusion.py``; the kernels themselves
are ``csrc/imn_newton.cu`` behind ``imn_solve``.
"""

from __future__ import annotations

import ctypes as C
from typing import Any

from .. import _lib, abi, binding, types
from ..arrays import is_device

# CTAs per SM requested from the compiler for the reference's Warp kernel
# (newton_fusion.py:27-33).  The CUDA kernel here is one warp per world and is
# limited by shared memory, not registers; the function is kept because callers
# and tests of the reference use it.
_NEWTON_MAX_BLOCKS_PER_SM = 12


def newton_min_blocks_per_sm(nworld: int, sm_count: int) -> int:
    """CTAs per SM worth demanding for a grid of ``nworld`` worlds, 0 for none
    (newton_fusion.py:36-49)."""
    if nworld <= 0 or sm_count <= 0:
        return 0
    return max(1, min(nworld // sm_count, _NEWTON_MAX_BLOCKS_PER_SM))


def _use_incremental(m: Any) -> bool:
    """Upstream ``solver._use_incremental``: the Newton solver keeps H between
    iterations."""
    return int(m.opt.solver) == binding.upstream_constants()["solver_newton"]


def _sparse_compact(ctx: Any) -> bool:
    return bool(getattr(ctx, "sparse_compact", False))


def _on_cuda(m: Any) -> bool:
    ref = getattr(m, "body_parentid", None)
    device = getattr(ref, "device", None)
    if device is not None and hasattr(device, "is_cuda"):
        return bool(device.is_cuda)
    if device is not None and hasattr(device, "type"):
        return device.type == "cuda"
    return ref is not None and is_device(ref)


def eligible(m: Any, ctx: Any, *, compact: bool = False) -> bool:
    """Structural gates of the fused path (newton_fusion.py:307-322)."""
    return bool(
        not compact
        and _on_cuda(m)
        and 0 < m.nv <= 79
        and m.nv_pad % 16 == 0
        and m.nv_pad <= 80
        and _use_incremental(m)
        and int(m.opt.integrator) != binding.upstream_constants()["integrator_discrete"]
        and int(m.opt.cone) == binding.upstream_constants()["cone_pyramidal"]
        and not m.is_sparse
        and not _sparse_compact(ctx)
        and m.opt.iterations > 0
        and m.block_dim.linesearch_iterative == 32
    )


def ineligible_reasons(m: Any, ctx: Any, *, compact: bool = False) -> list[str]:
    """The gates of ``eligible`` that this model fails, in words."""
    checks = [
        (not compact, "compact (sleeping-island) solve"),
        (_on_cuda(m), "model buffers are not on a CUDA device"),
        (0 < m.nv <= 79, f"nv {m.nv} outside 1..79"),
        (m.nv_pad % 16 == 0 and m.nv_pad <= 80, f"nv_pad {m.nv_pad} is not a multiple of 16 up to 80"),
        (_use_incremental(m), "solver is not Newton"),
        (int(m.opt.integrator) != binding.upstream_constants()["integrator_discrete"], "DISCRETE integrator"),
        (int(m.opt.cone) == binding.upstream_constants()["cone_pyramidal"], "elliptic friction cones"),
        (not m.is_sparse, "sparse constraint Jacobian"),
        (not _sparse_compact(ctx), "sparse-compact solver context"),
        (m.opt.iterations > 0, "opt.iterations is 0"),
        (m.block_dim.linesearch_iterative == 32, "line-search block width is not 32"),
    ]
    return [why for ok, why in checks if not ok]


def newton_block_dim(m: Any) -> int:
    """Logical block width of one world (newton_fusion.py:325-327).  It fixes the
    order of the per-thread partial sums; the CUDA kernel reproduces that order
    inside one physical warp."""
    return 64 if m.nv_pad >= 64 else m.block_dim.linesearch_iterative


def attach_scratch(m: Any, d: Any, ctx: Any, device: Any) -> None:
    """``ctx.newton_dof_union``: the dofs the changed rows touch and their count
    (newton_fusion.py:301-304)."""
    import torch

    ctx.newton_dof_union = torch.zeros((d.nworld, m.nv + 1), dtype=torch.int32, device=device)


class SolveCall:
    """The structs of one (Model, Data, context) triple, built once.

    Struct construction walks ~60 attributes; a step pipeline calls the solve every
    substep with the same buffers, so the result is cached on the scratch object
    and only revalidated by address."""

    def __init__(self, m: Any, d: Any, ctx: Any, nsolving: Any):
        self.m = binding.model_struct(m)
        self.d = binding.data_struct(m, d)
        plan = getattr(ctx, "sparse_hessian_plan", None)
        self.plan_struct = getattr(plan, "struct", None) if plan is not None and plan.path == "fused" else None
        self.c = binding.ctx_struct(self.d, ctx, nsolving, self.plan_struct)
        self.key = _key(m, d, ctx, nsolving)

    def launch_info(self) -> abi.ImnLaunchInfo:
        info = abi.ImnLaunchInfo()
        _lib.check(
            _lib.lib().imn_launch_info(C.byref(self.m), C.byref(self.d), C.byref(self.c), C.byref(info)),
            "imn_launch_info",
        )
        return info

    def __call__(self, stream=None) -> None:
        with _lib.nvtx("imn_solve"):
            rc = _lib.lib().imn_solve(
                C.byref(self.m), C.byref(self.d), C.byref(self.c), _lib.current_stream_handle(stream)
            )
        _lib.check(rc, "imn_solve")


_KEY_DATA = ("nefc", "ne", "nf", "qacc_smooth", "qacc_warmstart", "qfrc_smooth", "M", "qacc",
             "qfrc_constraint", "solver_niter", "overflow")
_KEY_EFC = ("J", "D", "aref", "frictionloss", "force", "state", "Ma", "J_world_offset")
_KEY_CTX = ("Jaref", "jv", "search", "mv", "grad", "h", "hfactor", "quad_changed_ids", "newton_dof_union",
            "world_order", "stats") + binding._CTX_WORLD_ARRAYS


def _key(m, d, ctx, nsolving):
    """Everything the cached structs were built from: the address of every buffer the
    kernel is handed and the scalar options.  A caller that rebinds any of them gets
    fresh structs instead of stale pointers."""
    from ..arrays import addr

    plan = getattr(ctx, "sparse_hessian_plan", None)
    return (
        id(m), id(d), id(ctx), id(plan), addr(nsolving),
        tuple(addr(getattr(d, n)) for n in _KEY_DATA),
        tuple(addr(getattr(d.efc, n, None)) for n in _KEY_EFC),
        tuple(addr(getattr(ctx, n, None)) for n in _KEY_CTX),
        addr(m.opt.tolerance), addr(m.opt.ls_tolerance), addr(m.stat.meaninertia),
        int(m.opt.iterations), int(m.opt.ls_iterations), int(m.opt.disableflags),
        int(getattr(m.opt, "warn_overflow", 0) or 0), int(d.nworld), int(d.njmax),
    )


def solve_call(m: Any, d: Any, ctx: Any, nsolving: Any, cache_on: Any = None) -> SolveCall:
    holder = cache_on if cache_on is not None else ctx
    call = getattr(holder, "_imn_solve_call", None)
    if call is None or call.key != _key(m, d, ctx, nsolving):
        call = SolveCall(m, d, ctx, nsolving)
        try:
            holder._imn_solve_call = call
        except AttributeError:
            pass
    return call


def run(m: Any, d: Any, ctx: Any, nsolving: Any, stream=None) -> None:
    """Init, every Newton iteration and the final force of all worlds: one launch
    (reference: init_context + run + qfrc_constraint_from_grad,
    newton_fusion.py:330-409, 431-472, 522-539)."""
    solve_call(m, d, ctx, nsolving)(stream)
