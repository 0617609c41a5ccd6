"""Step-pipeline entry points of the Newton solve and the M-side factor/solve.

Same names, arguments and error behaviour as the functions of the reference's
``src/instantmimic/utils/mjw_step_optimized.py`` that sit on the solver path:
``solve_with_scratch`` (:2683-2742), ``make_optimized_fwd_position_scratch``
(solver part, :2510-2585), ``_factor_solve_i_dense`` (:1030-1070).  Everything is
a launch of hand-written CUDA through the C ABI; there is no other code path.
"""

from __future__ import annotations

import ctypes as C
import functools
import logging
from dataclasses import dataclass
from typing import Any, Sequence

import numpy as np

from . import _lib, binding
from .arrays import to_host
from .mjw_kernels import newton_fusion

logger = logging.getLogger(__name__)


class SolverContext:
    """The arrays of upstream ``solver._create_solver_context`` that the fused path
    can report (call site mjw_step_optimized.py:2517).  The kernel keeps its
    working set on chip; these buffers receive the final values per world."""

    def __init__(self, m: Any, d: Any, device: Any, *, with_matrices: bool = False, with_stats: bool = False):
        import torch

        W, nv, R, P = d.nworld, m.nv, d.njmax, m.nv_pad
        f = lambda *s: torch.zeros(s, dtype=torch.float32, device=device)  # noqa: E731
        i = lambda *s: torch.zeros(s, dtype=torch.int32, device=device)  # noqa: E731
        b = lambda *s: torch.zeros(s, dtype=torch.uint8, device=device)  # noqa: E731
        self.Jaref, self.jv = f(W, R), f(W, R)
        self.search, self.mv = f(W, nv), f(W, nv)
        self.grad = f(W, P)
        self.h = f(W, P, P) if with_matrices else None
        self.hfactor = f(W, P, P) if with_matrices else None
        self.search_dot, self.grad_dot, self.grad_scale = f(W), f(W), f(W)
        self.newton_decrement, self.improvement, self.alpha = f(W), f(W), f(W)
        self.done, self.search_unchanged, self.ls_exhausted = b(W), b(W), b(W)
        self.quad_changed_ids = i(W, R)
        self.quad_changed_count, self.state_changed_count = i(W), i(W)
        self.sparse_hessian_plan = None
        # scratch of the fused kernel: worlds ordered by row count (no counterpart upstream)
        self.world_order = i(W)
        # work counters of each world's solve (passes, flips, factorisations, gradients);
        # counting costs the kernel ~9 %, so the array exists only on request
        self.stats = i(W, 4) if with_stats else None


@dataclass
class OptimizedFwdPositionScratch:
    """Solver-facing part of the reference's scratch object
    (mjw_step_optimized.py:459-519)."""

    solver_context: Any = None
    solver_nsolving: Any = None
    solver_uses_compact: bool = False
    constraint_free: bool = False
    mul_m_call: Any = None
    dense_factor_solve: Any = None
    tree_factor_solve: Any = None
    unroll_solver_iterations: bool = False
    # single-tile factor/solve of M for models below the blocked kernel's dof count
    # that have no tree plan (the reference's per-tile kernels, :672-750, 793-838)
    tile_factor_solve: Any = None
    # implicit-fast integrator buffers (mjw_step_optimized.py:470-480): M - h qDeriv in
    # M's layout, the solved acceleration, the actuators' velocity gains
    implicit_qderiv: Any = None
    implicit_qacc: Any = None
    implicit_actuator_vel: Any = None
    implicit_gain_coefficients: Any = None  # (g2, b2) per actuator, prepared at set-up
    advance_call: Any = None
    pre_advance_modifier: Any = None
    # directional ball-joint limit rows (mjw_step_optimized.py:2241-2249)
    ball_limit_buffers: Any = None
    # level tables of the body tree for subtree_com / crb / rne / com_vel
    # (mjw_step_optimized.py:518, 2575-2577)
    tree_reduction: Any = None


def _constraint_rows_impossible(m: Any, ball_joint_limits: Sequence[Any] = ()) -> bool:
    """True when the constraint producer can never emit a row for this model, so that
    MuJoCo's ``nefc == 0`` result holds on every step (mjw_step_optimized.py:116-147).

    Rows can come from equalities, friction loss (dofs, tendons), joint and tendon
    limits, contacts of any candidate geom pair, flexes, collision sensors and the
    caller's ball-joint limit rows.  The answer is True only when the model states the
    absence of each of them; a model that lacks one of the fields (this package's
    stand-in ``Model`` carries none) keeps the general path."""
    opt = getattr(m, "opt", None)
    if opt is None or not getattr(opt, "run_collision_detection", False):
        return False
    if ball_joint_limits or _solver_compact_enabled(m):
        return False
    for count in ("neq", "nflex", "nsensorcollision"):
        if int(getattr(m, count, 1)):
            return False
    for name in ("jnt_limited_slide_hinge_adr", "jnt_limited_ball_adr", "tendon_limited_adr"):
        rows = getattr(m, name, None)
        if rows is None or int(np.size(to_host(rows))):
            return False
    for name in ("dof_frictionloss", "tendon_frictionloss"):
        loss = getattr(m, name, None)
        if loss is None:
            return False
        loss = to_host(loss)
        if loss.size and bool((loss > 0.0).any()):
            return False
    pairs = getattr(m, "nxn_pairid_filtered", None)
    if pairs is None:
        return False
    # a pair id of -2 in the first column marks a geom pair that is filtered out
    return not bool((to_host(pairs).reshape(-1, 2)[:, 0] > -2).any())


def optimized_kernel_capabilities(m: Any, scratch: "OptimizedFwdPositionScratch", *, enabled: bool = True) -> dict:
    """Which kernel variants this model gets, without changing any state
    (mjw_step_optimized.py:2862-2875), extended by the choices this library makes
    below the reference's granularity."""
    ctx = getattr(scratch, "solver_context", None)
    fused = bool(enabled and ctx is not None and newton_fusion.eligible(m, ctx, compact=scratch.solver_uses_compact))
    plan = getattr(ctx, "sparse_hessian_plan", None) if ctx is not None else None
    tree = getattr(scratch, "tree_factor_solve", None)
    return {
        "tree": bool(enabled and getattr(scratch, "tree_reduction", None) is not None),
        "indexed_factor": bool(enabled and getattr(scratch, "dense_factor_solve", None) is not None),
        "persistent_newton": fused,
        "constraint_free": bool(getattr(scratch, "constraint_free", False)),
        "hessian_factor": (f"sparse pattern ({plan.path})" if plan is not None else "dense blocked Cholesky") if fused else None,
        "m_factor_solve": (
            f"tree L'DL, {tree.groups} group(s), {'generated' if tree.kernel is not None else 'interpreted'} kernel"
            if tree is not None
            else "blocked dense Cholesky" if scratch.dense_factor_solve is not None
            else "single-tile dense Cholesky" if scratch.tile_factor_solve is not None else None
        ),
    }


def log_kernel_selection(m: Any, d: Any, scratch: "OptimizedFwdPositionScratch") -> str:
    """One INFO line per model naming the kernel variants chosen (the counterpart of
    the reference's MJW_KERNEL_PATH / MJW_SPARSE_HESSIAN records,
    src/instantmimic/envs/direct_rl_env.py:873-884, 2909-2925)."""
    caps = optimized_kernel_capabilities(m, scratch)
    parts = [f"nv {int(m.nv)}", f"njmax {int(d.njmax)}", f"nworld {int(d.nworld)}"]
    if caps["constraint_free"] or d.njmax == 0:
        parts.append("solve: rowless hand-off (no constraint rows possible)")
    elif caps["persistent_newton"]:
        info = newton_fusion.solve_call(m, d, scratch.solver_context, scratch.solver_nsolving,
                                        cache_on=scratch).launch_info()
        parts.append(
            f"solve: fused Newton kernel, J {'resident in shared memory' if info.j_resident else 'streamed in 32-row tiles'}, "
            f"{info.smem_bytes} B shared memory per world, {caps['hessian_factor']}")
    else:
        parts.append("solve: outside the fused path")
    parts.append(f"M factor/solve: {caps['m_factor_solve']}")
    parts.append("M v: " + ("generated kernel" if isinstance(getattr(scratch, "mul_m_call", None), functools.partial) else "table kernels"))
    parts.append("body-tree stages: " + ("fused" if caps["tree"] else "none"))
    line = "IMN_KERNEL_PATH " + "; ".join(parts)
    logger.info(line)
    return line


# Below this many worlds the tiles of the generated M v do not fill the GPU.
_GENERATED_MUL_M_MIN_WORLDS = 4096


def generated_mul_m_kernel(m: Any, d: Any):
    """The model's generated M v kernel (compiled once per model, kept on it), or None."""
    if int(d.nworld) < _GENERATED_MUL_M_MIN_WORLDS or getattr(m, "M_mulm_rowadr", None) is None:
        return None
    cached = getattr(m, "_imn_mul_m_kernel", "unset")
    if cached != "unset":
        return cached
    from .mjw_kernels import mul_m_generated

    kernel = mul_m_generated.compile_mul_m(m)
    try:
        m._imn_mul_m_kernel = kernel
    except AttributeError:
        pass
    return kernel


def mul_m(m: Any, d: Any, res: Any, vec: Any, stream=None, kernel: Any = None) -> None:
    """res = M vec per world (upstream ``support.mul_m`` through the preallocated
    call, mjw_step_optimized.py:2252-2255).  With ``kernel`` (the model's generated
    straight-line kernel, ``mul_m_generated.compile_mul_m``) batches that fill the GPU run
    through it; the bits are the same."""
    from .arrays import addr, elem_strides

    if kernel is not None and int(d.nworld) >= _GENERATED_MUL_M_MIN_WORLDS and addr(res) != addr(vec):
        from .mjw_kernels import mul_m_generated

        with _lib.nvtx("mul_m_generated"):
            mul_m_generated.mul_m(kernel, d.M, res, vec, stream)
        return
    ms = binding.model_struct(m)
    rc = _lib.lib().imn_mul_m(
        C.byref(ms), addr(d.M), elem_strides(d.M)[0], addr(vec), elem_strides(vec)[0], addr(res),
        elem_strides(res)[0], int(d.nworld), _lib.current_stream_handle(stream),
    )
    _lib.check(rc, "imn_mul_m")


def make_optimized_fwd_position_scratch(
    m: Any,
    d: Any,
    device: Any = "cuda",
    *,
    include_optimized_kernel_scratch: bool = True,
    with_matrices: bool = False,
    with_stats: bool = False,
    ball_joint_limits: Sequence[Any] = (),
) -> OptimizedFwdPositionScratch:
    """Solver context, nsolving counter, the M-side factor/solve plans and the
    ``constraint_free`` decision (mjw_step_optimized.py:2237-2255, 2510-2585)."""
    import torch

    from .mjw_kernels import indexed_factor, tree_ldl

    ctx = nsolving = None
    if d.njmax > 0 and m.nv > 0:
        ctx = SolverContext(m, d, device, with_matrices=with_matrices, with_stats=with_stats)
        newton_fusion.attach_scratch(m, d, ctx, device)
        nsolving = torch.zeros((1,), dtype=torch.int32, device=device)
    dense = indexed_factor.create_blocked_dense_factor_solve_scratch(m, d, device)
    tree = tree_ldl.create_tree_factor_solve_scratch(m, device) if include_optimized_kernel_scratch else None
    tile = None
    if dense is None and m.nv > 0 and getattr(d, "M", None) is not None:
        # below the blocked kernel's dof count the reference factors M tile by tile; the
        # same kernel does it here with one 16- or 32-wide tile per world
        tile = indexed_factor.create_blocked_dense_factor_solve_scratch(m, d, device, minimum_nv=1)
    ball_buffers = None
    if ball_joint_limits and all(hasattr(d.efc, n) for n in ("pos", "margin", "vel", "type", "id")):
        from .mjw_kernels import ball_limits

        ball_buffers = ball_limits.make_ball_limit_buffers(ball_joint_limits, m, d, device)
    tree_reduction = None
    if include_optimized_kernel_scratch and getattr(m, "body_tree", None):
        from .mjw_kernels import tree_fusion

        tree_reduction = tree_fusion.create_tree_reduction_scratch(m)
    mul_m_kernel = generated_mul_m_kernel(m, d) if include_optimized_kernel_scratch else None
    scratch = OptimizedFwdPositionScratch(
        tree_reduction=tree_reduction,
        ball_limit_buffers=ball_buffers,
        solver_context=ctx,
        solver_nsolving=nsolving,
        constraint_free=_constraint_rows_impossible(m, ball_joint_limits),
        mul_m_call=functools.partial(mul_m, kernel=mul_m_kernel) if mul_m_kernel is not None else mul_m,
        dense_factor_solve=dense,
        tree_factor_solve=tree,
        tile_factor_solve=tile,
    )
    try:
        m._imn_tile_factor_solve = tile
    except AttributeError:
        pass
    if logger.isEnabledFor(logging.INFO) and newton_fusion._on_cuda(m):
        log_kernel_selection(m, d, scratch)
    return scratch


def _select_tree_reduction(scratch: Any, use_optimized_kernel: bool | None):
    """The tree scratch a step uses (mjw_step_optimized.py:2887-2894): the optimized
    kernels when asked for, and always when the scratch was made for ordered sums (a
    numerical requirement of its owner, not a speed choice)."""
    tree = getattr(scratch, "tree_reduction", None)
    if use_optimized_kernel or (tree is not None and tree.deterministic):
        return tree
    return None


def _solver_compact_enabled(m: Any) -> bool:
    return bool(getattr(m, "solver_compact", False))


def _rowless_handoff(m: Any, d: Any, stream=None) -> None:
    ms = binding.model_struct(m)
    ds = binding.data_struct(m, d)
    with _lib.nvtx("imn_rowless_handoff"):
        rc = _lib.lib().imn_rowless_handoff(C.byref(ms), C.byref(ds), _lib.current_stream_handle(stream))
    _lib.check(rc, "imn_rowless_handoff")


def solve_with_scratch(
    m: Any,
    d: Any,
    scratch: OptimizedFwdPositionScratch,
    *,
    use_optimized_kernel: bool = False,
    stream=None,
) -> None:
    """Solve the constraints of every world (mjw_step_optimized.py:2683-2742).

    ``use_optimized_kernel`` selects between the reference's stock and fused Warp
    launches; both compute the same solve, and here both are the one CUDA kernel.
    Sleeping-island (compact) contexts are not part of this path and raise."""
    if getattr(scratch, "constraint_free", False) or d.njmax == 0 or m.nv == 0:
        # MuJoCo's nefc == 0 result; implicit integration reads efc.Ma = M qacc.
        if m.nv:
            _rowless_handoff(m, d, stream)
        else:
            d.solver_niter.zero_()
        return
    ctx = scratch.solver_context
    nsolving = scratch.solver_nsolving
    if ctx is None or nsolving is None:
        raise RuntimeError("optimized solver scratch is not initialized")
    expected_compact = _solver_compact_enabled(m)
    if bool(scratch.solver_uses_compact) != expected_compact:
        raise RuntimeError("optimized solver scratch layout no longer matches model")
    if expected_compact:
        raise RuntimeError("compact (sleeping-island) solves are outside this solver's path")
    if not newton_fusion.eligible(m, ctx, compact=False):
        raise RuntimeError(
            "model is outside the fused Newton path: " + "; ".join(newton_fusion.ineligible_reasons(m, ctx))
            + ".  This library has no other solver path: route such models to the upstream solve"
        )
    del use_optimized_kernel
    newton_fusion.solve_call(m, d, ctx, nsolving, cache_on=scratch)(stream)


def _factor_solve_i_dense(
    m: Any,
    d: Any,
    M: Any,
    x: Any,
    y: Any,
    dense_factor_solve: Any = None,
    *,
    retain_factor: bool = False,
    factor_workspace: Any = None,
    tree_factor_solve: Any = None,
    stream=None,
) -> None:
    """x = M^-1 y for M (or M - h qDeriv) in the model's CSR layout, choosing the
    kernel as the reference does (mjw_step_optimized.py:1030-1070): the tree L'DL when
    a plan exists and no factor has to be kept, else the blocked dense Cholesky, else
    (nv < 32 without a tree plan, e.g. a short hinge chain) the single-tile dense
    Cholesky that stands in for the reference's per-tile kernels (:793-838).  The tile
    plan is made by ``make_optimized_fwd_position_scratch`` and remembered on the
    model; without it the first call builds it, which allocates (call once outside
    graph capture)."""
    from .mjw_kernels import indexed_factor, tree_ldl

    if factor_workspace is not None and dense_factor_solve is None:
        raise RuntimeError("a retained factor workspace requires the blocked dense path")
    if tree_factor_solve is not None and not retain_factor and factor_workspace is None:
        tree_ldl.tree_factor_solve(tree_factor_solve, M, x, y, stream=stream)
        return
    if dense_factor_solve is not None:
        indexed_factor.blocked_dense_factor_solve(
            d, M, x, y, dense_factor_solve, factor_workspace=factor_workspace, stream=stream
        )
        return
    if retain_factor:
        raise RuntimeError("a retained factor requires the blocked dense path (nv >= 32)")
    from .arrays import is_device

    if not is_device(M):
        raise RuntimeError("no factor/solve path for host buffers: the M-side kernels need CUDA arrays")
    tile = getattr(m, "_imn_tile_factor_solve", None)
    if tile is None or tile.U.shape[0] < d.nworld:
        from .arrays import device_of

        tile = indexed_factor.create_blocked_dense_factor_solve_scratch(m, d, device_of(M), minimum_nv=1)
        if tile is None:
            raise RuntimeError("no factor/solve plan for this model (nv == 0 or no inertia matrix)")
        try:
            m._imn_tile_factor_solve = tile
        except AttributeError:
            pass
    indexed_factor.blocked_dense_factor_solve(d, M, x, y, tile, stream=stream)


def refresh_sparse_hessian(m: Any, d: Any, scratch: OptimizedFwdPositionScratch, body_groups,
                           device: Any = "cuda") -> str:
    """Install (or remove) the sparse-Hessian plan on the solver context, as the
    reference's ``_refresh_mjw_sparse_hessian`` does
    (src/instantmimic/envs/direct_rl_env.py:2875-2925).  ``body_groups`` are the body
    sets that custom contact producers declare; ``None`` disables the plan.  Returns
    the reason string ("enabled" when a plan is installed)."""
    import torch

    from .mjw_kernels import sparse_hessian

    ctx = scratch.solver_context
    if ctx is None:
        return "no solver context"
    plan, reason = sparse_hessian.plan_for_model(m, ctx, body_groups, newton_fusion.newton_block_dim(m))
    ctx.sparse_hessian_plan = None
    if hasattr(scratch, "_imn_solve_call"):
        del scratch._imn_solve_call
    if plan is None:
        return reason
    sparse_hessian.upload(plan, device)
    if getattr(ctx, "hfactor", None) is None:
        ctx.hfactor = torch.zeros((d.nworld, m.nv_pad, m.nv_pad), dtype=torch.float32, device=device)
    if plan.path == "fused":
        sparse_hessian.violation_counter(ctx.hfactor, plan).zero_()
    ctx.sparse_hessian_plan = plan
    return reason


def check_sparse_hessian_violations(scratch: OptimizedFwdPositionScratch) -> None:
    """Raise when any world counted a constraint row or H update outside the declared
    pattern since the last check, and reset the counters
    (src/instantmimic/envs/direct_rl_env.py:2927-2951).  Reads device memory: call it
    at metric cadence, not every step."""
    from .mjw_kernels import sparse_hessian

    ctx = scratch.solver_context
    plan = getattr(ctx, "sparse_hessian_plan", None) if ctx is not None else None
    if plan is None or plan.path != "fused":
        return
    counter = sparse_hessian.violation_counter(ctx.hfactor, plan)
    total = float(counter.sum().item())
    if total > 0:
        worlds = int((counter > 0).sum().item())
        counter.zero_()
        raise RuntimeError(
            f"sparse Hessian: {int(total)} constraint rows or updates in {worlds} worlds fell outside the "
            "declared coupling pattern; a contact producer coupled bodies it did not declare"
        )


def fwd_acceleration_solve(m: Any, d: Any, scratch: OptimizedFwdPositionScratch, stream=None) -> None:
    """qacc_smooth = M^-1 qfrc_smooth, the factor/solve step of the reference's
    ``fwd_acceleration_optimized`` (mjw_step_optimized.py:1274-1329)."""
    _factor_solve_i_dense(
        m, d, d.M, d.qacc_smooth, d.qfrc_smooth, scratch.dense_factor_solve,
        tree_factor_solve=scratch.tree_factor_solve, stream=stream,
    )


def append_ball_limit_rows(m: Any, d: Any, scratch: OptimizedFwdPositionScratch, stream=None) -> None:
    """The directional ball-limit rows of this step, appended to the rows the constraint
    stage has produced so far: what the reference's ``_BallLimitConstraintCall`` does
    right after upstream's native ball-limit launch (mjw_step_optimized.py:355-388) --
    counters cleared, then ``BallLimitBuffers.launch``.  The upstream constraint stage
    itself is not part of this library; the caller invokes this at the same point."""
    buffers = scratch.ball_limit_buffers
    if buffers is None:
        return
    buffers.overflow.zero_()
    buffers.singular.zero_()
    buffers.launch(m, d, stream=stream)


# ---- the implicit-fast integrator's tail (mjw_step_optimized.py:5209-5297) --------------


def attach_implicit_scratch(m: Any, d: Any, scratch: OptimizedFwdPositionScratch, device: Any = "cuda") -> None:
    """Buffers of the implicit-fast tail: ``implicit_qderiv`` (nworld, nM),
    ``implicit_qacc`` (nworld, nv) and, for actuated models, ``implicit_actuator_vel``
    (nworld, nu) with the per-actuator coefficients its values are formed from.  The
    actuator tables are looked at here, once, so that a step reads nothing on the host."""
    import torch

    nM = int(m.M_colind.shape[0])
    scratch.implicit_qderiv = torch.zeros((d.nworld, nM), dtype=torch.float32, device=device)
    scratch.implicit_qacc = torch.zeros((d.nworld, m.nv), dtype=torch.float32, device=device)
    nu = int(getattr(m, "nu", 0) or 0)
    scratch.implicit_actuator_vel = torch.zeros((d.nworld, nu), dtype=torch.float32, device=device) if nu else None
    scratch.implicit_gain_coefficients = None
    if nu and getattr(m, "actuator_gaintype", None) is not None:
        scratch.implicit_gain_coefficients = _velocity_gain_coefficients(m)


def _velocity_gain_coefficients(m: Any):
    """(g2, b2) per actuator with d(force)/d(velocity) = g2 ctrl + b2, as tensors next to
    the model's tables; refuses actuator kinds whose derivative is upstream's."""
    from . import types as T
    from .arrays import as_torch, table_to_host

    gain_t, bias_t, dyn_t = (table_to_host(getattr(m, n))
                             for n in ("actuator_gaintype", "actuator_biastype", "actuator_dyntype"))
    if (dyn_t != int(T.DynType.NONE)).any():
        raise RuntimeError("actuators with activation dynamics are outside this integrator tail")
    if (gain_t > int(T.GainType.AFFINE)).any() or (bias_t > int(T.BiasType.AFFINE)).any():
        raise RuntimeError("muscle and user actuators need upstream's velocity derivative")
    g2 = as_torch(m.actuator_gainprm)[..., 2] * as_torch(m.actuator_gaintype).eq(int(T.GainType.AFFINE))
    b2 = as_torch(m.actuator_biasprm)[..., 2] * as_torch(m.actuator_biastype).eq(int(T.BiasType.AFFINE))
    return g2, b2


def actuator_velocity_gain(m: Any, d: Any, out: Any, scratch: Any = None) -> None:
    """out[w, a] = d(actuator force)/d(actuator velocity): the ``vel`` buffer of upstream's
    ``derivative._qderiv_actuator_passive_vel`` (call site mjw_step_optimized.py:4198-4225),
    RESTATED from MuJoCo's actuator model for stateless actuators with fixed or affine
    gain and bias: force = gain ctrl + bias with gain = g0 + g1 length + g2 velocity and
    bias = b0 + b1 length + b2 velocity, hence g2 ctrl + b2.  Muscle and user types, and
    actuators with activation dynamics, are refused.  With a scratch whose coefficients
    were prepared (``attach_implicit_scratch``) the call is device work only."""
    from .arrays import as_torch

    coefficients = getattr(scratch, "implicit_gain_coefficients", None) if scratch is not None else None
    g2, b2 = coefficients if coefficients is not None else _velocity_gain_coefficients(m)
    torch_out = as_torch(out)
    torch_out.copy_(as_torch(d.ctrl))
    torch_out.mul_(g2).add_(b2)


def deriv_smooth_vel_dense_actuator_centric(m: Any, d: Any, out: Any, scratch: OptimizedFwdPositionScratch,
                                            stream=None) -> None:
    """out = M - h qDeriv in M's layout (mjw_step_optimized.py:4172-4412): actuator term
    from ``scratch.implicit_actuator_vel`` and the per-world moment rows, joint damping.
    Models with tendons or fluid forces keep the upstream assembly."""
    if int(getattr(m, "ntendon", 0) or 0) or bool(getattr(m, "has_fluid", False)):
        raise RuntimeError("tendon damping and fluid terms are outside this assembly")
    from .arrays import addr, elem_strides

    ps = binding.implicit_struct(m, d, getattr(scratch, "implicit_actuator_vel", None))
    rc = _lib.lib().imn_implicit_matrix(C.byref(ps), addr(d.M), elem_strides(d.M)[0], addr(out),
                                        elem_strides(out)[0], int(d.nworld), _lib.current_stream_handle(stream))
    _lib.check(rc, "imn_implicit_matrix")


def _advance_with_scratch(m: Any, d: Any, qacc: Any, scratch: OptimizedFwdPositionScratch | None = None,
                          qvel: Any = None, stream=None) -> None:
    """qvel += h qacc, qpos moved with the new qvel, time += h
    (mjw_step_optimized.py:4823-4847).  A ``pre_advance_modifier`` or a preallocated
    ``advance_call`` on the scratch takes precedence, as in the reference."""
    modifier = getattr(scratch, "pre_advance_modifier", None) if scratch is not None else None
    if modifier is not None:
        qacc, qvel = modifier.apply(m, d, qacc, qvel)
    call = getattr(scratch, "advance_call", None) if scratch is not None else None
    if call is not None:
        call(m, d, qacc) if qvel is None else call(m, d, qacc, qvel)
        return
    if qvel is not None:
        raise RuntimeError("an externally integrated qvel needs the caller's advance_call")
    if int(getattr(m, "na", 0) or 0):
        raise RuntimeError("actuator activations are outside this advance")
    from .arrays import addr, elem_strides

    ps = binding.advance_struct(m, d)
    rc = _lib.lib().imn_advance(C.byref(ps), addr(qacc), elem_strides(qacc)[0], int(d.nworld),
                                _lib.current_stream_handle(stream))
    _lib.check(rc, "imn_advance")


def implicitfast_integrate(m: Any, d: Any, scratch: OptimizedFwdPositionScratch, stream=None) -> None:
    """The implicit-fast branch of ``_integrate`` (mjw_step_optimized.py:5241-5297):
    (M - h qDeriv) x = efc.Ma through the tree L'DL or blocked dense kernel, then the
    advance with x.  The free-body correction of mujoco-warp 3.16
    (``_implicit_free_body_correction``, :3768-3780) is upstream-only and not applied."""
    from . import binding as B

    if int(m.opt.integrator) != int(B.types.IntegratorType.IMPLICITFAST):
        raise NotImplementedError("only the implicit-fast integrator has a path here")
    if scratch.implicit_qderiv is None or scratch.implicit_qacc is None:
        raise RuntimeError("implicit-fast scratch is not attached (attach_implicit_scratch)")
    if int(getattr(m, "nu", 0) or 0) and not (int(m.opt.disableflags) & B.upstream_constants()["disable_actuation"]):
        actuator_velocity_gain(m, d, scratch.implicit_actuator_vel, scratch)
    deriv_smooth_vel_dense_actuator_centric(m, d, scratch.implicit_qderiv, scratch, stream=stream)
    _factor_solve_i_dense(
        m, d, scratch.implicit_qderiv, scratch.implicit_qacc, d.efc.Ma, scratch.dense_factor_solve,
        tree_factor_solve=scratch.tree_factor_solve, stream=stream,
    )
    _advance_with_scratch(m, d, scratch.implicit_qacc, scratch, stream=stream)
