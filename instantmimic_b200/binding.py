"""Builds the C-ABI structs of ``include/imnewton.h`` from Model / Data / context
objects.  Works on any array type ``arrays.addr`` understands, so the same code
describes device buffers for the CUDA library and host buffers for the oracle
used by the tests."""

from __future__ import annotations

import ctypes as C
from typing import Any

from . import abi, types
from .arrays import addr, elem_strides, is_contiguous, itemsize, length, shape


_UPSTREAM: dict | None = None


def upstream_constants(module_types: Any = None, module_solver: Any = None) -> dict:
    """Every constant this package shares with mujoco-warp, from the live upstream
    modules when they import (``mujoco_warp._src.types`` / ``.solver``; the arguments
    let a test pass stand-ins), else this package's defaults (``types``).

    MuJoCo has moved ``mjDSBL_*`` bits and enum members between releases, so nothing
    that is compared with a value stored in a caller's ``Model`` / ``Data`` is taken
    from this package when the real definition is at hand.  ``MJ_MINVAL`` /
    ``MJ_MAXVAL`` are compiled into the kernels: a live module that disagrees with
    them is an error, not an override."""
    global _UPSTREAM
    injected = module_types is not None or module_solver is not None
    if _UPSTREAM is not None and not injected:
        return _UPSTREAM
    if not injected:
        try:  # pragma: no cover - mujoco_warp is not installed in the build image
            from mujoco_warp._src import solver as module_solver
            from mujoco_warp._src import types as module_types
        except Exception:
            module_solver = module_types = None

    def member(enum_name: str, name: str, default: int) -> int:
        enum_cls = getattr(module_types, enum_name, None) if module_types is not None else None
        value = getattr(enum_cls, name, None)
        return int(default if value is None else value)

    out = {
        "source": "mujoco_warp" if module_types is not None else "package defaults",
        "alpha_noise_eps": float(getattr(module_solver, "_ALPHA_NOISE_EPS", types.ALPHA_NOISE_EPS)),
        "overflow_iterations": member("OverflowType", "ITERATIONS", types.OverflowType.ITERATIONS),
        "overflow_ls_iterations": member("OverflowType", "LS_ITERATIONS", types.OverflowType.LS_ITERATIONS),
        "disable_warmstart": member("DisableBit", "WARMSTART", types.DisableBit.WARMSTART),
        "disable_damper": member("DisableBit", "DAMPER", types.DisableBit.DAMPER),
        "disable_gravity": member("DisableBit", "GRAVITY", types.DisableBit.GRAVITY),
        "disable_actuation": member("DisableBit", "ACTUATION", types.DisableBit.ACTUATION),
        "disable_refsafe": member("DisableBit", "REFSAFE", types.DisableBit.REFSAFE),
        "constraint_limit_joint": member("ConstraintType", "LIMIT_JOINT", types.ConstraintType.LIMIT_JOINT),
        "solver_newton": member("SolverType", "NEWTON", types.SolverType.NEWTON),
        "cone_pyramidal": member("ConeType", "PYRAMIDAL", types.ConeType.PYRAMIDAL),
        "integrator_discrete": member("IntegratorType", "DISCRETE", types.IntegratorType.DISCRETE),
    }
    for name in ("SATISFIED", "QUADRATIC", "LINEARNEG", "LINEARPOS"):
        live = member("ConstraintState", name, getattr(types.ConstraintState, name))
        if live != int(getattr(types.ConstraintState, name)):
            raise RuntimeError(
                f"mujoco_warp ConstraintState.{name} = {live} differs from the value compiled into the kernels "
                f"({int(getattr(types.ConstraintState, name))})")
    for name in ("MJ_MINVAL", "MJ_MAXVAL"):
        live = getattr(module_types, name, None) if module_types is not None else None
        if live is not None and float(live) != float(getattr(types, name)):
            raise RuntimeError(
                f"mujoco_warp {name} = {live} differs from the value compiled into the kernels "
                f"({getattr(types, name)})")
    if not injected:
        _UPSTREAM = out
    return out


def _upstream_constants() -> tuple[float, int, int]:
    c = upstream_constants()
    return c["alpha_noise_eps"], c["overflow_iterations"], c["overflow_ls_iterations"]


def _mulm_pack(m: Any):
    """The packed M_mulm table of a model; built once (and cached on the model) for
    Model objects that come from mujoco-warp and do not carry it."""
    pack = getattr(m, "M_mulm_pack", None)
    if pack is None:
        pack = getattr(m, "_imn_mulm_pack", None)
    if pack is None:
        import numpy as np

        from .arrays import device_of, to_host
        from .mjw_model import pack_mulm

        col, madr = m.M_mulm_col, m.M_mulm_madr
        host = pack_mulm(to_host(col), to_host(madr))
        if isinstance(col, np.ndarray):
            pack = host
        else:
            import torch

            # on the device that holds the model's tables, not torch's current one
            pack = torch.from_numpy(host).to(device_of(col))
        try:
            m._imn_mulm_pack = pack
        except AttributeError:
            pass
    return pack


def model_struct(m: Any) -> abi.ImnModel:
    eps, ovf_it, ovf_ls = _upstream_constants()
    s = abi.ImnModel()
    s.nv = int(m.nv)
    s.nv_pad = int(m.nv_pad)
    s.nM = int(shape(m.M_colind)[0])
    s.iterations = int(m.opt.iterations)
    s.ls_iterations = int(m.opt.ls_iterations)
    s.warmstart = 0 if (int(m.opt.disableflags) & upstream_constants()["disable_warmstart"]) else 1
    s.n_tolerance = length(m.opt.tolerance)
    s.n_ls_tolerance = length(m.opt.ls_tolerance)
    s.n_meaninertia = length(m.stat.meaninertia)
    s.opt_tolerance = addr(m.opt.tolerance)
    s.opt_ls_tolerance = addr(m.opt.ls_tolerance)
    s.stat_meaninertia = addr(m.stat.meaninertia)
    s.M_rowadr = addr(m.M_rowadr)
    s.M_rownnz = addr(m.M_rownnz)
    s.M_colind = addr(m.M_colind)
    s.M_mulm_rowadr = addr(m.M_mulm_rowadr)
    s.M_mulm_col = addr(m.M_mulm_col)
    s.M_mulm_madr = addr(m.M_mulm_madr)
    s.M_mulm_pack = addr(_mulm_pack(m))
    s.alpha_noise_eps = eps
    s.overflow_iterations = ovf_it
    s.overflow_ls_iterations = ovf_ls
    s.warn_overflow = int(getattr(m.opt, "warn_overflow", 0) or 0)
    return s


def _row_ld(a: Any) -> int:
    st = elem_strides(a)
    if st[-1] != 1:
        raise ValueError("solver buffers need a unit innermost stride")
    return st[0]


def _same_ld(name: str, arrays: list[Any]) -> int:
    lds = {_row_ld(a) for a in arrays if a is not None}
    if len(lds) != 1:
        raise ValueError(f"{name} arrays must share one world stride, got {sorted(lds)}")
    return lds.pop()


def data_struct(m: Any, d: Any) -> abi.ImnData:
    s = abi.ImnData()
    s.nworld = int(d.nworld)
    s.njmax = int(d.njmax)
    s.nefc, s.ne, s.nf = addr(d.nefc), addr(d.ne), addr(d.nf)
    s.qacc_smooth = addr(d.qacc_smooth)
    s.qacc_warmstart = addr(d.qacc_warmstart)
    s.qfrc_smooth = addr(d.qfrc_smooth)
    s.dof_ld = _same_ld(
        "dof",
        [d.qacc_smooth, d.qacc_warmstart, d.qfrc_smooth, d.qacc, d.qfrc_constraint, d.efc.Ma],
    )
    s.efc_J = addr(d.efc.J)
    if s.njmax > 0 and getattr(d.efc, "J_world_offset", None) is not None:
        s.efc_ld = _same_ld(
            "efc", [d.efc.D, d.efc.aref, d.efc.frictionloss, d.efc.force, d.efc.state]
        )
    elif s.njmax > 0:
        js = elem_strides(d.efc.J)
        if js[2] != 1:
            raise ValueError("efc.J needs a unit innermost stride")
        s.J_ld_world, s.J_ld_row = js[0], js[1]
        s.efc_ld = _same_ld(
            "efc", [d.efc.D, d.efc.aref, d.efc.frictionloss, d.efc.force, d.efc.state]
        )
    else:
        # a model without constraint storage: the row arrays are empty, their strides
        # carry no information, and only the rowless hand-off may be called
        s.J_ld_world = s.J_ld_row = s.efc_ld = 0
    s.efc_D = addr(d.efc.D)
    s.efc_aref = addr(d.efc.aref)
    s.efc_frictionloss = addr(d.efc.frictionloss)
    s.M = addr(d.M)
    s.M_ld = _row_ld(d.M)
    s.qacc = addr(d.qacc)
    s.qfrc_constraint = addr(d.qfrc_constraint)
    s.efc_Ma = addr(d.efc.Ma)
    s.efc_force = addr(d.efc.force)
    s.efc_state = addr(d.efc.state)
    s.solver_niter = addr(d.solver_niter)
    s.overflow = addr(d.overflow)
    offsets = getattr(d.efc, "J_world_offset", None)
    if offsets is not None:
        # compact J: (total rows, >= nv) with one int64 element offset per world
        if itemsize(offsets) != 8 or length(offsets) < s.nworld:
            raise ValueError("efc.J_world_offset must hold one int64 per world")
        js = elem_strides(d.efc.J)
        if len(js) != 2 or js[1] != 1:
            raise ValueError("a compact efc.J is a (rows, nv) array with a unit innermost stride")
        s.J_world_offset = addr(offsets)
        s.J_ld_world, s.J_ld_row = 0, js[0]
        s.J_elems = int(shape(d.efc.J)[0]) * js[0]
    return s


_CTX_WORLD_ARRAYS = (
    "search_dot",
    "grad_dot",
    "grad_scale",
    "newton_decrement",
    "improvement",
    "alpha",
    "done",
    "search_unchanged",
    "ls_exhausted",
    "quad_changed_count",
    "state_changed_count",
)


def ctx_struct(d_struct: abi.ImnData, ctx: Any, nsolving: Any, sparse_plan_struct=None) -> abi.ImnCtx:
    """``ctx`` may omit any array (attribute missing or None): the kernel then skips
    writing it back."""
    s = abi.ImnCtx()

    def get(name):
        return getattr(ctx, name, None) if ctx is not None else None

    for name in ("Jaref", "jv", "quad_changed_ids"):
        a = get(name)
        if a is not None and _row_ld(a) != d_struct.efc_ld:
            raise ValueError(f"ctx.{name} must share the world stride of the efc arrays")
        setattr(s, name, addr(a))
    for name in ("search", "mv"):
        a = get(name)
        if a is not None and _row_ld(a) != d_struct.dof_ld:
            raise ValueError(f"ctx.{name} must share the world stride of the dof arrays")
        setattr(s, name, addr(a))
    g = get("grad")
    s.grad = addr(g)
    s.grad_ld = _row_ld(g) if g is not None else 0
    s.h = addr(get("h"))
    s.hfactor = addr(get("hfactor"))
    for name in _CTX_WORLD_ARRAYS:
        setattr(s, name, addr(get(name)))
    s.dof_union = addr(get("newton_dof_union"))
    s.nsolving = addr(nsolving)
    if sparse_plan_struct is not None:
        s.sparse_plan = C.pointer(sparse_plan_struct)
    order = get("world_order")
    if order is not None and length(order) < d_struct.nworld:
        raise ValueError("ctx.world_order must hold one int32 per world")
    s.world_order = addr(order)
    stats = get("stats")
    if stats is not None and (tuple(shape(stats)) != (d_struct.nworld, 4) or elem_strides(stats) != (4, 1)):
        raise ValueError("ctx.stats must be a contiguous (nworld, 4) int32 array")
    s.stats = addr(stats)
    return s


def _timestep(m: Any) -> tuple[int, int]:
    """Address and length of opt.timestep, mujoco-warp's per-world float array (world w
    reads element w % n, in the kernels, like every other per-world option)."""
    h = m.opt.timestep
    if isinstance(h, (int, float)) or h is None:
        raise ValueError("m.opt.timestep must be a float array of length 1 or nworld, next to the other arrays")
    n = length(h)
    if n <= 0 or not is_contiguous(h):
        raise ValueError("m.opt.timestep must be a contiguous, non-empty float array")
    return addr(h), n


def implicit_struct(m: Any, d: Any, velocity_gain: Any) -> abi.ImnImplicit:
    """``velocity_gain``: (nworld, nu) d(actuator force)/d(actuator velocity), or None."""
    c = upstream_constants()
    s = abi.ImnImplicit()
    flags = int(m.opt.disableflags)
    s.nv, s.nM = int(m.nv), int(shape(m.M_colind)[0])
    s.nu = int(getattr(m, "nu", 0) or 0)
    s.actuation = 0 if flags & c["disable_actuation"] else 1
    s.damper = 0 if flags & c["disable_damper"] else 1
    s.timestep, s.n_timestep = _timestep(m)
    s.dof_damping = addr(m.dof_damping)
    s.M_elemid = addr(m.M_elemid)
    if s.nu and s.actuation:
        if velocity_gain is None:
            raise ValueError("an actuated model needs the actuators' velocity gains")
        for name in ("moment_rownnz", "moment_rowadr"):
            a = getattr(d, name)
            if tuple(shape(a)) != (int(d.nworld), s.nu) or elem_strides(a) != (s.nu, 1):
                raise ValueError(f"d.{name} must be a contiguous (nworld, nu) array")
            setattr(s, name, addr(a))
        if elem_strides(d.moment_colind) != elem_strides(d.actuator_moment) or elem_strides(d.actuator_moment)[1] != 1:
            raise ValueError("d.moment_colind and d.actuator_moment must share one layout")
        if tuple(shape(velocity_gain)) != (int(d.nworld), s.nu) or elem_strides(velocity_gain) != (s.nu, 1):
            raise ValueError("velocity gains must be a contiguous (nworld, nu) array")
        s.moment_colind, s.actuator_moment = addr(d.moment_colind), addr(d.actuator_moment)
        s.moment_ld = elem_strides(d.actuator_moment)[0]
        s.actuator_velocity_gain = addr(velocity_gain)
    return s


def advance_struct(m: Any, d: Any) -> abi.ImnAdvance:
    s = abi.ImnAdvance()
    s.nv, s.nq, s.njnt = int(m.nv), int(m.nq), int(m.njnt)
    s.timestep, s.n_timestep = _timestep(m)
    s.jnt_type, s.jnt_dofadr, s.jnt_qposadr = addr(m.jnt_type), addr(m.jnt_dofadr), addr(m.jnt_qposadr)
    s.qvel, s.qvel_ld = addr(d.qvel), _row_ld(d.qvel)
    s.qpos, s.qpos_ld = addr(d.qpos), _row_ld(d.qpos)
    s.time = addr(getattr(d, "time", None))
    return s
