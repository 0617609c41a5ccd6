"""Directional ball-joint limit rows.

Host side of the reference's ``src/instantmimic/utils/mjw_kernels/ball_limits.py``
(``BallLimitBuffers`` :205-282, ``make_ball_limit_buffers`` :285-318) and of the limit
description it consumes (``src/instantmimic/utils/ball_joint_limits.py``:
``BallJointLimitCfg`` :11-31, ``ResolvedBallJointLimit`` :34-40, validation :51-83).  The
row kernel is ``ball_limit_kernel`` in ``csrc/imn_ball_limits.cu`` behind
``imn_ball_limit_rows``.  Resolving joint names against a MuJoCo model
(``configure_ball_joint_limits``, which edits the model's scalar safety cap) needs
MuJoCo and stays with the caller: entries arrive here already resolved.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Any, Sequence

import numpy as np

from .. import _lib, abi, binding
from ..arrays import addr, elem_strides

LIMIT_JOINT = 3  # mjtConstraint mjCNSTR_LIMIT_JOINT


@dataclass(frozen=True)
class BallJointLimitCfg:
    """Angles in radians; the frame's local Z is the twist axis, X / Y the swing axes.
    ``neutral`` is the joint quaternion at zero anatomical rotation, ``frame`` rotates
    anatomical coordinates into the joint's local ones (ball_joint_limits.py:11-31)."""

    joint: str
    swing: tuple
    twist: tuple
    neutral: tuple = (1.0, 0.0, 0.0, 0.0)
    frame: tuple = (1.0, 0.0, 0.0, 0.0)
    safety_angle: float | None = None
    margin: float = 0.0
    solref: tuple = (0.02, 1.0)
    solimp: tuple = (0.9, 0.95, 0.001, 0.5, 2.0)
    swing_lower: tuple | None = None


@dataclass(frozen=True)
class ResolvedBallJointLimit:
    cfg: BallJointLimitCfg
    joint_id: int
    qposadr: int
    dofadr: int
    minimum_h: float


def unit_quaternion(values, name: str) -> np.ndarray:
    q = np.asarray(values, dtype=np.float64)
    if q.shape != (4,) or not np.isfinite(q).all() or np.linalg.norm(q) < 1e-12:
        raise ValueError(f"{name} must be a finite nonzero wxyz quaternion")
    return q / np.linalg.norm(q)


def validate(cfg: BallJointLimitCfg) -> None:
    """The reference's configuration checks (ball_joint_limits.py:51-83)."""
    angles = lambda v, lo, hi: len(v) == 2 and all(math.isfinite(a) and lo < a < hi for a in v)  # noqa: E731
    if not angles(cfg.swing, 0.0, math.pi):
        raise ValueError("swing requires two angles strictly between 0 and pi")
    if len(cfg.twist) != 2 or not all(math.isfinite(v) for v in cfg.twist):
        raise ValueError("twist requires two finite angles")
    if not -math.pi < cfg.twist[0] < cfg.twist[1] < math.pi:
        raise ValueError("twist requires -pi < lower < upper < pi")
    if cfg.swing_lower is not None and not angles(cfg.swing_lower, -math.pi, 0.0):
        raise ValueError("swing_lower requires two angles strictly between -pi and 0")
    if cfg.safety_angle is not None and not (math.isfinite(cfg.safety_angle) and 0 < cfg.safety_angle < math.pi):
        raise ValueError("safety_angle must be strictly between 0 and pi")
    if not math.isfinite(cfg.margin) or cfg.margin < 0:
        raise ValueError("margin must be finite and nonnegative")
    if len(cfg.solref) != 2 or not all(math.isfinite(v) for v in cfg.solref):
        raise ValueError("solref requires two finite values")
    if not ((cfg.solref[0] > 0 and cfg.solref[1] > 0) or (cfg.solref[0] <= 0 and cfg.solref[1] <= 0)):
        raise ValueError("solref must use positive time/damping or nonpositive direct format")
    if len(cfg.solimp) != 5 or not all(math.isfinite(v) for v in cfg.solimp):
        raise ValueError("solimp requires five finite values")
    unit_quaternion(cfg.frame, "frame")
    unit_quaternion(cfg.neutral, "neutral")


def minimum_h(cfg: BallJointLimitCfg, cap: float) -> float:
    """cos^2 of half the largest relative rotation the scalar safety cap admits: the swing
    chart's denominators stay above it (ball_joint_limits.py:131-147)."""
    neutral_angle = 2 * math.acos(min(1.0, abs(float(unit_quaternion(cfg.neutral, "neutral")[0]))))
    if cap + neutral_angle >= math.radians(175):
        raise ValueError("safety_angle + neutral rotation must remain below 175 degrees")
    return math.cos((cap + neutral_angle) / 2) ** 2


def limit_tables(entries: Sequence[ResolvedBallJointLimit]) -> dict:
    """Per-joint arrays of the row kernel (ball_limits.py:296-315): addresses, unit
    quaternions, swing coefficients 1 / tan^2(angle / 2) for +x, +y, -x, -y, twist ends,
    chart bound, margin, solver parameters."""
    f32, i32 = np.float32, np.int32
    for e in entries:
        validate(e.cfg)
    swing = [[1 / math.tan(v / 2) ** 2 for v in (*e.cfg.swing, *(e.cfg.swing_lower or e.cfg.swing))] for e in entries]
    return {
        "qadr": np.asarray([e.qposadr for e in entries], i32),
        "dadr": np.asarray([e.dofadr for e in entries], i32),
        "joint": np.asarray([e.joint_id for e in entries], i32),
        "neutral": np.asarray([unit_quaternion(e.cfg.neutral, "neutral") for e in entries], f32).reshape(-1, 4),
        "frame": np.asarray([unit_quaternion(e.cfg.frame, "frame") for e in entries], f32).reshape(-1, 4),
        "swing": np.asarray(swing, f32).reshape(-1, 4),
        "twist": np.asarray([e.cfg.twist for e in entries], f32).reshape(-1, 2),
        "minimum_h": np.asarray([e.minimum_h for e in entries], f32),
        "margin": np.asarray([e.cfg.margin for e in entries], f32),
        "solref": np.asarray([e.cfg.solref for e in entries], f32).reshape(-1, 2),
        "solimp": np.asarray([e.cfg.solimp for e in entries], f32).reshape(-1, 5),
    }


@dataclass
class BallLimitBuffers:
    """Device copies of the tables plus the two diagnostic counters
    (ball_limits.py:205-219)."""

    tables: dict
    overflow: Any
    singular: Any
    njoint: int

    def launch(self, m: Any, d: Any, stream=None) -> None:
        """Append the violated rows of every world (ball_limits.py:221-282)."""
        ps = rows_struct(self.tables, self.njoint, m, d, self.overflow, self.singular)
        with _lib.nvtx("imn_ball_limit_rows"):
            rc = _lib.lib().imn_ball_limit_rows(C.byref(ps), int(d.nworld), _lib.current_stream_handle(stream))
        _lib.check(rc, "imn_ball_limit_rows")


def rows_struct(tables: dict, njoint: int, m: Any, d: Any, overflow: Any, singular: Any) -> abi.ImnBallLimits:
    c = binding.upstream_constants()
    s = abi.ImnBallLimits()
    s.njoint, s.nv, s.njmax = int(njoint), int(m.nv), int(d.njmax)
    s.refsafe = 0 if int(m.opt.disableflags) & c["disable_refsafe"] else 1
    s.limit_joint_type = c["constraint_limit_joint"]
    s.timestep, s.n_timestep = binding._timestep(m)
    for name in ("qadr", "dadr", "joint", "neutral", "frame", "swing", "twist", "minimum_h", "margin", "solref", "solimp"):
        setattr(s, name, addr(tables[name]))
    s.invweight = addr(m.dof_invweight0)
    s.n_invweight = int(m.dof_invweight0.shape[0])
    s.qpos, s.qpos_ld = addr(d.qpos), elem_strides(d.qpos)[0]
    s.qvel, s.qvel_ld = addr(d.qvel), elem_strides(d.qvel)[0]
    s.nefc, s.nl = addr(d.nefc), addr(getattr(d, "nl", None))
    efc = d.efc
    js = elem_strides(efc.J)
    if len(js) != 3 or js[2] != 1:
        raise ValueError("directional ball rows are written into a dense (nworld, njmax, nv) efc.J")
    s.efc_J, s.J_ld_world, s.J_ld_row = addr(efc.J), js[0], js[1]
    lds = set()
    for name, field in (("type", "efc_type"), ("id", "efc_id"), ("pos", "efc_pos"), ("margin", "efc_margin"), ("D", "efc_D"),
                        ("vel", "efc_vel"), ("aref", "efc_aref"), ("frictionloss", "efc_frictionloss")):
        a = getattr(efc, name)
        setattr(s, field, addr(a))
        lds.add(elem_strides(a)[0])
    if len(lds) != 1:
        raise ValueError("the efc row arrays must share one world stride")
    s.efc_ld = lds.pop()
    s.overflow, s.singular = addr(overflow), addr(singular)
    return s


def make_ball_limit_buffers(entries: Sequence[ResolvedBallJointLimit], m: Any, d: Any, device: Any = "cuda") -> BallLimitBuffers:
    """Buffers for the given limits (ball_limits.py:285-318): refuses the DISCRETE
    integrator, too few reserved rows, and a sparse Jacobian (outside this library)."""
    import torch

    if int(m.opt.integrator) == binding.upstream_constants()["integrator_discrete"]:
        raise ValueError("directional ball constraints do not support the DISCRETE integrator")
    if d.njmax < 3 * len(entries):
        raise ValueError("directional ball constraints need three reserved rows per joint")
    if bool(getattr(m, "is_sparse", False)):
        raise ValueError("directional ball constraints with a sparse Jacobian are outside this library")
    tables = {k: torch.from_numpy(v).to(device) for k, v in limit_tables(entries).items()}
    z = lambda: torch.zeros(d.nworld, dtype=torch.int32, device=device)  # noqa: E731
    return BallLimitBuffers(tables=tables, overflow=z(), singular=z(), njoint=len(entries))
