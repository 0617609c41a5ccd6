"""Enumerations and constants of the solver interface.

Values follow MuJoCo's public headers (mjtConstraintState, mjtCone, mjtSolver,
mjtIntegrator, mjtDisableBit); the reference reads them from
``mujoco_warp._src.types`` (src/instantmimic/utils/mjw_kernels/private.py:8-55).
``OverflowType`` and ``ALPHA_NOISE_EPS`` belong to mujoco-warp 3.16.0, whose
source is not available; the values here are this package's defaults and the
adapter overrides them from the live upstream module when one is importable.
"""

from __future__ import annotations

import enum


class ConstraintState(enum.IntEnum):
    SATISFIED = 0
    QUADRATIC = 1
    LINEARNEG = 2
    LINEARPOS = 3
    CONE = 4


class ConeType(enum.IntEnum):
    PYRAMIDAL = 0
    ELLIPTIC = 1


class SolverType(enum.IntEnum):
    PGS = 0
    CG = 1
    NEWTON = 2


class IntegratorType(enum.IntEnum):
    EULER = 0
    RK4 = 1
    IMPLICIT = 2
    IMPLICITFAST = 3
    DISCRETE = 4


class DisableBit(enum.IntFlag):
    # mjtDisableBit as laid out since MuJoCo split PASSIVE into SPRING and DAMPER (the
    # reference names both, so it runs on such a release); the adapter reads the live
    # values when mujoco-warp is importable
    SPRING = 1 << 5
    DAMPER = 1 << 6
    GRAVITY = 1 << 7
    WARMSTART = 1 << 9
    ACTUATION = 1 << 11
    REFSAFE = 1 << 12


class ConstraintType(enum.IntEnum):
    EQUALITY = 0
    FRICTION_DOF = 1
    FRICTION_TENDON = 2
    LIMIT_JOINT = 3
    LIMIT_TENDON = 4
    CONTACT_FRICTIONLESS = 5
    CONTACT_PYRAMIDAL = 6
    CONTACT_ELLIPTIC = 7


class JointType(enum.IntEnum):
    FREE = 0
    BALL = 1
    SLIDE = 2
    HINGE = 3


class GainType(enum.IntEnum):
    FIXED = 0
    AFFINE = 1
    MUSCLE = 2
    USER = 3


class BiasType(enum.IntEnum):
    NONE = 0
    AFFINE = 1
    MUSCLE = 2
    USER = 3


class DynType(enum.IntEnum):
    NONE = 0


class OverflowType(enum.IntFlag):
    ITERATIONS = 1
    LS_ITERATIONS = 2
    BROADPHASE = 4


MJ_MINVAL = 1e-15
MJ_MAXVAL = 1e10
ALPHA_NOISE_EPS = 1e-6
