"""Writes ball_limit_reference.npz:  python tests/golden/make_ball_limit_golden.py [reference root]

Golden vectors for the directional ball-limit rows, produced by the REFERENCE's own host
function ``limit_residuals`` (src/instantmimic/utils/ball_joint_limits.py:166-212), the
function its CUDA test uses as the truth for the row kernel
(tests/test_ball_joint_limits_cuda.py:45-80).  The module imports ``mujoco`` at the top
for its configuration helpers; ``limit_residuals`` itself is numpy only, so the import is
satisfied with a stand-in module that carries the one name an annotation uses.  The reference tree is read only by this
script, never at test time: the vectors are committed.

Per case: joint quaternion q (wxyz), configuration (swing, swing_lower, twist, neutral,
frame), and the reference's residuals (3,) and local angular Jacobians (3, 3), float64.
"""

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def load_reference(root: Path):
    if "mujoco" not in sys.modules:
        stand_in = types.ModuleType("mujoco")
        stand_in.MjModel = object  # only named in a type annotation
        sys.modules["mujoco"] = stand_in
    path = root / "src" / "instantmimic" / "utils" / "ball_joint_limits.py"
    spec = importlib.util.spec_from_file_location("ref_ball_joint_limits", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    root = Path(sys.argv[1]) if len(sys.argv) > 1 else Path("/root/reference")
    ref = load_reference(root)
    rng = np.random.default_rng(0)
    out = {k: [] for k in ("q", "swing", "swing_lower", "has_lower", "twist", "neutral", "frame", "residual", "jac")}

    def unit(v):
        return v / np.linalg.norm(v)

    for case in range(96):
        swing = tuple(rng.uniform(0.4, 2.2, 2))
        lower = tuple(-rng.uniform(0.3, 2.0, 2)) if case % 3 == 0 else None
        lo = rng.uniform(-2.0, 0.2)
        twist = (lo, lo + rng.uniform(0.3, 2.0))
        neutral = unit(np.r_[1.0, 0.15 * rng.normal(size=3)]) if case % 2 else np.array([1.0, 0, 0, 0])
        frame = unit(rng.normal(size=4)) if case % 4 >= 2 else np.array([1.0, 0, 0, 0])
        cfg = ref.BallJointLimitCfg(joint="j", swing=swing, twist=twist, neutral=tuple(neutral), frame=tuple(frame),
                                    swing_lower=lower)
        # rotations up to ~2.4 rad about random axes, kept inside the chart (h = w^2 + z^2 of
        # the relative quaternion away from 0)
        while True:
            axis, angle = unit(rng.normal(size=3)), rng.uniform(0.0, 2.4)
            q = np.r_[np.cos(angle / 2), np.sin(angle / 2) * axis]
            try:
                r, j = ref.limit_residuals(q, cfg)
            except ValueError:
                continue
            if np.isfinite(r).all() and np.isfinite(j).all() and np.abs(j).max() < 50:
                break
        if case % 5 == 0:
            q = -q  # the double cover: same rotation
            r, j = ref.limit_residuals(q, cfg)
        out["q"].append(q), out["swing"].append(swing), out["twist"].append(twist)
        out["swing_lower"].append(lower if lower is not None else (0.0, 0.0)), out["has_lower"].append(lower is not None)
        out["neutral"].append(neutral), out["frame"].append(frame)
        out["residual"].append(r), out["jac"].append(j)
    np.savez_compressed(HERE / "ball_limit_reference.npz", **{k: np.asarray(v) for k, v in out.items()})
    print("cases", len(out["q"]), "violated rows", int((np.asarray(out["residual"]) < 0).sum()))


if __name__ == "__main__":
    main()
