"""Writes plan_pins.json:  python tests/golden/make_plan_pins.py

SHA-256 of the sparse-Hessian plan tables and of the tree L'DL plans of the named
workloads and of a few synthetic trees.  The tables fix the summation order of every
factor entry, so a planner change that alters them changes results bit for bit; the
pins make such a change visible in the CPU test suite (tests/test_plan_pins.py)."""

import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from instantmimic_b200 import synthetic  # noqa: E402
from instantmimic_b200.mjw_kernels import sparse_hessian, tree_ldl  # noqa: E402
from instantmimic_b200.mjw_model import put_model  # noqa: E402


def sparse_digest(plan) -> str:
    h = hashlib.sha256()
    for name in sorted(plan.tables):
        h.update(name.encode())
        h.update(np.ascontiguousarray(plan.tables[name]).tobytes())
    h.update(repr((plan.nfac, plan.nslots, plan.levels, plan.nterms, round(plan.density, 6))).encode())
    return h.hexdigest()


def tree_digest(plan) -> str:
    return hashlib.sha256(repr((plan.groups, plan.trunk, plan.span, plan.dense_cost)).encode()).hexdigest()


def pins() -> dict:
    out = {}
    for name in ("humanoid", "snu", "g1"):
        m, _, _ = synthetic.make_workload(name, 1)
        groups = [[b] for b in range(1, len(m.body_dofadr))]
        out[f"{name}/sparse/fused"] = sparse_digest(
            sparse_hessian.build_plan(m, groups, 32 if m.nv_pad < 64 else 64, "fused"))
        out[f"{name}/sparse/nonfused"] = sparse_digest(sparse_hessian.build_plan(m, groups, 64, "nonfused"))
        structure = tree_ldl.tree_ldl_structure(m.M_rowadr, m.M_rownnz, m.M_colind)
        for g in range(1, 5):
            out[f"{name}/tree/{g}"] = tree_digest(tree_ldl.plan_tree_ldl(*structure, g))
        out[f"{name}/tree/best"] = tree_digest(tree_ldl.best_tree_ldl_plan(*structure))
    for nv in (35, 64):
        m, _, _ = synthetic.make_sweep_point(nv, 32, 1)
        groups = [[b] for b in range(1, len(m.body_dofadr))]
        out[f"limbs{nv}/sparse/fused"] = sparse_digest(
            sparse_hessian.build_plan(m, groups, 32 if m.nv_pad < 64 else 64, "fused"))
    for nv in (13, 31, 40):
        parent, body = synthetic.chain_tree(nv)
        m = put_model(parent, body_of_dof=body)
        structure = tree_ldl.tree_ldl_structure(m.M_rowadr, m.M_rownnz, m.M_colind)
        out[f"chain{nv}/tree/best"] = tree_digest(tree_ldl.best_tree_ldl_plan(*structure))
    return out


if __name__ == "__main__":
    (HERE / "plan_pins.json").write_text(json.dumps(pins(), indent=1) + "\n")
    print(len(pins()), "pins written")
