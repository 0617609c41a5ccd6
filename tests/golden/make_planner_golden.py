"""Writes planner_reference.npz:  python tests/golden/make_planner_golden.py [reference root]

Golden outputs of the REFERENCE's own host planners, run in the build container:

* ``sparse_hessian.build_plan`` (src/instantmimic/utils/mjw_kernels/sparse_hessian.py:229-702):
  the ``SH_*`` index tables it bakes into its generated source, parsed back out of the
  snippets the way the reference's own test does (tests/test_mjw_sparse_hessian.py:190-196),
  plus nslots / nterms / levels / density;
* ``tree_ldl.plan_tree_ldl`` / ``best_tree_ldl_plan`` (tree_ldl.py:105-185): groups, trunk,
  span, dense cost.

Both modules are plain Python + numpy on the host; their one module-level import that is
absent here, ``warp``, is only used inside kernel factories that this script never calls,
so an empty stand-in module satisfies it (and a one-value stand-in for the upstream shim
``private.types``, whose ``ConstraintState.QUADRATIC`` goes into generated kernel text only).  Models are this repository's synthetic trees,
handed over through a ``.numpy()`` adapter.  The reference tree is read only by this
script, never at test time: the outputs are committed.
"""

import importlib.util
import re
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
sys.path.insert(0, str(HERE.parent))

from instantmimic_b200 import synthetic  # noqa: E402
from instantmimic_b200.mjw_model import put_model  # noqa: E402

# reference table name -> field of ImnSparsePlan
TABLES = {
    "SH_LP": "lvl_ptr", "SH_LT": "lvl_team", "SH_ES": "ent_slot", "SH_EC": "ent_col", "SH_RP": "run_ptr",
    "SH_RAB": "run_ab", "SH_RKL": "run_kl", "SH_ORIG": "orig", "SH_BL": "b_lvl", "SH_BS": "b_slot", "SH_BI": "b_src",
    "SH_BJ": "b_dst", "SH_PAIR": "pair", "SH_FL": "f_lvl", "SH_FR": "f_row", "SH_RS": "row_start", "SH_RKP": "rk_ptr",
    "SH_RK": "rk", "SH_PM": "pmask", "SH_SA": "s_a", "SH_SB": "s_b", "SH_SM": "s_m", "SH_GAT": "gat",
}


def _stand_ins():
    """``warp`` (never called) and the reference's upstream shim, of which build_plan reads one
    enum value that goes into generated kernel text, not into any table."""
    import enum

    sys.modules.setdefault("warp", types.ModuleType("warp"))

    class ConstraintState(enum.IntEnum):
        QUADRATIC = 1

    chain = "instantmimic.utils.mjw_kernels.private".split(".")
    for k in range(1, len(chain) + 1):
        sys.modules.setdefault(".".join(chain[:k]), types.ModuleType(".".join(chain[:k])))
    sys.modules["instantmimic.utils.mjw_kernels.private"].types = types.SimpleNamespace(ConstraintState=ConstraintState)


def load(root: Path, name: str):
    _stand_ins()
    path = root / "src" / "instantmimic" / "utils" / "mjw_kernels" / f"{name}.py"
    spec = importlib.util.spec_from_file_location(f"ref_{name}", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


class _Arr:
    """What the reference expects of a model array: ``numpy()``, ``shape``, ``size``."""

    def __init__(self, a):
        self._a = np.asarray(a)
        self.shape, self.size = self._a.shape, self._a.size

    def numpy(self):
        return self._a


def adapt(m):
    out = types.SimpleNamespace(nv=m.nv, nv_pad=m.nv_pad, neq=0, nflex=0, ntendon=0)
    for name in ("dof_parentid", "body_parentid", "body_dofadr", "body_dofnum", "geom_bodyid", "nxn_geom_pair_filtered",
                 "M_colind", "M_hinit_i"):
        setattr(out, name, _Arr(getattr(m, name)))
    return out


def tables_of(plan) -> dict:
    text = "\n".join(getattr(plan, n, "") or "" for n in ("factor_snippet", "init_snippet", "nonfused_snippet"))
    found = re.findall(r"static const [a-z ]+ (SH_\w+)\[\] = \{([^}]*)\};", text)
    out = {}
    for name, vals in found:
        arr = np.array([int(v.rstrip("u")) for v in vals.split(",")], dtype=np.int64)
        if name in out:
            assert np.array_equal(out[name], arr), name
        out[name] = arr
    return out


def cases():
    from test_sparse_hessian import BOX_A, BOX_B, FOOT_L, FOOT_R, FORE_R, _legged_model

    single = lambda m: [[b] for b in range(1, len(m.body_dofadr))]  # noqa: E731
    for name in ("humanoid", "snu", "g1"):
        m, _, _ = synthetic.make_workload(name, 1)
        yield name, m, single(m)
    m = _legged_model()
    for i, groups in enumerate([[], [[FOOT_L, BOX_B]], [[FOOT_L, FOOT_R, BOX_B], [FORE_R, BOX_A]]]):
        yield f"legged{i}", m, groups
    m = _legged_model()
    m.geom_bodyid = np.array([0, FOOT_R, BOX_B], np.int32)
    m.nxn_geom_pair_filtered = np.array([[1, 2]], np.int32)
    yield "legged_pairs", m, [[FOOT_L, BOX_A]]
    for nv in (35, 64):
        m, _, _ = synthetic.make_sweep_point(nv, 32, 1)
        yield f"limbs{nv}", m, single(m)


def main():
    root = Path(sys.argv[1]) if len(sys.argv) > 1 else Path("/root/reference")
    sh, tl = load(root, "sparse_hessian"), load(root, "tree_ldl")
    out = {}
    names = []
    for name, m, groups in cases():
        names.append(name)
        out[f"{name}/groups"] = np.asarray([len(g) for g in groups] + [b for g in groups for b in g], np.int64)
        for path, block in (("fused", 32 if m.nv_pad < 64 else 64), ("nonfused", 64)):
            plan = sh.build_plan(adapt(m), groups, block, path)
            for ref_name, arr in tables_of(plan).items():
                out[f"{name}/{path}/{TABLES[ref_name]}"] = arr
            out[f"{name}/{path}/meta"] = np.asarray([plan.nslots, plan.nterms, plan.levels, block], np.int64)
            out[f"{name}/{path}/density"] = np.asarray(plan.density)
        st = tl.tree_ldl_structure(np.asarray(m.M_rowadr), np.asarray(m.M_rownnz), np.asarray(m.M_colind))
        plans = {str(g): tl.plan_tree_ldl(*st, g) for g in range(1, 5)}
        plans["best"] = tl.best_tree_ldl_plan(*st)
        for key, p in plans.items():
            out[f"{name}/tree/{key}/groups"] = np.asarray([len(g) for g in p.groups] + [k for g in p.groups for k in g], np.int64)
            out[f"{name}/tree/{key}/trunk"] = np.asarray(p.trunk, np.int64)
            out[f"{name}/tree/{key}/cost"] = np.asarray([p.span, p.dense_cost], np.int64)
            out[f"{name}/tree/{key}/beats_dense"] = np.asarray(bool(tl.tree_ldl_beats_dense(p)))
    for nv in (13, 26, 31, 40):
        parent, body = synthetic.chain_tree(nv)
        m = put_model(parent, body_of_dof=body)
        st = tl.tree_ldl_structure(np.asarray(m.M_rowadr), np.asarray(m.M_rownnz), np.asarray(m.M_colind))
        p = tl.best_tree_ldl_plan(*st)
        out[f"chain{nv}/tree/best/cost"] = np.asarray([p.span, p.dense_cost, len(p.groups), int(tl.tree_ldl_beats_dense(p))], np.int64)
    out["names"] = np.asarray(names)
    np.savez_compressed(HERE / "planner_reference.npz", **out)
    print(len(out), "arrays,", (HERE / "planner_reference.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
