"""Writes the fixtures of this folder:  python tests/golden/make_golden.py

The reference cannot run where this repository is built (mujoco, mujoco-warp and warp
are not installed), so these vectors come from the CPU oracle (oracle/), not from the
reference: they freeze the oracle's results so that neither the oracle nor the CUDA
kernels can drift unnoticed.  The files use the solver-state format of
instantmimic_b200/solver_state.py; on a machine with the reference installed,
solver_state.capture around its solve_with_scratch writes files of the same format,
which the same tests can then replay (tests/test_golden.py reads every newton_*.npz
here).
"""

import copy
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
sys.path.insert(0, str(HERE.parent))

from helpers import host_ctx  # noqa: E402

from instantmimic_b200 import solver_state, synthetic  # noqa: E402
from instantmimic_b200.mjw_kernels import indexed_factor, sparse_hessian, tree_ldl  # noqa: E402
from instantmimic_b200.mjw_model import put_model  # noqa: E402
from oracle import oracle  # noqa: E402


def newton_case(name, m, d, sparse_groups=None):
    entries = solver_state.snapshot_inputs(m, d)
    d2 = copy.deepcopy(d)
    ctx = host_ctx(m, d2)
    oracle.solve(m, d2, ctx, np.zeros(1, np.int32))
    entries.update(solver_state.snapshot_outputs(m, d2, ctx))
    if sparse_groups is not None:
        # the same inputs through the sparse-pattern factor (different rounding, own results)
        plan = sparse_hessian.build_plan(m, sparse_groups, 32 if m.nv_pad < 64 else 64, "fused")
        d3 = copy.deepcopy(d)
        ctx3 = host_ctx(m, d3)
        oracle.solve(m, d3, ctx3, np.zeros(1, np.int32), sparse_plan_struct=sparse_hessian.host_struct(plan))
        entries["sparse/qacc"] = d3.qacc
        entries["sparse/solver_niter"] = d3.solver_niter
        entries["sparse/efc_force"] = d3.efc.force
        entries["sparse/efc_state"] = d3.efc.state
        entries["sparse/groups"] = np.asarray([g[0] for g in sparse_groups], np.int32)
    solver_state.save(HERE / f"newton_{name}.npz", entries)


def main():
    oracle.build()
    m, d, _ = synthetic.make_workload("humanoid", 8, seed=11, rowless_fraction=0.2)
    groups = [[b] for b in range(1, len(m.body_dofadr))]
    newton_case("humanoid", m, d, groups)
    m, d, _ = synthetic.make_workload("snu", 3, seed=12)
    newton_case("snu", m, d)
    parent, body = synthetic.humanoid_tree()
    m = put_model(parent, body_of_dof=body, iterations=100, ls_iterations=50)
    d, _ = synthetic.make_problem(m, 6, 48, seed=13, ne=3, nf=5, nefc_range=(8, 48))
    newton_case("eq_friction", m, d)
    # worlds at rest: aref = 0 and a zero warm start make Jaref exactly 0, so equality and
    # friction-loss rows are QUADRATIC with a force of exactly 0 and still enter the Hessian
    d, _ = synthetic.make_problem(m, 6, 48, seed=15, ne=4, nf=5, nefc_range=(12, 48))
    d.efc.aref[:] = 0.0
    d.qacc_warmstart[:] = 0.0
    newton_case("at_rest", m, d)

    # M-side: tree L'DL (1 and 4 groups) and blocked dense (3 right-hand sides)
    parent, body = synthetic.humanoid_tree()
    m = put_model(parent, body_of_dof=body)
    rng = np.random.default_rng(14)
    Mv, _ = synthetic.random_mass_matrices(m, 5, rng)
    y = rng.normal(size=(5, m.nv)).astype(np.float32)
    structure = tree_ldl.tree_ldl_structure(m.M_rowadr, m.M_rownnz, m.M_colind)
    out = {"M": Mv, "y": y}
    for groups in (1, 4):
        plan = tree_ldl.plan_tree_ldl(*structure, groups)
        out[f"x_tree_{groups}"] = oracle.tree_ldl_solve(structure, plan, Mv, y)
    pad = indexed_factor._round_up(m.nv, 16)
    layout = indexed_factor.block_major_layout(indexed_factor.dense_index_table(m), pad, m.nM)
    ident = indexed_factor.pad_identity(m.nv, pad)
    y3 = rng.normal(size=(5, m.nv, 3)).astype(np.float32)
    x3, U = oracle.blocked_dense_factor_solve(m.nv, pad, layout, ident, Mv, y3)
    out.update(y3=y3, x_blocked=x3, U=U)
    np.savez_compressed(HERE / "msolve_humanoid.npz", **out)
    for p in sorted(HERE.glob("*.npz")):
        print(p.name, p.stat().st_size)


if __name__ == "__main__":
    main()
