"""CPU checks of the oracle itself (no GPU): converged solves satisfy the
optimality conditions of MuJoCo's convex constraint problem and agree with an
independent float64 Newton solver; structural outputs are consistent."""

import copy

import numpy as np
import pytest

from instantmimic_b200 import synthetic, types
from instantmimic_b200.mjw_model import put_model

from helpers import reference_f64, run_oracle


@pytest.mark.parametrize("name,nworld", [("humanoid", 48), ("snu", 12)])
def test_oracle_matches_independent_float64_solver(oracle, name, nworld):
    m, d, Md = synthetic.make_workload(name, nworld, seed=3, iterations=100, ls_iterations=50)
    got, _, _ = run_oracle(oracle, m, d)
    want = reference_f64(m, d, Md)
    scale = np.maximum(1.0, np.linalg.norm(want, axis=1))
    err = np.linalg.norm(got.qacc - want, axis=1) / scale
    assert err.max() < 1e-4, err.max()
    assert np.all(got.solver_niter < 100)


def test_oracle_equality_and_friction_rows(oracle):
    parent, body = synthetic.chain_tree(35)
    m = put_model(parent, body_of_dof=body, iterations=100, ls_iterations=50)
    d, Md = synthetic.make_problem(m, 24, 96, seed=5, nefc_range=(20, 90), ne=6, nf=5)
    got, ctx, _ = run_oracle(oracle, m, d)
    want = reference_f64(m, d, Md)
    scale = np.maximum(1.0, np.linalg.norm(want, axis=1))
    assert (np.linalg.norm(got.qacc - want, axis=1) / scale).max() < 1e-4
    # equality rows are always quadratic; friction rows use all three friction states
    assert np.all(got.efc.state[:, :6] == types.ConstraintState.QUADRATIC)
    fr = got.efc.state[:, 6:11]
    assert set(np.unique(fr)) <= {1, 2, 3}
    lin = fr != types.ConstraintState.QUADRATIC
    assert np.allclose(np.abs(got.efc.force[:, 6:11][lin]), d.efc.frictionloss[:, 6:11][lin])


def test_oracle_outputs_are_self_consistent(oracle):
    m, d, Md = synthetic.make_workload("humanoid", 64, seed=11, rowless_fraction=0.25)
    got, ctx, nsolving = run_oracle(oracle, m, d)
    rowless = d.nefc == 0
    assert rowless.any() and (~rowless).any()
    # rowless worlds: MuJoCo's nefc == 0 result, exactly
    np.testing.assert_array_equal(got.qacc[rowless], d.qacc_smooth[rowless])
    np.testing.assert_array_equal(got.qfrc_constraint[rowless], 0.0)
    np.testing.assert_array_equal(got.solver_niter[rowless], 0)
    # Ma = M qacc for every world
    Ma = np.einsum("wij,wj->wi", Md.astype(np.float64), got.qacc.astype(np.float64))
    assert np.abs(Ma - got.efc_Ma if hasattr(got, "efc_Ma") else Ma - got.efc.Ma).max() < 2e-3
    # qfrc_constraint = J^T force
    for w in np.flatnonzero(~rowless)[:16]:
        n = min(int(d.nefc[w]), d.njmax)
        jtf = d.efc.J[w, :n].astype(np.float64).T @ got.efc.force[w, :n]
        assert np.abs(jtf - got.qfrc_constraint[w]).max() < 5e-3 * max(1.0, np.abs(jtf).max())
    assert nsolving[0] == int(rowless.sum())
    assert np.all(ctx.done == 1)
    # the changed-row list of the last iteration is strictly ascending
    for w in range(d.nworld):
        ids = ctx.quad_changed_ids[w, : ctx.quad_changed_count[w]]
        assert np.all(np.diff(ids) > 0)


def test_oracle_iteration_budget_sets_overflow_bits(oracle):
    m, d, _ = synthetic.make_workload("humanoid", 32, seed=2, iterations=1, ls_iterations=1)
    got, _, _ = run_oracle(oracle, m, d)
    assert np.all(got.solver_niter == 1)
    assert np.any(got.overflow & int(types.OverflowType.ITERATIONS))
    assert np.all((got.overflow & ~3) == 0)


def test_oracle_is_deterministic_across_thread_counts(oracle):
    m, d, _ = synthetic.make_workload("humanoid", 40, seed=7)
    a, _, _ = run_oracle(oracle, m, d, threads=1)
    b, _, _ = run_oracle(oracle, m, copy.deepcopy(d), threads=4)
    for x, y in ((a.qacc, b.qacc), (a.efc.force, b.efc.force), (a.efc.state, b.efc.state)):
        np.testing.assert_array_equal(x, y)


def test_work_counters_are_consistent(oracle):
    """ctx.stats: line-search passes, flipped rows, factorisations, gradient evaluations."""
    from helpers import run_oracle

    m, d, _ = synthetic.make_workload("humanoid", 64, seed=2, rowless_fraction=0.1)
    got, ctx, _ = run_oracle(oracle, m, d)
    st, niter = ctx.stats, got.solver_niter
    rows = d.nefc > 0
    assert (st[~rows] == 0).all()
    assert (st[rows, 3] >= 1).all() and (st[rows, 3] <= niter[rows] + 1).all()  # one gradient at init, at most one per iteration
    assert (st[rows, 2] >= 1).all() and (st[rows, 2] <= st[rows, 3]).all()      # a factorisation needs a gradient
    assert (st[rows, 0] >= niter[rows]).all() and (st[rows, 0] <= niter[rows] * (m.opt.ls_iterations + 2)).all()
    assert (st[rows, 1] >= st[rows, 2] - 1).all()                                # every refactorisation had a flip


def test_compact_jacobian_layout_gives_the_same_solve(oracle):
    """efc.J handed over as the nefc rows of each world back to back (J_world_offset)."""
    from instantmimic_b200 import mjw_model

    m, d, _ = synthetic.make_workload("humanoid", 40, seed=6, rowless_fraction=0.1)
    want, _, _ = run_oracle(oracle, m, d)
    dc = mjw_model.compact_jacobian(d)
    assert dc.efc.J.shape == (int(d.nefc.sum()), m.nv) and dc.efc.J_world_offset[1] == d.nefc[0] * m.nv
    got, _, _ = run_oracle(oracle, m, dc)
    np.testing.assert_array_equal(got.qacc.view(np.uint32), want.qacc.view(np.uint32))
    np.testing.assert_array_equal(got.solver_niter, want.solver_niter)
    np.testing.assert_array_equal(got.efc.state, want.efc.state)
