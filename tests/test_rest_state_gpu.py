"""Worlds at rest: qvel = 0 and a zero warm start give aref = 0 and qacc = 0, so
Jaref = J qacc - aref is exactly 0 on every row.  Equality rows and friction-loss
rows are then QUADRATIC with a force of exactly 0; they still contribute
D J^T J to the Hessian (upstream's JTDAJ and sparse_hessian.py:589 select rows
by state alone).  The kernels must agree with the oracle bit for bit here, with
the dense factor and with the sparse-pattern plan."""

import copy

import numpy as np
import pytest

from instantmimic_b200 import synthetic
from instantmimic_b200.mjw_model import put_model

from helpers import run_cuda, run_oracle
from test_newton_gpu import _check

pytestmark = pytest.mark.gpu


def _at_rest(name="humanoid", worlds=96, ne=5, nf=6, seed=11):
    tree, njmax, nefc_range = synthetic.WORKLOADS[name]
    parent, body = tree()
    m = put_model(parent, body_of_dof=body, iterations=50, ls_iterations=50, tolerance=1e-8)
    d, _ = synthetic.make_problem(m, worlds, njmax, seed, nefc_range=nefc_range, ne=ne, nf=nf)
    d.efc.aref[:] = 0.0
    d.qacc_warmstart[:] = 0.0
    return m, d


def test_zero_force_quadratic_rows_enter_the_dense_hessian(oracle, cuda_device):
    m, d = _at_rest()
    want, wctx, _ = run_oracle(oracle, m, d)
    # the case is the intended one: QUADRATIC rows whose force is exactly zero exist
    # after the first constraint update (all of them: Jaref == 0 everywhere)
    assert (want.solver_niter > 0).any()
    got, gctx, _, _ = run_cuda(m, d, cuda_device)
    _check(got, want, gctx, wctx)
    np.testing.assert_array_equal(got.qacc, want.qacc)
    np.testing.assert_array_equal(gctx.h, wctx.h)


def test_zero_force_quadratic_rows_enter_the_sparse_hessian(oracle, cuda_device):
    from test_sparse_hessian import _cuda_sparse, _oracle_sparse, _single_body_groups

    m, d = _at_rest(worlds=64)
    # single-dof equality rows stay inside any pattern (friction rows already are)
    d.efc.J[:, :5] = 0.0
    rng = np.random.default_rng(3)
    dofs = rng.integers(0, m.nv, (d.nworld, 5))
    d.efc.J[np.arange(d.nworld)[:, None], np.arange(5)[None, :], dofs] = 1.0
    got, scratch, _ = _cuda_sparse(m, copy.deepcopy(d), cuda_device, _single_body_groups(m))
    plan = scratch.solver_context.sparse_hessian_plan
    want, wctx = _oracle_sparse(oracle, m, d, plan)
    np.testing.assert_array_equal(got.solver_niter, want.solver_niter)
    np.testing.assert_array_equal(got.overflow, want.overflow)
    live = np.arange(d.njmax)[None, :] < d.nefc[:, None]
    np.testing.assert_array_equal(got.efc.state[live], want.efc.state[live])
    np.testing.assert_array_equal(got.qacc, want.qacc)
    hf = scratch.solver_context.hfactor.cpu().numpy().reshape(d.nworld, -1)
    whf = wctx.hfactor.reshape(d.nworld, -1)
    np.testing.assert_array_equal(hf[:, : 2 * plan.nfac + m.nv], whf[:, : 2 * plan.nfac + m.nv])
