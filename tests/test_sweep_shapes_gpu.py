"""The nine (nv, nefc) shapes of the isolated sweep -- nv in {27, 35, 64} x nefc in
{32, 128, 512}, generic rows on kinematic-tree ancestor patterns -- on a 64-world
sample each, against the oracle bit for bit, with the dense factor and (where the
sparse-pattern plan admits the model: nv >= 33) with the sparse factor."""

import copy

import numpy as np
import pytest

from instantmimic_b200 import synthetic
from instantmimic_b200.mjw_kernels import sparse_hessian

from helpers import run_cuda, run_oracle
from test_newton_gpu import _check

pytestmark = pytest.mark.gpu

SHAPES = [(nv, nefc) for nv in (27, 35, 64) for nefc in (32, 128, 512)]


@pytest.mark.parametrize("nv,nefc", SHAPES)
def test_sweep_shape_dense_factor(oracle, cuda_device, nv, nefc):
    m, d, _ = synthetic.make_sweep_point(nv, nefc, 64, seed=0, iterations=50, ls_iterations=50)
    want, wctx, _ = run_oracle(oracle, m, d)
    got, gctx, _, _ = run_cuda(m, d, cuda_device)
    _check(got, want, gctx, wctx)
    np.testing.assert_array_equal(got.qacc.view(np.uint32), want.qacc.view(np.uint32))
    np.testing.assert_array_equal(got.efc.force.view(np.uint32), want.efc.force.view(np.uint32))


@pytest.mark.parametrize("nv,nefc", [s for s in SHAPES if s[0] >= sparse_hessian.MIN_NV])
def test_sweep_shape_sparse_factor(oracle, cuda_device, nv, nefc):
    """Rows on one ancestor chain each stay inside the tree-ancestry pattern, which is
    what the sparse plan's density gate admits (rows that couple two arbitrary chains
    need a dense pattern, for which the reference keeps the dense factor too)."""
    from test_sparse_hessian import _cuda_sparse, _oracle_sparse, _single_body_groups

    m, d, _ = synthetic.make_sweep_point(nv, nefc, 64, seed=0, couple=False, iterations=50, ls_iterations=50)
    got, scratch, _ = _cuda_sparse(m, copy.deepcopy(d), cuda_device, _single_body_groups(m))
    plan = scratch.solver_context.sparse_hessian_plan
    want, _ = _oracle_sparse(oracle, m, d, plan)
    np.testing.assert_array_equal(got.solver_niter, want.solver_niter)
    np.testing.assert_array_equal(got.overflow, want.overflow)
    np.testing.assert_array_equal(got.efc.state, want.efc.state)
    np.testing.assert_array_equal(got.qacc.view(np.uint32), want.qacc.view(np.uint32))
    np.testing.assert_array_equal(got.efc.force.view(np.uint32), want.efc.force.view(np.uint32))
    assert sparse_hessian.violations(scratch.solver_context.hfactor, plan).sum() == 0
