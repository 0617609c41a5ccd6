"""Whole-batch rowless hand-off (the reference's tests/test_mjw_rowless_handoff.py:20-101):
with ``scratch.constraint_free`` set, or with njmax == 0, solve_with_scratch leaves
MuJoCo's nefc == 0 result for every world: qacc == qacc_smooth exactly, a freshly
computed efc.Ma = M qacc (the implicit integrator reads it), qfrc_constraint == 0,
solver_niter == 0.  Checked against the oracle's restatement bit for bit and against
a float64 product."""

import copy

import numpy as np
import pytest

from instantmimic_b200 import mjw_model, synthetic
from instantmimic_b200 import mjw_step_optimized as runtime

pytestmark = pytest.mark.gpu


def _dense(m, Mv):
    """(W, nv, nv) symmetric M from the ancestor CSR values."""
    W, nv = Mv.shape[0], m.nv
    out = np.zeros((W, nv, nv))
    for i in range(nv):
        for k in range(int(m.M_rownnz[i])):
            e = int(m.M_rowadr[i]) + k
            c = int(m.M_colind[e])
            out[:, i, c] = out[:, c, i] = Mv[:, e]
    return out


def _run(m, d, device, *, constraint_free, sparse=False):
    import torch

    md, dd = mjw_model.to_device(m, device), mjw_model.to_device(copy.deepcopy(d), device)
    # stale values everywhere the hand-off must write
    dd.qacc.fill_(7.0), dd.efc.Ma.fill_(7.0), dd.qfrc_constraint.fill_(7.0), dd.solver_niter.fill_(9)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, device)
    if sparse:
        groups = [[b] for b in range(1, len(m.body_dofadr))]
        assert runtime.refresh_sparse_hessian(md, dd, scratch, groups, device) == "enabled"
    scratch.constraint_free = constraint_free
    runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
    torch.cuda.synchronize()
    return mjw_model.to_host(dd)


@pytest.mark.parametrize("name,worlds", [("humanoid", 300), ("snu", 70)])
@pytest.mark.parametrize("sparse", [False, True])
def test_constraint_free_scratch_hands_off_the_whole_batch(oracle, cuda_device, name, worlds, sparse):
    m, d, _ = synthetic.make_workload(name, worlds, seed=4)
    # rows are present in the buffers but the scratch says they cannot occur: they must be ignored
    want = copy.deepcopy(d)
    oracle.rowless_handoff(m, want)
    got = _run(m, d, cuda_device, constraint_free=True, sparse=sparse)
    np.testing.assert_array_equal(got.qacc, d.qacc_smooth)
    np.testing.assert_array_equal(got.qfrc_constraint, 0.0)
    np.testing.assert_array_equal(got.solver_niter, 0)
    np.testing.assert_array_equal(got.efc.Ma.view(np.uint32), want.efc.Ma.view(np.uint32))
    exact = np.einsum("wij,wj->wi", _dense(m, d.M.astype(np.float64)), d.qacc_smooth.astype(np.float64))
    assert np.abs(got.efc.Ma - exact).max() <= 1e-5 * (np.abs(exact).max() + 1)


def test_model_without_constraint_rows_hands_off(oracle, cuda_device):
    parent, body = synthetic.humanoid_tree()
    m = mjw_model.put_model(parent, body_of_dof=body)
    d, _ = synthetic.make_problem(m, 129, 0, seed=2)  # njmax == 0: no efc storage at all
    want = copy.deepcopy(d)
    oracle.rowless_handoff(m, want)
    got = _run(m, d, cuda_device, constraint_free=False)
    np.testing.assert_array_equal(got.qacc, d.qacc_smooth)
    np.testing.assert_array_equal(got.qfrc_constraint, 0.0)
    np.testing.assert_array_equal(got.solver_niter, 0)
    np.testing.assert_array_equal(got.efc.Ma.view(np.uint32), want.efc.Ma.view(np.uint32))
