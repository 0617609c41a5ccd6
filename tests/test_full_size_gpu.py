"""The benchmark configurations at their full batch sizes.  The CPU oracle is too slow
to redo whole batches in a test, so the full-size runs are checked through properties
that do not depend on size: a strided sample of worlds against the oracle bit for bit,
consistency of forces, states and qfrc_constraint with the inputs, and idempotence (a
solve warm-started at the solution stops at once at the same point)."""

import copy

import numpy as np
import pytest

from instantmimic_b200 import mjw_model, synthetic

from helpers import run_cuda, run_oracle

pytestmark = pytest.mark.gpu

CASES = {
    # name: (builder, worlds); the sweep point keeps 4096 worlds of its 65536 (10.7 GB of J at full size)
    "humanoid_8192": (lambda: synthetic.make_workload("humanoid", 8192, seed=0), 8192),
    "snu_4096": (lambda: synthetic.make_workload("snu", 4096, seed=0), 4096),
    "g1_16384": (lambda: synthetic.make_workload("g1", 16384, seed=0, iterations=10, ls_iterations=20), 16384),
    "sweep_nv64_nefc512_4096": (lambda: synthetic.make_sweep_point(64, 512, 4096, seed=0, iterations=50, ls_iterations=50), 4096),
}


def _pick(d, idx):
    """Host Data of the worlds ``idx`` (copies)."""
    out = copy.copy(d)
    out.nworld = len(idx)
    for name in ("nefc", "ne", "nf", "qacc_smooth", "qacc_warmstart", "qfrc_smooth", "M", "qacc", "qfrc_constraint",
                 "solver_niter", "overflow"):
        setattr(out, name, getattr(d, name)[idx].copy())
    out.efc = copy.copy(d.efc)
    for name in ("J", "D", "aref", "frictionloss", "force", "state", "Ma"):
        setattr(out.efc, name, getattr(d.efc, name)[idx].copy())
    return out


@pytest.mark.parametrize("case", list(CASES))
def test_full_batch_properties(oracle, cuda_device, case):
    build, W = CASES[case]
    m, d, _ = build()
    got, _, _, _ = run_cuda(m, d, cuda_device, matrices=False)
    assert np.isfinite(got.qacc).all() and (got.solver_niter >= 0).all()
    assert (got.solver_niter <= m.opt.iterations).all()

    # 1. a strided sample of the batch, bit for bit against the oracle
    idx = np.arange(0, W, max(1, W // 96))
    want, _, _ = run_oracle(oracle, m, _pick(d, idx), matrices=False)
    assert np.array_equal(got.solver_niter[idx], want.solver_niter)
    assert np.array_equal(got.overflow[idx], want.overflow)
    assert np.array_equal(got.qacc[idx].view(np.uint32), want.qacc.view(np.uint32))
    live_s = np.arange(d.njmax)[None, :] < np.minimum(d.nefc[idx], d.njmax)[:, None]
    assert np.array_equal(got.efc.state[idx][live_s], want.efc.state[live_s])
    assert np.array_equal(got.efc.force[idx][live_s].view(np.uint32), want.efc.force[live_s].view(np.uint32))

    # 2. forces and states agree with the inputs at the solution (float64 recomputation)
    live = np.arange(d.njmax)[None, :] < np.minimum(d.nefc, d.njmax)[:, None]
    J = np.where(live[..., None], d.efc.J[..., : m.nv], 0.0).astype(np.float64)
    jar = np.einsum("wrv,wv->wr", J, got.qacc.astype(np.float64)) - np.where(live, d.efc.aref, 0.0)
    D = np.where(live, d.efc.D, 0.0).astype(np.float64)
    state, force = got.efc.state, np.where(live, got.efc.force, 0.0).astype(np.float64)
    scale = 1.0 + np.abs(jar)
    ineq = live & (np.arange(d.njmax)[None, :] >= (d.ne + d.nf)[:, None])
    quad = ineq & (state == 1)
    sat = ineq & (state == 0)
    assert (jar[quad] < 1e-3 * scale[quad]).all()          # active rows are violated (up to rounding)
    assert (jar[sat] > -1e-3 * scale[sat]).all()           # satisfied rows are not
    assert (force[sat] == 0).all()
    np.testing.assert_allclose(force[quad], (-D * jar)[quad], rtol=2e-3, atol=2e-3 * np.abs(force).max())
    # qfrc_constraint = J^T force for worlds that converged
    conv = (got.overflow == 0) & (d.nefc > 0)
    jtf = np.einsum("wrv,wr->wv", J, force)
    err = np.abs(got.qfrc_constraint - jtf)[conv].max() / (1.0 + np.abs(jtf[conv]).max())
    assert err < 5e-3, err
    assert (got.qfrc_constraint[d.nefc == 0] == 0).all()

    # 3. idempotence: warm-started at the solution the solver stops within one iteration
    d2 = copy.deepcopy(d)
    d2.qacc_warmstart[:] = got.qacc
    again, _, _, _ = run_cuda(m, d2, cuda_device, matrices=False)
    assert (again.solver_niter[conv] <= 2).all()
    assert np.abs(again.qacc - got.qacc)[conv].max() <= 1e-3 * (1.0 + np.abs(got.qacc).max())
    # the active set is the same up to rows that sit on their boundary (|Jaref| ~ rounding)
    sel = live & conv[:, None]
    flipped = sel & (again.efc.state != got.efc.state)
    assert flipped.sum() <= 1e-4 * sel.sum()
    assert (np.abs(jar[flipped]) < 1e-3 * scale[flipped]).all()


@pytest.mark.parametrize("name,worlds", [("humanoid", 8192), ("snu", 4096)])
def test_full_batch_m_side_kernels(oracle, cuda_device, name, worlds):
    """tree L'DL, blocked dense Cholesky and M v on a whole batch: M x = y holds to
    rounding, both solvers agree, M v is linear, and a strided sample equals the oracle."""
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime
    from instantmimic_b200.mjw_kernels import indexed_factor, tree_ldl

    m, d, Mdense = synthetic.make_workload(name, worlds, seed=1)
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(d, cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    assert scratch.tree_factor_solve is not None and scratch.dense_factor_solve is not None
    y = dd.qfrc_smooth
    x_tree, x_dense, back = torch.zeros_like(y), torch.zeros_like(y), torch.zeros_like(y)
    tree_ldl.tree_factor_solve(scratch.tree_factor_solve, dd.M, x_tree, y)
    indexed_factor.blocked_dense_factor_solve(dd, dd.M, x_dense, y, scratch.dense_factor_solve)
    runtime.mul_m(md, dd, back, x_tree)
    torch.cuda.synchronize()
    yh, xt, xd = d.qfrc_smooth.astype(np.float64), x_tree.cpu().numpy(), x_dense.cpu().numpy()
    scale = 1.0 + np.abs(yh).max(axis=1, keepdims=True)
    assert (np.abs(back.cpu().numpy() - yh) / scale).max() < 2e-4          # M (M^-1 y) = y
    assert (np.abs(xt - xd) / (1.0 + np.abs(xd).max(axis=1, keepdims=True))).max() < 2e-3
    # linearity of M v: M (2 a + b) = 2 M a + M b up to rounding
    a, b = dd.qacc_smooth, dd.qacc_warmstart
    Ma, Mb, Mab = torch.zeros_like(a), torch.zeros_like(a), torch.zeros_like(a)
    runtime.mul_m(md, dd, Ma, a)
    runtime.mul_m(md, dd, Mb, b)
    runtime.mul_m(md, dd, Mab, 2.0 * a + b)
    torch.cuda.synchronize()
    lin = (Mab - (2.0 * Ma + Mb)).abs().max().item() / (1.0 + Mab.abs().max().item())
    assert lin < 1e-5, lin
    # strided sample against the oracle, bit for bit
    idx = np.arange(0, worlds, worlds // 64)
    structure = tree_ldl.tree_ldl_structure(m.M_rowadr, m.M_rownnz, m.M_colind)
    want = oracle.tree_ldl_solve(structure, scratch.tree_factor_solve.plan, np.ascontiguousarray(d.M[idx]),
                                 np.ascontiguousarray(d.qfrc_smooth[idx]))
    assert np.array_equal(xt[idx].view(np.uint32), want.view(np.uint32))
    want_ma = np.zeros((len(idx), m.nv), np.float32)
    oracle.mul_m(m, np.ascontiguousarray(d.M[idx]), np.ascontiguousarray(d.qacc_smooth[idx]), want_ma)
    assert np.array_equal(Ma.cpu().numpy()[idx].view(np.uint32), want_ma.view(np.uint32))
