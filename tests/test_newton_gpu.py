"""GPU parity of the fused Newton solve against the CPU oracle, through
solve_with_scratch -> C ABI -> CUDA.  Bar: efc.state, solver_niter and overflow
identical; qacc, qfrc_constraint, efc.force, efc.Ma within 1e-4 in the scaled
norm (the tests also report how many are bit-identical)."""

import copy

import numpy as np
import pytest

from instantmimic_b200 import synthetic
from instantmimic_b200.mjw_model import put_model

from helpers import run_cuda, run_oracle, scaled_err

pytestmark = pytest.mark.gpu

TOL = 1e-4


def _check(got, want, gctx=None, wctx=None):
    np.testing.assert_array_equal(got.solver_niter, want.solver_niter)
    np.testing.assert_array_equal(got.overflow, want.overflow)
    for w in range(want.nworld):
        n = min(int(want.nefc[w]), want.njmax)
        np.testing.assert_array_equal(got.efc.state[w, :n], want.efc.state[w, :n])
    for a, b in (
        (got.qacc, want.qacc),
        (got.qfrc_constraint, want.qfrc_constraint),
        (got.efc.Ma, want.efc.Ma),
    ):
        assert np.isfinite(a).all()
        assert scaled_err(a, b) < TOL
    mask = np.arange(want.njmax)[None, :] < np.minimum(want.nefc, want.njmax)[:, None]
    f_got = np.where(mask, got.efc.force, 0.0)
    f_want = np.where(mask, want.efc.force, 0.0)
    assert scaled_err(f_got, f_want) < TOL
    if gctx is not None:
        np.testing.assert_array_equal(gctx.quad_changed_count, wctx.quad_changed_count)
        np.testing.assert_array_equal(gctx.state_changed_count, wctx.state_changed_count)
        np.testing.assert_array_equal(gctx.search_unchanged, wctx.search_unchanged)
        if gctx.stats is not None:
            np.testing.assert_array_equal(gctx.stats, wctx.stats)  # passes, flips, factorisations, gradients
        for w in range(want.nworld):
            k = wctx.quad_changed_count[w]
            np.testing.assert_array_equal(gctx.quad_changed_ids[w, :k], wctx.quad_changed_ids[w, :k])


@pytest.mark.parametrize("name,nworld", [("humanoid", 256), ("snu", 64), ("g1", 32)])
@pytest.mark.parametrize("iters", [(4, 4), (50, 50)])
def test_named_workloads_match_oracle(oracle, cuda_device, name, nworld, iters):
    m, d, _ = synthetic.make_workload(
        name, nworld, seed=1, iterations=iters[0], ls_iterations=iters[1], rowless_fraction=0.1
    )
    want, wctx, wn = run_oracle(oracle, m, d)
    got, gctx, gn, _ = run_cuda(m, d, cuda_device)
    _check(got, want, gctx, wctx)
    assert gn[0] == wn[0]
    # bit-exactness is expected, not only tolerance
    assert np.array_equal(got.qacc, want.qacc)


@pytest.mark.parametrize("nv", [13, 16, 29, 31, 32, 33, 35, 56, 60, 61, 62, 70, 79])
@pytest.mark.parametrize("iters", [(4, 4), (100, 50)])
@pytest.mark.parametrize("warmstart_scale", [0.0, 50.0])
def test_layout_boundaries_match_oracle(oracle, cuda_device, nv, iters, warmstart_scale):
    """DOF counts at the tile / block-width boundaries of the reference's parity
    test (tests/test_mjw_newton_fusion.py:269-278)."""
    parent, body = synthetic.chain_tree(nv)
    m = put_model(parent, body_of_dof=body, iterations=iters[0], ls_iterations=iters[1])
    d, _ = synthetic.make_problem(m, 8, 256, seed=29, nefc_range=(8, 200), warmstart_scale=warmstart_scale)
    want, wctx, _ = run_oracle(oracle, m, d)
    got, gctx, _, _ = run_cuda(m, d, cuda_device)
    _check(got, want, gctx, wctx)


@pytest.mark.parametrize("chains,nv", [(2, 40), (3, 45), (4, 68), (5, 79)])
def test_rows_touching_few_dofs(oracle, cuda_device, chains, nv):
    parent, body = synthetic.multi_chain_tree(chains, nv)
    m = put_model(parent, body_of_dof=body, iterations=100, ls_iterations=50)
    d, _ = synthetic.make_problem(m, 8, 128, seed=4, nefc_range=(16, 128), warmstart_scale=50.0)
    want, wctx, _ = run_oracle(oracle, m, d)
    got, gctx, _, _ = run_cuda(m, d, cuda_device)
    _check(got, want, gctx, wctx)


def test_equality_and_friction_rows(oracle, cuda_device):
    parent, body = synthetic.chain_tree(35)
    m = put_model(parent, body_of_dof=body, iterations=100, ls_iterations=50)
    d, _ = synthetic.make_problem(m, 64, 96, seed=5, nefc_range=(20, 90), ne=6, nf=5)
    want, wctx, _ = run_oracle(oracle, m, d)
    got, gctx, _, _ = run_cuda(m, d, cuda_device)
    _check(got, want, gctx, wctx)


def test_rows_beyond_nefc_are_never_read(oracle, cuda_device):
    m, d, _ = synthetic.make_workload("humanoid", 64, seed=9)
    dp = copy.deepcopy(d)
    beyond = np.arange(d.njmax)[None, :] >= d.nefc[:, None]
    dp.efc.J[beyond] = np.nan
    dp.efc.D[beyond] = np.nan
    dp.efc.aref[beyond] = np.nan
    want, _, _ = run_oracle(oracle, m, d)
    got, _, _, _ = run_cuda(m, dp, cuda_device)
    _check(got, want)


def test_rowless_worlds_finish_at_the_smooth_acceleration(oracle, cuda_device):
    """tests/test_mjw_newton_fusion.py:349-415."""
    m, d, _ = synthetic.make_workload("humanoid", 64, seed=3)
    d.nefc[::2] = 0
    d.ne[::2] = 0
    d.nf[::2] = 0
    want, _, _ = run_oracle(oracle, m, d)
    got, _, _, _ = run_cuda(m, d, cuda_device)
    np.testing.assert_array_equal(got.qacc[::2], d.qacc_smooth[::2])
    np.testing.assert_array_equal(got.qfrc_constraint[::2], 0.0)
    np.testing.assert_array_equal(got.solver_niter[::2], 0)
    _check(got, want)


def test_world_order_changes_nothing_but_the_schedule(oracle, cuda_device):
    """With the context's world_order scratch the kernel takes worlds by descending row
    count; the scratch then holds a permutation sorted that way, and every result
    equals the index-order launch bit for bit."""
    m, d, _ = synthetic.make_workload("humanoid", 700, seed=9, rowless_fraction=0.1)
    a, actx, an, _ = run_cuda(m, d, cuda_device)
    b, bctx, bn, _ = run_cuda(m, d, cuda_device, ordered=False)
    order = actx.world_order
    assert bctx.world_order is None
    assert sorted(order.tolist()) == list(range(700))
    cls = (64 * (d.njmax - np.minimum(d.nefc[order], d.njmax).astype(np.int64))) // (d.njmax + 1)
    assert (np.diff(cls) >= 0).all() and d.nefc[order[0]] >= d.nefc.max() - 1 and d.nefc[order[-1]] == 0
    assert an[0] == bn[0]
    for name in ("qacc", "qfrc_constraint", "solver_niter", "overflow"):
        assert np.array_equal(getattr(a, name), getattr(b, name)), name
    assert np.array_equal(a.efc.Ma, b.efc.Ma)
    live = np.arange(d.njmax)[None, :] < np.minimum(d.nefc, d.njmax)[:, None]
    assert np.array_equal(a.efc.force[live], b.efc.force[live])
    assert np.array_equal(a.efc.state[live], b.efc.state[live])
    want, _, _ = run_oracle(oracle, m, d)
    assert np.array_equal(a.qacc, want.qacc)


@pytest.mark.parametrize("name,worlds,jpad", [("humanoid", 96, 48), ("humanoid", 96, 37), ("g1", 24, 37), ("snu", 24, 64)])
def test_padded_strides_are_read_from_the_arrays(oracle, cuda_device, name, worlds, jpad):
    """Upstream allocates efc.J with a third extent >= nv and may pad other arrays; the
    library takes every stride from the live arrays.  Padding is poisoned with NaN.
    jpad 37 makes the rows of J unaligned for the bulk copies (resident and streamed)."""
    import torch

    from instantmimic_b200 import mjw_model
    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, _ = synthetic.make_workload(name, worlds, seed=17, rowless_fraction=0.1)
    want, _, _ = run_oracle(oracle, m, d)
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(copy.deepcopy(d), cuda_device)
    nan = float("nan")

    def padded(t, extra):
        full = torch.full((*t.shape[:-1], t.shape[-1] + extra), nan if t.is_floating_point() else -7,
                          dtype=t.dtype, device=t.device)
        view = full[..., : t.shape[-1]]
        view.copy_(t)
        return view

    for field in ("qacc_smooth", "qacc_warmstart", "qfrc_smooth", "qacc", "qfrc_constraint"):
        setattr(dd, field, padded(getattr(dd, field), 6))
    dd.efc.Ma = padded(dd.efc.Ma, 6)
    dd.M = padded(dd.M, 3)
    for field in ("D", "aref", "frictionloss", "force", "state"):
        setattr(dd.efc, field, padded(getattr(dd.efc, field), 8))
    dd.efc.J = padded(dd.efc.J, jpad - m.nv)
    assert not dd.efc.J.is_contiguous() and dd.efc.J.stride() == (d.njmax * jpad, jpad, 1)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    ctx = scratch.solver_context  # its row / dof arrays share the strides of the data arrays
    for field in ("Jaref", "jv", "quad_changed_ids"):
        setattr(ctx, field, padded(getattr(ctx, field), 8))
    for field in ("search", "mv"):
        setattr(ctx, field, padded(getattr(ctx, field), 6))
    runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
    torch.cuda.synchronize()
    assert np.array_equal(dd.solver_niter.cpu().numpy(), want.solver_niter)
    assert np.array_equal(dd.qacc.cpu().numpy(), want.qacc)
    assert np.array_equal(dd.qfrc_constraint.cpu().numpy(), want.qfrc_constraint)
    live = np.arange(d.njmax)[None, :] < np.minimum(d.nefc, d.njmax)[:, None]
    assert np.array_equal(dd.efc.state.cpu().numpy()[live], want.efc.state[live])
    assert np.array_equal(dd.efc.force.cpu().numpy()[live], want.efc.force[live])


def test_iteration_limits_set_overflow_bits_and_warn_when_asked(oracle, cuda_device, capfd):
    """newton_fusion.py:284-293, newton_stages.py:435-439: hitting the iteration or
    line-search limit ORs the upstream overflow bits into d.overflow; the device prints
    the upstream messages only when opt.warn_overflow has the bit."""
    import torch

    m, d, _ = synthetic.make_workload("humanoid", 64, seed=23, iterations=1, ls_iterations=1)
    m.opt.warn_overflow = 3
    want, _, _ = run_oracle(oracle, m, d)
    got, _, _, _ = run_cuda(m, d, cuda_device)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(got.overflow, want.overflow)
    assert (got.overflow & 1).any() and (got.overflow & 2).any()
    out = capfd.readouterr().out
    assert "solver iterations limit reached - please increase iterations to 1" in out
    assert "linesearch iterations limit reached - please increase ls_iterations to 1" in out
    m.opt.warn_overflow = 0
    quiet, _, _, _ = run_cuda(m, d, cuda_device)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(quiet.overflow, want.overflow)
    assert "limit reached" not in capfd.readouterr().out


def test_repeated_solves_are_bitwise_identical(cuda_device):
    """tests/test_mjw_newton_fusion.py:290-346: eight solves, identical qacc."""
    m, d, _ = synthetic.make_workload("snu", 64, seed=29, iterations=3, ls_iterations=50)
    runs = [run_cuda(m, d, cuda_device)[0] for _ in range(8)]
    for r in runs[1:]:
        np.testing.assert_array_equal(runs[0].qacc, r.qacc)
        np.testing.assert_array_equal(runs[0].efc.force, r.efc.force)


def test_streamed_jacobian_variant_matches_oracle(oracle, cuda_device):
    """njmax large enough that J does not stay resident in shared memory."""
    m, d, _ = synthetic.make_sweep_point(64, 512, 24, seed=0, iterations=20, ls_iterations=20)
    want, wctx, _ = run_oracle(oracle, m, d)
    got, gctx, _, handles = run_cuda(m, d, cuda_device)
    from instantmimic_b200.mjw_kernels import newton_fusion

    md, dd, scratch = handles
    info = newton_fusion.solve_call(md, dd, scratch.solver_context, scratch.solver_nsolving, cache_on=scratch).launch_info()
    assert info.j_resident == 0
    _check(got, want, gctx, wctx)


def test_graph_capture_replay_matches_eager(cuda_device):
    """The solve is one stream-ordered launch and allocates nothing, so it can be
    captured and replayed (the reference runs inside CUDA graphs)."""
    import torch

    from instantmimic_b200 import mjw_model
    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, _ = synthetic.make_workload("humanoid", 128, seed=6)
    md = mjw_model.to_device(m, cuda_device)
    dd = mjw_model.to_device(d, cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
    torch.cuda.synchronize()
    eager = dd.qacc.clone()
    dd.qacc.zero_()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(eager, dd.qacc)


def test_torch_library_op_matches_the_direct_call(oracle, cuda_device):
    """torch.ops.imnewton.solve: the same launch behind a registered torch operator."""
    import torch

    from instantmimic_b200 import mjw_model, torch_ops
    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, _ = synthetic.make_workload("humanoid", 128, seed=14)
    want, _, _ = run_oracle(oracle, m, d)
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(d, cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    handle = torch_ops.register_model(md, scratch)
    torch_ops.solve_data(handle, dd)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(dd.qacc.cpu().numpy().view(np.uint32), want.qacc.view(np.uint32))
    np.testing.assert_array_equal(dd.solver_niter.cpu().numpy(), want.solver_niter)
    assert torch.library.opcheck is not None and hasattr(torch.ops.imnewton, "solve")


@pytest.mark.parametrize("name,worlds", [("humanoid", 200), ("snu", 48)])
def test_compact_jacobian_layout(oracle, cuda_device, name, worlds):
    """efc.J as only the nefc rows of each world (J_world_offset), resident and streamed
    kernels: same bits as the padded layout."""
    from instantmimic_b200 import mjw_model

    m, d, _ = synthetic.make_workload(name, worlds, seed=15, rowless_fraction=0.1)
    want, wctx, _ = run_oracle(oracle, m, d)
    got, gctx, _, _ = run_cuda(m, mjw_model.compact_jacobian(d), cuda_device)
    _check(got, want, gctx, wctx)
    np.testing.assert_array_equal(got.qacc.view(np.uint32), want.qacc.view(np.uint32))
