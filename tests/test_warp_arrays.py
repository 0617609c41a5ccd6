"""The host mirror fed with Warp-style arrays (tests/fake_warp.py): byte strides, dtype
classes without ``itemsize``, ``is_contiguous`` as a bool attribute, no torch methods.
This is the array type the reference's Model / Data / solver context hold, so these
tests are the drop-in check of the boundary.  CPU: struct building and the oracle on
the wrapped host buffers.  GPU: every public entry of the mirror on wrapped device
buffers, compared with the same call on plain torch tensors bit for bit."""

import copy
import ctypes

import numpy as np
import pytest

from instantmimic_b200 import arrays, binding, mjw_model, synthetic

from fake_warp import FakeWarpArray, wrap
from helpers import host_ctx, run_oracle


def test_array_helpers_on_warp_style_arrays():
    import torch

    t = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4)
    a = FakeWarpArray(t[:, :, :3])  # padded rows
    assert arrays.addr(a) == t.data_ptr()
    assert arrays.elem_strides(a) == (12, 4, 1)
    assert arrays.itemsize(a) == 4 and not arrays.is_contiguous(a)
    assert arrays.is_contiguous(FakeWarpArray(t)) and not arrays.is_device(a)
    flags = FakeWarpArray(torch.zeros(5, dtype=torch.bool))
    assert arrays.itemsize(flags) == 1 and arrays.elem_strides(flags) == (1,)

    class vec3(ctypes.Array):  # noqa: N801 - Warp's vector types are ctypes arrays
        _type_ = ctypes.c_float
        _length_ = 3

    v = FakeWarpArray(torch.zeros(4, 3), dtype=vec3)
    v.shape, v.strides = (4,), (12,)
    assert arrays.itemsize(v) == 12 and arrays.elem_strides(v) == (1,)

    class mystery:  # noqa: N801
        pass

    with pytest.raises(TypeError, match="element size"):
        arrays.itemsize(FakeWarpArray(torch.zeros(3), dtype=mystery))
    np.testing.assert_array_equal(arrays.to_host(a), t[:, :, :3].numpy())
    assert arrays.as_torch(FakeWarpArray(t)).data_ptr() == t.data_ptr()


def test_structs_from_warp_style_buffers_equal_the_numpy_ones(oracle):
    m, d, _ = synthetic.make_workload("humanoid", 6, seed=3)
    want, wctx, _ = run_oracle(oracle, m, d)
    d2 = copy.deepcopy(d)
    ctx = host_ctx(m, d2)
    mw, dw, cw = wrap(m), wrap(d2), wrap(ctx)
    ms, ds = binding.model_struct(mw), binding.data_struct(mw, dw)
    ref = binding.data_struct(m, d2)
    for name in ("dof_ld", "J_ld_world", "J_ld_row", "efc_ld", "M_ld", "nworld", "njmax"):
        assert getattr(ds, name) == getattr(ref, name), name
    assert ms.nM == m.nM and ds.efc_J == d2.efc.J.ctypes.data
    oracle.solve(mw, dw, cw, np.zeros(1, np.int32))  # the oracle reads and writes through the same structs
    np.testing.assert_array_equal(d2.qacc.view(np.uint32), want.qacc.view(np.uint32))
    np.testing.assert_array_equal(d2.solver_niter, want.solver_niter)
    np.testing.assert_array_equal(ctx.search.view(np.uint32), wctx.search.view(np.uint32))


def test_body_tree_stages_on_warp_style_vector_arrays(oracle):
    """mujoco-warp holds cinert, crb, cdof, cvel, ... as 2-D arrays of vector types (vec10,
    spatial_vector): shape (nworld, nbody), the components folded into the dtype.  The
    mirror must read them as the same bytes."""
    import torch

    from instantmimic_b200.mjw_kernels import tree_fusion

    def vector_type(n):
        return type(f"vec{n}", (ctypes.Array,), {"_type_": ctypes.c_float, "_length_": n})

    def folded(a):
        w = FakeWarpArray(torch.from_numpy(a), dtype=vector_type(a.shape[-1]))
        w.shape, w.strides, w.ndim = a.shape[:-1], tuple(s for s in a.strides[:-1]), a.ndim - 1
        return w

    m, d, _ = synthetic.make_workload("humanoid", 3, seed=2)
    synthetic.add_smooth_state(m, d, seed=4)
    want = copy.deepcopy(d)
    scratch = tree_fusion.create_tree_reduction_scratch(m, deterministic=True)
    oracle.com_vel(m, want, scratch)
    oracle.crb(m, want, scratch)
    oracle.rne(m, want, scratch)
    dw = copy.copy(d)
    for name in ("cinert", "crb", "cdof", "cdof_dot", "cvel", "cacc", "cfrc_int"):
        setattr(dw, name, folded(getattr(d, name)))
    dw.qvel, dw.M, dw.qfrc_bias = FakeWarpArray(torch.from_numpy(d.qvel)), FakeWarpArray(torch.from_numpy(d.M)), \
        FakeWarpArray(torch.from_numpy(d.qfrc_bias))
    mw = wrap(m)
    mw.body_tree = m.body_tree  # a list of arrays on the reference side too
    sw = tree_fusion.create_tree_reduction_scratch(mw, deterministic=True)
    assert tree_fusion._per_body(dw.cinert, 3, 14, 10, "d.cinert") == d.cinert.ctypes.data
    oracle.com_vel(mw, dw, sw)
    oracle.crb(mw, dw, sw)
    oracle.rne(mw, dw, sw)
    for name in ("cvel", "cdof_dot", "crb", "M", "cacc", "cfrc_int", "qfrc_bias"):
        np.testing.assert_array_equal(getattr(d, name), getattr(want, name), err_msg=name)
    with pytest.raises(ValueError, match="d.cvel"):
        tree_fusion._per_body(folded(d.cvel[:, :5]), 3, 14, 6, "d.cvel")


# ---------------------------------------------------------------------------- GPU


@pytest.mark.gpu
def test_solve_with_scratch_on_warp_style_buffers(oracle, cuda_device):
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, _ = synthetic.make_workload("humanoid", 96, seed=7, rowless_fraction=0.1)
    want, _, _ = run_oracle(oracle, m, d)
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(copy.deepcopy(d), cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device, with_matrices=True)
    mw, dw = wrap(md), wrap(dd)
    sw = copy.copy(scratch)
    sw.solver_context = wrap(scratch.solver_context)
    sw.solver_nsolving = wrap(scratch.solver_nsolving)
    runtime.solve_with_scratch(mw, dw, sw, use_optimized_kernel=True)
    torch.cuda.synchronize()
    got = mjw_model.to_host(dd)
    np.testing.assert_array_equal(got.qacc.view(np.uint32), want.qacc.view(np.uint32))
    np.testing.assert_array_equal(got.solver_niter, want.solver_niter)
    # worlds without rows are finished before the loop and never count down (as in the reference)
    assert int(scratch.solver_nsolving.item()) == int((d.nefc == 0).sum())
    # the sparse plan is installed on, and its counter read from, a Warp-style context
    groups = [[b] for b in range(1, len(m.body_dofadr))]
    assert runtime.refresh_sparse_hessian(mw, dw, sw, groups, cuda_device) == "enabled"
    runtime.solve_with_scratch(mw, dw, sw, use_optimized_kernel=True)
    torch.cuda.synchronize()
    runtime.check_sparse_hessian_violations(sw)
    np.testing.assert_array_equal(dd.solver_niter.cpu().numpy(), want.solver_niter)
    # whole-batch hand-off and M v through the same objects
    sw.constraint_free = True
    runtime.solve_with_scratch(mw, dw, sw, use_optimized_kernel=True)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(dd.qacc.cpu().numpy(), d.qacc_smooth)
    line = runtime.log_kernel_selection(mw, dw, sw)
    assert "rowless hand-off" in line and "M factor/solve: tree L'DL" in line


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["humanoid", "chain31"])
def test_m_factor_solve_on_warp_style_buffers(cuda_device, name):
    """Tree L'DL, blocked dense (fresh and retained factor), multi-RHS and the small
    single-tile path, on Warp-style buffers vs plain tensors bit for bit and vs
    numpy.linalg.solve."""
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime
    from instantmimic_b200.mjw_kernels import indexed_factor

    if name == "humanoid":
        parent, body = synthetic.humanoid_tree()
    else:
        parent, body = synthetic.chain_tree(31)  # a 31-dof chain: too long for the tree plan, below the blocked kernel
    m = mjw_model.put_model(parent, body_of_dof=body)
    d, Mdense = synthetic.make_problem(m, 37, 8, seed=9)
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(d, cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    if name == "chain31":
        assert scratch.tree_factor_solve is None and scratch.dense_factor_solve is None
        assert scratch.tile_factor_solve is not None
    mw, dw = wrap(md), wrap(dd)
    exact = np.linalg.solve(Mdense.astype(np.float64), d.qfrc_smooth.astype(np.float64)[..., None])[..., 0]

    def solve(m_, d_, **kw):
        x = torch.zeros_like(dd.qacc_smooth)
        xa = FakeWarpArray(x) if m_ is mw else x
        runtime._factor_solve_i_dense(m_, d_, d_.M, xa, d_.qfrc_smooth, scratch.dense_factor_solve,
                                      tree_factor_solve=scratch.tree_factor_solve, **kw)
        torch.cuda.synchronize()
        return x.cpu().numpy()

    plain, warp = solve(md, dd), solve(mw, dw)
    np.testing.assert_array_equal(plain.view(np.uint32), warp.view(np.uint32))
    np.testing.assert_allclose(warp, exact, rtol=2e-4, atol=2e-5 * np.abs(exact).max())
    if scratch.dense_factor_solve is not None:
        U = torch.zeros_like(scratch.dense_factor_solve.U)
        kept = solve(mw, dw, retain_factor=True, factor_workspace=FakeWarpArray(U))
        np.testing.assert_allclose(kept, exact, rtol=2e-4, atol=2e-5 * np.abs(exact).max())
        # three right-hand sides, factor reuse, one inactive world
        bs = scratch.dense_factor_solve
        y3 = torch.randn(37, m.nv, 3, device=cuda_device)
        act = torch.ones(37, dtype=torch.int32, device=cuda_device)
        act[5] = 0
        x3 = torch.full_like(y3, 7.0)
        indexed_factor.factor_multi_solve(bs, dw.M, FakeWarpArray(y3), FakeWarpArray(act), FakeWarpArray(U),
                                          FakeWarpArray(x3), 3)
        x3b = torch.full_like(y3, 7.0)
        indexed_factor.multi_solve(bs, FakeWarpArray(U), FakeWarpArray(y3), FakeWarpArray(act), FakeWarpArray(x3b), 3)
        torch.cuda.synchronize()
        assert torch.equal(x3, x3b) and bool((x3[5] == 7.0).all())
        ex3 = np.linalg.solve(Mdense.astype(np.float64), y3.cpu().numpy().astype(np.float64))
        live = np.arange(37) != 5
        np.testing.assert_allclose(x3.cpu().numpy()[live], ex3[live], rtol=2e-3, atol=2e-4 * np.abs(ex3).max())
