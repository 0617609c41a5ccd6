"""The reference's own CUDA text as the arbiter of the factor arithmetic.

tests/golden/ref_snippets.npz holds inputs and outputs of the reference's generated CUDA
for the sparse-pattern Hessian factor and the tree L'DL of M (compiled with nvcc, run on a
B200; tests/golden/make_ref_snippet_golden.py, oracle/ref_snippets.py).  The CPU oracle
and the CUDA kernels must reproduce every output bit for bit."""

from pathlib import Path

import numpy as np
import pytest

from instantmimic_b200 import synthetic
from instantmimic_b200.mjw_kernels import sparse_hessian, tree_ldl
from oracle import oracle, ref_snippets

GOLDEN = Path(__file__).parent / "golden" / "ref_snippets.npz"
# the cases the committed file holds (written by tests/golden/make_ref_snippet_golden.py)
CASES = [str(name) for name in np.load(GOLDEN)["names"]]


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def model_of(name):
    """Model and body groups of a case: the list the golden file was made from."""
    for case, m, groups in ref_snippets.case_models():
        if case == name:
            return m, groups
    raise KeyError(name)


def inputs(g, name):
    keys = ("J", "D", "state", "state2", "nefc", "M", "ids", "count", "uni", "H", "grad", "y")
    return {k: g[f"{name}/in/{k}"] for k in keys}


def check(g, name, tag, U, search, sd, dec, nfac, parts):
    """Compare the meaningful part of U (the reference leaves the rest untouched) and the
    solve's results."""
    ref_U = g[f"{name}/{tag}/U"].reshape(U.shape[0], -1)
    got_U = U.reshape(U.shape[0], -1)
    for lo, hi in parts:
        np.testing.assert_array_equal(got_U[:, lo:hi], ref_U[:, lo:hi], err_msg=f"{name}/{tag}/U[{lo}:{hi}]")
    np.testing.assert_array_equal(search, g[f"{name}/{tag}/search"], err_msg=f"{name}/{tag}/search")
    np.testing.assert_array_equal(sd, g[f"{name}/{tag}/search_dot"], err_msg=f"{name}/{tag}/search_dot")
    np.testing.assert_array_equal(dec, g[f"{name}/{tag}/decrement"], err_msg=f"{name}/{tag}/decrement")


def test_golden_file_covers_the_bench_models_and_names_known_cases(golden):
    known = [name for name, _, _ in ref_snippets.case_models()]
    assert set(CASES) <= set(known)
    assert {"humanoid", "snu", "g1", "limbs64"} <= set(CASES)


@pytest.mark.parametrize("name", CASES)
def test_oracle_tree_ldl_equals_the_reference_code(golden, name):
    m, _ = model_of(name)
    x = inputs(golden, name)
    st = tree_ldl.tree_ldl_structure(np.asarray(m.M_rowadr), np.asarray(m.M_rownnz), np.asarray(m.M_colind))
    plan = tree_ldl.best_tree_ldl_plan(*st)
    got = oracle.tree_ldl_solve(st, plan, x["M"], x["y"])
    np.testing.assert_array_equal(got, golden[f"{name}/tree/x"])


@pytest.mark.parametrize("name", CASES)
def test_oracle_fused_stages_equal_the_reference_code(golden, name):
    m, groups = model_of(name)
    x = inputs(golden, name)
    plan = sparse_hessian.build_plan(m, groups, 32 if m.nv_pad < 64 else 64, "fused")
    st = sparse_hessian.host_struct(plan)
    nfac, nv, P = plan.nfac, m.nv, m.nv_pad
    W = x["J"].shape[0]
    U = np.zeros((W, P, P), np.float32)
    search, sd, dec = oracle.sparse_stage(st, 3, x, x["grad"][0], U, nv)
    check(golden, name, "init", U, search, sd, dec, nfac, [(0, 2 * nfac + nv), (P * P - 1, P * P)])
    x2 = dict(x, state=x["state2"])
    search, sd, dec = oracle.sparse_stage(st, 0, x2, x["grad"][1], U, nv)
    check(golden, name, "update", U, search, sd, dec, nfac, [(0, nfac), (P * P - 1, P * P)])
    U = golden[f"{name}/init/U"].copy()
    search, sd, dec = oracle.sparse_stage(st, 1, x, x["grad"][2], U, nv)
    check(golden, name, "resident", U, search, sd, dec, nfac, [(0, 2 * nfac + nv)])


@pytest.mark.parametrize("name", CASES)
def test_oracle_nonfused_equals_the_reference_code(golden, name):
    m, groups = model_of(name)
    x = inputs(golden, name)
    plan = sparse_hessian.build_plan(m, groups, 64, "nonfused")
    st = sparse_hessian.host_struct(plan)
    nfac, nv, P = plan.nfac, m.nv, m.nv_pad
    W = x["H"].shape[0]
    U = np.zeros((W, P, P), np.float32)
    search, sd, dec = oracle.sparse_factor_nonfused(st, x["grad"][0], x["H"], U, nv)
    check(golden, name, "nonfused_factor", U, search, sd, dec, nfac, [(0, nfac + nv)])
    search, sd, dec = oracle.sparse_factor_nonfused(st, x["grad"][1], x["H"], U, nv, quad_changed=np.zeros(W, np.int32),
                                                    skip_unchanged=True)
    check(golden, name, "nonfused_solve", U, search, sd, dec, nfac, [(0, nfac + nv)])


# ---- CUDA -----------------------------------------------------------------------------


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_cuda_tree_ldl_equals_the_reference_code(golden, name):
    import torch

    from instantmimic_b200 import mjw_model

    dev = torch.device("cuda:0")
    m, _ = model_of(name)
    x = inputs(golden, name)
    md = mjw_model.to_device(m, dev)
    for generate in (True, False):
        scratch = tree_ldl.create_tree_factor_solve_scratch(md, dev, generate=generate)
        assert scratch is not None
        M, y = torch.from_numpy(x["M"]).to(dev), torch.from_numpy(x["y"]).to(dev)
        out = torch.zeros_like(y)
        tree_ldl.tree_factor_solve(scratch, M, out, y)
        np.testing.assert_array_equal(out.cpu().numpy(), golden[f"{name}/tree/x"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_cuda_nonfused_equals_the_reference_code(golden, name):
    import torch
    from types import SimpleNamespace

    dev = torch.device("cuda:0")
    m, groups = model_of(name)
    x = inputs(golden, name)
    plan = sparse_hessian.upload(sparse_hessian.build_plan(m, groups, 64, "nonfused"), dev)
    nfac, nv, P = plan.nfac, m.nv, m.nv_pad
    W = x["H"].shape[0]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    ctx = SimpleNamespace(
        done=torch.zeros(W, dtype=torch.uint8, device=dev), grad=t(x["grad"][0]), h=t(x["H"]),
        quad_changed_count=torch.ones(W, dtype=torch.int32, device=dev),
        state_changed_count=torch.ones(W, dtype=torch.int32, device=dev), hfactor=torch.zeros(W, P, P, device=dev),
        search=torch.zeros(W, nv, device=dev), search_dot=torch.zeros(W, device=dev),
        newton_decrement=torch.zeros(W, device=dev))
    sparse_hessian.nonfused_factor_solve(plan, ctx, W)
    torch.cuda.synchronize()
    check(golden, name, "nonfused_factor", ctx.hfactor.cpu().numpy(), ctx.search.cpu().numpy(),
          ctx.search_dot.cpu().numpy(), ctx.newton_decrement.cpu().numpy(), nfac, [(0, nfac + nv)])
    ctx.grad = t(x["grad"][1])
    ctx.quad_changed_count.zero_()
    sparse_hessian.nonfused_factor_solve(plan, ctx, W, skip_unchanged=True)
    torch.cuda.synchronize()
    check(golden, name, "nonfused_solve", ctx.hfactor.cpu().numpy(), ctx.search.cpu().numpy(),
          ctx.search_dot.cpu().numpy(), ctx.newton_decrement.cpu().numpy(), nfac, [(0, nfac + nv)])
