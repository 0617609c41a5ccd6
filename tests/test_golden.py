"""Committed fixtures (tests/golden, written by tests/golden/make_golden.py): the CPU
oracle must still reproduce them bit for bit, and so must the CUDA kernels.  Also the
round trip of the solver-state format the fixtures are stored in."""

import copy
from pathlib import Path

import numpy as np
import pytest

from instantmimic_b200 import solver_state, synthetic
from instantmimic_b200.mjw_kernels import indexed_factor, sparse_hessian, tree_ldl
from instantmimic_b200.mjw_model import put_model

from helpers import host_ctx, run_cuda, run_oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
NEWTON = sorted(p.name for p in GOLDEN.glob("newton_*.npz"))


def _bits(a, b, what):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape, what
    assert np.array_equal(np.ascontiguousarray(a).view(np.uint8), np.ascontiguousarray(b).view(np.uint8)), what


def _check_solution(d, out, what):
    live = np.arange(d.njmax)[None, :] < np.minimum(d.nefc, d.njmax)[:, None]
    for name in ("qacc", "qfrc_constraint", "solver_niter", "overflow"):
        _bits(getattr(d, name), getattr(out, name), f"{what}: {name}")
    _bits(d.efc.Ma, out.efc_Ma, f"{what}: efc.Ma")
    _bits(np.where(live, d.efc.force, 0), np.where(live, out.efc_force, 0), f"{what}: efc.force")
    _bits(np.where(live, d.efc.state, 0), np.where(live, out.efc_state, 0), f"{what}: efc.state")


def test_fixture_folder_is_complete():
    assert NEWTON == ["newton_at_rest.npz", "newton_eq_friction.npz", "newton_humanoid.npz", "newton_snu.npz"]
    assert (GOLDEN / "msolve_humanoid.npz").exists() and (GOLDEN / "make_golden.py").exists()


@pytest.mark.parametrize("name", NEWTON)
def test_oracle_reproduces_newton_fixture(oracle, name):
    m, d, out, ctx = solver_state.load(GOLDEN / name)
    got, gctx, _ = run_oracle(oracle, m, d)
    _check_solution(got, out, name)
    solved = d.nefc > 0
    for field in ("search", "grad", "alpha", "quad_changed_count", "state_changed_count", "search_unchanged"):
        _bits(getattr(gctx, field)[solved], getattr(ctx, field)[solved], f"{name}: ctx.{field}")


def test_oracle_reproduces_sparse_factor_fixture(oracle):
    e = solver_state.read(GOLDEN / "newton_humanoid.npz")
    m, d, _, _ = solver_state.load(GOLDEN / "newton_humanoid.npz")
    groups = [[int(b)] for b in e["sparse/groups"]]
    plan = sparse_hessian.build_plan(m, groups, 32, "fused")
    d2 = copy.deepcopy(d)
    oracle.solve(m, d2, host_ctx(m, d2), np.zeros(1, np.int32), sparse_plan_struct=sparse_hessian.host_struct(plan))
    _bits(d2.qacc, e["sparse/qacc"], "sparse qacc")
    _bits(d2.solver_niter, e["sparse/solver_niter"], "sparse niter")


def test_oracle_reproduces_msolve_fixture(oracle):
    z = np.load(GOLDEN / "msolve_humanoid.npz")
    parent, body = synthetic.humanoid_tree()
    m = put_model(parent, body_of_dof=body)
    structure = tree_ldl.tree_ldl_structure(m.M_rowadr, m.M_rownnz, m.M_colind)
    for groups in (1, 4):
        plan = tree_ldl.plan_tree_ldl(*structure, groups)
        _bits(oracle.tree_ldl_solve(structure, plan, z["M"], z["y"]), z[f"x_tree_{groups}"], f"tree {groups}")
    pad = indexed_factor._round_up(m.nv, 16)
    layout = indexed_factor.block_major_layout(indexed_factor.dense_index_table(m), pad, m.nM)
    x, U = oracle.blocked_dense_factor_solve(m.nv, pad, layout, indexed_factor.pad_identity(m.nv, pad), z["M"], z["y3"])
    _bits(x, z["x_blocked"], "blocked x")
    _bits(U, z["U"], "blocked U")


def test_state_file_round_trip_and_capture(oracle, tmp_path):
    """dump -> load gives containers on which the solve gives the same bits; capture()
    around a solve callable records inputs and results of its first calls."""
    m, d, _ = synthetic.make_workload("humanoid", 5, seed=21)
    path = solver_state.dump(tmp_path / "state.npz", m, d)
    m2, d2, out, ctx = solver_state.load(path)
    assert out is None and ctx is None
    a, _, _ = run_oracle(oracle, m, d)
    b, _, _ = run_oracle(oracle, m2, d2)
    _bits(a.qacc, b.qacc, "round trip qacc")
    _bits(a.solver_niter, b.solver_niter, "round trip niter")

    def solve(m_, d_, scratch, *, use_optimized_kernel=False):
        oracle.solve(m_, d_, scratch.solver_context, np.zeros(1, np.int32))

    from types import SimpleNamespace

    wrapped = solver_state.capture(solve, tmp_path / "cap", limit=2)
    for _ in range(3):
        dd = copy.deepcopy(d)
        wrapped(m, dd, SimpleNamespace(solver_context=host_ctx(m, dd)), use_optimized_kernel=True)
    files = sorted((tmp_path / "cap").glob("*.npz"))
    assert [f.name for f in files] == ["solve_0000.npz", "solve_0001.npz"]
    m3, d3, out3, ctx3 = solver_state.load(files[0])
    _check_solution(a, out3, "captured")
    assert ctx3 is not None and ctx3.search.shape == (5, m.nv)
    with pytest.raises(ValueError, match="not a imnewton-solver-state"):
        np.savez(tmp_path / "other.npz", format=np.asarray("x"))
        solver_state.read(tmp_path / "other.npz")


# ---------------------------------------------------------------------------- GPU


@pytest.mark.gpu
@pytest.mark.parametrize("name", NEWTON)
def test_cuda_reproduces_newton_fixture(cuda_device, name):
    m, d, out, ctx = solver_state.load(GOLDEN / name)
    got, gctx, _, _ = run_cuda(m, d, cuda_device)
    _check_solution(got, out, name)
    solved = d.nefc > 0
    for field in ("quad_changed_count", "state_changed_count", "search_unchanged"):
        _bits(getattr(gctx, field)[solved], getattr(ctx, field)[solved].astype(getattr(gctx, field).dtype),
              f"{name}: ctx.{field}")


@pytest.mark.gpu
def test_cuda_reproduces_sparse_and_msolve_fixtures(cuda_device):
    import torch

    from instantmimic_b200 import mjw_model
    from instantmimic_b200 import mjw_step_optimized as runtime

    e = solver_state.read(GOLDEN / "newton_humanoid.npz")
    m, d, _, _ = solver_state.load(GOLDEN / "newton_humanoid.npz")
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(d, cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device, with_matrices=True)
    assert runtime.refresh_sparse_hessian(md, dd, scratch, [[int(b)] for b in e["sparse/groups"]], cuda_device) == "enabled"
    runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
    torch.cuda.synchronize()
    _bits(dd.qacc.cpu().numpy(), e["sparse/qacc"], "sparse qacc")
    _bits(dd.solver_niter.cpu().numpy(), e["sparse/solver_niter"], "sparse niter")

    z = np.load(GOLDEN / "msolve_humanoid.npz")
    parent, body = synthetic.humanoid_tree()
    mm = put_model(parent, body_of_dof=body)
    structure = tree_ldl.tree_ldl_structure(mm.M_rowadr, mm.M_rownnz, mm.M_colind)
    Mt, yt = torch.from_numpy(z["M"]).to(cuda_device), torch.from_numpy(z["y"]).to(cuda_device)
    for groups in (1, 4):
        sc = tree_ldl.compile_plan(structure, tree_ldl.plan_tree_ldl(*structure, groups), cuda_device)
        x = torch.zeros_like(yt)
        tree_ldl.tree_factor_solve(sc, Mt, x, yt)
        torch.cuda.synchronize()
        _bits(x.cpu().numpy(), z[f"x_tree_{groups}"], f"tree {groups}")
    md2 = mjw_model.to_device(mm, cuda_device)
    dd2 = mjw_model.to_device(mjw_model.make_data(mm, 5, 4), cuda_device)
    bs = indexed_factor.create_blocked_dense_factor_solve_scratch(md2, dd2, cuda_device)
    y3 = torch.from_numpy(z["y3"]).to(cuda_device)
    x3 = torch.zeros_like(y3)
    U = torch.zeros((5, bs.pad, bs.pad), dtype=torch.float32, device=cuda_device)
    indexed_factor.factor_multi_solve(bs, Mt, y3, torch.ones(5, dtype=torch.int32, device=cuda_device), U, x3, 3)
    torch.cuda.synchronize()
    _bits(x3.cpu().numpy(), z["x_blocked"], "blocked x")
    _bits(U.cpu().numpy(), z["U"], "blocked U")
