"""Static-pattern sparse L'DL of the Hessian: symbolic factor, tables, gates (CPU)
and the numeric kernels (GPU).  The CPU checks restate the reference's self-contained
ones (tests/test_mjw_sparse_hessian.py:73-98, 199-291) on synthetic kinematic trees."""

import copy
from types import SimpleNamespace

import numpy as np
import pytest

from instantmimic_b200 import synthetic
from instantmimic_b200.mjw_kernels import sparse_hessian
from instantmimic_b200.mjw_model import put_model


def test_symbolic_fill_contains_the_numeric_factor():
    rng = np.random.default_rng(3)
    for _ in range(5):
        n = 30
        adj = [set() for _ in range(n)]
        for _ in range(60):
            a, b = rng.integers(0, n, 2)
            if a != b:
                adj[a].add(int(b))
                adj[b].add(int(a))
        rowstruct, colstruct, levels = sparse_hessian._symbolic(adj)
        H = np.zeros((n, n))
        for a in range(n):
            for b in adj[a]:
                H[a, b] = rng.normal()
        H = (H + H.T) / 2 + 2 * n * np.eye(n)
        L = np.linalg.cholesky(H)
        for j in range(n):
            for i in range(j + 1, n):
                if abs(L[i, j]) > 1e-12:
                    assert i in colstruct[j], (i, j)
        level = {k: lv for lv, cols in enumerate(levels) for k in cols}
        for i in range(n):
            assert all(level[k] < level[i] for k in rowstruct[i])


def _legged_model():
    """Torso (6) + two 6-dof legs + two 3-dof arms + two free boxes: nv 36, nv_pad 48
    (the shape of tests/test_mjw_sparse_hessian.py:14-49).  Body ids: 1 torso, 2-4 left
    leg (thigh, shin, foot), 5-7 right leg, 8-9 left arm, 10-11 right arm, 12 box A,
    13 box B."""
    joints = [(6, -1), (3, 0), (1, 1), (2, 2), (3, 0), (1, 4), (2, 5), (1, 0), (2, 7), (1, 0), (2, 9),
              (6, -1), (6, -1)]
    parent, body = synthetic._tree_from_joints(joints)
    return put_model(parent, body_of_dof=body)


FOOT_L, FOOT_R, FORE_R, BOX_A, BOX_B = 4, 7, 11, 12, 13


def test_pattern_couples_tree_groups_and_collision_pairs():
    m = _legged_model()
    m.geom_bodyid = np.array([0, FOOT_R, BOX_B], np.int32)
    m.nxn_geom_pair_filtered = np.array([[1, 2]], np.int32)  # right foot vs box B
    adj = sparse_hessian.hessian_pattern(m, [[FOOT_L, BOX_A]])
    dofs = lambda b: list(range(m.body_dofadr[b], m.body_dofadr[b] + m.body_dofnum[b]))  # noqa: E731
    torso, foot_l, foot_r, arm_l = dofs(1), dofs(FOOT_L), dofs(FOOT_R), dofs(8)
    assert set(torso) <= adj[foot_l[0]]  # tree ancestry
    assert arm_l[0] not in adj[foot_l[0]]  # sibling branches stay uncoupled
    assert set(foot_l) <= adj[dofs(BOX_A)[0]]  # declared group
    assert foot_r[0] not in adj[dofs(BOX_A)[0]]
    assert set(foot_r) <= adj[dofs(BOX_B)[0]]  # collision candidate pair


def _body_dofs(m, b):
    return list(range(int(m.body_dofadr[b]), int(m.body_dofadr[b]) + int(m.body_dofnum[b])))


def test_equalities_and_site_welds_couple_their_bodies():
    """tests/test_mjw_sparse_hessian.py:100-150: a connect between the two boxes, a weld
    given through two sites, and a joint equality between two joints' first dofs."""
    m = _legged_model()
    m.neq = 3
    m.eq_type = np.array([sparse_hessian.EQ_CONNECT, sparse_hessian.EQ_WELD, sparse_hessian.EQ_JOINT], np.int32)
    m.eq_obj1id = np.array([BOX_A, 0, 2], np.int32)   # body, site, joint ids
    m.eq_obj2id = np.array([BOX_B, 1, 5], np.int32)
    m.eq_objtype = np.array([1, sparse_hessian.OBJ_SITE, 3], np.int32)
    m.site_bodyid = np.array([FOOT_L, FORE_R], np.int32)
    m.jnt_dofadr = np.array([0, 6, 9, 10, 12, 15, 16], np.int32)
    adj = sparse_hessian.hessian_pattern(m, [])
    a, b = _body_dofs(m, BOX_A), _body_dofs(m, BOX_B)
    assert set(b) <= adj[a[0]] and set(a) <= adj[b[3]]
    foot, fore = _body_dofs(m, FOOT_L), _body_dofs(m, FORE_R)
    assert set(fore) <= adj[foot[0]]                      # the weld's sites sit on these bodies
    assert set(_body_dofs(m, 10)) <= adj[foot[0]]         # ... and the fore-arm's chain comes along
    assert 15 in adj[9] and 16 not in adj[9]              # joint equality: first dofs only
    m.eq_type[2] = 3
    with pytest.raises(ValueError, match="no coupling rule"):
        sparse_hessian.hessian_pattern(m, [])


def test_flex_couplings():
    """sparse_hessian.py:121-170 / tests/test_mjw_sparse_hessian.py:174-188: every element
    couples its vertices' bodies; a geom that may collide with the flex joins each
    element; an interpolated flex couples all its nodes; flexes that may collide with
    each other are coupled whole."""
    # six free bodies (6 dofs each): bodies 1-4 carry the vertices of flex 0 (two
    # triangles 0-1-2 and 1-2-3), bodies 5-6 are the nodes of the interpolated flex 1
    joints = [(6, -1)] * 6 + [(6, -1)]  # body 7: a free box with a geom
    parent, body = synthetic._tree_from_joints(joints)
    m = put_model(parent, body_of_dof=body)
    m.nflex = 2
    m.flex_vertadr, m.flex_vertnum = np.array([0, 4], np.int32), np.array([4, 0], np.int32)
    m.flex_vertbodyid = np.array([1, 2, 3, 4], np.int32)
    m.flex_elemadr, m.flex_elemnum = np.array([0, 2], np.int32), np.array([2, 1], np.int32)
    m.flex_elemdataadr, m.flex_dim = np.array([0, 6], np.int32), np.array([2, 2], np.int32)
    m.flex_elem = np.array([0, 1, 2, 1, 2, 3, 0, 0, 0], np.int32)
    m.flex_interp = np.array([0, 1], np.int32)
    m.flex_nodeadr, m.flex_nodenum = np.array([0, 0], np.int32), np.array([0, 2], np.int32)
    m.flex_nodebodyid = np.array([5, 6], np.int32)
    m.flex_contype, m.flex_conaffinity = np.array([1, 0], np.int32), np.array([2, 0], np.int32)
    m.flex_selfcollide = np.array([0, 0], np.int32)
    m.ngeom = 1
    m.geom_contype, m.geom_conaffinity = np.array([2], np.int32), np.array([0], np.int32)
    m.geom_bodyid = np.array([7], np.int32)
    adj = sparse_hessian.hessian_pattern(m, [])
    d = lambda b: _body_dofs(m, b)  # noqa: E731
    assert set(d(2)) | set(d(3)) <= adj[d(1)[0]]       # first triangle
    assert set(d(4)) <= adj[d(2)[0]]                   # second triangle
    assert d(4)[0] not in adj[d(1)[0]]                 # vertices 0 and 3 share no element
    assert set(d(6)) <= adj[d(5)[0]]                   # interpolated flex: all nodes
    assert set(d(1)) | set(d(4)) <= adj[d(7)[0]]       # the geom's body meets every element
    assert d(5)[0] not in adj[d(7)[0]] and d(5)[0] not in adj[d(1)[0]]
    m.flex_selfcollide[0] = 1
    m.flex_conaffinity[0] = 3                          # flex 0 may now collide with itself
    adj = sparse_hessian.hessian_pattern(m, [])
    assert set(d(4)) <= adj[d(1)[0]]                   # coupled whole


def test_tendon_gate_reads_the_model_arrays():
    """sparse_hessian.py:729-733: tendons are fine unless one has a limit or friction loss."""
    m = _legged_model()

    class _Dev(np.ndarray):
        device = SimpleNamespace(is_cuda=True)

    m.body_parentid = m.body_parentid.view(_Dev)
    ctx = SimpleNamespace()
    groups = [[FOOT_L], [FOOT_R]]
    m.ntendon = 2
    plan, reason = sparse_hessian.plan_for_model(m, ctx, groups, 32)
    assert plan is None and "tendon" in reason            # arrays absent: refused
    m.tendon_limited_adr = np.zeros(0, np.int32)
    m.tendon_frictionloss = np.zeros(2, np.float32)
    plan, reason = sparse_hessian.plan_for_model(m, ctx, groups, 32)
    assert plan is not None and reason == "enabled"
    m.tendon_frictionloss = np.array([0.0, 0.3], np.float32)
    assert sparse_hessian.plan_for_model(m, ctx, groups, 32)[0] is None
    m.tendon_frictionloss = np.zeros(2, np.float32)
    m.tendon_limited_adr = np.array([1], np.int32)
    assert sparse_hessian.plan_for_model(m, ctx, groups, 32)[0] is None


def _run_tables(plan, H, g):
    """Execute the factor and solve tables in numpy float64, each level as one
    parallel sweep over a snapshot, asserting no level writes what another lane of
    it reads or writes."""
    T = {k: v.astype(np.int64) for k, v in plan.tables.items()}
    nv, nfac = plan.nv, plan.nfac
    N, iD = np.zeros(plan.nslots), np.zeros(nv)
    pair = T["pair"].reshape(nv, nv)
    for s in range(nfac):
        a, b = T["s_a"][s], T["s_b"][s]
        assert pair[a, b] == s
        N[s] = H[a, b]
    words = (nv + 31) // 32
    for a in range(nv):
        for b in range(a, nv):
            in_mask = (T["pmask"][a * words + b // 32] >> (b % 32)) & 1
            assert bool(in_mask) == (pair[a, b] >= 0 or a == b)
            assert H[a, b] == 0.0 or pair[a, b] >= 0
    orig = T["orig"]
    N[nfac:] = g[orig]
    LP, ES, EC, RP, RAB, RKL = (T[k] for k in ("lvl_ptr", "ent_slot", "ent_col", "run_ptr", "run_ab", "run_kl"))
    for lvl in range(len(LP) - 1):
        n0, d0 = N.copy(), iD.copy()
        written, read = set(), set()
        for e in range(LP[lvl], LP[lvl + 1]):
            v = 0.0
            for r in range(RP[e], RP[e + 1]):
                a, b, k, ln = RAB[r] & 0xFFFF, RAB[r] >> 16, RKL[r] & 0xFFFF, RKL[r] >> 16
                v += float(np.sum(n0[a : a + ln] * n0[b : b + ln] * d0[k : k + ln]))
                read |= {*range(a, a + ln), *range(b, b + ln), *range(-k - ln, -k)}
            assert ES[e] not in written
            written.add(ES[e])
            N[ES[e]] = n0[ES[e]] - v
            if EC[e] >= 0:
                iD[EC[e]] = 1.0 / N[ES[e]]
                written.add(-1 - EC[e])
        assert not written & read
    BL, BS, BI, BJ = (T[k] for k in ("b_lvl", "b_slot", "b_src", "b_dst"))
    for lvl in range(len(BL) - 1):
        z = N[nfac:].copy()
        src, dst = set(), set()
        for p in range(BL[lvl], BL[lvl + 1]):
            i, j = BI[p], BJ[p]
            assert j not in dst, "two pushes to one unknown in a level"
            src.add(i)
            dst.add(j)
            N[nfac + j] = z[j] - N[BS[p]] * (z[i] * iD[i])
        assert not src & dst
    x = np.zeros(nv)
    x[orig] = N[nfac:] * iD
    return x


def test_tables_solve_h_without_a_race_inside_any_level():
    m = _legged_model()
    cases = [[], [[FOOT_L, BOX_B]], [[FOOT_L, FOOT_R, BOX_B], [FORE_R, BOX_A]]]
    rng = np.random.default_rng(5)
    for groups in cases:
        plan = sparse_hessian.build_plan(m, groups, 64, "fused")
        adj, nv = plan.adjacency, m.nv
        H = np.zeros((nv, nv))
        for a in range(nv):
            for b in adj[a]:
                if a < b:
                    H[a, b] = H[b, a] = rng.normal()
        H += np.diag(np.abs(H).sum(1) + 1.0 + rng.random(nv))
        g = rng.normal(size=nv)
        x = _run_tables(plan, H, g)
        assert plan.levels > 1
        np.testing.assert_allclose(x, np.linalg.solve(H, g), rtol=1e-10, atol=1e-12)
        # M's stored entries map onto pattern slots
        sm = plan.tables["s_m"]
        assert (sm >= 0).sum() == m.nM


def test_plan_gates():
    m = _legged_model()
    ctx = SimpleNamespace()
    plan, reason = sparse_hessian.plan_for_model(m, ctx, None, 32)
    assert plan is None and "declare" in reason
    plan, reason = sparse_hessian.plan_for_model(m, ctx, [], 32)  # host arrays: not CUDA
    assert plan is None and "CPU" in reason
    m.body_parentid = SimpleNamespace(device=SimpleNamespace(is_cuda=True))
    small_parent, small_body = synthetic.chain_tree(20)
    small = put_model(small_parent, body_of_dof=small_body)
    small.body_parentid = m.body_parentid
    plan, reason = sparse_hessian.plan_for_model(small, ctx, [], 32)
    assert plan is None and "nv 20" in reason
    # hessian_pattern needs the real body tree again
    m2 = _legged_model()
    on_cuda = copy.copy(m2)
    host_parent = m2.body_parentid

    class _Dev(np.ndarray):  # a host array that claims a CUDA device
        device = SimpleNamespace(is_cuda=True)

    arr = host_parent.view(_Dev)
    on_cuda.body_parentid = arr
    plan, reason = sparse_hessian.plan_for_model(on_cuda, ctx, [[FOOT_L], [FOOT_R]], 32)
    assert plan is not None and reason == "enabled" and plan.path == "fused"
    assert plan.density <= sparse_hessian.MAX_DENSITY
    # a single chain is dense: rejected by density
    cp, cb = synthetic.chain_tree(40)
    chain = put_model(cp, body_of_dof=cb)
    chain.body_parentid = chain.body_parentid.view(_Dev)
    plan, reason = sparse_hessian.plan_for_model(chain, ctx, [], 32)
    assert plan is None and "density" in reason


def test_pattern_misses_counts_entries_outside_the_adjacency():
    m = _legged_model()
    adj = sparse_hessian.hessian_pattern(m, [])
    h = np.zeros((2, m.nv_pad, m.nv_pad), np.float32)
    h[0, 0, 1] = 1.0  # inside (tree ancestry)
    left, right = int(m.body_dofadr[FOOT_L]), int(m.body_dofadr[FOOT_R])
    h[1, min(left, right), max(left, right)] = 2.0  # the two feet are not coupled
    assert sparse_hessian.pattern_misses(h, adj) == 1


def _single_body_groups(m):
    return [[b] for b in range(1, len(m.body_dofadr))]


def _oracle_sparse(oracle, m, d, plan):
    from helpers import host_ctx

    d2 = copy.deepcopy(d)
    ctx = host_ctx(m, d2)
    oracle.solve(m, d2, ctx, np.zeros(1, np.int32), sparse_plan_struct=sparse_hessian.host_struct(plan))
    return d2, ctx


def test_sparse_oracle_agrees_with_dense_oracle(oracle):
    """tests/test_mjw_sparse_hessian.py:349-377: same iteration counts, |dqacc| <= 2e-4
    (max|qacc| + 1), no violations when rows stay inside the declared pattern."""
    from helpers import run_oracle

    for name, worlds in (("humanoid", 128), ("snu", 32)):
        m, d, _ = synthetic.make_workload(name, worlds, seed=2)
        plan = sparse_hessian.build_plan(m, _single_body_groups(m), 32 if m.nv_pad < 64 else 64, "fused")
        dense, _, _ = run_oracle(oracle, m, d)
        sparse, ctx = _oracle_sparse(oracle, m, d, plan)
        np.testing.assert_array_equal(sparse.solver_niter, dense.solver_niter)
        assert np.abs(sparse.qacc - dense.qacc).max() <= 2e-4 * (np.abs(dense.qacc).max() + 1)
        assert ctx.hfactor[:, -1, -1].sum() == 0


# ---------------------------------------------------------------------------- GPU


def _cuda_sparse(m, d, device, groups):
    import torch

    from instantmimic_b200 import mjw_model
    from instantmimic_b200 import mjw_step_optimized as runtime

    md, dd = mjw_model.to_device(m, device), mjw_model.to_device(copy.deepcopy(d), device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, device, with_matrices=True)
    reason = runtime.refresh_sparse_hessian(md, dd, scratch, groups, device)
    assert reason == "enabled", reason
    runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
    torch.cuda.synchronize()
    return mjw_model.to_host(dd), scratch, (md, dd)


@pytest.mark.gpu
@pytest.mark.parametrize("name,worlds", [("humanoid", 128), ("snu", 48)])
def test_fused_sparse_kernel_matches_oracle(oracle, cuda_device, name, worlds):
    m, d, _ = synthetic.make_workload(name, worlds, seed=2, rowless_fraction=0.1)
    groups = _single_body_groups(m)
    got, scratch, _ = _cuda_sparse(m, d, cuda_device, groups)
    plan = scratch.solver_context.sparse_hessian_plan
    want, wctx = _oracle_sparse(oracle, m, d, plan)
    np.testing.assert_array_equal(got.solver_niter, want.solver_niter)
    np.testing.assert_array_equal(got.overflow, want.overflow)
    live = np.arange(d.njmax)[None, :] < np.minimum(d.nefc, d.njmax)[:, None]
    np.testing.assert_array_equal(got.efc.state[live], want.efc.state[live])
    np.testing.assert_array_equal(got.qacc, want.qacc)  # bit for bit
    np.testing.assert_array_equal(got.efc.force[live], want.efc.force[live])
    # the packed H, the factor and 1/D land in hfactor as the reference lays them out
    hf = scratch.solver_context.hfactor.cpu().numpy().reshape(worlds, -1)
    whf = wctx.hfactor.reshape(worlds, -1)
    rows = d.nefc > 0
    np.testing.assert_array_equal(hf[rows, : 2 * plan.nfac + m.nv], whf[rows, : 2 * plan.nfac + m.nv])
    assert sparse_hessian.violations(scratch.solver_context.hfactor, plan).sum() == 0


@pytest.mark.gpu
def test_fused_sparse_matches_dense_steps(oracle, cuda_device):
    from helpers import run_cuda

    m, d, _ = synthetic.make_workload("humanoid", 256, seed=8)
    dense, _, _, _ = run_cuda(m, d, cuda_device)
    sparse, scratch, _ = _cuda_sparse(m, d, cuda_device, _single_body_groups(m))
    np.testing.assert_array_equal(sparse.solver_niter, dense.solver_niter)
    assert np.abs(sparse.qacc - dense.qacc).max() <= 2e-4 * (np.abs(dense.qacc).max() + 1)
    # bitwise repeatable
    again, _, _ = _cuda_sparse(m, d, cuda_device, _single_body_groups(m))
    np.testing.assert_array_equal(again.qacc, sparse.qacc)


@pytest.mark.gpu
def test_violation_counter_accumulates_and_resets(cuda_device):
    """tests/test_mjw_sparse_hessian.py:426-452: rows that couple undeclared bodies
    are counted, the count accumulates across solves and the check raises and resets."""
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, _ = synthetic.make_workload("humanoid", 32, seed=3)
    # make row 0 of every world couple the two feet (not a declared group)
    left, right = int(m.body_dofadr[9 + 1]), int(m.body_dofadr[12 + 1])
    d.efc.J[:, 0, left] = 1.0
    d.efc.J[:, 0, right] = 1.0
    d.efc.aref[:, 0] = 5.0  # active (Jaref < 0) at the start
    got, scratch, (md, dd) = _cuda_sparse(m, d, cuda_device, _single_body_groups(m))
    plan = scratch.solver_context.sparse_hessian_plan
    first = sparse_hessian.violations(scratch.solver_context.hfactor, plan).copy()
    assert (first > 0).sum() > 16
    runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
    torch.cuda.synchronize()
    second = sparse_hessian.violations(scratch.solver_context.hfactor, plan)
    assert (second >= first).all() and second.sum() > first.sum()
    with pytest.raises(RuntimeError, match="outside the declared coupling pattern"):
        runtime.check_sparse_hessian_violations(scratch)
    assert sparse_hessian.violations(scratch.solver_context.hfactor, plan).sum() == 0
    runtime.check_sparse_hessian_violations(scratch)  # clean now


@pytest.mark.gpu
def test_nonfused_sparse_factor_matches_oracle_and_dense_search(oracle, cuda_device):
    """sparse_hessian_upstream_factor: factor the dense H the iteration maintains
    (mode 4), then solve again from the stored factor (mode 5)."""
    import ctypes as C

    import torch

    from helpers import run_cuda
    from instantmimic_b200 import abi

    m, d, _ = synthetic.make_workload("humanoid", 64, seed=6, iterations=1, ls_iterations=50)
    _, hctx, _, (md, dd, scratch) = run_cuda(m, d, cuda_device, matrices=True)
    ctx = scratch.solver_context
    plan = sparse_hessian.build_plan(m, _single_body_groups(m), 64, "nonfused")
    sparse_hessian.upload(plan, cuda_device)
    dense_search = ctx.search.clone()
    ctx.done.zero_()
    ctx.hfactor.zero_()
    sparse_hessian.nonfused_factor_solve(plan, ctx, d.nworld)
    torch.cuda.synchronize()
    got = ctx.search.cpu().numpy()
    rows = d.nefc > 0
    scale = np.abs(dense_search.cpu().numpy()).max() + 1
    assert np.abs(got - dense_search.cpu().numpy())[rows].max() <= 2e-4 * scale
    # oracle, same tables on the host
    lib = oracle.lib()
    st = sparse_hessian.host_struct(plan)
    W, P = d.nworld, m.nv_pad
    o_search = np.zeros((W, m.nv), np.float32)
    o_hf = np.zeros((W, P, P), np.float32)
    o_sd, o_dec = np.zeros(W, np.float32), np.zeros(W, np.float32)
    grad, h = hctx.grad.copy(), hctx.h.copy()
    lib.oracle_sparse_factor_nonfused.restype = C.c_int
    lib.oracle_sparse_factor_nonfused.argtypes = [C.POINTER(abi.ImnSparsePlan)] + [abi.P] * 2 + [abi.I64] + [
        abi.P] * 5 + [abi.I64, abi.P, abi.P, C.c_int, C.c_int, C.c_int]
    lib.oracle_sparse_factor_nonfused(
        C.byref(st), None, grad.ctypes.data, grad.strides[0] // 4, h.ctypes.data, None, None, o_hf.ctypes.data,
        o_search.ctypes.data, m.nv, o_sd.ctypes.data, o_dec.ctypes.data, W, 0, 0)
    np.testing.assert_array_equal(got, o_search)
    np.testing.assert_array_equal(ctx.search_dot.cpu().numpy(), o_sd)
    np.testing.assert_array_equal(ctx.newton_decrement.cpu().numpy(), o_dec)
    # solve-only from the stored factor: same bits as the fresh factor's solve
    ctx.search.zero_()
    ctx.quad_changed_count.zero_()
    sparse_hessian.nonfused_factor_solve(plan, ctx, d.nworld, skip_unchanged=True)
    torch.cuda.synchronize()
    np.testing.assert_allclose(ctx.search.cpu().numpy(), got, rtol=2e-4, atol=2e-5)


def test_sweep_records_restate_the_level_tables():
    """The per-(sweep, lane) records the fused kernel reads (include/imnewton.h) carry the
    same entries, runs and level boundaries as the level tables they are packed from."""
    for name in ("humanoid", "snu"):
        m, _, _ = synthetic.make_workload(name, 1, seed=0)
        plan = sparse_hessian.build_plan(m, _single_body_groups(m), 32 if m.nv_pad < 64 else 64, "fused")
        t = plan.tables
        fs = t["fsweep"].reshape(-1, 32, 4).astype(np.int64)
        seen, sweep = [], 0
        for lvl, team in enumerate(int(v) for v in t["lvl_team"]):
            e0, e1, per = int(t["lvl_ptr"][lvl]), int(t["lvl_ptr"][lvl + 1]), 32 // team
            starts = list(range(e0, e1, per))
            for eb in starts:
                rec = fs[sweep]
                sweep += 1
                assert ((rec[:, 3] >> 1) & 1 == (eb == starts[-1])).all()        # last sweep of the level
                assert ((rec[:, 3] >> 2) & 7 == team.bit_length() - 1).all()     # team width
                for lane in range(32):
                    e = eb + lane // team
                    has = rec[lane, 3] & 1
                    assert bool(has) == (e < e1)
                    if not has:
                        continue
                    seen.append(e) if lane % team == 0 else None
                    assert rec[lane, 0] & 0xFFFF == t["ent_slot"][e]
                    assert (rec[lane, 0] >> 16) - 1 == t["ent_col"][e]
                    r0, r1 = int(t["run_ptr"][e]), int(t["run_ptr"][e + 1])
                    assert (rec[lane, 3] >> 8) & 0xFF == max(r1 - r0 - 1, 0)
                    if r1 > r0:
                        assert rec[lane, 1] == t["run_ab"][r0] and rec[lane, 2] == t["run_kl"][r0]
                        assert rec[lane, 3] >> 16 == r0 + 1
        assert sweep == fs.shape[0] and seen == list(range(len(t["ent_slot"])))
        # backward records: every (slot, src, dst) once, levels closed by the last-of-level bit
        bs = t["bsweep"].astype(np.int64)
        live = bs[(bs >> 30) & 1 == 1]
        assert len(live) == len(t["b_slot"])
        assert sorted(zip(live & 0xFFFF, (live >> 16) & 0x7F, (live >> 23) & 0x7F)) == sorted(
            zip(t["b_slot"].astype(int), t["b_src"].astype(int), t["b_dst"].astype(int)))
        nonempty = int((np.diff(t["b_lvl"].astype(int)) > 0).sum())
        assert int(((bs.reshape(-1, 32)[:, 0] >> 31) & 1).sum()) == nonempty
    # the non-fused plan carries no records
    big, _, _ = synthetic.make_workload("humanoid", 1, seed=0)
    nf = sparse_hessian.build_plan(big, _single_body_groups(big), 64, "nonfused")
    assert nf.tables["fsweep"].size == 0 and sparse_hessian.host_struct(nf).nfsweep == 0


@pytest.mark.gpu
def test_library_uploaded_plan_gives_the_same_bits(cuda_device):
    """imn_sparse_plan_create: the tables in one device allocation made by the library."""
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, _ = synthetic.make_workload("humanoid", 64, seed=12)
    got, scratch, (md, dd) = _cuda_sparse(m, d, cuda_device, _single_body_groups(m))
    plan = scratch.solver_context.sparse_hessian_plan
    native = sparse_hessian.NativePlan(plan)
    assert native.struct.nfac == plan.nfac and native.struct.nfsweep == plan.struct.nfsweep
    plan.struct = native.struct
    del scratch._imn_solve_call  # structs are cached per scratch
    dd.qacc.zero_()
    runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(dd.qacc.cpu().numpy().view(np.uint32), got.qacc.view(np.uint32))
    np.testing.assert_array_equal(dd.solver_niter.cpu().numpy(), got.solver_niter)
    native.close()
    native.close()  # idempotent
