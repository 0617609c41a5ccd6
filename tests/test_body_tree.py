"""Body-tree reductions, crb, rne and com_vel: the oracle against the reference's own
statement of the ordered sum and against independent float64 forms; the CUDA kernels
against the oracle, bit for bit.

The topologies, component counts and the cancellation case follow the reference's
tests/test_mjw_tree_fusion.py:11-75, 137-160; the selection table follows :163-177."""

from types import SimpleNamespace

import numpy as np
import pytest

from instantmimic_b200 import mjw_model, synthetic, types
from instantmimic_b200.mjw_kernels import tree_fusion, velocity_fusion
from oracle import oracle

COUNT = 97


def topology(kind: str):
    if kind == "wide":
        parents = np.zeros(COUNT, dtype=np.int32)
    elif kind == "deep":
        parents = np.maximum(np.arange(COUNT, dtype=np.int32) - 1, 0)
    else:  # several bodies hang on the world body
        parents = np.maximum(np.arange(COUNT, dtype=np.int32) - 3, 0)
    depths = np.zeros(COUNT, dtype=np.int32)
    for body in range(1, COUNT):
        depths[body] = depths[parents[body]] + 1
    levels = [np.flatnonzero(depths == k).astype(np.int32) for k in range(int(depths.max()) + 1)]
    return parents, levels


def depth_ordered_sum(initial, parents, levels, skip_root):
    """The reference test's own statement of the result (test_mjw_tree_fusion.py:36-41)."""
    out = initial.copy()
    for level in reversed(levels):
        for body in level:
            parent = parents[body]
            if body and (not skip_root or parent):
                out[:, parent, :] += out[:, body, :]
    return out


CASES = [(3, False), (6, False), (10, True)]


@pytest.mark.parametrize("kind", ["wide", "deep", "multiple_roots"])
@pytest.mark.parametrize("components,skip_root", CASES)
def test_oracle_accumulate_equals_the_depth_ordered_sum(kind, components, skip_root):
    parents, levels = topology(kind)
    model = SimpleNamespace(body_parentid=parents, body_tree=levels)
    scratch = tree_fusion.create_tree_reduction_scratch(model, deterministic=True)
    assert scratch.levels == len(levels)
    initial = np.random.default_rng(7).uniform(0.1, 1.0, (3, COUNT, components)).astype(np.float32)
    values = initial.copy()
    oracle.body_tree_accumulate(model, scratch, values, components, skip_root)
    np.testing.assert_array_equal(values, depth_ordered_sum(initial, parents, levels, skip_root))


def cancellation_case():
    parents = np.array([0, 0, 0, 0, 1, 1, 2, 2], dtype=np.int32)
    levels = [np.array(x, dtype=np.int32) for x in ([0], [1, 2, 3], [4, 5, 6, 7])]
    initial = np.array([[[1], [1e8], [1], [-1e8], [1], [-1], [2], [3]]], np.float32)
    return parents, levels, initial


def test_oracle_accumulate_keeps_the_float32_cancellation_order():
    parents, levels, initial = cancellation_case()
    model = SimpleNamespace(body_parentid=parents, body_tree=levels)
    scratch = tree_fusion.create_tree_reduction_scratch(model, deterministic=True, cooperative=False)
    values = initial.copy()
    oracle.body_tree_accumulate(model, scratch, values, 1, False)
    np.testing.assert_array_equal(values, depth_ordered_sum(initial, parents, levels, False))
    # the world body: ((1 + 1e8) + 6) - 1e8 in float32 = 8 (1e8 swallows the 1, the 6 rounds
    # to 8 on 1e8's grid); any other order of the three children gives another number
    assert values[0, 0, 0] == np.float32(8.0)


def test_level_tables_list_children_in_level_order():
    parents, levels = topology("multiple_roots")
    t = tree_fusion.level_tables(levels, parents)
    assert t["bodies"].tolist() == np.concatenate(levels).tolist()
    for pos, parent in enumerate(t["bodies"].tolist()):
        kids = t["child_ids"][t["child_ptr"][pos]:t["child_ptr"][pos + 1]].tolist()
        assert kids == [b for b in t["bodies"].tolist() if b != 0 and parents[b] == parent]
    with pytest.raises(ValueError, match="one level below"):
        tree_fusion.level_tables([np.array([0]), np.array([1, 2])], np.array([0, 0, 1]))
    with pytest.raises(ValueError, match="every body"):
        tree_fusion.level_tables([np.array([0]), np.array([1])], np.array([0, 0, 1]))


def test_tree_selection_keeps_the_kernel_flag():
    from instantmimic_b200.mjw_step_optimized import _select_tree_reduction

    atomic = SimpleNamespace(deterministic=False)
    ordered = SimpleNamespace(deterministic=True, cooperative=False)
    assert _select_tree_reduction(SimpleNamespace(tree_reduction=atomic), False) is None
    assert _select_tree_reduction(SimpleNamespace(tree_reduction=atomic), True) is atomic
    assert _select_tree_reduction(SimpleNamespace(tree_reduction=ordered), False) is ordered
    assert _select_tree_reduction(None, True) is None
    # the capability record names the tree scratch (mjw_step_optimized.py:2862-2875)
    from instantmimic_b200.mjw_step_optimized import optimized_kernel_capabilities

    bare = dict(solver_context=None, solver_uses_compact=False, dense_factor_solve=None, tile_factor_solve=None,
                tree_factor_solve=None, constraint_free=False)
    model = SimpleNamespace(nv=3)
    assert optimized_kernel_capabilities(model, SimpleNamespace(tree_reduction=ordered, **bare))["tree"] is True
    assert optimized_kernel_capabilities(model, SimpleNamespace(tree_reduction=None, **bare))["tree"] is False
    assert optimized_kernel_capabilities(model, SimpleNamespace(tree_reduction=ordered, **bare), enabled=False)["tree"] is False


def test_missing_scratch_is_an_error_not_a_fallback():
    m, d, _ = synthetic.make_workload("humanoid", 2, seed=0)
    synthetic.add_smooth_state(m, d)
    for call in (tree_fusion.crb, tree_fusion.rne, tree_fusion.subtree_com_accumulate):
        with pytest.raises(RuntimeError, match="no per-level upstream path"):
            call(m, d, None)
    with pytest.raises(RuntimeError, match="no per-level upstream path"):
        velocity_fusion.com_vel(m, d, None)
    assert tree_fusion.create_tree_reduction_scratch(SimpleNamespace(body_tree=[])) is None


# ---- independent float64 forms ----------------------------------------------------


def inertia_matrix(i10):
    """6x6 spatial inertia of the 10 numbers (rotational about the origin, m c, m)."""
    ixx, iyy, izz, ixy, ixz, iyz, mx, my, mz, mass = [float(v) for v in i10]
    rot = np.array([[ixx, ixy, ixz], [ixy, iyy, iyz], [ixz, iyz, izz]])
    skew = np.array([[0, -mz, my], [mz, 0, -mx], [-my, mx, 0]])  # [m c]x
    out = np.zeros((6, 6))
    out[:3, :3], out[:3, 3:], out[3:, :3], out[3:, 3:] = rot, skew, skew.T, mass * np.eye(3)
    return out


def dof_ancestry(m):
    """anc[b] = the dofs on the path from the root to body b (its own included)."""
    parent, nbody = np.asarray(m.body_parentid), len(m.body_parentid)
    anc = [[] for _ in range(nbody)]
    for b in range(1, nbody):
        own = list(range(int(m.body_dofadr[b]), int(m.body_dofadr[b]) + int(m.body_dofnum[b])))
        anc[b] = anc[parent[b]] + own
    return anc


def smooth_case(name, nworld=3, seed=5):
    m, d, _ = synthetic.make_workload(name, nworld, seed=seed)
    synthetic.add_smooth_state(m, d, seed=seed + 1)
    scratch = tree_fusion.create_tree_reduction_scratch(m, deterministic=True)
    return m, d, scratch


def cross_motion(vel, a):
    return np.concatenate([np.cross(vel[:3], a[:3]), np.cross(vel[:3], a[3:]) + np.cross(vel[3:], a[:3])])


def cross_force(vel, f):
    return np.concatenate([np.cross(vel[:3], f[:3]) + np.cross(vel[3:], f[3:]), np.cross(vel[:3], f[3:])])


@pytest.mark.parametrize("name", ["humanoid", "snu", "g1"])
def test_oracle_crb_equals_the_sum_over_bodies(name):
    """M = sum_b J_b^T I_b J_b with J_b the motion axes on the path to body b: the
    composite-inertia recursion is that sum reordered."""
    m, d, scratch = smooth_case(name)
    oracle.crb(m, d, scratch)
    anc = dof_ancestry(m)
    nbody = len(m.body_parentid)
    for w in range(d.nworld):
        dense = np.zeros((m.nv, m.nv))
        for b in range(1, nbody):
            J = np.zeros((6, m.nv))
            J[:, anc[b]] = d.cdof[w, anc[b]].astype(np.float64).T
            dense += J.T @ inertia_matrix(d.cinert[w, b]) @ J
        dense += np.diag(m.dof_armature[0].astype(np.float64))
        got = np.zeros((m.nv, m.nv))
        for i in range(m.nv):
            for k in range(int(m.M_rownnz[i])):
                got[i, m.M_colind[m.M_rowadr[i] + k]] = d.M[w, m.M_rowadr[i] + k]
        lower = np.tril(dense) * (got != 0)
        np.testing.assert_allclose(got, lower, rtol=2e-5, atol=2e-5 * np.abs(dense).max())
        assert np.count_nonzero(got) == m.nM
        # composite inertias: every body's own plus its descendants', the world body untouched
        np.testing.assert_array_equal(d.crb[w, 0], d.cinert[w, 0])
        leaf = [b for b in range(1, nbody) if b not in set(np.asarray(m.body_parentid)[1:].tolist())]
        np.testing.assert_array_equal(d.crb[w, leaf], d.cinert[w, leaf])


@pytest.mark.parametrize("name", ["humanoid", "snu", "g1"])
def test_oracle_com_vel_and_rne_equal_the_path_sums(name):
    m, d, scratch = smooth_case(name)
    oracle.com_vel(m, d, scratch)
    oracle.rne(m, d, scratch)
    anc = dof_ancestry(m)
    nbody = len(m.body_parentid)
    g = m.opt.gravity[0].astype(np.float64)
    for w in range(d.nworld):
        cdof, qv = d.cdof[w].astype(np.float64), d.qvel[w].astype(np.float64)
        cvel = np.zeros((nbody, 6))
        for b in range(1, nbody):
            cvel[b] = (cdof[anc[b]] * qv[anc[b], None]).sum(0)
        np.testing.assert_allclose(d.cvel[w], cvel, rtol=1e-5, atol=1e-5)
        # cdof_dot of a dof: the velocity accumulated before that dof's joint (after the
        # three translations for the rotations of a free joint) crossed with the axis
        dot = np.zeros((m.nv, 6))
        for b in range(1, nbody):
            v = cvel[m.body_parentid[b]].copy()
            dof = int(m.body_dofadr[b])
            for j in range(int(m.body_jntadr[b]), int(m.body_jntadr[b]) + int(m.body_jntnum[b])):
                kind = int(m.jnt_type[j])
                if kind == types.JointType.FREE:
                    for k in range(3):
                        v += cdof[dof + k] * qv[dof + k]
                    for k in range(3, 6):
                        dot[dof + k] = cross_motion(v, cdof[dof + k])
                    for k in range(3, 6):
                        v += cdof[dof + k] * qv[dof + k]
                    dof += 6
                elif kind == types.JointType.BALL:
                    for k in range(3):
                        dot[dof + k] = cross_motion(v, cdof[dof + k])
                    for k in range(3):
                        v += cdof[dof + k] * qv[dof + k]
                    dof += 3
                else:
                    dot[dof] = cross_motion(v, cdof[dof])
                    v += cdof[dof] * qv[dof]
                    dof += 1
        np.testing.assert_allclose(d.cdof_dot[w], dot, rtol=1e-5, atol=1e-5)
        # bias forces: qfrc_bias = sum_b J_b^T (I_b a_b + v_b x* I_b v_b), a_b the path sum
        # of cdof_dot qvel on top of -gravity
        bias = np.zeros(m.nv)
        for b in range(1, nbody):
            a = np.concatenate([np.zeros(3), -g]) + (dot[anc[b]] * qv[anc[b], None]).sum(0)
            I = inertia_matrix(d.cinert[w, b])
            f = I @ a + cross_force(cvel[b], I @ cvel[b])
            bias[anc[b]] += cdof[anc[b]] @ f
            np.testing.assert_allclose(d.cacc[w, b], a, rtol=1e-4, atol=1e-4)
        np.testing.assert_allclose(d.qfrc_bias[w], bias, rtol=2e-4, atol=2e-4 * max(1.0, np.abs(bias).max()))


def test_gravity_switch():
    m, d, scratch = smooth_case("humanoid", nworld=1)
    d.qvel[:] = 0
    oracle.com_vel(m, d, scratch)
    oracle.rne(m, d, scratch)
    assert np.abs(d.qfrc_bias).max() > 0
    m.opt.disableflags |= int(types.DisableBit.GRAVITY)
    oracle.rne(m, d, scratch)
    assert np.abs(d.qfrc_bias).max() == 0 and np.abs(d.cacc).max() == 0


# ---- CUDA against the oracle ----------------------------------------------------------


def _device():
    import torch

    return torch.device("cuda:0")


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["wide", "deep", "multiple_roots"])
@pytest.mark.parametrize("components,skip_root", CASES)
def test_cuda_accumulate_bit_exact(kind, components, skip_root):
    import torch

    parents, levels = topology(kind)
    host = SimpleNamespace(body_parentid=parents, body_tree=levels)
    dev = SimpleNamespace(body_parentid=torch.from_numpy(parents).to(_device()),
                          body_tree=[torch.from_numpy(x).to(_device()) for x in levels])
    scratch = tree_fusion.create_tree_reduction_scratch(dev, deterministic=True)
    assert scratch.team_lanes == (32 if kind == "wide" else 8)
    for nworld in (3, 1027):
        initial = np.random.default_rng(7).uniform(0.1, 1.0, (nworld, COUNT, components)).astype(np.float32)
        values = torch.from_numpy(initial).to(_device())
        data = SimpleNamespace(nworld=nworld)
        tree_fusion.accumulate(dev, data, values, components, skip_root, scratch)
        expected = depth_ordered_sum(initial, parents, levels, skip_root)
        np.testing.assert_array_equal(values.cpu().numpy(), expected)
        # replays give the same bits
        values.copy_(torch.from_numpy(initial))
        tree_fusion.accumulate(dev, data, values, components, skip_root, scratch)
        np.testing.assert_array_equal(values.cpu().numpy(), expected)
    ref = initial.copy()
    oracle.body_tree_accumulate(host, tree_fusion.create_tree_reduction_scratch(host), ref, components, skip_root)
    np.testing.assert_array_equal(ref, expected)


@pytest.mark.gpu
def test_cuda_accumulate_cancellation_order():
    import torch

    parents, levels, initial = cancellation_case()
    dev = SimpleNamespace(body_parentid=torch.from_numpy(parents).to(_device()),
                          body_tree=[torch.from_numpy(x).to(_device()) for x in levels])
    scratch = tree_fusion.create_tree_reduction_scratch(dev, deterministic=True, cooperative=False)
    values = torch.from_numpy(initial).to(_device())
    tree_fusion.accumulate(dev, SimpleNamespace(nworld=1), values, 1, False, scratch)
    np.testing.assert_array_equal(values.cpu().numpy(), depth_ordered_sum(initial, parents, levels, False))


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["humanoid", "snu", "g1"])
@pytest.mark.parametrize("nworld,team", [(5, None), (2051, None), (37, 16), (37, 32), (4096 + 13, None)])
def test_cuda_smooth_stages_bit_exact(name, nworld, team):
    """Every width of the per-world lane team (8 is what these models get; 16 and 32 forced)
    and batches that leave the last warp with surplus teams; from 4096 worlds on the
    lane-per-world kernels run (32 worlds per block; the last block is partial)."""
    from dataclasses import replace

    m, d, scratch = smooth_case(name, nworld=nworld)
    md, dd = mjw_model.to_device(m, _device()), mjw_model.to_device(d, _device())
    sd = tree_fusion.create_tree_reduction_scratch(md, deterministic=True)
    assert sd.team_lanes == 8
    if team is not None:
        sd = replace(sd, team_lanes=team)
    dd.M.fill_(float("nan"))  # every stored entry of M is written
    velocity_fusion.com_vel(md, dd, sd)
    tree_fusion.crb(md, dd, sd)
    tree_fusion.rne(md, dd, sd)
    tree_fusion.subtree_com_accumulate(md, dd, sd)
    oracle.com_vel(m, d, scratch)
    oracle.crb(m, d, scratch)
    oracle.rne(m, d, scratch)
    oracle.body_tree_accumulate(m, scratch, d.subtree_com, 3, False)
    got = mjw_model.to_host(dd)
    for field in ("cvel", "cdof_dot", "crb", "M", "cacc", "cfrc_int", "qfrc_bias", "subtree_com"):
        np.testing.assert_array_equal(getattr(got, field), getattr(d, field), err_msg=field)


@pytest.mark.gpu
def test_cuda_tree_entry_points_check_their_arguments():
    import torch

    m, d, _ = smooth_case("humanoid", nworld=2)
    md, dd = mjw_model.to_device(m, _device()), mjw_model.to_device(d, _device())
    sd = tree_fusion.create_tree_reduction_scratch(md)
    with pytest.raises(ValueError, match="contiguous"):
        tree_fusion.accumulate(md, dd, torch.zeros(2, 3, 3, device=_device()), 3, False, sd)
    dd.cinert = dd.cinert[:, :, :9]
    with pytest.raises(ValueError, match="d.cinert"):
        tree_fusion.crb(md, dd, sd)
