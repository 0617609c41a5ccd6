"""The implicit-fast integrator's tail: A = M - h qDeriv (joint damping + actuator-centric
actuation term), (A) x = efc.Ma, advance.  CPU: the oracle against float64 numpy
(dense algebra, rotation by the axis-angle formula).  GPU: the CUDA kernels against the
oracle -- A bit for bit, the advanced state within 2e-6 (sinf / cosf differ in the last
place between libm and the GPU), the solved acceleration against a float64 dense solve
with the tolerance the reference uses for its M-side solves (2e-4 relative)."""

import copy

import numpy as np
import pytest

from instantmimic_b200 import mjw_model, synthetic, types

ADVANCE_TOL = 2e-6
SOLVE_RTOL = 2e-4


def _problem(worlds=70, nu=20, seed=3, damping=True, single=False):
    rng = np.random.default_rng(seed)
    m, d, Mdense = synthetic.make_workload("humanoid", worlds, seed=seed)
    m.dof_damping = rng.uniform(0.0, 2.0, m.nv).astype(np.float32) if damping else np.zeros(m.nv, np.float32)
    m.nu = nu
    # moment rows: most actuators act on one dof, some span a dof and a few of its ancestors
    parent = np.asarray(m.dof_parentid)
    chains = [[[] for _ in range(nu)] for _ in range(worlds)]
    for w in range(worlds):
        for a in range(nu):
            want = 1 if single or rng.random() < 0.7 else int(rng.integers(2, 5))
            chain = [int(rng.integers(6, m.nv))]
            while len(chain) < want and parent[chain[-1]] >= 0:
                chain.append(int(parent[chain[-1]]))
            chains[w][a] = sorted(chain)
    nnz = np.array([[len(c) for c in row] for row in chains], np.int32)
    adr = np.zeros((worlds, nu), np.int32)
    if nu:
        adr[:, 1:] = np.cumsum(nnz, axis=1)[:, :-1]
    ld = max(int(nnz.sum(axis=1).max()) if nu else 1, 1)
    colind = np.zeros((worlds, ld), np.int32)
    moment = np.zeros((worlds, ld), np.float32)
    for w in range(worlds):
        for a in range(nu):
            c = chains[w][a]
            colind[w, adr[w, a] : adr[w, a] + len(c)] = c
            moment[w, adr[w, a] : adr[w, a] + len(c)] = rng.normal(size=len(c))
    d.moment_rownnz, d.moment_rowadr, d.moment_colind, d.actuator_moment = nnz, adr, colind, moment
    gain = (-rng.uniform(0.0, 30.0, (worlds, nu)) * (rng.random((worlds, nu)) < 0.8)).astype(np.float32)
    d.qpos = np.zeros((worlds, m.nq), np.float32)
    for j in range(m.njnt):
        p = int(m.jnt_qposadr[j])
        if m.jnt_type[j] == types.JointType.FREE:
            d.qpos[:, p : p + 3] = rng.normal(size=(worlds, 3))
            p += 3
        if m.jnt_type[j] in (types.JointType.FREE, types.JointType.BALL):
            q = rng.normal(size=(worlds, 4))
            d.qpos[:, p : p + 4] = q / np.linalg.norm(q, axis=1, keepdims=True)
        else:
            d.qpos[:, p] = rng.normal(size=worlds)
    d.qvel = rng.normal(0.0, 2.0, (worlds, m.nv)).astype(np.float32)
    d.time = rng.uniform(0, 5, worlds).astype(np.float32)
    d.efc.Ma[:] = rng.normal(size=(worlds, m.nv)).astype(np.float32)
    return m, d, Mdense, gain


def _dense_a(m, d, Mdense, gain):
    """float64 A = M - h (sum_a gain_a mom_a mom_a^T - diag(damping)) restricted to M's pattern."""
    h = float(m.opt.timestep[0])
    W, nv = d.nworld, m.nv
    pattern = np.asarray(m.M_elemid) >= 0
    pattern = pattern | pattern.T
    A = Mdense.astype(np.float64).copy()
    for w in range(W):
        qd = -np.diag(m.dof_damping.astype(np.float64))
        for a in range(m.nu):
            n, s = int(d.moment_rownnz[w, a]), int(d.moment_rowadr[w, a])
            mom = np.zeros(nv)
            mom[d.moment_colind[w, s : s + n]] = d.actuator_moment[w, s : s + n]
            qd += float(gain[w, a]) * np.outer(mom, mom)
        A[w] -= h * qd * pattern
    return A


def _quat_rotate_reference(q, w, h):
    """float64 q (x) exp(h w / 2), normalised."""
    out = np.empty_like(q, dtype=np.float64)
    for k in range(q.shape[0]):
        a = np.linalg.norm(w[k])
        r = np.array([1.0, 0, 0, 0]) if a < 1e-15 else np.concatenate(([np.cos(0.5 * h * a)], np.sin(0.5 * h * a) * w[k] / a))
        p = q[k].astype(np.float64)
        o = np.array([p[0] * r[0] - p[1:] @ r[1:], *(p[0] * r[1:] + r[0] * p[1:] + np.cross(p[1:], r[1:]))])
        out[k] = o / np.linalg.norm(o)
    return out


def test_oracle_matrix_and_advance_against_float64(oracle):
    m, d, Mdense, gain = _problem()
    A = oracle.implicit_matrix(m, d, gain)
    want = _dense_a(m, d, Mdense, gain)
    rows, cols = np.nonzero(np.asarray(m.M_elemid) >= 0)
    got_dense = np.zeros_like(want)
    got_dense[:, rows, cols] = A[:, np.asarray(m.M_elemid)[rows, cols]]
    got_dense[:, cols, rows] = got_dense[:, rows, cols]
    assert np.abs(got_dense - want).max() <= 1e-5 * np.abs(want).max()
    # without actuators and damping A is M itself, bit for bit
    m0, d0, _, _ = _problem(nu=0, damping=False)
    np.testing.assert_array_equal(oracle.implicit_matrix(m0, d0, None), d0.M)
    # advance
    h = float(m.opt.timestep[0])
    d1 = copy.deepcopy(d)
    qacc = np.random.default_rng(9).normal(0, 5, (d.nworld, m.nv)).astype(np.float32)
    oracle.advance(m, d1, qacc)
    v = d.qvel.astype(np.float64) + h * qacc
    assert np.abs(d1.qvel - v).max() < 1e-5
    np.testing.assert_allclose(d1.time, d.time + np.float32(h), rtol=0, atol=1e-6)
    for j in range(m.njnt):
        p, k = int(m.jnt_qposadr[j]), int(m.jnt_dofadr[j])
        if m.jnt_type[j] == types.JointType.FREE:
            assert np.abs(d1.qpos[:, p : p + 3] - (d.qpos[:, p : p + 3] + h * v[:, k : k + 3])).max() < 1e-5
            p, k = p + 3, k + 3
        if m.jnt_type[j] in (types.JointType.FREE, types.JointType.BALL):
            ref = _quat_rotate_reference(d.qpos[:, p : p + 4], v[:, k : k + 3], h)
            assert np.abs(d1.qpos[:, p : p + 4] - ref).max() < 1e-5
            assert np.abs(np.linalg.norm(d1.qpos[:, p : p + 4], axis=1) - 1).max() < 1e-5
        else:
            assert np.abs(d1.qpos[:, p] - (d.qpos[:, p] + h * v[:, k])).max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("nu", [33, 70])
def test_cuda_single_dof_actuators_add_in_actuator_order(oracle, cuda_device, nu):
    """Batches of single-dof actuators take the ranked one-step path; several actuators on
    one dof (70 actuators on 28 dofs) must still add in ascending actuator order."""
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, _, gain = _problem(nu=nu, single=True, seed=9)
    assert (d.moment_rownnz == 1).all()
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(copy.deepcopy(d), cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    runtime.attach_implicit_scratch(md, dd, scratch, cuda_device)
    scratch.implicit_actuator_vel.copy_(torch.from_numpy(gain))
    runtime.deriv_smooth_vel_dense_actuator_centric(md, dd, scratch.implicit_qderiv, scratch)
    torch.cuda.synchronize()
    A = oracle.implicit_matrix(m, d, gain)
    np.testing.assert_array_equal(scratch.implicit_qderiv.cpu().numpy().view(np.uint32), A.view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("nu", [0, 20])
def test_cuda_implicitfast_tail_matches_oracle(oracle, cuda_device, nu):
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, Mdense, gain = _problem(nu=nu)
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(copy.deepcopy(d), cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    runtime.attach_implicit_scratch(md, dd, scratch, cuda_device)
    if nu:
        scratch.implicit_actuator_vel.copy_(torch.from_numpy(gain))
    # 1. the matrix, bit for bit
    runtime.deriv_smooth_vel_dense_actuator_centric(md, dd, scratch.implicit_qderiv, scratch)
    torch.cuda.synchronize()
    A = oracle.implicit_matrix(m, d, gain if nu else None)
    np.testing.assert_array_equal(scratch.implicit_qderiv.cpu().numpy().view(np.uint32), A.view(np.uint32))
    # 2. solve + advance through the tree L'DL kernel
    runtime._factor_solve_i_dense(md, dd, scratch.implicit_qderiv, scratch.implicit_qacc, dd.efc.Ma,
                                  scratch.dense_factor_solve, tree_factor_solve=scratch.tree_factor_solve)
    runtime._advance_with_scratch(md, dd, scratch.implicit_qacc, scratch)
    torch.cuda.synchronize()
    x = scratch.implicit_qacc.cpu().numpy()
    exact = np.linalg.solve(_dense_a(m, d, Mdense, gain), d.efc.Ma.astype(np.float64)[..., None])[..., 0]
    np.testing.assert_allclose(x, exact, rtol=SOLVE_RTOL, atol=SOLVE_RTOL * np.abs(exact).max())
    want = copy.deepcopy(d)
    oracle.advance(m, want, x)  # same acceleration in: compares the advance alone
    got = mjw_model.to_host(dd)
    np.testing.assert_array_equal(got.qvel.view(np.uint32), want.qvel.view(np.uint32))
    assert np.abs(got.qpos - want.qpos).max() <= ADVANCE_TOL
    np.testing.assert_array_equal(got.time, want.time)


@pytest.mark.gpu
def test_implicitfast_integrate_entry(oracle, cuda_device):
    """The whole tail through one call, on a model with affine (position-servo) actuators:
    the velocity gains come from the actuator parameters."""
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, Mdense, _ = _problem(nu=20)
    rng = np.random.default_rng(4)
    m.actuator_gaintype = np.zeros(m.nu, np.int32)
    m.actuator_biastype = np.full(m.nu, int(types.BiasType.AFFINE), np.int32)
    m.actuator_dyntype = np.zeros(m.nu, np.int32)
    m.actuator_gainprm = np.zeros((m.nu, 10), np.float32)
    m.actuator_biasprm = np.zeros((m.nu, 10), np.float32)
    m.actuator_biasprm[:, 2] = -rng.uniform(1.0, 20.0, m.nu)  # -kd
    d.ctrl = rng.uniform(-1, 1, (d.nworld, m.nu)).astype(np.float32)
    gain = np.broadcast_to(m.actuator_biasprm[:, 2], (d.nworld, m.nu)).astype(np.float32)
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(copy.deepcopy(d), cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    runtime.attach_implicit_scratch(md, dd, scratch, cuda_device)
    runtime.implicitfast_integrate(md, dd, scratch)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(scratch.implicit_actuator_vel.cpu().numpy(), gain)
    exact = np.linalg.solve(_dense_a(m, d, Mdense, gain), d.efc.Ma.astype(np.float64)[..., None])[..., 0]
    h = float(m.opt.timestep[0])
    got = mjw_model.to_host(dd)
    assert np.abs(got.qvel - (d.qvel + h * exact)).max() <= 1e-4 * (np.abs(exact).max() + 1)
