"""One substep's worth of this library's calls -- body velocities, composite inertias and M,
bias forces, the constraint solve, the implicit-fast tail -- captured in a single CUDA
graph: nothing on the way allocates, synchronises or reads a device array on the host
(the reference runs its step inside a captured graph, docs/reference/simulation.md:3-11)."""

import copy

import numpy as np
import pytest

from instantmimic_b200 import mjw_model, synthetic, types

pytestmark = pytest.mark.gpu


def test_a_whole_substep_is_one_capturable_graph(cuda_device):
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime
    from instantmimic_b200.mjw_kernels import tree_fusion, velocity_fusion

    rng = np.random.default_rng(8)
    m, d, _ = synthetic.make_workload("humanoid", 96, seed=11)
    synthetic.add_smooth_state(m, d, seed=12)
    m.nu = m.nv - 6
    m.dof_damping = rng.uniform(0.0, 1.0, m.nv).astype(np.float32)
    m.actuator_gaintype = np.zeros(m.nu, np.int32)
    m.actuator_biastype = np.full(m.nu, int(types.BiasType.AFFINE), np.int32)
    m.actuator_dyntype = np.zeros(m.nu, np.int32)
    m.actuator_gainprm = np.zeros((m.nu, 10), np.float32)
    m.actuator_biasprm = np.zeros((m.nu, 10), np.float32)
    m.actuator_biasprm[:, 2] = -rng.uniform(1.0, 20.0, m.nu)
    W = d.nworld
    d.ctrl = rng.uniform(-1, 1, (W, m.nu)).astype(np.float32)
    d.moment_rownnz = np.ones((W, m.nu), np.int32)
    d.moment_rowadr = np.tile(np.arange(m.nu, dtype=np.int32), (W, 1))
    d.moment_colind = np.tile(np.arange(6, m.nv, dtype=np.int32), (W, 1))
    d.actuator_moment = np.ones((W, m.nu), np.float32)
    d.qpos = np.zeros((W, m.nq), np.float32)
    for j in range(m.njnt):
        p = int(m.jnt_qposadr[j])
        if m.jnt_type[j] == types.JointType.FREE:
            p += 3
        if m.jnt_type[j] in (types.JointType.FREE, types.JointType.BALL):
            d.qpos[:, p] = 1.0
    d.time = np.zeros(W, np.float32)
    Mkeep = d.M.copy()  # crb overwrites M with the inertia of the random state: keep the solve's own

    def fresh():
        md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(copy.deepcopy(d), cuda_device)
        scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
        runtime.attach_implicit_scratch(md, dd, scratch, cuda_device)
        assert scratch.tree_reduction is not None
        return md, dd, scratch

    # the reference's order writes M (crb) before the solve reads it; here the solve's batch
    # brings its own positive definite M, so crb writes into a copy
    def step(md, dd, scratch):
        solve_M = dd.M
        dd.M = dd.crb_M
        tree = runtime._select_tree_reduction(scratch, True)
        velocity_fusion.com_vel(md, dd, tree)
        tree_fusion.subtree_com_accumulate(md, dd, tree)
        tree_fusion.crb(md, dd, tree)
        tree_fusion.rne(md, dd, tree)
        dd.M = solve_M
        runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
        runtime.implicitfast_integrate(md, dd, scratch)

    md, dd, scratch = fresh()
    dd.crb_M = torch.zeros_like(dd.M)
    step(md, dd, scratch)
    torch.cuda.synchronize()
    eager = {k: getattr(dd, k).clone() for k in ("cvel", "cdof_dot", "crb", "crb_M", "cfrc_int", "qfrc_bias", "qacc",
                                                  "qvel", "qpos", "time", "solver_niter", "subtree_com")}
    assert int(dd.solver_niter.max()) > 0 and np.array_equal(dd.M.cpu().numpy(), Mkeep)

    md, dd, scratch = fresh()
    dd.crb_M = torch.zeros_like(dd.M)
    # one untimed call outside the capture: set-up work of first calls (function attributes,
    # cached host copies of constant tables) is not part of a step
    warm = fresh()
    warm[1].crb_M = torch.zeros_like(warm[1].M)
    step(*warm)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            step(md, dd, scratch)
    g.replay()
    torch.cuda.synchronize()
    for k, want in eager.items():
        assert torch.equal(getattr(dd, k), want), k
