"""Host-side gates and error behaviour of the solver entry points (no GPU).  The
tables are the reference's (tests/test_mjw_newton_fusion.py:30-96, 418-447)."""

from types import SimpleNamespace

import numpy as np
import pytest

from instantmimic_b200 import mjw_model, synthetic, types
from instantmimic_b200 import mjw_step_optimized as runtime
from instantmimic_b200.mjw_kernels import newton_fusion as fusion


def _model(**updates):
    model = SimpleNamespace(
        nv=34,
        nv_pad=48,
        is_sparse=False,
        opt=SimpleNamespace(
            solver=types.SolverType.NEWTON,
            cone=types.ConeType.PYRAMIDAL,
            iterations=4,
            integrator=types.IntegratorType.IMPLICITFAST,
        ),
        block_dim=SimpleNamespace(linesearch_iterative=32),
        body_parentid=SimpleNamespace(device=SimpleNamespace(is_cuda=True)),
    )
    for key, value in updates.items():
        setattr(model, key, value)
    return model


@pytest.mark.parametrize(
    "nv,pad,expected",
    [
        (0, 0, False), (12, 12, False), (13, 16, True), (16, 16, True), (17, 32, True),
        (31, 32, True), (32, 32, True), (32, 48, True), (33, 48, True), (35, 48, True),
        (56, 64, True), (60, 64, True), (61, 64, True), (64, 80, True), (70, 80, True),
        (79, 80, True), (80, 96, False), (34, 40, False),
    ],
)
def test_eligibility_uses_dof_layout(nv, pad, expected):
    assert fusion.eligible(_model(nv=nv, nv_pad=pad), object()) is expected


@pytest.mark.parametrize("pad,expected", [(32, 32), (48, 32), (64, 64), (80, 64)])
def test_block_width_uses_padded_dof_layout(pad, expected):
    assert fusion.newton_block_dim(_model(nv_pad=pad)) == expected


@pytest.mark.parametrize(
    "reason",
    ["compact", "sparse", "sparse_compact", "cg", "discrete", "elliptic", "zero_iterations",
     "reduction_layout", "cpu_device"],
)
def test_unsupported_solver_modes_are_not_eligible(reason):
    model = _model()
    ctx = SimpleNamespace(sparse_compact=reason == "sparse_compact")
    if reason == "sparse":
        model.is_sparse = True
    if reason == "discrete":
        model.opt.integrator = types.IntegratorType.DISCRETE
    if reason == "cg":
        model.opt.solver = types.SolverType.CG
    if reason == "elliptic":
        model.opt.cone = types.ConeType.ELLIPTIC
    if reason == "zero_iterations":
        model.opt.iterations = 0
    if reason == "reduction_layout":
        model.block_dim.linesearch_iterative = 64
    if reason == "cpu_device":
        model.body_parentid.device.is_cuda = False
    assert not fusion.eligible(model, ctx, compact=reason == "compact")


@pytest.mark.parametrize(
    "nworld,sm_count,expected",
    [(1024, 170, 6), (2048, 170, 12), (4096, 170, 12), (8192, 170, 12), (512, 170, 3), (100, 170, 1),
     (1024, 108, 9), (1024, 132, 7), (0, 170, 0), (1024, 0, 0), (-1, 170, 0), (8192, 148, 12)],
)
def test_min_blocks_tracks_grid_and_device(nworld, sm_count, expected):
    assert fusion.newton_min_blocks_per_sm(nworld, sm_count) == expected


def test_nv_pad_rule_and_dense_cap():
    assert [mjw_model.newton_nv_pad(nv) for nv in (13, 15, 16, 31, 32, 34, 63, 64, 79)] == [
        16, 16, 32, 32, 48, 48, 64, 80, 80]
    assert mjw_model.DENSE_NV_MAX == 79


def test_solve_with_scratch_error_behaviour():
    """mjw_step_optimized.py:2701-2707: missing scratch and layout mismatch raise."""
    m, d, _ = synthetic.make_workload("humanoid", 2, seed=0)
    empty = runtime.OptimizedFwdPositionScratch()
    with pytest.raises(RuntimeError, match="not initialized"):
        runtime.solve_with_scratch(m, d, empty)
    scratch = runtime.OptimizedFwdPositionScratch(solver_context=object(), solver_nsolving=object(),
                                                  solver_uses_compact=True)
    with pytest.raises(RuntimeError, match="no longer matches"):
        runtime.solve_with_scratch(m, d, scratch)
    # host arrays are not CUDA buffers: the model is outside the fused path and there
    # is no other path
    scratch.solver_uses_compact = False
    with pytest.raises(RuntimeError, match="outside the fused Newton path"):
        runtime.solve_with_scratch(m, d, scratch)
    with pytest.raises(RuntimeError, match="factor workspace requires"):
        runtime._factor_solve_i_dense(m, d, d.M, d.qacc, d.qfrc_smooth, None, factor_workspace=d.M)
    with pytest.raises(RuntimeError, match="retained factor requires"):
        runtime._factor_solve_i_dense(m, d, d.M, d.qacc, d.qfrc_smooth, None, retain_factor=True)
    with pytest.raises(RuntimeError, match="need CUDA arrays"):
        runtime._factor_solve_i_dense(m, d, d.M, d.qacc, d.qfrc_smooth, None)


def test_struct_builder_checks_strides():
    from instantmimic_b200 import binding

    m, d, _ = synthetic.make_workload("humanoid", 4, seed=0)
    d.qacc = np.zeros((4, m.nv + 2), np.float32)[:, : m.nv]  # different world stride
    with pytest.raises(ValueError, match="share one world stride"):
        binding.data_struct(m, d)
    m2, d2, _ = synthetic.make_workload("humanoid", 4, seed=0)
    d2.efc.J = np.zeros((4, d2.njmax, 2 * m2.nv), np.float32)[:, :, ::2]
    with pytest.raises(ValueError, match="unit innermost stride"):
        binding.data_struct(m2, d2)
    # a J with padded rows is accepted and described by its strides
    m3, d3, _ = synthetic.make_workload("humanoid", 4, seed=0)
    d3.efc.J = np.zeros((4, d3.njmax, 48), np.float32)[:, :, : m3.nv]
    s = binding.data_struct(m3, d3)
    assert (s.J_ld_row, s.J_ld_world) == (48, 48 * d3.njmax)


def test_shard_bounds_cover_the_batch():
    for n, g in ((8192, 8), (1000, 3), (5, 8)):
        b = mjw_model.shard_bounds(n, g)
        assert b[0][0] == 0 and b[-1][1] == n
        assert all(lo2 == hi1 for (_, hi1), (lo2, _) in zip(b, b[1:]))
        sizes = [hi - lo for lo, hi in b]
        assert max(sizes) - min(sizes) <= 1


def test_constants_follow_a_live_upstream_module():
    """Bits and enum members that are compared with values stored in a caller's Model
    come from the upstream module when there is one; constants compiled into the
    kernels must agree with it."""
    import enum
    from types import SimpleNamespace

    from instantmimic_b200 import binding, types

    class DisableBit(enum.IntFlag):
        WARMSTART = 1 << 9  # moved by one bit, as MuJoCo releases have done

    class OverflowType(enum.IntFlag):
        ITERATIONS = 8
        LS_ITERATIONS = 16

    live = SimpleNamespace(DisableBit=DisableBit, OverflowType=OverflowType, MJ_MINVAL=1e-15, MJ_MAXVAL=1e10)
    c = binding.upstream_constants(live, SimpleNamespace(_ALPHA_NOISE_EPS=2e-6))
    assert c["disable_warmstart"] == 512 and c["overflow_iterations"] == 8 and c["overflow_ls_iterations"] == 16
    assert c["alpha_noise_eps"] == 2e-6 and c["solver_newton"] == int(types.SolverType.NEWTON)
    with pytest.raises(RuntimeError, match="MJ_MINVAL"):
        binding.upstream_constants(SimpleNamespace(MJ_MINVAL=1e-12), None)

    class ConstraintState(enum.IntEnum):
        SATISFIED = 0
        QUADRATIC = 2

    with pytest.raises(RuntimeError, match="ConstraintState.QUADRATIC"):
        binding.upstream_constants(SimpleNamespace(ConstraintState=ConstraintState), None)
    assert binding.upstream_constants()["source"] == "package defaults"


def test_constraint_rows_impossible_gate():
    """mjw_step_optimized.py:116-147: True only when the model rules out every row
    source; a model without the fields keeps the general path."""
    from types import SimpleNamespace

    m, _, _ = synthetic.make_workload("humanoid", 1, seed=0)
    assert runtime._constraint_rows_impossible(m, ()) is False  # the stand-in carries none of the fields
    e = np.zeros(0, np.int32)
    free = SimpleNamespace(
        opt=SimpleNamespace(run_collision_detection=True), neq=0, nflex=0, nsensorcollision=0,
        jnt_limited_slide_hinge_adr=e, jnt_limited_ball_adr=e, tendon_limited_adr=e,
        dof_frictionloss=np.zeros(5, np.float32), tendon_frictionloss=np.zeros(0, np.float32),
        nxn_pairid_filtered=np.full((3, 2), -2, np.int32))
    assert runtime._constraint_rows_impossible(free, ()) is True
    assert runtime._constraint_rows_impossible(free, [object()]) is False  # ball-limit rows declared
    for change in (dict(neq=1), dict(nflex=2), dict(nsensorcollision=1),
                   dict(jnt_limited_slide_hinge_adr=np.array([3], np.int32)),
                   dict(dof_frictionloss=np.array([0, 0.2], np.float32)),
                   dict(nxn_pairid_filtered=np.array([[-2, -2], [-1, 4]], np.int32)),
                   dict(solver_compact=True), dict(opt=SimpleNamespace(run_collision_detection=False))):
        assert runtime._constraint_rows_impossible(SimpleNamespace(**{**vars(free), **change}), ()) is False, change


def test_timestep_is_handed_over_as_an_array_and_model_tables_are_read_once():
    """opt.timestep goes to the kernels as mujoco-warp stores it (a per-world float array);
    constant model tables that host code has to look at are copied from the device once per
    buffer, so that a step neither synchronises the stream nor breaks a graph capture."""
    import torch

    from instantmimic_b200 import arrays, binding

    m, _, _ = synthetic.make_workload("humanoid", 2, seed=0)
    ptr, n = binding._timestep(m)
    assert ptr == m.opt.timestep.ctypes.data and n == 1
    m.opt.timestep = 0.002
    with pytest.raises(ValueError, match="float array"):
        binding._timestep(m)
    table = torch.arange(5, dtype=torch.int32)
    first = arrays.table_to_host(table)
    table += 1  # a later change of the buffer is not seen: the table is declared constant
    assert arrays.table_to_host(table) is first and first.tolist() == [0, 1, 2, 3, 4]
    host = np.arange(3)
    assert arrays.table_to_host(host) is host


def test_packed_transfer_layouts_are_aligned_and_disjoint():
    """The one-buffer transport of host batches: every segment starts on a 256-byte boundary,
    segments do not overlap, and the typed views address exactly their segment."""
    import torch

    from instantmimic_b200 import host_batch

    W, R, nv, nM = 37, 64, 34, 310
    for offsets, end in (host_batch.packed_layout(W, R, nv, nM), host_batch.result_layout(W, R, nv)):
        spans = []
        for name, (o, dtype, shape) in offsets.items():
            n = int(np.prod(shape)) * np.dtype(dtype).itemsize
            assert o % 256 == 0, name
            spans.append((o, o + n))
        spans.sort()
        assert all(a_end <= b_start for (_, a_end), (b_start, _) in zip(spans, spans[1:]))
        assert end % 256 == 0 and end >= spans[-1][1]
        buf = torch.zeros(end, dtype=torch.uint8)
        views = host_batch._views(buf, offsets)
        for name, (o, dtype, shape) in offsets.items():
            v = views[name]
            assert tuple(v.shape) == tuple(shape) and str(v.dtype) == "torch." + dtype
            assert v.data_ptr() == buf.data_ptr() + o
    fixed = host_batch.packed_layout(W, R, nv, nM)[0]
    assert fixed["Joff"][1] == "int64" and "D" not in fixed  # per-row inputs travel compacted


def test_host_near_device_binds_to_the_gpus_node_and_restores(tmp_path):
    """Pinned staging buffers should live on the NUMA node of their GPU: the context manager
    narrows the thread's CPUs to that node's (read from sysfs) and puts them back."""
    import os

    from instantmimic_b200 import host_batch

    assert host_batch._cpu_list("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    before = os.sched_getaffinity(0)
    one = min(before)
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text(f"{one}\n")
    with host_batch.host_near_device(pci_bus_id="0000:1B:00.0", sysfs=str(tmp_path)) as near:
        assert near.node == 1 and os.sched_getaffinity(0) == {one}
    assert os.sched_getaffinity(0) == before
    # a platform that does not say (numa_node -1, or no such file): nothing changes
    (dev / "numa_node").write_text("-1\n")
    with host_batch.host_near_device(pci_bus_id="0000:1b:00.0", sysfs=str(tmp_path)) as near:
        assert near.node is None and os.sched_getaffinity(0) == before
    with host_batch.host_near_device(pci_bus_id="0000:ff:00.0", sysfs=str(tmp_path)) as near:
        assert near.node is None and os.sched_getaffinity(0) == before
