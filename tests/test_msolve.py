"""M-side factor + solve: tree L'DL plans, the blocked dense Cholesky and their
kernels.  CPU tests pin the oracle against numpy.linalg.solve of the dense matrix
(the pin the reference's own tests use, tests/test_tree_ldl.py:99-120,
tests/test_blocked_dense_factor_solve.py:616-626); GPU tests compare the CUDA
kernels with the oracle bit for bit."""

import numpy as np
import pytest

from instantmimic_b200 import synthetic
from instantmimic_b200.mjw_kernels import indexed_factor, tree_ldl
from instantmimic_b200.mjw_model import put_model


def _branched_tree():
    """Free root with two branches (one with a ball joint) and a second free body:
    nested ancestor rows, a 3-dof joint and two separate trees
    (tests/test_tree_ldl.py:22-37)."""
    joints = [(6, -1), (1, 0), (1, 1), (3, 0), (1, 3), (6, -1)]
    return synthetic._tree_from_joints(joints)


def _limbs_tree(limbs=4, links=6):
    return synthetic.limb_tree(6 + limbs * links, limbs)


TREES = {"branched": _branched_tree, "limbs": _limbs_tree, "humanoid": synthetic.humanoid_tree}


def _model_and_matrices(tree, worlds, seed=0):
    parent, body = tree()
    m = put_model(parent, body_of_dof=body)
    rng = np.random.default_rng(seed)
    Mv, Md = synthetic.random_mass_matrices(m, worlds, rng)
    return m, Mv, Md.astype(np.float64)


def _structure(m):
    return tree_ldl.tree_ldl_structure(m.M_rowadr, m.M_rownnz, m.M_colind)


@pytest.mark.parametrize("tree", ["branched", "limbs", "humanoid", "random7", "random8"])
@pytest.mark.parametrize("groups", [1, 2, 4])
def test_tree_oracle_matches_a_dense_solve(oracle, tree, groups):
    worlds = 37
    m, Mv, Md = _model_and_matrices(TREES.get(tree) or _random_forest(int(tree[6:])), worlds)
    structure = _structure(m)
    assert structure is not None
    plan = tree_ldl.plan_tree_ldl(*structure, groups)
    y = np.random.default_rng(1).normal(size=(worlds, m.nv)).astype(np.float32)
    x = oracle.tree_ldl_solve(structure, plan, Mv, y)
    want = np.stack([np.linalg.solve(a, b) for a, b in zip(Md, y)])
    np.testing.assert_allclose(x, want, rtol=2e-4, atol=2e-5)


def test_plans_cover_every_dof_once_and_split_limbs_off_a_trunk():
    """tests/test_tree_ldl.py:123-138."""
    m, _, _ = _model_and_matrices(_limbs_tree, 1)
    structure = _structure(m)
    for groups in (1, 2, 4):
        plan = tree_ldl.plan_tree_ldl(*structure, groups)
        dofs = sorted([*plan.trunk, *(k for nodes in plan.groups for k in nodes)])
        assert dofs == list(range(m.nv))
    single = tree_ldl.plan_tree_ldl(*structure, 1)
    split = tree_ldl.plan_tree_ldl(*structure, 4)
    assert not single.trunk
    assert split.trunk == tuple(range(6))
    assert sorted(len(nodes) for nodes in split.groups) == [6, 6, 6, 6]
    assert split.span < single.span


def test_tree_solve_is_used_only_where_it_beats_the_dense_cost():
    limbs, _, _ = _model_and_matrices(_limbs_tree, 1)
    assert tree_ldl.tree_ldl_beats_dense(tree_ldl.best_tree_ldl_plan(*_structure(limbs)))
    parent, body = synthetic._tree_from_joints([(6, -1)] + [(1, i) for i in range(40)])
    chain = put_model(parent, body_of_dof=body)
    plan = tree_ldl.best_tree_ldl_plan(*_structure(chain))
    assert plan.span > tree_ldl.MAX_SHORT_SPAN
    assert not tree_ldl.tree_ldl_beats_dense(plan)


def test_structure_check_rejects_rows_that_are_not_nested_ancestor_chains():
    m, _, _ = _model_and_matrices(_branched_tree, 1)
    rowadr, rownnz, colind = (np.array(a) for a in (m.M_rowadr, m.M_rownnz, m.M_colind))
    assert tree_ldl.tree_ldl_structure(rowadr, rownnz, colind) is not None
    bad = colind.copy()
    bad[rowadr[7]] = 1  # row 7 no longer starts with its root ancestor
    assert tree_ldl.tree_ldl_structure(rowadr, rownnz, bad) is None
    assert tree_ldl.tree_ldl_structure(rowadr, rownnz[:-1], colind) is None
    assert tree_ldl.tree_ldl_structure(np.zeros(0), np.zeros(0), np.zeros(0)) is None


@pytest.mark.parametrize("tree", ["humanoid", "snu", "random4", "random5", "random6"])
def test_compiled_program_matches_the_plan_interpreter(oracle, tree):
    """The instruction list the CUDA kernel runs, interpreted in numpy float64,
    solves M x = y (checks compilation independently of any kernel)."""
    worlds = 5
    build = {"humanoid": synthetic.humanoid_tree, "snu": synthetic.snu_tree}.get(tree) or _random_forest(int(tree[6:]))
    m, Mv, Md = _model_and_matrices(build, worlds)
    structure = _structure(m)
    y = np.random.default_rng(2).normal(size=(worlds, m.nv))
    for groups in (1, 3, 4):
        plan = tree_ldl.plan_tree_ldl(*structure, groups)
        program = tree_ldl._Program(*structure, plan)
        prog, ptr = program.encode()
        G = len(plan.groups)
        col = np.zeros((program.nslot, worlds))
        x = np.zeros((worlds, m.nv))

        def run(lo, hi):
            for op, dst, ab, c in prog[lo:hi]:
                a, b = ab & 0xFFFF, (ab >> 16) & 0xFFFF
                if op == tree_ldl.OP_LOAD_M:
                    col[dst] = Mv[:, a]
                elif op == tree_ldl.OP_LOAD_Y:
                    col[dst] = y[:, a]
                elif op == tree_ldl.OP_ZERO:
                    col[dst] = 0
                elif op == tree_ldl.OP_INV:
                    col[dst] = 1.0 / col[a]
                elif op == tree_ldl.OP_UPD:
                    col[dst] = col[dst] - col[a] * col[b] * col[c]
                elif op == tree_ldl.OP_SCALE:
                    col[dst] = col[dst] * col[a]
                elif op == tree_ldl.OP_SUBMUL:
                    col[dst] = col[dst] - col[a] * col[b]
                elif op == tree_ldl.OP_MUL:
                    col[dst] = col[a] * col[b]
                elif op == tree_ldl.OP_ADD:
                    col[dst] = col[dst] + col[a]
                elif op == tree_ldl.OP_MULSUB:
                    col[dst] = col[a] * col[b] - col[dst]
                elif op == tree_ldl.OP_STORE_X:
                    x[:, dst] = col[a]

        for j in range(G):
            run(ptr[j], ptr[j + 1])
        run(ptr[G], ptr[G + 1])
        for j in range(G):
            run(ptr[G + 1 + j], ptr[G + 2 + j])
        want = np.stack([np.linalg.solve(a, b) for a, b in zip(Md, y)])
        np.testing.assert_allclose(x, want, rtol=1e-5, atol=1e-6)


def _blocked_case(nv, worlds, rhs, seed=0):
    parent, body = synthetic.limb_tree(nv)
    m = put_model(parent, body_of_dof=body)
    rng = np.random.default_rng(seed)
    Mv, Md = synthetic.random_mass_matrices(m, worlds, rng)
    pad = indexed_factor._round_up(nv, 16)
    layout = indexed_factor.block_major_layout(indexed_factor.dense_index_table(m), pad, m.nM)
    ident = indexed_factor.pad_identity(nv, pad)
    y = rng.normal(size=(worlds, nv, rhs)).astype(np.float32)
    return m, Mv, Md.astype(np.float64), pad, layout, ident, y


@pytest.mark.parametrize("nv", [32, 35, 48, 56, 70])
def test_blocked_oracle_matches_numpy_and_reuses_its_factor(oracle, nv):
    worlds, rhs = 6, 3
    m, Mv, Md, pad, layout, ident, y = _blocked_case(nv, worlds, rhs)
    x, U = oracle.blocked_dense_factor_solve(nv, pad, layout, ident, Mv, y)
    want = np.stack([np.linalg.solve(a, b) for a, b in zip(Md, y)])
    np.testing.assert_allclose(x, want, rtol=2e-3, atol=2e-4)
    # U^T U reproduces M; the padded block is the identity
    for w in range(worlds):
        np.testing.assert_allclose(U[w, :nv, :nv].T @ U[w, :nv, :nv], Md[w], rtol=1e-4, atol=1e-4)
        np.testing.assert_array_equal(U[w, nv:, nv:], np.eye(pad - nv, dtype=np.float32))
    # a second solve from the stored factor is bit-identical to the fresh one
    x2, _ = oracle.blocked_dense_factor_solve(nv, pad, layout, ident, None, y, U=U, mode=1)
    np.testing.assert_array_equal(x, x2)


def test_plan_compiles_to_a_straight_line_kernel_without_a_gpu():
    """tree_ldl.py:362-390 builds its kernel from generated source at run time; so does
    imn_tree_ldl_compile (no GPU needed to compile).  Values that one warp keeps to
    itself become registers: only the trunk exchange is left in shared memory."""
    m, _, _ = _model_and_matrices(synthetic.humanoid_tree, 1)
    structure = _structure(m)
    plan = tree_ldl.plan_tree_ldl(*structure, 4)
    program = tree_ldl._Program(*structure, plan)
    prog, ptr = program.encode()
    kernel = tree_ldl.GeneratedKernel(prog, ptr, m.nv, m.nM, len(plan.groups), program.owner, program.nslot)
    info = kernel.info()
    assert info["code_bytes"] > 0
    assert 0 < info["shared_slots"] < program.nslot // 2
    src = info["source"]
    assert src.count("fmaf(") == int(np.isin(prog[:, 0], (tree_ldl.OP_UPD, tree_ldl.OP_SUBMUL, tree_ldl.OP_MULSUB)).sum())
    assert src.count("bar.sync") == 2 * len(plan.groups)
    # the values that cross warps live in cells of the staged tile whose entry the writing
    # warp has already read: the exchange takes no shared memory of its own
    import re

    body = src[src.index("switch (part)"):]
    assert len(set(re.findall(r"Mw\[\d+\]", body))) == info["shared_slots"] and "S[" not in body
    # malformed programs are rejected before any compilation
    from instantmimic_b200 import _lib

    bad = prog.copy()
    bad[0, 1] = program.nslot  # destination slot out of range
    with pytest.raises(_lib.ImnError, match="out of range"):
        tree_ldl.GeneratedKernel(bad, ptr, m.nv, m.nM, len(plan.groups), program.owner, program.nslot)


def test_mul_m_program_forms_every_row_in_table_order_and_compiles(oracle):
    """M v as a generated program: interpreted in float32 with one fmaf per stored entry it
    equals the oracle's mul_m bit for bit, every warp loads v only before the barriers, and
    the source compiles without a GPU with one fmaf per stored entry."""
    from instantmimic_b200.mjw_kernels import mul_m_generated as mg

    for tree in ("humanoid", "limbs", "branched"):
        worlds = 5
        m, Mv, _ = _model_and_matrices(TREES[tree], worlds)
        v = np.random.default_rng(5).normal(size=(worlds, m.nv)).astype(np.float32)
        want = np.zeros_like(v)
        oracle.mul_m(m, Mv, v, want)
        prog, ptr, nslot = mg.mul_m_program(m.M_mulm_rowadr, m.M_mulm_col, m.M_mulm_madr, m.nv)
        G = mg.WARPS
        assert ptr.size == 2 * G + 2 and ptr[G] == ptr[G + 1]  # empty trunk
        assert set(prog[: ptr[G], 0]) <= {tree_ldl.OP_LOAD_Y}
        assert tree_ldl.OP_LOAD_Y not in set(prog[ptr[G + 1] :, 0])
        x = _interpret_mul_m(prog, nslot, Mv, v, m.nv)
        np.testing.assert_array_equal(x.view(np.uint32), want.view(np.uint32))
        kernel = mg.GeneratedMulM(prog, ptr, m.nv, m.nM, nslot)
        src = kernel.info()["source"]
        assert "mul_m_generated(" in src and src.count("fmaf(") == int(m.M_mulm_rowadr[m.nv])
        assert kernel.info()["shared_slots"] == 0  # nothing crosses warps


def _random_forest(seed):
    """A bushy random forest of 20 to 60 dofs (several limbs, so that the plan has groups)."""
    rng = np.random.default_rng(seed)
    nv = int(rng.integers(20, 61))
    parent = np.full(nv, -1, np.int32)
    for i in range(1, nv):
        parent[i] = int(rng.integers(max(i - 6, 0), i)) if rng.random() < 0.97 else -1
    return lambda: (parent, None)


@pytest.mark.parametrize("tree", ["branched", "limbs", "humanoid", "snu", "random1", "random2", "random3"])
def test_lent_tile_cells_are_dead_before_they_are_reused(tree):
    """A cross-warp value may live in the tile cell of an entry of M only if that entry is
    read exactly once in the whole kernel, by the warp that first writes the value, before
    that write (nobody else ever looks at the cell again)."""
    import re

    build = TREES.get(tree) or (_random_forest(int(tree[6:])) if tree.startswith("random") else synthetic.snu_tree)
    m, _, _ = _model_and_matrices(build, 1)
    structure = _structure(m)
    plan = tree_ldl.best_tree_ldl_plan(*structure)
    program = tree_ldl._Program(*structure, plan)
    prog, ptr = program.encode()
    G = len(plan.groups)
    src = tree_ldl.GeneratedKernel(prog, ptr, m.nv, m.nM, G, program.owner, program.nslot).info()["source"]
    if "tileM" not in src:
        pytest.skip("tile not staged for this model")
    body = src[src.index("switch (part)"):]
    cases = re.split(r"\n  case \d+: \{\n", body)[1:]
    assert len(cases) == G
    lent = set(re.findall(r"Mw\[(\d+)\]", body))
    for e in lent:
        loads = [(j, mt.start()) for j, c in enumerate(cases) for mt in re.finditer(r"= Mt\[%s\];" % e, c)]
        assert len(loads) == 1, e
        j, at = loads[0]
        first_use = {k: c.find("Mw[%s]" % e) for k, c in enumerate(cases) if "Mw[%s]" % e in c}
        # the loading warp writes it first (an assignment), after its load
        assert j in first_use and first_use[j] > at
        assert re.match(r"Mw\[%s\] = " % e, cases[j][first_use[j]:])
        # program order across phases: the writer's first use sits in an earlier phase than, or
        # the same warp as, every other use (phases are separated by the two barriers)
        phase = lambda c, pos: c[:pos].count("bar.sync")  # noqa: E731
        for k, pos in first_use.items():
            assert k == j or phase(cases[k], pos) > phase(cases[j], first_use[j])


def _interpret_mul_m(prog, nslot, Mv, v, nv):
    """float32 interpretation of an M v program (a float32 product is exact in a double, so
    one rounding of the double sum is the fused multiply-add)."""
    from instantmimic_b200.mjw_kernels import mul_m_generated as mg

    col = np.zeros((nslot, Mv.shape[0]), np.float32)
    x = np.full((Mv.shape[0], nv), np.nan, np.float32)
    for op, dst, ab, _c in prog:
        a, b = ab & 0xFFFF, (ab >> 16) & 0xFFFF
        if op == tree_ldl.OP_LOAD_M:
            col[dst] = Mv[:, a]
        elif op == tree_ldl.OP_LOAD_Y:
            col[dst] = v[:, a]
        elif op == tree_ldl.OP_ZERO:
            col[dst] = 0
        elif op == mg.OP_MULADD:
            col[dst] = (col[a].astype(np.float64) * col[b].astype(np.float64) + col[dst].astype(np.float64)).astype(np.float32)
        elif op == tree_ldl.OP_STORE_X:
            x[:, dst] = col[a]
    return x


def test_mul_m_program_on_random_forests(oracle):
    """Random kinematic forests (several roots, chains, bushy trees, nv 1 .. 70), 1 to 4
    warps: the program returns the oracle's bits and every row is stored once."""
    from instantmimic_b200.mjw_kernels import mul_m_generated as mg

    rng = np.random.default_rng(11)
    for trial in range(12):
        nv = int(rng.integers(1, 71))
        style = trial % 3
        parent = np.full(nv, -1, np.int32)
        for i in range(1, nv):
            if style == 0:
                parent[i] = i - 1 if rng.random() < 0.9 else -1           # chains, now and then a new root
            elif style == 1:
                parent[i] = int(rng.integers(-1, i))                       # anything goes
            else:
                parent[i] = int(rng.integers(max(i - 3, -1), i))           # shallow and bushy
        m = put_model(parent)
        worlds = 3
        Mv, _ = synthetic.random_mass_matrices(m, worlds, rng)
        v = rng.normal(size=(worlds, nv)).astype(np.float32)
        want = np.zeros_like(v)
        oracle.mul_m(m, Mv, v, want)
        warps = 1 + trial % 4
        prog, ptr, nslot = mg.mul_m_program(m.M_mulm_rowadr, m.M_mulm_col, m.M_mulm_madr, nv, warps)
        assert ptr.size == 2 * warps + 2
        stores = prog[prog[:, 0] == tree_ldl.OP_STORE_X, 1]
        assert sorted(stores.tolist()) == list(range(nv))
        got = _interpret_mul_m(prog, nslot, Mv, v, nv)
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32), err_msg=f"trial {trial}")


# ---------------------------------------------------------------------------- GPU


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["contiguous", "padded"])
def test_generated_mul_m_returns_the_bits_of_mul_m(oracle, cuda_device, layout):
    """The generated M v (tiles by bulk copies when contiguous, plain loads for padded
    strides and the last partial tile) against the oracle, bit for bit."""
    import torch

    from instantmimic_b200 import mjw_model
    from instantmimic_b200.mjw_kernels import mul_m_generated as mg

    worlds = 4096 + 13
    m, Mv, _ = _model_and_matrices(TREES["humanoid"], worlds)
    v = np.random.default_rng(4).normal(size=(worlds, m.nv)).astype(np.float32)
    want = np.zeros_like(v)
    oracle.mul_m(m, Mv, v, want)
    md = mjw_model.to_device(m, cuda_device)
    kernel = mg.compile_mul_m(md)
    assert kernel is not None and kernel.staged
    pad = 0 if layout == "contiguous" else 3
    Mt = torch.zeros((worlds, m.nM + pad), device=cuda_device)[:, : m.nM]
    vt = torch.zeros((worlds, m.nv + pad), device=cuda_device)[:, : m.nv]
    Mt.copy_(torch.from_numpy(Mv)), vt.copy_(torch.from_numpy(v))
    out = torch.full((worlds, m.nv + pad), 7.0, device=cuda_device)[:, : m.nv]
    mg.mul_m(kernel, Mt, out, vt)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    np.testing.assert_array_equal(vt.cpu().numpy(), v)  # the input is left alone
    with pytest.raises(ValueError, match="alias"):
        mg.mul_m(kernel, Mt, vt, vt)


@pytest.mark.gpu
@pytest.mark.parametrize("tree", ["branched", "limbs", "humanoid"])
@pytest.mark.parametrize("groups", [1, 2, 4])
@pytest.mark.parametrize("generate", [True, False])
def test_tree_kernel_matches_oracle_bitwise(oracle, cuda_device, tree, groups, generate):
    """Both forms of the plan -- the straight-line kernel generated and compiled at run
    time, and the interpreted instruction list -- against the oracle, bit for bit."""
    import torch

    worlds = 37  # not a multiple of the 32 worlds a block serves
    m, Mv, Md = _model_and_matrices(TREES[tree], worlds)
    structure = _structure(m)
    plan = tree_ldl.plan_tree_ldl(*structure, groups)
    scratch = tree_ldl.compile_plan(structure, plan, cuda_device, generate)
    assert (scratch.kernel is not None) == generate
    y = np.random.default_rng(1).normal(size=(worlds, m.nv)).astype(np.float32)
    x = torch.zeros((worlds, m.nv), dtype=torch.float32, device=cuda_device)
    tree_ldl.tree_factor_solve(scratch, torch.from_numpy(Mv).to(cuda_device), x, torch.from_numpy(y).to(cuda_device))
    torch.cuda.synchronize()
    want = oracle.tree_ldl_solve(structure, plan, Mv, y)
    np.testing.assert_array_equal(x.cpu().numpy(), want)
    dense = np.stack([np.linalg.solve(a, b) for a, b in zip(Md, y)])
    np.testing.assert_allclose(x.cpu().numpy(), dense, rtol=2e-4, atol=2e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["contiguous", "padded", "offset"])
def test_generated_tree_kernel_tile_paths(oracle, cuda_device, layout):
    """The generated kernel brings a block's 32 worlds of M and y into shared memory:
    by TMA bulk copies when worlds are contiguous and 16-byte aligned, by plain loads
    for padded strides, an unaligned base, and the last partial block.  Same bits on
    every path."""
    import torch

    worlds = 32 * 3 + 5
    m, Mv, _ = _model_and_matrices(TREES["humanoid"], worlds)
    structure = _structure(m)
    plan = tree_ldl.best_tree_ldl_plan(*structure)
    scratch = tree_ldl.compile_plan(structure, plan, cuda_device, True)
    assert scratch.kernel is not None and "tileM" in scratch.kernel.info()["source"]
    y = np.random.default_rng(2).normal(size=(worlds, m.nv)).astype(np.float32)
    want = oracle.tree_ldl_solve(structure, plan, Mv, y)
    if layout == "contiguous":
        Mt, yt = torch.from_numpy(Mv).to(cuda_device), torch.from_numpy(y).to(cuda_device)
        x = torch.full((worlds, m.nv), 7.0, device=cuda_device)
    elif layout == "padded":
        Mt = torch.zeros((worlds, m.nM + 2), device=cuda_device)[:, : m.nM]
        yt = torch.zeros((worlds, m.nv + 6), device=cuda_device)[:, : m.nv]
        Mt.copy_(torch.from_numpy(Mv)), yt.copy_(torch.from_numpy(y))
        x = torch.full((worlds, m.nv + 1), 7.0, device=cuda_device)[:, : m.nv]
    else:  # contiguous worlds whose first element sits 4 bytes past a 16-byte boundary
        Mt = torch.zeros(worlds * m.nM + 1, device=cuda_device)[1:].view(worlds, m.nM)
        yt = torch.zeros(worlds * m.nv + 1, device=cuda_device)[1:].view(worlds, m.nv)
        Mt.copy_(torch.from_numpy(Mv)), yt.copy_(torch.from_numpy(y))
        x = torch.full((worlds, m.nv), 7.0, device=cuda_device)
    tree_ldl.tree_factor_solve(scratch, Mt, x, yt)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(x.cpu().numpy(), want)


@pytest.mark.gpu
def test_model_scratch_selects_tree_solve_and_solves_qacc_smooth(oracle, cuda_device):
    import torch

    from instantmimic_b200 import mjw_model
    from instantmimic_b200 import mjw_step_optimized as runtime

    m, d, Md = synthetic.make_workload("humanoid", 100, seed=4)
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(d, cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    assert scratch.tree_factor_solve is not None and scratch.dense_factor_solve is not None
    dd.qacc_smooth.zero_()
    runtime.fwd_acceleration_solve(md, dd, scratch)
    torch.cuda.synchronize()
    want = np.stack([np.linalg.solve(a.astype(np.float64), b) for a, b in zip(Md, d.qfrc_smooth)])
    np.testing.assert_allclose(dd.qacc_smooth.cpu().numpy(), want, rtol=2e-4, atol=2e-4)
    # the blocked dense path gives the same answer within its own tolerance
    out = torch.zeros_like(dd.qacc_smooth)
    runtime._factor_solve_i_dense(md, dd, dd.M, out, dd.qfrc_smooth, scratch.dense_factor_solve, retain_factor=True)
    torch.cuda.synchronize()
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=2e-3, atol=2e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("nv,rhs", [(32, 3), (35, 1), (35, 3), (48, 2), (56, 3), (70, 1), (70, 30), (79, 5)])
def test_blocked_kernel_matches_oracle_bitwise(oracle, cuda_device, nv, rhs):
    """rhs 30 at nv 70 exceeds the columns that ride through the factorisation, so
    part of them takes the substitution with the stored factor."""
    import torch

    from instantmimic_b200 import mjw_model

    worlds = 9
    m, Mv, Md, pad, layout, ident, y = _blocked_case(nv, worlds, rhs)
    md = mjw_model.to_device(m, cuda_device)
    dd = mjw_model.to_device(mjw_model.make_data(m, worlds, 4), cuda_device)
    scratch = indexed_factor.create_blocked_dense_factor_solve_scratch(md, dd, cuda_device)
    assert scratch is not None and scratch.pad == pad
    Mt = torch.from_numpy(Mv).to(cuda_device)
    yt = torch.from_numpy(y).to(cuda_device)
    active = torch.ones(worlds, dtype=torch.int32, device=cuda_device)
    active[3] = 0
    xt = torch.full_like(yt, 7.0)
    U = torch.zeros((worlds, pad, pad), dtype=torch.float32, device=cuda_device)
    indexed_factor.factor_multi_solve(scratch, Mt, yt, active, U, xt, rhs)
    torch.cuda.synchronize()
    want_x, want_U = oracle.blocked_dense_factor_solve(nv, pad, layout, ident, Mv, y)
    got = xt.cpu().numpy()
    live = np.arange(worlds) != 3
    np.testing.assert_array_equal(got[live], want_x[live])
    np.testing.assert_array_equal(got[3], 7.0)  # inactive world untouched
    np.testing.assert_array_equal(U.cpu().numpy()[live], want_U[live])
    # reuse of the stored factor == fresh solve, bit for bit
    x2 = torch.zeros_like(yt)
    active.fill_(1)
    active[3] = 0
    indexed_factor.multi_solve(scratch, U, yt, active, x2, rhs)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(x2.cpu().numpy()[live], got[live])
    dense = np.stack([np.linalg.solve(a, b) for a, b in zip(Md, y)])
    np.testing.assert_allclose(got[live], dense[live], rtol=2e-3, atol=2e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("nv,rhs", [(32, 1), (35, 1), (35, 3), (47, 1), (47, 2), (56, 1)])
def test_two_worlds_per_warp_return_the_same_bits(oracle, cuda_device, nv, rhs):
    """From 2048 worlds on, models whose columns fit 16 lanes (nv + right-hand sides that ride
    along <= 48) are factored two worlds per warp; (47, 2) and nv 56 stay on a warp per world.
    An odd batch leaves the last warp with one world; inactive worlds are skipped."""
    import torch

    from instantmimic_b200 import mjw_model

    worlds = 2051
    m, Mv, Md, pad, layout, ident, y = _blocked_case(nv, worlds, rhs)
    md = mjw_model.to_device(m, cuda_device)
    dd = mjw_model.to_device(mjw_model.make_data(m, worlds, 4), cuda_device)
    scratch = indexed_factor.create_blocked_dense_factor_solve_scratch(md, dd, cuda_device)
    Mt, yt = torch.from_numpy(Mv).to(cuda_device), torch.from_numpy(y).to(cuda_device)
    active = torch.ones(worlds, dtype=torch.int32, device=cuda_device)
    off = [3, 4, 5, 40, 2049, 2050]  # a lone inactive world, an inactive pair, the ragged end
    active[off] = 0
    live = active.cpu().numpy() != 0
    xt = torch.full_like(yt, 7.0)
    U = torch.full((worlds, pad, pad), 5.0, dtype=torch.float32, device=cuda_device)
    indexed_factor.factor_multi_solve(scratch, Mt, yt, active, U, xt, rhs)
    torch.cuda.synchronize()
    want_x, want_U = oracle.blocked_dense_factor_solve(nv, pad, layout, ident, Mv, y)
    np.testing.assert_array_equal(xt.cpu().numpy()[live], want_x[live])
    np.testing.assert_array_equal(xt.cpu().numpy()[~live], 7.0)
    np.testing.assert_array_equal(U.cpu().numpy()[live], want_U[live])
    np.testing.assert_array_equal(U.cpu().numpy()[~live], 5.0)
    x2 = torch.zeros_like(yt)
    indexed_factor.multi_solve(scratch, U, yt, active, x2, rhs)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(x2.cpu().numpy()[live], want_x[live])


@pytest.mark.gpu
def test_small_models_have_no_blocked_scratch(cuda_device):
    from instantmimic_b200 import mjw_model

    parent, body = synthetic.chain_tree(16)
    m = put_model(parent, body_of_dof=body)
    md = mjw_model.to_device(m, cuda_device)
    dd = mjw_model.to_device(mjw_model.make_data(m, 4, 4), cuda_device)
    assert indexed_factor.create_blocked_dense_factor_solve_scratch(md, dd, cuda_device) is None


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["contiguous", "padded"])
def test_mul_m_tile_paths_match_the_oracle(oracle, cuda_device, layout):
    """M v and the whole-batch hand-off at a batch large enough for the tiled kernel
    (32 worlds per block, tiles by TMA bulk copies when contiguous and aligned, plain
    loads for padded strides and the last partial tile), against the oracle bit for bit."""
    import torch

    from instantmimic_b200 import mjw_model
    from instantmimic_b200 import mjw_step_optimized as runtime

    worlds = 4096 + 13
    m, Mv, _ = _model_and_matrices(TREES["humanoid"], worlds)
    v = np.random.default_rng(3).normal(size=(worlds, m.nv)).astype(np.float32)
    want = np.zeros_like(v)
    oracle.mul_m(m, Mv, v, want)
    md = mjw_model.to_device(m, cuda_device)
    pad = 0 if layout == "contiguous" else 3
    Mt = torch.zeros((worlds, m.nM + pad), device=cuda_device)[:, : m.nM]
    vt = torch.zeros((worlds, m.nv + pad), device=cuda_device)[:, : m.nv]
    Mt.copy_(torch.from_numpy(Mv)), vt.copy_(torch.from_numpy(v))
    out = torch.full((worlds, m.nv + pad), 7.0, device=cuda_device)[:, : m.nv]
    from types import SimpleNamespace

    runtime.mul_m(md, SimpleNamespace(M=Mt, nworld=worlds), out, vt)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    if layout == "contiguous":
        d = mjw_model.make_data(m, worlds, 0)
        d.M[:], d.qacc_smooth[:] = Mv, v
        dd = mjw_model.to_device(d, cuda_device)
        dd.qacc.fill_(5.0), dd.qfrc_constraint.fill_(5.0), dd.solver_niter.fill_(5)
        runtime._rowless_handoff(md, dd)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(dd.efc.Ma.cpu().numpy().view(np.uint32), want.view(np.uint32))
        np.testing.assert_array_equal(dd.qacc.cpu().numpy(), v)
        assert float(dd.qfrc_constraint.abs().max()) == 0.0 and int(dd.solver_niter.abs().max()) == 0


@pytest.mark.gpu
def test_scratch_mul_m_call_takes_the_generated_kernel_from_4096_worlds(cuda_device):
    """make_optimized_fwd_position_scratch hands out the generated M v for batches that fill
    the GPU (the plain call below that); both return the bits of imn_mul_m."""
    import functools

    import torch

    from instantmimic_b200 import mjw_model
    from instantmimic_b200 import mjw_step_optimized as runtime

    for worlds, generated in ((4096, True), (64, False)):
        m, Mv, _ = _model_and_matrices(TREES["humanoid"], worlds)
        d = mjw_model.make_data(m, worlds, 0)
        d.M[:] = Mv
        d.qacc_smooth[:] = np.random.default_rng(8).normal(size=(worlds, m.nv)).astype(np.float32)
        md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(d, cuda_device)
        scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
        assert isinstance(scratch.mul_m_call, functools.partial) == generated
        a, b = torch.empty_like(dd.qacc_smooth), torch.empty_like(dd.qacc_smooth)
        scratch.mul_m_call(md, dd, a, dd.qacc_smooth)
        runtime.mul_m(md, dd, b, dd.qacc_smooth)
        torch.cuda.synchronize()
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))
