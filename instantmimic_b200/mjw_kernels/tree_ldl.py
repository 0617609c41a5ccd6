"""Tree-structured L'DL factor + solve of inertia-like matrices.

MuJoCo stores M (and the implicit-integration matrix M - h qDeriv, which has M's
sparsity) in CSR over each dof's ancestors: a row lists the dof's ancestors root
first and ends with the diagonal, and every ancestor's row is a prefix of it.
Eliminating dofs from the leaves towards the roots therefore creates no fill-in.

Interface and planning rules follow the reference's
``src/instantmimic/utils/mjw_kernels/tree_ldl.py`` (TreeLdlPlan :47-57, structure
check :66-91, planner :105-185, profitability gate :188-193, entry point :419-433).
The reference turns a plan into generated straight-line source per model and
compiles it at run time.  Here the plan is first compiled into a small instruction
list (``_Program``); ``csrc/imn_tree_jit.cu`` turns that list into straight-line CUDA C
and compiles it for sm_100a with NVRTC (values only one warp touches live in
registers), and ``csrc/imn_msolve.cu`` holds a generic kernel that interprets the same
list for machines without NVRTC.  Both map 32 worlds to a warp, one warp per group,
lane = world, and give the same bits.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any

import numpy as np

from .. import _lib, abi
from ..arrays import addr, elem_strides

MAX_GROUPS = 4
# Static shared memory the reference allows one block for the trunk exchange.
MAX_SHARED_BYTES = 48 * 1024
# The tree solve replaces the dense Cholesky when its critical path is short, or
# short relative to the dense flops per world (tree_ldl.py:33-44).
MAX_SHORT_SPAN = 4096
MIN_DENSE_TO_SPAN_RATIO = 8.0

# instruction opcodes of the interpreter (four int32 per instruction: op, dst, a | b << 16, c)
OP_LOAD_M, OP_LOAD_Y, OP_ZERO, OP_INV, OP_UPD, OP_SCALE, OP_SUBMUL, OP_MUL, OP_ADD, OP_STORE_X, OP_MULSUB = range(11)


@dataclass(frozen=True)
class TreeLdlPlan:
    """What `plan_tree_ldl` decides (the fields of the reference's plan, tree_ldl.py:43-53)."""

    groups: tuple[tuple[int, ...], ...]  # per group the dofs of its parts in elimination order (descending)
    trunk: tuple[int, ...]  # the dofs eliminated after all groups, ascending; closed under taking ancestors
    span: int  # update units on the longest path: the trunk's plus the heaviest group's
    dense_cost: int  # flops per world of a dense Cholesky over every tree of the model


@dataclass
class TreeFactorSolveScratch:
    plan: TreeLdlPlan
    groups: int
    cuda: bool
    struct: abi.ImnTreePlan
    tables: tuple  # device tensors the struct points into (kept alive)
    nv: int
    # generated straight-line kernel (None: the instruction list is interpreted)
    kernel: "GeneratedKernel | None" = None


class GeneratedKernel:
    """Owner of an ``ImnTreeKernel``: the plan's instruction list turned into CUDA C
    and compiled for sm_100a at run time, as the reference does through Warp
    (tree_ldl.py:362-390)."""

    def __init__(self, prog: np.ndarray, ptr: np.ndarray, nv: int, nM: int, groups: int, owner: int, nslot: int):
        prog = np.ascontiguousarray(prog, dtype=np.int32)
        ptr = np.ascontiguousarray(ptr, dtype=np.int32)
        handle = C.c_void_p()
        rc = _lib.lib().imn_tree_ldl_compile(
            prog.ctypes.data, ptr.ctypes.data, nv, nM, groups, owner, nslot, C.byref(handle)
        )
        _lib.check(rc, "imn_tree_ldl_compile")
        self.handle = handle

    def info(self) -> dict:
        slots, size, src = C.c_int32(), C.c_int64(), C.c_char_p()
        _lib.check(
            _lib.lib().imn_tree_ldl_kernel_info(self.handle, C.byref(slots), C.byref(size), C.byref(src)),
            "imn_tree_ldl_kernel_info",
        )
        return {"shared_slots": slots.value, "code_bytes": size.value, "source": src.value.decode()}

    def __del__(self):
        handle, self.handle = getattr(self, "handle", None), None
        if handle:
            try:
                _lib.lib().imn_tree_ldl_kernel_destroy(handle)
            except Exception:  # interpreter shutdown
                pass


def tree_ldl_structure(rowadr, rownnz, colind):
    """The CSR as tuples when it has the nested-ancestor form, else ``None``
    (tree_ldl.py:66-91).  Nested-ancestor form: every row ends with its own dof; a
    row of more than one entry is its parent's row (the dof before the last)
    followed by the dof itself.  By induction over the dofs this makes every
    ancestor's row a prefix of the row."""
    rowadr = np.asarray(rowadr, dtype=np.int64)
    rownnz = np.asarray(rownnz, dtype=np.int64)
    colind = np.asarray(colind, dtype=np.int64)
    nv = rowadr.size
    if nv == 0 or rownnz.size != nv or (rownnz < 1).any() or (rowadr < 0).any():
        return None
    if (rowadr + rownnz > colind.size).any():
        return None
    last = rowadr + rownnz - 1
    if (colind[last] != np.arange(nv)).any():
        return None
    for k in np.flatnonzero(rownnz > 1):
        head = colind[rowadr[k] : last[k]]
        p = int(head[-1])
        if p >= k or rownnz[p] != head.size or not np.array_equal(head, colind[rowadr[p] : rowadr[p] + head.size]):
            return None
    return tuple(rowadr.tolist()), tuple(rownnz.tolist()), tuple(colind.tolist())


def _tree(rowadr, rownnz, colind):
    """(parent, children) of the dof tree behind the CSR."""
    nv = len(rowadr)
    parent = [colind[rowadr[k] + rownnz[k] - 2] if rownnz[k] > 1 else -1 for k in range(nv)]
    children: list[list[int]] = [[] for _ in range(nv)]
    for k, p in enumerate(parent):
        if p >= 0:
            children[p].append(k)
    return parent, children


def _shared_bytes(rowadr, rownnz, groups: int, trunk) -> int:
    """Bytes of the reference's trunk exchange arrays for one block of 32 worlds: every
    group keeps its contribution to each trunk entry and trunk right-hand side, plus
    the trunk solution once (tree_ldl.py:98-102)."""
    if not trunk:
        return 0
    entries = int(sum(rownnz[i] for i in trunk))
    return 4 * 32 * (groups * (entries + len(trunk)) + len(trunk))


def _balance(parts, weight, groups: int):
    """Longest-processing-time packing: parts by falling weight (index breaks ties),
    each onto the currently lightest group (lowest group on ties).  Returns the
    heaviest group's load and the groups' part lists."""
    import heapq

    heap = [(0, g) for g in range(groups)]
    bins: list[list[int]] = [[] for _ in range(groups)]
    for r in sorted(parts, key=lambda r: (-weight[r], r)):
        load, g = heapq.heappop(heap)
        bins[g].append(r)
        heapq.heappush(heap, (load + weight[r], g))
    return max(load for load, _ in heap), bins


def plan_tree_ldl(rowadr, rownnz, colind, groups: int) -> TreeLdlPlan:
    """Plan with exactly ``groups`` groups and the shortest critical path found by the
    rule of tree_ldl.py:105-170: begin with whole trees as parts; keep cutting the
    heaviest part that can still be cut (its root dof moves to the trunk, its
    children become parts), and of all cuts seen keep the one whose heaviest group
    plus trunk is shortest.  Costs are in update units: eliminating a dof whose row
    has n entries takes n (n - 1) / 2 updates plus 2 n for scaling and the solves; a
    trunk dof costs 2 n more for the exchange."""
    import heapq

    nv = len(rowadr)
    parent, children = _tree(rowadr, rownnz, colind)
    own = [n * (n - 1) // 2 + 2 * n for n in rownnz]
    weight, size = list(own), [1] * nv
    for k in range(nv - 1, -1, -1):  # children before parents
        if parent[k] >= 0:
            weight[parent[k]] += weight[k]
            size[parent[k]] += size[k]
    roots = [k for k in range(nv) if parent[k] < 0]
    parts = set(roots)
    cuttable = [(-weight[r], r) for r in roots if children[r]]
    heapq.heapify(cuttable)
    trunk: list[int] = []
    trunk_cost = 0
    best_span, best_trunk, best_bins = None, None, None
    while True:
        heaviest, bins = _balance(parts, weight, groups)
        span = heaviest + trunk_cost
        if best_span is None or span < best_span:
            best_span, best_trunk, best_bins = span, sorted(trunk), bins
        if not cuttable:
            break
        _, r = heapq.heappop(cuttable)
        parts.discard(r)
        trunk.append(r)
        trunk_cost += own[r] + 2 * rownnz[r]
        for c in children[r]:
            parts.add(c)
            if children[c]:
                heapq.heappush(cuttable, (-weight[c], c))
    group_dofs = []
    for part_roots in best_bins:
        members, todo = [], list(part_roots)
        while todo:
            k = todo.pop()
            members.append(k)
            todo.extend(children[k])
        group_dofs.append(tuple(sorted(members, reverse=True)))  # leaves first
    return TreeLdlPlan(groups=tuple(group_dofs), trunk=tuple(best_trunk), span=best_span,
                       dense_cost=sum(size[r] ** 3 // 3 for r in roots))


def best_tree_ldl_plan(rowadr, rownnz, colind) -> TreeLdlPlan:
    """Of the plans with 1..MAX_GROUPS groups whose trunk exchange fits the
    shared-memory limit, the one with the shortest critical path (the fewest groups
    among equals).  One group needs no exchange, so a plan always exists."""
    fitting = []
    for groups in range(1, MAX_GROUPS + 1):
        plan = plan_tree_ldl(rowadr, rownnz, colind, groups)
        if _shared_bytes(rowadr, rownnz, groups, plan.trunk) <= MAX_SHARED_BYTES:
            fitting.append(plan)
    return min(fitting, key=lambda p: p.span)  # min keeps the first of equal spans


def tree_ldl_beats_dense(plan: TreeLdlPlan) -> bool:
    """The gate of tree_ldl.py:188-193."""
    return plan.span <= MAX_SHORT_SPAN or plan.dense_cost >= MIN_DENSE_TO_SPAN_RATIO * plan.span


class _Program:
    """Instruction streams of a plan: per group a forward and a backward stream, plus
    the trunk stream run by the owner group between two block barriers."""

    def __init__(self, rowadr, rownnz, colind, plan: TreeLdlPlan):
        nv, nM, G = len(rowadr), len(colind), len(plan.groups)
        trunk = set(plan.trunk)
        entries = [e for i in plan.trunk for e in range(rowadr[i], rowadr[i] + rownnz[i])]
        eslot = {e: n for n, e in enumerate(entries)}
        dslot = {i: n for n, i in enumerate(plan.trunk)}
        T, Tv = len(entries), len(plan.trunk)
        # slot map of one world's shared-memory column
        self.M0, self.S0, self.D0, self.X0 = 0, nM, nM + nv, nM + 2 * nv
        acc0 = nM + 3 * nv
        self.nslot = acc0 + G * (T + Tv)
        am = lambda j, e: acc0 + j * (T + Tv) + eslot[e]  # noqa: E731
        asol = lambda j, i: acc0 + j * (T + Tv) + T + dslot[i]  # noqa: E731
        m, s, d, x = (lambda e: e), (lambda k: self.S0 + k), (lambda k: self.D0 + k), (lambda k: self.X0 + k)

        def eliminate(k, out, target_m, target_s):
            start, count = rowadr[k], rownnz[k] - 1
            out.append((OP_INV, d(k), m(start + count), 0, 0))
            for p in range(count):
                anc = colind[start + p]
                for q in range(p + 1):
                    out.append((OP_UPD, target_m(anc, rowadr[anc] + q), m(start + p), m(start + q), d(k)))
            for p in range(count):
                out.append((OP_SCALE, m(start + p), d(k), 0, 0))
            for p in range(count):
                out.append((OP_SUBMUL, target_s(colind[start + p]), m(start + p), s(k), 0))

        def back_substitute(i, out):
            # x_i = s_i d_i - sum_p m_p x_anc(p).  The reference writes "x = s * d;
            # x = x - m0 * x0; x = x - m1 * x1; ..." (tree_ldl.py:258-266, 297-303); compiled
            # with contraction on, the first difference of two products fuses its LEFT
            # product, fma(s, d, -(m0 x0)), and every later term is fma(-m, x, acc)
            # (established against the reference's generated code run on a B200)
            start, count = rowadr[i], rownnz[i] - 1
            if count == 0:
                out.append((OP_MUL, x(i), s(i), d(i), 0))
                return
            out.append((OP_MUL, x(i), m(start), x(colind[start]), 0))
            out.append((OP_MULSUB, x(i), s(i), d(i), 0))
            for p in range(1, count):
                out.append((OP_SUBMUL, x(i), m(start + p), x(colind[start + p]), 0))

        self.forward, self.backward = [], []
        touched = []
        for j, nodes in enumerate(plan.groups):
            # what this group hands to the trunk: for every trunk ancestor of one of its dofs
            # (position p in that dof's row) the leading p + 1 entries of the ancestor's row,
            # and the ancestor's right-hand side
            trunk_entries, trunk_dofs = set(), set()
            for k in nodes:
                row = colind[rowadr[k] : rowadr[k] + rownnz[k] - 1]
                for p, anc in enumerate(row):
                    if anc in trunk:
                        trunk_dofs.add(int(anc))
                        trunk_entries.update(range(rowadr[anc], rowadr[anc] + p + 1))
            tm, ts = sorted(trunk_entries), sorted(trunk_dofs)
            touched.append((set(tm), set(ts)))
            f = []
            for k in nodes:
                for e in range(rowadr[k], rowadr[k] + rownnz[k]):
                    f.append((OP_LOAD_M, m(e), e, 0, 0))
            for k in nodes:
                f.append((OP_LOAD_Y, s(k), k, 0, 0))
            for e in tm:
                f.append((OP_ZERO, am(j, e), 0, 0, 0))
            for i in ts:
                f.append((OP_ZERO, asol(j, i), 0, 0, 0))
            tgt_m = lambda anc, index, j=j: index if anc not in trunk else am(j, index)  # noqa: E731
            tgt_s = lambda anc, j=j: s(anc) if anc not in trunk else asol(j, anc)  # noqa: E731
            for k in nodes:
                eliminate(k, f, tgt_m, tgt_s)
            self.forward.append(f)
            b, own = [], set()
            for i in reversed(nodes):
                back_substitute(i, b)
                own.add(i)
                b.append((OP_STORE_X, i, x(i), 0, 0))
            self.backward.append(b)
        t = []
        for e in entries:
            t.append((OP_LOAD_M, m(e), e, 0, 0))
            for j in range(G):
                if e in touched[j][0]:
                    t.append((OP_ADD, m(e), am(j, e), 0, 0))
        for i in plan.trunk:
            t.append((OP_LOAD_Y, s(i), i, 0, 0))
            for j in range(G):
                if i in touched[j][1]:
                    t.append((OP_ADD, s(i), asol(j, i), 0, 0))
        for k in reversed(plan.trunk):
            eliminate(k, t, lambda anc, index: index, lambda anc: s(anc))
        for i in plan.trunk:
            # the trunk solution lands in x(i), where the groups' backward streams read it
            back_substitute(i, t)
            t.append((OP_STORE_X, i, x(i), 0, 0))
        self.trunk = t
        self.owner = min(range(G), key=lambda j: sum(rownnz[k] ** 2 for k in plan.groups[j]))
        self.ntrunk, self.ntrunk_entries = Tv, T

    def encode(self):
        """(prog int32 (n, 4), prog_ptr int32 (3 G + 2)): streams are stored as
        forward_0..forward_{G-1}, trunk, backward_0..backward_{G-1}."""
        streams = [*self.forward, self.trunk, *self.backward]
        ptr, flat = [0], []
        for st in streams:
            for op, dst, a, b, c in st:
                if max(dst, a, b, c) >= 1 << 16:
                    raise ValueError("tree L'DL program exceeds 16-bit slots")
                flat.append((op, dst, a | (b << 16), c))
            ptr.append(len(flat))
        prog = np.asarray(flat, dtype=np.int32).reshape(-1, 4)
        return prog, np.asarray(ptr, dtype=np.int32)


def compile_plan(structure, plan: TreeLdlPlan, device: Any, generate: bool = True) -> TreeFactorSolveScratch:
    """Upload a plan's instruction streams, build its C-ABI struct and (``generate``)
    compile the streams into a straight-line kernel.  Without a run-time compiler on
    the machine the instruction list is interpreted instead; same results."""
    import torch

    rowadr, rownnz, colind = structure
    program = _Program(rowadr, rownnz, colind, plan)
    prog, ptr = program.encode()
    t_prog = torch.from_numpy(prog).to(device)
    t_ptr = torch.from_numpy(ptr).to(device)
    st = abi.ImnTreePlan()
    st.nv, st.nM = len(rowadr), len(colind)
    st.groups = len(plan.groups)
    st.ntrunk, st.ntrunk_entries = program.ntrunk, program.ntrunk_entries
    st.nslot = program.nslot
    st.prog, st.prog_ptr = addr(t_prog), addr(t_ptr)
    st.owner = program.owner
    kernel = None
    if generate:
        try:
            kernel = GeneratedKernel(prog, ptr, st.nv, st.nM, st.groups, st.owner, st.nslot)
        except _lib.ImnError as e:
            if "NVRTC" not in str(e):
                raise
    return TreeFactorSolveScratch(
        plan=plan, groups=len(plan.groups), cuda=True, struct=st, tables=(t_prog, t_ptr), nv=len(rowadr),
        kernel=kernel,
    )


def _to_numpy(a):
    from ..arrays import to_host

    return to_host(a)


def create_tree_factor_solve_scratch(m: Any, device: Any = "cuda", generate: bool = True) -> TreeFactorSolveScratch | None:
    """The compiled factor+solve for this model, or ``None`` when ineligible
    (tree_ldl.py:403-416)."""
    if getattr(m, "nv", 0) <= 0:
        return None
    arrays = [getattr(m, name, None) for name in ("M_rowadr", "M_rownnz", "M_colind")]
    if any(a is None for a in arrays):
        return None
    structure = tree_ldl_structure(*(_to_numpy(a) for a in arrays))
    if structure is None:
        return None
    plan = best_tree_ldl_plan(*structure)
    if not tree_ldl_beats_dense(plan):
        return None
    return compile_plan(structure, plan, device, generate)


def tree_factor_solve(scratch: TreeFactorSolveScratch, M: Any, x: Any, y: Any, stream=None) -> None:
    """x = M^-1 y for an M in the model's CSR layout (tree_ldl.py:419-433)."""
    for array in (M, x, y):
        if elem_strides(array)[1] != 1:
            raise ValueError("tree_factor_solve needs rows of contiguous floats")
    nworld = int(M.shape[0])
    if scratch.kernel is not None:
        with _lib.nvtx("imn_tree_ldl_compiled_solve"):
            rc = _lib.lib().imn_tree_ldl_compiled_solve(
                scratch.kernel.handle, addr(M), elem_strides(M)[0], addr(y), elem_strides(y)[0], addr(x),
                elem_strides(x)[0], nworld, _lib.current_stream_handle(stream),
            )
        _lib.check(rc, "imn_tree_ldl_compiled_solve")
        return
    rc = _lib.lib().imn_tree_ldl_solve(
        C.byref(scratch.struct), addr(M), elem_strides(M)[0], addr(y), elem_strides(y)[0], addr(x),
        elem_strides(x)[0], nworld, _lib.current_stream_handle(stream),
    )
    _lib.check(rc, "imn_tree_ldl_solve")
