"""Static-pattern sparse L'DL of the Newton Hessian.

H = M + J^T D J has a sparsity fixed by the model: M couples a dof with its tree
ancestors and a constraint row couples the dofs of the ancestor chains of the bodies
it touches.  The symbolic factor is computed once per model on the host; the numeric
factor runs left-looking over elimination-tree levels inside the world's warp.

Interface, gates and table semantics follow the reference's
``src/instantmimic/utils/mjw_kernels/sparse_hessian.py`` (pattern :62-118, symbolic
factor :192-212, lane teams :215-221, tables :229-402, gates :176-189, :705-758,
counter :786-801, validation helper :946-957).  The reference bakes the tables into
generated source text; here they are plain arrays uploaded once and read by generic
kernels (``csrc/imn_sparse.cuh``), so no code is generated per model.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

import numpy as np

from .. import abi, types
from ..arrays import addr

EQ_CONNECT, EQ_WELD, EQ_JOINT = 0, 1, 2
EQ_FLEX, EQ_FLEXVERT, EQ_FLEXSTRAIN = 4, 5, 6
OBJ_SITE = 6
# Largest per-world factor (bytes) the reference keeps in static shared memory.
MAX_SHARED_BYTES = 46 * 1024
# Above this fill density the dense blocked factor is kept (sparse_hessian.py:179-183).
MAX_DENSITY = 0.6
MIN_NV = 33  # below, the fused Newton uses the single-tile Cholesky
NONFUSED_MIN_NV = 80  # the upstream iteration keeps the dense factor below this


@dataclass
class SparseHessianPlan:
    nv: int
    nv_pad: int
    block: int
    nslots: int
    nterms: int
    levels: int
    density: float
    path: str  # "fused" (persistent Newton) or "nonfused" (upstream iteration)
    nfac: int
    tables: dict = field(repr=False)
    adjacency: list = field(repr=False)
    struct: Any = field(default=None, repr=False)
    device_tables: Any = field(default=None, repr=False)

    def __hash__(self):
        return id(self)


def _np(a):
    if a is None:
        return None
    from ..arrays import to_host

    return to_host(a)


def _chain(body: int, body_parentid, body_dofadr, body_dofnum) -> list[int]:
    """Dofs of a body and of all its ancestors."""
    out = []
    b = int(body)
    while b > 0:
        first = int(body_dofadr[b])
        if first >= 0:
            out.extend(range(first, first + int(body_dofnum[b])))
        b = int(body_parentid[b])
    return out


def hessian_pattern(m: Any, body_groups: Sequence[Sequence[int]]) -> list[set[int]]:
    """Upper bound of H's off-diagonal pattern as a dof adjacency (MuJoCo dof order):
    tree ancestry, every declared body group, equality constraints, and the native
    collision candidates (sparse_hessian.py:62-118)."""
    nv = int(m.nv)
    dof_parentid = _np(m.dof_parentid)
    body_parentid, body_dofadr, body_dofnum = _np(m.body_parentid), _np(m.body_dofadr), _np(m.body_dofnum)
    adj: list[set[int]] = [set() for _ in range(nv)]
    for d in range(nv):
        p = int(dof_parentid[d])
        while p >= 0:
            adj[d].add(p)
            adj[p].add(d)
            p = int(dof_parentid[p])

    def clique(bodies):
        dofs = sorted({d for b in bodies for d in _chain(b, body_parentid, body_dofadr, body_dofnum)})
        for a in dofs:
            adj[a].update(x for x in dofs if x != a)

    for group in body_groups:
        clique(group)
    if int(getattr(m, "neq", 0) or 0):
        eq_type, obj1, obj2 = _np(m.eq_type), _np(m.eq_obj1id), _np(m.eq_obj2id)
        objtype = _np(m.eq_objtype)
        site_bodyid = _np(getattr(m, "site_bodyid", None))
        jnt_dofadr = _np(getattr(m, "jnt_dofadr", None))
        for t, a, b, ot in zip(eq_type, obj1, obj2, objtype):
            if t in (EQ_CONNECT, EQ_WELD):
                if ot == OBJ_SITE:
                    a, b = site_bodyid[a], site_bodyid[b]
                clique((int(a), max(int(b), 0)))
            elif t in (EQ_FLEX, EQ_FLEXVERT, EQ_FLEXSTRAIN):
                continue
            elif t == EQ_JOINT:
                dofs = [int(jnt_dofadr[a])] + ([int(jnt_dofadr[b])] if b >= 0 else [])
                for x in dofs:
                    adj[x].update(y for y in dofs if y != x)
            else:
                raise ValueError(f"equality type {int(t)} is not supported")
    if int(getattr(m, "nflex", 0) or 0):
        raise ValueError("flex objects are not supported by this pattern builder")
    geom_bodyid = _np(getattr(m, "geom_bodyid", None))
    pairs = _np(getattr(m, "nxn_geom_pair_filtered", None))
    if pairs is not None and pairs.shape[0]:
        for g1, g2 in pairs:
            clique((int(geom_bodyid[g1]), int(geom_bodyid[g2])))
    return adj


def _symbolic(adj_e: list[set[int]]):
    """Symbolic L'DL in elimination order: fill, row/column structures and the
    elimination-tree levels (sparse_hessian.py:192-212)."""
    n = len(adj_e)
    upper = [{a for a in adj_e[k] if a > k} for k in range(n)]
    for k in range(n):
        later = sorted(upper[k])
        for pos, a in enumerate(later):
            upper[a].update(later[pos + 1 :])
    colstruct = [sorted(upper[k]) for k in range(n)]
    rowstruct: list[list[int]] = [[] for _ in range(n)]
    for k in range(n):
        for i in colstruct[k]:
            rowstruct[i].append(k)
    parent = [c[0] if c else -1 for c in colstruct]
    level = [0] * n
    for k in range(n):
        if parent[k] >= 0:
            level[parent[k]] = max(level[parent[k]], level[k] + 1)
    levels: list[list[int]] = [[] for _ in range(max(level, default=0) + 1)]
    for k in range(n):
        levels[level[k]].append(k)
    return rowstruct, colstruct, levels


def _team(nentries: int, maxterms: int, lanes: int) -> int:
    """Lanes per entry of one level: the power of two that minimises sweeps x
    (terms per lane + tree depth) (sparse_hessian.py:215-221)."""
    best, best_cost = 1, None
    for T in (1, 2, 4, 8, 16, 32):
        sweeps = -(-nentries // (lanes // T))
        cost = sweeps * (-(-maxterms // T) + 2 * int(np.log2(T)))
        if best_cost is None or cost < best_cost:
            best, best_cost = T, cost
    return best


def build_plan(m: Any, body_groups: Sequence[Sequence[int]], block: int, path: str = "fused") -> SparseHessianPlan:
    """Symbolic factor and every index table of the numeric kernels
    (sparse_hessian.py:229-402).  Elimination index e = nv - 1 - dof (leaves first).
    Slots are row-major over L's rows (row structure, then the diagonal), followed by
    one augmented row for the right-hand side."""
    nv, nv_pad = int(m.nv), int(m.nv_pad)
    adj = hessian_pattern(m, body_groups)
    n = nv
    orig = [nv - 1 - e for e in range(n)]
    adj_e = [{nv - 1 - a for a in adj[orig[e]]} for e in range(n)]
    rowstruct, colstruct, levels = _symbolic(adj_e)
    slot: dict[tuple[int, int], int] = {}
    for i in range(n):
        for k in rowstruct[i]:
            slot[i, k] = len(slot)
        slot[i, i] = len(slot)
    nfac = len(slot)
    rhs = nfac
    for k in range(n):
        slot[n, k] = len(slot)
    nslots = len(slot)
    if nslots >= 65536 or nfac + n > nv_pad * nv_pad:
        raise ValueError("sparse Hessian factor does not fit the packed layout")
    rs = [set(r) for r in rowstruct]
    lvl_ptr, lvl_team, ent_slot, ent_col, run_ptr, run_ab, run_kl = [0], [], [], [], [0], [], []
    nterms = 0
    for cols in levels:
        entries = []
        for j in cols:
            for i in [j, *colstruct[j], n]:
                ks = sorted(rs[j]) if i in (j, n) else sorted(rs[j] & rs[i])
                runs: list[list[int]] = []
                for k in ks:
                    a, b = slot[i, k], slot[j, k]
                    last = runs[-1] if runs else None
                    if last and k == last[2] + last[3] and a == last[0] + last[3] and b == last[1] + last[3]:
                        last[3] += 1
                    else:
                        runs.append([a, b, k, 1])
                entries.append((slot[i, j], j if i == j else -1, runs, len(ks)))
        entries.sort(key=lambda e: -e[3])  # stable: longest entries first
        for s, c, runs, nt in entries:
            ent_slot.append(s)
            ent_col.append(c)
            for a, b, k, ln in runs:
                run_ab.append(a | (b << 16))
                run_kl.append(k | (ln << 16))
            run_ptr.append(len(run_ab))
            nterms += nt
        lvl_ptr.append(len(ent_slot))
        lvl_team.append(_team(len(entries), max(e[3] for e in entries), block))
    by_slot = sorted(((s, ij) for ij, s in slot.items() if s < nfac))
    gat, s_a, s_b, s_m = [], [], [], []
    colind, rowi = _np(m.M_colind), _np(m.M_hinit_i)
    csr = {(min(int(r), int(c)), max(int(r), int(c))): e for e, (r, c) in enumerate(zip(rowi, colind))}
    for s, (i, j) in by_slot:
        a, b = sorted((orig[i], orig[j]))
        gat.append(a * nv_pad + b)
        s_a.append(a)
        s_b.append(b)
        s_m.append(csr.get((a, b), -1))
    f_lvl, f_row = [0], []
    for cols in levels:
        f_row += cols
        f_lvl.append(len(f_row))
    row_start = [slot[j, rowstruct[j][0]] if rowstruct[j] else slot[j, j] for j in range(n)]
    rk_ptr, rk = [0], []
    for j in range(n):
        rk += rowstruct[j]
        rk_ptr.append(len(rk))
    # backward solve, root level first: a level's finished unknowns push their column
    # terms to their descendants; an unknown receives at most one push per level
    b_lvl, b_slot, b_src, b_dst = [0], [], [], []
    for cols in reversed(levels):
        for i in cols:
            for j in rowstruct[i]:
                b_slot.append(slot[i, j])
                b_src.append(i)
                b_dst.append(j)
        b_lvl.append(len(b_slot))
    for a in (lvl_ptr, ent_slot, run_ptr, f_lvl, f_row, row_start, rk_ptr, rk, b_lvl, b_slot, b_src, b_dst):
        if max(a, default=0) >= 65536:
            raise ValueError("sparse Hessian tables exceed 16-bit indices")
    pair = [-1] * (nv * nv)
    for a in range(nv):
        for b in range(a, nv):
            i, j = nv - 1 - a, nv - 1 - b
            if (i, j) in slot and slot[i, j] < nfac:
                pair[a * nv + b] = slot[i, j]
    words = (nv + 31) // 32
    pmask = []
    for a in range(nv):
        bits = [0] * words
        for b in range(nv):
            if b == a or pair[min(a, b) * nv + max(a, b)] >= 0:
                bits[b // 32] |= 1 << (b % 32)
        pmask += bits
    nw = block // 32
    if 2 * nfac + n >= nv_pad * nv_pad - 1:
        raise ValueError("packed H and factor do not fit hfactor")
    init_tile = 4 * nv + 4 if path == "fused" else 0
    if 4 * (nslots + n + 2 * nw + init_tile) > MAX_SHARED_BYTES:
        raise ValueError("the factor does not fit the block's shared memory")
    raw = dict(
        lvl_ptr=lvl_ptr, lvl_team=lvl_team, ent_slot=ent_slot, ent_col=ent_col, run_ptr=run_ptr,
        run_ab=run_ab, run_kl=run_kl, orig=orig, b_lvl=b_lvl, b_slot=b_slot, b_src=b_src, b_dst=b_dst,
        pair=pair, f_lvl=f_lvl, f_row=f_row, row_start=row_start, rk_ptr=rk_ptr, rk=rk or [0],
        pmask=pmask, s_a=s_a, s_b=s_b, s_m=s_m, gat=gat,
    )
    raw["fsweep"], raw["bsweep"] = _pack_sweeps(raw) if path == "fused" else ([], [])
    tables = {}
    for name, dtype in abi.SPARSE_TABLES:
        vals = raw[name] if len(raw[name]) else [0]
        tables[name] = np.asarray(vals, dtype=np.int64).astype(dtype)
    if path != "fused":
        tables["fsweep"], tables["bsweep"] = tables["fsweep"][:0], tables["bsweep"][:0]
    return SparseHessianPlan(
        nv=nv, nv_pad=nv_pad, block=block, nslots=nslots, nterms=nterms, levels=len(levels),
        density=nfac / (nv * (nv + 1) / 2), path=path, nfac=nfac, tables=tables, adjacency=adj,
    )


def _pack_sweeps(raw: dict) -> tuple[list[int], list[int]]:
    """The level tables as one record per (sweep, lane) for the fused kernel (layout in
    include/imnewton.h).  A sweep is the 32 / team entries of a level that the warp
    works on at once; lanes of a team carry the same record."""
    lvl_ptr, lvl_team = raw["lvl_ptr"], raw["lvl_team"]
    run_ptr, run_ab, run_kl = raw["run_ptr"], raw["run_ab"], raw["run_kl"]
    fs: list[int] = []
    for lvl, team in enumerate(lvl_team):
        e0, e1, per = lvl_ptr[lvl], lvl_ptr[lvl + 1], 32 // team
        starts = list(range(e0, e1, per))
        for eb in starts:
            base = (2 if eb == starts[-1] else 0) | ((team.bit_length() - 1) << 2)
            for lane in range(32):
                e = eb + lane // team
                if e >= e1:
                    fs += [0, 0, 0, base]
                    continue
                r0, r1 = run_ptr[e], run_ptr[e + 1]
                extra = max(r1 - r0 - 1, 0)
                if extra > 255 or r0 + 1 > 0xFFFF or raw["ent_col"][e] + 1 > 0xFFFF:
                    raise ValueError("sparse plan exceeds the packed sweep record")
                fs += [
                    raw["ent_slot"][e] | ((raw["ent_col"][e] + 1) << 16),
                    run_ab[r0] if r1 > r0 else 0,
                    run_kl[r0] if r1 > r0 else 0,
                    base | 1 | (extra << 8) | ((r0 + 1) << 16),
                ]
    bs: list[int] = []
    b_lvl = raw["b_lvl"]
    for lvl in range(len(b_lvl) - 1):
        p0, p1 = b_lvl[lvl], b_lvl[lvl + 1]
        starts = list(range(p0, p1, 32))
        for pb in starts:
            last = (1 << 31) if pb == starts[-1] else 0
            for lane in range(32):
                p = pb + lane
                if p >= p1:
                    bs.append(last)
                    continue
                src, dst = raw["b_src"][p], raw["b_dst"][p]
                if src > 127 or dst > 127:
                    raise ValueError("sparse plan exceeds the packed sweep record")
                bs.append(raw["b_slot"][p] | (src << 16) | (dst << 23) | (1 << 30) | last)
    return fs, bs


def plan_struct(plan: SparseHessianPlan, arrays: dict) -> abi.ImnSparsePlan:
    """C-ABI struct over ``arrays`` (host numpy for the oracle, device tensors for CUDA)."""
    st = abi.ImnSparsePlan()
    st.nv, st.nv_pad, st.block = plan.nv, plan.nv_pad, plan.block
    st.nfac, st.nslots, st.nlevels = plan.nfac, plan.nslots, plan.levels
    st.nentries = int(plan.tables["ent_slot"].shape[0])
    st.nruns = int(plan.tables["run_ab"].shape[0])
    st.nback = int(plan.tables["b_slot"].shape[0])
    for name, _ in abi.SPARSE_TABLES:
        setattr(st, name, addr(arrays[name]))
    st.nfsweep = int(plan.tables["fsweep"].shape[0]) // 128
    st.nbsweep = int(plan.tables["bsweep"].shape[0]) // 32
    if not st.nfsweep:
        st.fsweep = st.bsweep = None
    return st


def host_struct(plan: SparseHessianPlan) -> abi.ImnSparsePlan:
    return plan_struct(plan, plan.tables)


def upload(plan: SparseHessianPlan, device: Any = "cuda") -> SparseHessianPlan:
    """Copy the tables to ``device`` and attach the device-side struct to the plan."""
    import torch

    dev = {}
    for name, _ in abi.SPARSE_TABLES:
        t = plan.tables[name]
        # torch has no uint16/uint32 arithmetic types; ship the raw bytes
        dev[name] = torch.from_numpy(t.view(np.uint8).copy()).to(device)
    plan.device_tables = dev
    plan.struct = plan_struct(plan, dev)
    return plan


def plan_for_model(m: Any, ctx: Any, body_groups, block: int, *, compact: bool = False,
                   fused_runtime: bool = True):
    """(plan, reason): the plan when the model qualifies, else ``None`` and why
    (sparse_hessian.py:705-758)."""
    from . import newton_fusion

    if body_groups is None:
        return None, "a custom contact producer did not declare its body groups"
    if not newton_fusion._on_cuda(m):
        return None, "fused Newton not eligible (CPU)"
    if int(m.nv) < MIN_NV:
        return None, f"nv {int(m.nv)} < {MIN_NV}"
    if int(getattr(m, "ntendon", 0) or 0) and getattr(m, "tendon_rows_possible", True):
        return None, "tendon limit or frictionloss rows"
    if fused_runtime and newton_fusion.eligible(m, ctx, compact=compact):
        if int(getattr(m, "nflex", 0) or 0):
            return None, "flex objects on the fused path"
        path, width = "fused", block
    elif (
        int(m.opt.solver) == int(types.SolverType.NEWTON)
        and int(m.opt.cone) == int(types.ConeType.PYRAMIDAL)
        and int(m.opt.integrator) != int(types.IntegratorType.DISCRETE)
        and m.opt.iterations > 0
        and not compact
        and not newton_fusion._sparse_compact(ctx)
    ):
        if int(m.nv) < NONFUSED_MIN_NV:
            return None, f"upstream iteration with nv {int(m.nv)} < {NONFUSED_MIN_NV}"
        path, width = "nonfused", 64 if int(m.nv) <= 96 else 128
    else:
        return None, "Newton solver structure not supported"
    try:
        plan = build_plan(m, body_groups, width, path)
    except ValueError as exc:
        return None, str(exc)
    if plan.density > MAX_DENSITY:
        return None, f"pattern density {plan.density:.2f} > {MAX_DENSITY}"
    return plan, "enabled"


def violation_counter(hfactor: Any, plan: SparseHessianPlan):
    """Fused path: per-world view of the pattern-violation counter, the last element
    of each world's ``hfactor``.  It counts active rows at the initial assembly and
    incremental H updates outside the pattern (must stay zero) and accumulates across
    solves; zero it when the plan is installed and after a nonzero read
    (sparse_hessian.py:786-801)."""
    if plan.path != "fused":
        raise ValueError("the violation counter exists on the fused path only")
    from ..arrays import as_torch

    last = plan.nv_pad - 1
    return as_torch(hfactor)[:, last, last]


def violations(hfactor: Any, plan: SparseHessianPlan) -> np.ndarray:
    return _np(violation_counter(hfactor, plan))


def nonfused_factor_solve(plan: SparseHessianPlan, ctx: Any, nworld: int, *, skip_unchanged: bool = False,
                          skip_noflip: bool = False, stream=None) -> None:
    """The upstream ``_cholesky_factorize_solve`` step with the sparse factor
    (sparse_hessian.py:849-894, 914-931): refactor the dense ``ctx.h`` when rows changed
    QUADRATIC state (always without ``skip_unchanged``), else solve with the factor kept in
    ``ctx.hfactor``; ``skip_noflip`` leaves worlds without state changes untouched.  Writes
    ``ctx.search``, ``ctx.search_dot``, ``ctx.newton_decrement``."""
    import ctypes as C

    from .. import _lib
    from ..arrays import elem_strides

    if plan.struct is None:
        raise RuntimeError("upload() the plan before using it on the device")
    state = ctx.state_changed_count if skip_noflip else ctx.quad_changed_count
    rc = _lib.lib().imn_sparse_factor_nonfused(
        C.byref(plan.struct), addr(ctx.done), addr(ctx.grad), elem_strides(ctx.grad)[0], addr(ctx.h),
        addr(ctx.quad_changed_count), addr(state), addr(ctx.hfactor), addr(ctx.search),
        elem_strides(ctx.search)[0], addr(ctx.search_dot), addr(ctx.newton_decrement), int(nworld),
        int(bool(skip_unchanged)), int(bool(skip_noflip)), _lib.current_stream_handle(stream),
    )
    _lib.check(rc, "imn_sparse_factor_nonfused")


def pattern_misses(h: np.ndarray, plan_adj: list[set[int]], tol: float = 0.0) -> int:
    """Nonzero upper-triangle entries of dense Hessians ``h`` (nworld, nv_pad, nv_pad)
    outside a dof adjacency (sparse_hessian.py:946-957)."""
    nv = len(plan_adj)
    mask = np.eye(nv, dtype=bool)
    for a in range(nv):
        for b in plan_adj[a]:
            mask[a, b] = True
    off = np.triu(np.ones((nv, nv), bool)) & ~mask
    return int((np.abs(h[:, :nv, :nv][:, off]) > tol).sum())
