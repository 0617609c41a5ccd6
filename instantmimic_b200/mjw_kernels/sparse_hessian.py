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


def _strict_ancestors(dof_parentid: np.ndarray) -> np.ndarray:
    """(nv, nv) bool: entry [d, a] says dof a is a strict tree ancestor of dof d.  A
    dof's parent precedes it, so one pass in dof order inherits the parent's row."""
    nv = int(dof_parentid.size)
    anc = np.zeros((nv, nv), bool)
    for d in range(nv):
        p = int(dof_parentid[d])
        if p >= 0:
            anc[d] = anc[p]
            anc[d, p] = True
    return anc


def _chain_masks(body_parentid, body_dofadr, body_dofnum, nv: int) -> np.ndarray:
    """(nbody, nv) bool: the dofs that move body b, i.e. its own and those of every
    body between it and the world.  Bodies follow their parents, so a body's mask is
    its parent's plus its own dofs."""
    nbody = int(body_parentid.size)
    masks = np.zeros((nbody, nv), bool)
    for b in range(1, nbody):
        masks[b] = masks[int(body_parentid[b])]
        first = int(body_dofadr[b])
        if first >= 0:
            masks[b, first : first + int(body_dofnum[b])] = True
    return masks


class _Coupling:
    """Symmetric dof-coupling matrix under construction."""

    def __init__(self, m: Any):
        self.nv = int(m.nv)
        anc = _strict_ancestors(_np(m.dof_parentid).astype(np.int64))
        self.P = anc | anc.T
        self.masks = _chain_masks(_np(m.body_parentid), _np(m.body_dofadr), _np(m.body_dofnum), self.nv)

    def bodies(self, ids) -> None:
        """One constraint row may touch all these bodies at once: every dof that moves
        one of them couples with every other."""
        ids = [int(b) for b in ids if int(b) > 0]
        if ids:
            self.dofs(np.flatnonzero(self.masks[ids].any(axis=0)))

    def dofs(self, ids) -> None:
        ids = np.asarray(ids, dtype=np.int64)
        self.P[np.ix_(ids, ids)] = True

    def adjacency(self) -> list[set[int]]:
        P = self.P.copy()
        np.fill_diagonal(P, False)
        return [set(int(b) for b in np.flatnonzero(P[a])) for a in range(self.nv)]


def _couple_equalities(m: Any, cp: _Coupling) -> None:
    """connect / weld rows couple two bodies (given directly or through two sites),
    joint rows couple the first dof of one or two joints; flex equalities live inside
    the flex couplings."""
    eq_type, obj1, obj2, objtype = (_np(getattr(m, n)) for n in ("eq_type", "eq_obj1id", "eq_obj2id", "eq_objtype"))
    for t, a, b, kind in zip(eq_type, obj1, obj2, objtype):
        t, a, b = int(t), int(a), int(b)
        if t in (EQ_FLEX, EQ_FLEXVERT, EQ_FLEXSTRAIN):
            continue
        if t in (EQ_CONNECT, EQ_WELD):
            if int(kind) == OBJ_SITE:
                site_bodyid = _np(m.site_bodyid)
                a, b = int(site_bodyid[a]), int(site_bodyid[b])
            cp.bodies([a, b])
        elif t == EQ_JOINT:
            jnt_dofadr = _np(m.jnt_dofadr)
            cp.dofs([int(jnt_dofadr[a])] + ([int(jnt_dofadr[b])] if b >= 0 else []))
        else:
            raise ValueError(f"equality constraint of type {t} has no coupling rule")


def _couple_flexes(m: Any, cp: _Coupling) -> None:
    """Bodies one flex row can touch (sparse_hessian.py:121-170).  A flex with
    interpolation couples all its nodes; otherwise each element couples its vertices'
    bodies (elasticity, edge equalities, contacts inside an element).  A geom that may
    collide with a flex (contype / conaffinity either way) adds its body to each of the
    flex's elements; two flexes that may collide (or one with itself when it
    self-collides) are coupled as wholes."""
    nflex = int(m.nflex)
    get = lambda name: _np(getattr(m, name))  # noqa: E731
    vertadr, vertnum, vertbody = get("flex_vertadr"), get("flex_vertnum"), get("flex_vertbodyid")
    elemnum, dataadr, dim, elem = get("flex_elemnum"), get("flex_elemdataadr"), get("flex_dim"), get("flex_elem")
    interp, nodeadr, nodenum, nodebody = get("flex_interp"), get("flex_nodeadr"), get("flex_nodenum"), get("flex_nodebodyid")
    whole: list[list[int]] = []          # all bodies of flex f
    elements: list[list[list[int]]] = []  # per flex, the body list of each element
    for f in range(nflex):
        if int(interp[f]) != 0:
            nodes = [int(b) for b in nodebody[int(nodeadr[f]) : int(nodeadr[f]) + int(nodenum[f])]]
            whole.append(nodes)
            elements.append([nodes] * int(elemnum[f]))
            cp.bodies(nodes)
            continue
        v0 = int(vertadr[f])
        whole.append([int(b) for b in vertbody[v0 : v0 + int(vertnum[f])]])
        per = int(dim[f]) + 1
        data = np.asarray(elem[int(dataadr[f]) : int(dataadr[f]) + per * int(elemnum[f])]).reshape(-1, per)
        elements.append([[int(vertbody[v0 + int(v)]) for v in row] for row in data])
        for bodies in elements[-1]:
            cp.bodies(bodies)
    f_type, f_aff = get("flex_contype"), get("flex_conaffinity")
    g_type, g_aff, geom_bodyid = get("geom_contype"), get("geom_conaffinity"), get("geom_bodyid")
    for f in range(nflex):
        hits = np.flatnonzero((int(f_type[f]) & g_aff) | (g_type & int(f_aff[f])))
        for g in hits:
            for bodies in elements[f]:
                cp.bodies([*bodies, int(geom_bodyid[g])])
    selfcollide = get("flex_selfcollide")
    for f in range(nflex):
        for h in range(f, nflex):
            may = (int(f_type[f]) & int(f_aff[h])) or (int(f_type[h]) & int(f_aff[f]))
            if may and (f != h or int(selfcollide[f])):
                cp.bodies(whole[f] + whole[h])


def hessian_pattern(m: Any, body_groups: Sequence[Sequence[int]]) -> list[set[int]]:
    """Upper bound of H's off-diagonal pattern as a dof adjacency (MuJoCo dof order):
    tree ancestry, every declared body group, equality constraints, flex couplings and
    the native collision candidates (sparse_hessian.py:62-170)."""
    cp = _Coupling(m)
    for group in body_groups:
        cp.bodies(group)
    if int(getattr(m, "neq", 0) or 0):
        _couple_equalities(m, cp)
    if int(getattr(m, "nflex", 0) or 0):
        _couple_flexes(m, cp)
    pairs = _np(getattr(m, "nxn_geom_pair_filtered", None))
    if pairs is not None and pairs.shape[0]:
        geom_bodyid = _np(m.geom_bodyid)
        for g1, g2 in np.asarray(pairs).reshape(-1, 2):
            cp.bodies([int(geom_bodyid[g1]), int(geom_bodyid[g2])])
    return cp.adjacency()


def _filled_upper(adj_e: list[set[int]]) -> np.ndarray:
    """Boolean upper triangle of the factor's structure for a symmetric pattern given as
    an adjacency in elimination order: eliminating k joins all its later neighbours."""
    n = len(adj_e)
    U = np.zeros((n, n), bool)
    for k, nb in enumerate(adj_e):
        later = [a for a in nb if a > k]
        U[k, later] = True
    for k in range(n):
        later = np.flatnonzero(U[k])
        if later.size > 1:
            block = U[np.ix_(later, later)]
            block |= np.triu(np.ones((later.size, later.size), bool), 1)
            U[np.ix_(later, later)] = block
    return U


def _etree_levels(U: np.ndarray) -> list[list[int]]:
    """Elimination-tree levels: a column's parent is its first later neighbour; a node
    sits one level above its deepest child."""
    n = U.shape[0]
    depth = np.zeros(n, np.int64)
    for k in range(n):
        later = np.flatnonzero(U[k])
        if later.size:
            depth[later[0]] = max(depth[later[0]], depth[k] + 1)
    return [[int(k) for k in np.flatnonzero(depth == lv)] for lv in range(int(depth.max(initial=0)) + 1)]


def _symbolic(adj_e: list[set[int]]):
    """Symbolic L'DL in elimination order: (row structure, column structure, levels)
    (sparse_hessian.py:192-212)."""
    U = _filled_upper(adj_e)
    n = U.shape[0]
    colstruct = [[int(i) for i in np.flatnonzero(U[k])] for k in range(n)]
    rowstruct = [[int(k) for k in np.flatnonzero(U[:, i])] for i in range(n)]
    return rowstruct, colstruct, _etree_levels(U)


def _team(nentries: int, maxterms: int, lanes: int) -> int:
    """Lanes per entry of one level: the power of two with the fewest steps, a step
    count being sweeps x (terms per lane + two per stage of the team's reduction
    tree) (sparse_hessian.py:215-221)."""
    log2 = np.arange(6)
    width = 1 << log2
    sweeps = -(-nentries // (lanes // width))
    steps = sweeps * (-(-maxterms // width) + 2 * log2)
    return int(width[int(np.argmin(steps))])


def _runs(ks: np.ndarray, a: np.ndarray, b: np.ndarray):
    """Maximal stretches over which the elimination index and both slots advance by one:
    (first a, first b, first k, length) per stretch."""
    if ks.size == 0:
        return []
    step = (np.diff(ks) != 1) | (np.diff(a) != 1) | (np.diff(b) != 1)
    starts = np.concatenate(([0], np.flatnonzero(step) + 1))
    ends = np.concatenate((starts[1:], [ks.size]))
    return [(int(a[s]), int(b[s]), int(ks[s]), int(e - s)) for s, e in zip(starts, ends)]


def build_plan(m: Any, body_groups: Sequence[Sequence[int]], block: int, path: str = "fused") -> SparseHessianPlan:
    """Symbolic factor and every index table of the numeric kernels (table semantics of
    sparse_hessian.py:229-402).  Elimination index e = nv - 1 - dof (leaves first).
    Slots are row-major over L's rows (a row's off-diagonal entries in ascending
    column order, then its diagonal), followed by one augmented row for the right-hand
    side."""
    nv, nv_pad = int(m.nv), int(m.nv_pad)
    n = nv
    adj = hessian_pattern(m, body_groups)
    orig = np.arange(n - 1, -1, -1)
    U = _filled_upper([{nv - 1 - a for a in adj[orig[e]]} for e in range(n)])
    L = U.T  # L[i, k]: entry (i, k), k < i, is in the factor
    levels = _etree_levels(U)
    # slot numbers: numpy walks the lower triangle (diagonal included) row-major
    slot_of = np.full((n + 1, n), -1, np.int64)
    rows, cols = np.nonzero(L | np.eye(n, dtype=bool))
    slot_of[rows, cols] = np.arange(rows.size)
    nfac = int(rows.size)
    slot_of[n] = nfac + np.arange(n)
    nslots = nfac + n
    if nslots >= 65536 or nslots > nv_pad * nv_pad:
        raise ValueError(f"sparse Hessian factor of {nslots} slots exceeds the packed (nv_pad, nv_pad) storage")
    Lx = np.vstack([L, np.ones((1, n), bool)])  # the augmented row meets every column
    lvl_ptr, lvl_team, ent_slot, ent_col, run_ptr, run_ab, run_kl = [0], [], [], [], [0], [], []
    nterms = 0
    for columns in levels:
        found = []  # (slot, diagonal column or -1, runs, term count)
        for j in columns:
            below = np.flatnonzero(U[j])
            for i in (j, *below.tolist(), n):
                # terms: earlier columns k present in both row j and row i (the diagonal
                # entry and the augmented row meet all of row j)
                ks = np.flatnonzero(L[j] if i == j else (L[j] & Lx[i]))
                found.append((int(slot_of[i, j]), j if i == j else -1, _runs(ks, slot_of[i, ks], slot_of[j, ks]),
                              int(ks.size)))
        # entries with many terms first (stable), so that a sweep's lanes finish together
        order = np.argsort([-f[3] for f in found], kind="stable")
        for q in order:
            s, c, runs, nt = found[int(q)]
            ent_slot.append(s)
            ent_col.append(c)
            run_ab += [a | (b << 16) for a, b, _, _ in runs]
            run_kl += [k | (ln << 16) for _, _, k, ln in runs]
            run_ptr.append(len(run_ab))
            nterms += nt
        lvl_ptr.append(len(ent_slot))
        lvl_team.append(_team(len(found), max(f[3] for f in found), block))
    # dense position and CSR entry of M behind every factor slot
    colind, rowi = _np(m.M_colind).astype(np.int64), _np(m.M_hinit_i).astype(np.int64)
    m_entry = np.full((nv, nv), -1, np.int64)
    m_entry[np.minimum(rowi, colind), np.maximum(rowi, colind)] = np.arange(colind.size)
    dof_hi, dof_lo = orig[rows], orig[cols]  # elimination row >= column  <=>  dof row <= column
    s_a, s_b = np.minimum(dof_hi, dof_lo), np.maximum(dof_hi, dof_lo)
    gat = s_a * nv_pad + s_b
    s_m = m_entry[s_a, s_b]
    pair = np.full((nv, nv), -1, np.int64)
    pair[s_a, s_b] = np.arange(nfac)
    reach = (pair >= 0) | (pair.T >= 0) | np.eye(nv, dtype=bool)
    words = (nv + 31) // 32
    bits = np.zeros((nv, words * 32), np.uint64)
    bits[:, :nv] = reach
    pmask = (bits.reshape(nv, words, 32) << np.arange(32, dtype=np.uint64)).sum(axis=2)
    # forward solve: unknowns by level, each with its row's slots and source columns
    f_row = [k for columns in levels for k in columns]
    f_lvl = np.concatenate(([0], np.cumsum([len(c) for c in levels])))
    row_nnz = L.sum(axis=1)
    row_first = np.where(row_nnz > 0, slot_of[np.arange(n), np.argmax(L, axis=1)], slot_of[np.arange(n), np.arange(n)])
    rk = cols[rows != cols]
    rk_ptr = np.concatenate(([0], np.cumsum(row_nnz)))
    # backward solve, root level first: a finished unknown pushes its column terms down
    # to the unknowns of its row; an unknown receives at most one push per level
    b_lvl, b_slot, b_src, b_dst = [0], [], [], []
    for columns in reversed(levels):
        for i in columns:
            js = np.flatnonzero(L[i])
            b_slot += slot_of[i, js].tolist()
            b_src += [i] * js.size
            b_dst += js.tolist()
        b_lvl.append(len(b_slot))
    for table in (lvl_ptr, ent_slot, run_ptr, f_lvl, f_row, row_first, rk_ptr, rk, b_lvl, b_slot, b_src, b_dst):
        if np.max(table, initial=0) >= 65536:
            raise ValueError("a sparse Hessian index table does not fit 16 bits")
    nw = block // 32
    if 2 * nfac + n >= nv_pad * nv_pad - 1:
        raise ValueError("packed H, factor and 1/D leave no room for the violation counter in hfactor")
    init_tile = 4 * nv + 4 if path == "fused" else 0
    if 4 * (nslots + n + 2 * nw + init_tile) > MAX_SHARED_BYTES:
        raise ValueError("the per-world factor exceeds the shared-memory budget of one block")
    raw = dict(
        lvl_ptr=lvl_ptr, lvl_team=lvl_team, ent_slot=ent_slot, ent_col=ent_col, run_ptr=run_ptr,
        run_ab=run_ab, run_kl=run_kl, orig=orig.tolist(), b_lvl=b_lvl, b_slot=b_slot, b_src=b_src, b_dst=b_dst,
        pair=pair.reshape(-1).tolist(), f_lvl=f_lvl.tolist(), f_row=f_row, row_start=row_first.tolist(),
        rk_ptr=rk_ptr.tolist(), rk=rk.tolist() or [0], pmask=pmask.reshape(-1).tolist(), s_a=s_a.tolist(),
        s_b=s_b.tolist(), s_m=s_m.tolist(), gat=gat.tolist(),
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


class NativePlan:
    """Owner of a plan uploaded by the library itself (``imn_sparse_plan_create``): one
    device allocation for all tables, freed with the object.  ``struct`` is the C-ABI
    plan with device pointers.  Equivalent to ``upload``, without torch."""

    def __init__(self, plan: SparseHessianPlan):
        import ctypes as C

        from .. import _lib

        host = host_struct(plan)
        self._keep = plan.tables  # the host tables must outlive the call only
        out = C.POINTER(abi.ImnSparsePlan)()
        _lib.check(_lib.lib().imn_sparse_plan_create(C.byref(host), C.byref(out)), "imn_sparse_plan_create")
        self._ptr = out
        self.struct = out.contents

    def close(self) -> None:
        ptr, self._ptr = getattr(self, "_ptr", None), None
        if ptr:
            from .. import _lib

            _lib.lib().imn_sparse_plan_destroy(ptr)

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass


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
    if int(getattr(m, "ntendon", 0) or 0):
        # tendon limit and friction-loss rows couple the dofs a tendon spans, which the
        # pattern does not cover: read the live model arrays (sparse_hessian.py:729-733);
        # a model that has tendons but lacks the arrays is refused
        limited = getattr(m, "tendon_limited_adr", None)
        loss = getattr(m, "tendon_frictionloss", None)
        if limited is None or loss is None or int(_np(limited).shape[0]) or bool((_np(loss) > 0).any()):
            return None, "tendon limit or frictionloss rows"
    from .. import binding

    const = binding.upstream_constants()
    if fused_runtime and newton_fusion.eligible(m, ctx, compact=compact):
        if int(getattr(m, "nflex", 0) or 0):
            return None, "flex objects on the fused path"
        path, width = "fused", block
    elif (
        int(m.opt.solver) == const["solver_newton"]
        and int(m.opt.cone) == const["cone_pyramidal"]
        and int(m.opt.integrator) != const["integrator_discrete"]
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
