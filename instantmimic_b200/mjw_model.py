"""Model / Data containers with the fields the Newton solve reads.

The reference receives ``Model`` and ``Data`` from ``mujoco_warp.put_model`` /
``put_data`` (src/instantmimic/utils/mjw_model.py:60-82).  MuJoCo is not a
dependency of this package, so the same fields are built here from a kinematic
tree (one parent index per dof).  Field names, shapes and meaning follow
mujoco-warp so that ``solve_with_scratch`` works unchanged on either kind of
object.  Arrays are numpy on the host; ``to_device`` moves every array of a
container to a CUDA device as torch tensors.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields, is_dataclass, replace
from types import SimpleNamespace
from typing import Any

import numpy as np

from . import types

UPSTREAM_DENSE_NV_MAX = 60
# Newton pads nv + 1 to a multiple of 16: nv <= 79 keeps nv_pad <= 80
# (src/instantmimic/utils/mjw_model.py:29-30).
DENSE_NV_MAX = 79
WIDE_JTDAJ_BLOCK_DIM = 256


def newton_nv_pad(nv: int) -> int:
    """nv + 1 rounded up to 16 (src/instantmimic/utils/mjw_model.py:5-6)."""
    return ((nv + 1 + 15) // 16) * 16


@dataclass
class Option:
    iterations: int = 100
    ls_iterations: int = 50
    tolerance: Any = None  # float array, length 1 or nworld
    ls_tolerance: Any = None
    impratio_invsqrt: Any = None
    cone: int = types.ConeType.PYRAMIDAL
    solver: int = types.SolverType.NEWTON
    integrator: int = types.IntegratorType.IMPLICITFAST
    disableflags: int = 0
    warn_overflow: int = 0
    graph_conditional: bool = True
    timestep: Any = None  # float array, length 1 or nworld
    gravity: Any = None  # (1 or nworld, 3)


@dataclass
class Statistic:
    meaninertia: Any = None  # float array, length 1 or nworld


@dataclass
class Model:
    nv: int
    nv_pad: int
    opt: Option
    stat: Statistic
    is_sparse: bool
    dof_parentid: Any
    M_rowadr: Any
    M_rownnz: Any
    M_colind: Any
    M_hinit_i: Any  # row (dof) of every stored entry of M
    M_mulm_rowadr: Any
    M_mulm_col: Any
    M_mulm_madr: Any
    M_mulm_pack: Any  # col | madr << 16 per entry of the M_mulm tables
    block_dim: SimpleNamespace = field(
        default_factory=lambda: SimpleNamespace(linesearch_iterative=32)
    )
    # body tree, used only by the sparse-Hessian pattern
    body_parentid: Any = None
    body_dofadr: Any = None
    body_dofnum: Any = None
    neq: int = 0
    nflex: int = 0
    ntendon: int = 0
    geom_bodyid: Any = None
    nxn_geom_pair_filtered: Any = None
    # integrator-facing tables (joints, damping, M's dense-position index, actuators)
    nq: int = 0
    njnt: int = 0
    nu: int = 0
    jnt_type: Any = None
    jnt_dofadr: Any = None
    jnt_qposadr: Any = None
    dof_damping: Any = None
    M_elemid: Any = None  # (nv, nv): CSR entry of (i, j) for j an ancestor of i or i itself, else -1
    actuator_gaintype: Any = None
    actuator_biastype: Any = None
    actuator_dyntype: Any = None
    actuator_gainprm: Any = None  # (nu, 10)
    actuator_biasprm: Any = None  # (nu, 10)
    # body tree and the tables of the smooth-dynamics stages (tree_fusion / velocity_fusion)
    body_tree: Any = None  # list of int arrays: the bodies of each depth, world body first
    body_jntadr: Any = None
    body_jntnum: Any = None
    dof_bodyid: Any = None
    dof_armature: Any = None  # (1 or nworld, nv)

    @property
    def nactuator(self) -> int:
        return self.nu

    @property
    def nM(self) -> int:
        return int(self.M_colind.shape[0])


@dataclass
class Constraint:
    J: Any
    D: Any
    aref: Any
    frictionloss: Any
    force: Any
    state: Any
    Ma: Any
    # optional compact layout of J: (total rows, nv) with one int64 element offset per
    # world (see compact_jacobian); None for mujoco-warp's padded (nworld, njmax, nv)
    J_world_offset: Any = None


@dataclass
class Data:
    nworld: int
    njmax: int
    nefc: Any
    ne: Any
    nf: Any
    qacc_smooth: Any
    qacc_warmstart: Any
    qfrc_smooth: Any
    M: Any
    qacc: Any
    qfrc_constraint: Any
    efc: Constraint
    solver_niter: Any
    overflow: Any
    # integrator state and the actuator moments (mujoco-warp's per-world CSR); None
    # when only the solve is used
    qpos: Any = None
    qvel: Any = None
    time: Any = None
    moment_rownnz: Any = None
    moment_rowadr: Any = None
    moment_colind: Any = None
    actuator_moment: Any = None
    ctrl: Any = None
    # smooth-dynamics state (None when only the solve is used): per-body spatial
    # inertias (10), composite inertias, velocities, accelerations, forces (6), per-dof
    # motion axes and their time derivatives (6), subtree centres of mass (3)
    cinert: Any = None
    crb: Any = None
    cdof: Any = None
    cdof_dot: Any = None
    cvel: Any = None
    cacc: Any = None
    cfrc_int: Any = None
    qfrc_bias: Any = None
    subtree_com: Any = None


def ancestor_csr(dof_parentid: np.ndarray):
    """M's CSR over ancestors: each row lists the dof's ancestors root first and ends
    with the diagonal (src/instantmimic/utils/mjw_kernels/tree_ldl.py:3-8)."""
    parent = np.asarray(dof_parentid, dtype=np.int64)
    nv = parent.size
    rowadr, rownnz, colind, rowidx = [], [], [], []
    for k in range(nv):
        chain = []
        p = k
        while p >= 0:
            chain.append(p)
            p = int(parent[p])
        chain.reverse()
        rowadr.append(len(colind))
        rownnz.append(len(chain))
        colind += chain
        rowidx += [k] * len(chain)
    as32 = lambda v: np.asarray(v, dtype=np.int32)  # noqa: E731
    return as32(rowadr), as32(rownnz), as32(colind), as32(rowidx)


def mulm_tables(rowadr, rownnz, colind, nv: int):
    """Full symmetric rows of M for ``M v``: for each dof the stored entries of its
    row and column in ascending column order (upstream ``M_mulm_*`` tables read at
    src/instantmimic/utils/mjw_kernels/newton_fusion.py:171-176)."""
    rows: list[list[tuple[int, int]]] = [[] for _ in range(nv)]
    for k in range(nv):
        for q in range(int(rownnz[k])):
            e = int(rowadr[k]) + q
            c = int(colind[e])
            rows[k].append((c, e))
            if c != k:
                rows[c].append((k, e))
    adr, col, madr = [0], [], []
    for k in range(nv):
        for c, e in sorted(rows[k]):
            col.append(c)
            madr.append(e)
        adr.append(len(col))
    as32 = lambda v: np.asarray(v, dtype=np.int32)  # noqa: E731
    return as32(adr), as32(col), as32(madr)


def pack_mulm(col, madr) -> np.ndarray:
    """One word per entry of the M_mulm tables: col | madr << 16."""
    col = np.asarray(col).astype(np.int64)
    madr = np.asarray(madr).astype(np.int64)
    if col.size and (col.max() >= 1 << 16 or madr.max() >= 1 << 16):
        raise ValueError("M_mulm indices exceed 16 bits")
    return (col | (madr << 16)).astype(np.uint32).view(np.int32)


def put_model(
    dof_parentid,
    *,
    iterations: int = 100,
    ls_iterations: int = 50,
    tolerance: float = 1e-8,
    ls_tolerance: float = 0.01,
    meaninertia: float = 1.0,
    warmstart: bool = True,
    nv_pad: int | None = None,
    body_of_dof=None,
    timestep: float = 1.0 / 120.0,
) -> Model:
    """Host ``Model`` of a kinematic tree given one parent index per dof."""
    parent = np.asarray(dof_parentid, dtype=np.int32)
    nv = int(parent.size)
    rowadr, rownnz, colind, rowidx = ancestor_csr(parent)
    madr_row, mcol, madr = mulm_tables(rowadr, rownnz, colind, nv)
    opt = Option(
        iterations=iterations,
        ls_iterations=ls_iterations,
        tolerance=np.array([tolerance], np.float32),
        ls_tolerance=np.array([ls_tolerance], np.float32),
        impratio_invsqrt=np.array([1.0], np.float32),
        disableflags=0 if warmstart else int(types.DisableBit.WARMSTART),
        timestep=np.array([timestep], np.float32),
    )
    if body_of_dof is None:
        # one body per dof: a chain of single-dof bodies under the world body 0
        body_of_dof = np.arange(1, nv + 1)
    body_of_dof = np.asarray(body_of_dof, dtype=np.int32)
    nbody = int(body_of_dof.max()) + 1 if nv else 1
    body_dofadr = np.full(nbody, -1, np.int32)
    body_dofnum = np.zeros(nbody, np.int32)
    body_parentid = np.zeros(nbody, np.int32)
    for dof in range(nv):
        b = int(body_of_dof[dof])
        if body_dofadr[b] < 0:
            body_dofadr[b] = dof
            p = int(parent[dof])
            body_parentid[b] = int(body_of_dof[p]) if p >= 0 else 0
        body_dofnum[b] += 1
    # joints: a body with 6 dofs hangs on a free joint, with 3 on a ball joint, any other
    # count is that many hinges
    jnt_type, jnt_dofadr, jnt_qposadr, nq = [], [], [], 0
    body_jntnum = np.zeros(nbody, np.int32)
    for b in range(1, nbody):
        first, count = int(body_dofadr[b]), int(body_dofnum[b])
        if first < 0:
            continue
        body_jntnum[b] = 1 if count in (3, 6) else count
        kinds = [(types.JointType.FREE, 6, 7)] if count == 6 else (
            [(types.JointType.BALL, 3, 4)] if count == 3 else [(types.JointType.HINGE, 1, 1)] * count)
        for kind, ndof, npos in kinds:
            jnt_type.append(int(kind)), jnt_dofadr.append(first), jnt_qposadr.append(nq)
            first += ndof
            nq += npos
    order = np.argsort(jnt_dofadr, kind="stable")
    jnt_type = np.asarray(jnt_type, np.int32)[order]
    jnt_dofadr = np.asarray(jnt_dofadr, np.int32)[order]
    sizes = np.where(jnt_type == int(types.JointType.FREE), 7, np.where(jnt_type == int(types.JointType.BALL), 4, 1))
    jnt_qposadr = np.concatenate(([0], np.cumsum(sizes)[:-1])).astype(np.int32)
    # bodies are numbered in dof order, so a body's joints are consecutive
    body_jntadr = np.concatenate(([0], np.cumsum(body_jntnum)[:-1])).astype(np.int32)
    depth = np.zeros(nbody, np.int32)
    for b in range(1, nbody):
        depth[b] = depth[body_parentid[b]] + 1
    body_tree = [np.flatnonzero(depth == k).astype(np.int32) for k in range(int(depth.max()) + 1)]
    opt.gravity = np.array([[0.0, 0.0, -9.81]], np.float32)
    elemid = np.full((nv, nv), -1, np.int32)
    elemid[rowidx, colind] = np.arange(colind.size, dtype=np.int32)
    return Model(
        nq=int(nq),
        njnt=int(jnt_type.size),
        jnt_type=jnt_type,
        jnt_dofadr=jnt_dofadr,
        jnt_qposadr=jnt_qposadr,
        dof_damping=np.zeros(nv, np.float32),
        M_elemid=elemid,
        nv=nv,
        nv_pad=newton_nv_pad(nv) if nv_pad is None else int(nv_pad),
        opt=opt,
        stat=Statistic(meaninertia=np.array([meaninertia], np.float32)),
        is_sparse=False,
        dof_parentid=parent,
        M_rowadr=rowadr,
        M_rownnz=rownnz,
        M_colind=colind,
        M_hinit_i=rowidx,
        M_mulm_rowadr=madr_row,
        M_mulm_col=mcol,
        M_mulm_madr=madr,
        M_mulm_pack=pack_mulm(mcol, madr),
        body_parentid=body_parentid,
        body_dofadr=body_dofadr,
        body_dofnum=body_dofnum,
        body_tree=body_tree,
        body_jntadr=body_jntadr,
        body_jntnum=body_jntnum,
        dof_bodyid=body_of_dof.copy(),
        dof_armature=np.zeros((1, nv), np.float32),
        geom_bodyid=np.zeros(0, np.int32),
        nxn_geom_pair_filtered=np.zeros((0, 2), np.int32),
    )


def make_data(m: Model, nworld: int, njmax: int) -> Data:
    """Host ``Data`` with zeroed solver-facing buffers."""
    nv = m.nv
    f = lambda *s: np.zeros(s, np.float32)  # noqa: E731
    i = lambda *s: np.zeros(s, np.int32)  # noqa: E731
    return Data(
        nworld=nworld,
        njmax=njmax,
        nefc=i(nworld),
        ne=i(nworld),
        nf=i(nworld),
        qacc_smooth=f(nworld, nv),
        qacc_warmstart=f(nworld, nv),
        qfrc_smooth=f(nworld, nv),
        M=f(nworld, m.nM),
        qacc=f(nworld, nv),
        qfrc_constraint=f(nworld, nv),
        efc=Constraint(
            J=f(nworld, njmax, nv),
            D=f(nworld, njmax),
            aref=f(nworld, njmax),
            frictionloss=f(nworld, njmax),
            force=f(nworld, njmax),
            state=i(nworld, njmax),
            Ma=f(nworld, nv),
        ),
        solver_niter=i(nworld),
        overflow=i(nworld),
    )


def compact_jacobian(d: Data) -> Data:
    """Host ``Data`` whose ``efc.J`` holds only the ``nefc`` rows of each world, one world
    after the other (as MuJoCo C stores ``mjData.efc_J``), with ``efc.J_world_offset``
    naming each world's first element.  The solver reads the same rows; nothing else
    changes."""
    nefc = np.minimum(np.asarray(d.nefc), d.njmax).astype(np.int64)
    ld = int(d.efc.J.shape[2])
    live = np.arange(d.njmax)[None, :] < nefc[:, None]
    rows = np.ascontiguousarray(d.efc.J[live])  # world-major, rows ascending
    if rows.shape[0] == 0:
        rows = np.zeros((1, ld), np.float32)
    offsets = (np.concatenate(([0], np.cumsum(nefc)[:-1])) * ld).astype(np.int64)
    return replace(d, efc=replace(d.efc, J=rows, J_world_offset=offsets))


def _map_arrays(obj: Any, fn):
    """Copy of a (nested) dataclass / namespace with ``fn`` applied to every array."""
    if isinstance(obj, np.ndarray):
        return fn(obj)
    if isinstance(obj, list):
        return [_map_arrays(v, fn) for v in obj]
    if is_dataclass(obj) and not isinstance(obj, type):
        return replace(obj, **{f.name: _map_arrays(getattr(obj, f.name), fn) for f in fields(obj)})
    if isinstance(obj, SimpleNamespace):
        return SimpleNamespace(**{k: _map_arrays(v, fn) for k, v in vars(obj).items()})
    return obj


def to_device(obj: Any, device: Any = "cuda"):
    """Move every numpy array of a container to ``device`` as torch tensors."""
    import torch

    return _map_arrays(obj, lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device))


def to_host(obj: Any):
    """Inverse of ``to_device``: numpy copies of every tensor."""
    import torch

    def conv(o):
        if isinstance(o, torch.Tensor):
            return o.detach().cpu().numpy()
        if isinstance(o, np.ndarray):
            return o.copy()
        if isinstance(o, list):
            return [conv(v) for v in o]
        if is_dataclass(o) and not isinstance(o, type):
            return replace(o, **{f.name: conv(getattr(o, f.name)) for f in fields(o)})
        if isinstance(o, SimpleNamespace):
            return SimpleNamespace(**{k: conv(v) for k, v in vars(o).items()})
        return o

    return conv(obj)


def slice_worlds(d: Data, lo: int, hi: int) -> Data:
    """The contiguous world range [lo, hi) of a batch: the shard one GPU solves.

    Worlds are independent, so a shard is a view of every world-major array; nothing
    is exchanged between shards."""

    def cut(a):
        return a[lo:hi]

    if d.efc.J_world_offset is not None:
        raise ValueError("slice_worlds works on the padded efc.J layout")
    efc = replace(d.efc, **{f.name: cut(getattr(d.efc, f.name)) for f in fields(d.efc) if f.name != "J_world_offset"})
    out = replace(
        d,
        nworld=hi - lo,
        efc=efc,
        **{
            name: cut(getattr(d, name))
            for name in (
                "nefc",
                "ne",
                "nf",
                "qacc_smooth",
                "qacc_warmstart",
                "qfrc_smooth",
                "M",
                "qacc",
                "qfrc_constraint",
                "solver_niter",
                "overflow",
            )
        },
    )
    return out


def shard_bounds(nworld: int, nshards: int) -> list[tuple[int, int]]:
    """Contiguous, near-equal world ranges, one per GPU."""
    base, extra = divmod(nworld, nshards)
    out, lo = [], 0
    for g in range(nshards):
        hi = lo + base + (1 if g < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out
