"""Bottom-up rigid-body reductions: the subtree centres of mass, the composite inertias
with the joint-space inertia M, and the bias forces.

Host side of the reference's ``src/instantmimic/utils/mjw_kernels/tree_fusion.py``
(``TreeReductionScratch`` :27-33, ``create_tree_reduction_scratch`` :36-50, ``accumulate``
:138-170, ``subtree_com_accumulate`` :173-183, ``crb`` :186-206, ``rne`` :209-222).  The
kernels are in ``csrc/imn_body_tree.cu`` behind ``imn_body_tree_accumulate``, ``imn_crb``
and ``imn_rne``: a world is one warp that walks the levels of ``m.body_tree`` in its slice
of shared memory.

The reference's scratch selects between atomic and ordered ("deterministic") sums and
between one cooperative launch and one launch per level.  Here there is one kernel, it is
ordered (children join their parent in level-list order, one writer per parent) and it is
one launch; the two flags are kept on the scratch because callers read them
(``_select_tree_reduction``, mjw_step_optimized.py:2887-2894).  Without a scratch the
reference runs upstream mujoco-warp's per-level launches; this package has no second
path, so a missing scratch is an error.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from .. import _lib, abi, binding
from ..arrays import addr, device_of, elem_strides, is_contiguous, is_device, length, shape, to_host


@dataclass(frozen=True)
class TreeReductionScratch:
    bodies: Any
    offsets: Any
    levels: int
    deterministic: bool = False
    cooperative: bool = True
    # per parent (by position in ``bodies``) its children in level-list order; no
    # counterpart in the reference, which scans the whole next level for every parent
    child_ptr: Any = None
    child_ids: Any = None
    # lanes of a warp per world: the smallest of 8, 16, 32 that covers the widest level
    team_lanes: int = 32
    keep: tuple = field(default=(), repr=False, compare=False)


def level_tables(body_tree, body_parentid) -> dict[str, np.ndarray]:
    """Level list, level offsets and the per-parent child lists of a body tree."""
    levels = [np.asarray(to_host(level), dtype=np.int32).reshape(-1) for level in body_tree]
    parent = np.asarray(to_host(body_parentid), dtype=np.int32).reshape(-1)
    bodies = np.concatenate(levels).astype(np.int32)
    offsets = np.cumsum([0] + [len(level) for level in levels]).astype(np.int32)
    if sorted(bodies.tolist()) != list(range(len(parent))):
        raise ValueError("m.body_tree must list every body exactly once")
    position = np.empty(len(parent), dtype=np.int64)
    position[bodies] = np.arange(len(bodies))
    depth = np.searchsorted(offsets, position, side="right") - 1
    for body in range(1, len(parent)):
        if depth[body] != depth[parent[body]] + 1:
            raise ValueError(f"body {body} is not one level below its parent {parent[body]}")
    children: list[list[int]] = [[] for _ in bodies]
    for body in bodies.tolist():  # level-list order
        if body != 0:
            children[position[parent[body]]].append(body)
    child_ptr = np.cumsum([0] + [len(c) for c in children]).astype(np.int32)
    child_ids = np.asarray([b for c in children for b in c] or [0], dtype=np.int32)
    widest = max(len(level) for level in levels)
    team = 8 if widest <= 8 else (16 if widest <= 16 else 32)
    return {"bodies": bodies, "offsets": offsets, "child_ptr": child_ptr, "child_ids": child_ids, "team_lanes": team}


def _place(table: np.ndarray, like: Any):
    """A table next to ``like``: a torch tensor on its device, or the numpy array itself."""
    if is_device(like):
        import torch

        return torch.from_numpy(table).to(device_of(like))
    return table


def create_tree_reduction_scratch(m: Any, *, deterministic: bool = False, cooperative: bool = True):
    if not getattr(m, "body_tree", None):
        return None
    t = level_tables(m.body_tree, m.body_parentid)
    return TreeReductionScratch(
        _place(t["bodies"], m.body_parentid),
        _place(t["offsets"], m.body_parentid),
        len(m.body_tree),
        deterministic,
        cooperative,
        _place(t["child_ptr"], m.body_parentid),
        _place(t["child_ids"], m.body_parentid),
        int(t["team_lanes"]),
    )


def _need(scratch: Any, who: str) -> None:
    if scratch is None:
        raise RuntimeError(
            f"{who}: this library has no per-level upstream path; pass the scratch of create_tree_reduction_scratch")


def tree_struct(m: Any, scratch: TreeReductionScratch, *, dofs: bool = False, joints: bool = False,
                inertia: bool = False, gravity: bool = False) -> abi.ImnBodyTree:
    """The C struct over the model's tables; the flags name what the call reads."""
    s = abi.ImnBodyTree()
    s.nbody = length(m.body_parentid)
    s.nlevels = int(scratch.levels)
    s.body_parentid = addr(m.body_parentid)
    s.level_bodies, s.level_offsets = addr(scratch.bodies), addr(scratch.offsets)
    s.child_ptr, s.child_ids = addr(scratch.child_ptr), addr(scratch.child_ids)
    s.team_lanes = int(getattr(scratch, "team_lanes", 32))
    if dofs:
        s.nv = int(m.nv)
        s.body_dofadr, s.body_dofnum = addr(m.body_dofadr), addr(m.body_dofnum)
        s.dof_bodyid, s.dof_parentid = addr(m.dof_bodyid), addr(m.dof_parentid)
    if joints:
        s.body_jntadr, s.body_jntnum, s.jnt_type = addr(m.body_jntadr), addr(m.body_jntnum), addr(m.jnt_type)
    if inertia:
        s.nM = length(m.M_colind)
        arm = m.dof_armature
        dims = shape(arm)
        if dims[-1] != m.nv or not is_contiguous(arm):
            raise ValueError("m.dof_armature must be a contiguous (n, nv) or (nv) array")
        s.dof_armature, s.n_armature = addr(arm), (dims[0] if len(dims) == 2 else 1)
        s.M_rowidx, s.M_colind = addr(m.M_hinit_i), addr(m.M_colind)
    if gravity:
        g = m.opt.gravity
        dims = shape(g)
        if dims[-1] != 3 or not is_contiguous(g):
            raise ValueError("m.opt.gravity must be a contiguous (n, 3) or (3) array")
        s.gravity, s.n_gravity = addr(g), (dims[0] if len(dims) == 2 else 1)
        s.gravity_enabled = 0 if int(m.opt.disableflags) & binding.upstream_constants()["disable_gravity"] else 1
    return s


def _per_body(a: Any, nworld: int, nbody: int, width: int, name: str) -> int:
    """Address of a contiguous (nworld, nbody, width) float array (a Warp vector array has
    the same bytes with the last extent folded into its dtype)."""
    dims = tuple(shape(a))
    if dims not in ((nworld, nbody, width), (nworld, nbody)) or not is_contiguous(a):
        raise ValueError(f"{name} must be a contiguous ({nworld}, {nbody}, {width}) float array")
    return addr(a)


def _row_ld(a: Any) -> int:
    return elem_strides(a)[0]


def accumulate(m: Any, d: Any, values: Any, components: int, skip_root_parent: bool, scratch: TreeReductionScratch,
               stream=None) -> None:
    """values[:, parent] += values[:, body], deepest level first (tree_fusion.py:138-170)."""
    _need(scratch, "accumulate")
    nbody = length(m.body_parentid)
    ptr = _per_body(values, d.nworld, nbody, components, "values")
    with _lib.nvtx("imn_body_tree_accumulate"):
        rc = _lib.lib().imn_body_tree_accumulate(
            C.byref(tree_struct(m, scratch)), ptr, nbody * components, int(components), int(bool(skip_root_parent)),
            int(d.nworld), _lib.current_stream_handle(stream))
    _lib.check(rc, "imn_body_tree_accumulate")


def subtree_com_accumulate(m: Any, d: Any, scratch: TreeReductionScratch | None = None, stream=None) -> None:
    _need(scratch, "subtree_com_accumulate")
    accumulate(m, d, d.subtree_com, 3, False, scratch, stream)


def crb(m: Any, d: Any, scratch: TreeReductionScratch | None = None, stream=None) -> None:
    """d.crb and d.M from d.cinert and d.cdof (tree_fusion.py:186-206)."""
    _need(scratch, "crb")
    nbody = length(m.body_parentid)
    t = tree_struct(m, scratch, dofs=True, inertia=True)
    with _lib.nvtx("imn_crb"):
        rc = _lib.lib().imn_crb(
            C.byref(t), _per_body(d.cinert, d.nworld, nbody, 10, "d.cinert"),
            _per_body(d.cdof, d.nworld, m.nv, 6, "d.cdof"), _per_body(d.crb, d.nworld, nbody, 10, "d.crb"),
            addr(d.M), _row_ld(d.M), int(d.nworld), _lib.current_stream_handle(stream))
    _lib.check(rc, "imn_crb")


def rne(m: Any, d: Any, scratch: TreeReductionScratch | None = None, stream=None) -> None:
    """d.cacc, d.cfrc_int and d.qfrc_bias (tree_fusion.py:209-222)."""
    _need(scratch, "rne")
    nbody = length(m.body_parentid)
    t = tree_struct(m, scratch, dofs=True, gravity=True)
    with _lib.nvtx("imn_rne"):
        rc = _lib.lib().imn_rne(
            C.byref(t), _per_body(d.cinert, d.nworld, nbody, 10, "d.cinert"),
            _per_body(d.cvel, d.nworld, nbody, 6, "d.cvel"), _per_body(d.cdof, d.nworld, m.nv, 6, "d.cdof"),
            _per_body(d.cdof_dot, d.nworld, m.nv, 6, "d.cdof_dot"), addr(d.qvel), _row_ld(d.qvel),
            _per_body(d.cacc, d.nworld, nbody, 6, "d.cacc"), _per_body(d.cfrc_int, d.nworld, nbody, 6, "d.cfrc_int"),
            addr(d.qfrc_bias), _row_ld(d.qfrc_bias), int(d.nworld), _lib.current_stream_handle(stream))
    _lib.check(rc, "imn_rne")
