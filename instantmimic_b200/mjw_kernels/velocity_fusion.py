"""Depth-ordered body velocities.

Host side of the reference's ``src/instantmimic/utils/mjw_kernels/velocity_fusion.py``
(``com_vel`` :105-126, kernel :15-103); the kernel is ``com_vel_kernel`` in
``csrc/imn_body_tree.cu`` behind ``imn_com_vel``.  Without a tree scratch the reference
runs upstream mujoco-warp's per-level launches; this package has no second path.
"""

from __future__ import annotations

import ctypes as C
from typing import Any

from .. import _lib
from ..arrays import addr, length
from . import tree_fusion


def com_vel(m: Any, d: Any, tree: Any, stream=None) -> None:
    """d.cvel and d.cdof_dot from d.qvel and d.cdof."""
    tree_fusion._need(tree, "com_vel")
    nbody = length(m.body_parentid)
    t = tree_fusion.tree_struct(m, tree, dofs=True, joints=True)
    with _lib.nvtx("imn_com_vel"):
        rc = _lib.lib().imn_com_vel(
            C.byref(t), addr(d.qvel), tree_fusion._row_ld(d.qvel),
            tree_fusion._per_body(d.cdof, d.nworld, m.nv, 6, "d.cdof"),
            tree_fusion._per_body(d.cvel, d.nworld, nbody, 6, "d.cvel"),
            tree_fusion._per_body(d.cdof_dot, d.nworld, m.nv, 6, "d.cdof_dot"), int(d.nworld),
            _lib.current_stream_handle(stream))
    _lib.check(rc, "imn_com_vel")
