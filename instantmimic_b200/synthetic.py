"""Seeded synthetic solver inputs with the shapes of the reference's models.

The reference obtains ``efc.*``, ``M`` and ``qfrc_smooth`` from MuJoCo-Warp's
collision and constraint pipeline, which is not part of this package.  The
generators here produce inputs with the same layout, sizes and value ranges:
kinematic trees transcribed from the reference's model files (dof counts and
parent structure only), tree-structured SPD mass matrices, pyramidal contact rows
in groups of four that touch the ancestor chain of one body, joint-limit rows on
single dofs, and optional equality / friction-loss rows.
"""

from __future__ import annotations

import numpy as np

from .mjw_model import Data, Model, make_data, put_model


def _tree_from_joints(joints):
    """joints: list of (ndof, parent_joint_index or -1) -> (dof_parentid, body_of_dof)."""
    parent, body, last = [], [], []
    for j, (ndof, pj) in enumerate(joints):
        prev = last[pj] if pj >= 0 else -1
        for _ in range(ndof):
            parent.append(prev)
            prev = len(parent) - 1
            body.append(j + 1)
        last.append(prev)
    return np.asarray(parent, np.int32), np.asarray(body, np.int32)


def humanoid_tree():
    """The PD humanoid of data/humanoid/mjcf/humanoid_pd.xml:50-127: free root, 8 ball
    joints, 4 hinges, nv 34."""
    joints = [
        (6, -1),  # 0 pelvis (free)
        (3, 0),  # 1 abdomen
        (3, 1),  # 2 neck
        (3, 1),  # 3 right shoulder
        (1, 3),  # 4 right elbow
        (3, 1),  # 5 left shoulder
        (1, 5),  # 6 left elbow
        (3, 0),  # 7 right hip
        (1, 7),  # 8 right knee
        (3, 8),  # 9 right ankle
        (3, 0),  # 10 left hip
        (1, 10),  # 11 left knee
        (3, 11),  # 12 left ankle
    ]
    return _tree_from_joints(joints)


def humanoid_mjcf(iterations: int = 50, ls_iterations: int = 50, tolerance: float = 1e-8) -> str:
    """MJCF text of a humanoid with the joint tree of ``humanoid_tree`` (free root, 8 ball
    joints, 4 hinges, nv 34), capsule links, box feet and a floor plane, with the
    benchmark's solver options (Newton, pyramidal cones, dense Jacobian).  Geometry is
    generated, not taken from the reference's model file: it serves the CPU baseline
    that steps MuJoCo C on a model of the same structure."""
    names = ["pelvis", "abdomen", "neck", "r_shoulder", "r_elbow", "l_shoulder", "l_elbow", "r_hip", "r_knee",
             "r_ankle", "l_hip", "l_knee", "l_ankle"]
    joints = [(6, -1), (3, 0), (3, 1), (3, 1), (1, 3), (3, 1), (1, 5), (3, 0), (1, 7), (3, 8), (3, 0), (1, 10),
              (3, 11)]
    # offset of each body in its parent's frame, and the link capsule's end point
    pos = {"pelvis": (0, 0, 0.98), "abdomen": (0, 0, 0.12), "neck": (0, 0, 0.32), "r_shoulder": (0, -0.18, 0.26),
           "r_elbow": (0, 0, -0.28), "l_shoulder": (0, 0.18, 0.26), "l_elbow": (0, 0, -0.28),
           "r_hip": (0, -0.09, -0.06), "r_knee": (0, 0, -0.42), "r_ankle": (0, 0, -0.41),
           "l_hip": (0, 0.09, -0.06), "l_knee": (0, 0, -0.42), "l_ankle": (0, 0, -0.41)}
    tip = {"pelvis": (0, 0, 0.08), "abdomen": (0, 0, 0.28), "neck": (0, 0, 0.14), "r_shoulder": (0, 0, -0.26),
           "r_elbow": (0, 0, -0.24), "l_shoulder": (0, 0, -0.26), "l_elbow": (0, 0, -0.24), "r_hip": (0, 0, -0.40),
           "r_knee": (0, 0, -0.39), "l_hip": (0, 0, -0.40), "l_knee": (0, 0, -0.39)}
    children: dict[int, list[int]] = {}
    for j, (_, pj) in enumerate(joints):
        children.setdefault(pj, []).append(j)
    vec = lambda v: " ".join(f"{x:g}" for x in v)  # noqa: E731

    def body(j: int, indent: str) -> str:
        name, ndof = names[j], joints[j][0]
        out = [f'{indent}<body name="{name}" pos="{vec(pos[name])}">']
        if ndof == 6:
            out.append(f'{indent}  <freejoint name="{name}"/>')
        elif ndof == 3:
            out.append(f'{indent}  <joint name="{name}" type="ball" damping="1"/>')
        else:
            out.append(f'{indent}  <joint name="{name}" type="hinge" axis="0 1 0" range="-140 5" damping="1"/>')
        if name.endswith("ankle"):
            out.append(f'{indent}  <geom name="{name}_foot" type="box" size="0.09 0.045 0.03" pos="0.045 0 -0.03"/>')
        else:
            out.append(f'{indent}  <geom name="{name}_link" type="capsule" size="0.05" '
                       f'fromto="0 0 0 {vec(tip[name])}" contype="0" conaffinity="0"/>')
        for c in children.get(j, []):
            out.append(body(c, indent + "  "))
        out.append(f"{indent}</body>")
        return "\n".join(out)

    return f"""<mujoco model="generated_humanoid">
  <compiler angle="degree"/>
  <option timestep="{1 / 120:.8f}" integrator="implicitfast" solver="Newton" cone="pyramidal" jacobian="dense"
          iterations="{iterations}" ls_iterations="{ls_iterations}" tolerance="{tolerance:g}"/>
  <default><geom density="1000" friction="1 0.005 0.0001"/></default>
  <worldbody>
    <geom name="floor" type="plane" size="0 0 0.05" conaffinity="1"/>
{body(0, "    ")}
  </worldbody>
</mujoco>
"""


def snu_tree():
    """The SNU muscle humanoid's joint tree, transcribed from
    data/snu_humanoid/mjcf/include/body.xml:50-897 (bodies in document order, which
    is MuJoCo's body order): free root, 14 ball joints, 8 hinges, nv 56."""
    joints = [
        (6, -1),  # 0 Pelvis (free)
        (3, 0),  # 1 FemurR
        (1, 1),  # 2 TibiaR
        (3, 2),  # 3 TalusR
        (1, 3),  # 4 FootThumbR
        (1, 3),  # 5 FootPinkyR
        (3, 0),  # 6 FemurL
        (1, 6),  # 7 TibiaL
        (3, 7),  # 8 TalusL
        (1, 8),  # 9 FootThumbL
        (1, 8),  # 10 FootPinkyL
        (3, 0),  # 11 Spine
        (3, 11),  # 12 Torso
        (3, 12),  # 13 Neck
        (3, 13),  # 14 Head
        (3, 12),  # 15 ShoulderR
        (3, 15),  # 16 ArmR
        (1, 16),  # 17 ForeArmR
        (3, 17),  # 18 HandR
        (3, 12),  # 19 ShoulderL
        (3, 19),  # 20 ArmL
        (1, 20),  # 21 ForeArmL
        (3, 21),  # 22 HandL
    ]
    parent, body = _tree_from_joints(joints)
    assert parent.size == 56, parent.size
    return parent, body


def g1_like_tree():
    """Shape stand-in for the Unitree G1 (nv 35: free root and 29 hinges in chains of
    6/6/3/7/7; the model itself is not distributed with the reference)."""
    joints = [(6, -1)]
    for _ in range(2):  # legs, 6 hinges each
        prev = 0
        for _ in range(6):
            joints.append((1, prev))
            prev = len(joints) - 1
    prev = 0
    for _ in range(3):  # waist
        joints.append((1, prev))
        prev = len(joints) - 1
    waist = prev
    for _ in range(2):  # arms, 7 hinges each
        prev = waist
        for _ in range(7):
            joints.append((1, prev))
            prev = len(joints) - 1
    parent, body = _tree_from_joints(joints)
    assert parent.size == 35
    return parent, body


def limb_tree(nv: int, limbs: int = 4):
    """Free root plus ``limbs`` hinge chains sharing the remaining dofs."""
    if nv < 6:
        return _tree_from_joints([(nv, -1)])
    joints = [(6, -1)]
    rest = nv - 6
    per, extra = divmod(rest, limbs)
    for c in range(limbs):
        prev = 0
        for _ in range(per + (1 if c < extra else 0)):
            joints.append((1, prev))
            prev = len(joints) - 1
    return _tree_from_joints(joints)


def chain_tree(nv: int):
    """Free root, then ball joints and hinges in one chain (the layout of the
    reference's parity models, tests/test_mjw_newton_fusion.py:99-115)."""
    balls, hinges = divmod(max(nv - 6, 0), 3)
    joints = [(min(nv, 6), -1)]
    for _ in range(balls):
        joints.append((3, len(joints) - 1))
    for _ in range(hinges):
        joints.append((1, len(joints) - 1))
    return _tree_from_joints(joints)


def multi_chain_tree(chains: int, nv: int):
    """``chains`` separate floating chains (tests/test_mjw_newton_fusion.py:118-142)."""
    per, extra = divmod(nv, chains)
    joints = []
    for c in range(chains):
        n = per + (1 if c < extra else 0)
        joints.append((6, -1))
        for _ in range(n - 6):
            joints.append((1, len(joints) - 1))
    return _tree_from_joints(joints)


def ancestor_masks(dof_parentid: np.ndarray) -> np.ndarray:
    """mask[d, a] = True when a is d or one of its ancestors."""
    nv = dof_parentid.size
    mask = np.zeros((nv, nv), bool)
    for d in range(nv):
        p = d
        while p >= 0:
            mask[d, p] = True
            p = int(dof_parentid[p])
    return mask


def random_mass_matrices(m: Model, nworld: int, rng: np.random.Generator):
    """(W, nM) CSR values of M = L^T D L, L unit lower on the ancestor pattern with
    N(0, 0.3) entries and D ~ U(0.5, 2); also returns the dense matrices."""
    nv, nM = m.nv, m.nM
    rows = np.asarray(m.M_hinit_i)
    cols = np.asarray(m.M_colind)
    offdiag = rows != cols
    out = np.empty((nworld, nM), np.float32)
    dense_all = np.empty((nworld, nv, nv), np.float32)
    chunk = max(1, min(nworld, (1 << 24) // max(nv * nv, 1)))
    for lo in range(0, nworld, chunk):
        hi = min(nworld, lo + chunk)
        n = hi - lo
        L = np.zeros((n, nv, nv), np.float32)
        vals = rng.normal(0.0, 0.3, (n, nM)).astype(np.float32)
        L[:, rows[offdiag], cols[offdiag]] = vals[:, offdiag]
        L[:, np.arange(nv), np.arange(nv)] = 1.0
        D = rng.uniform(0.5, 2.0, (n, nv)).astype(np.float32)
        dense = np.einsum("wki,wk,wkj->wij", L, D, L, optimize=True).astype(np.float32)
        dense = 0.5 * (dense + dense.transpose(0, 2, 1))
        out[lo:hi] = dense[:, rows, cols]
        dense_all[lo:hi] = dense
    return out, dense_all


def make_problem(
    m: Model,
    nworld: int,
    njmax: int,
    seed: int = 0,
    *,
    nefc_range: tuple[int, int] | None = None,
    ne: int = 0,
    nf: int = 0,
    rows: str = "contacts",
    rowless_fraction: float = 0.0,
    warmstart_scale: float = 0.1,
    poison: bool = False,
    d_range: tuple[float, float] = (0.1, 10.0),
    couple: bool = True,
) -> tuple[Data, np.ndarray]:
    """Seeded solver inputs for ``nworld`` worlds; returns (Data, dense M).

    rows = "contacts": inequality rows come in groups of four pyramid edges
    (Jn +- mu Jt1, Jn +- mu Jt2) on the ancestor chain of one random dof, followed by
    single-dof joint-limit rows.  rows = "generic": every row is N(0,1) on the union
    of the ancestor chains of one or two random dofs (of one only with ``couple=False``, so that every row stays
    inside the tree-ancestry pattern).  Rows [0, ne) are equality rows,
    [ne, ne+nf) friction-loss rows on single dofs.  ``poison`` fills rows at and
    beyond nefc with NaN so that a kernel that reads them is caught.
    """
    rng = np.random.default_rng(seed)
    nv = m.nv
    d = make_data(m, nworld, njmax)
    parent = np.asarray(m.dof_parentid)
    masks = ancestor_masks(parent).astype(np.float32)
    lo, hi = nefc_range if nefc_range is not None else (njmax // 4, njmax)
    hi = min(hi, njmax)
    lo = min(max(lo, ne + nf), hi)
    nefc = rng.integers(lo, hi + 1, nworld).astype(np.int32)
    if rowless_fraction > 0:
        nefc[rng.random(nworld) < rowless_fraction] = 0
    d.nefc[:] = nefc
    d.ne[:] = np.where(nefc > 0, ne, 0)
    d.nf[:] = np.where(nefc > 0, nf, 0)
    Mv, Mdense = random_mass_matrices(m, nworld, rng)
    d.M[:] = Mv

    J = d.efc.J
    R = njmax
    if rows == "generic":
        a = rng.integers(0, nv, (nworld, R))
        b = rng.integers(0, nv, (nworld, R))
        two = (rng.random((nworld, R)) < 0.5) & couple
        mask = masks[a]
        mask = np.maximum(mask, masks[b] * two[..., None])
        J[:] = rng.normal(0.0, 1.0, (nworld, R, nv)).astype(np.float32) * mask
    else:
        ncon = (R + 3) // 4
        body = rng.integers(0, nv, (nworld, ncon))
        mk = masks[body]  # (W, ncon, nv)
        jn = rng.normal(0.0, 1.0, (nworld, ncon, nv)).astype(np.float32) * mk
        jt1 = rng.normal(0.0, 1.0, (nworld, ncon, nv)).astype(np.float32) * mk
        jt2 = rng.normal(0.0, 1.0, (nworld, ncon, nv)).astype(np.float32) * mk
        mu = rng.uniform(0.5, 1.0, (nworld, ncon, 1)).astype(np.float32)
        quad = np.stack([jn + mu * jt1, jn - mu * jt1, jn + mu * jt2, jn - mu * jt2], axis=2)
        J[:] = quad.reshape(nworld, ncon * 4, nv)[:, :R]
        # the last rows of every world are joint limits on one dof each
        nlim = rng.integers(0, 7, nworld)
        for w in range(nworld):
            k = int(min(nlim[w], max(int(nefc[w]) - ne - nf, 0)))
            if k:
                r0 = int(nefc[w]) - k
                dofs = rng.integers(min(6, nv - 1), nv, k)
                J[w, r0 : r0 + k] = 0.0
                J[w, np.arange(r0, r0 + k), dofs] = rng.choice([-1.0, 1.0], k)
    if ne:
        a = rng.integers(0, nv, (nworld, ne))
        J[:, :ne] = rng.normal(0.0, 1.0, (nworld, ne, nv)).astype(np.float32) * masks[a]
    if nf:
        dofs = rng.integers(0, nv, (nworld, nf))
        J[:, ne : ne + nf] = 0.0
        wi = np.repeat(np.arange(nworld), nf)
        ri = np.tile(np.arange(ne, ne + nf), nworld)
        J[wi, ri, dofs.reshape(-1)] = 1.0
        d.efc.frictionloss[:, ne : ne + nf] = rng.uniform(0.1, 1.0, (nworld, nf)).astype(np.float32)
    d.efc.D[:] = rng.uniform(d_range[0], d_range[1], (nworld, R)).astype(np.float32)
    d.efc.aref[:] = rng.normal(0.0, 1.0, (nworld, R)).astype(np.float32)

    qs = rng.normal(0.0, 1.0, (nworld, nv)).astype(np.float32)
    d.qacc_smooth[:] = qs
    d.qfrc_smooth[:] = np.einsum("wij,wj->wi", Mdense.astype(np.float64), qs.astype(np.float64)).astype(
        np.float32
    )
    d.qacc_warmstart[:] = qs + warmstart_scale * rng.normal(0.0, 1.0, (nworld, nv)).astype(np.float32)
    if poison:
        beyond = np.arange(R)[None, :] >= nefc[:, None]
        J[beyond] = np.nan
        d.efc.D[beyond] = np.nan
        d.efc.aref[beyond] = np.nan
    return d, Mdense


# Named workloads: the shapes of the reference's benchmark models (see make_workload).
WORKLOADS = {
    # name: (tree, njmax, nefc_range, iterations, ls_iterations)
    "humanoid": (humanoid_tree, 64, (16, 64)),
    "snu": (snu_tree, 128, (24, 128)),
    "g1": (g1_like_tree, 250, (16, 200)),
}


def make_workload(
    name: str,
    nworld: int,
    seed: int = 0,
    *,
    iterations: int = 50,
    ls_iterations: int = 50,
    tolerance: float = 1e-8,
    rowless_fraction: float = 0.0,
) -> tuple[Model, Data, np.ndarray]:
    """(Model, Data, dense M) of a named workload on the host."""
    tree, njmax, nefc_range = WORKLOADS[name]
    parent, body = tree()
    m = put_model(
        parent,
        iterations=iterations,
        ls_iterations=ls_iterations,
        tolerance=tolerance,
        body_of_dof=body,
    )
    d, Mdense = make_problem(
        m, nworld, njmax, seed, nefc_range=nefc_range, rowless_fraction=rowless_fraction
    )
    return m, d, Mdense


def make_sweep_point(nv: int, nefc: int, nworld: int, seed: int = 0, *, couple: bool = True, **opts):
    """One point of the isolated sweep: generic rows, ne = nf = 0, R = nefc."""
    parent, body = limb_tree(nv)
    m = put_model(parent, body_of_dof=body, **opts)
    d, Mdense = make_problem(m, nworld, nefc, seed, nefc_range=(nefc, nefc), rows="generic", couple=couple)
    return m, d, Mdense


def add_smooth_state(m: Model, d, seed: int = 0):
    """Fills host ``Data`` with a random but physical smooth-dynamics state: per-body
    spatial inertias about a common origin (positive mass, positive definite rotational
    part), motion axes ``cdof`` of unit scale, joint velocities, and empty outputs
    (``crb``, ``M``, ``cvel``, ``cdof_dot``, ``cacc``, ``cfrc_int``, ``qfrc_bias``,
    ``subtree_com``).  ``cvel`` / ``cdof_dot`` are left zero: run ``com_vel`` to make them
    consistent with ``qvel``."""
    rng = np.random.default_rng(seed)
    W, nv, nbody = d.nworld, m.nv, int(np.asarray(m.body_parentid).size)
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)  # noqa: E731
    mass = rng.uniform(0.5, 5.0, (W, nbody))
    com = rng.uniform(-0.3, 0.3, (W, nbody, 3))
    a = rng.normal(0.0, 0.1, (W, nbody, 3, 3))
    inertia = a @ np.swapaxes(a, -1, -2) + 0.02 * np.eye(3)
    c2 = (com * com).sum(-1)
    about_origin = inertia + mass[..., None, None] * (c2[..., None, None] * np.eye(3) - com[..., :, None] * com[..., None, :])
    cinert = np.concatenate(
        [
            np.stack([about_origin[..., 0, 0], about_origin[..., 1, 1], about_origin[..., 2, 2],
                      about_origin[..., 0, 1], about_origin[..., 0, 2], about_origin[..., 1, 2]], -1),
            mass[..., None] * com,
            mass[..., None],
        ],
        -1,
    )
    cinert[:, 0] = 0.0  # the world body carries no inertia
    d.cinert = f32(cinert)
    d.cdof = f32(rng.normal(0.0, 0.6, (W, nv, 6)))
    d.qvel = f32(rng.normal(0.0, 0.5, (W, nv)))
    z = lambda *s: np.zeros(s, np.float32)  # noqa: E731
    d.crb, d.cvel, d.cacc, d.cfrc_int = z(W, nbody, 10), z(W, nbody, 6), z(W, nbody, 6), z(W, nbody, 6)
    d.cdof_dot, d.qfrc_bias, d.subtree_com = z(W, nv, 6), z(W, nv), f32(rng.uniform(0.1, 1.0, (W, nbody, 3)))
    m.dof_armature = f32(rng.uniform(0.0, 0.05, (1, nv)))
    return d
