"""ctypes mirror of ``include/imnewton.h``.

The structures carry raw addresses only, so the same definitions describe device
buffers (for the CUDA library) and host buffers (for the CPU oracle the tests
check against).  Field order and types must match the header exactly;
``tests/test_abi.py`` checks the sizes against the compiled library.
"""

from __future__ import annotations

import ctypes as C

P = C.c_void_p
I32 = C.c_int32
I64 = C.c_int64
F32 = C.c_float

IMN_ABI_VERSION = 4

IMN_OK = 0
IMN_ERR_NULL = -1
IMN_ERR_SHAPE = -2
IMN_ERR_UNSUPPORTED = -3
IMN_ERR_LAUNCH = -4
IMN_ERR_LIMIT = -5


class ImnModel(C.Structure):
    _fields_ = [
        ("nv", I32),
        ("nv_pad", I32),
        ("nM", I32),
        ("iterations", I32),
        ("ls_iterations", I32),
        ("warmstart", I32),
        ("n_tolerance", I32),
        ("n_ls_tolerance", I32),
        ("n_meaninertia", I32),
        ("opt_tolerance", P),
        ("opt_ls_tolerance", P),
        ("stat_meaninertia", P),
        ("M_rowadr", P),
        ("M_rownnz", P),
        ("M_colind", P),
        ("M_mulm_rowadr", P),
        ("M_mulm_col", P),
        ("M_mulm_madr", P),
        ("M_mulm_pack", P),
        ("alpha_noise_eps", F32),
        ("overflow_iterations", I32),
        ("overflow_ls_iterations", I32),
        ("warn_overflow", I32),
    ]


class ImnData(C.Structure):
    _fields_ = [
        ("nworld", I32),
        ("njmax", I32),
        ("nefc", P),
        ("ne", P),
        ("nf", P),
        ("qacc_smooth", P),
        ("qacc_warmstart", P),
        ("qfrc_smooth", P),
        ("dof_ld", I64),
        ("efc_J", P),
        ("J_ld_world", I64),
        ("J_ld_row", I64),
        ("efc_D", P),
        ("efc_aref", P),
        ("efc_frictionloss", P),
        ("efc_ld", I64),
        ("M", P),
        ("M_ld", I64),
        ("qacc", P),
        ("qfrc_constraint", P),
        ("efc_Ma", P),
        ("efc_force", P),
        ("efc_state", P),
        ("solver_niter", P),
        ("overflow", P),
        ("J_world_offset", P),
        ("J_elems", I64),
    ]


SPARSE_TABLES = (
    # (field, numpy dtype)
    ("lvl_ptr", "uint16"),
    ("lvl_team", "uint8"),
    ("ent_slot", "uint16"),
    ("ent_col", "int16"),
    ("run_ptr", "uint16"),
    ("run_ab", "uint32"),
    ("run_kl", "uint32"),
    ("orig", "uint16"),
    ("b_lvl", "uint16"),
    ("b_slot", "uint16"),
    ("b_src", "uint16"),
    ("b_dst", "uint16"),
    ("pair", "int32"),
    ("f_lvl", "uint16"),
    ("f_row", "uint16"),
    ("row_start", "uint16"),
    ("rk_ptr", "uint16"),
    ("rk", "uint16"),
    ("pmask", "uint32"),
    ("s_a", "uint16"),
    ("s_b", "uint16"),
    ("s_m", "int32"),
    ("gat", "uint32"),
    ("fsweep", "uint32"),
    ("bsweep", "uint32"),
)


class ImnSparsePlan(C.Structure):
    _fields_ = [
        ("nv", I32),
        ("nv_pad", I32),
        ("block", I32),
        ("nfac", I32),
        ("nslots", I32),
        ("nlevels", I32),
        ("nentries", I32),
        ("nruns", I32),
        ("nback", I32),
    ] + [(name, P) for name, _ in SPARSE_TABLES] + [("nfsweep", I32), ("nbsweep", I32)]


class ImnCtx(C.Structure):
    _fields_ = [
        ("Jaref", P),
        ("jv", P),
        ("search", P),
        ("mv", P),
        ("grad", P),
        ("grad_ld", I64),
        ("h", P),
        ("hfactor", P),
        ("search_dot", P),
        ("grad_dot", P),
        ("grad_scale", P),
        ("newton_decrement", P),
        ("improvement", P),
        ("alpha", P),
        ("done", P),
        ("search_unchanged", P),
        ("ls_exhausted", P),
        ("quad_changed_ids", P),
        ("quad_changed_count", P),
        ("state_changed_count", P),
        ("dof_union", P),
        ("nsolving", P),
        ("sparse_plan", C.POINTER(ImnSparsePlan)),
        ("world_order", P),
        ("stats", P),
    ]


class ImnTreePlan(C.Structure):
    _fields_ = [
        ("nv", I32),
        ("nM", I32),
        ("groups", I32),
        ("ntrunk", I32),
        ("ntrunk_entries", I32),
        ("nslot", I32),
        ("prog", P),
        ("prog_ptr", P),
        ("owner", I32),
    ]


class ImnBlockedPlan(C.Structure):
    _fields_ = [
        ("nv", I32),
        ("pad", I32),
        ("indices", P),
        ("identity", P),
        ("nM", I32),
    ]


class ImnImplicit(C.Structure):
    _fields_ = [
        ("nv", I32), ("nM", I32), ("nu", I32), ("actuation", I32), ("damper", I32), ("timestep", P), ("n_timestep", I32),
        ("dof_damping", P), ("M_elemid", P), ("moment_rownnz", P), ("moment_rowadr", P), ("moment_colind", P),
        ("actuator_moment", P), ("moment_ld", I64), ("actuator_velocity_gain", P),
    ]


class ImnAdvance(C.Structure):
    _fields_ = [
        ("nv", I32), ("nq", I32), ("njnt", I32), ("timestep", P), ("n_timestep", I32), ("jnt_type", P), ("jnt_dofadr", P),
        ("jnt_qposadr", P), ("qvel", P), ("qvel_ld", I64), ("qpos", P), ("qpos_ld", I64), ("time", P),
    ]


class ImnBodyTree(C.Structure):
    _fields_ = [
        ("nbody", I32), ("nv", I32), ("nM", I32), ("nlevels", I32), ("body_parentid", P), ("level_bodies", P),
        ("level_offsets", P), ("child_ptr", P), ("child_ids", P), ("body_jntnum", P), ("body_jntadr", P),
        ("body_dofadr", P), ("body_dofnum", P), ("jnt_type", P), ("dof_bodyid", P), ("dof_parentid", P),
        ("dof_armature", P), ("n_armature", I32), ("M_rowidx", P), ("M_colind", P), ("gravity", P),
        ("n_gravity", I32), ("gravity_enabled", I32), ("team_lanes", I32),
    ]


class ImnBallLimits(C.Structure):
    _fields_ = [
        ("njoint", I32), ("nv", I32), ("njmax", I32), ("refsafe", I32), ("limit_joint_type", I32),
        ("timestep", P), ("n_timestep", I32), ("qadr", P), ("dadr", P), ("joint", P), ("neutral", P), ("frame", P), ("swing", P),
        ("twist", P), ("minimum_h", P), ("margin", P), ("solref", P), ("solimp", P), ("invweight", P),
        ("n_invweight", I32), ("qpos", P), ("qpos_ld", I64), ("qvel", P), ("qvel_ld", I64), ("nefc", P), ("nl", P),
        ("efc_type", P), ("efc_id", P), ("efc_J", P), ("J_ld_world", I64), ("J_ld_row", I64), ("efc_pos", P),
        ("efc_margin", P), ("efc_D", P), ("efc_vel", P), ("efc_aref", P), ("efc_frictionloss", P), ("efc_ld", I64),
        ("overflow", P), ("singular", P),
    ]


class ImnLaunchInfo(C.Structure):
    _fields_ = [
        ("world_threads", I32),
        ("worlds_per_cta", I32),
        ("smem_bytes", I32),
        ("j_resident", I32),
        ("grid", I32),
    ]


# name -> (restype, argtypes) of every symbol the header declares
SYMBOLS = {
    "imn_solve": (C.c_int, [C.POINTER(ImnModel), C.POINTER(ImnData), C.POINTER(ImnCtx), P]),
    "imn_rowless_handoff": (C.c_int, [C.POINTER(ImnModel), C.POINTER(ImnData), P]),
    "imn_mul_m": (C.c_int, [C.POINTER(ImnModel), P, I64, P, I64, P, I64, I32, P]),
    "imn_tree_ldl_solve": (C.c_int, [C.POINTER(ImnTreePlan), P, I64, P, I64, P, I64, I32, P]),
    "imn_tree_ldl_compile": (C.c_int, [P, P, I32, I32, I32, I32, I32, C.POINTER(C.c_void_p)]),
    "imn_mul_m_compile": (C.c_int, [P, P, I32, I32, I32, I32, C.POINTER(C.c_void_p)]),
    "imn_tree_ldl_kernel_info": (
        C.c_int,
        [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int64), C.POINTER(C.c_char_p)],
    ),
    "imn_tree_ldl_kernel_destroy": (None, [C.c_void_p]),
    "imn_tree_ldl_compiled_solve": (C.c_int, [C.c_void_p, P, I64, P, I64, P, I64, I32, P]),
    "imn_blocked_dense_factor_solve": (
        C.c_int,
        [C.POINTER(ImnBlockedPlan), P, I64, P, P, P, P, I32, I32, I32, P],
    ),
    "imn_blocked_dense_factor_solve_static": (
        C.c_int,
        [C.POINTER(ImnBlockedPlan), P, I64, P, P, P, I32, I32, P],
    ),
    "imn_sparse_factor_nonfused": (
        C.c_int,
        [C.POINTER(ImnSparsePlan), P, P, I64, P, P, P, P, P, I64, P, P, I32, I32, I32, P],
    ),
    "imn_implicit_matrix": (C.c_int, [C.POINTER(ImnImplicit), P, I64, P, I64, I32, P]),
    "imn_advance": (C.c_int, [C.POINTER(ImnAdvance), P, I64, I32, P]),
    "imn_ball_limit_rows": (C.c_int, [C.POINTER(ImnBallLimits), I32, P]),
    "imn_expand_row_vectors": (C.c_int, [P, P, P, P, I64, P, I32, P, P, P, I64, I32, P]),
    "imn_expand_rows": (C.c_int, [P, P, I32, P, I32, I32, P, I64, P]),
    "imn_body_tree_accumulate": (C.c_int, [C.POINTER(ImnBodyTree), P, I64, I32, I32, I32, P]),
    "imn_crb": (C.c_int, [C.POINTER(ImnBodyTree), P, P, P, P, I64, I32, P]),
    "imn_rne": (C.c_int, [C.POINTER(ImnBodyTree), P, P, P, P, P, I64, P, P, P, I64, I32, P]),
    "imn_com_vel": (C.c_int, [C.POINTER(ImnBodyTree), P, I64, P, P, P, I32, P]),
    "imn_sparse_plan_create": (C.c_int, [C.POINTER(ImnSparsePlan), C.POINTER(C.POINTER(ImnSparsePlan))]),
    "imn_sparse_plan_destroy": (None, [C.POINTER(ImnSparsePlan)]),
    "imn_launch_info": (
        C.c_int,
        [C.POINTER(ImnModel), C.POINTER(ImnData), C.POINTER(ImnCtx), C.POINTER(ImnLaunchInfo)],
    ),
    "imn_set_copy_wait_limit": (C.c_int, [I32, I32]),
    "imn_copy_rows": (C.c_int, [P, I64, P, I64, I64, I32, I32, P]),
    "imn_last_error": (C.c_char_p, []),
    "imn_abi_version": (C.c_int, []),
}


def bind(lib: C.CDLL, symbols=SYMBOLS) -> C.CDLL:
    """Attach restype/argtypes; raises AttributeError when a symbol is missing."""
    for name, (restype, argtypes) in symbols.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib
