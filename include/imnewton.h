/*
 * imnewton.h -- C ABI of the B200-native Newton constraint solver.
 *
 * Every entry point replaces one interface of InstantMimic's MuJoCo-Warp step
 * (reference paths are given per declaration, relative to the InstantMimic
 * source tree).  The structs are plain-old-data: device pointers, extents and
 * element strides of buffers that the CALLER owns.  The library allocates no
 * device memory; plans (index tables) are uploaded once by the caller and
 * passed as pointers.  All work is enqueued on the CUDA stream handed in and
 * no call synchronises, so every entry point may be recorded into a CUDA
 * graph like the Warp launches it stands in for.
 *
 * Return value: 0 on success, a negative ImnStatus when host-side validation
 * fails (nothing is launched).  Device-side conditions never surface here: they
 * go to the per-world `overflow` bits and to the sparse-pattern violation
 * counter exactly as the reference does.
 *
 * Conventions shared by all structs
 *   - W = nworld, nv = degrees of freedom, P = nv_pad, R = njmax.
 *   - every array is world-major; `*_ld` fields are the stride, in ELEMENTS,
 *     between consecutive worlds (or rows where stated).
 *   - float is IEEE binary32; int is int32_t; flags are uint8_t (0/1).
 */
#ifndef IMNEWTON_H_
#define IMNEWTON_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IMN_ABI_VERSION 4

typedef enum ImnStatus {
  IMN_OK = 0,
  IMN_ERR_NULL = -1,        /* a required pointer is NULL                      */
  IMN_ERR_SHAPE = -2,       /* nv / nv_pad / njmax / stride out of range       */
  IMN_ERR_UNSUPPORTED = -3, /* model outside the fused path's eligibility      */
  IMN_ERR_LAUNCH = -4,      /* cudaGetLastError() after the launch             */
  IMN_ERR_LIMIT = -5        /* size beyond a stated fixed maximum              */
} ImnStatus;

/* mujoco ConstraintState values (efc.state). */
enum {
  IMN_STATE_SATISFIED = 0,
  IMN_STATE_QUADRATIC = 1,
  IMN_STATE_LINEARNEG = 2,
  IMN_STATE_LINEARPOS = 3
};

/* Model-side constants of the solve: the fields of mujoco_warp `Model` that
 * solve_with_scratch reads (mjw_step_optimized.py:2588-2680,
 * newton_fusion.py:330-409). */
typedef struct ImnModel {
  int32_t nv;
  int32_t nv_pad;        /* roundup(nv + 1, 16) on the Newton path             */
  int32_t nM;            /* number of stored entries of M (CSR over ancestors) */
  int32_t iterations;    /* opt.iterations                                     */
  int32_t ls_iterations; /* opt.ls_iterations                                  */
  int32_t warmstart;     /* !(opt.disableflags & WARMSTART)                    */
  /* per-world option arrays, indexed world % n (newton_stages.py:183-186)      */
  int32_t n_tolerance, n_ls_tolerance, n_meaninertia;
  const float* opt_tolerance;
  const float* opt_ls_tolerance;
  const float* stat_meaninertia;
  /* M in CSR over each dof's ancestors, root first, diagonal last
   * (tree_ldl.py:3-8): rowadr[nv], rownnz[nv], colind[nM]                      */
  const int32_t* M_rowadr;
  const int32_t* M_rownnz;
  const int32_t* M_colind;
  /* full symmetric rows for M*v: rowadr[nv+1], col[], madr[]
   * (newton_fusion.py:171-176, 378-380)                                        */
  const int32_t* M_mulm_rowadr;
  const int32_t* M_mulm_col;
  const int32_t* M_mulm_madr;
  /* the same table, one word per entry: col | madr << 16 (2 nM - nv entries);
   * built once per model by the host layer                                    */
  const uint32_t* M_mulm_pack;
  /* constants that live in the upstream solver module                         */
  float alpha_noise_eps;          /* solver._ALPHA_NOISE_EPS                    */
  int32_t overflow_iterations;    /* types.OverflowType.ITERATIONS bit          */
  int32_t overflow_ls_iterations; /* types.OverflowType.LS_ITERATIONS bit       */
  int32_t warn_overflow;          /* opt.warn_overflow mask (device printf)     */
} ImnModel;

/* Data-side buffers of one batch of worlds: the fields of mujoco_warp `Data`
 * that the solve reads and writes (newton_fusion.py:330-395). */
typedef struct ImnData {
  int32_t nworld;
  int32_t njmax;
  const int32_t* nefc; /* (W) */
  const int32_t* ne;   /* (W) */
  const int32_t* nf;   /* (W) */
  /* (W, nv) inputs, stride dof_ld */
  const float* qacc_smooth;
  const float* qacc_warmstart;
  const float* qfrc_smooth;
  int64_t dof_ld;
  /* efc.J (W, R, >=nv): world stride J_ld_world, row stride J_ld_row */
  const float* efc_J;
  int64_t J_ld_world;
  int64_t J_ld_row;
  /* (W, R) row arrays, stride efc_ld */
  const float* efc_D;
  const float* efc_aref;
  const float* efc_frictionloss;
  int64_t efc_ld;
  /* M (W, nM), stride M_ld */
  const float* M;
  int64_t M_ld;
  /* outputs */
  float* qacc;            /* (W, nv)  stride dof_ld */
  float* qfrc_constraint; /* (W, nv)  stride dof_ld */
  float* efc_Ma;          /* (W, nv)  stride dof_ld */
  float* efc_force;       /* (W, R)   stride efc_ld */
  int32_t* efc_state;     /* (W, R)   stride efc_ld */
  int32_t* solver_niter;  /* (W) */
  int32_t* overflow;      /* (W), bits are OR-ed in */
  /* Optional, no counterpart in the reference (mujoco-warp pads every world to njmax
   * rows): when non-NULL, world w's Jacobian starts at efc_J + J_world_offset[w]
   * (elements) instead of efc_J + w * J_ld_world, and efc_J holds J_elems elements
   * in all.  Lets a producer hand over J compactly -- only the nefc rows of each
   * world, one world after the other, as MuJoCo C stores mjData.efc_J -- so that no
   * dead row crosses PCIe.  Rows are still J_ld_row apart. */
  const int64_t* J_world_offset; /* (W) or NULL */
  int64_t J_elems;               /* extent of efc_J when J_world_offset is given */
} ImnData;

/* Static-pattern sparse L'DL of the Hessian: the tables that
 * sparse_hessian.build_plan (sparse_hessian.py:229-402) bakes into generated
 * source, here as device arrays.  Names follow the SH_* tables.  */
typedef struct ImnSparsePlan {
  int32_t nv, nv_pad, block;
  int32_t nfac;    /* factor slots (rows of L incl. diagonal)                  */
  int32_t nslots;  /* nfac + nv (augmented right-hand-side row)                */
  int32_t nlevels;
  int32_t nentries, nruns, nback;
  const uint16_t* lvl_ptr;  /* SH_LP  [nlevels+1]                              */
  const uint8_t* lvl_team;  /* SH_LT  [nlevels]                                */
  const uint16_t* ent_slot; /* SH_ES  [nentries]                               */
  const int16_t* ent_col;   /* SH_EC  [nentries]                               */
  const uint16_t* run_ptr;  /* SH_RP  [nentries+1]                             */
  const uint32_t* run_ab;   /* SH_RAB [nruns]                                  */
  const uint32_t* run_kl;   /* SH_RKL [nruns]                                  */
  const uint16_t* orig;     /* SH_ORIG[nv]                                     */
  const uint16_t* b_lvl;    /* SH_BL  [nlevels+1]                              */
  const uint16_t* b_slot;   /* SH_BS  [nback]                                  */
  const uint16_t* b_src;    /* SH_BI  [nback]                                  */
  const uint16_t* b_dst;    /* SH_BJ  [nback]                                  */
  const int32_t* pair;      /* SH_PAIR[nv*nv]                                  */
  const uint16_t* f_lvl;    /* SH_FL  [nlevels+1]                              */
  const uint16_t* f_row;    /* SH_FR  [nv]                                     */
  const uint16_t* row_start;/* SH_RS  [nv]                                     */
  const uint16_t* rk_ptr;   /* SH_RKP [nv+1]                                   */
  const uint16_t* rk;       /* SH_RK  []                                       */
  const uint32_t* pmask;    /* SH_PM  [nv*words]                               */
  const uint16_t* s_a;      /* SH_SA  [nfac]                                   */
  const uint16_t* s_b;      /* SH_SB  [nfac]                                   */
  const int32_t* s_m;       /* SH_SM  [nfac]                                   */
  const uint32_t* gat;      /* SH_GAT [nfac] (non-fused path)                  */
  /* The level tables once more, laid out for the fused kernel: one record per
   * (sweep, lane), so that a lane fetches all it needs for a sweep with one load
   * and can fetch the next sweep's record ahead of time.  A sweep is 32 / team
   * entries of one level.
   *   fsweep [nfsweep][32][4]: {slot | (col+1) << 16, run_ab, run_kl of the entry's
   *     first run, flags}; flags bit 0 = the lane has an entry, bit 1 = last sweep
   *     of its level, bits 2-4 = log2(team), bits 8-15 = further runs of the entry,
   *     bits 16-31 = index of the first of those in run_ab / run_kl.
   *   bsweep [nbsweep][32]: slot | src << 16 | dst << 23 | has-work << 30 |
   *     last-of-level << 31 (backward solve).
   * NULL / 0 when the plan is only used by the non-fused kernel. */
  const uint32_t* fsweep;
  const uint32_t* bsweep;
  int32_t nfsweep, nbsweep;
} ImnSparsePlan;

/* Solver context: the arrays mujoco_warp's `_create_solver_context` allocates
 * (mjw_step_optimized.py:2517) plus newton_dof_union
 * (newton_fusion.py:301-304).  The fused kernel keeps its working set in
 * shared memory; any pointer that is non-NULL receives the final value of the
 * corresponding quantity when a world finishes, so a caller that inspects the
 * context (the reference's tests do) still finds it.  NULL pointers are
 * skipped.  `hfactor` is REQUIRED only on the sparse path: its last element per
 * world is the pattern-violation counter; the packed H | N | 1/D layout of
 * sparse_hessian.py:488-489 is written there only when `h` is non-NULL too. */
typedef struct ImnCtx {
  float* Jaref; /* (W, R) stride efc_ld of ImnData */
  float* jv;    /* (W, R) */
  float* search; /* (W, nv) stride dof_ld */
  float* mv;     /* (W, nv) */
  float* grad;   /* (W, grad_ld) */
  int64_t grad_ld;
  float* h;       /* (W, P, P) dense Hessian, upper triangle maintained */
  float* hfactor; /* (W, P, P) dense upper factor | packed sparse layout */
  float* search_dot;
  float* grad_dot;
  float* grad_scale;
  float* newton_decrement;
  float* improvement;
  float* alpha;
  uint8_t* done;
  uint8_t* search_unchanged;
  uint8_t* ls_exhausted;
  int32_t* quad_changed_ids;   /* (W, R) stride efc_ld */
  int32_t* quad_changed_count; /* (W) */
  int32_t* state_changed_count;/* (W) */
  int32_t* dof_union;          /* (W, nv + 1) */
  int32_t* nsolving;           /* (1): nworld minus the worlds that finished */
  const ImnSparsePlan* sparse_plan; /* HOST pointer or NULL (dense factor)    */
  int32_t* world_order; /* optional scratch (W): when given, imn_solve fills it with
                         * the worlds ordered by descending row count and hands the
                         * worlds to the GPU in that order (long solves first, which
                         * shortens the tail of the launch); results do not depend
                         * on it                                                  */
  int32_t* stats;       /* optional (W, 4), no counterpart in the reference: work
                         * counters of each world's solve, from which the flop count
                         * of a batch is computed -- [0] row-evaluation passes of the
                         * line searches, [1] rows whose QUADRATIC membership flipped
                         * (summed over iterations), [2] factorisations (the initial
                         * one included), [3] full gradient evaluations (the initial
                         * one included)                                          */
} ImnCtx;

/* Tree-structured L'DL plan (tree_ldl.py:47-57, 105-170) as an instruction
 * list instead of generated source.  One instruction is four int32:
 * {op, a, b, c}; see imn_tree_ldl_solve.  */
typedef struct ImnTreePlan {
  int32_t nv, nM;
  int32_t groups;       /* warps per block of 32 worlds                        */
  int32_t ntrunk;       /* trunk dofs                                          */
  int32_t ntrunk_entries;
  int32_t nslot;        /* per-world scratch slots in shared memory            */
  const int32_t* prog;      /* device: concatenated instruction streams        */
  const int32_t* prog_ptr;  /* device: [2*groups + 2] stream offsets           */
  int32_t owner;        /* group that finishes the trunk                       */
} ImnTreePlan;

/* Blocked dense Cholesky of M gathered by index
 * (indexed_factor.py:15-173, mjw_step_optimized.py:893-955). */
typedef struct ImnBlockedPlan {
  int32_t nv;
  int32_t pad;            /* roundup(nv, 16)                                   */
  const int32_t* indices; /* device (pad*pad) block-major gather; nM = zero    */
  const float* identity;  /* device (256): ones on the padded diagonal         */
  int32_t nM;
} ImnBlockedPlan;

/* mujoco mjtJoint values (Model.jnt_type). */
enum { IMN_JNT_FREE = 0, IMN_JNT_BALL = 1, IMN_JNT_SLIDE = 2, IMN_JNT_HINGE = 3 };

/* Inputs of the implicit-fast matrix A = M - h qDeriv (mjw_step_optimized.py:4172-4295):
 * the passive joint damping and the actuator-centric actuation term
 * sum_a moment_a moment_a^T gain_a, with the actuator moments in mujoco-warp's
 * per-world CSR (Data.moment_rownnz / moment_rowadr / moment_colind /
 * actuator_moment) and gain_a = d(actuator force)/d(actuator velocity), the
 * `vel` buffer that upstream's _qderiv_actuator_passive_vel fills. */
typedef struct ImnImplicit {
  int32_t nv, nM, nu;
  int32_t actuation;           /* !(opt.disableflags & ACTUATION)                */
  int32_t damper;              /* !(opt.disableflags & DAMPER)                   */
  const float* timestep;       /* opt.timestep (n_timestep): world w reads w % n  */
  int32_t n_timestep;
  const float* dof_damping;    /* (nv)                                           */
  const int32_t* M_elemid;     /* (nv, nv): entry of M for (i, j), -1 if none    */
  const int32_t* moment_rownnz; /* (W, nu)                                       */
  const int32_t* moment_rowadr; /* (W, nu)                                       */
  const int32_t* moment_colind; /* (W, moment_ld) dofs, ascending within a row   */
  const float* actuator_moment; /* (W, moment_ld)                                */
  int64_t moment_ld;
  const float* actuator_velocity_gain; /* (W, nu)                                */
} ImnImplicit;

/* State advanced by the integrator (upstream _advance, called through
 * _advance_with_scratch, mjw_step_optimized.py:4823-4847). */
typedef struct ImnAdvance {
  int32_t nv, nq, njnt;
  const float* timestep;      /* opt.timestep (n_timestep): world w reads w % n   */
  int32_t n_timestep;
  const int32_t* jnt_type;    /* (njnt) IMN_JNT_*                                */
  const int32_t* jnt_dofadr;  /* (njnt)                                          */
  const int32_t* jnt_qposadr; /* (njnt)                                          */
  float* qvel;                /* (W, nv)  in/out                                 */
  int64_t qvel_ld;
  float* qpos;                /* (W, nq)  in/out                                 */
  int64_t qpos_ld;
  float* time;                /* (W) in/out, may be NULL                         */
} ImnAdvance;

/* Body tree and the model tables of the smooth-dynamics stages that walk it
 * (tree_fusion.py:27-50 TreeReductionScratch / create_tree_reduction_scratch; the
 * kernels' model arguments, tree_fusion.py:192-206, 209-222, velocity_fusion.py:15-29).
 * All pointers are device pointers.  Tables a call does not read may be NULL. */
typedef struct ImnBodyTree {
  int32_t nbody, nv, nM, nlevels;
  const int32_t* body_parentid; /* (nbody)                                          */
  const int32_t* level_bodies;  /* (nbody) m.body_tree concatenated, level 0 first  */
  const int32_t* level_offsets; /* (nlevels + 1)                                    */
  const int32_t* child_ptr;     /* (nbody + 1) by position in level_bodies: the     */
  const int32_t* child_ids;     /* children of that body in level-list order (the
                                 * world body is nobody's child); no counterpart in
                                 * the reference, which scans the whole next level  */
  const int32_t* body_jntnum;   /* (nbody) */
  const int32_t* body_jntadr;   /* (nbody) */
  const int32_t* body_dofadr;   /* (nbody) */
  const int32_t* body_dofnum;   /* (nbody) */
  const int32_t* jnt_type;      /* (njnt) IMN_JNT_*                                 */
  const int32_t* dof_bodyid;    /* (nv) */
  const int32_t* dof_parentid;  /* (nv) */
  const float* dof_armature;    /* (n_armature, nv), world w reads row w % n        */
  int32_t n_armature;
  const int32_t* M_rowidx;      /* (nM) dof (row) of every stored entry of M        */
  const int32_t* M_colind;      /* (nM) its column: an ancestor of the row, or itself */
  const float* gravity;         /* (n_gravity, 3) opt.gravity, world w reads w % n  */
  int32_t n_gravity;
  int32_t gravity_enabled;      /* !(opt.disableflags & GRAVITY)                    */
  int32_t team_lanes;           /* lanes of a warp that work on one world: 8, 16 or
                                 * 32 (any other value: 32); pass the smallest that
                                 * covers the widest level.  rne (16) and crb (32) raise
                                 * it to their own minimum.  Results do not depend on it   */
} ImnBodyTree;

/* Directional ball-joint limits (ball_limits.py:205-318 BallLimitBuffers /
 * make_ball_limit_buffers) and the constraint-row arrays of mujoco_warp `Data` they are
 * appended to (ball_limits.py:259-281).  Dense Jacobian only. */
typedef struct ImnBallLimits {
  int32_t njoint;              /* limited ball joints                             */
  int32_t nv, njmax;
  int32_t refsafe;             /* !(opt.disableflags & REFSAFE)                   */
  int32_t limit_joint_type;    /* types.ConstraintType.LIMIT_JOINT                */
  const float* timestep;       /* opt.timestep (n_timestep): world w reads w % n  */
  int32_t n_timestep;
  const int32_t* qadr;         /* (njoint) qpos address of the joint's quaternion */
  const int32_t* dadr;         /* (njoint) first dof                              */
  const int32_t* joint;        /* (njoint) joint id (efc.id)                      */
  const float* neutral;        /* (njoint, 4) wxyz                                */
  const float* frame;          /* (njoint, 4) wxyz                                */
  const float* swing;          /* (njoint, 4) 1 / tan^2(angle / 2): +x, +y, -x, -y */
  const float* twist;          /* (njoint, 2) lower, upper                        */
  const float* minimum_h;      /* (njoint)                                        */
  const float* margin;         /* (njoint)                                        */
  const float* solref;         /* (njoint, 2)                                     */
  const float* solimp;         /* (njoint, 5)                                     */
  const float* invweight;      /* (n_invweight, nv) dof_invweight0, world % n     */
  int32_t n_invweight;
  const float* qpos;           /* (W, nq) */
  int64_t qpos_ld;
  const float* qvel;           /* (W, nv) */
  int64_t qvel_ld;
  int32_t* nefc;               /* (W) in/out */
  int32_t* nl;                 /* (W) in/out, may be NULL */
  int32_t* efc_type;           /* (W, R) stride efc_ld */
  int32_t* efc_id;
  float* efc_J;                /* (W, R, >= nv) */
  int64_t J_ld_world, J_ld_row;
  float* efc_pos;
  float* efc_margin;
  float* efc_D;
  float* efc_vel;
  float* efc_aref;
  float* efc_frictionloss;
  int64_t efc_ld;
  int32_t* overflow;           /* (W) rows that found no room, may be NULL        */
  int32_t* singular;           /* (W) candidates at the chart's antipode, may be NULL */
} ImnBallLimits;

/* ---- entry points ------------------------------------------------------- */

/* Replaces solve_with_scratch's monolithic fused branch:
 * _solve_monolithic_with_scratch (mjw_step_optimized.py:2588-2680) =
 * _solve_init_dof + newton_fusion.init_context (newton_fusion.py:431-472) +
 * newton_fusion.run (newton_fusion.py:330-409) + qfrc_constraint_from_grad
 * (newton_fusion.py:522-539), as ONE persistent kernel.  `stream` is a
 * cudaStream_t. */
int imn_solve(const ImnModel* m, const ImnData* d, const ImnCtx* ctx, void* stream);

/* Replaces the rowless branch of solve_with_scratch
 * (mjw_step_optimized.py:2692-2699): qacc = qacc_smooth, efc.Ma = M qacc,
 * qfrc_constraint = 0, solver_niter = 0 for every world. */
int imn_rowless_handoff(const ImnModel* m, const ImnData* d, void* stream);

/* Replaces support.mul_m through the preallocated call
 * (mjw_step_optimized.py:2252-2255): out = M v per world. */
int imn_mul_m(const ImnModel* m, const float* M, int64_t M_ld, const float* v,
              int64_t v_ld, float* out, int64_t out_ld, int32_t nworld, void* stream);

/* Replaces tree_ldl.tree_factor_solve (tree_ldl.py:419-433): x = M^-1 y with
 * M in the model's ancestor CSR; nothing but x is written. */
int imn_tree_ldl_solve(const ImnTreePlan* plan, const float* M, int64_t M_ld,
                       const float* y, int64_t y_ld, float* x, int64_t x_ld,
                       int32_t nworld, void* stream);

/* Replaces make_tree_ldl_factor_solve_kernel (tree_ldl.py:362-390, source text
 * from _generate_source, tree_ldl.py:196-359): turns the plan's instruction list
 * into straight-line CUDA C and compiles it for sm_100a at run time (NVRTC,
 * looked up with dlopen; IMN_ERR_UNSUPPORTED when it is not installed -- callers
 * then keep imn_tree_ldl_solve).  `prog` (n x 4 int32) and `prog_ptr`
 * (2*groups + 2 offsets) are HOST copies of the arrays of ImnTreePlan.  Needs no
 * GPU; the machine code is handed to the CUDA runtime on the first
 * imn_tree_ldl_compiled_solve (make that call outside stream capture). */
typedef struct ImnTreeKernel ImnTreeKernel;
int imn_tree_ldl_compile(const int32_t* prog, const int32_t* prog_ptr, int32_t nv,
                         int32_t nM, int32_t groups, int32_t owner, int32_t nslot,
                         ImnTreeKernel** out);
/* Shared-memory slots per world, bytes of machine code, and the generated source
 * (owned by the kernel object); any pointer may be NULL. */
int imn_tree_ldl_kernel_info(const ImnTreeKernel* kernel, int32_t* shared_slots,
                             int64_t* code_bytes, const char** source);
void imn_tree_ldl_kernel_destroy(ImnTreeKernel* kernel);

/* out = M v (upstream support.mul_m, called at mjw_step_optimized.py:2252-2255) as
 * generated straight-line code of the same kind.  The program is built by the caller from
 * the model's symmetric-row tables (M_mulm_rowadr / col / madr): streams 0..groups-1 load
 * the entries of v each warp needs (LOAD_Y), the trunk stream is empty, streams
 * groups+1..2*groups form each row's sum in table order -- ZERO, then LOAD_M + MULADD
 * (dst = fmaf(a, b, dst)) per stored entry -- and STORE_X it.  The results equal
 * imn_mul_m's bit for bit.  Launch with imn_tree_ldl_compiled_solve (y = v, x = out; out
 * must not alias v); kernel_info / kernel_destroy as for the tree kernels. */
int imn_mul_m_compile(const int32_t* prog, const int32_t* prog_ptr, int32_t nv, int32_t nM,
                      int32_t groups, int32_t nslot, ImnTreeKernel** out);

/* tree_ldl.tree_factor_solve (tree_ldl.py:419-433) through the generated kernel;
 * arguments and results as imn_tree_ldl_solve, bit for bit. */
int imn_tree_ldl_compiled_solve(ImnTreeKernel* kernel, const float* M, int64_t M_ld,
                                const float* y, int64_t y_ld, float* x, int64_t x_ld,
                                int32_t nworld, void* stream);

/* Replaces factor_solve_indexed_cholesky_kernel and its multi-RHS variants
 * (indexed_factor.py:176-214, 217-391, 394-493;
 * mjw_step_optimized.py:958-993).
 *   mode 0: factor M into U (W, pad, pad) and solve rhs_count columns
 *   mode 1: solve with the U already stored
 * y and x are (W, nv, rhs_count) contiguous; `active` (W) may be NULL; worlds
 * whose flag is 0 are left untouched.  U is caller-owned scratch. */
int imn_blocked_dense_factor_solve(const ImnBlockedPlan* plan, const float* M,
                                   int64_t M_ld, const float* y, float* U, float* x,
                                   const int32_t* active, int32_t nworld,
                                   int32_t rhs_count, int32_t mode, void* stream);

/* Floats of the factor workspace built into the library (32 MiB per GPU). */
#define IMN_STATIC_FACTOR_FLOATS (8 * 1024 * 1024)

/* No counterpart in the reference.  Factor + solve (mode 0 of
 * imn_blocked_dense_factor_solve) for callers that cannot provide the
 * (W, pad, pad) factor workspace because they may not allocate device memory
 * where they call: a step being recorded into a CUDA graph, a process whose
 * device memory belongs to another framework's pool, a host that forbids
 * cudaMalloc after start-up.  The workspace is a fixed array inside the library;
 * every GPU that loads the library holds its 32 MiB until the process exits.
 *   - nworld * pad * pad must not exceed IMN_STATIC_FACTOR_FLOATS, else
 *     IMN_ERR_LIMIT is returned and nothing runs;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress with that device current); make that first call
 *     outside any stream capture; the address is cached per device (first calls
 *     from several host threads are safe) and belongs to the device's primary
 *     context: it does not survive cudaDeviceReset;
 *   - all calls share the one array and it keeps the last call's factor: two
 *     calls whose kernels overlap on the GPU (different streams) race, and the
 *     stored factor cannot be reused by a later solve-only call;
 *   - inputs, outputs, `active` and results are as for
 *     imn_blocked_dense_factor_solve; no allocation happens in any call. */
int imn_blocked_dense_factor_solve_static(const ImnBlockedPlan* plan, const float* M,
                                          int64_t M_ld, const float* y, float* x,
                                          const int32_t* active, int32_t nworld,
                                          int32_t rhs_count, void* stream);

/* Replaces sparse_hessian_upstream_factor, the sparse factor of the
 * non-fused iteration (sparse_hessian.py:849-894): mode 4 gathers the dense H
 * and factors, mode 5 solves with the stored factor.  hfactor layout:
 * [0,nfac) N, [nfac,nfac+nv) 1/D.  search is (W, nv), grad (W, grad_ld). */
int imn_sparse_factor_nonfused(const ImnSparsePlan* plan, const uint8_t* done,
                               const float* grad, int64_t grad_ld, const float* h,
                               const int32_t* quad_changed,
                               const int32_t* state_changed, float* hfactor,
                               float* search, int64_t search_ld, float* search_dot,
                               float* decrement, int32_t nworld,
                               int32_t skip_unchanged, int32_t skip_noflip,
                               void* stream);

/* Replaces deriv_smooth_vel_dense_actuator_centric (mjw_step_optimized.py:4172-4412;
 * kernels :629-669 and upstream derivative._qderiv_actuator_passive): out = M - h qDeriv
 * in M's CSR layout, (W, nM).  The factor/solve of the result is
 * imn_tree_ldl_compiled_solve / imn_blocked_dense_factor_solve with y = efc.Ma.
 * Tendon damping and fluid terms are not included. */
int imn_implicit_matrix(const ImnImplicit* p, const float* M, int64_t M_ld, float* out,
                        int64_t out_ld, int32_t nworld, void* stream);

/* Replaces upstream _advance as called by _advance_with_scratch
 * (mjw_step_optimized.py:4823-4847) for models without actuator activations:
 * qvel += h qacc; qpos moves with the new qvel (free and ball joints on the unit
 * quaternions); time += h. */
int imn_advance(const ImnAdvance* p, const float* qacc, int64_t qacc_ld, int32_t nworld,
                void* stream);

/* Replaces BallLimitBuffers.launch (ball_limits.py:221-282, kernel :36-203): appends the
 * violated directional limit rows of every limited ball joint to each world's rows, in
 * (joint, kind) order. */
int imn_ball_limit_rows(const ImnBallLimits* p, int32_t nworld, void* stream);

/* Replaces accumulate (tree_fusion.py:138-170; kernels :52-135): every body's value is
 * added to its parent's, deepest level first, `components` floats per body, in place.
 * values is (W, nbody, components) with world stride `world_ld` floats.  With
 * skip_root_parent the world body receives nothing.  Children are added in level-list
 * order, one writer per parent: the reference's deterministic mode, bit for bit.
 * subtree_com_accumulate (:173-183) is this call with 3 components. */
int imn_body_tree_accumulate(const ImnBodyTree* tree, float* values, int64_t world_ld,
                             int32_t components, int32_t skip_root_parent, int32_t nworld,
                             void* stream);

/* Replaces crb (tree_fusion.py:186-206): crb = cinert summed up the tree (10 floats per
 * body, the world body kept out), then M on its CSR rows (ancestors ascending, diagonal
 * last; every stored entry is written).  cinert, crb: (W, nbody, 10); cdof: (W, nv, 6). */
int imn_crb(const ImnBodyTree* tree, const float* cinert, const float* cdof, float* crb,
            float* M, int64_t M_ld, int32_t nworld, void* stream);

/* Replaces rne (tree_fusion.py:209-222; no acceleration term): cacc down the tree from
 * -gravity, cfrc_int = cinert cacc + cvel x* (cinert cvel) summed up the tree,
 * qfrc_bias = cdof . cfrc_int[dof's body].  cacc, cfrc_int, cvel: (W, nbody, 6);
 * cdof, cdof_dot: (W, nv, 6). */
int imn_rne(const ImnBodyTree* tree, const float* cinert, const float* cvel, const float* cdof,
            const float* cdof_dot, const float* qvel, int64_t qvel_ld, float* cacc,
            float* cfrc_int, float* qfrc_bias, int64_t bias_ld, int32_t nworld, void* stream);

/* Replaces com_vel (velocity_fusion.py:105-126, kernel :15-103): body velocities cvel by
 * depth and cdof_dot = cvel x cdof per dof, joint by joint. */
int imn_com_vel(const ImnBodyTree* tree, const float* qvel, int64_t qvel_ld, const float* cdof,
                float* cvel, float* cdof_dot, int32_t nworld, void* stream);

/* Uploads a sparse plan (sparse_hessian.build_plan's tables, sparse_hessian.py:229-402,
 * which the reference bakes into generated source instead).  `host_tables` holds HOST
 * pointers and the counts; the call copies every table into one device allocation
 * of the current device and returns a plan whose pointers are device pointers, ready
 * for ImnCtx.sparse_plan and imn_sparse_factor_nonfused.  This and
 * imn_tree_ldl_compile / imn_mul_m_compile are the only entry points that allocate; they
 * belong to model set-up, not to the step.  imn_sparse_plan_destroy frees the allocation. */
int imn_sparse_plan_create(const ImnSparsePlan* host_tables, ImnSparsePlan** out);
void imn_sparse_plan_destroy(ImnSparsePlan* plan);

/* Launch geometry the library would use for (m, d): block width of one world
 * (newton_fusion.newton_block_dim, newton_fusion.py:325-327), worlds per CTA,
 * dynamic shared memory per CTA, whether J stays resident in shared memory. */
typedef struct ImnLaunchInfo {
  int32_t world_threads;
  int32_t worlds_per_cta;
  int32_t smem_bytes;
  int32_t j_resident;
  int32_t grid;
} ImnLaunchInfo;
int imn_launch_info(const ImnModel* m, const ImnData* d, const ImnCtx* ctx,
                    ImnLaunchInfo* out);

/* No counterpart in the reference (its fused path takes a dense Jacobian that is already
 * on the GPU).  For callers whose constraint rows are sparse on the host -- MuJoCo C with
 * jacobian="sparse" stores efc_J as values + efc_J_colind + efc_J_rowadr -- so that only
 * the nonzeros cross PCIe: writes `nrows` dense rows of `nv` floats (row stride `ld_row`
 * floats) from the device copies of values, colind and rowadr (nrows + 1 starts).
 * `colind_bytes` is 4 (int32, MuJoCo's) or 1 (uint8: a fused-path model has at most 79
 * dofs, and a producer that emits bytes moves 5 instead of 8 bytes per nonzero).  Rows
 * are cleared first; indices outside [0, nv) are skipped. */
int imn_expand_rows(const float* values, const void* colind, int32_t colind_bytes,
                    const int32_t* rowadr, int32_t nrows, int32_t nv, float* dense,
                    int64_t ld_row, void* stream);

/* Companion of imn_expand_rows for efc.D, efc.aref and efc.frictionloss: the values of the
 * live rows only (worlds back to back, in the order of the compact Jacobian whose per-world
 * element offsets are `J_world_offset`, row stride `J_ld_row`) written into the padded
 * (nworld, efc_ld) arrays.  Rows at or beyond a world's nefc are left as they are. */
int imn_expand_row_vectors(const float* D_rows, const float* aref_rows,
                           const float* frictionloss_rows, const int64_t* J_world_offset,
                           int64_t J_ld_row, const int32_t* nefc, int32_t njmax, float* D,
                           float* aref, float* frictionloss, int64_t efc_ld, int32_t nworld,
                           void* stream);

/* No counterpart in the reference, whose solver buffers never leave the GPU.  For
 * callers that keep a batch in pinned host memory: copies the leading `width` bytes
 * of each of `nworld` per-world blocks (block strides `dst_pitch` / `src_pitch`
 * bytes) between host and device with ONE cudaMemcpy2DAsync on `stream`.  Used to
 * move only rows [0, max nefc) of efc.J / D / aref / frictionloss in and of
 * efc.force / state out: the solver never reads or writes rows at or beyond nefc.
 * to_host 0: host -> device, 1: device -> host. */
int imn_copy_rows(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t width,
                  int32_t nworld, int32_t to_host, void* stream);

/* Failure detection of the input copies (no counterpart in the reference, whose
 * Warp kernels use plain loads).  A world's inputs arrive by TMA bulk copies on an
 * mbarrier; a world waits at most `polls` polls for them (default 1 << 22), then
 * ORs bit 30 into its `overflow` word, waits once more with the same limit for the
 * copies in flight and returns with no result written.  `withhold_copies` is the
 * host-side fault injection of that path: bit 0 makes the initial load, bit 1 the
 * streamed row tiles, bring their data with plain loads while the barrier is still
 * told to expect bytes, so that the wait runs out although nothing is in flight.
 * Process-wide; read when a launch is planned.  Pass (1 << 22, 0) to restore. */
int imn_set_copy_wait_limit(int32_t polls, int32_t withhold_copies);

/* Text of the last validation failure on the calling thread. */
const char* imn_last_error(void);
int imn_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* IMNEWTON_H_ */
