// imn_body_tree.cu -- bottom-up body-tree reductions and the smooth-dynamics stages
// built on them (reference: src/instantmimic/utils/mjw_kernels/tree_fusion.py,
// velocity_fusion.py):
//
//   imn_body_tree_accumulate   accumulate()      tree_fusion.py:52-170  (also
//                              subtree_com_accumulate, :173-183, with 3 components)
//   imn_crb                    crb()             tree_fusion.py:186-206 (composite
//                              inertias, then the joint-space inertia M)
//   imn_rne                    rne()             tree_fusion.py:209-222 (bias forces)
//   imn_com_vel                com_vel()         velocity_fusion.py:15-126
//
// The reference walks m.body_tree inside one cooperative block per world, one level
// after the other with a block barrier in between.  Here a world is a team of 8, 16 or 32
// lanes of a warp: its per-body values sit in the team's slice of shared memory, a level
// is a strided loop over (body, component) entries, and __syncwarp() separates levels.  Inputs arrive
// and results leave as contiguous per-world runs (coalesced); nothing is read twice
// from HBM.
//
// Summation order.  A parent receives its children in the order in which they stand
// in the level list, one writer per (parent, component): the reference's
// deterministic kernels (tree_fusion.py:80-135), which its own test pins bit for bit
// against a sequential depth-ordered sum.  The unordered (atomic) mode of the
// reference has no order to reproduce; the ordered result satisfies its tolerance.
//
// RESTATED: the per-body arithmetic of crb / rne (spatial inertia times motion vector,
// force cross product, the ancestor walk of M, the bias projection) lives in
// mujoco-warp's smooth.py and math.py, whose source is not available; what follows is
// MuJoCo's published mj_crb / mj_rne / mj_comVel arithmetic with sums written as
// left-to-right fused multiply-add chains.  velocity_fusion.py spells its joint
// branches out, and those are followed statement by statement.
#include "imn_common.cuh"

namespace imn {

static const int kTreeWarps = 4;

struct Sp6 {
  float v[6];
};

__device__ __forceinline__ Sp6 ld6(const float* p) {
  Sp6 r;
#pragma unroll
  for (int k = 0; k < 6; ++k) r.v[k] = p[k];
  return r;
}
__device__ __forceinline__ void st6(float* p, const Sp6& a) {
#pragma unroll
  for (int k = 0; k < 6; ++k) p[k] = a.v[k];
}
// a + b * s, component by component
__device__ __forceinline__ Sp6 axpy6(const Sp6& a, const Sp6& b, float s) {
  Sp6 r;
#pragma unroll
  for (int k = 0; k < 6; ++k) r.v[k] = fmaf(b.v[k], s, a.v[k]);
  return r;
}
__device__ __forceinline__ float dot6(const Sp6& a, const Sp6& b) {
  float acc = a.v[0] * b.v[0];
#pragma unroll
  for (int k = 1; k < 6; ++k) acc = fmaf(a.v[k], b.v[k], acc);
  return acc;
}
// x y' - y x'
__device__ __forceinline__ float det2(float x, float yp, float y, float xp) { return fmaf(x, yp, -(y * xp)); }
__device__ __forceinline__ void cross3(const float* a, const float* b, float* r) {
  r[0] = det2(a[1], b[2], a[2], b[1]);
  r[1] = det2(a[2], b[0], a[0], b[2]);
  r[2] = det2(a[0], b[1], a[1], b[0]);
}
// Spatial motion cross product (MuJoCo mju_crossMotion): angular = w x a_ang,
// linear = w x a_lin + v x a_ang, for vel = (w, v).
__device__ __forceinline__ Sp6 motion_cross(const Sp6& vel, const Sp6& a) {
  Sp6 r;
  float t[3], u[3];
  cross3(vel.v, a.v, r.v);
  cross3(vel.v, a.v + 3, t);
  cross3(vel.v + 3, a.v, u);
#pragma unroll
  for (int k = 0; k < 3; ++k) r.v[3 + k] = t[k] + u[k];
  return r;
}
// Spatial force cross product (MuJoCo mju_crossForce): angular = w x f_ang + v x f_lin,
// linear = w x f_lin.
__device__ __forceinline__ Sp6 motion_cross_force(const Sp6& vel, const Sp6& f) {
  Sp6 r;
  float t[3], u[3];
  cross3(vel.v, f.v, t);
  cross3(vel.v + 3, f.v + 3, u);
#pragma unroll
  for (int k = 0; k < 3; ++k) r.v[k] = t[k] + u[k];
  cross3(vel.v, f.v + 3, r.v + 3);
  return r;
}
// 10-number spatial inertia (Ixx Iyy Izz Ixy Ixz Iyz, m*cx m*cy m*cz, m) times a motion
// vector (MuJoCo mju_mulInertVec), each sum a left-to-right chain contracted the way
// nvcc contracts "a*b + c*d + ..." (the first sum or difference of two products fuses
// its LEFT product and rounds the right one; every later product is fused into the
// running value) -- the rule the reference's generated tree L'DL code follows when run.
__device__ __forceinline__ Sp6 inert_vec(const float* i, const Sp6& a) {
  const float* v = a.v;
  Sp6 r;
  r.v[0] = fmaf(i[7], v[5], fmaf(-i[8], v[4], fmaf(i[4], v[2], fmaf(i[0], v[0], i[3] * v[1]))));
  r.v[1] = fmaf(-i[6], v[5], fmaf(i[8], v[3], fmaf(i[5], v[2], fmaf(i[3], v[0], i[1] * v[1]))));
  r.v[2] = fmaf(i[6], v[4], fmaf(-i[7], v[3], fmaf(i[2], v[2], fmaf(i[4], v[0], i[5] * v[1]))));
  r.v[3] = fmaf(i[9], v[3], fmaf(i[8], v[1], -(i[7] * v[2])));
  r.v[4] = fmaf(i[9], v[4], fmaf(i[6], v[2], -(i[8] * v[0])));
  r.v[5] = fmaf(i[9], v[5], fmaf(i[7], v[0], -(i[6] * v[1])));
  return r;
}

// A world is worked on by a team of GW lanes (8, 16 or 32): the levels of a body tree are a
// few bodies wide, so a whole warp per world would leave most lanes idle through the
// per-body arithmetic (measured: 8 of 32 lanes active per instruction, the kernels bound by
// instruction issue).  A warp therefore takes 32 / GW consecutive worlds; control flow is the
// same for all of them (one model), so __syncwarp() separates levels for every team at once.
// The last warp's surplus teams run on the last world and store nothing.
template <int GW>
struct Team {
  int sl;      // lane within the team
  int w;       // the team's world (clamped to the batch)
  int slot;    // the team's slice of the CTA's shared memory
  bool live;   // false: surplus team, no stores
  bool none;   // the whole warp is surplus
};
template <int GW>
__device__ __forceinline__ Team<GW> make_team(int nworld) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, per = 32 / GW;
  const int first = (blockIdx.x * kTreeWarps + warp) * per, sub = lane / GW;
  Team<GW> t;
  t.sl = lane - sub * GW;
  t.live = first + sub < nworld;
  t.w = t.live ? first + sub : nworld - 1;
  t.slot = warp * per + sub;
  t.none = first >= nworld;
  return t;
}

// Bottom-up sweep over the team's values (nbody x C floats in shared memory): the
// parents of a level take their children of the next level, in level-list order
// (tree_fusion.py:94-112).  child_ptr is indexed by the parent's position in the level
// list.
template <int GW>
__device__ __forceinline__ void sweep_up(const ImnBodyTree& T, float* v, int C, bool skip_root_parent, int sl) {
#pragma unroll 1
  for (int level = T.nlevels - 1; level > 0; --level) {
    const int pstart = T.level_offsets[level - 1];
    const int pcount = T.level_offsets[level] - pstart;
#pragma unroll 1
    for (int entry = sl; entry < pcount * C; entry += GW) {
      const int pos = pstart + entry / C, comp = entry - (entry / C) * C;
      const int parent = T.level_bodies[pos];
      if (skip_root_parent && parent == 0) continue;
      float value = v[parent * C + comp];
      const int cend = T.child_ptr[pos + 1];
#pragma unroll 1
      for (int k = T.child_ptr[pos]; k < cend; ++k) value = value + v[T.child_ids[k] * C + comp];
      v[parent * C + comp] = value;
    }
    __syncwarp();
  }
}

// Per-world runs are a few hundred floats: four loads in flight per lane.
template <int GW>
__device__ __forceinline__ void copy_in(float* dst, const float* __restrict__ src, int n, int sl) {
  int i = sl;
#pragma unroll 1
  for (; i + 3 * GW < n; i += 4 * GW) {
    const float a = src[i], b = src[i + GW], c = src[i + 2 * GW], d = src[i + 3 * GW];
    dst[i] = a, dst[i + GW] = b, dst[i + 2 * GW] = c, dst[i + 3 * GW] = d;
  }
#pragma unroll 1
  for (; i < n; i += GW) dst[i] = src[i];
}
template <int GW>
__device__ __forceinline__ void copy_out(float* __restrict__ dst, const float* src, int n, int sl, bool live) {
  if (!live) return;
#pragma unroll 4
  for (int i = sl; i < n; i += GW) dst[i] = src[i];
}

template <int GW>
__global__ void __launch_bounds__(32 * kTreeWarps)
    tree_accumulate_kernel(const ImnBodyTree T, float* __restrict__ values, const int64_t world_ld, const int C,
                           const int skip_root_parent, const int nworld) {
  extern __shared__ __align__(16) float tree_smem[];
  const Team<GW> t = make_team<GW>(nworld);
  if (t.none) return;
  const int n = T.nbody * C;
  float* v = tree_smem + (size_t)t.slot * ((n + 3) & ~3);
  float* g = values + (size_t)t.w * world_ld;
  copy_in<GW>(v, g, n, t.sl);
  __syncwarp();
  sweep_up<GW>(T, v, C, skip_root_parent != 0, t.sl);
  copy_out<GW>(g, v, n, t.sl, t.live);
}

// crb: composite inertias (cinert summed up the tree, the world body's children kept
// out of it: tree_fusion.py:190-191), then M (tree_fusion.py:192-206): row i of M holds
// i's ancestors in ascending order with the diagonal last; entry (i, j) is
// cdof_j . (crb[body_i] cdof_i), the diagonal on top of the armature.
template <int GW>
__global__ void __launch_bounds__(32 * kTreeWarps)
    crb_kernel(const ImnBodyTree T, const float* __restrict__ cinert, const float* __restrict__ cdof,
               float* __restrict__ crb, float* __restrict__ M, const int64_t M_ld, const int nworld) {
  extern __shared__ __align__(16) float tree_smem[];
  const Team<GW> t = make_team<GW>(nworld);
  if (t.none) return;
  const int sl = t.sl, w = t.w;
  const int nb10 = T.nbody * 10, nv6 = T.nv * 6;
  float* c = tree_smem + (size_t)t.slot * (((nb10 + 3) & ~3) + 2 * ((nv6 + 3) & ~3));
  float* dof = c + ((nb10 + 3) & ~3);
  float* bufs = dof + ((nv6 + 3) & ~3);
  copy_in<GW>(c, cinert + (size_t)w * nb10, nb10, sl);
  copy_in<GW>(dof, cdof + (size_t)w * nv6, nv6, sl);
  __syncwarp();
  sweep_up<GW>(T, c, 10, true, sl);
  copy_out<GW>(crb + (size_t)w * nb10, c, nb10, sl, t.live);
  const float* arm = T.dof_armature + (size_t)(w % T.n_armature) * T.nv;
  float* Mw = M + (size_t)w * M_ld;
  // crb[body_i] cdof_i per dof, then one stored entry of M per lane: entry e = (i, j) is
  // cdof_j . buf_i -- the ancestor walk of the reference flattened over M's CSR, so that
  // every lane is busy and consecutive lanes store consecutive entries
#pragma unroll 1
  for (int i = sl; i < T.nv; i += GW) st6(bufs + 6 * i, inert_vec(c + 10 * T.dof_bodyid[i], ld6(dof + 6 * i)));
  __syncwarp();
#pragma unroll 2
  for (int e = sl; e < T.nM; e += GW) {
    const int i = T.M_rowidx[e], j = T.M_colind[e];
    float v = dot6(ld6(dof + 6 * j), ld6(bufs + 6 * i));
    if (i == j) v = arm[i] + v;
    if (t.live) Mw[e] = v;
  }
}

// rne without accelerations (tree_fusion.py:209-222): cacc down the tree from
// -gravity, per-body forces cinert cacc + cvel x* (cinert cvel), summed up the tree,
// projected on the dofs.
template <int GW>
__global__ void __launch_bounds__(32 * kTreeWarps)
    rne_kernel(const ImnBodyTree T, const float* __restrict__ cinert, const float* __restrict__ cvel,
               const float* __restrict__ cdof, const float* __restrict__ cdof_dot, const float* __restrict__ qvel,
               const int64_t qvel_ld, float* __restrict__ cacc_out, float* __restrict__ cfrc_out,
               float* __restrict__ qfrc_bias, const int64_t bias_ld, const int nworld) {
  extern __shared__ __align__(16) float tree_smem[];
  const Team<GW> t = make_team<GW>(nworld);
  if (t.none) return;
  const int sl = t.sl, w = t.w;
  const int nb6 = T.nbody * 6, nv6 = T.nv * 6, nb6p = (nb6 + 3) & ~3, nv6p = (nv6 + 3) & ~3;
  float* cacc = tree_smem + (size_t)t.slot * (2 * nb6p + nv6p);
  float* cfrc = cacc + nb6p;
  float* dd = cfrc + nb6p;  // cdof_dot, then cdof
  copy_in<GW>(dd, cdof_dot + (size_t)w * nv6, nv6, sl);
  if (sl < 6) {
    const float* g = T.gravity + 3 * (size_t)(w % T.n_gravity);
    cacc[sl] = (sl < 3 || !T.gravity_enabled) ? 0.0f : -g[sl - 3];
    cfrc[sl] = 0.0f;
  }
  __syncwarp();
  const float* qv = qvel + (size_t)w * qvel_ld;
#pragma unroll 1
  for (int level = 1; level < T.nlevels; ++level) {
    const int end = T.level_offsets[level + 1];
#pragma unroll 1
    for (int pos = T.level_offsets[level] + sl; pos < end; pos += GW) {
      const int b = T.level_bodies[pos];
      Sp6 a = ld6(cacc + 6 * T.body_parentid[b]);
      const int d0 = T.body_dofadr[b], d1 = d0 + T.body_dofnum[b];
#pragma unroll 1
      for (int dofid = d0; dofid < d1; ++dofid) a = axpy6(a, ld6(dd + 6 * dofid), qv[dofid]);
      st6(cacc + 6 * b, a);
    }
    __syncwarp();
  }
  copy_out<GW>(cacc_out + (size_t)w * nb6, cacc, nb6, sl, t.live);
#pragma unroll 1
  for (int b = 1 + sl; b < T.nbody; b += GW) {
    const float* I = cinert + ((size_t)w * T.nbody + b) * 10;
    float in[10];
#pragma unroll
    for (int k = 0; k < 10; ++k) in[k] = I[k];
    const Sp6 v = ld6(cvel + ((size_t)w * T.nbody + b) * 6);
    const Sp6 f = inert_vec(in, ld6(cacc + 6 * b));
    const Sp6 x = motion_cross_force(v, inert_vec(in, v));
    Sp6 r;
#pragma unroll
    for (int k = 0; k < 6; ++k) r.v[k] = f.v[k] + x.v[k];
    st6(cfrc + 6 * b, r);
  }
  __syncwarp();
  copy_in<GW>(dd, cdof + (size_t)w * nv6, nv6, sl);  // cdof_dot is no longer needed
  sweep_up<GW>(T, cfrc, 6, false, sl);
  __syncwarp();
  copy_out<GW>(cfrc_out + (size_t)w * nb6, cfrc, nb6, sl, t.live);
  float* bias = qfrc_bias + (size_t)w * bias_ld;
#pragma unroll 1
  for (int i = sl; i < T.nv; i += GW) {
    const float e = dot6(ld6(dd + 6 * i), ld6(cfrc + 6 * T.dof_bodyid[i]));
    if (t.live) bias[i] = e;
  }
}

// Body velocities by depth (velocity_fusion.py:15-103): cvel of a body is its parent's
// plus cdof qvel of its own dofs; cdof_dot of a dof is cvel x cdof taken before that
// dof's own contribution (for a free joint: the three translations first, zero
// cdof_dot; then the rotations against the velocity that includes the translations).
template <int GW>
__global__ void __launch_bounds__(32 * kTreeWarps)
    com_vel_kernel(const ImnBodyTree T, const float* __restrict__ qvel, const int64_t qvel_ld,
                   const float* __restrict__ cdof, float* __restrict__ cvel_out, float* __restrict__ cdof_dot_out,
                   const int nworld) {
  extern __shared__ __align__(16) float tree_smem[];
  const Team<GW> t = make_team<GW>(nworld);
  if (t.none) return;
  const int sl = t.sl, w = t.w;
  const int nb6 = T.nbody * 6, nv6 = T.nv * 6, nb6p = (nb6 + 3) & ~3, nv6p = (nv6 + 3) & ~3;
  float* cvel = tree_smem + (size_t)t.slot * (nb6p + 2 * nv6p);
  float* dof = cvel + nb6p;
  float* dot = dof + nv6p;
  copy_in<GW>(dof, cdof + (size_t)w * nv6, nv6, sl);
  __syncwarp();
  const float* qv = qvel + (size_t)w * qvel_ld;
#pragma unroll 1
  for (int level = 0; level < T.nlevels; ++level) {
    const int end = T.level_offsets[level + 1];
#pragma unroll 1
    for (int pos = T.level_offsets[level] + sl; pos < end; pos += GW) {
      const int b = T.level_bodies[pos];
      Sp6 v;
      if (b == 0) {
#pragma unroll
        for (int k = 0; k < 6; ++k) v.v[k] = 0.0f;
      } else {
        v = ld6(cvel + 6 * T.body_parentid[b]);
        int dofid = T.body_dofadr[b];
        const int j1 = T.body_jntadr[b] + T.body_jntnum[b];
#pragma unroll 1
        for (int j = T.body_jntadr[b]; j < j1; ++j) {
          const int type = T.jnt_type[j];
          if (type == IMN_JNT_FREE) {
            Sp6 zero;
#pragma unroll
            for (int k = 0; k < 6; ++k) zero.v[k] = 0.0f;
#pragma unroll 1
            for (int k = 0; k < 3; ++k) {
              v = axpy6(v, ld6(dof + 6 * (dofid + k)), qv[dofid + k]);
              st6(dot + 6 * (dofid + k), zero);
            }
#pragma unroll 1
            for (int k = 3; k < 6; ++k) st6(dot + 6 * (dofid + k), motion_cross(v, ld6(dof + 6 * (dofid + k))));
#pragma unroll 1
            for (int k = 3; k < 6; ++k) v = axpy6(v, ld6(dof + 6 * (dofid + k)), qv[dofid + k]);
            dofid += 6;
          } else if (type == IMN_JNT_BALL) {
#pragma unroll 1
            for (int k = 0; k < 3; ++k) st6(dot + 6 * (dofid + k), motion_cross(v, ld6(dof + 6 * (dofid + k))));
#pragma unroll 1
            for (int k = 0; k < 3; ++k) v = axpy6(v, ld6(dof + 6 * (dofid + k)), qv[dofid + k]);
            dofid += 3;
          } else {
            st6(dot + 6 * dofid, motion_cross(v, ld6(dof + 6 * dofid)));
            v = axpy6(v, ld6(dof + 6 * dofid), qv[dofid]);
            dofid += 1;
          }
        }
      }
      st6(cvel + 6 * b, v);
    }
    __syncwarp();
  }
  copy_out<GW>(cvel_out + (size_t)w * nb6, cvel, nb6, sl, t.live);
  copy_out<GW>(cdof_dot_out + (size_t)w * nv6, dot, nv6, sl, t.live);
}

}  // namespace imn

#include "imn_body_tree_tile.cuh"

namespace imn {

static int check_tree(const ImnBodyTree* T, const char* who, bool need_dofs) {
  if (!T) return set_error("%s: NULL tree", who), IMN_ERR_NULL;
  if (T->nbody <= 0 || T->nlevels <= 0) return set_error("%s: empty body tree", who), IMN_ERR_SHAPE;
  if (!T->body_parentid || !T->level_bodies || !T->level_offsets || !T->child_ptr || !T->child_ids)
    return set_error("%s: a body-tree table is NULL", who), IMN_ERR_NULL;
  if (need_dofs) {
    if (T->nv <= 0) return set_error("%s: nv must be positive", who), IMN_ERR_SHAPE;
    if (!T->dof_bodyid || !T->dof_parentid || !T->body_dofadr || !T->body_dofnum)
      return set_error("%s: a dof table is NULL", who), IMN_ERR_NULL;
  }
  return IMN_OK;
}

// Lanes per world: the tree's team_lanes when it is 8, 16 or 32 (the host mirror sets the
// smallest that covers the widest level), else a whole warp.
// Per kernel the width is raised to what was measured fastest on a B200 (65536 worlds,
// 14-body / 34-dof and 24-body / 56-dof humanoids, widths 8 / 16 / 32 in us):
//   tree sum, 3 components   19 / 25 / 41     29 / 39 / 64    -> the tree's width
//   com_vel                  64 / 70 / 111   132 / 121 / 163  -> the tree's width
//   rne                      99 / 74 / 113   189 / 139 / 159  -> at least 16
//   crb                     141 / 101 / 88   473 / 255 / 187  -> 32
// A narrow team fills the lanes during the per-body arithmetic but multiplies the shared
// memory of a CTA (16 worlds instead of 4), which costs resident warps: crb keeps three
// per-world arrays on chip and its entry loop fills a whole warp anyway.
static int team_lanes(const ImnBodyTree* T, int at_least = 8) {
  const int lanes = (T->team_lanes == 8 || T->team_lanes == 16) ? T->team_lanes : 32;
  return lanes > at_least ? lanes : at_least;
}

template <typename... Args>
static int launch_tree(const char* who, void (*kernel)(Args...), int gw, size_t floats_per_world, int nworld,
                       void* stream, Args... args) {
  if (nworld < 0) return set_error("%s: negative world count", who), IMN_ERR_SHAPE;
  if (nworld == 0) return IMN_OK;
  const int per_cta = kTreeWarps * (32 / gw);
  const size_t bytes = floats_per_world * 4 * per_cta;
  if (bytes > 227 * 1024)
    return set_error("%s: %zu bytes of shared memory per block exceed the 227 KB of an SM", who, bytes), IMN_ERR_LIMIT;
  if (bytes > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return set_error("%s: cudaFuncSetAttribute: %s", who, cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  }
  kernel<<<(nworld + per_cta - 1) / per_cta, 32 * kTreeWarps, bytes, (cudaStream_t)stream>>>(args...);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("%s: launch failed: %s", who, cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}

static size_t up4z(size_t n) { return (n + 3) & ~(size_t)3; }

// The lane-per-world kernels take over from 4096 worlds on (128 blocks of 32 worlds: below
// that the teams fill the GPU better) when two blocks' rows fit an SM's shared memory.
static bool use_tiles(int nworld, size_t bytes) { return nworld >= 4096 && bytes <= 113 * 1024; }

template <typename... Args>
static int launch_tile(const char* who, void (*kernel)(Args...), size_t bytes, int nworld, void* stream, Args... args) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return set_error("%s: cudaFuncSetAttribute: %s", who, cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  }
  kernel<<<(nworld + 31) / 32, 32 * kTileWarps, bytes, (cudaStream_t)stream>>>(args...);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("%s: launch failed: %s", who, cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}
static size_t oddz(size_t n) { return n | 1; }

// KERNEL<8 | 16 | 32> by the tree's team width
#define IMN_TEAM_LAUNCH(LANES, KERNEL, FLOATS, NWORLD, STREAM, ...)                                \
  ((LANES) == 8    ? imn::launch_tree(who, KERNEL<8>, 8, FLOATS, NWORLD, STREAM, __VA_ARGS__)   \
   : (LANES) == 16 ? imn::launch_tree(who, KERNEL<16>, 16, FLOATS, NWORLD, STREAM, __VA_ARGS__) \
                   : imn::launch_tree(who, KERNEL<32>, 32, FLOATS, NWORLD, STREAM, __VA_ARGS__))

}  // namespace imn

extern "C" int imn_body_tree_accumulate(const ImnBodyTree* T, float* values, int64_t world_ld, int32_t components,
                                        int32_t skip_root_parent, int32_t nworld, void* stream) {
  const char* who = "imn_body_tree_accumulate";
  int rc = imn::check_tree(T, who, false);
  if (rc) return rc;
  if (!values) return imn::set_error("%s: NULL values", who), IMN_ERR_NULL;
  if (components <= 0 || world_ld < (int64_t)T->nbody * components)
    return imn::set_error("%s: components %d / world stride %lld do not hold %d bodies", who, components,
                          (long long)world_ld, T->nbody),
           IMN_ERR_SHAPE;
  return IMN_TEAM_LAUNCH(imn::team_lanes(T), imn::tree_accumulate_kernel, imn::up4z((size_t)T->nbody * components), nworld, stream, *T,
                         values, world_ld, (int)components, (int)skip_root_parent, (int)nworld);
}

extern "C" int imn_crb(const ImnBodyTree* T, const float* cinert, const float* cdof, float* crb, float* M,
                       int64_t M_ld, int32_t nworld, void* stream) {
  const char* who = "imn_crb";
  int rc = imn::check_tree(T, who, true);
  if (rc) return rc;
  if (!cinert || !cdof || !crb || !M || !T->dof_armature || !T->M_rowidx || !T->M_colind)
    return imn::set_error("%s: NULL array", who), IMN_ERR_NULL;
  if (T->n_armature <= 0 || M_ld < T->nM) return imn::set_error("%s: bad armature count or M stride", who), IMN_ERR_SHAPE;
  return IMN_TEAM_LAUNCH(imn::team_lanes(T, 32), imn::crb_kernel,
                         imn::up4z((size_t)T->nbody * 10) + 2 * imn::up4z((size_t)T->nv * 6), nworld,
                         stream, *T, cinert, cdof, crb, M, M_ld, (int)nworld);
}

extern "C" int imn_rne(const ImnBodyTree* T, const float* cinert, const float* cvel, const float* cdof,
                       const float* cdof_dot, const float* qvel, int64_t qvel_ld, float* cacc, float* cfrc_int,
                       float* qfrc_bias, int64_t bias_ld, int32_t nworld, void* stream) {
  const char* who = "imn_rne";
  int rc = imn::check_tree(T, who, true);
  if (rc) return rc;
  if (!cinert || !cvel || !cdof || !cdof_dot || !qvel || !cacc || !cfrc_int || !qfrc_bias || !T->gravity)
    return imn::set_error("%s: NULL array", who), IMN_ERR_NULL;
  if (T->n_gravity <= 0 || qvel_ld < T->nv || bias_ld < T->nv)
    return imn::set_error("%s: bad gravity count or stride", who), IMN_ERR_SHAPE;
  return IMN_TEAM_LAUNCH(imn::team_lanes(T, 16), imn::rne_kernel, 2 * imn::up4z((size_t)T->nbody * 6) + imn::up4z((size_t)T->nv * 6), nworld,
                         stream, *T, cinert, cvel, cdof, cdof_dot, qvel, qvel_ld, cacc, cfrc_int, qfrc_bias, bias_ld,
                         (int)nworld);
}

extern "C" int imn_com_vel(const ImnBodyTree* T, const float* qvel, int64_t qvel_ld, const float* cdof, float* cvel,
                           float* cdof_dot, int32_t nworld, void* stream) {
  const char* who = "imn_com_vel";
  int rc = imn::check_tree(T, who, true);
  if (rc) return rc;
  if (!qvel || !cdof || !cvel || !cdof_dot || !T->body_jntadr || !T->body_jntnum || !T->jnt_type)
    return imn::set_error("%s: NULL array", who), IMN_ERR_NULL;
  if (qvel_ld < T->nv) return imn::set_error("%s: qvel stride < nv", who), IMN_ERR_SHAPE;
  {
    const size_t bytes =
        128 * (imn::oddz((size_t)T->nbody * 6) + 2 * imn::oddz((size_t)T->nv * 6) + imn::oddz(T->nv));
    if (imn::use_tiles(nworld, bytes))
      return imn::launch_tile(who, imn::com_vel_tile_kernel, bytes, nworld, stream, *T, qvel, qvel_ld, cdof, cvel,
                              cdof_dot, (int)nworld);
  }
  return IMN_TEAM_LAUNCH(imn::team_lanes(T), imn::com_vel_kernel, imn::up4z((size_t)T->nbody * 6) + 2 * imn::up4z((size_t)T->nv * 6),
                         nworld, stream, *T, qvel, qvel_ld, cdof, cvel, cdof_dot, (int)nworld);
}
