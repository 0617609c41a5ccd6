// imn_integrate.cu -- the implicit-fast integrator's tail, the step right after the
// constraint solve (reference: _integrate, mjw_step_optimized.py:5209-5297):
//
//   1. A = M - h qDeriv on M's sparsity, qDeriv = d(qfrc_smooth)/d(qvel) restricted to
//      the actuator term  sum_a moment_a moment_a^T dforce_a/dvelocity_a  (the
//      actuator-centric assembly, mjw_step_optimized.py:629-669, 4172-4295) and the
//      passive joint damping  -diag(dof_damping)  (upstream _qderiv_actuator_passive);
//   2. x = A^-1 efc.Ma  -- the tree L'DL / blocked dense kernels (imn_msolve.cu,
//      imn_tree_jit.cu), launched by the host layer between the two kernels here;
//   3. the advance  qvel += h x, qpos integrated on its manifold with the new qvel,
//      time += h  (upstream _advance through _advance_with_scratch,
//      mjw_step_optimized.py:4823-4847).
//
// RESTATED: the arithmetic of steps 1 and 3 lives in mujoco-warp (derivative.py,
// forward.py), whose source is not available; what follows is MuJoCo's published
// semi-implicit update (mj_advance, mju_quatIntegrate) and the derivative terms named
// above, with a fixed summation order.  The reference adds the actuator products with
// atomics in whatever order the hardware picks; here an entry receives them in
// ascending actuator order, so results are reproducible bit for bit (and equal to the
// CPU oracle's).  Tendon damping, fluid forces and the free-body correction of
// mujoco-warp 3.16 are not part of this file.
#include "imn_common.cuh"

namespace imn {

// One warp per world.  qD is assembled in the warp's shared-memory row (nM floats),
// then A = M - h qD leaves coalesced.
static const int kMatrixWarps = 8;

__global__ void __launch_bounds__(32 * kMatrixWarps)
    implicit_matrix_kernel(const ImnImplicit P, const float* __restrict__ M, const int64_t M_ld,
                           float* __restrict__ out, const int64_t out_ld, const int nworld) {
  extern __shared__ float qd_all[];
  const int lane = threadIdx.x & 31, w = blockIdx.x * kMatrixWarps + (threadIdx.x >> 5);
  if (w >= nworld) return;
  float* qd = qd_all + (threadIdx.x >> 5) * ((P.nM + 3) & ~3);
  for (int e = lane; e < P.nM; e += 32) qd[e] = 0.0f;
  __syncwarp();
  if (P.nu > 0 && P.actuation) {
    const int* rownnz = P.moment_rownnz + (size_t)w * P.nu;
    const int* rowadr = P.moment_rowadr + (size_t)w * P.nu;
    const int* colind = P.moment_colind + (size_t)w * P.moment_ld;
    const float* moment = P.actuator_moment + (size_t)w * P.moment_ld;
    const float* gain = P.actuator_velocity_gain + (size_t)w * P.nu;
    // Actuators are taken 32 at a time, in ascending order.  A batch whose actuators all
    // act on a single dof (position / velocity servos: the usual case) is added in one
    // step: lane = actuator, lanes that hit the same diagonal entry are ranked by lane and
    // add one rank after the other, which is ascending actuator order.  Any other batch
    // goes actuator by actuator.
#pragma unroll 1
    for (int a0 = 0; a0 < P.nu; a0 += 32) {
      const int a = a0 + lane;
      const bool mine = a < P.nu;
      const int n_mine = mine ? rownnz[a] : 0;
      const float vel_mine = mine ? gain[a] : 0.0f;
      if (__all_sync(IMN_FULL_MASK, n_mine <= 1)) {
        int e = -1;
        float c = 0.0f;
        if (n_mine == 1 && vel_mine != 0.0f) {
          const int base = rowadr[a], di = colind[base];
          e = P.M_elemid[di * P.nv + di];
          c = (moment[base] * moment[base]) * vel_mine;
          if (c == 0.0f) e = -1;
        }
        const unsigned peers = __match_any_sync(IMN_FULL_MASK, e);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const int rounds = __reduce_max_sync(IMN_FULL_MASK, e >= 0 ? __popc(peers) : 0);
#pragma unroll 1
        for (int r = 0; r < rounds; ++r) {
          if (e >= 0 && rank == r) qd[e] = qd[e] + c;
          __syncwarp();
        }
        continue;
      }
      const int a1 = min(a0 + 32, P.nu);
#pragma unroll 1
      for (int s = a0; s < a1; ++s) {
        const float vel = gain[s];
        const int n = rownnz[s];
        if (vel == 0.0f || n <= 0) continue;  // warp-uniform
        const int base = rowadr[s];
        // pairs (ri >= rj) of the actuator's moment row; distinct pairs hit distinct
        // entries of M, so the lanes never collide within one actuator
#pragma unroll 1
        for (int p = lane; p < n * (n + 1) / 2; p += 32) {
          int ri = (int)((sqrtf(8.0f * (float)p + 1.0f) - 1.0f) * 0.5f);
          while ((ri + 1) * (ri + 2) / 2 <= p) ++ri;
          while (ri * (ri + 1) / 2 > p) --ri;
          const int rj = p - ri * (ri + 1) / 2;
          const int di = colind[base + ri], dj = colind[base + rj];
          const int e = P.M_elemid[di * P.nv + dj];
          if (e < 0) continue;
          const float c = (moment[base + ri] * moment[base + rj]) * vel;
          if (c != 0.0f) qd[e] = qd[e] + c;
        }
        __syncwarp();
      }
    }
  }
  if (P.damper)
    for (int i = lane; i < P.nv; i += 32) {
      const int e = P.M_elemid[i * P.nv + i];
      qd[e] = qd[e] - P.dof_damping[i];
    }
  __syncwarp();
  const float* Mw = M + (size_t)w * M_ld;
  float* ow = out + (size_t)w * out_ld;
  const float h = P.timestep[w % P.n_timestep];
#pragma unroll 4
  for (int e = lane; e < P.nM; e += 32) ow[e] = Mw[e] - h * qd[e];
}

__device__ __forceinline__ void quat_integrate(float q[4], const float w[3], float h) {
  // q <- normalise(q (x) [cos(a/2), axis sin(a/2)]),  a = h |w|,  axis = w / |w|
  const float norm = sqrtf(w[0] * w[0] + w[1] * w[1] + w[2] * w[2]);
  float r[4] = {1.0f, 0.0f, 0.0f, 0.0f};
  if (norm >= IMN_MJ_MINVAL) {
    const float half = 0.5f * (h * norm);
    const float s = sinf(half) / norm;
    r[0] = cosf(half), r[1] = w[0] * s, r[2] = w[1] * s, r[3] = w[2] * s;
  }
  const float a = q[0], b = q[1], c = q[2], d = q[3];
  float o[4] = {a * r[0] - b * r[1] - c * r[2] - d * r[3], a * r[1] + b * r[0] + c * r[3] - d * r[2],
                a * r[2] - b * r[3] + c * r[0] + d * r[1], a * r[3] + b * r[2] - c * r[1] + d * r[0]};
  const float len = sqrtf(o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3]);
  if (len < IMN_MJ_MINVAL) {
    q[0] = 1.0f, q[1] = q[2] = q[3] = 0.0f;
    return;
  }
  const float inv = 1.0f / len;
  q[0] = o[0] * inv, q[1] = o[1] * inv, q[2] = o[2] * inv, q[3] = o[3] * inv;
}

// The advance of one joint of one world: its dofs get their new velocity, then its
// coordinates move with it.  `qvel`, `qpos`, `acc` point at the joint's first entry.
__device__ __forceinline__ void advance_joint(int type, float h, float* qvel, float* qpos, const float* acc) {
  const int ndof = type == IMN_JNT_FREE ? 6 : (type == IMN_JNT_BALL ? 3 : 1);
  float v[6];
  for (int k = 0; k < ndof; ++k) {
    v[k] = qvel[k] + h * acc[k];
    qvel[k] = v[k];
  }
  if (type == IMN_JNT_FREE) {
    for (int k = 0; k < 3; ++k) qpos[k] = qpos[k] + h * v[k];
    float q[4] = {qpos[3], qpos[4], qpos[5], qpos[6]};
    quat_integrate(q, v + 3, h);
    for (int k = 0; k < 4; ++k) qpos[3 + k] = q[k];
  } else if (type == IMN_JNT_BALL) {
    float q[4] = {qpos[0], qpos[1], qpos[2], qpos[3]};
    quat_integrate(q, v, h);
    for (int k = 0; k < 4; ++k) qpos[k] = q[k];
  } else {
    qpos[0] = qpos[0] + h * v[0];
  }
}

// A block advances 32 consecutive worlds: their qpos, qvel and qacc rows come into shared
// memory with coalesced loads, lane = world, the warps share the joints (a warp works on
// one joint of 32 worlds at a time, so its lanes take the same branch: with a thread per
// (world, joint) every warp held a free joint next to hinges and ran the quaternion path
// for one lane in 29), and the rows leave with coalesced stores.
static const int kAdvanceWarps = 4;
__host__ __device__ inline int advance_stride(int n) { return (n & 3) == 0 ? (n | 1) : n; }

__global__ void __launch_bounds__(32 * kAdvanceWarps)
    advance_kernel(const ImnAdvance P, const float* __restrict__ qacc, const int64_t qacc_ld, const int nworld) {
  extern __shared__ __align__(16) float rows[];
  // row strides: the lanes of a warp read the same element of 32 rows; a row length that
  // shares a factor of 4 or more with the 32 banks is padded to an odd stride
  const int tq = advance_stride(P.nq), tv = advance_stride(P.nv);
  float* sq = rows;            // [32][tq]
  float* sv = sq + 32 * tq;    // [32][tv]
  float* sa = sv + 32 * tv;    // [32][tv]
  const int w0 = blockIdx.x * 32, nw = min(32, nworld - w0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // the block's rows as one run of nw * n elements over all threads (consecutive threads,
  // consecutive addresses).  Row and column come from a multiplication by 1 / n, exact for
  // these few thousand elements ((e + 1/2) / n is at least 1 / (2 n) away from an integer),
  // so that the iterations do not depend on each other and their loads overlap.
  auto move = [&](float* tile, int stride, float* global, const float* source, int64_t ld, int n, bool store) {
    if (stride == n && ld == n) {  // rows back to back on both sides: one straight copy
      float* g = global ? global + (size_t)w0 * ld : nullptr;
      const float* src = source ? source + (size_t)w0 * ld : g;
#pragma unroll 4
      for (int e = threadIdx.x; e < nw * n; e += 32 * kAdvanceWarps)
        if (store) g[e] = tile[e];
        else tile[e] = src[e];
      return;
    }
    const float inv = 1.0f / (float)n;
#pragma unroll 4
    for (int e = threadIdx.x; e < nw * n; e += 32 * kAdvanceWarps) {
      const int r = (int)(((float)e + 0.5f) * inv), c = e - r * n;
      const size_t at = (size_t)(w0 + r) * ld + c;
      if (store) global[at] = tile[r * stride + c];
      else tile[r * stride + c] = source ? source[at] : global[at];
    }
  };
  move(sq, tq, P.qpos, nullptr, P.qpos_ld, P.nq, false);
  move(sv, tv, P.qvel, nullptr, P.qvel_ld, P.nv, false);
  move(sa, tv, nullptr, qacc, qacc_ld, P.nv, false);
  __syncthreads();
  if (lane < nw) {
    const int w = w0 + lane;
    const float h = P.timestep[w % P.n_timestep];
#pragma unroll 1
    for (int j = warp; j < P.njnt; j += kAdvanceWarps) {
      const int dof = P.jnt_dofadr[j], pos = P.jnt_qposadr[j];
      advance_joint(P.jnt_type[j], h, sv + lane * tv + dof, sq + lane * tq + pos, sa + lane * tv + dof);
    }
    if (warp == 0 && P.time) P.time[w] = P.time[w] + h;
  }
  __syncthreads();
  move(sq, tq, P.qpos, nullptr, P.qpos_ld, P.nq, true);
  move(sv, tv, P.qvel, nullptr, P.qvel_ld, P.nv, true);
}

}  // namespace imn

extern "C" int imn_implicit_matrix(const ImnImplicit* p, const float* M, int64_t M_ld, float* out, int64_t out_ld,
                                   int32_t nworld, void* stream) {
  if (!p || !M || !out || !p->M_elemid || !p->timestep)
    return imn::set_error("imn_implicit_matrix: NULL argument"), IMN_ERR_NULL;
  if (p->n_timestep <= 0) return imn::set_error("imn_implicit_matrix: empty opt.timestep"), IMN_ERR_SHAPE;
  if (p->nv <= 0 || p->nM <= 0 || p->nu < 0 || nworld < 0 || M_ld < p->nM || out_ld < p->nM)
    return imn::set_error("imn_implicit_matrix: bad extent or stride"), IMN_ERR_SHAPE;
  if (p->damper && !p->dof_damping) return imn::set_error("imn_implicit_matrix: dof_damping is NULL"), IMN_ERR_NULL;
  if (p->nu > 0 && p->actuation &&
      (!p->moment_rownnz || !p->moment_rowadr || !p->moment_colind || !p->actuator_moment ||
       !p->actuator_velocity_gain || p->moment_ld <= 0))
    return imn::set_error("imn_implicit_matrix: an actuator array is NULL"), IMN_ERR_NULL;
  if (nworld == 0) return IMN_OK;
  const size_t bytes = sizeof(float) * (size_t)((p->nM + 3) & ~3) * imn::kMatrixWarps;
  if (bytes > 227 * 1024) return imn::set_error("imn_implicit_matrix: nM %d too large", p->nM), IMN_ERR_LIMIT;
  if (bytes > 48 * 1024) {
    cudaError_t e =
        cudaFuncSetAttribute(imn::implicit_matrix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess)
      return imn::set_error("imn_implicit_matrix: cudaFuncSetAttribute: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  }
  imn::implicit_matrix_kernel<<<(nworld + imn::kMatrixWarps - 1) / imn::kMatrixWarps, 32 * imn::kMatrixWarps, bytes,
                                (cudaStream_t)stream>>>(*p, M, M_ld, out, out_ld, nworld);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return imn::set_error("imn_implicit_matrix: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}

extern "C" int imn_advance(const ImnAdvance* p, const float* qacc, int64_t qacc_ld, int32_t nworld, void* stream) {
  if (!p || !qacc || !p->qvel || !p->qpos || !p->jnt_type || !p->jnt_dofadr || !p->jnt_qposadr || !p->timestep)
    return imn::set_error("imn_advance: NULL argument"), IMN_ERR_NULL;
  if (p->n_timestep <= 0) return imn::set_error("imn_advance: empty opt.timestep"), IMN_ERR_SHAPE;
  if (p->njnt <= 0 || p->nv <= 0 || p->nq < p->nv || nworld < 0 || qacc_ld < p->nv || p->qvel_ld < p->nv ||
      p->qpos_ld < p->nq)
    return imn::set_error("imn_advance: bad extent or stride"), IMN_ERR_SHAPE;
  if (nworld == 0) return IMN_OK;
  const size_t bytes = sizeof(float) * 32 * ((size_t)imn::advance_stride(p->nq) + 2 * (size_t)imn::advance_stride(p->nv));
  if (bytes > 227 * 1024) return imn::set_error("imn_advance: nq %d too large", p->nq), IMN_ERR_LIMIT;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(imn::advance_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess)
      return imn::set_error("imn_advance: cudaFuncSetAttribute: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  }
  imn::advance_kernel<<<(unsigned)((nworld + 31) / 32), 32 * imn::kAdvanceWarps, bytes, (cudaStream_t)stream>>>(
      *p, qacc, qacc_ld, nworld);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return imn::set_error("imn_advance: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}
