// imn_body_tree_tile.cuh -- com_vel for batches that fill the GPU: a block takes 32
// consecutive worlds, lane = world.
//
// With a team of lanes per world (imn_body_tree.cu) every lane walks the model's tables
// for its own body, and a level a few bodies wide leaves most of a team idle: 1600 warp
// instructions per world, 8 of 32 lanes active, the kernel bound by instruction issue at a
// third of the HBM rate.  Here the 32 lanes of a warp work on the same body of 32 worlds:
// table lookups and control flow are uniform (one instruction serves 32 worlds), every
// lane is busy, and the per-body arithmetic is the team kernel's own (same helpers, same
// order), so the bits are the same.  Measured per 65536 worlds on a B200: 14-body / 34-dof
// humanoid 62.6 -> 54.6 us, 24-body / 56-dof 130.5 -> 98.0 us, 31-body / 35-dof 103.7 -> 93.7.
// The same mapping of crb and rne was slower than their team kernels (140 vs 86 us, 123 vs
// 72 us): with two blocks of 80 KB per SM the serial chain of uniform table lookups and
// shared-memory reads per body is not covered by other warps; they keep the teams.
//
// Memory.  Each per-world array comes into shared memory as 32 rows (coalesced loads by
// the block's warps) with an odd row stride, so that the lanes of a warp, which read the
// same element of 32 different rows, hit 32 different banks.  Results leave the same way.
// The warps of a block share the bodies of a level and meet at a block barrier between
// levels.
#pragma once

namespace imn {

static const int kTileWarps = 8;

__device__ __forceinline__ int odd(int n) { return n | 1; }

// tile[r][0..n) <- g[(w0 + r) * ld + ...], rows past the batch repeat the last world.  A warp
// takes four rows at a time and four 128-byte runs of each, so that sixteen loads per lane
// are in flight before the first store: with 8 to 24 warps per SM the loads' latency, not
// HBM, would otherwise bound the kernels (measured: 0.7 TB/s with four loads in flight).
__device__ __forceinline__ void rows_in(float* tile, int stride, const float* __restrict__ g, int64_t ld, int n, int w0,
                                        int nworld) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int R = 4, U = 4;
  static_assert(32 % (R * kTileWarps) == 0, "rows are dealt in groups of R per warp");
#pragma unroll 1
  for (int r0 = warp; r0 < 32; r0 += R * kTileWarps) {
    const float* src[R];
#pragma unroll
    for (int q = 0; q < R; ++q) src[q] = g + (size_t)min(w0 + r0 + q * kTileWarps, nworld - 1) * ld;
#pragma unroll 1
    for (int c0 = lane; c0 < n; c0 += 32 * U) {
      float v[R][U];
#pragma unroll
      for (int q = 0; q < R; ++q)
#pragma unroll
        for (int u = 0; u < U; ++u) v[q][u] = c0 + 32 * u < n ? src[q][c0 + 32 * u] : 0.0f;
#pragma unroll
      for (int q = 0; q < R; ++q)
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (c0 + 32 * u < n) tile[(r0 + q * kTileWarps) * stride + c0 + 32 * u] = v[q][u];
    }
  }
}
__device__ __forceinline__ void rows_out(float* __restrict__ g, int64_t ld, const float* tile, int stride, int n, int w0,
                                         int nworld) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll 1
  for (int r = warp; r < 32 && w0 + r < nworld; r += kTileWarps) {
    float* dst = g + (size_t)(w0 + r) * ld;
    const float* src = tile + r * stride;
#pragma unroll 4
    for (int c = lane; c < n; c += 32) dst[c] = src[c];
  }
}

// com_vel (velocity_fusion.py:15-103), top-down by level.
__global__ void __launch_bounds__(32 * kTileWarps)
    com_vel_tile_kernel(const ImnBodyTree T, const float* __restrict__ qvel, const int64_t qvel_ld,
                        const float* __restrict__ cdof, float* __restrict__ cvel_out, float* __restrict__ cdof_dot_out,
                        const int nworld) {
  extern __shared__ __align__(16) float tile_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, w0 = blockIdx.x * 32;
  const int nb6 = T.nbody * 6, nv6 = T.nv * 6, sb = odd(nb6), sv = odd(nv6), sq = odd(T.nv);
  float* cvel_t = tile_smem;
  float* dof_t = cvel_t + 32 * sb;
  float* dot_t = dof_t + 32 * sv;
  float* qv_t = dot_t + 32 * sv;
  rows_in(dof_t, sv, cdof, nv6, nv6, w0, nworld);
  rows_in(qv_t, sq, qvel, qvel_ld, T.nv, w0, nworld);
  __syncthreads();
  float* cvel = cvel_t + lane * sb;
  const float* dof = dof_t + lane * sv;
  float* dot = dot_t + lane * sv;
  const float* qv = qv_t + lane * sq;
#pragma unroll 1
  for (int level = 0; level < T.nlevels; ++level) {
    const int end = T.level_offsets[level + 1];
#pragma unroll 1
    for (int pos = T.level_offsets[level] + warp; pos < end; pos += kTileWarps) {
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
    __syncthreads();
  }
  rows_out(cvel_out, nb6, cvel_t, sb, nb6, w0, nworld);
  rows_out(cdof_dot_out, nv6, dot_t, sv, nv6, w0, nworld);
}

}  // namespace imn
