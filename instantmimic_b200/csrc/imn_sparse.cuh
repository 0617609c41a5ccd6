// imn_sparse.cuh -- numeric phases of the static-pattern sparse L'DL of the Newton
// Hessian, executed by one warp on shared-memory operands.
//
// The reference generates these bodies per model with the index tables baked in
// (sparse_hessian.py:410-480 level factor and backward solve, :528-544 forward
// solve, :571-637 initial assembly, :501-527 incremental update).  Here the tables
// are device arrays (ImnSparsePlan) and the code is generic.  Entries hold N = L D;
// slots are row-major, so an entry's terms are runs of contiguous slots; a level is
// one parallel sweep; levels with few long entries split each entry over a team of
// T lanes joined by a shuffle-down tree of width T.  Every entry sums its terms in
// a fixed order, so results do not depend on scheduling.
#pragma once

#include "imn_common.cuh"

namespace imn {

// N[rhs + j] = grad[dof of elimination index j]
__device__ __forceinline__ void sp_load_rhs(const ImnSparsePlan& P, float* N, const float* grad, int lane) {
#pragma unroll 1
  for (int j = lane; j < P.nv; j += 32) N[P.nfac + j] = grad[__ldg(P.orig + j)];
  __syncwarp();
}

// Left-looking numeric factor over elimination-tree levels; the right-hand side
// rides as the augmented last row (forward solve).
__device__ __forceinline__ void sp_factor_levels(const ImnSparsePlan& P, float* N, float* iD, int lane) {
#pragma unroll 1
  for (int l = 0; l < P.nlevels; ++l) {
    const int e0 = __ldg(P.lvl_ptr + l), e1 = __ldg(P.lvl_ptr + l + 1);
    const int T = __ldg(P.lvl_team + l);
    const int tl = lane & (T - 1), team = lane / T, per = 32 / T;
#pragma unroll 1
    for (int eb = e0; eb < e1; eb += per) {
      const int e = eb + team;
      float v = 0.0f;
      int sl = 0, col = -1;
      if (e < e1) {
        sl = __ldg(P.ent_slot + e);
        col = __ldg(P.ent_col + e);
        const int r1 = __ldg(P.run_ptr + e + 1);
#pragma unroll 1
        for (int r = __ldg(P.run_ptr + e); r < r1; ++r) {
          const uint32_t ab = __ldg(P.run_ab + r), kl = __ldg(P.run_kl + r);
          const float* pa = N + (ab & 0xFFFFu);
          const float* pb = N + (ab >> 16);
          const float* pd = iD + (kl & 0xFFFFu);
          const int len = (int)(kl >> 16);
#pragma unroll 2
          for (int t = tl; t < len; t += T) v = fmaf(pa[t] * pb[t], pd[t], v);
        }
      }
#pragma unroll 1
      for (int off = T >> 1; off > 0; off >>= 1) v = v + __shfl_down_sync(IMN_FULL_MASK, v, off, T);
      if (e < e1 && tl == 0) {
        const float w = N[sl] - v;
        N[sl] = w;
        if (col >= 0) iD[col] = 1.0f / w;
      }
    }
    __syncwarp();
  }
}

// The same factorisation driven by the per-(sweep, lane) records (ImnSparsePlan::
// fsweep): one 128-bit load gives a lane its entry, the entry's first run and the
// sweep's team width, and the next sweep's record is fetched while the current one is
// worked on, so no table load sits on the dependent path.  The term loop is kept
// rolled: taking terms in groups of four or two (loads first) was measured 2-4 % slower
// on the whole kernel, which is bound by instruction fetch.
__device__ __forceinline__ float sp_run_terms(const float* N, const float* iD, uint32_t ab, uint32_t kl, int tl,
                                              int T, float v) {
  const float* pa = N + (ab & 0xFFFFu);
  const float* pb = N + (ab >> 16);
  const float* pd = iD + (kl & 0xFFFFu);
  const int len = (int)(kl >> 16);
  int t = tl;
#pragma unroll 1
  for (; t < len; t += T) v = fmaf(pa[t] * pb[t], pd[t], v);
  return v;
}

__device__ __forceinline__ void sp_factor_sweeps(const ImnSparsePlan& P, float* N, float* iD, int lane) {
  const uint4* tab = reinterpret_cast<const uint4*>(P.fsweep) + lane;
  const int ns = P.nfsweep;
  uint4 cur = __ldg(tab);
#pragma unroll 1
  for (int s = 0; s < ns; ++s) {
    const uint4 nxt = __ldg(tab + 32 * min(s + 1, ns - 1));
    const uint32_t fl = cur.w;
    const int T = 1 << ((fl >> 2) & 7), tl = lane & (T - 1);
    const bool has = (fl & 1u) != 0u;
    float v = 0.0f;
    if (has) {
      v = sp_run_terms(N, iD, cur.y, cur.z, tl, T, v);
      const int extra = (fl >> 8) & 0xFF, r0 = fl >> 16;
#pragma unroll 1
      for (int r = r0; r < r0 + extra; ++r) v = sp_run_terms(N, iD, __ldg(P.run_ab + r), __ldg(P.run_kl + r), tl, T, v);
    }
#pragma unroll 1
    for (int off = T >> 1; off > 0; off >>= 1) v = v + __shfl_down_sync(IMN_FULL_MASK, v, off, T);
    if (has && tl == 0) {
      const int sl = cur.x & 0xFFFF, col = (int)(cur.x >> 16) - 1;
      const float w = N[sl] - v;
      N[sl] = w;
      if (col >= 0) iD[col] = 1.0f / w;
    }
    if (fl & 2u) __syncwarp();
    cur = nxt;
  }
}

// Forward solve with a stored factor (rows by level).
__device__ __forceinline__ void sp_forward(const ImnSparsePlan& P, float* N, const float* iD,
                                           const float* grad, int lane) {
  const int rhs = P.nfac;
#pragma unroll 1
  for (int l = 0; l < P.nlevels; ++l) {
    const int q1 = __ldg(P.f_lvl + l + 1);
#pragma unroll 1
    for (int q = __ldg(P.f_lvl + l) + lane; q < q1; q += 32) {
      const int j = __ldg(P.f_row + q);
      float v = grad[__ldg(P.orig + j)];
      const float* rowp = N + __ldg(P.row_start + j);
      const int k0 = __ldg(P.rk_ptr + j), cnt = __ldg(P.rk_ptr + j + 1) - k0;
#pragma unroll 1
      for (int t = 0; t < cnt; ++t) {
        const int k = __ldg(P.rk + k0 + t);
        v = fmaf(-(rowp[t] * iD[k]), N[rhs + k], v);
      }
      N[rhs + j] = v;
    }
    __syncwarp();
  }
}

// Backward solve (levels in reverse, each finished unknown pushes its column terms
// to its descendants), search = -x, and the sums (sum x^2, sum grad x) in the order
// of a block of `bd` threads: strided partials, a tree per warp, warps in order.
__device__ __forceinline__ void sp_backward(const ImnSparsePlan& P, float* N, const float* iD,
                                            const float* grad, float* search, int bd, int lane,
                                            float& sum0, float& sum1) {
  const int rhs = P.nfac, n = P.nv;
#pragma unroll 1
  for (int l = 0; l < P.nlevels; ++l) {
    const int p1 = __ldg(P.b_lvl + l + 1);
#pragma unroll 1
    for (int p = __ldg(P.b_lvl + l) + lane; p < p1; p += 32) {
      const int i = __ldg(P.b_src + p), j = __ldg(P.b_dst + p);
      N[rhs + j] = fmaf(-N[__ldg(P.b_slot + p)], N[rhs + i] * iD[i], N[rhs + j]);
    }
    __syncwarp();
  }
  float ra = 0.0f, rb = 0.0f;
#pragma unroll 1
  for (int w = 0; w < bd / 32; ++w) {
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll 1
    for (int j = lane + 32 * w; j < n; j += bd) {
      const int d = __ldg(P.orig + j);
      const float v = N[rhs + j] * iD[j];
      search[d] = -v;
      s0 = fmaf(v, v, s0);
      s1 = fmaf(grad[d], v, s1);
    }
    ra = ra + warp_tree_sum(s0);
    rb = rb + warp_tree_sum(s1);
  }
  sum0 = ra, sum1 = rb;
  __syncwarp();
}

// sp_backward driven by the per-(sweep, lane) records (ImnSparsePlan::bsweep).
__device__ __forceinline__ void sp_backward_sweeps(const ImnSparsePlan& P, float* N, const float* iD,
                                                   const float* grad, float* search, int bd, int lane,
                                                   float& sum0, float& sum1) {
  const int rhs = P.nfac, n = P.nv, ns = P.nbsweep;
  const uint32_t* tab = P.bsweep + lane;
  uint32_t cur = ns ? __ldg(tab) : 0u;
#pragma unroll 1
  for (int s = 0; s < ns; ++s) {
    const uint32_t nxt = __ldg(tab + 32 * min(s + 1, ns - 1));
    if (cur & (1u << 30)) {
      const int i = (cur >> 16) & 0x7F, j = (cur >> 23) & 0x7F;
      N[rhs + j] = fmaf(-N[cur & 0xFFFFu], N[rhs + i] * iD[i], N[rhs + j]);
    }
    if (cur >> 31) __syncwarp();
    cur = nxt;
  }
  float ra = 0.0f, rb = 0.0f;
#pragma unroll 1
  for (int w = 0; w < bd / 32; ++w) {
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll 1
    for (int j = lane + 32 * w; j < n; j += bd) {
      const int d = __ldg(P.orig + j);
      const float v = N[rhs + j] * iD[j];
      search[d] = -v;
      s0 = fmaf(v, v, s0);
      s1 = fmaf(grad[d], v, s1);
    }
    ra = ra + warp_tree_sum(s0);
    rb = rb + warp_tree_sum(s1);
  }
  sum0 = ra, sum1 = rb;
  __syncwarp();
}

// Count one pattern violation in the world's counter (last element of its hfactor);
// the first one of a world is reported (sparse_hessian.py:521-523, 619-620).
__device__ __forceinline__ void sp_violation(float* counter, int world, const char* what) {
  if (counter && atomicAdd(counter, 1.0f) == 0.0f)
    printf("sparse Hessian: world %d %s outside the declared coupling pattern\n", world, what);
}

}  // namespace imn
