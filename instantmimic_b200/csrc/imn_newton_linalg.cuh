// imn_newton_linalg.cuh -- per-world linear algebra of the fused Newton kernel,
// executed by one warp on shared-memory operands.  Every function is called from
// exactly one place in the kernel so that the machine code stays small (the
// kernel is bound by instruction fetch and latency, not by arithmetic).
#pragma once

#include <stdio.h>

#include "imn_newton_dev.cuh"
#include "imn_sparse.cuh"

namespace imn {

// Shared-memory view of one world plus the per-world constants.
struct World {
  int nv, ldj, ldu, bd, nefc, ne, nef, lane, nM;
  float *Jsm, *A, *qacc, *Ma, *search, *mv, *grad, *qfs, *xsm, *dinv;
  // the world's M stays in global memory: its nM values are read once per iteration by
  // `products` (independent loads, issued together) and once by the Hessian assembly, and
  // the shared memory they would take holds more worlds per SM instead (measured: humanoid
  // 0.792 -> 0.785 ms per 8192 worlds, SNU-like 1.820 -> 1.736 ms per 4096)
  const float* M;
  float *Jaref, *jv, *Dsm, *floss, *force;
  // row states and the two row lists are 16-bit (njmax < 65536): shared memory per
  // world decides how many worlds an SM holds
  uint16_t *state, *ids, *frows;
  int* uni;
  const float* Jg;    // this world's J in global memory
  const float *Jbeg, *Jend;  // first element and one past the last row of the whole J array
  // streamed J: the copy barrier of the row tile, the parity of its next phase and the
  // flag a timed-out copy raises (all in shared memory); wait limit in polls and the
  // failure-path test switch that withholds the copies
  void* jbar;
  int* jphase;
  int* jfail;
  int wait_polls, withhold_copies;
  const int* mulm_rowadr;
  const uint32_t* mulm_pack;
  // sparse plan only: packed H, N = L D with the carried row, 1/D, the world's
  // violation counter in global memory, the world index (for messages)
  float *Hp, *N, *iD, *viol;
  int world;
#ifdef IMN_PROFILE
  long long* prof_acc;
  long long* prof_t;
#endif
};

#ifdef IMN_PROFILE
#define IMN_MARK(s, k) do { const long long t_ = clock64(); (s).prof_acc[k] += t_ - *(s).prof_t; *(s).prof_t = t_; } while (0)
#else
#define IMN_MARK(s, k)
#endif

// Rows [base, base+32) of J: resident rows are addressed in place, otherwise they
// are staged through the 32-row tile.
template <bool JRES>
__device__ __forceinline__ const float* j_tile(const World& s, int base) {
  if (JRES) return s.Jsm + base * s.ldj;
  __syncwarp();  // every lane is done with the previous tile
  const int n = min(32, s.nefc - base) * s.ldj;
  const float* src = s.Jg + (size_t)base * s.ldj;
  // One TMA bulk copy on the world's mbarrier; the wait is bounded.  A bulk copy wants
  // 16-byte aligned ends, so the smallest aligned range around the rows is copied (up
  // to three floats of the neighbouring rows on either side, still inside the J
  // array) and the tile starts `head` floats into the buffer.
  const int head = (int)((reinterpret_cast<uintptr_t>(src) & 15) >> 2);
  const uint32_t bytes = (uint32_t)((head + n + 3) & ~3) * 4u;
  // after a copy that timed out the barrier's phase is unknown: the world is lost (the
  // caller checks jfail at the end of the pass) and the rest of the pass uses plain loads
  if (src - head >= s.Jbeg && src - head + (bytes >> 2) <= s.Jend && !*s.jfail) {
    const uint32_t parity = (uint32_t)*s.jphase;
    __syncwarp();
    if (s.lane == 0) {
      mbar_expect_tx(s.jbar, bytes);
      if (!(s.withhold_copies & 2)) bulk_g2s(s.Jsm, src - head, bytes, s.jbar);
      *s.jphase = (int)(parity ^ 1u);
    }
    bool arrived = false;
#pragma unroll 1
    for (int tries = 0; tries < s.wait_polls && !arrived; ++tries) arrived = mbar_try_wait(s.jbar, parity);
    if (!arrived && s.lane == 0) *s.jfail = 1;
    __syncwarp();
    return s.Jsm + head;
  }
#pragma unroll 4
  for (int i = s.lane; i < n; i += 32) s.Jsm[i] = src[i];
  // the next tile may arrive through the async proxy into the same buffer
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  return s.Jsm;
}
template <bool JRES>
__device__ __forceinline__ float j_at(const World& s, int r, int i) {
  return JRES ? s.Jsm[r * s.ldj + i] : s.Jg[(size_t)r * s.ldj + i];
}

// outM = M v over the symmetric rows (newton_fusion.py:171-176) and
// outJ[r] = J[r,:] v (- minus[r]): one running sum per row; above 50 dofs in
// 20-dof partials joined by plain adds (newton_stages.py:157-174).
template <bool JRES>
__device__ __forceinline__ void products(const World& s, const float* v, float* outM, float* outJ,
                                         const float* minus) {
  const int lane = s.lane, nv = s.nv;
#pragma unroll 1
  for (int i = lane; i < nv; i += 32) {
    float acc = 0.0f;
    const int k1 = __ldg(s.mulm_rowadr + i + 1);
#pragma unroll 4
    for (int k = __ldg(s.mulm_rowadr + i); k < k1; ++k) {
      const uint32_t p = __ldg(s.mulm_pack + k);
      acc = fmaf(__ldg(s.M + (p >> 16)), v[p & 0xFFFF], acc);
    }
    outM[i] = acc;
  }
  const int chunk = nv > 50 ? 20 : nv;
#pragma unroll 1
  for (int base = 0; base < s.nefc; base += 32) {
    const float* Jt = j_tile<JRES>(s, base);
    const int r = base + lane;
    if (r < s.nefc) {
      const float* Jr = Jt + lane * s.ldj;
      const float sub = minus ? minus[r] : 0.0f;
      float total = 0.0f;
#pragma unroll 1
      for (int s0 = 0; s0 < nv; s0 += chunk) {
        float p = 0.0f;
        const int e = min(s0 + chunk, nv);
#pragma unroll 4
        for (int i = s0; i < e; ++i) p = fmaf(Jr[i], v[i], p);
        if (s0 == 0)
          total = minus ? p - sub : (nv > 50 ? 0.0f + p : p);
        else
          total = total + p;
      }
      outJ[r] = total;
    }
    if (!JRES) __syncwarp();
  }
}

// grad = Ma - qfrc_smooth - J^T force over the rows with a nonzero force (a zero
// force leaves the running sums unchanged), then grad_dot
// (newton_stages.py:785-795).
template <bool JRES>
__device__ __forceinline__ float full_gradient(const World& s, int nfr) {
  const int lane = s.lane, nv = s.nv;
  float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f;
  const int i0 = lane, i1 = lane + 32, i2 = lane + 64;
  const bool h0 = i0 < nv, h1 = i1 < nv, h2 = i2 < nv;
  int a = 0;
#pragma unroll 1
  for (int base = 0; base < s.nefc; base += 32) {
    const float* Jt = j_tile<JRES>(s, base);
    const int hi = JRES ? s.nefc : base + 32;
#pragma unroll 2
    for (; a < nfr; ++a) {
      const int r = s.frows[a];
      if (r >= hi) break;
      const float f = s.force[r];
      const float* Jr = Jt + (r - base) * s.ldj;
      if (h0) s0 = fmaf(Jr[i0], f, s0);
      if (h1) s1 = fmaf(Jr[i1], f, s1);
      if (h2) s2 = fmaf(Jr[i2], f, s2);
    }
    if (JRES) break;
    __syncwarp();
  }
  if (h0) s.grad[i0] = (s.Ma[i0] - s.qfs[i0]) - s0;
  if (h1) s.grad[i1] = (s.Ma[i1] - s.qfs[i1]) - s1;
  if (h2) s.grad[i2] = (s.Ma[i2] - s.qfs[i2]) - s2;
  __syncwarp();
  return logical_block_sum(nv, s.bd, lane, [&](int i, float acc) { return fmaf(s.grad[i], s.grad[i], acc); });
}

// H = M + J^T diag(D, QUADRATIC rows) J on the upper triangle, every entry summing
// its rows in ascending order.  H[r][c] (r <= c) lives at A[(c+1)*ldu + r].
// The QUADRATIC rows arrive as the ascending list s.ids[0, nq) (built by the row
// update of the initial pass).
template <bool JRES>
__device__ __forceinline__ void assemble_hessian(const World& s, int nq) {
  const int lane = s.lane, nv = s.nv, ldu = s.ldu;
  float* A = s.A;
#pragma unroll 4
  for (int e = lane; e < (nv + 1) * ldu; e += 32) A[e] = 0.0f;
  __syncwarp();
#pragma unroll 1
  for (int i = lane; i < nv; i += 32) {
    // the symmetric row of dof i lists every stored entry (i, c); keep c >= i
    const int k1 = __ldg(s.mulm_rowadr + i + 1);
#pragma unroll 1
    for (int k = __ldg(s.mulm_rowadr + i); k < k1; ++k) {
      const uint32_t p = __ldg(s.mulm_pack + k);
      const int c = p & 0xFFFF;
      if (c >= i) A[(c + 1) * ldu + i] = __ldg(s.M + (p >> 16));
    }
  }
  __syncwarp();
  const int npair = nv * (nv + 1) / 2;
  // six entries per lane at a time: a row's D is read once per six entries and the six
  // running sums overlap; every entry still receives its rows in ascending order
  constexpr int Q = 6;
  int k_lo = 0;
#pragma unroll 1
  for (int base = 0; base < s.nefc && k_lo < nq; base += 32) {
    const float* Jt = j_tile<JRES>(s, base);
    const int row_hi = JRES ? s.nefc : base + 32;
    int k_hi = k_lo;
    while (k_hi < nq && s.ids[k_hi] < row_hi) ++k_hi;
#pragma unroll 1
    for (int e0 = 0; e0 < npair && k_hi > k_lo; e0 += 32 * Q) {
      float acc[Q];
      int ij[Q];
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        const int e = e0 + 32 * q + lane;
        int pi = 0, pj = 0;
        if (e < npair) pair_lookup(e, pi, pj);
        ij[q] = e < npair ? (pi | (pj << 16)) : -1;
        acc[q] = e < npair ? A[(pj + 1) * ldu + pi] : 0.0f;
      }
#pragma unroll 1
      for (int k = k_lo; k < k_hi; ++k) {
        const int r = s.ids[k];
        const float Dr = s.Dsm[r];
        const float* Jr = Jt + (r - base) * s.ldj;
#pragma unroll
        for (int q = 0; q < Q; ++q) {
          const int pi = ij[q] < 0 ? 0 : (ij[q] & 0xFFFF), pj = ij[q] < 0 ? 0 : (ij[q] >> 16);
          acc[q] = fmaf(Jr[pi] * Dr, Jr[pj], acc[q]);
        }
      }
#pragma unroll
      for (int q = 0; q < Q; ++q)
        if (ij[q] >= 0) A[((ij[q] >> 16) + 1) * ldu + (ij[q] & 0xFFFF)] = acc[q];
    }
    k_lo = k_hi;
    if (JRES) break;
    __syncwarp();
  }
  __syncwarp();
}

// Rows whose QUADRATIC membership flipped -> dofs they touch (ascending), then
// the pair update of H in the listed row order (newton_stages.py:651-701).
// With a sparse plan (SP != nullptr) the entry lands in the packed H through the
// plan's pair table; an entry outside the pattern is dropped and counted
// (sparse_hessian.py:501-527).
template <bool JRES, bool SPARSE>
__device__ __forceinline__ void update_hessian(const World& s, int count, const ImnSparsePlan& SP) {
  const int lane = s.lane, nv = s.nv, ldu = s.ldu;
  int n = 0;
#pragma unroll 1
  for (int base = 0; base < nv; base += 32) {
    const int dof = base + lane;
    bool hit = false;
    if (dof < nv)
#pragma unroll 1
      for (int t = 0; t < count && !hit; ++t) hit = j_at<JRES>(s, s.ids[t], dof) != 0.0f;
    const unsigned hm = __ballot_sync(IMN_FULL_MASK, hit);
    if (hit) s.uni[n + __popc(hm & ((1u << lane) - 1u))] = dof;
    n += __popc(hm);
  }
  if (lane == 0) s.uni[nv] = n;
  __syncwarp();
  IMN_MARK(s, 12);
  const int npu = n * (n + 1) / 2;
  // several pairs per lane at a time: the listed rows are walked once per group and the
  // sums overlap their latencies; each sum still takes its rows in list order.  Four,
  // except two in the resident-J kernel with the sparse plan, where the smaller code is
  // worth more (measured: 2 % faster there; 1-3 % slower with the dense factor, 2-8 %
  // slower with streamed J).
  constexpr int Q = (JRES && SPARSE) ? 2 : 4;
#pragma unroll 1
  for (int base = 0; base < npu; base += 32 * Q) {
    int row[Q], col[Q], sl[Q];
    float delta[Q];
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      const bool in = base + 32 * q + lane < npu;
      int pi = 0, pj = 0;
      if (in) pair_lookup(base + 32 * q + lane, pi, pj);
      row[q] = in ? s.uni[pi] : 0, col[q] = in ? s.uni[pj] : 0;
      // looked up ahead of the sum so that the table's latency is hidden behind it
      sl[q] = in ? (SPARSE ? __ldg(SP.pair + row[q] * nv + col[q]) : 0) : -2;
      delta[q] = 0.0f;
    }
#pragma unroll 1
    for (int t = 0; t < count; ++t) {
      const int r = s.ids[t];
      const float Dr = s.state[r] == IMN_STATE_QUADRATIC ? s.Dsm[r] : -s.Dsm[r];
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        const float a = j_at<JRES>(s, r, row[q]), b = j_at<JRES>(s, r, col[q]);
        if (a != 0.0f && b != 0.0f) delta[q] = fmaf(Dr * a, b, delta[q]);
      }
    }
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      if (sl[q] != -2 && delta[q] != 0.0f) {
        if (SPARSE) {
          if (sl[q] >= 0)
            s.Hp[sl[q]] = s.Hp[sl[q]] + delta[q];
          else
            sp_violation(s.viol, s.world, "updates an H entry");
        } else {
          s.A[(col[q] + 1) * ldu + row[q]] = s.A[(col[q] + 1) * ldu + row[q]] + delta[q];
        }
      }
    }
  }
  __syncwarp();
  IMN_MARK(s, 13);
}

// Sparse plan: H = M + J^T diag(D, QUADRATIC rows) J on the pattern slots, each slot
// summing its rows in ascending order; every active row's dof support must lie in
// the pattern (sparse_hessian.py:571-637).  Leaves the packed H in both N and Hp.
// A lane keeps the running sums of ten slots in registers and walks the QUADRATIC
// rows once per ten slots: the row's D is read once, and ten independent sums overlap
// their latencies.  The QUADRATIC rows arrive as the ascending list s.ids[0, nq).
template <bool JRES>
__device__ __forceinline__ void assemble_hessian_sparse(const World& s, int nq, const ImnSparsePlan& SP) {
  const int lane = s.lane, nv = s.nv, nfac = SP.nfac, words = (nv + 31) >> 5;
#pragma unroll 1
  for (int a = 0; a < nq; ++a) {
    const int r = s.ids[a];
    if (s.Dsm[r] == 0.0f) continue;
    unsigned rm[3] = {0u, 0u, 0u};
#pragma unroll
    for (int q = 0; q < 3; ++q)
      if (q < words) {
        const int d = q * 32 + lane;
        rm[q] = __ballot_sync(IMN_FULL_MASK, d < nv && j_at<JRES>(s, r, d) != 0.0f);
      }
    bool bad = false;
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const int d = q * 32 + lane;
      if (q < words && d < nv && ((rm[q] >> lane) & 1u)) {
#pragma unroll
        for (int p = 0; p < 3; ++p)
          if (p < words) bad = bad || (rm[p] & ~__ldg(SP.pmask + d * words + p)) != 0u;
      }
    }
    if (__any_sync(IMN_FULL_MASK, bad) && lane == 0) sp_violation(s.viol, s.world, "has a constraint row");
  }
  __syncwarp();
  constexpr int Q = 10;
#pragma unroll 1
  for (int base = 0; base < nfac; base += 32 * Q) {
    float acc[Q];
    int ab[Q];
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      const int sl = base + 32 * q + lane;
      acc[q] = 0.0f, ab[q] = 0;
      if (sl < nfac) {
        const int e = __ldg(SP.s_m + sl);
        ab[q] = (int)__ldg(SP.s_a + sl) | ((int)__ldg(SP.s_b + sl) << 16);
        acc[q] = e >= 0 ? __ldg(s.M + e) : 0.0f;
      }
    }
    // rows in ascending order; a streamed J passes through its 32-row tile
    int k = 0;
#pragma unroll 1
    for (int row0 = 0; row0 < s.nefc && k < nq; row0 += 32) {
      const float* Jt = j_tile<JRES>(s, row0);
      const int row1 = JRES ? s.nefc : row0 + 32;
#pragma unroll 1
      for (; k < nq; ++k) {
        const int r = s.ids[k];
        if (r >= row1) break;
        const float Dr = s.Dsm[r];
        const float* Jr = Jt + (r - row0) * s.ldj;
#pragma unroll
        for (int q = 0; q < Q; ++q) acc[q] = fmaf(Jr[ab[q] & 0xFFFF] * Dr, Jr[ab[q] >> 16], acc[q]);
      }
      if (JRES) break;
      __syncwarp();
    }
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      const int sl = base + 32 * q + lane;
      if (sl < nfac) s.N[sl] = acc[q], s.Hp[sl] = acc[q];
    }
  }
  __syncwarp();
}

}  // namespace imn
