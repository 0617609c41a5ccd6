// imn_newton_dev.cuh -- device helpers of the fused Newton kernel: TMA bulk copy
// and mbarrier wrappers, the piecewise row costs of the line search, and the
// reductions that reproduce the reference's summation orders.
#pragma once

#include "imn_common.cuh"

namespace imn {

// ---- TMA bulk copy + mbarrier (sm_90+ PTX) -----------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(void* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, void* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(void* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// ---- row cost pieces (the statement is in oracle/newton_oracle.c) -------------
__device__ __forceinline__ int row_zone(float x, bool fr, float rf) {
  if (fr) return x <= -rf ? IMN_STATE_LINEARNEG : (x >= rf ? IMN_STATE_LINEARPOS : IMN_STATE_QUADRATIC);
  return x >= 0.0f ? IMN_STATE_SATISFIED : IMN_STATE_QUADRATIC;
}
__device__ __forceinline__ float zone_cost(int z, float x, float D, float f, float rf) {
  if (z == IMN_STATE_QUADRATIC) return ((0.5f * D) * x) * x;
  if (z == IMN_STATE_LINEARNEG) return f * (-0.5f * rf - x);
  if (z == IMN_STATE_LINEARPOS) return f * (-0.5f * rf + x);
  return 0.0f;
}
// One constraint row prepared for repeated evaluation along the search direction.
struct Row {
  float D, ja, j, f, rf, jvD, h, q1r, cost0;
  int z0;  // -1: no row
};
__device__ __forceinline__ Row make_row(bool valid, bool fr, float f, float D, float ja, float j) {
  Row r;
  r.f = fr ? f : 0.0f, r.D = D, r.ja = ja, r.j = j;
  r.rf = fr ? safe_div(f, D) : -1.0f;  // rf < 0 marks an inequality row
  r.z0 = valid ? row_zone(ja, fr, r.rf) : -1;
  r.jvD = j * D;
  r.h = j * r.jvD;
  r.q1r = r.jvD * ja;
  r.cost0 = zone_cost(r.z0, ja, D, r.f, r.rf);
  return r;
}
// (cost(alpha) - cost(0), slope, curvature) at alpha; with `absolute` the first
// component is the cost itself (used at alpha = 0 only).
__device__ __forceinline__ Vec3 row_at(const Row& r, float alpha, bool absolute) {
  if (r.z0 < 0) return v3(0.0f, 0.0f, 0.0f);
  const float x = fmaf(alpha, r.j, r.ja);
  Vec3 o = v3(0.0f, 0.0f, 0.0f);
  int z;
  if (r.rf < 0.0f) {
    z = x < 0.0f ? IMN_STATE_QUADRATIC : IMN_STATE_SATISFIED;
  } else {
    z = row_zone(x, true, r.rf);
    if (z == IMN_STATE_LINEARNEG) o.c1 = -r.f * r.j;
    if (z == IMN_STATE_LINEARPOS) o.c1 = r.f * r.j;
  }
  if (z == IMN_STATE_QUADRATIC) o.c1 = r.jvD * x, o.c2 = r.h;
  if (absolute)
    o.c0 = r.cost0;
  else if (z != r.z0)
    o.c0 = zone_cost(z, x, r.D, r.f, r.rf) - r.cost0;
  else if (z == IMN_STATE_QUADRATIC)
    o.c0 = alpha * fmaf(0.5f * alpha, r.h, r.q1r);
  else if (z == IMN_STATE_LINEARNEG)
    o.c0 = -r.f * (alpha * r.j);
  else if (z == IMN_STATE_LINEARPOS)
    o.c0 = r.f * (alpha * r.j);
  return o;
}
// The same for a plain inequality row (limit or pyramidal contact edge): cost
// 0.5 D x^2 while x < 0, else nothing.  Branch-free; identical values to row_at.
__device__ __forceinline__ Row make_row_ineq(bool valid, float D, float ja, float j) {
  Row r;
  r.f = 0.0f, r.D = D, r.ja = ja, r.j = j, r.rf = -1.0f;
  r.z0 = valid ? (ja >= 0.0f ? IMN_STATE_SATISFIED : IMN_STATE_QUADRATIC) : -1;
  r.jvD = j * D;
  r.h = j * r.jvD;
  r.q1r = r.jvD * ja;
  r.cost0 = r.z0 == IMN_STATE_QUADRATIC ? ((0.5f * D) * ja) * ja : 0.0f;
  return r;
}
__device__ __forceinline__ Vec3 row_at_ineq(const Row& r, float alpha, bool absolute) {
  const float x = fmaf(alpha, r.j, r.ja);
  const bool valid = r.z0 >= 0, on = valid && x < 0.0f, on0 = r.z0 == IMN_STATE_QUADRATIC;
  const float cx = on ? ((0.5f * r.D) * x) * x : 0.0f;
  float c0 = on == on0 ? (on ? alpha * fmaf(0.5f * alpha, r.h, r.q1r) : 0.0f) : cx - r.cost0;
  if (absolute) c0 = r.cost0;
  if (!valid) c0 = 0.0f;
  return v3(c0, on ? r.jvD * x : 0.0f, on ? r.h : 0.0f);
}
__device__ __forceinline__ Vec3 eval_quad(float q1, float q2, float alpha) {
  return v3(fmaf(alpha, q1, (alpha * alpha) * q2) + 0.0f, fmaf(2.0f * alpha, q2, q1), 2.0f * q2);
}
__device__ __forceinline__ bool in_bracket(Vec3 x, Vec3 y) {
  return (x.c1 < y.c1 && y.c1 < 0.0f) || (x.c1 > y.c1 && y.c1 > 0.0f);
}
__device__ __forceinline__ void eval_constraint(bool is_eq, bool is_fr, float jaref, float D,
                                                float floss, float& force, int& state) {
  force = -D * jaref, state = IMN_STATE_QUADRATIC;
  if (is_eq) return;
  if (is_fr) {
    const float rf = safe_div(floss, D);
    if (jaref <= -rf)
      force = floss, state = IMN_STATE_LINEARNEG;
    else if (jaref >= rf)
      force = -floss, state = IMN_STATE_LINEARPOS;
    return;
  }
  if (jaref >= 0.0f) force = 0.0f, state = IMN_STATE_SATISFIED;
}

// One value per thread of the reference's logical block (32 or 64 threads),
// each thread summing its strided elements, then Warp's block reduction: a tree
// per warp and the later warp added to the first (newton_stages.py:34-38).  The
// physical warp plays both logical warps when bd == 64.
template <class F>
__device__ __forceinline__ float logical_block_sum(int n, int bd, int lane, F term) {
  float a = 0.0f;
#pragma unroll 1
  for (int i = lane; i < n; i += bd) a = term(i, a);
  float s = warp_tree_sum(a);
  if (bd == 64) {
    float b = 0.0f;
#pragma unroll 1
    for (int i = lane + 32; i < n; i += 64) b = term(i, b);
    s = s + warp_tree_sum(b);
  }
  return s;
}

// Shuffle-down trees of N values at once (independent chains interleave), lane 0
// broadcast, then "+0" per later logical warp of the line search
// (newton_stages.py:39-49).
template <int N>
__device__ __forceinline__ void ls_sum(float (&v)[N], int bd) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = v[k] + __shfl_down_sync(IMN_FULL_MASK, v[k], off);
  }
#pragma unroll
  for (int k = 0; k < N; ++k) {
    v[k] = __shfl_sync(IMN_FULL_MASK, v[k], 0);
    if (bd == 64) v[k] = v[k] + 0.0f;
  }
}

// advance an upper-triangle pair (i <= j), enumerated column by column, by `step`
__device__ __forceinline__ void pair_advance(int& i, int& j, int step) {
  i += step;
  while (i > j) i -= j + 1, ++j;
}

// The same enumeration as a table: entry e holds i | j << 8 of the e-th pair (i <= j),
// for every pair of up to 80 indices.  One coalesced load replaces the stepping loop.
struct PairTable {
  uint16_t v[80 * 81 / 2];
  constexpr PairTable() : v() {
    int e = 0;
    for (int j = 0; j < 80; ++j)
      for (int i = 0; i <= j; ++i) v[e++] = (uint16_t)(i | (j << 8));
  }
};
__device__ const PairTable g_pairs = PairTable();
__device__ __forceinline__ void pair_lookup(int e, int& i, int& j) {
  const int p = g_pairs.v[e];
  i = p & 0xFF, j = p >> 8;
}

}  // namespace imn
