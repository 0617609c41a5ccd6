// imn_newton.cu -- the fused Newton constraint solve, one warp per world.
//
// One launch replaces the reference's whole solve pipeline
// (mjw_step_optimized.py:2588-2680): _solve_init_dof, the init of
// newton_fusion.py:431-472 (Jaref, Ma = M qacc, constraint update, gradient,
// Hessian, factor, first search direction), the persistent iteration loop of
// newton_fusion.py:170-296 and the final qfrc_constraint_from_grad.
//
// B200 mapping.  The solve is latency-bound small dense algebra (nv <= 79), not a
// tensor-core contraction, so the design goal is to touch HBM exactly once: a CTA
// is one warp that owns one world.  Its J, M and row data arrive in shared memory
// through TMA bulk copies (cp.async.bulk, one mbarrier), the Hessian, its
// Cholesky factor and every vector stay on chip for all iterations, and the
// results are written once.  A warp needs no block barrier (only __syncwarp),
// lane reductions are shuffle trees, and the hardware CTA scheduler balances
// worlds whose iteration counts differ.  Worlds with more rows than fit on chip
// stream J through a 32-row staging tile.
//
// Arithmetic contract.  Every value that decides an active set or an iteration
// count is formed by the same float32 operations in the same order as the CPU
// oracle used by the tests: explicit fmaf chains in ascending index order,
// shuffle-down trees for lane sums, IEEE sqrt and division.  Blocking, register
// tiling and the lane mapping never change the order in which one value
// receives its terms.
#include <stdio.h>

#include "imn_common.cuh"

namespace imn {

// Phase timers, compiled only into the profiling build (-DIMN_PROFILE).
#ifdef IMN_PROFILE
__device__ unsigned long long g_prof[16];
#define PROF_DECL long long prof_t = clock64(); long long prof_acc[12] = {0}
#define PROF(k) do { const long long t_ = clock64(); prof_acc[k] += t_ - prof_t; prof_t = t_; } while (0)
#define PROF_FLUSH do { if (lane == 0) for (int k_ = 0; k_ < 12; ++k_) atomicAdd(&g_prof[k_], (unsigned long long)prof_acc[k_]); } while (0)
#else
#define PROF_DECL
#define PROF(k)
#define PROF_FLUSH
#endif

// Internal error bit OR-ed into `overflow` when the input copies of a world do not
// complete within the wait limit (the world is left unsolved).
#define IMN_OVERFLOW_COPY_TIMEOUT (1 << 30)

struct Geom {
  int nv, njmax, ldj, ldu, nM, bd;
  int jrows;  // rows of J held in shared memory (njmax when resident, else 32)
  // offsets in 4-byte words; every region starts on a 16-byte boundary
  int oBar, oJ, oA, oVec, nv4, oM, oRowF, oRowI, r4, oUni, total;
};

static inline int up4(int n) { return (n + 3) & ~3; }

static Geom make_geom(const ImnModel& m, const ImnData& d, bool resident) {
  Geom g;
  g.nv = m.nv;
  g.njmax = d.njmax;
  g.ldj = (int)d.J_ld_row;
  g.ldu = up4(m.nv + 1);
  g.nM = m.nM;
  g.bd = m.nv_pad >= 64 ? 64 : 32;
  g.jrows = resident ? d.njmax : 32;
  g.nv4 = up4(m.nv);
  g.r4 = up4(d.njmax);
  int o = 0;
  g.oBar = o, o += 4;
  g.oJ = o, o += up4(g.jrows * g.ldj);
  g.oA = o, o += (m.nv + 1) * g.ldu;
  g.oVec = o, o += 8 * g.nv4;
  g.oM = o, o += up4(m.nM);
  g.oRowF = o, o += 5 * g.r4;
  g.oRowI = o, o += 3 * g.r4;
  g.oUni = o, o += up4(m.nv + 1);
  g.total = o;
  return g;
}

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
  int z0;
  bool fr, valid;
};
__device__ __forceinline__ Row make_row(bool valid, bool fr, float f, float D, float ja, float j) {
  Row r;
  r.valid = valid, r.fr = fr, r.f = fr ? f : 0.0f, r.D = D, r.ja = ja, r.j = j;
  r.rf = fr ? safe_div(f, D) : 0.0f;
  r.z0 = row_zone(ja, fr, r.rf);
  r.jvD = j * D;
  r.h = j * r.jvD;
  r.q1r = r.jvD * ja;
  r.cost0 = zone_cost(r.z0, ja, D, r.f, r.rf);
  return r;
}
// (cost, slope, curvature) at alpha = 0
__device__ __forceinline__ Vec3 row_at_zero(const Row& r) {
  if (!r.valid) return v3(0.0f, 0.0f, 0.0f);
  if (r.z0 == IMN_STATE_QUADRATIC) return v3(r.cost0, r.q1r, r.h);
  if (r.z0 == IMN_STATE_LINEARNEG) return v3(r.cost0, -r.f * r.j, 0.0f);
  if (r.z0 == IMN_STATE_LINEARPOS) return v3(r.cost0, r.f * r.j, 0.0f);
  return v3(0.0f, 0.0f, 0.0f);
}
// (cost(alpha) - cost(0), slope, curvature) at alpha
__device__ __forceinline__ Vec3 row_at(const Row& r, float alpha) {
  if (!r.valid) return v3(0.0f, 0.0f, 0.0f);
  const float x = fmaf(alpha, r.j, r.ja);
  if (!r.fr) {
    const bool on = x < 0.0f, on0 = r.z0 == IMN_STATE_QUADRATIC;
    float c = 0.0f;
    if (on && on0)
      c = alpha * fmaf(0.5f * alpha, r.h, r.q1r);
    else if (on != on0)
      c = (on ? ((0.5f * r.D) * x) * x : 0.0f) - r.cost0;
    return v3(c, on ? r.jvD * x : 0.0f, on ? r.h : 0.0f);
  }
  const int z = row_zone(x, true, r.rf);
  Vec3 o = v3(0.0f, 0.0f, 0.0f);
  if (z == IMN_STATE_QUADRATIC) o.c1 = r.jvD * x, o.c2 = r.h;
  if (z == IMN_STATE_LINEARNEG) o.c1 = -r.f * r.j;
  if (z == IMN_STATE_LINEARPOS) o.c1 = r.f * r.j;
  if (z != r.z0)
    o.c0 = zone_cost(z, x, r.D, r.f, r.rf) - r.cost0;
  else if (z == IMN_STATE_QUADRATIC)
    o.c0 = alpha * fmaf(0.5f * alpha, r.h, r.q1r);
  else if (z == IMN_STATE_LINEARNEG)
    o.c0 = -r.f * (alpha * r.j);
  else
    o.c0 = r.f * (alpha * r.j);
  return o;
}
__device__ __forceinline__ Vec3 eval_quad(float q1, float q2, float alpha) {
  return v3(fmaf(alpha, q1, (alpha * alpha) * q2) + 0.0f, fmaf(2.0f * alpha, q2, q1), 2.0f * q2);
}
__device__ __forceinline__ bool in_bracket(Vec3 x, Vec3 y) {
  return (x.c1 < y.c1 && y.c1 < 0.0f) || (x.c1 > y.c1 && y.c1 > 0.0f);
}
__device__ __forceinline__ void eval_constraint(bool is_eq, bool is_fr, float jaref, float D,
                                                float floss, float& force, int& state) {
  if (is_eq) {
    force = -D * jaref, state = IMN_STATE_QUADRATIC;
    return;
  }
  if (is_fr) {
    const float rf = safe_div(floss, D);
    if (jaref <= -rf) {
      force = floss, state = IMN_STATE_LINEARNEG;
      return;
    }
    if (jaref >= rf) {
      force = -floss, state = IMN_STATE_LINEARPOS;
      return;
    }
    force = -D * jaref, state = IMN_STATE_QUADRATIC;
    return;
  }
  if (jaref >= 0.0f) {
    force = 0.0f, state = IMN_STATE_SATISFIED;
    return;
  }
  force = -D * jaref, state = IMN_STATE_QUADRATIC;
}

// One value per thread of the reference's logical block (32 or 64 threads),
// each thread summing its strided elements, then Warp's block reduction: a tree
// per warp and the later warp added to the first (newton_stages.py:34-38).  The
// physical warp plays both logical warps when bd == 64.
template <class F>
__device__ __forceinline__ float logical_block_sum(int n, int bd, int lane, F term) {
  float a = 0.0f;
  for (int i = lane; i < n; i += bd) a = term(i, a);
  float s = warp_tree_sum(a);
  if (bd == 64) {
    float b = 0.0f;
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

template <bool JRES>
__global__ void __launch_bounds__(32) newton_kernel(const ImnModel m, const ImnData d, const ImnCtx cx,
                                                    const Geom g) {
  extern __shared__ __align__(16) float smem[];
  const int lane = threadIdx.x;
  const int w = blockIdx.x;
  const int nv = g.nv, ldj = g.ldj, ldu = g.ldu, bd = g.bd, R = g.njmax, nv4 = g.nv4, r4 = g.r4;

  void* bar = smem + g.oBar;
  float* Jsm = smem + g.oJ;
  // A is (nv+1) x ldu.  U[r][c] (r <= c <= nv; column nv carries the right-hand
  // side) lives at A[r*ldu + c]; H[r][c] (r <= c < nv) at A[(c+1)*ldu + r].
  float* A = smem + g.oA;
  float* qacc = smem + g.oVec;
  float* Ma = qacc + nv4;
  float* search = Ma + nv4;
  float* mv = search + nv4;
  float* grad = mv + nv4;
  float* qfs = grad + nv4;
  float* xsm = qfs + nv4;
  float* dinv = xsm + nv4;
  float* Msm = smem + g.oM;
  float* Jaref = smem + g.oRowF;
  float* jv = Jaref + r4;
  float* Dsm = jv + r4;
  float* floss = Dsm + r4;
  float* force = floss + r4;
  int* state = reinterpret_cast<int*>(smem + g.oRowI);
  int* ids = state + r4;
  int* frows = ids + r4;  // rows with a nonzero force, ascending
  int* uni = reinterpret_cast<int*>(smem + g.oUni);

  PROF_DECL;
  const int nefc_in = d.nefc[w];
  const int nefc = min(R, nefc_in);
  const int ne = d.ne[w], nf = d.nf[w], nef = ne + nf;
  const bool rowless = nefc_in == 0;
  const size_t dofo = (size_t)w * d.dof_ld, efco = (size_t)w * d.efc_ld;
  const float* Jg = d.efc_J + (size_t)w * d.J_ld_world;

  // ---- load: TMA bulk copies for the 16-byte-aligned bulk of every array, plain
  // loads for the ragged ends -----------------------------------------------------
  {
    const float* q0 = (m.warmstart && !rowless) ? d.qacc_warmstart : d.qacc_smooth;
    struct Src {
      float* dst;
      const float* src;
      int n;
    };
    const Src srcs[7] = {
        {Jsm, Jg, JRES ? nefc * ldj : 0},
        {Msm, d.M + (size_t)w * d.M_ld, g.nM},
        {Dsm, d.efc_D + efco, nefc},
        {floss, d.efc_frictionloss + efco, nefc},
        {jv, d.efc_aref + efco, nefc},  // aref is parked in jv until Jaref is formed
        {qacc, q0 + dofo, nv},
        {qfs, d.qfrc_smooth + dofo, nv},
    };
    if (lane == 0) mbar_init(bar, 1);
    __syncwarp();
    uint32_t tx = 0;
#pragma unroll
    for (int k = 0; k < 7; ++k)
      if ((reinterpret_cast<uintptr_t>(srcs[k].src) & 15) == 0) tx += (uint32_t)(srcs[k].n & ~3) * 4u;
    if (lane == 0) {
      mbar_expect_tx(bar, tx);
#pragma unroll
      for (int k = 0; k < 7; ++k) {
        const uint32_t bytes =
            (reinterpret_cast<uintptr_t>(srcs[k].src) & 15) == 0 ? (uint32_t)(srcs[k].n & ~3) * 4u : 0u;
        if (bytes) bulk_g2s(srcs[k].dst, srcs[k].src, bytes, bar);
      }
    }
#pragma unroll
    for (int k = 0; k < 7; ++k) {
      const int done_n = (reinterpret_cast<uintptr_t>(srcs[k].src) & 15) == 0 ? (srcs[k].n & ~3) : 0;
      for (int i = done_n + lane; i < srcs[k].n; i += 32) srcs[k].dst[i] = srcs[k].src[i];
    }
    for (int i = lane; i < nv; i += 32) search[i] = 0.0f, mv[i] = 0.0f, grad[i] = 0.0f;
    for (int i = lane; i <= nv; i += 32) uni[i] = 0;
    // bounded wait for the copies
    bool arrived = false;
    for (int tries = 0; tries < (1 << 22) && !arrived; ++tries) arrived = mbar_try_wait(bar, 0);
    if (!arrived) {
      if (lane == 0) d.overflow[w] |= IMN_OVERFLOW_COPY_TIMEOUT;
      return;
    }
  }
  __syncwarp();
  PROF(0);

  // stage rows [base, base+32) of J when it is not resident
  auto tile = [&](int base) -> const float* {
    if (JRES) return Jsm + base * ldj;
    __syncwarp();
    const int n = min(32, nefc - base) * ldj;
    const float* src = Jg + (size_t)base * ldj;
    for (int i = lane; i < n; i += 32) Jsm[i] = src[i];
    __syncwarp();
    return Jsm;
  };
  auto Jat = [&](int r, int i) -> float { return JRES ? Jsm[r * ldj + i] : Jg[(size_t)r * ldj + i]; };
  // out = M v over the symmetric rows (newton_fusion.py:171-176)
  auto mul_m = [&](const float* v, float* out) {
    for (int i = lane; i < nv; i += 32) {
      float s = 0.0f;
      const int k1 = __ldg(m.M_mulm_rowadr + i + 1);
      int k = __ldg(m.M_mulm_rowadr + i);
      for (; k + 4 <= k1; k += 4) {
        const uint32_t p0 = __ldg(m.M_mulm_pack + k), p1 = __ldg(m.M_mulm_pack + k + 1);
        const uint32_t p2 = __ldg(m.M_mulm_pack + k + 2), p3 = __ldg(m.M_mulm_pack + k + 3);
        const float a0 = Msm[p0 >> 16], a1 = Msm[p1 >> 16], a2 = Msm[p2 >> 16], a3 = Msm[p3 >> 16];
        const float b0 = v[p0 & 0xFFFF], b1 = v[p1 & 0xFFFF], b2 = v[p2 & 0xFFFF], b3 = v[p3 & 0xFFFF];
        s = fmaf(a0, b0, s);
        s = fmaf(a1, b1, s);
        s = fmaf(a2, b2, s);
        s = fmaf(a3, b3, s);
      }
      for (; k < k1; ++k) {
        const uint32_t p = __ldg(m.M_mulm_pack + k);
        s = fmaf(Msm[p >> 16], v[p & 0xFFFF], s);
      }
      out[i] = s;
    }
  };
  // one running sum per row of J v; above 50 dofs in 20-dof partials
  // (newton_stages.py:157-174); `minus` is subtracted from the first partial
  auto row_dots = [&](const float* v, float* out, const float* minus) {
    for (int base = 0; base < nefc; base += 32) {
      const float* Jt = tile(base);
      const int r = base + lane;
      if (r < nefc) {
        const float* Jr = Jt + lane * ldj;
        const float sub = minus ? minus[r] : 0.0f;
        float res;
        if (nv > 50) {
          float total = 0.0f;
          for (int s0 = 0; s0 < nv; s0 += 20) {
            float p = 0.0f;
            const int e = min(s0 + 20, nv);
#pragma unroll 4
            for (int i = s0; i < e; ++i) p = fmaf(Jr[i], v[i], p);
            if (s0 == 0)
              total = minus ? p - sub : 0.0f + p;
            else
              total = total + p;
          }
          res = total;
        } else {
          float p = 0.0f;
#pragma unroll 8
          for (int i = 0; i < nv; ++i) p = fmaf(Jr[i], v[i], p);
          res = minus ? p - sub : p;
        }
        out[r] = res;
      }
      if (!JRES) __syncwarp();
    }
  };
  // grad = Ma - qfrc_smooth - J^T force over the rows with a nonzero force
  // (a zero force leaves the running sums unchanged), then grad_dot
  // (newton_stages.py:785-795)
  auto full_gradient = [&](int nfr) -> float {
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f;
    const int i0 = lane, i1 = lane + 32, i2 = lane + 64;
    const bool h1 = i1 < nv, h2 = i2 < nv;
    if (JRES) {
      int a = 0;
      for (; a + 2 <= nfr; a += 2) {
        const int ra = frows[a], rb = frows[a + 1];
        const float fa = force[ra], fb = force[rb];
        const float* Ja = Jsm + ra * ldj;
        const float* Jb = Jsm + rb * ldj;
        if (i0 < nv) s0 = fmaf(Jb[i0], fb, fmaf(Ja[i0], fa, s0));
        if (h1) s1 = fmaf(Jb[i1], fb, fmaf(Ja[i1], fa, s1));
        if (h2) s2 = fmaf(Jb[i2], fb, fmaf(Ja[i2], fa, s2));
      }
      if (a < nfr) {
        const int ra = frows[a];
        const float fa = force[ra];
        const float* Ja = Jsm + ra * ldj;
        if (i0 < nv) s0 = fmaf(Ja[i0], fa, s0);
        if (h1) s1 = fmaf(Ja[i1], fa, s1);
        if (h2) s2 = fmaf(Ja[i2], fa, s2);
      }
    } else {
      int a = 0;
      for (int base = 0; base < nefc; base += 32) {
        const float* Jt = tile(base);
        for (; a < nfr && frows[a] < base + 32; ++a) {
          const int r = frows[a];
          const float f = force[r];
          const float* Jr = Jt + (r - base) * ldj;
          if (i0 < nv) s0 = fmaf(Jr[i0], f, s0);
          if (h1) s1 = fmaf(Jr[i1], f, s1);
          if (h2) s2 = fmaf(Jr[i2], f, s2);
        }
        __syncwarp();
      }
    }
    if (i0 < nv) grad[i0] = (Ma[i0] - qfs[i0]) - s0;
    if (h1) grad[i1] = (Ma[i1] - qfs[i1]) - s1;
    if (h2) grad[i2] = (Ma[i2] - qfs[i2]) - s2;
    __syncwarp();
    return logical_block_sum(nv, bd, lane, [&](int i, float a) { return fmaf(grad[i], grad[i], a); });
  };

  // Upper Cholesky H = U^T U with the right-hand side as column nv (forward solve),
  // then back substitution (newton_stages.py:546-609).  Left-looking in blocks of
  // 16 rows: a block first takes the updates of all earlier rows (independent
  // running sums, register-tiled four rows at a time), then finishes row by row.
  // Every entry still receives its terms in ascending row order.
  auto factor_solve = [&](bool factor, float& sum0, float& sum1) {
    if (factor) {
      for (int b0 = 0; b0 < nv; b0 += 16) {
        const int b1 = min(b0 + 16, nv);
        // phase 1: terms of rows t < b0
        for (int r0 = b0; r0 < b1; r0 += 4) {
          for (int c = r0 + lane; c <= nv; c += 32) {
            float a0, a1, a2, a3;
            if (c < nv) {
              const float* Hc = A + (c + 1) * ldu;
              a0 = Hc[r0];
              a1 = (r0 + 1 <= c) ? Hc[r0 + 1] : 0.0f;
              a2 = (r0 + 2 <= c) ? Hc[r0 + 2] : 0.0f;
              a3 = (r0 + 3 <= c) ? Hc[r0 + 3] : 0.0f;
            } else {
              a0 = grad[r0];
              a1 = r0 + 1 < nv ? grad[r0 + 1] : 0.0f;
              a2 = r0 + 2 < nv ? grad[r0 + 2] : 0.0f;
              a3 = r0 + 3 < nv ? grad[r0 + 3] : 0.0f;
            }
#pragma unroll 4
            for (int t = 0; t < b0; ++t) {
              const float* Ut = A + t * ldu;
              const float uc = Ut[c];
              const float4 ur = *reinterpret_cast<const float4*>(Ut + r0);  // r0 % 4 == 0
              a0 = fmaf(-ur.x, uc, a0);
              a1 = fmaf(-ur.y, uc, a1);
              a2 = fmaf(-ur.z, uc, a2);
              a3 = fmaf(-ur.w, uc, a3);
            }
            A[r0 * ldu + c] = a0;
            if (r0 + 1 < b1 && r0 + 1 <= c) A[(r0 + 1) * ldu + c] = a1;
            if (r0 + 2 < b1 && r0 + 2 <= c) A[(r0 + 2) * ldu + c] = a2;
            if (r0 + 3 < b1 && r0 + 3 <= c) A[(r0 + 3) * ldu + c] = a3;
          }
        }
        __syncwarp();
        // phase 2: terms of rows b0 <= t < r, pivot, scale
        for (int r = b0; r < b1; ++r) {
          float acc[3];
          float dg = 0.0f;
#pragma unroll
          for (int k = 0; k < 3; ++k) {
            const int c = r + lane + 32 * k;
            if (c <= nv) {
              float a = A[r * ldu + c];
              for (int t = b0; t < r; ++t) a = fmaf(-A[t * ldu + r], A[t * ldu + c], a);
              acc[k] = a;
              if (k == 0 && lane == 0) dg = sqrtf(a);
            }
          }
          dg = __shfl_sync(IMN_FULL_MASK, dg, 0);
          const float rinv = 1.0f / dg;
#pragma unroll
          for (int k = 0; k < 3; ++k) {
            const int c = r + lane + 32 * k;
            if (c <= nv) A[r * ldu + c] = (c == r) ? dg : acc[k] * rinv;
          }
          if (lane == 0) dinv[r] = rinv;
          __syncwarp();
        }
      }
    } else {
      // forward substitution with the stored factor; an unknown receives its
      // terms in ascending order exactly as the factor's carried column does
      float acc[3];
#pragma unroll
      for (int k = 0; k < 3; ++k) acc[k] = (lane + 32 * k) < nv ? grad[lane + 32 * k] : 0.0f;
      for (int t = 0; t < nv; ++t) {
        const int k0 = t >> 5;
        const float mine = k0 == 0 ? acc[0] : (k0 == 1 ? acc[1] : acc[2]);
        float yt = mine * dinv[t];
        yt = __shfl_sync(IMN_FULL_MASK, yt, t & 31);
        if (lane == 0) A[t * ldu + nv] = yt;
        const float* Ut = A + t * ldu;
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          const int r = lane + 32 * k;
          if (r > t && r < nv) acc[k] = fmaf(-Ut[r], yt, acc[k]);
        }
      }
      __syncwarp();
    }
    // back substitution, 16-row blocks from the last: later blocks' columns in
    // ascending order first, then the block's own columns from its last inwards
    for (int b0 = ((nv - 1) / 16) * 16; b0 >= 0; b0 -= 16) {
      const int b1 = min(b0 + 16, nv);
      const int r = b0 + lane;
      const float* Ur = A + r * ldu;
      float acc = 0.0f, di = 0.0f;
      if (r < b1) {
        acc = Ur[nv];
        di = dinv[r];
#pragma unroll 4
        for (int c = b1; c < nv; ++c) acc = fmaf(-Ur[c], xsm[c], acc);
      }
      for (int c = b1 - 1; c >= b0; --c) {
        const float xc = __shfl_sync(IMN_FULL_MASK, acc * di, c - b0);
        if (r < c) acc = fmaf(-Ur[c], xc, acc);
        if (lane == 0) xsm[c] = xc;
      }
      __syncwarp();
    }
    sum0 = logical_block_sum(nv, bd, lane, [&](int i, float a) { return fmaf(xsm[i], xsm[i], a); });
    sum1 = logical_block_sum(nv, bd, lane, [&](int i, float a) { return fmaf(grad[i], xsm[i], a); });
    for (int i = lane; i < nv; i += 32) search[i] = -xsm[i];
    __syncwarp();
  };

  // ---- init ----------------------------------------------------------------
  row_dots(qacc, Jaref, jv);  // Jaref = J qacc - aref (aref parked in jv)
  mul_m(qacc, Ma);
  __syncwarp();

  float search_dot = 0.0f, grad_dot = 0.0f, grad_scale = 1.0f, decrement = 0.0f;
  float improvement = 0.0f, alpha = 0.0f;
  int quad_count = 0, state_count = 0, niter = 0, overflow = 0, nfr = 0;
  bool search_unchanged = false, ls_exhausted = false;

  if (!rowless) {
    // _update_constraint: force / state of every row; rows with a force, ascending
    for (int base = 0; base < nefc; base += 32) {
      const int r = base + lane;
      float f = 0.0f;
      if (r < nefc) {
        const bool is_eq = r < ne, is_fr = !is_eq && r < nef;
        int st;
        eval_constraint(is_eq, is_fr, Jaref[r], Dsm[r], is_fr ? floss[r] : 0.0f, f, st);
        force[r] = f;
        state[r] = st;
        jv[r] = 0.0f;
      }
      const unsigned mask = __ballot_sync(IMN_FULL_MASK, f != 0.0f);
      if (f != 0.0f) frows[nfr + __popc(mask & ((1u << lane) - 1u))] = r;
      nfr += __popc(mask);
    }
    __syncwarp();
    PROF(1);
    grad_dot = full_gradient(nfr);
    PROF(2);
    // H = M + J^T diag(D, QUADRATIC rows) J on the upper triangle, rows ascending
    for (int e = lane; e < (nv + 1) * ldu; e += 32) A[e] = 0.0f;
    __syncwarp();
    for (int i = lane; i < nv; i += 32) {
      // the symmetric row of dof i lists every stored entry (i, c); keep c >= i
      const int k1 = __ldg(m.M_mulm_rowadr + i + 1);
      for (int k = __ldg(m.M_mulm_rowadr + i); k < k1; ++k) {
        const uint32_t p = __ldg(m.M_mulm_pack + k);
        const int c = p & 0xFFFF;
        if (c >= i) A[(c + 1) * ldu + i] = Msm[p >> 16];
      }
    }
    __syncwarp();
    const int npair = nv * (nv + 1) / 2;
    {
      int a_lo = 0;
      for (int base = 0; base < nefc; base += 32) {
        const float* Jt = tile(base);
        const int row_hi = JRES ? nefc : min(base + 32, nefc);
        int a_hi = a_lo;
        while (a_hi < nfr && frows[a_hi] < row_hi) ++a_hi;
        // two entries per lane per pass so that their running sums overlap
        int i0 = lane, j0 = 0, i1 = lane + 32, j1 = 0;
        pair_advance(i0, j0, 0);
        pair_advance(i1, j1, 0);
        for (int e = lane; e < npair; e += 64) {
          const bool two = e + 32 < npair;
          float v0 = A[(j0 + 1) * ldu + i0];
          float v1 = two ? A[(j1 + 1) * ldu + i1] : 0.0f;
          const int i1c = two ? i1 : i0, j1c = two ? j1 : j0;
          for (int a = a_lo; a < a_hi; ++a) {
            const int r = frows[a];
            if (state[r] != IMN_STATE_QUADRATIC) continue;
            const float Dr = Dsm[r];
            const float* Jr = Jt + (r - base) * ldj;
            v0 = fmaf(Jr[i0] * Dr, Jr[j0], v0);
            v1 = fmaf(Jr[i1c] * Dr, Jr[j1c], v1);
          }
          A[(j0 + 1) * ldu + i0] = v0;
          if (two) A[(j1 + 1) * ldu + i1] = v1;
          pair_advance(i0, j0, 64);
          pair_advance(i1, j1, 64);
        }
        a_lo = a_hi;
        if (JRES) break;
        __syncwarp();
      }
    }
    __syncwarp();
    PROF(3);
    factor_solve(true, search_dot, decrement);
    PROF(4);
  }

  // ---- Newton iterations (newton_fusion.py:170-296) -----------------------------
  bool done = rowless;
  const float tolerance = m.opt_tolerance[w % m.n_tolerance];
  const float ls_tolerance = m.opt_ls_tolerance[w % m.n_ls_tolerance];
  const float scale = m.stat_meaninertia[w % m.n_meaninertia] * (float)nv;
  const float eps = m.alpha_noise_eps;
  while (!done) {
    if (!search_unchanged) {
      mul_m(search, mv);
      row_dots(search, jv, nullptr);
    }
    __syncwarp();
    PROF(5);
    // ---- exact line search (newton_stages.py:182-367) ------------------------
    float noise_floor;
    bool ls_converged;
    {
      const float snorm = sqrtf(search_dot);
      const float gtol = fmaxf(tolerance * ls_tolerance * snorm * scale, 1e-06f);
      float gq[2] = {0.0f, 0.0f};
      for (int i = lane; i < nv; i += 32) {
        gq[0] = fmaf(search[i], Ma[i] - qfs[i], gq[0]);
        gq[1] = fmaf(0.5f * search[i], mv[i], gq[1]);
      }
      for (int r = lane; r < ne; r += 32) {
        const float jvD = jv[r] * Dsm[r];
        gq[0] = fmaf(jvD, Jaref[r], gq[0]);
        gq[1] = fmaf(0.5f * jv[r], jvD, gq[1]);
      }
      ls_sum(gq, bd);
      const float q1 = gq[0], q2 = gq[1];
      // the lane's first two rows stay in registers; further rows are re-read
      const int ra = ne + lane, rb = ra + 32;
      const Row rowa = ra < nefc ? make_row(true, ra < nef, floss[ra], Dsm[ra], Jaref[ra], jv[ra])
                                 : make_row(false, false, 0.0f, 1.0f, 0.0f, 0.0f);
      const Row rowb = rb < nefc ? make_row(true, rb < nef, floss[rb], Dsm[rb], Jaref[rb], jv[rb])
                                 : make_row(false, false, 0.0f, 1.0f, 0.0f, 0.0f);
      const bool more = ne + 64 < nefc;
      float p[3];
      {
        Vec3 acc = v3(0.0f, 0.0f, 0.0f) + row_at_zero(rowa);  // running sums start at zero
        acc = acc + row_at_zero(rowb);
        if (more)
          for (int r = rb + 32; r < nefc; r += 32)
            acc = acc + row_at_zero(make_row(true, r < nef, floss[r], Dsm[r], Jaref[r], jv[r]));
        p[0] = acc.c0, p[1] = acc.c1, p[2] = acc.c2;
      }
      ls_sum(p, bd);
      const Vec3 rows = v3(p[0], p[1], p[2]);
      const Vec3 p0 = v3(0.0f, q1, 2.0f * q2) + rows;
      const Vec3 p0_delta = v3(0.0f, p0.c1, p0.c2);
      const float q1_abs = sqrtf(2.0f * fmaxf(rows.c0, 0.0f) * fmaxf(rows.c2, 0.0f)) + fabsf(q1);
      const float gtol_accept = fmaxf(gtol, eps * q1_abs);
      noise_floor = eps * fmaxf(1.0f, safe_div(q1_abs, p0.c2));
      alpha = 0.0f, improvement = 0.0f;
      ls_converged = fabsf(p0.c1) < eps * q1_abs;
      const float lo_alpha_in = -safe_div(p0.c1, p0.c2);
      Vec3 lo_in = v3(0.0f, 0.0f, 0.0f);
      if (!ls_converged) {
        Vec3 acc = v3(0.0f, 0.0f, 0.0f) + row_at(rowa, lo_alpha_in);
        acc = acc + row_at(rowb, lo_alpha_in);
        if (more)
          for (int r = rb + 32; r < nefc; r += 32)
            acc = acc + row_at(make_row(true, r < nef, floss[r], Dsm[r], Jaref[r], jv[r]), lo_alpha_in);
        p[0] = acc.c0, p[1] = acc.c1, p[2] = acc.c2;
        ls_sum(p, bd);
        lo_in = eval_quad(q1, q2, lo_alpha_in) + v3(p[0], p[1], p[2]);
        if (fabsf(lo_in.c1) < gtol_accept && lo_in.c0 < 0.0f) {
          ls_converged = true;
          alpha = lo_alpha_in;
          improvement = -lo_in.c0;
        }
      }
      if (!ls_converged) {
        const bool lo_less = lo_in.c1 < p0.c1;
        Vec3 lo = lo_less ? lo_in : p0_delta;
        float lo_alpha = lo_less ? lo_alpha_in : 0.0f;
        Vec3 hi = lo_less ? p0_delta : lo_in;
        float hi_alpha = lo_less ? 0.0f : lo_alpha_in;
        for (int it = 0; it < m.ls_iterations; ++it) {
          const float a_lo = lo_alpha - safe_div(lo.c1, lo.c2);
          const float a_hi = hi_alpha - safe_div(hi.c1, hi.c2);
          const float a_mid = 0.5f * (lo_alpha + hi_alpha);
          const Vec3 z3 = v3(0.0f, 0.0f, 0.0f);
          Vec3 s_lo = z3 + row_at(rowa, a_lo), s_hi = z3 + row_at(rowa, a_hi), s_mid = z3 + row_at(rowa, a_mid);
          s_lo = s_lo + row_at(rowb, a_lo);
          s_hi = s_hi + row_at(rowb, a_hi);
          s_mid = s_mid + row_at(rowb, a_mid);
          if (more)
            for (int r = rb + 32; r < nefc; r += 32) {
              const Row rr = make_row(true, r < nef, floss[r], Dsm[r], Jaref[r], jv[r]);
              s_lo = s_lo + row_at(rr, a_lo);
              s_hi = s_hi + row_at(rr, a_hi);
              s_mid = s_mid + row_at(rr, a_mid);
            }
          float q[9] = {s_lo.c0, s_lo.c1, s_lo.c2, s_hi.c0, s_hi.c1, s_hi.c2, s_mid.c0, s_mid.c1, s_mid.c2};
          ls_sum(q, bd);
          const Vec3 lo_next = eval_quad(q1, q2, a_lo) + v3(q[0], q[1], q[2]);
          const Vec3 hi_next = eval_quad(q1, q2, a_hi) + v3(q[3], q[4], q[5]);
          const Vec3 mid = eval_quad(q1, q2, a_mid) + v3(q[6], q[7], q[8]);
          const bool conv_lo = fabsf(lo_next.c1) < gtol_accept && lo_next.c0 < 0.0f;
          const bool conv_hi = fabsf(hi_next.c1) < gtol_accept && hi_next.c0 < 0.0f;
          const bool conv_mid = fabsf(mid.c1) < gtol_accept && mid.c0 < 0.0f;
          const bool converged = conv_lo || conv_hi || conv_mid;
          bool swap_lo = false, swap_hi = false;
          if (converged) {
            Vec3 best = v3(IMN_MJ_MAXVAL, 0.0f, 0.0f);
            float best_alpha = 0.0f;
            if (conv_lo && lo_next.c0 < best.c0) best = lo_next, best_alpha = a_lo;
            if (conv_hi && hi_next.c0 < best.c0) best = hi_next, best_alpha = a_hi;
            if (conv_mid && mid.c0 < best.c0) best = mid, best_alpha = a_mid;
            lo = hi = best;
            lo_alpha = hi_alpha = best_alpha;
          } else {
            bool s;
            s = in_bracket(lo, lo_next);
            if (s) lo = lo_next, lo_alpha = a_lo;
            swap_lo |= s;
            s = in_bracket(lo, mid);
            if (s) lo = mid, lo_alpha = a_mid;
            swap_lo |= s;
            s = in_bracket(lo, hi_next);
            if (s) lo = hi_next, lo_alpha = a_hi;
            swap_lo |= s;
            s = in_bracket(hi, hi_next) || (hi.c1 < 0.0f && hi_next.c1 > 0.0f);
            if (s) hi = hi_next, hi_alpha = a_hi;
            swap_hi |= s;
            s = in_bracket(hi, mid);
            if (s) hi = mid, hi_alpha = a_mid;
            swap_hi |= s;
            s = in_bracket(hi, lo_next);
            if (s) hi = lo_next, hi_alpha = a_lo;
            swap_hi |= s;
          }
          const bool ls_done = converged || (!swap_lo && !swap_hi) ||
                               (lo.c0 < 0.0f && lo.c1 < 0.0f && lo.c1 > -gtol) ||
                               (hi.c0 < 0.0f && hi.c1 > 0.0f && hi.c1 < gtol);
          if (lo.c0 < 0.0f || hi.c0 < 0.0f) {
            const bool lo_better = lo.c0 < hi.c0;
            alpha = lo_better ? lo_alpha : hi_alpha;
            improvement = -(lo_better ? lo.c0 : hi.c0);
          }
          if (ls_done) {
            ls_converged = true;
            break;
          }
        }
      }
    }
    PROF(6);
    // ---- move, re-evaluate rows, list QUADRATIC flips (newton_stages.py:373-426)
    for (int i = lane; i < nv; i += 32) {
      qacc[i] = fmaf(alpha, search[i], qacc[i]);
      Ma[i] = fmaf(alpha, mv[i], Ma[i]);
    }
    quad_count = 0;
    state_count = 0;
    nfr = 0;
    for (int base = 0; base < nefc; base += 32) {
      const int r = base + lane;
      bool flip = false, changed = false;
      float f = 0.0f;
      if (r < nefc) {
        const float nj = rounded_step(Jaref[r], alpha, jv[r]);
        Jaref[r] = nj;
        const bool is_eq = r < ne, is_fr = !is_eq && r < nef;
        int ns;
        eval_constraint(is_eq, is_fr, nj, Dsm[r], is_fr ? floss[r] : 0.0f, f, ns);
        const int old = state[r];
        force[r] = f;
        state[r] = ns;
        flip = (old == IMN_STATE_QUADRATIC) != (ns == IMN_STATE_QUADRATIC);
        changed = old != ns;
      }
      const unsigned below = (1u << lane) - 1u;
      const unsigned fm = __ballot_sync(IMN_FULL_MASK, flip);
      if (flip) ids[quad_count + __popc(fm & below)] = r;
      quad_count += __popc(fm);
      state_count += __popc(__ballot_sync(IMN_FULL_MASK, changed));
      const unsigned nz = __ballot_sync(IMN_FULL_MASK, f != 0.0f);
      if (f != 0.0f) frows[nfr + __popc(nz & below)] = r;
      nfr += __popc(nz);
    }
    ls_exhausted = fabsf(alpha) < noise_floor;
    if (ls_exhausted) state_count += 1;
    if (!ls_converged) {
      if ((m.warn_overflow & m.overflow_ls_iterations) && lane == 0)
        printf("linesearch iterations limit reached - please increase ls_iterations to %u\n",
               (unsigned)m.ls_iterations);
      overflow |= m.overflow_ls_iterations;
    }
    __syncwarp();
    PROF(7);
    // ---- gradient (newton_stages.py:745-798) and factor (newton_stages.py:629-740)
    const bool changed = state_count != 0;
    search_unchanged = !changed;
    if (!changed) {
      const float sigma = grad_scale, ns = sigma - alpha;
      const float ratio = sigma != 0.0f ? ns / sigma : 0.0f;
      const float rsq = ratio * ratio;
      grad_dot *= rsq;
      decrement *= rsq;
      grad_scale = ns;
    } else {
      grad_dot = full_gradient(nfr);
      PROF(8);
      decrement = 0.0f;
      grad_scale = 1.0f;
      if (quad_count > 0) {
        // dofs the changed rows touch, ascending (newton_stages.py:657-680)
        int n = 0;
        for (int base = 0; base < nv; base += 32) {
          const int dof = base + lane;
          bool hit = false;
          if (dof < nv)
            for (int t = 0; t < quad_count && !hit; ++t) hit = Jat(ids[t], dof) != 0.0f;
          const unsigned hm = __ballot_sync(IMN_FULL_MASK, hit);
          if (hit) uni[n + __popc(hm & ((1u << lane) - 1u))] = dof;
          n += __popc(hm);
        }
        if (lane == 0) uni[nv] = n;
        __syncwarp();
        const int npu = n * (n + 1) / 2;
        int pi = lane, pj = 0;
        pair_advance(pi, pj, 0);
        for (int e = lane; e < npu; e += 32) {
          const int row = uni[pi], col = uni[pj];
          float delta = 0.0f;
          for (int t = 0; t < quad_count; ++t) {
            const int r = ids[t];
            const float a = Jat(r, row), b = Jat(r, col);
            float da = Dsm[r] * a;
            if (state[r] != IMN_STATE_QUADRATIC) da = -da;
            if (a != 0.0f && b != 0.0f) delta = fmaf(da, b, delta);
          }
          if (delta != 0.0f) A[(col + 1) * ldu + row] = A[(col + 1) * ldu + row] + delta;
          pair_advance(pi, pj, 32);
        }
        __syncwarp();
      }
      PROF(9);
      factor_solve(quad_count > 0, search_dot, decrement);
      PROF(10);
    }
    // ---- convergence (newton_fusion.py:267-295) -------------------------------
    ++niter;
    const bool converged = alpha == 0.0f || (improvement > 0.0f && improvement / scale < tolerance) ||
                           sqrtf(grad_dot) / scale < tolerance ||
                           0.5f * decrement / scale < tolerance;
    if (converged || niter == m.iterations) {
      if (!converged) {
        if ((m.warn_overflow & m.overflow_iterations) && lane == 0)
          printf("solver iterations limit reached - please increase iterations to %u\n",
                 (unsigned)m.iterations);
        overflow |= m.overflow_iterations;
      }
      done = true;
      if (lane == 0 && cx.nsolving) atomicAdd(cx.nsolving, -1);
    }
  }

  // ---- results (once) ---------------------------------------------------------
  for (int i = lane; i < nv; i += 32) {
    d.qacc[dofo + i] = qacc[i];
    d.efc_Ma[dofo + i] = Ma[i];
    d.qfrc_constraint[dofo + i] = rowless ? 0.0f : fmaf(-grad_scale, grad[i], Ma[i] - qfs[i]);
    if (cx.search) cx.search[dofo + i] = search[i];
    if (cx.mv) cx.mv[dofo + i] = mv[i];
    if (cx.grad) cx.grad[(size_t)w * cx.grad_ld + i] = grad[i];
  }
  for (int r = lane; r < nefc; r += 32) {
    d.efc_force[efco + r] = force[r];
    d.efc_state[efco + r] = state[r];
    if (cx.Jaref) cx.Jaref[efco + r] = Jaref[r];
    if (cx.jv) cx.jv[efco + r] = jv[r];
    if (cx.quad_changed_ids && r < quad_count) cx.quad_changed_ids[efco + r] = ids[r];
  }
  if (cx.dof_union && !rowless)
    for (int i = lane; i <= nv; i += 32) cx.dof_union[(size_t)w * (nv + 1) + i] = uni[i];
  if (!rowless) {
    const size_t ho = (size_t)w * m.nv_pad * m.nv_pad;
    if (cx.h)
      for (int r = 0; r < nv; ++r)
        for (int c = r + lane; c < nv; c += 32) cx.h[ho + (size_t)r * m.nv_pad + c] = A[(c + 1) * ldu + r];
    if (cx.hfactor && !cx.sparse_plan)
      for (int r = 0; r < nv; ++r)
        for (int c = r + lane; c < nv; c += 32) cx.hfactor[ho + (size_t)r * m.nv_pad + c] = A[r * ldu + c];
  }
  PROF(11);
  PROF_FLUSH;
  if (lane == 0) {
    d.solver_niter[w] = niter;
    if (overflow) d.overflow[w] |= overflow;
    if (cx.search_dot) cx.search_dot[w] = search_dot;
    if (cx.done) cx.done[w] = 1;
    if (!rowless) {
      if (cx.grad_dot) cx.grad_dot[w] = grad_dot;
      if (cx.grad_scale) cx.grad_scale[w] = grad_scale;
      if (cx.newton_decrement) cx.newton_decrement[w] = decrement;
      if (cx.improvement) cx.improvement[w] = improvement;
      if (cx.alpha) cx.alpha[w] = alpha;
      if (cx.search_unchanged) cx.search_unchanged[w] = search_unchanged;
      if (cx.ls_exhausted) cx.ls_exhausted[w] = ls_exhausted;
      if (cx.quad_changed_count) cx.quad_changed_count[w] = quad_count;
      if (cx.state_changed_count) cx.state_changed_count[w] = state_count;
    }
  }
}

__global__ void fill_nsolving(int* nsolving, int value) { *nsolving = value; }

// Largest dynamic shared memory one CTA may opt into on sm_100 (227 KB).
static const int kMaxSmem = 227 * 1024;
// Resident-J budget per world: keep at least 4 worlds per SM.
static const int kResidentBudget = kMaxSmem / 4;

static int validate(const ImnModel* m, const ImnData* d, const ImnCtx* cx) {
  if (!m || !d || !cx) return set_error("imn_solve: NULL struct"), IMN_ERR_NULL;
  if (d->nworld < 0 || d->njmax < 0) return set_error("imn_solve: negative extent"), IMN_ERR_SHAPE;
  if (m->nv <= 0 || m->nv > 79 || m->nv_pad % 16 != 0 || m->nv_pad > 80 || m->nv_pad <= m->nv)
    return set_error("imn_solve: nv %d / nv_pad %d outside the fused path (0 < nv <= 79, nv_pad %% 16 == 0, nv < nv_pad <= 80)",
                     m->nv, m->nv_pad),
           IMN_ERR_UNSUPPORTED;
  if (m->iterations <= 0) return set_error("imn_solve: iterations must be positive"), IMN_ERR_UNSUPPORTED;
  if (m->n_tolerance <= 0 || m->n_ls_tolerance <= 0 || m->n_meaninertia <= 0)
    return set_error("imn_solve: empty option array"), IMN_ERR_SHAPE;
  const void* need[] = {m->opt_tolerance, m->opt_ls_tolerance, m->stat_meaninertia, m->M_mulm_rowadr,
                        m->M_mulm_pack, d->nefc, d->ne, d->nf, d->qacc_smooth, d->qacc_warmstart,
                        d->qfrc_smooth, d->efc_J, d->efc_D, d->efc_aref, d->efc_frictionloss, d->M, d->qacc,
                        d->qfrc_constraint, d->efc_Ma, d->efc_force, d->efc_state, d->solver_niter,
                        d->overflow};
  for (const void* p : need)
    if (!p) return set_error("imn_solve: a required Model/Data pointer is NULL"), IMN_ERR_NULL;
  if (d->dof_ld < m->nv || d->J_ld_row < m->nv || d->efc_ld < d->njmax || d->M_ld < m->nM ||
      d->J_ld_world < (int64_t)d->njmax * d->J_ld_row)
    return set_error("imn_solve: a stride is smaller than its extent"), IMN_ERR_SHAPE;
  if (d->J_ld_row > 4 * (int64_t)m->nv + 64)
    return set_error("imn_solve: efc.J row stride %lld is far larger than nv %d", (long long)d->J_ld_row, m->nv),
           IMN_ERR_SHAPE;
  if (m->nM >= (1 << 16)) return set_error("imn_solve: nM exceeds 16-bit indices"), IMN_ERR_LIMIT;
  if (cx->grad && cx->grad_ld < m->nv) return set_error("imn_solve: ctx.grad stride < nv"), IMN_ERR_SHAPE;
  if (cx->sparse_plan) return set_error("imn_solve: sparse plan not supported by this kernel"), IMN_ERR_UNSUPPORTED;
  return IMN_OK;
}

static int plan_launch(const ImnModel* m, const ImnData* d, Geom* g, bool* resident) {
  Geom gr = make_geom(*m, *d, true);
  if (gr.total * 4 <= kResidentBudget) {
    *g = gr, *resident = true;
    return IMN_OK;
  }
  Geom gs = make_geom(*m, *d, false);
  if (gs.total * 4 > kMaxSmem)
    return set_error("imn_solve: njmax %d needs %d bytes of shared memory per world (max %d)", d->njmax,
                     gs.total * 4, kMaxSmem),
           IMN_ERR_LIMIT;
  *g = gs, *resident = false;
  return IMN_OK;
}

}  // namespace imn

#ifdef IMN_PROFILE
extern "C" int imn_debug_profile(unsigned long long* out, int reset) {
  cudaMemcpyFromSymbol(out, imn::g_prof, sizeof(unsigned long long) * 16);
  if (reset) {
    unsigned long long z[16] = {0};
    cudaMemcpyToSymbol(imn::g_prof, z, sizeof z);
  }
  return 0;
}
extern "C" int imn_debug_occupancy(int bytes, int resident) {
  int n = 0;
  if (resident)
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, imn::newton_kernel<true>, 32, bytes);
  else
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, imn::newton_kernel<false>, 32, bytes);
  return n;
}
#endif

extern "C" int imn_launch_info(const ImnModel* m, const ImnData* d, const ImnCtx* cx, ImnLaunchInfo* out) {
  if (!out) return imn::set_error("imn_launch_info: NULL out"), IMN_ERR_NULL;
  int rc = imn::validate(m, d, cx);
  if (rc) return rc;
  imn::Geom g;
  bool res;
  rc = imn::plan_launch(m, d, &g, &res);
  if (rc) return rc;
  out->world_threads = g.bd;
  out->worlds_per_cta = 1;
  out->smem_bytes = g.total * 4;
  out->j_resident = res ? 1 : 0;
  out->grid = d->nworld;
  return IMN_OK;
}

extern "C" int imn_solve(const ImnModel* m, const ImnData* d, const ImnCtx* cx, void* stream_) {
  int rc = imn::validate(m, d, cx);
  if (rc) return rc;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (d->nworld == 0) return IMN_OK;
  imn::Geom g;
  bool res;
  rc = imn::plan_launch(m, d, &g, &res);
  if (rc) return rc;
  const int bytes = g.total * 4;
  auto kern = res ? imn::newton_kernel<true> : imn::newton_kernel<false>;
  {
    // many one-warp CTAs share an SM: ask for the largest shared-memory carve-out,
    // otherwise the driver sizes it for a single CTA
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                         cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess && bytes > 48 * 1024)
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess)
      return imn::set_error("imn_solve: cudaFuncSetAttribute: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  }
  if (cx->nsolving) imn::fill_nsolving<<<1, 1, 0, stream>>>(cx->nsolving, d->nworld);
  kern<<<d->nworld, 32, bytes, stream>>>(*m, *d, *cx, g);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return imn::set_error("imn_solve: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}
