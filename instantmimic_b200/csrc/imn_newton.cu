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
// is one warp that owns one world, loads that world's J, M and row data into
// shared memory with coalesced reads, keeps the Hessian, its Cholesky factor and
// every vector on chip for all iterations, and writes the results once.  A warp
// needs no block barrier (only __syncwarp), lane reductions are shuffle trees,
// and the hardware CTA scheduler balances worlds whose iteration counts differ.
// Worlds with more rows than fit on chip stream J through a 32-row staging tile.
//
// Arithmetic contract.  Every value that decides an active set or an iteration
// count is formed by the same float32 operations in the same order as the CPU
// oracle used by the tests: explicit fmaf chains in ascending index order,
// shuffle-down trees for lane sums, IEEE sqrt and division.
#include <stdio.h>

#include "imn_common.cuh"

namespace imn {

struct Geom {
  int nv, njmax, ldj, lda, nM, bd;
  int jrows;  // rows of J held in shared memory (njmax when resident, else 32)
  // offsets in 4-byte words
  int oJ, oA, oVec, oM, oRowF, oRowI, oUni, total;
};

__host__ __device__ inline int odd_up(int n) { return n | 1; }

static Geom make_geom(const ImnModel& m, const ImnData& d, bool resident) {
  Geom g;
  g.nv = m.nv;
  g.njmax = d.njmax;
  g.ldj = odd_up(m.nv);
  g.lda = odd_up(m.nv + 1);
  g.nM = m.nM;
  g.bd = m.nv_pad >= 64 ? 64 : 32;
  g.jrows = resident ? d.njmax : 32;
  int o = 0;
  g.oJ = o, o += g.jrows * g.ldj;
  g.oA = o, o += (m.nv + 1) * g.lda;
  g.oVec = o, o += 8 * m.nv;
  g.oM = o, o += m.nM;
  g.oRowF = o, o += 5 * d.njmax;
  g.oRowI = o, o += 3 * d.njmax;
  g.oUni = o, o += m.nv + 1;
  g.total = o;
  return g;
}

// ---- row cost pieces (see oracle/newton_oracle.c for the statement) ---------
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
__device__ __forceinline__ Vec3 zone_slope(int z, float x, float D, float f, float jv) {
  if (z == IMN_STATE_QUADRATIC) {
    const float jvD = jv * D;
    return v3(0.0f, jvD * x, jv * jvD);
  }
  if (z == IMN_STATE_LINEARNEG) return v3(0.0f, -f * jv, 0.0f);
  if (z == IMN_STATE_LINEARPOS) return v3(0.0f, f * jv, 0.0f);
  return v3(0.0f, 0.0f, 0.0f);
}
__device__ __forceinline__ Vec3 eval_row_zero(bool fr, float f, float D, float jaref, float jv) {
  const float rf = fr ? safe_div(f, D) : 0.0f;
  const int z = row_zone(jaref, fr, rf);
  Vec3 r = zone_slope(z, jaref, D, f, jv);
  r.c0 = zone_cost(z, jaref, D, f, rf);
  return r;
}
__device__ __forceinline__ Vec3 eval_row(bool fr, float f, float alpha, float D, float jaref,
                                         float jv) {
  const float rf = fr ? safe_div(f, D) : 0.0f;
  const float x = fmaf(alpha, jv, jaref);
  const int z0 = row_zone(jaref, fr, rf), z = row_zone(x, fr, rf);
  Vec3 r = zone_slope(z, x, D, f, jv);
  if (z != z0) {
    r.c0 = zone_cost(z, x, D, f, rf) - zone_cost(z0, jaref, D, f, rf);
  } else if (z == IMN_STATE_QUADRATIC) {
    const float jvD = jv * D;
    r.c0 = alpha * fmaf(0.5f * alpha, jv * jvD, jvD * jaref);
  } else if (z == IMN_STATE_LINEARNEG) {
    r.c0 = -f * (alpha * jv);
  } else if (z == IMN_STATE_LINEARPOS) {
    r.c0 = f * (alpha * jv);
  }
  return r;
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

// First-warp reduction of the line search plus "+0" per later logical warp.
__device__ __forceinline__ float ls_sum(float v, int bd) {
  float s = warp_tree_sum(v);
  if (bd == 64) s = s + 0.0f;
  return s;
}
__device__ __forceinline__ Vec3 ls_sum(Vec3 v, int bd) {
  return v3(ls_sum(v.c0, bd), ls_sum(v.c1, bd), ls_sum(v.c2, bd));
}

template <bool JRES>
__global__ void __launch_bounds__(32) newton_kernel(const ImnModel m, const ImnData d, const ImnCtx cx,
                                                    const Geom g) {
  extern __shared__ __align__(16) float smem[];
  const int lane = threadIdx.x;
  const int w = blockIdx.x;
  const int nv = g.nv, ldj = g.ldj, lda = g.lda, bd = g.bd, R = g.njmax;

  float* Jsm = smem + g.oJ;
  float* A = smem + g.oA;  // H[r][c] at A[r*lda+c] (r<=c); U[r][c] at A[(c+1)*lda+r] (r<=c)
  float* qacc = smem + g.oVec;
  float* Ma = qacc + nv;
  float* search = Ma + nv;
  float* mv = search + nv;
  float* grad = mv + nv;
  float* qfs = grad + nv;
  float* ysm = qfs + nv;
  float* xsm = ysm + nv;
  float* Msm = smem + g.oM;
  float* Jaref = smem + g.oRowF;
  float* jv = Jaref + R;
  float* Dsm = jv + R;
  float* floss = Dsm + R;
  float* force = floss + R;
  int* state = reinterpret_cast<int*>(smem + g.oRowI);
  int* ids = state + R;
  int* act = ids + R;
  int* uni = reinterpret_cast<int*>(smem + g.oUni);

  const int nefc_in = d.nefc[w];
  const int nefc = min(R, nefc_in);
  const int ne = d.ne[w], nf = d.nf[w], nef = ne + nf;
  const bool rowless = nefc_in == 0;
  const size_t dofo = (size_t)w * d.dof_ld, efco = (size_t)w * d.efc_ld;
  const float* Jg = d.efc_J + (size_t)w * d.J_ld_world;
  const int ldjg = (int)d.J_ld_row;

  // ---- load (coalesced, once) ------------------------------------------------
  {
    const float* q0 = (m.warmstart && !rowless) ? d.qacc_warmstart : d.qacc_smooth;
    for (int i = lane; i < nv; i += 32) {
      qacc[i] = q0[dofo + i];
      qfs[i] = d.qfrc_smooth[dofo + i];
      search[i] = 0.0f, mv[i] = 0.0f, grad[i] = 0.0f;
    }
    for (int i = lane; i <= nv; i += 32) uni[i] = 0;
    const float* Mg = d.M + (size_t)w * d.M_ld;
    for (int e = lane; e < g.nM; e += 32) Msm[e] = Mg[e];
    for (int r = lane; r < nefc; r += 32) {
      Dsm[r] = d.efc_D[efco + r];
      floss[r] = d.efc_frictionloss[efco + r];
      jv[r] = 0.0f;
    }
    if (JRES) {
      int rr = 0, cc = lane;
      while (cc >= nv) cc -= nv, ++rr;
      while (rr < nefc) {
        Jsm[rr * ldj + cc] = Jg[(size_t)rr * ldjg + cc];
        cc += 32;
        while (cc >= nv) cc -= nv, ++rr;
      }
    }
  }
  __syncwarp();

  // stage rows [base, base+32) of J when it is not resident
  auto tile = [&](int base) -> const float* {
    if (JRES) return Jsm + base * ldj;
    __syncwarp();
    const int rows = min(32, nefc - base);
    int rr = 0, cc = lane;
    while (cc >= nv) cc -= nv, ++rr;
    while (rr < rows) {
      Jsm[rr * ldj + cc] = Jg[(size_t)(base + rr) * ldjg + cc];
      cc += 32;
      while (cc >= nv) cc -= nv, ++rr;
    }
    __syncwarp();
    return Jsm;
  };
  auto Jat = [&](int r, int i) -> float {
    return JRES ? Jsm[r * ldj + i] : Jg[(size_t)r * ldjg + i];
  };
  // out = M v over the symmetric rows (newton_fusion.py:171-176)
  auto mul_m = [&](const float* v, float* out) {
    for (int i = lane; i < nv; i += 32) {
      float s = 0.0f;
      const int k1 = m.M_mulm_rowadr[i + 1];
      for (int k = m.M_mulm_rowadr[i]; k < k1; ++k) s = fmaf(Msm[m.M_mulm_madr[k]], v[m.M_mulm_col[k]], s);
      out[i] = s;
    }
  };
  // one running sum per row of J v; above 50 dofs in 20-dof partials
  // (newton_stages.py:157-174); first_minus is subtracted from the first partial
  auto row_dots = [&](const float* v, float* out, const float* minus) {
    for (int base = 0; base < nefc; base += 32) {
      const float* Jt = tile(base);
      const int r = base + lane;
      if (r < nefc) {
        const float* Jr = Jt + lane * ldj;
        float res;
        if (nv > 50) {
          float total = 0.0f;
          for (int s0 = 0; s0 < nv; s0 += 20) {
            float p = 0.0f;
            const int e = min(s0 + 20, nv);
            for (int i = s0; i < e; ++i) p = fmaf(Jr[i], v[i], p);
            if (s0 == 0)
              total = minus ? p - minus[efco + r] : 0.0f + p;
            else
              total = total + p;
          }
          res = total;
        } else {
          float p = 0.0f;
          for (int i = 0; i < nv; ++i) p = fmaf(Jr[i], v[i], p);
          res = minus ? p - minus[efco + r] : p;
        }
        out[r] = res;
      }
    }
  };
  // grad = Ma - qfrc_smooth - J^T force, grad_dot (newton_stages.py:785-795)
  auto full_gradient = [&]() -> float {
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f;
    const int i0 = lane, i1 = lane + 32, i2 = lane + 64;
    for (int base = 0; base < nefc; base += 32) {
      const float* Jt = tile(base);
      const int rows = JRES ? nefc : min(32, nefc - base);
      for (int rr = 0; rr < rows; ++rr) {
        const float f = force[base + rr];
        if (f != 0.0f) {
          const float* Jr = Jt + rr * ldj;
          if (i0 < nv) s0 = fmaf(Jr[i0], f, s0);
          if (i1 < nv) s1 = fmaf(Jr[i1], f, s1);
          if (i2 < nv) s2 = fmaf(Jr[i2], f, s2);
        }
      }
      if (JRES) break;
    }
    if (i0 < nv) grad[i0] = (Ma[i0] - qfs[i0]) - s0;
    if (i1 < nv) grad[i1] = (Ma[i1] - qfs[i1]) - s1;
    if (i2 < nv) grad[i2] = (Ma[i2] - qfs[i2]) - s2;
    __syncwarp();
    return logical_block_sum(nv, bd, lane, [&](int i, float a) { return fmaf(grad[i], grad[i], a); });
  };
  // Upper Cholesky with the right-hand side as one more column, then the back
  // substitution (newton_stages.py:546-609).  Returns (sum x^2, sum grad x).
  auto factor_solve = [&](bool factor, float& sum0, float& sum1) {
    if (factor) {
      for (int r = 0; r < nv; ++r) {
        const float* colr = A + (r + 1) * lda;
        float acc[3];
        float diag = 0.0f;
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          const int c = r + lane + 32 * k;
          if (c <= nv) {
            float a = c < nv ? A[r * lda + c] : grad[r];
            const float* colc = c < nv ? A + (c + 1) * lda : ysm;
            for (int t = 0; t < r; ++t) a = fmaf(-colr[t], colc[t], a);
            acc[k] = a;
            if (c == r) diag = sqrtf(a);
          }
        }
        diag = __shfl_sync(IMN_FULL_MASK, diag, 0);
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          const int c = r + lane + 32 * k;
          if (c <= nv) {
            float* colc = c < nv ? A + (c + 1) * lda : ysm;
            colc[r] = (c == r) ? diag : acc[k] / diag;
          }
        }
        __syncwarp();
      }
    } else {
      // forward substitution with the stored factor: updates reach each
      // unknown in ascending order, as in the factor's augmented column
      float acc[3];
#pragma unroll
      for (int k = 0; k < 3; ++k) acc[k] = (lane + 32 * k) < nv ? grad[lane + 32 * k] : 0.0f;
      for (int t = 0; t < nv; ++t) {
        const int k0 = t >> 5;
        float mine = k0 == 0 ? acc[0] : (k0 == 1 ? acc[1] : acc[2]);
        float yt = 0.0f;
        if ((t & 31) == lane) yt = mine / A[(t + 1) * lda + t];
        yt = __shfl_sync(IMN_FULL_MASK, yt, t & 31);
        if (lane == 0) ysm[t] = yt;
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          const int r = lane + 32 * k;
          if (r > t && r < nv) acc[k] = fmaf(-A[(r + 1) * lda + t], yt, acc[k]);
        }
      }
      __syncwarp();
    }
    // back substitution, 16-row blocks from the last: later blocks' columns in
    // ascending order first, then the block's own columns from its last inwards
    for (int b0 = ((nv - 1) / 16) * 16; b0 >= 0; b0 -= 16) {
      const int b1 = min(b0 + 16, nv);
      const int r = b0 + lane;
      float acc = 0.0f;
      if (r < b1) {
        acc = ysm[r];
        for (int c = b1; c < nv; ++c) acc = fmaf(-A[(c + 1) * lda + r], xsm[c], acc);
      }
      for (int c = b1 - 1; c >= b0; --c) {
        float xc = 0.0f;
        if (r == c) xc = acc / A[(c + 1) * lda + c];
        xc = __shfl_sync(IMN_FULL_MASK, xc, c - b0);
        if (r < c && r >= b0) acc = fmaf(-A[(c + 1) * lda + r], xc, acc);
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
  row_dots(qacc, Jaref, d.efc_aref);
  mul_m(qacc, Ma);
  __syncwarp();

  float search_dot = 0.0f, grad_dot = 0.0f, grad_scale = 1.0f, decrement = 0.0f;
  float improvement = 0.0f, alpha = 0.0f;
  int quad_count = 0, state_count = 0, niter = 0, overflow = 0;
  bool search_unchanged = false, ls_exhausted = false;

  if (!rowless) {
    // _update_constraint: force / state of every row, and the list of QUADRATIC rows
    int nact = 0;
    for (int base = 0; base < nefc; base += 32) {
      const int r = base + lane;
      int st = IMN_STATE_SATISFIED;
      if (r < nefc) {
        const bool is_eq = r < ne, is_fr = !is_eq && r < nef;
        float f;
        eval_constraint(is_eq, is_fr, Jaref[r], Dsm[r], is_fr ? floss[r] : 0.0f, f, st);
        force[r] = f;
        state[r] = st;
      }
      const unsigned mask = __ballot_sync(IMN_FULL_MASK, r < nefc && st == IMN_STATE_QUADRATIC);
      if (r < nefc && st == IMN_STATE_QUADRATIC) act[nact + __popc(mask & ((1u << lane) - 1u))] = r;
      nact += __popc(mask);
    }
    __syncwarp();
    grad_dot = full_gradient();
    // H = M + J^T diag(D, QUADRATIC rows) J on the upper triangle, rows ascending
    for (int e = lane; e < (nv + 1) * lda; e += 32) A[e] = 0.0f;
    __syncwarp();
    for (int i = lane; i < nv; i += 32) {
      // the symmetric row of dof i lists every stored entry (i, c); keep c >= i
      const int k1 = m.M_mulm_rowadr[i + 1];
      for (int k = m.M_mulm_rowadr[i]; k < k1; ++k) {
        const int c = m.M_mulm_col[k];
        if (c >= i) A[i * lda + c] = Msm[m.M_mulm_madr[k]];
      }
    }
    __syncwarp();
    const int npair = nv * (nv + 1) / 2;
    for (int base = 0; base < nefc; base += 32) {
      const float* Jt = tile(base);
      const int row_hi = JRES ? nefc : min(base + 32, nefc);
      for (int e = lane; e < npair; e += 32) {
        int cj = (int)((sqrtf((float)(8 * e + 1)) - 1.0f) * 0.5f);
        while ((cj + 1) * (cj + 2) / 2 <= e) ++cj;
        while (cj * (cj + 1) / 2 > e) --cj;
        const int i = e - cj * (cj + 1) / 2;
        float v = A[i * lda + cj];
        for (int a = 0; a < nact; ++a) {
          const int r = act[a];
          if (r < base) continue;
          if (r >= row_hi) break;
          const float* Jr = Jt + (r - base) * ldj;
          v = fmaf(Jr[i] * Dsm[r], Jr[cj], v);
        }
        A[i * lda + cj] = v;
      }
      if (JRES) break;
    }
    __syncwarp();
    factor_solve(true, search_dot, decrement);
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
    // ---- exact line search (newton_stages.py:182-367) ------------------------
    float noise_floor;
    bool ls_converged;
    {
      const float snorm = sqrtf(search_dot);
      const float gtol = fmaxf(tolerance * ls_tolerance * snorm * scale, 1e-06f);
      float g0 = 0.0f, g1 = 0.0f;
      for (int i = lane; i < nv; i += 32) {
        g0 = fmaf(search[i], Ma[i] - qfs[i], g0);
        g1 = fmaf(0.5f * search[i], mv[i], g1);
      }
      for (int r = lane; r < ne; r += 32) {
        const float jvD = jv[r] * Dsm[r];
        g0 = fmaf(jvD, Jaref[r], g0);
        g1 = fmaf(0.5f * jv[r], jvD, g1);
      }
      const float q1 = ls_sum(g0, bd), q2 = ls_sum(g1, bd);
      Vec3 acc = v3(0.0f, 0.0f, 0.0f);
      for (int r = ne + lane; r < nefc; r += 32)
        acc = acc + eval_row_zero(r < nef, floss[r], Dsm[r], Jaref[r], jv[r]);
      const Vec3 rows = ls_sum(acc, bd);
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
        Vec3 a1 = v3(0.0f, 0.0f, 0.0f);
        for (int r = ne + lane; r < nefc; r += 32)
          a1 = a1 + eval_row(r < nef, floss[r], lo_alpha_in, Dsm[r], Jaref[r], jv[r]);
        lo_in = eval_quad(q1, q2, lo_alpha_in) + ls_sum(a1, bd);
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
          Vec3 s_lo = v3(0.0f, 0.0f, 0.0f), s_hi = s_lo, s_mid = s_lo;
          for (int r = ne + lane; r < nefc; r += 32) {
            const bool fr = r < nef;
            const float f = floss[r], D = Dsm[r], ja = Jaref[r], j = jv[r];
            s_lo = s_lo + eval_row(fr, f, a_lo, D, ja, j);
            s_hi = s_hi + eval_row(fr, f, a_hi, D, ja, j);
            s_mid = s_mid + eval_row(fr, f, a_mid, D, ja, j);
          }
          const Vec3 lo_next = eval_quad(q1, q2, a_lo) + ls_sum(s_lo, bd);
          const Vec3 hi_next = eval_quad(q1, q2, a_hi) + ls_sum(s_hi, bd);
          const Vec3 mid = eval_quad(q1, q2, a_mid) + ls_sum(s_mid, bd);
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
    // ---- move, re-evaluate rows, list QUADRATIC flips (newton_stages.py:373-426)
    for (int i = lane; i < nv; i += 32) {
      qacc[i] = fmaf(alpha, search[i], qacc[i]);
      Ma[i] = fmaf(alpha, mv[i], Ma[i]);
    }
    quad_count = 0;
    state_count = 0;
    for (int base = 0; base < nefc; base += 32) {
      const int r = base + lane;
      bool flip = false, changed = false;
      if (r < nefc) {
        const float nj = rounded_step(Jaref[r], alpha, jv[r]);
        Jaref[r] = nj;
        const bool is_eq = r < ne, is_fr = !is_eq && r < nef;
        float f;
        int ns;
        eval_constraint(is_eq, is_fr, nj, Dsm[r], is_fr ? floss[r] : 0.0f, f, ns);
        const int old = state[r];
        force[r] = f;
        state[r] = ns;
        flip = (old == IMN_STATE_QUADRATIC) != (ns == IMN_STATE_QUADRATIC);
        changed = old != ns;
      }
      const unsigned fm = __ballot_sync(IMN_FULL_MASK, flip);
      if (flip) ids[quad_count + __popc(fm & ((1u << lane) - 1u))] = r;
      quad_count += __popc(fm);
      state_count += __popc(__ballot_sync(IMN_FULL_MASK, changed));
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
      grad_dot = full_gradient();
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
        for (int e = lane; e < n * (n + 1) / 2; e += 32) {
          int cj = (int)((sqrtf((float)(8 * e + 1)) - 1.0f) * 0.5f);
          while ((cj + 1) * (cj + 2) / 2 <= e) ++cj;
          while (cj * (cj + 1) / 2 > e) --cj;
          const int row = uni[e - cj * (cj + 1) / 2], col = uni[cj];
          float delta = 0.0f;
          for (int t = 0; t < quad_count; ++t) {
            const int r = ids[t];
            const float a = Jat(r, row), b = Jat(r, col);
            float da = Dsm[r] * a;
            if (state[r] != IMN_STATE_QUADRATIC) da = -da;
            if (a != 0.0f && b != 0.0f) delta = fmaf(da, b, delta);
          }
          if (delta != 0.0f) A[row * lda + col] = A[row * lda + col] + delta;
        }
        __syncwarp();
      }
      factor_solve(quad_count > 0, search_dot, decrement);
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
        for (int c = r + lane; c < nv; c += 32) cx.h[ho + (size_t)r * m.nv_pad + c] = A[r * lda + c];
    if (cx.hfactor && !cx.sparse_plan)
      for (int r = 0; r < nv; ++r)
        for (int c = r + lane; c < nv; c += 32)
          cx.hfactor[ho + (size_t)r * m.nv_pad + c] = A[(c + 1) * lda + r];
  }
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
  const void* need[] = {m->opt_tolerance, m->opt_ls_tolerance, m->stat_meaninertia, m->M_rowadr,
                        m->M_colind, m->M_mulm_rowadr, m->M_mulm_col, m->M_mulm_madr, d->nefc, d->ne,
                        d->nf, d->qacc_smooth, d->qacc_warmstart, d->qfrc_smooth, d->efc_J, d->efc_D,
                        d->efc_aref, d->efc_frictionloss, d->M, d->qacc, d->qfrc_constraint, d->efc_Ma,
                        d->efc_force, d->efc_state, d->solver_niter, d->overflow};
  for (const void* p : need)
    if (!p) return set_error("imn_solve: a required Model/Data pointer is NULL"), IMN_ERR_NULL;
  if (d->dof_ld < m->nv || d->J_ld_row < m->nv || d->efc_ld < d->njmax || d->M_ld < m->nM ||
      d->J_ld_world < (int64_t)d->njmax * d->J_ld_row)
    return set_error("imn_solve: a stride is smaller than its extent"), IMN_ERR_SHAPE;
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
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return imn::set_error("imn_solve: cudaFuncSetAttribute: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  }
  if (cx->nsolving) imn::fill_nsolving<<<1, 1, 0, stream>>>(cx->nsolving, d->nworld);
  kern<<<d->nworld, 32, bytes, stream>>>(*m, *d, *cx, g);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return imn::set_error("imn_solve: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}
