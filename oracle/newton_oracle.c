/*
 * newton_oracle.c -- CPU restatement of InstantMimic's fused Newton solve.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA path: the
 * tests, the smoke run and the CPU-baseline leg of the benchmark may call it;
 * no product code may.  It walks one world at a time through the same float32
 * operations, in the same order, that the reference performs per world:
 *
 *   driver        src/instantmimic/utils/mjw_step_optimized.py:2588-2680
 *   init          src/instantmimic/utils/mjw_kernels/newton_fusion.py:412-472
 *   Newton loop   src/instantmimic/utils/mjw_kernels/newton_fusion.py:170-296
 *   line search   src/instantmimic/utils/mjw_kernels/newton_stages.py:95-442
 *   gradient      src/instantmimic/utils/mjw_kernels/newton_stages.py:745-798
 *   H update      src/instantmimic/utils/mjw_kernels/newton_stages.py:451-470, 614-742
 *   factor/solve  src/instantmimic/utils/mjw_kernels/newton_stages.py:473-611
 *   final force   src/instantmimic/utils/mjw_kernels/newton_fusion.py:522-539
 *
 * PARITY UNPINNED for the full solve: the reference delegates part of the
 * arithmetic to mujoco-warp 3.16.0 (solver.py, block_cholesky.py, support.py,
 * math.py), whose source is not part of the reference tree and is not
 * installed.  Functions marked RESTATED follow MuJoCo's published convex
 * solver (pyramidal cones, piecewise-quadratic row costs) and the argument
 * lists visible at the reference's call sites.  What IS pinned: the sparse-pattern
 * Hessian factor stages this file calls (sparse_oracle.c) bit for bit against the
 * reference's own generated CUDA code run on a B200; the KKT residual of converged
 * solves against an independent float64 solver; the self-contained linear-algebra
 * pieces against numpy.
 *
 * Rounding contract (shared with the CUDA kernels): compile with
 * -ffp-contract=off; every fused multiply-add is an explicit fmaf(); sqrtf and
 * '/' are IEEE correctly rounded; reductions over lanes follow a 32-lane
 * shuffle-down tree and later warps are added in order.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/imnewton.h"
#include "oracle_common.h"
#include "sparse_oracle.h"

#define MJ_MAXVAL 1.0e10f

typedef struct Vec3 {
  float c[3];
} Vec3;

static inline Vec3 v3(float a, float b, float c) {
  Vec3 r = {{a, b, c}};
  return r;
}
static inline Vec3 v3add(Vec3 a, Vec3 b) { return v3(a.c[0] + b.c[0], a.c[1] + b.c[1], a.c[2] + b.c[2]); }

/* RESTATED: upstream solver._eval_constraint for pyramidal rows
 * (call site newton_stages.py:385-399). */
static inline void eval_constraint(int is_equality, int is_friction, float jaref, float D,
                                   float frictionloss, float* force, int* state) {
  if (is_equality) {
    *force = -D * jaref;
    *state = IMN_STATE_QUADRATIC;
    return;
  }
  if (is_friction) {
    const float rf = safe_div(frictionloss, D);
    if (jaref <= -rf) {
      *force = frictionloss;
      *state = IMN_STATE_LINEARNEG;
      return;
    }
    if (jaref >= rf) {
      *force = -frictionloss;
      *state = IMN_STATE_LINEARPOS;
      return;
    }
    *force = -D * jaref;
    *state = IMN_STATE_QUADRATIC;
    return;
  }
  if (jaref >= 0.0f) {
    *force = 0.0f;
    *state = IMN_STATE_SATISFIED;
    return;
  }
  *force = -D * jaref;
  *state = IMN_STATE_QUADRATIC;
}

/* RESTATED: upstream solver._compute_efc_eval_pt_pyramidal and its alpha = 0
 * form (call sites newton_stages.py:209-217, 241-250, 271-282).  A row's cost is
 * piecewise in x = Jaref + alpha jv: zero (inequality, x >= 0), quadratic
 * 0.5 D x^2, or linear beyond +-frictionloss / D (friction rows).
 *   eval_row_zero: (cost, slope, curvature) at alpha = 0.
 *   eval_row:      (cost(alpha) - cost(0), slope, curvature) at alpha; the
 *                  search brackets on cost CHANGES (the reference zeroes the
 *                  cost of its alpha = 0 point, newton_stages.py:223), and a
 *                  change within one piece is formed without cancellation. */
static inline int row_zone(float x, int is_friction, float rf) {
  if (is_friction) return x <= -rf ? IMN_STATE_LINEARNEG : (x >= rf ? IMN_STATE_LINEARPOS : IMN_STATE_QUADRATIC);
  return x >= 0.0f ? IMN_STATE_SATISFIED : IMN_STATE_QUADRATIC;
}
static inline float zone_cost(int zone, float x, float D, float f, float rf) {
  switch (zone) {
    case IMN_STATE_QUADRATIC: return ((0.5f * D) * x) * x;
    case IMN_STATE_LINEARNEG: return f * (-0.5f * rf - x);
    case IMN_STATE_LINEARPOS: return f * (-0.5f * rf + x);
    default: return 0.0f;
  }
}
static inline Vec3 zone_slope(int zone, float x, float D, float f, float jv) {
  switch (zone) {
    case IMN_STATE_QUADRATIC: {
      const float jvD = jv * D;
      return v3(0.0f, jvD * x, jv * jvD);
    }
    case IMN_STATE_LINEARNEG: return v3(0.0f, -f * jv, 0.0f);
    case IMN_STATE_LINEARPOS: return v3(0.0f, f * jv, 0.0f);
    default: return v3(0.0f, 0.0f, 0.0f);
  }
}
static inline Vec3 eval_row_zero(int efcid, int nef, float D, const float* frictionloss,
                                 float jaref, float jv) {
  const int fr = efcid < nef;
  const float f = fr ? frictionloss[efcid] : 0.0f;
  const float rf = fr ? safe_div(f, D) : 0.0f;
  const int z = row_zone(jaref, fr, rf);
  Vec3 r = zone_slope(z, jaref, D, f, jv);
  r.c[0] = zone_cost(z, jaref, D, f, rf);
  return r;
}
static inline Vec3 eval_row(int efcid, float alpha, int nef, float D, const float* frictionloss,
                            float jaref, float jv) {
  const int fr = efcid < nef;
  const float f = fr ? frictionloss[efcid] : 0.0f;
  const float rf = fr ? safe_div(f, D) : 0.0f;
  const float x = fmaf(alpha, jv, jaref);
  const int z0 = row_zone(jaref, fr, rf), z = row_zone(x, fr, rf);
  Vec3 r = zone_slope(z, x, D, f, jv);
  if (z != z0) {
    r.c[0] = zone_cost(z, x, D, f, rf) - zone_cost(z0, jaref, D, f, rf);
  } else if (z == IMN_STATE_QUADRATIC) {
    const float jvD = jv * D;
    r.c[0] = alpha * fmaf(0.5f * alpha, jv * jvD, jvD * jaref);
  } else if (z == IMN_STATE_LINEARNEG) {
    r.c[0] = -f * (alpha * jv);
  } else if (z == IMN_STATE_LINEARPOS) {
    r.c[0] = f * (alpha * jv);
  }
  return r;
}

/* RESTATED: upstream solver._eval_pt on the Gauss quadratic
 * (call site newton_stages.py:252). */
static inline Vec3 eval_quad(const float q[3], float alpha) {
  return v3(fmaf(alpha, q[1], (alpha * alpha) * q[2]) + q[0], fmaf(2.0f * alpha, q[2], q[1]),
            2.0f * q[2]);
}
/* RESTATED: upstream solver._in_bracket (call sites newton_stages.py:331-349). */
static inline int in_bracket(Vec3 x, Vec3 y) {
  return (x.c[1] < y.c[1] && y.c[1] < 0.0f) || (x.c[1] > y.c[1] && y.c[1] > 0.0f);
}

typedef struct World {
  int nv, nefc, ne, nf, bd, nwarps, ldj;
  const float* J;
  const float *D, *aref, *floss, *qfs, *M;
  float *qacc, *Ma, *search, *mv, *grad, *H, *U, *y, *x;
  float *Jaref, *jv, *force;
  int *state, *ids, *uni;
  float search_dot, grad_dot, grad_scale, decrement, improvement, alpha;
  int quad_count, state_count, search_unchanged, ls_exhausted, done, niter, overflow;
  /* work counters reported through ctx->stats */
  int st_passes, st_flips, st_factor, st_grad;
  /* static-pattern sparse factor (NULL: dense): packed H, N = L D with the carried
   * right-hand-side row, 1/D, and the count of pattern violations of this solve */
  const ImnSparsePlan* sp;
  float *Hp, *N, *iD;
  int violations;
} World;

/* Sparse counterpart of factor_solve: mode 0 refactors the packed H, mode 1 solves
 * with the resident factor (sparse_hessian.py:490-547). */
static void factor_solve_sparse(World* w, int factor, float sums[2]) {
  if (factor) {
    memcpy(w->N, w->Hp, sizeof(float) * w->sp->nfac);
    sparse_load_rhs(w->sp, w->N, w->grad);
    sparse_factor_levels(w->sp, w->N, w->iD);
  } else {
    sparse_forward(w->sp, w->N, w->iD, w->grad);
  }
  sparse_backward(w->sp, w->N, w->iD, w->grad, w->search, w->sp->block, sums);
}

/* ctx.grad_dot: Warp tile_sum of one partial per thread of the logical block
 * (newton_stages.py:785-795). */
static float strided_square_sum(const float* g, int nv, int bd) {
  float part[64];
  for (int t = 0; t < bd; ++t) {
    float s = 0.0f;
    for (int i = t; i < nv; i += bd) s = fmaf(g[i], g[i], s);
    part[t] = s;
  }
  return block_sum(part, bd);
}

static void mul_m(const ImnModel* m, const float* M, const float* v, float* out) {
  for (int i = 0; i < m->nv; ++i) {
    float s = 0.0f;
    for (int k = m->M_mulm_rowadr[i]; k < m->M_mulm_rowadr[i + 1]; ++k)
      s = fmaf(M[m->M_mulm_madr[k]], v[m->M_mulm_col[k]], s);
    out[i] = s;
  }
}

/* J row times a dof vector: one running sum per row; above 50 dofs the sum is
 * split into 20-dof partials joined by plain adds (newton_stages.py:157-174). */
static float row_dot(const float* Jr, const float* v, int nv) {
  if (nv > 50) {
    float total = 0.0f;
    for (int s = 0; s < nv; s += 20) {
      float p = 0.0f;
      const int e = s + 20 < nv ? s + 20 : nv;
      for (int i = s; i < e; ++i) p = fmaf(Jr[i], v[i], p);
      total = total + p;
    }
    return total;
  }
  float p = 0.0f;
  for (int i = 0; i < nv; ++i) p = fmaf(Jr[i], v[i], p);
  return p;
}

/* qfrc_constraint = J^T force, one running sum per dof over ascending rows
 * (newton_stages.py:786-790), then grad and its squared norm. */
static void full_gradient(World* w) {
  for (int i = 0; i < w->nv; ++i) {
    float s = 0.0f;
    for (int r = 0; r < w->nefc; ++r) s = fmaf(w->J[(size_t)r * w->ldj + i], w->force[r], s);
    w->grad[i] = (w->Ma[i] - w->qfs[i]) - s;
  }
  w->grad_dot = strided_square_sum(w->grad, w->nv, w->bd);
}

/* Upper Cholesky H = U^T U with the right-hand side carried as one more
 * column (forward solve), then back substitution in 16-wide block order
 * (newton_stages.py:546-609).  Each entry subtracts its inner products in
 * ascending row order with fused multiply-adds.  factor == 0 reuses U
 * (newton_stages.py:736-737).  Returns (sum x^2, sum grad x); search = -x. */
static void factor_solve(World* w, int factor, float sums[2]) {
  const int nv = w->nv;
  float *U = w->U, *y = w->y, *x = w->x;
  const float* H = w->H;
  for (int r = 0; r < nv; ++r) {
    if (factor) {
      float acc = H[r * nv + r];
      for (int t = 0; t < r; ++t) acc = fmaf(-U[t * nv + r], U[t * nv + r], acc);
      const float d = sqrtf(acc);
      const float rinv = 1.0f / d; /* the row is scaled by the reciprocal pivot */
      U[r * nv + r] = d;
      for (int c = r + 1; c < nv; ++c) {
        acc = H[r * nv + c];
        for (int t = 0; t < r; ++t) acc = fmaf(-U[t * nv + r], U[t * nv + c], acc);
        U[r * nv + c] = acc * rinv;
      }
    }
    float acc = w->grad[r];
    for (int t = 0; t < r; ++t) acc = fmaf(-U[t * nv + r], y[t], acc);
    y[r] = acc * (1.0f / U[r * nv + r]);
  }
  for (int r = nv - 1; r >= 0; --r) {
    const int tile_end = ((r / 16) + 1) * 16 < nv ? ((r / 16) + 1) * 16 : nv;
    float acc = y[r];
    /* later 16-wide blocks first, in ascending order (newton_stages.py:605-607),
     * then the row's own diagonal block from its last column inwards */
    for (int c = tile_end; c < nv; ++c) acc = fmaf(-U[r * nv + c], x[c], acc);
    for (int c = tile_end - 1; c > r; --c) acc = fmaf(-U[r * nv + c], x[c], acc);
    x[r] = acc * (1.0f / U[r * nv + r]);
  }
  float p0[64], p1[64];
  for (int t = 0; t < w->bd; ++t) {
    float s0 = 0.0f, s1 = 0.0f;
    for (int i = t; i < nv; i += w->bd) {
      s0 = fmaf(x[i], x[i], s0);
      s1 = fmaf(w->grad[i], x[i], s1);
    }
    p0[t] = s0;
    p1[t] = s1;
  }
  sums[0] = block_sum(p0, w->bd);
  sums[1] = block_sum(p1, w->bd);
  for (int i = 0; i < nv; ++i) w->search[i] = -x[i];
}

/* H = M + sum over QUADRATIC rows of D J^T J, upper triangle, rows ascending. */
static void assemble_hessian(const ImnModel* m, World* w) {
  const int nv = w->nv;
  memset(w->H, 0, sizeof(float) * nv * nv);
  for (int j = 0; j < nv; ++j)
    for (int k = 0; k < m->M_rownnz[j]; ++k) {
      const int e = m->M_rowadr[j] + k;
      w->H[m->M_colind[e] * nv + j] = w->M[e];
    }
  for (int i = 0; i < nv; ++i)
    for (int j = i; j < nv; ++j) {
      float v = w->H[i * nv + j];
      for (int r = 0; r < w->nefc; ++r)
        if (w->state[r] == IMN_STATE_QUADRATIC)
          v = fmaf(w->J[(size_t)r * w->ldj + i] * w->D[r], w->J[(size_t)r * w->ldj + j], v);
      w->H[i * nv + j] = v;
    }
}

/* Exact line search of newton_stages.py:182-367 on lanes 0..31. */
static void line_search(const ImnModel* m, World* w, int worldid, float* noise_floor_out,
                        int* ls_converged_out) {
  const int nv = w->nv, ne = w->ne, nef = w->ne + w->nf, nefc = w->nefc;
  const float eps = m->alpha_noise_eps;
  const float tolerance = m->opt_tolerance[worldid % m->n_tolerance];
  const float ls_tolerance = m->opt_ls_tolerance[worldid % m->n_ls_tolerance];
  const float snorm = sqrtf(w->search_dot);
  const float scale = m->stat_meaninertia[worldid % m->n_meaninertia] * (float)nv;
  const float gtol = fmaxf(tolerance * ls_tolerance * snorm * scale, 1e-06f);
  float lane0[32], lane1[32], lane2[32];
  for (int l = 0; l < 32; ++l) {
    float g0 = 0.0f, g1 = 0.0f;
    for (int i = l; i < nv; i += 32) {
      g0 = fmaf(w->search[i], w->Ma[i] - w->qfs[i], g0);
      g1 = fmaf(0.5f * w->search[i], w->mv[i], g1);
    }
    for (int r = l; r < ne; r += 32) {
      const float jvD = w->jv[r] * w->D[r];
      g0 = fmaf(jvD, w->Jaref[r], g0);
      g1 = fmaf(0.5f * w->jv[r], jvD, g1);
    }
    lane0[l] = g0;
    lane1[l] = g1;
  }
  const float qg[3] = {0.0f, block_sum32(lane0, w->nwarps), block_sum32(lane1, w->nwarps)};

#define ROW_SUM(OUT, EXPR)                                      \
  do {                                                          \
    for (int l = 0; l < 32; ++l) {                              \
      Vec3 acc = v3(0.0f, 0.0f, 0.0f);                          \
      for (int r = ne + l; r < nefc; r += 32) {                 \
        acc = v3add(acc, (EXPR));                               \
      }                                                         \
      lane0[l] = acc.c[0];                                      \
      lane1[l] = acc.c[1];                                      \
      lane2[l] = acc.c[2];                                      \
    }                                                           \
    (OUT) = v3(block_sum32(lane0, w->nwarps), block_sum32(lane1, w->nwarps), \
               block_sum32(lane2, w->nwarps));                  \
  } while (0)

  Vec3 rows;
  w->st_passes += 1;
  ROW_SUM(rows, eval_row_zero(r, nef, w->D[r], w->floss, w->Jaref[r], w->jv[r]));
  const Vec3 p0 = v3add(v3(qg[0], qg[1], 2.0f * qg[2]), rows);
  const Vec3 p0_delta = v3(0.0f, p0.c[1], p0.c[2]);
  const float q1_abs =
      sqrtf(2.0f * fmaxf(rows.c[0], 0.0f) * fmaxf(rows.c[2], 0.0f)) + fabsf(qg[1]);
  const float gtol_accept = fmaxf(gtol, eps * q1_abs);
  const float noise_floor = eps * fmaxf(1.0f, safe_div(q1_abs, p0.c[2]));
  float alpha = 0.0f, improvement = 0.0f;
  int ls_converged = fabsf(p0.c[1]) < eps * q1_abs;
  const float lo_alpha_in = -safe_div(p0.c[1], p0.c[2]);
  Vec3 lo_in = v3(0.0f, 0.0f, 0.0f);
  if (!ls_converged) {
    Vec3 s;
    w->st_passes += 1;
    ROW_SUM(s, eval_row(r, lo_alpha_in, nef, w->D[r], w->floss, w->Jaref[r], w->jv[r]));
    lo_in = v3add(eval_quad(qg, lo_alpha_in), s);
    if (fabsf(lo_in.c[1]) < gtol_accept && lo_in.c[0] < 0.0f) {
      ls_converged = 1;
      alpha = lo_alpha_in;
      improvement = -lo_in.c[0];
    }
  }
  if (!ls_converged) {
    const int lo_less = lo_in.c[1] < p0.c[1];
    Vec3 lo = lo_less ? lo_in : p0_delta;
    float lo_alpha = lo_less ? lo_alpha_in : 0.0f;
    Vec3 hi = lo_less ? p0_delta : lo_in;
    float hi_alpha = lo_less ? 0.0f : lo_alpha_in;
    for (int it = 0; it < m->ls_iterations; ++it) {
      const float a_lo = lo_alpha - safe_div(lo.c[1], lo.c[2]);
      const float a_hi = hi_alpha - safe_div(hi.c[1], hi.c[2]);
      const float a_mid = 0.5f * (lo_alpha + hi_alpha);
      Vec3 s_lo, s_hi, s_mid;
      w->st_passes += 1;
      ROW_SUM(s_lo, eval_row(r, a_lo, nef, w->D[r], w->floss, w->Jaref[r], w->jv[r]));
      ROW_SUM(s_hi, eval_row(r, a_hi, nef, w->D[r], w->floss, w->Jaref[r], w->jv[r]));
      ROW_SUM(s_mid, eval_row(r, a_mid, nef, w->D[r], w->floss, w->Jaref[r], w->jv[r]));
      const Vec3 lo_next = v3add(eval_quad(qg, a_lo), s_lo);
      const Vec3 hi_next = v3add(eval_quad(qg, a_hi), s_hi);
      const Vec3 mid = v3add(eval_quad(qg, a_mid), s_mid);
      const int conv_lo = fabsf(lo_next.c[1]) < gtol_accept && lo_next.c[0] < 0.0f;
      const int conv_hi = fabsf(hi_next.c[1]) < gtol_accept && hi_next.c[0] < 0.0f;
      const int conv_mid = fabsf(mid.c[1]) < gtol_accept && mid.c[0] < 0.0f;
      const int converged = conv_lo || conv_hi || conv_mid;
      int swap_lo = 0, swap_hi = 0;
      if (converged) {
        Vec3 best = v3(MJ_MAXVAL, 0.0f, 0.0f);
        float best_alpha = 0.0f;
        if (conv_lo && lo_next.c[0] < best.c[0]) best = lo_next, best_alpha = a_lo;
        if (conv_hi && hi_next.c[0] < best.c[0]) best = hi_next, best_alpha = a_hi;
        if (conv_mid && mid.c[0] < best.c[0]) best = mid, best_alpha = a_mid;
        lo = hi = best;
        lo_alpha = hi_alpha = best_alpha;
      } else {
        /* candidates are tried in the order lo_next, mid, hi_next for the low
         * end and hi_next, mid, lo_next for the high end; each compares with the
         * bracket end as already moved by the earlier candidates */
        int s;
        s = in_bracket(lo, lo_next);
        if (s) lo = lo_next, lo_alpha = a_lo;
        swap_lo |= s;
        s = in_bracket(lo, mid);
        if (s) lo = mid, lo_alpha = a_mid;
        swap_lo |= s;
        s = in_bracket(lo, hi_next);
        if (s) lo = hi_next, lo_alpha = a_hi;
        swap_lo |= s;
        s = in_bracket(hi, hi_next) || (hi.c[1] < 0.0f && hi_next.c[1] > 0.0f);
        if (s) hi = hi_next, hi_alpha = a_hi;
        swap_hi |= s;
        s = in_bracket(hi, mid);
        if (s) hi = mid, hi_alpha = a_mid;
        swap_hi |= s;
        s = in_bracket(hi, lo_next);
        if (s) hi = lo_next, hi_alpha = a_lo;
        swap_hi |= s;
      }
      const int ls_done = converged || (!swap_lo && !swap_hi) ||
                          (lo.c[0] < 0.0f && lo.c[1] < 0.0f && lo.c[1] > -gtol) ||
                          (hi.c[0] < 0.0f && hi.c[1] > 0.0f && hi.c[1] < gtol);
      if (lo.c[0] < 0.0f || hi.c[0] < 0.0f) {
        const int lo_better = lo.c[0] < hi.c[0];
        alpha = lo_better ? lo_alpha : hi_alpha;
        improvement = -(lo_better ? lo.c[0] : hi.c[0]);
      }
      if (ls_done) {
        ls_converged = 1;
        break;
      }
    }
  }
#undef ROW_SUM
  w->alpha = alpha;
  w->improvement = improvement;
  *noise_floor_out = noise_floor;
  *ls_converged_out = ls_converged;
}

/* Changed rows -> dofs they touch (ascending), then the pair update of H
 * (newton_stages.py:651-701). */
static void update_hessian(World* w) {
  const int nv = w->nv, count = w->quad_count;
  int n = 0;
  for (int dof = 0; dof < nv; ++dof) {
    int hit = 0;
    for (int t = 0; t < count && !hit; ++t)
      hit = w->J[(size_t)w->ids[t] * w->ldj + dof] != 0.0f;
    if (hit) w->uni[n++] = dof;
  }
  w->uni[nv] = n;
  if (w->sp) {
    /* sparse plan: the same pair loop lands in the packed H (sparse_hessian.py:501-527) */
    w->violations += sparse_update(w->sp, w->Hp, w->J, w->ldj, w->D, w->state, w->ids, count, w->uni, n);
    return;
  }
  for (int cj = 0; cj < n; ++cj)
    for (int ri = 0; ri <= cj; ++ri) {
      const int row = w->uni[ri], col = w->uni[cj];
      float delta = 0.0f;
      for (int t = 0; t < count; ++t) {
        const int r = w->ids[t];
        const float a = w->J[(size_t)r * w->ldj + row];
        const float b = w->J[(size_t)r * w->ldj + col];
        float da = w->D[r] * a;
        if (w->state[r] != IMN_STATE_QUADRATIC) da = -da;
        if (a != 0.0f && b != 0.0f) delta = fmaf(da, b, delta);
      }
      if (delta != 0.0f) w->H[row * nv + col] = w->H[row * nv + col] + delta;
    }
}

typedef struct Workspace {
  float* f;
  int* i;
} Workspace;

static void solve_world(const ImnModel* m, const ImnData* d, const ImnCtx* ctx, int wid,
                        Workspace* ws, int* finished) {
  const int nv = m->nv, R = d->njmax;
  World w;
  memset(&w, 0, sizeof w);
  w.nv = nv;
  w.bd = m->nv_pad >= 64 ? 64 : 32;
  w.nwarps = w.bd / 32;
  const int nefc_in = d->nefc[wid];
  w.nefc = nefc_in < R ? nefc_in : R;
  w.ne = d->ne[wid];
  w.nf = d->nf[wid];
  w.ldj = (int)d->J_ld_row;
  w.J = d->efc_J + (d->J_world_offset ? (size_t)d->J_world_offset[wid] : (size_t)wid * d->J_ld_world);
  w.D = d->efc_D + (size_t)wid * d->efc_ld;
  w.aref = d->efc_aref + (size_t)wid * d->efc_ld;
  w.floss = d->efc_frictionloss + (size_t)wid * d->efc_ld;
  w.qfs = d->qfrc_smooth + (size_t)wid * d->dof_ld;
  w.M = d->M + (size_t)wid * d->M_ld;
  float* f = ws->f;
  w.qacc = f, f += nv;
  w.Ma = f, f += nv;
  w.search = f, f += nv;
  w.mv = f, f += nv;
  w.grad = f, f += nv;
  w.y = f, f += nv;
  w.x = f, f += nv;
  w.H = f, f += nv * nv;
  w.U = f, f += nv * nv;
  w.Jaref = f, f += R;
  w.jv = f, f += R;
  w.force = f, f += R;
  w.state = ws->i;
  w.ids = ws->i + R;
  w.uni = ws->i + 2 * R;
  w.sp = ctx ? ctx->sparse_plan : NULL;
  if (w.sp) {
    w.Hp = f, f += w.sp->nfac;
    w.N = f, f += w.sp->nslots;
    w.iD = f, f += nv;
  }
  const float* qsm = d->qacc_smooth + (size_t)wid * d->dof_ld;
  const float* qws = d->qacc_warmstart + (size_t)wid * d->dof_ld;
  const int rowless = nefc_in == 0;

  /* _solve_init_dof + _init_efc_settling_empty_worlds */
  for (int i = 0; i < nv; ++i) w.qacc[i] = (m->warmstart && !rowless) ? qws[i] : qsm[i];
  w.done = rowless;
  /* Jaref = J qacc - aref (RESTATED: upstream _solve_init_jaref_kernel; the
   * first partial carries -aref, later 20-dof partials are added in order) */
  for (int r = 0; r < w.nefc; ++r) {
    const float* Jr = w.J + (size_t)r * w.ldj;
    if (nv > 50) {
      float total = 0.0f;
      for (int s = 0; s < nv; s += 20) {
        float p = 0.0f;
        const int e = s + 20 < nv ? s + 20 : nv;
        for (int i = s; i < e; ++i) p = fmaf(Jr[i], w.qacc[i], p);
        total = (s == 0) ? p - w.aref[r] : total + p;
      }
      w.Jaref[r] = total;
    } else {
      w.Jaref[r] = row_dot(Jr, w.qacc, nv) - w.aref[r];
    }
  }
  mul_m(m, w.M, w.qacc, w.Ma);
  memset(w.mv, 0, sizeof(float) * nv);
  memset(w.search, 0, sizeof(float) * nv);
  memset(w.grad, 0, sizeof(float) * nv);
  memset(w.jv, 0, sizeof(float) * R);
  w.grad_scale = 1.0f;
  if (!rowless) {
    /* _update_constraint, _update_gradient (RESTATED, upstream) */
    for (int r = 0; r < w.nefc; ++r)
      eval_constraint(r < w.ne, r >= w.ne && r < w.ne + w.nf, w.Jaref[r], w.D[r],
                      (r >= w.ne && r < w.ne + w.nf) ? w.floss[r] : 0.0f, &w.force[r],
                      &w.state[r]);
    full_gradient(&w);
    w.st_grad = 1, w.st_factor = 1;
    float sums[2];
    if (w.sp) {
      /* H on the pattern slots, kept packed, then the level factor
       * (sparse_hessian.py:571-637) */
      w.violations += sparse_assemble(w.sp, w.N, w.M, w.J, w.ldj, w.D, w.state, w.nefc);
      memcpy(w.Hp, w.N, sizeof(float) * w.sp->nfac);
      factor_solve_sparse(&w, 1, sums);
    } else {
      assemble_hessian(m, &w);
      factor_solve(&w, 1, sums);
    }
    w.search_dot = sums[0];
    w.decrement = sums[1];
  }
  int overflow = 0;
  while (!w.done) {
    if (!w.search_unchanged) mul_m(m, w.M, w.search, w.mv);
    w.quad_count = 0;
    w.state_count = 0;
    if (!w.search_unchanged)
      for (int r = 0; r < w.nefc; ++r) w.jv[r] = row_dot(w.J + (size_t)r * w.ldj, w.search, nv);
    float noise_floor;
    int ls_converged;
    line_search(m, &w, wid, &noise_floor, &ls_converged);
    const float alpha = w.alpha;
    for (int i = 0; i < nv; ++i) {
      w.qacc[i] = fmaf(alpha, w.search[i], w.qacc[i]);
      w.Ma[i] = fmaf(alpha, w.mv[i], w.Ma[i]);
    }
    for (int r = 0; r < w.nefc; ++r) {
      const float nj = w.Jaref[r] + alpha * w.jv[r]; /* two roundings, never fused */
      w.Jaref[r] = nj;
      const int is_eq = r < w.ne, is_fr = !is_eq && r < w.ne + w.nf;
      int ns;
      eval_constraint(is_eq, is_fr, nj, w.D[r], is_fr ? w.floss[r] : 0.0f, &w.force[r], &ns);
      const int old = w.state[r];
      w.state[r] = ns;
      if ((old == IMN_STATE_QUADRATIC) != (ns == IMN_STATE_QUADRATIC)) w.ids[w.quad_count++] = r;
      if (old != ns) w.state_count++;
    }
    w.ls_exhausted = fabsf(alpha) < noise_floor;
    if (w.ls_exhausted) w.state_count++;
    if (!ls_converged) overflow |= m->overflow_ls_iterations;
    /* gradient */
    const int changed = w.state_count != 0;
    w.search_unchanged = !changed;
    if (!changed) {
      const float sigma = w.grad_scale, ns = sigma - alpha;
      const float ratio = sigma != 0.0f ? ns / sigma : 0.0f;
      const float rsq = ratio * ratio;
      w.grad_dot *= rsq;
      w.decrement *= rsq;
      w.grad_scale = ns;
    } else {
      full_gradient(&w);
      w.st_grad++, w.st_flips += w.quad_count, w.st_factor += w.quad_count > 0;
      w.decrement = 0.0f;
      w.grad_scale = 1.0f;
      /* factor */
      if (w.quad_count > 0) update_hessian(&w);
      float sums[2];
      if (w.sp)
        factor_solve_sparse(&w, w.quad_count > 0, sums);
      else
        factor_solve(&w, w.quad_count > 0, sums);
      w.search_dot = sums[0];
      w.decrement = sums[1];
    }
    /* convergence (newton_fusion.py:267-295) */
    w.niter++;
    const float tol = m->opt_tolerance[wid % m->n_tolerance];
    const float scale = m->stat_meaninertia[wid % m->n_meaninertia] * (float)nv;
    const int converged = w.alpha == 0.0f ||
                          (w.improvement > 0.0f && w.improvement / scale < tol) ||
                          sqrtf(w.grad_dot) / scale < tol || 0.5f * w.decrement / scale < tol;
    if (converged || w.niter == m->iterations) {
      if (!converged) overflow |= m->overflow_iterations;
      w.done = 1;
      (*finished)++;
    }
  }
  /* outputs */
  float* qacc = d->qacc + (size_t)wid * d->dof_ld;
  float* qfc = d->qfrc_constraint + (size_t)wid * d->dof_ld;
  float* Ma = d->efc_Ma + (size_t)wid * d->dof_ld;
  for (int i = 0; i < nv; ++i) {
    qacc[i] = w.qacc[i];
    Ma[i] = w.Ma[i];
    qfc[i] = rowless ? 0.0f : fmaf(-w.grad_scale, w.grad[i], w.Ma[i] - w.qfs[i]);
  }
  for (int r = 0; r < w.nefc; ++r) {
    d->efc_force[(size_t)wid * d->efc_ld + r] = w.force[r];
    d->efc_state[(size_t)wid * d->efc_ld + r] = w.state[r];
  }
  d->solver_niter[wid] = w.niter;
  d->overflow[wid] |= overflow;
  if (ctx) {
#define PUT(ARR, LD, N, SRC)                                                        \
  if (ctx->ARR)                                                                     \
    for (int q = 0; q < (N); ++q) ctx->ARR[(size_t)wid * (LD) + q] = (SRC)[q]
    PUT(Jaref, d->efc_ld, w.nefc, w.Jaref);
    PUT(jv, d->efc_ld, w.nefc, w.jv);
    PUT(search, d->dof_ld, nv, w.search);
    PUT(mv, d->dof_ld, nv, w.mv);
    PUT(grad, ctx->grad_ld, nv, w.grad);
    PUT(quad_changed_ids, d->efc_ld, w.quad_count, w.ids);
#undef PUT
    if (ctx->search_dot) ctx->search_dot[wid] = w.search_dot;
    if (ctx->grad_dot && !rowless) ctx->grad_dot[wid] = w.grad_dot;
    if (ctx->grad_scale && !rowless) ctx->grad_scale[wid] = w.grad_scale;
    if (ctx->newton_decrement && !rowless) ctx->newton_decrement[wid] = w.decrement;
    if (ctx->improvement && !rowless) ctx->improvement[wid] = w.improvement;
    if (ctx->alpha && !rowless) ctx->alpha[wid] = w.alpha;
    if (ctx->done) ctx->done[wid] = 1;
    if (ctx->stats) {
      int32_t* st = ctx->stats + 4 * (size_t)wid;
      st[0] = w.st_passes, st[1] = w.st_flips, st[2] = w.st_factor, st[3] = w.st_grad;
    }
    if (ctx->search_unchanged && !rowless) ctx->search_unchanged[wid] = (uint8_t)w.search_unchanged;
    if (ctx->ls_exhausted && !rowless) ctx->ls_exhausted[wid] = (uint8_t)w.ls_exhausted;
    if (ctx->quad_changed_count && !rowless) ctx->quad_changed_count[wid] = w.quad_count;
    if (ctx->state_changed_count && !rowless) ctx->state_changed_count[wid] = w.state_count;
    if (ctx->h && !rowless && !w.sp)
      for (int r = 0; r < nv; ++r)
        for (int c = r; c < nv; ++c)
          ctx->h[((size_t)wid * m->nv_pad + r) * m->nv_pad + c] = w.H[r * nv + c];
    if (ctx->hfactor && !rowless && w.sp) {
      /* packed H | N | 1/D, and the violation counter in the last element
       * (sparse_hessian.py:488-489, 795-796) */
      float* Uf = ctx->hfactor + (size_t)wid * m->nv_pad * m->nv_pad;
      const int nfac = w.sp->nfac;
      for (int q = 0; q < nfac; ++q) Uf[q] = w.Hp[q], Uf[nfac + q] = w.N[q];
      for (int q = 0; q < nv; ++q) Uf[2 * nfac + q] = w.iD[q];
      Uf[m->nv_pad * m->nv_pad - 1] += (float)w.violations;
    }
    if (ctx->hfactor && !rowless && !ctx->sparse_plan)
      for (int r = 0; r < nv; ++r)
        for (int c = r; c < nv; ++c)
          ctx->hfactor[((size_t)wid * m->nv_pad + r) * m->nv_pad + c] = w.U[r * nv + c];
  }
}

/* Same contract as imn_solve, on host pointers.  threads <= 0: all cores. */
int oracle_solve(const ImnModel* m, const ImnData* d, const ImnCtx* ctx, int threads) {
  const int nv = m->nv, R = d->njmax;
  size_t nf = (size_t)7 * nv + (size_t)2 * nv * nv + (size_t)3 * R + 64;
  if (ctx && ctx->sparse_plan) nf += (size_t)ctx->sparse_plan->nfac + ctx->sparse_plan->nslots + nv;
  const size_t ni = (size_t)2 * R + nv + 8;
  int finished = 0;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
#pragma omp parallel reduction(+ : finished)
  {
    Workspace ws;
    ws.f = (float*)malloc(nf * sizeof(float));
    ws.i = (int*)malloc(ni * sizeof(int));
#pragma omp for schedule(dynamic, 8)
    for (int wid = 0; wid < d->nworld; ++wid) solve_world(m, d, ctx, wid, &ws, &finished);
    free(ws.f);
    free(ws.i);
  }
  if (ctx && ctx->nsolving) ctx->nsolving[0] = d->nworld - finished;
  return 0;
}

/* Rowless hand-off (mjw_step_optimized.py:2692-2699). */
int oracle_rowless_handoff(const ImnModel* m, const ImnData* d) {
  for (int wid = 0; wid < d->nworld; ++wid) {
    const float* qsm = d->qacc_smooth + (size_t)wid * d->dof_ld;
    float* qacc = d->qacc + (size_t)wid * d->dof_ld;
    for (int i = 0; i < m->nv; ++i) qacc[i] = qsm[i];
    mul_m(m, d->M + (size_t)wid * d->M_ld, qacc, d->efc_Ma + (size_t)wid * d->dof_ld);
    for (int i = 0; i < m->nv; ++i) d->qfrc_constraint[(size_t)wid * d->dof_ld + i] = 0.0f;
    d->solver_niter[wid] = 0;
  }
  return 0;
}

int oracle_mul_m(const ImnModel* m, const float* M, int64_t M_ld, const float* v, int64_t v_ld,
                 float* out, int64_t out_ld, int nworld) {
  for (int w = 0; w < nworld; ++w)
    mul_m(m, M + (size_t)w * M_ld, v + (size_t)w * v_ld, out + (size_t)w * out_ld);
  return 0;
}
