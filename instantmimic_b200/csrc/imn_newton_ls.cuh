// imn_newton_ls.cuh -- exact line search on the piecewise-quadratic cost along the
// search direction (reference: newton_stages.py:182-367), one warp, rows over lanes.
//
// The search is a sequence of evaluation passes over the inequality / friction
// rows: pass 0 at alpha = 0 (absolute costs), pass 1 at the first Newton step, then
// one pass per bracket iteration at three step sizes.  All passes run through ONE
// evaluation site (three step sizes per pass; the first two passes use one of
// them), which keeps the machine code small.  A lane keeps its first two rows in
// registers; further rows are re-read from shared memory in ascending order, so
// each lane adds its rows in the same order as a strided loop would.
#pragma once

#include "imn_newton_linalg.cuh"

namespace imn {

// Row sums of one lane at step size `al` in the general form (friction-loss rows,
// or more than two rows per lane): rows ne+lane, ne+lane+32, ... in ascending order,
// each prepared from shared memory.  Kept out of line: models without friction-loss
// rows and with at most 64 inequality rows never run it, and the line search's
// resident code stays small (the kernel is bound by instruction fetch).
__device__ __noinline__ Vec3 ls_rows_general(const float* floss, const float* D, const float* Jaref,
                                             const float* jv, int ne, int nef, int nefc, int lane, float al,
                                             bool absolute) {
  Vec3 acc = v3(0.0f, 0.0f, 0.0f);
#pragma unroll 1
  for (int r = ne + lane; r < nefc; r += 32)
    acc = acc + row_at(make_row(true, r < nef, floss[r], D[r], Jaref[r], jv[r]), al, absolute);
  return acc;
}

struct LineSearchResult {
  float alpha, improvement, noise_floor;
  bool converged;
  int passes;  // row-evaluation passes made
};

__device__ __forceinline__ LineSearchResult line_search(const World& s, float search_dot, float tolerance,
                                                        float ls_tolerance, float scale, float eps,
                                                        int ls_iterations) {
  const int lane = s.lane, nv = s.nv, ne = s.ne, nef = s.nef, nefc = s.nefc, bd = s.bd;
  const float snorm = sqrtf(search_dot);
  const float gtol = fmaxf(tolerance * ls_tolerance * snorm * scale, 1e-06f);
  float gq[2] = {0.0f, 0.0f};
#pragma unroll 1
  for (int i = lane; i < nv; i += 32) {
    gq[0] = fmaf(s.search[i], s.Ma[i] - s.qfs[i], gq[0]);
    gq[1] = fmaf(0.5f * s.search[i], s.mv[i], gq[1]);
  }
#pragma unroll 1
  for (int r = lane; r < ne; r += 32) {
    const float jvD = s.jv[r] * s.Dsm[r];
    gq[0] = fmaf(jvD, s.Jaref[r], gq[0]);
    gq[1] = fmaf(0.5f * s.jv[r], jvD, gq[1]);
  }
  ls_sum(gq, bd);
  const float q1 = gq[0], q2 = gq[1];
  const int ra = ne + lane, rb = ra + 32;
  const bool va = ra < nefc, vb = rb < nefc;
  // friction-loss rows are rare: without any (warp-uniform test) the rows are plain
  // inequalities and the short branch-free evaluation is used
  const bool fric = nef > ne;
  const bool more = ne + 64 < nefc;
  const Row rowa = make_row_ineq(va, va ? s.Dsm[ra] : 1.0f, va ? s.Jaref[ra] : 0.0f, va ? s.jv[ra] : 0.0f);
  const Row rowb = make_row_ineq(vb, vb ? s.Dsm[rb] : 1.0f, vb ? s.Jaref[rb] : 0.0f, vb ? s.jv[rb] : 0.0f);

  LineSearchResult out;
  out.alpha = 0.0f, out.improvement = 0.0f, out.noise_floor = 0.0f, out.converged = false, out.passes = 0;
  Vec3 p0 = v3(0.0f, 0.0f, 0.0f), lo = p0, hi = p0;
  float gtol_accept = 0.0f, lo_alpha = 0.0f, hi_alpha = 0.0f;
  float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f;  // step sizes of the coming pass
  // pass 0: alpha = 0; pass 1: first Newton step; pass >= 2: bracket iterations
#pragma unroll 1
  for (int pass = 0; pass < ls_iterations + 2; ++pass) {
    const bool absolute = pass == 0;
    out.passes = pass + 1;
    const Vec3 z3 = v3(0.0f, 0.0f, 0.0f);  // running sums start at zero
    Vec3 s0 = z3, s1 = z3, s2 = z3;
    if (!fric && !more) {
      s0 = (z3 + row_at_ineq(rowa, a0, absolute)) + row_at_ineq(rowb, a0, absolute);
      if (pass >= 2) {
        s1 = (z3 + row_at_ineq(rowa, a1, absolute)) + row_at_ineq(rowb, a1, absolute);
        s2 = (z3 + row_at_ineq(rowa, a2, absolute)) + row_at_ineq(rowb, a2, absolute);
      }
    } else {
      // general form, one step size at a time
      s0 = ls_rows_general(s.floss, s.Dsm, s.Jaref, s.jv, ne, nef, nefc, lane, a0, absolute);
      if (pass >= 2) {
        s1 = ls_rows_general(s.floss, s.Dsm, s.Jaref, s.jv, ne, nef, nefc, lane, a1, absolute);
        s2 = ls_rows_general(s.floss, s.Dsm, s.Jaref, s.jv, ne, nef, nefc, lane, a2, absolute);
      }
    }
    float q[9] = {s0.c0, s0.c1, s0.c2, s1.c0, s1.c1, s1.c2, s2.c0, s2.c1, s2.c2};
    if (pass >= 2) {
      ls_sum(q, bd);
    } else {
      float q3[3] = {q[0], q[1], q[2]};
      ls_sum(q3, bd);
      q[0] = q3[0], q[1] = q3[1], q[2] = q3[2];
    }
    if (pass == 0) {
      const Vec3 rows = v3(q[0], q[1], q[2]);
      p0 = v3(0.0f, q1, 2.0f * q2) + rows;
      const float q1_abs = sqrtf(2.0f * fmaxf(rows.c0, 0.0f) * fmaxf(rows.c2, 0.0f)) + fabsf(q1);
      gtol_accept = fmaxf(gtol, eps * q1_abs);
      out.noise_floor = eps * fmaxf(1.0f, safe_div(q1_abs, p0.c2));
      if (fabsf(p0.c1) < eps * q1_abs) {
        out.converged = true;
        break;
      }
      a0 = a1 = a2 = -safe_div(p0.c1, p0.c2);
      continue;
    }
    if (pass == 1) {
      const Vec3 lo_in = eval_quad(q1, q2, a0) + v3(q[0], q[1], q[2]);
      if (fabsf(lo_in.c1) < gtol_accept && lo_in.c0 < 0.0f) {
        out.converged = true;
        out.alpha = a0;
        out.improvement = -lo_in.c0;
        break;
      }
      const Vec3 p0_delta = v3(0.0f, p0.c1, p0.c2);
      const bool lo_less = lo_in.c1 < p0.c1;
      lo = lo_less ? lo_in : p0_delta;
      lo_alpha = lo_less ? a0 : 0.0f;
      hi = lo_less ? p0_delta : lo_in;
      hi_alpha = lo_less ? 0.0f : a0;
    } else {
      const Vec3 lo_next = eval_quad(q1, q2, a0) + v3(q[0], q[1], q[2]);
      const Vec3 hi_next = eval_quad(q1, q2, a1) + v3(q[3], q[4], q[5]);
      const Vec3 mid = eval_quad(q1, q2, a2) + v3(q[6], q[7], q[8]);
      const bool conv_lo = fabsf(lo_next.c1) < gtol_accept && lo_next.c0 < 0.0f;
      const bool conv_hi = fabsf(hi_next.c1) < gtol_accept && hi_next.c0 < 0.0f;
      const bool conv_mid = fabsf(mid.c1) < gtol_accept && mid.c0 < 0.0f;
      const bool converged = conv_lo || conv_hi || conv_mid;
      bool swap_lo = false, swap_hi = false;
      if (converged) {
        Vec3 best = v3(IMN_MJ_MAXVAL, 0.0f, 0.0f);
        float best_alpha = 0.0f;
        if (conv_lo && lo_next.c0 < best.c0) best = lo_next, best_alpha = a0;
        if (conv_hi && hi_next.c0 < best.c0) best = hi_next, best_alpha = a1;
        if (conv_mid && mid.c0 < best.c0) best = mid, best_alpha = a2;
        lo = hi = best;
        lo_alpha = hi_alpha = best_alpha;
      } else {
        // candidates in the order lo_next, mid, hi_next for the low end and
        // hi_next, mid, lo_next for the high end, each against the end as moved
        bool t;
        t = in_bracket(lo, lo_next);
        if (t) lo = lo_next, lo_alpha = a0;
        swap_lo |= t;
        t = in_bracket(lo, mid);
        if (t) lo = mid, lo_alpha = a2;
        swap_lo |= t;
        t = in_bracket(lo, hi_next);
        if (t) lo = hi_next, lo_alpha = a1;
        swap_lo |= t;
        t = in_bracket(hi, hi_next) || (hi.c1 < 0.0f && hi_next.c1 > 0.0f);
        if (t) hi = hi_next, hi_alpha = a1;
        swap_hi |= t;
        t = in_bracket(hi, mid);
        if (t) hi = mid, hi_alpha = a2;
        swap_hi |= t;
        t = in_bracket(hi, lo_next);
        if (t) hi = lo_next, hi_alpha = a0;
        swap_hi |= t;
      }
      const bool ls_done = converged || (!swap_lo && !swap_hi) ||
                           (lo.c0 < 0.0f && lo.c1 < 0.0f && lo.c1 > -gtol) ||
                           (hi.c0 < 0.0f && hi.c1 > 0.0f && hi.c1 < gtol);
      if (lo.c0 < 0.0f || hi.c0 < 0.0f) {
        const bool lo_better = lo.c0 < hi.c0;
        out.alpha = lo_better ? lo_alpha : hi_alpha;
        out.improvement = -(lo_better ? lo.c0 : hi.c0);
      }
      if (ls_done) {
        out.converged = true;
        break;
      }
    }
    // step sizes of the next bracket pass
    a0 = lo_alpha - safe_div(lo.c1, lo.c2);
    a1 = hi_alpha - safe_div(hi.c1, hi.c2);
    a2 = 0.5f * (lo_alpha + hi_alpha);
  }
  return out;
}

}  // namespace imn
