/*
 * sparse_oracle.c -- CPU restatement of the static-pattern sparse L'DL of the
 * Newton Hessian.  TEST INFRASTRUCTURE ONLY (see newton_oracle.c).
 *
 * Follows the numeric bodies the reference generates in
 * src/instantmimic/utils/mjw_kernels/sparse_hessian.py:
 *   level factor with lane teams        :410-452
 *   backward solve, search, sums        :453-480
 *   forward solve with a stored factor  :528-544
 *   initial assembly on pattern slots   :571-637
 *   incremental update of packed H      :501-527
 *   non-fused gather / reload           :651-676
 * PINNED bit for bit against that generated CUDA code, compiled with nvcc and run on a
 * B200 (oracle/ref_snippets.py, tests/golden/ref_snippets.npz, tests/test_ref_snippets.py):
 * initial assembly, update with flipped rows, solve with the resident factor, non-fused
 * factor and solve-only call, on four models.
 * Entries hold N = L D; an entry's terms are summed by a team of T lanes (lane tl
 * takes elements tl, tl+T, ... of every run) and joined by a shuffle-down tree of
 * width T, which this file reproduces lane by lane.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/imnewton.h"
#include "oracle_common.h"
#include "sparse_oracle.h"

void sparse_factor_levels(const ImnSparsePlan* P, float* N, float* iD) {
  for (int l = 0; l < P->nlevels; ++l) {
    const int T = P->lvl_team[l];
    for (int e = P->lvl_ptr[l]; e < P->lvl_ptr[l + 1]; ++e) {
      float part[32];
      for (int i = 0; i < T; ++i) part[i] = 0.0f;
      for (int r = P->run_ptr[e]; r < P->run_ptr[e + 1]; ++r) {
        const uint32_t ab = P->run_ab[r], kl = P->run_kl[r];
        const float* pa = N + (ab & 0xFFFFu);
        const float* pb = N + (ab >> 16);
        const float* pd = iD + (kl & 0xFFFFu);
        const int len = (int)(kl >> 16);
        for (int tl = 0; tl < T; ++tl)
          for (int t = tl; t < len; t += T) part[tl] = fmaf(pa[t] * pb[t], pd[t], part[tl]);
      }
      for (int off = T >> 1; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) part[i] = part[i] + part[i + off];
      const int sl = P->ent_slot[e], col = P->ent_col[e];
      const float w = N[sl] - part[0];
      N[sl] = w;
      if (col >= 0) iD[col] = 1.0f / w;
    }
  }
}

void sparse_load_rhs(const ImnSparsePlan* P, float* N, const float* grad) {
  for (int j = 0; j < P->nv; ++j) N[P->nfac + j] = grad[P->orig[j]];
}

void sparse_forward(const ImnSparsePlan* P, float* N, const float* iD, const float* grad) {
  const int rhs = P->nfac;
  for (int l = 0; l < P->nlevels; ++l)
    for (int q = P->f_lvl[l]; q < P->f_lvl[l + 1]; ++q) {
      const int j = P->f_row[q];
      float v = grad[P->orig[j]];
      const float* rowp = N + P->row_start[j];
      const int k0 = P->rk_ptr[j];
      for (int t = 0; t < P->rk_ptr[j + 1] - k0; ++t) {
        const int k = P->rk[k0 + t];
        v = fmaf(-(rowp[t] * iD[k]), N[rhs + k], v);
      }
      N[rhs + j] = v;
    }
}

void sparse_backward(const ImnSparsePlan* P, float* N, const float* iD, const float* grad, float* search,
                     int bd, float sums[2]) {
  const int rhs = P->nfac, n = P->nv;
  for (int l = 0; l < P->nlevels; ++l)
    for (int p = P->b_lvl[l]; p < P->b_lvl[l + 1]; ++p) {
      const int i = P->b_src[p], j = P->b_dst[p];
      N[rhs + j] = fmaf(-N[P->b_slot[p]], N[rhs + i] * iD[i], N[rhs + j]);
    }
  float p0[128], p1[128];
  for (int t = 0; t < bd; ++t) {
    float s0 = 0.0f, s1 = 0.0f;
    for (int j = t; j < n; j += bd) {
      const int d = P->orig[j];
      const float v = N[rhs + j] * iD[j];
      search[d] = -v;
      s0 = fmaf(v, v, s0);
      s1 = fmaf(grad[d], v, s1);
    }
    p0[t] = s0, p1[t] = s1;
  }
  float ra = 0.0f, rb = 0.0f;
  for (int w = 0; w < bd / 32; ++w) {
    ra = ra + warp_tree(p0 + 32 * w);
    rb = rb + warp_tree(p1 + 32 * w);
  }
  sums[0] = ra, sums[1] = rb;
}

int sparse_assemble(const ImnSparsePlan* P, float* N, const float* M, const float* J, int ldj,
                    const float* D, const int* state, int nefc) {
  const int nv = P->nv, words = (nv + 31) / 32;
  int violations = 0;
  for (int s = 0; s < P->nfac; ++s) N[s] = P->s_m[s] >= 0 ? M[P->s_m[s]] : 0.0f;
  for (int r = 0; r < nefc; ++r) {
    if (state[r] != IMN_STATE_QUADRATIC || D[r] == 0.0f) continue;
    /* the row's dof support must lie inside the pattern */
    uint32_t rm[4] = {0, 0, 0, 0};
    for (int d = 0; d < nv; ++d)
      if (J[(size_t)r * ldj + d] != 0.0f) rm[d >> 5] |= 1u << (d & 31);
    int bad = 0;
    for (int d = 0; d < nv && !bad; ++d)
      if ((rm[d >> 5] >> (d & 31)) & 1u)
        for (int p = 0; p < words; ++p) bad |= (rm[p] & ~P->pmask[d * words + p]) != 0u;
    violations += bad;
  }
  for (int s = 0; s < P->nfac; ++s) {
    const int a = P->s_a[s], b = P->s_b[s];
    float v = N[s];
    for (int r = 0; r < nefc; ++r)
      if (state[r] == IMN_STATE_QUADRATIC) v = fmaf(J[(size_t)r * ldj + a] * D[r], J[(size_t)r * ldj + b], v);
    N[s] = v;
  }
  return violations;
}

int sparse_update(const ImnSparsePlan* P, float* Hp, const float* J, int ldj, const float* D, const int* state,
                  const int* ids, int count, const int* uni, int n) {
  const int nv = P->nv;
  int violations = 0;
  for (int cj = 0; cj < n; ++cj)
    for (int ri = 0; ri <= cj; ++ri) {
      const int row = uni[ri], col = uni[cj];
      float delta = 0.0f;
      for (int t = 0; t < count; ++t) {
        const int r = ids[t];
        const float a = J[(size_t)r * ldj + row], b = J[(size_t)r * ldj + col];
        float da = D[r] * a;
        if (state[r] != IMN_STATE_QUADRATIC) da = -da;
        if (a != 0.0f && b != 0.0f) delta = fmaf(da, b, delta);
      }
      if (delta != 0.0f) {
        const int sl = P->pair[row * nv + col];
        if (sl >= 0)
          Hp[sl] = Hp[sl] + delta;
        else
          ++violations;
      }
    }
  return violations;
}

/* Sparse factor of the non-fused iteration (sparse_hessian.py:849-894): mode 4
 * gathers the dense H and factors, mode 5 solves with the stored factor.
 * hfactor: [0, nfac) N, [nfac, nfac + nv) 1/D. */
int oracle_sparse_factor_nonfused(const ImnSparsePlan* P, const uint8_t* done, const float* grad,
                                  int64_t grad_ld, const float* h, const int32_t* quad_changed,
                                  const int32_t* state_changed, float* hfactor, float* search,
                                  int64_t search_ld, float* search_dot, float* decrement, int nworld,
                                  int skip_unchanged, int skip_noflip) {
  const int P2 = P->nv_pad * P->nv_pad, nfac = P->nfac, n = P->nv;
  float* N = (float*)malloc(sizeof(float) * P->nslots);
  float* iD = (float*)malloc(sizeof(float) * n);
  for (int w = 0; w < nworld; ++w) {
    if (done && done[w]) continue;
    if (skip_noflip && state_changed[w] == 0) continue;
    const int mode = (skip_unchanged && quad_changed[w] == 0) ? 5 : 4;
    const float* g = grad + (size_t)w * grad_ld;
    float* Uf = hfactor + (size_t)w * P2;
    if (mode == 4) {
      const float* Hd = h + (size_t)w * P2;
      for (int s = 0; s < nfac; ++s) N[s] = Hd[P->gat[s]];
      sparse_load_rhs(P, N, g);
      sparse_factor_levels(P, N, iD);
      for (int s = 0; s < nfac; ++s) Uf[s] = N[s];
      for (int j = 0; j < n; ++j) Uf[nfac + j] = iD[j];
    } else {
      for (int s = 0; s < nfac; ++s) N[s] = Uf[s];
      for (int j = 0; j < n; ++j) iD[j] = Uf[nfac + j];
      sparse_forward(P, N, iD, g);
    }
    float sums[2];
    sparse_backward(P, N, iD, g, search + (size_t)w * search_ld, P->block, sums);
    search_dot[w] = sums[0];
    decrement[w] = sums[1];
  }
  free(N), free(iD);
  return 0;
}

/* One stage of the fused path per world, for stage-level checks against the reference's
 * own generated code (sparse_hessian.py:483-547 factor_snippet, :571-637 init_snippet):
 *   stage 0  incremental update of the packed H in U with the flipped rows `ids` over
 *            the dof union `uni`, refactor, solve;
 *   stage 1  the factor is reloaded from U (the reference's mode 2), forward solve with
 *            it (mode 1), solve;
 *   stage 3  initial assembly H = M + J'DJ on the pattern, factor, solve; U receives
 *            packed H | N | 1/D.
 * J (W, njmax, nv), D / state / ids (W, njmax), uni (W, nv + 1), M (W, nM), grad
 * (W, grad_ld), U (W, P, P), search (W, nv).  The violation counter in U's last element
 * counts as in the kernels. */
int oracle_sparse_stage(const ImnSparsePlan* P, int stage, const float* J, int njmax, const float* D,
                        const int32_t* state, const int32_t* nefc, const float* M, int nM, const int32_t* ids,
                        const int32_t* count, const int32_t* uni, const float* grad, int64_t grad_ld, float* U,
                        float* search, float* search_dot, float* decrement, int nworld) {
  const int P2 = P->nv_pad * P->nv_pad, nfac = P->nfac, n = P->nv;
  float* N = (float*)malloc(sizeof(float) * P->nslots);
  float* iD = (float*)malloc(sizeof(float) * n);
  for (int w = 0; w < nworld; ++w) {
    const float* g = grad + (size_t)w * grad_ld;
    const float* Jw = J ? J + (size_t)w * njmax * n : NULL;
    const float* Dw = D ? D + (size_t)w * njmax : NULL;
    const int32_t* sw = state ? state + (size_t)w * njmax : NULL;
    float* Uf = U + (size_t)w * P2;
    if (stage == 3) {
      const int rows = nefc[w] < njmax ? nefc[w] : njmax;
      const int bad = sparse_assemble(P, N, M + (size_t)w * nM, Jw, n, Dw, sw, rows);
      Uf[P2 - 1] += (float)bad;
      for (int s = 0; s < nfac; ++s) Uf[s] = N[s];
      sparse_load_rhs(P, N, g);
      sparse_factor_levels(P, N, iD);
      for (int s = 0; s < nfac; ++s) Uf[nfac + s] = N[s];
      for (int j = 0; j < n; ++j) Uf[2 * nfac + j] = iD[j];
    } else if (stage == 0) {
      const int32_t* u = uni + (size_t)w * (n + 1);
      const int bad = sparse_update(P, Uf, Jw, n, Dw, sw, ids + (size_t)w * njmax, count[w], u, u[n]);
      Uf[P2 - 1] += (float)bad;
      for (int s = 0; s < nfac; ++s) N[s] = Uf[s];
      sparse_load_rhs(P, N, g);
      sparse_factor_levels(P, N, iD);
    } else {
      for (int s = 0; s < nfac; ++s) N[s] = Uf[nfac + s];
      for (int j = 0; j < n; ++j) iD[j] = Uf[2 * nfac + j];
      sparse_forward(P, N, iD, g);
    }
    float sums[2];
    sparse_backward(P, N, iD, g, search + (size_t)w * n, P->block, sums);
    search_dot[w] = sums[0];
    decrement[w] = sums[1];
  }
  free(N), free(iD);
  return 0;
}
