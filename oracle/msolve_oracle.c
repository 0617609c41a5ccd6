/*
 * msolve_oracle.c -- CPU restatement of the M-side factor + solve paths.
 *
 * TEST INFRASTRUCTURE ONLY (see newton_oracle.c).
 *
 *   tree L'DL       src/instantmimic/utils/mjw_kernels/tree_ldl.py:196-359 (the
 *                   serial CPU form of the generated code: every group's forward
 *                   pass, the trunk, every group's backward pass)
 *   blocked dense   src/instantmimic/utils/mjw_kernels/indexed_factor.py:15-173,
 *                   217-493 (gather through the block-major index table, upper
 *                   Cholesky, forward and backward substitution)
 *
 * Parity pins: the tree L'DL is PINNED bit for bit against the reference's own generated
 * CUDA code, compiled with nvcc and run on a B200 (oracle/ref_snippets.py,
 * tests/golden/ref_snippets.npz, tests/test_ref_snippets.py).  Both paths are also
 * checked against numpy.linalg.solve of the dense matrix
 * (the reference's own tests use the same pin, tests/test_tree_ldl.py:99-120 and
 * tests/test_blocked_dense_factor_solve.py:616-626).  PARITY UNPINNED at the bit
 * level for the blocked dense path: Warp's tile_cholesky / tile_matmul internal
 * summation orders are not visible; entries here subtract their inner products
 * in ascending order with fused multiply-adds.
 *
 * The tree oracle works from the PLAN (groups, trunk) and the CSR, not from the
 * product's compiled instruction list, so it also checks that compilation.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "oracle_common.h"

typedef struct TreeCtx {
  int nv, nM, G;
  const int *rowadr, *rownnz, *colind;
  const unsigned char* in_trunk;
  float *m, *s, *d, *x; /* per entry / per dof */
  float* am;            /* [G][nM] trunk matrix accumulators */
  float* as;            /* [G][nv] trunk solution accumulators */
} TreeCtx;

/* Leaves-first elimination of dof k plus its share of the L^-T y solve
 * (tree_ldl.py:215-232).  j < 0: trunk pass (targets are the trunk's own). */
static void eliminate(TreeCtx* t, int k, int j) {
  const int start = t->rowadr[k], count = t->rownnz[k] - 1;
  const float dk = 1.0f / t->m[start + count];
  t->d[k] = dk;
  for (int p = 0; p < count; ++p) {
    const int anc = t->colind[start + p];
    for (int q = 0; q <= p; ++q) {
      const int e = t->rowadr[anc] + q;
      float* dst = (j >= 0 && t->in_trunk[anc]) ? &t->am[(size_t)j * t->nM + e] : &t->m[e];
      *dst = fmaf(-(t->m[start + p] * t->m[start + q]), dk, *dst);
    }
  }
  for (int p = 0; p < count; ++p) t->m[start + p] = t->m[start + p] * dk;
  for (int p = 0; p < count; ++p) {
    const int anc = t->colind[start + p];
    float* dst = (j >= 0 && t->in_trunk[anc]) ? &t->as[(size_t)j * t->nv + anc] : &t->s[anc];
    *dst = fmaf(-t->m[start + p], t->s[k], *dst);
  }
}

/* x_k = s_k d_k - sum_p m_p x_anc(p)  (tree_ldl.py:258-266, 297-303).  The reference
 * writes "x = s * d; x = x - m0 * x0; x = x - m1 * x1; ..."; compiled with contraction
 * on, the first difference of two products fuses its LEFT product -- fma(s, d, -(m0 x0)),
 * the right product rounded on its own -- and every later term is fma(-m, x, acc).
 * Established against the reference's generated code run on a B200
 * (tests/golden/ref_snippets.npz). */
static float back_substitute(const TreeCtx* t, int k) {
  const int start = t->rowadr[k], count = t->rownnz[k] - 1;
  if (count == 0) return t->s[k] * t->d[k];
  float u = fmaf(t->s[k], t->d[k], -(t->m[start] * t->x[t->colind[start]]));
  for (int p = 1; p < count; ++p) u = fmaf(-t->m[start + p], t->x[t->colind[start + p]], u);
  return u;
}

int oracle_tree_ldl_solve(int nv, int nM, const int* rowadr, const int* rownnz, const int* colind,
                          int ngroups, const int* group_ptr, const int* group_nodes, int ntrunk,
                          const int* trunk, const float* M, int64_t M_ld, const float* y, int64_t y_ld,
                          float* x, int64_t x_ld, int nworld) {
  TreeCtx t;
  t.nv = nv, t.nM = nM, t.G = ngroups;
  t.rowadr = rowadr, t.rownnz = rownnz, t.colind = colind;
  unsigned char* in_trunk = (unsigned char*)calloc(nv, 1);
  for (int i = 0; i < ntrunk; ++i) in_trunk[trunk[i]] = 1;
  t.in_trunk = in_trunk;
  t.m = (float*)malloc(sizeof(float) * nM);
  t.s = (float*)malloc(sizeof(float) * nv);
  t.d = (float*)malloc(sizeof(float) * nv);
  t.x = (float*)malloc(sizeof(float) * nv);
  t.am = (float*)malloc(sizeof(float) * (size_t)ngroups * nM);
  t.as = (float*)malloc(sizeof(float) * (size_t)ngroups * nv);
  unsigned char* touched_m = (unsigned char*)malloc((size_t)ngroups * nM);
  unsigned char* touched_s = (unsigned char*)malloc((size_t)ngroups * nv);
  /* which trunk entries / dofs each group accumulates into (tree_ldl.py:236-245) */
  memset(touched_m, 0, (size_t)ngroups * nM);
  memset(touched_s, 0, (size_t)ngroups * nv);
  for (int j = 0; j < ngroups; ++j)
    for (int n = group_ptr[j]; n < group_ptr[j + 1]; ++n) {
      const int k = group_nodes[n];
      for (int p = 0; p < rownnz[k] - 1; ++p) {
        const int anc = colind[rowadr[k] + p];
        if (!in_trunk[anc]) continue;
        touched_s[(size_t)j * nv + anc] = 1;
        for (int q = 0; q <= p; ++q) touched_m[(size_t)j * nM + rowadr[anc] + q] = 1;
      }
    }
  for (int w = 0; w < nworld; ++w) {
    const float* Mr = M + (size_t)w * M_ld;
    const float* yr = y + (size_t)w * y_ld;
    float* xr = x + (size_t)w * x_ld;
    memset(t.am, 0, sizeof(float) * (size_t)ngroups * nM);
    memset(t.as, 0, sizeof(float) * (size_t)ngroups * nv);
    for (int j = 0; j < ngroups; ++j) {
      for (int n = group_ptr[j]; n < group_ptr[j + 1]; ++n) {
        const int k = group_nodes[n];
        for (int e = rowadr[k]; e < rowadr[k] + rownnz[k]; ++e) t.m[e] = Mr[e];
        t.s[k] = yr[k];
      }
      for (int n = group_ptr[j]; n < group_ptr[j + 1]; ++n) eliminate(&t, group_nodes[n], j);
    }
    /* trunk: own entries plus every group's contribution, in group order */
    for (int i = 0; i < ntrunk; ++i) {
      const int k = trunk[i];
      for (int e = rowadr[k]; e < rowadr[k] + rownnz[k]; ++e) {
        float v = Mr[e];
        for (int j = 0; j < ngroups; ++j)
          if (touched_m[(size_t)j * nM + e]) v = v + t.am[(size_t)j * nM + e];
        t.m[e] = v;
      }
      float u = yr[k];
      for (int j = 0; j < ngroups; ++j)
        if (touched_s[(size_t)j * nv + k]) u = u + t.as[(size_t)j * nv + k];
      t.s[k] = u;
    }
    for (int i = ntrunk - 1; i >= 0; --i) eliminate(&t, trunk[i], -1);
    for (int i = 0; i < ntrunk; ++i) {
      const int k = trunk[i];
      const float u = back_substitute(&t, k);
      t.x[k] = u;
      xr[k] = u;
    }
    for (int j = 0; j < ngroups; ++j)
      for (int n = group_ptr[j + 1] - 1; n >= group_ptr[j]; --n) {
        const int k = group_nodes[n];
        const float u = back_substitute(&t, k);
        t.x[k] = u;
        xr[k] = u;
      }
  }
  free(in_trunk), free(t.m), free(t.s), free(t.d), free(t.x), free(t.am), free(t.as);
  free(touched_m), free(touched_s);
  return 0;
}

/* Blocked dense Cholesky of M gathered through `indices` (block-major
 * (nblk, nblk, 16, 16); index nM = zero), identity on the padded diagonal.
 * mode 0: factor + solve; mode 1: solve with the stored U.  y, x: (W, nv, rhs). */
int oracle_blocked_dense_factor_solve(int nv, int pad, int nM, const int* indices, const float* identity,
                                      const float* M, int64_t M_ld, const float* y, float* U, float* x,
                                      const int* active, int nworld, int rhs, int mode) {
  const int nblk = pad / 16;
  float* A = (float*)malloc(sizeof(float) * pad * pad);
  float* dinv = (float*)malloc(sizeof(float) * pad);
  float* B = (float*)malloc(sizeof(float) * pad * rhs);
  for (int w = 0; w < nworld; ++w) {
    if (active && active[w] == 0) continue;
    float* Uw = U + (size_t)w * pad * pad;
    if (mode == 0) {
      const float* Mw = M + (size_t)w * M_ld;
      for (int kb = 0; kb < nblk; ++kb)
        for (int ib = 0; ib < nblk; ++ib)
          for (int r = 0; r < 16; ++r)
            for (int c = 0; c < 16; ++c) {
              const int idx = indices[((kb * nblk + ib) * 16 + r) * 16 + c];
              float v = idx < nM ? Mw[idx] : 0.0f;
              if (kb == ib && 16 * (kb + 1) > nv) v += identity[r * 16 + c];
              A[(16 * kb + r) * pad + 16 * ib + c] = v;
            }
      for (int r = 0; r < pad; ++r) {
        float acc = A[r * pad + r];
        for (int t = 0; t < r; ++t) acc = fmaf(-A[t * pad + r], A[t * pad + r], acc);
        const float dg = sqrtf(acc), rinv = 1.0f / dg;
        A[r * pad + r] = dg;
        dinv[r] = rinv;
        for (int c = r + 1; c < pad; ++c) {
          acc = A[r * pad + c];
          for (int t = 0; t < r; ++t) acc = fmaf(-A[t * pad + r], A[t * pad + c], acc);
          A[r * pad + c] = acc * rinv;
        }
      }
      for (int r = 0; r < pad; ++r)
        for (int c = 0; c < pad; ++c) Uw[r * pad + c] = c >= r ? A[r * pad + c] : 0.0f;
    } else {
      memcpy(A, Uw, sizeof(float) * pad * pad);
      for (int r = 0; r < pad; ++r) dinv[r] = 1.0f / A[r * pad + r];
    }
    const float* yw = y + (size_t)w * nv * rhs;
    for (int q = 0; q < pad * rhs; ++q) B[q] = q < nv * rhs ? yw[q] : 0.0f;
    for (int q = 0; q < rhs; ++q) {
      for (int r = 0; r < pad; ++r) {
        float acc = B[r * rhs + q];
        for (int t = 0; t < r; ++t) acc = fmaf(-A[t * pad + r], B[t * rhs + q], acc);
        B[r * rhs + q] = acc * dinv[r];
      }
      for (int r = pad - 1; r >= 0; --r) {
        const int b1 = (r / 16 + 1) * 16;
        float acc = B[r * rhs + q];
        for (int c = b1; c < pad; ++c) acc = fmaf(-A[r * pad + c], B[c * rhs + q], acc);
        for (int c = b1 - 1; c > r; --c) acc = fmaf(-A[r * pad + c], B[c * rhs + q], acc);
        B[r * rhs + q] = acc * dinv[r];
      }
    }
    float* xw = x + (size_t)w * nv * rhs;
    for (int q = 0; q < nv * rhs; ++q) xw[q] = B[q];
  }
  free(A), free(dinv), free(B);
  return 0;
}
