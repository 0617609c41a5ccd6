// imn_newton_factor.cuh -- upper Cholesky H = U^T U of one world with the
// right-hand side carried as one more column (forward solve), then the back
// substitution (reference: newton_stages.py:546-609).
//
// Storage: A is (nv+1) x ldu in shared memory.  U[r][c] (r <= c <= nv; column nv
// is the carried right-hand side) lives at A[r*ldu + c]; H[r][c] (r <= c < nv)
// at A[(c+1)*ldu + r], so H survives the factorisation for the next incremental
// update.  dinv[r] = 1 / U[r][r].
//
// Order of operations (identical to the CPU oracle): every entry starts from H
// (or grad) and subtracts U[t][r] * U[t][c] for t = 0, 1, ... with fused
// multiply-adds; the pivot is sqrtf; the row is scaled by the reciprocal pivot.
//
// Mapping: 16 rows at a time.  A lane owns up to three columns c = b0 + lane +
// 32k and keeps the block's 16 running sums of each in registers.  Phase 1 adds
// the terms of all earlier rows (one shared-memory read of U[t][c] and four
// 128-bit broadcast reads of U[t][b0..b0+15] feed 16 fused multiply-adds).
// Phase 2 eliminates the block's rows one by one with warp shuffles: the pivot
// row's entry of column b0+j is in lane j, so no shared-memory round trip and no
// barrier separates the 16 steps.  The register file is shifted by one row per
// step so that the loop body is the same code for every row.
#pragma once

#include "imn_newton_linalg.cuh"

namespace imn {

__device__ __forceinline__ void factor_solve(const World& s, bool factor, float& sum0, float& sum1) {
  const int lane = s.lane, nv = s.nv, ldu = s.ldu;
  float* A = s.A;
  if (factor) {
#pragma unroll 1
    for (int b0 = 0; b0 < nv; b0 += 16) {
      const int nr = min(16, nv - b0);
      const int ng = (nr + 3) >> 2;
      float acc[3][16];
      int cc[3];
      bool act[3], valid[3];
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        const int c = b0 + lane + 32 * k;
        act[k] = b0 + 32 * k <= nv;  // warp-uniform: the slot holds at least one column
        valid[k] = c <= nv;
        cc[k] = valid[k] ? c : nv;
        if (act[k]) {
          // H column cc (rows b0..), or grad for the carried column; rows below the
          // diagonal hold values that are never stored or read by another lane
          const float* src = (cc[k] < nv ? A + (cc[k] + 1) * ldu : s.grad) + b0;
#pragma unroll
          for (int gi = 0; gi < 4; ++gi) {
            float4 h = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (gi < ng) h = *reinterpret_cast<const float4*>(src + 4 * gi);
            acc[k][4 * gi] = h.x, acc[k][4 * gi + 1] = h.y, acc[k][4 * gi + 2] = h.z, acc[k][4 * gi + 3] = h.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[k][i] = 0.0f;
        }
      }
      // phase 1: terms of rows t < b0
#pragma unroll 1
      for (int t = 0; t < b0; ++t) {
        const float* Ut = A + t * ldu;
        float ur[16];
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
          float4 u = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          if (gi < ng) u = *reinterpret_cast<const float4*>(Ut + b0 + 4 * gi);
          ur[4 * gi] = u.x, ur[4 * gi + 1] = u.y, ur[4 * gi + 2] = u.z, ur[4 * gi + 3] = u.w;
        }
#pragma unroll
        for (int k = 0; k < 3; ++k)
          if (act[k]) {
            const float uc = Ut[cc[k]];
#pragma unroll
            for (int gi = 0; gi < 4; ++gi)
              if (gi < ng) {  // warp-uniform: a short last block skips its absent rows
#pragma unroll
                for (int i = 4 * gi; i < 4 * gi + 4; ++i) acc[k][i] = fmaf(-ur[i], uc, acc[k][i]);
              }
          }
      }
      IMN_MARK(s, 12);
      // phase 2: eliminate the block's rows; acc[k][0] is always the current row
#pragma unroll 1
      for (int r = 0; r < nr; ++r) {
        const float pv = __shfl_sync(IMN_FULL_MASK, acc[0][0], r);
        const float dg = sqrtf(pv);
        const float rinv = 1.0f / dg;
        float u[3];
        float* Ur = A + (b0 + r) * ldu;
#pragma unroll
        for (int k = 0; k < 3; ++k)
          if (act[k]) {
            u[k] = acc[k][0] * rinv;
            if (k == 0 && lane == r) u[k] = dg;
            if (valid[k] && cc[k] >= b0 + r) Ur[cc[k]] = u[k];
          }
        if (lane == 0) s.dinv[b0 + r] = rinv;
        float um[16];  // um[j] = U[b0+r][b0+r+j], held by lane r+j
#pragma unroll
        for (int j = 1; j < 16; ++j) um[j] = __shfl_sync(IMN_FULL_MASK, u[0], (r + j) & 31);
#pragma unroll
        for (int k = 0; k < 3; ++k)
          if (act[k]) {
#pragma unroll
            for (int j = 1; j < 16; ++j) acc[k][j - 1] = fmaf(-um[j], u[k], acc[k][j]);
            acc[k][15] = 0.0f;
          }
      }
      __syncwarp();
      IMN_MARK(s, 13);
    }
  } else {
    // forward substitution with the stored factor: unknown r receives its terms
    // in ascending order, exactly as the carried column of the factorisation
#pragma unroll 1
    for (int i = lane; i < nv; i += 32) s.xsm[i] = s.grad[i];
    __syncwarp();
#pragma unroll 1
    for (int t = 0; t < nv; ++t) {
      const float yt = s.xsm[t] * s.dinv[t];
      const float* Ut = A + t * ldu;
      __syncwarp();
#pragma unroll 1
      for (int r = t + 1 + lane; r < nv; r += 32) s.xsm[r] = fmaf(-Ut[r], yt, s.xsm[r]);
      if (lane == 0) A[t * ldu + nv] = yt;
      __syncwarp();
    }
  }
  // back substitution, 16-row blocks from the last: later blocks' columns in
  // ascending order first, then the block's own columns from its last inwards
#pragma unroll 1
  for (int b0 = ((nv - 1) / 16) * 16; b0 >= 0; b0 -= 16) {
    const int b1 = min(b0 + 16, nv);
    const int r = b0 + lane;
    const float* Ur = A + r * ldu;
    float acc = 0.0f, di = 0.0f;
    if (r < b1) {
      acc = Ur[nv];
      di = s.dinv[r];
#pragma unroll 2
      for (int c = b1; c < nv; ++c) acc = fmaf(-Ur[c], s.xsm[c], acc);
    }
#pragma unroll 1
    for (int c = b1 - 1; c >= b0; --c) {
      const float xc = __shfl_sync(IMN_FULL_MASK, acc * di, c - b0);
      if (r < c) acc = fmaf(-Ur[c], xc, acc);
      if (lane == 0) s.xsm[c] = xc;
    }
    __syncwarp();
  }
  IMN_MARK(s, 14);
  sum0 = logical_block_sum(nv, s.bd, lane, [&](int i, float a) { return fmaf(s.xsm[i], s.xsm[i], a); });
  sum1 = logical_block_sum(nv, s.bd, lane, [&](int i, float a) { return fmaf(s.grad[i], s.xsm[i], a); });
#pragma unroll 1
  for (int i = lane; i < nv; i += 32) s.search[i] = -s.xsm[i];
  __syncwarp();
  IMN_MARK(s, 15);
}

}  // namespace imn
