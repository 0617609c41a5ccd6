/*
 * oracle_common.h -- float32 helpers shared by the CPU oracle sources.
 * TEST INFRASTRUCTURE ONLY (see newton_oracle.c).
 */
#ifndef ORACLE_COMMON_H_
#define ORACLE_COMMON_H_

#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define MJ_MINVAL 1.0e-15f

/* RESTATED: upstream math.safe_div (call sites newton_stages.py:231-265). */
static inline float safe_div(float x, float y) { return x / (y != 0.0f ? y : MJ_MINVAL); }

/* Lane 0 of a 32-lane shuffle-down tree (offsets 16, 8, 4, 2, 1): the value a
 * warp's __shfl_down_sync reduction leaves in its first lane
 * (newton_stages.py:39-45). */
static inline float warp_tree(const float* v) {
  float s[32];
  for (int i = 0; i < 32; ++i) s[i] = v[i];
  for (int off = 16; off > 0; off >>= 1)
    for (int i = 0; i + off < 32; ++i)
      if (i < off) s[i] = s[i] + s[i + off];
  return s[0];
}

/* First-warp reduction of the line search: the tree, then one "+ 0" per later
 * warp of the logical block (newton_stages.py:46-49). */
static inline float block_sum32(const float* lanes, int nwarps) {
  float s = warp_tree(lanes);
  for (int w = 1; w < nwarps; ++w) s = s + 0.0f;
  return s;
}

/* Whole-block sum of one value per thread: per-warp trees, then the first
 * thread adds the later warps' partials in order (newton_stages.py:34-38). */
static inline float block_sum(const float* part, int bd) {
  float s = warp_tree(part);
  for (int w = 1; w < bd / 32; ++w) s = s + warp_tree(part + 32 * w);
  return s;
}

#endif /* ORACLE_COMMON_H_ */
