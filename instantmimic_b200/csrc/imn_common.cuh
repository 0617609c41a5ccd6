// imn_common.cuh -- helpers shared by the sm_100a kernels.
//
// Rounding contract: the translation units are compiled with -fmad=false, so a
// multiply followed by an add stays two roundings unless the source says
// fmaf(); sqrtf and '/' are the IEEE-rounded forms (nvcc defaults
// -prec-sqrt=true -prec-div=true, no fast-math).  Lane reductions follow a
// 32-lane shuffle-down tree whose lane-0 value is broadcast.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/imnewton.h"

#define IMN_FULL_MASK 0xFFFFFFFFu
#define IMN_MJ_MINVAL 1.0e-15f
#define IMN_MJ_MAXVAL 1.0e10f

namespace imn {

void set_error(const char* fmt, ...);

__device__ __forceinline__ float safe_div(float x, float y) {
  return x / (y != 0.0f ? y : IMN_MJ_MINVAL);
}

// Jaref + alpha * jv with both roundings kept (newton_stages.py:18-19).
__device__ __forceinline__ float rounded_step(float a, float b, float c) {
  return __fadd_rn(a, __fmul_rn(b, c));
}

// Lane 0 of the shuffle-down tree, broadcast to the warp
// (newton_stages.py:39-45).
__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = v + __shfl_down_sync(IMN_FULL_MASK, v, off);
  return __shfl_sync(IMN_FULL_MASK, v, 0);
}

struct Vec3 {
  float c0, c1, c2;
};
__device__ __forceinline__ Vec3 v3(float a, float b, float c) { return Vec3{a, b, c}; }
__device__ __forceinline__ Vec3 operator+(Vec3 a, Vec3 b) {
  return Vec3{a.c0 + b.c0, a.c1 + b.c1, a.c2 + b.c2};
}
__device__ __forceinline__ Vec3 warp_tree_sum(Vec3 v) {
  return Vec3{warp_tree_sum(v.c0), warp_tree_sum(v.c1), warp_tree_sum(v.c2)};
}

}  // namespace imn
