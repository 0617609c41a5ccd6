// imn_msolve.cu -- factor + solve of inertia-like matrices (M and M - h qDeriv):
// the tree-structured L'DL and the blocked dense Cholesky.
//
// Tree L'DL (reference: tree_ldl.py:196-359, 419-433).  The reference generates
// straight-line source per model; here one kernel interprets the plan's
// instruction list.  A block serves 32 worlds with one warp per group; lane l of
// every warp works on world 32*block + l, all operands of a world live in column
// l of a [slot][32] shared-memory array (bank = lane, so no conflicts), every
// lane of a warp executes the same instruction on its own world, and the only
// synchronisation is the pair of block barriers around the trunk.
//
// Blocked dense Cholesky (reference: indexed_factor.py:15-173, 217-493).  One warp
// per world gathers M through the plan's block-major index table into shared
// memory, factors it (same entry formula as the Newton Hessian factor), carries
// `rhs_count` right-hand sides through the forward and backward substitution and
// stores U (pad x pad, upper) in the caller's workspace.
#include "imn_common.cuh"

namespace imn {

enum { OP_LOAD_M, OP_LOAD_Y, OP_ZERO, OP_INV, OP_UPD, OP_SCALE, OP_SUBMUL, OP_MUL, OP_ADD, OP_STORE_X };

__device__ __forceinline__ void tree_run(const int4* __restrict__ prog, int lo, int hi, float* col,
                                         const float* __restrict__ Mr, const float* __restrict__ yr,
                                         float* __restrict__ xr, bool live) {
#pragma unroll 1
  for (int pc = lo; pc < hi; ++pc) {
    const int4 ins = __ldg(prog + pc);
    const int dst = ins.y, a = ins.z & 0xFFFF, b = (ins.z >> 16) & 0xFFFF, c = ins.w;
    switch (ins.x) {
      case OP_LOAD_M: col[dst * 32] = Mr[a]; break;
      case OP_LOAD_Y: col[dst * 32] = yr[a]; break;
      case OP_ZERO: col[dst * 32] = 0.0f; break;
      case OP_INV: col[dst * 32] = 1.0f / col[a * 32]; break;
      case OP_UPD: col[dst * 32] = fmaf(-(col[a * 32] * col[b * 32]), col[c * 32], col[dst * 32]); break;
      case OP_SCALE: col[dst * 32] = col[dst * 32] * col[a * 32]; break;
      case OP_SUBMUL: col[dst * 32] = fmaf(-col[a * 32], col[b * 32], col[dst * 32]); break;
      case OP_MUL: col[dst * 32] = col[a * 32] * col[b * 32]; break;
      case OP_ADD: col[dst * 32] = col[dst * 32] + col[a * 32]; break;
      case OP_STORE_X:
        if (live) xr[dst] = col[a * 32];
        break;
      default: break;
    }
  }
}

__global__ void tree_ldl_kernel(const int4* __restrict__ prog, const int* __restrict__ ptr, int groups,
                                int owner, const float* __restrict__ M, int64_t M_ld,
                                const float* __restrict__ y, int64_t y_ld, float* __restrict__ x,
                                int64_t x_ld, int nworld) {
  extern __shared__ float slots[];  // [nslot][32]
  const int lw = threadIdx.x & 31, part = threadIdx.x >> 5;
  const int world = blockIdx.x * 32 + lw;
  const bool live = world < nworld;
  const int src = live ? world : nworld - 1;
  const float* Mr = M + (size_t)src * M_ld;
  const float* yr = y + (size_t)src * y_ld;
  float* xr = x + (size_t)src * x_ld;
  float* col = slots + lw;
  // streams: forward_0..forward_{G-1}, trunk, backward_0..backward_{G-1}
  tree_run(prog, ptr[part], ptr[part + 1], col, Mr, yr, xr, live);
  __syncthreads();
  if (part == owner) tree_run(prog, ptr[groups], ptr[groups + 1], col, Mr, yr, xr, live);
  __syncthreads();
  tree_run(prog, ptr[groups + 1 + part], ptr[groups + 2 + part], col, Mr, yr, xr, live);
}

// ---- blocked dense Cholesky ------------------------------------------------------
__global__ void __launch_bounds__(32) blocked_dense_kernel(const int nv, const int pad, const int nM,
                                                           const int* __restrict__ indices,
                                                           const float* __restrict__ identity,
                                                           const float* __restrict__ M, const int64_t M_ld,
                                                           const float* __restrict__ y, float* __restrict__ Ug,
                                                           float* __restrict__ x,
                                                           const int* __restrict__ active, const int rhs,
                                                           const int mode) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x, w = blockIdx.x;
  if (active && active[w] == 0) return;
  const int ld = pad | 1;
  float* U = sm;                 // pad x ld, upper triangle
  float* dinv = U + pad * ld;    // pad
  float* B = dinv + pad;         // pad x rhs right-hand sides / solutions
  float* Uw = Ug + (size_t)w * pad * pad;
  const int nblk = pad >> 4;
  if (mode == 0) {
    // gather: table entry ((kb*nblk + ib)*16 + r)*16 + c addresses M's value of
    // (16 kb + r, 16 ib + c); index nM is the extra zero slot; the padded diagonal
    // of the last block gets the identity
    const float* Mw = M + (size_t)w * M_ld;
    for (int q = lane; q < pad * pad; q += 32) {
      const int c = q & 15, r = (q >> 4) & 15, blk = q >> 8;
      const int ib = blk % nblk, kb = blk / nblk;
      const int idx = indices[q];
      float v = idx < nM ? Mw[idx] : 0.0f;
      if (kb == ib && 16 * (kb + 1) > nv) v += identity[(r << 4) | c];
      U[(16 * kb + r) * ld + 16 * ib + c] = v;
    }
    __syncwarp();
    for (int r = 0; r < pad; ++r) {
      float dg = 0.0f;
      for (int c = r + lane; c < pad; c += 32) {
        float a = U[r * ld + c];
        for (int t = 0; t < r; ++t) a = fmaf(-U[t * ld + r], U[t * ld + c], a);
        U[r * ld + c] = a;
        if (c == r) dg = sqrtf(a);
      }
      dg = __shfl_sync(IMN_FULL_MASK, dg, 0);
      const float rinv = 1.0f / dg;
      for (int c = r + lane; c < pad; c += 32) U[r * ld + c] = (c == r) ? dg : U[r * ld + c] * rinv;
      if (lane == 0) dinv[r] = rinv;
      __syncwarp();
    }
    for (int q = lane; q < pad * pad; q += 32) {
      const int r = q / pad, c = q - r * pad;
      Uw[q] = c >= r ? U[r * ld + c] : 0.0f;
    }
  } else {
    for (int q = lane; q < pad * pad; q += 32) {
      const int r = q / pad, c = q - r * pad;
      U[r * ld + c] = Uw[q];
    }
    __syncwarp();
    for (int r = lane; r < pad; r += 32) dinv[r] = 1.0f / U[r * ld + r];
  }
  // right-hand sides: rows nv..pad-1 are zero
  const float* yw = y + (size_t)w * nv * rhs;
  for (int q = lane; q < pad * rhs; q += 32) B[q] = q < nv * rhs ? yw[q] : 0.0f;
  __syncwarp();
  // forward substitution: unknown r receives its terms in ascending order
  for (int t = 0; t < pad; ++t) {
    const float di = dinv[t];
    for (int q = lane; q < rhs; q += 32) B[t * rhs + q] = B[t * rhs + q] * di;
    __syncwarp();
    for (int e = lane; e < (pad - t - 1) * rhs; e += 32) {
      const int r = t + 1 + e / rhs, q = e % rhs;
      B[r * rhs + q] = fmaf(-U[t * ld + r], B[t * rhs + q], B[r * rhs + q]);
    }
    __syncwarp();
  }
  // back substitution in 16-row blocks from the last: later blocks' columns first
  // (ascending), then the block's own columns from its last inwards
  for (int b0 = pad - 16; b0 >= 0; b0 -= 16) {
    const int b1 = b0 + 16;
    for (int e = lane; e < 16 * rhs; e += 32) {
      const int r = b0 + e / rhs, q = e % rhs;
      float acc = B[r * rhs + q];
      for (int c = b1; c < pad; ++c) acc = fmaf(-U[r * ld + c], B[c * rhs + q], acc);
      B[r * rhs + q] = acc;
    }
    __syncwarp();
    for (int c = b1 - 1; c >= b0; --c) {
      const float di = dinv[c];
      for (int q = lane; q < rhs; q += 32) B[c * rhs + q] = B[c * rhs + q] * di;
      __syncwarp();
      for (int e = lane; e < (c - b0) * rhs; e += 32) {
        const int r = b0 + e / rhs, q = e % rhs;
        B[r * rhs + q] = fmaf(-U[r * ld + c], B[c * rhs + q], B[r * rhs + q]);
      }
      __syncwarp();
    }
  }
  float* xw = x + (size_t)w * nv * rhs;
  for (int q = lane; q < nv * rhs; q += 32) xw[q] = B[q];
}

}  // namespace imn

extern "C" int imn_tree_ldl_solve(const ImnTreePlan* plan, const float* M, int64_t M_ld, const float* y,
                                  int64_t y_ld, float* x, int64_t x_ld, int32_t nworld, void* stream) {
  if (!plan || !M || !y || !x || !plan->prog || !plan->prog_ptr)
    return imn::set_error("imn_tree_ldl_solve: NULL argument"), IMN_ERR_NULL;
  if (plan->nv <= 0 || plan->groups < 1 || plan->groups > 4 || plan->owner < 0 || plan->owner >= plan->groups ||
      plan->nslot <= 0)
    return imn::set_error("imn_tree_ldl_solve: malformed plan"), IMN_ERR_SHAPE;
  if (nworld < 0 || M_ld < plan->nM || y_ld < plan->nv || x_ld < plan->nv)
    return imn::set_error("imn_tree_ldl_solve: a stride is smaller than its extent"), IMN_ERR_SHAPE;
  if (nworld == 0) return IMN_OK;
  const size_t bytes = (size_t)plan->nslot * 32 * sizeof(float);
  if (bytes > 227 * 1024)
    return imn::set_error("imn_tree_ldl_solve: plan needs %zu bytes of shared memory per block (max %d)", bytes,
                          227 * 1024),
           IMN_ERR_LIMIT;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(imn::tree_ldl_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess)
      return imn::set_error("imn_tree_ldl_solve: cudaFuncSetAttribute: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  }
  imn::tree_ldl_kernel<<<(nworld + 31) / 32, 32 * plan->groups, bytes, (cudaStream_t)stream>>>(
      reinterpret_cast<const int4*>(plan->prog), plan->prog_ptr, plan->groups, plan->owner, M, M_ld, y, y_ld, x,
      x_ld, nworld);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return imn::set_error("imn_tree_ldl_solve: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}

extern "C" int imn_blocked_dense_factor_solve(const ImnBlockedPlan* plan, const float* M, int64_t M_ld,
                                              const float* y, float* U, float* x, const int32_t* active,
                                              int32_t nworld, int32_t rhs_count, int32_t mode, void* stream) {
  if (!plan || !y || !U || !x || (mode == 0 && (!M || !plan->indices || !plan->identity)))
    return imn::set_error("imn_blocked_dense_factor_solve: NULL argument"), IMN_ERR_NULL;
  if (plan->nv <= 0 || plan->pad % 16 != 0 || plan->pad < plan->nv || plan->pad >= plan->nv + 16)
    return imn::set_error("imn_blocked_dense_factor_solve: pad %d is not nv %d rounded up to 16", plan->pad,
                          plan->nv),
           IMN_ERR_SHAPE;
  if (mode != 0 && mode != 1) return imn::set_error("imn_blocked_dense_factor_solve: mode must be 0 or 1"), IMN_ERR_SHAPE;
  if (nworld < 0 || rhs_count < 1 || (mode == 0 && M_ld < plan->nM))
    return imn::set_error("imn_blocked_dense_factor_solve: bad extent or stride"), IMN_ERR_SHAPE;
  if (nworld == 0) return IMN_OK;
  const int ld = plan->pad | 1;
  const size_t bytes = sizeof(float) * ((size_t)plan->pad * ld + plan->pad + (size_t)plan->pad * rhs_count);
  if (bytes > 227 * 1024)
    return imn::set_error("imn_blocked_dense_factor_solve: %zu bytes of shared memory needed (max %d)", bytes,
                          227 * 1024),
           IMN_ERR_LIMIT;
  if (bytes > 48 * 1024) {
    cudaError_t e =
        cudaFuncSetAttribute(imn::blocked_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess)
      return imn::set_error("imn_blocked_dense_factor_solve: cudaFuncSetAttribute: %s", cudaGetErrorString(e)),
             IMN_ERR_LAUNCH;
  }
  imn::blocked_dense_kernel<<<nworld, 32, bytes, (cudaStream_t)stream>>>(
      plan->nv, plan->pad, plan->nM, plan->indices, plan->identity, M, M_ld, y, U, x, active, rhs_count, mode);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return imn::set_error("imn_blocked_dense_factor_solve: launch failed: %s", cudaGetErrorString(e)),
           IMN_ERR_LAUNCH;
  return IMN_OK;
}

// ---- factor + solve without any caller- or library-side allocation ---------------
//
// Some hosts of this library may not allocate device memory at the point where they
// need a factor + solve: a simulation step that is being recorded into a CUDA graph,
// a control loop that has handed all device memory to another framework's pool at
// start-up, or a plug-in whose host forbids cudaMalloc after initialisation (the call
// synchronises the device).  imn_blocked_dense_factor_solve needs a (W, pad, pad)
// workspace for the factor; this variant keeps that workspace inside the library, in
// a fixed-size array in device memory that every GPU loading the library holds until
// the process exits.
namespace imn {

static __device__ __align__(256) float g_static_factor[IMN_STATIC_FACTOR_FLOATS];

// Device address of g_static_factor per CUDA device.  In host code the array's name is
// only a handle; the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
static float* g_static_factor_ptr[64] = {nullptr};

static int static_factor_workspace(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error("static workspace: cudaGetDevice: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  if (dev < 0 || dev >= 64) return set_error("static workspace: device index %d out of range", dev), IMN_ERR_LIMIT;
  if (!g_static_factor_ptr[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_factor);
    if (e != cudaSuccess || !ptr)
      return set_error("static workspace: cudaGetSymbolAddress: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
    g_static_factor_ptr[dev] = ptr;
  }
  *out = g_static_factor_ptr[dev];
  return IMN_OK;
}

}  // namespace imn

extern "C" int imn_blocked_dense_factor_solve_static(const ImnBlockedPlan* plan, const float* M, int64_t M_ld,
                                                     const float* y, float* x, const int32_t* active,
                                                     int32_t nworld, int32_t rhs_count, void* stream) {
  if (!plan) return imn::set_error("imn_blocked_dense_factor_solve_static: NULL plan"), IMN_ERR_NULL;
  if (nworld < 0 || plan->pad <= 0)
    return imn::set_error("imn_blocked_dense_factor_solve_static: bad extent"), IMN_ERR_SHAPE;
  const int64_t need = (int64_t)nworld * plan->pad * plan->pad;
  if (need > (int64_t)IMN_STATIC_FACTOR_FLOATS)
    return imn::set_error("imn_blocked_dense_factor_solve_static: %d worlds x pad %d^2 = %lld floats exceed the "
                          "built-in workspace of %lld floats; use imn_blocked_dense_factor_solve with your own",
                          nworld, plan->pad, (long long)need, (long long)IMN_STATIC_FACTOR_FLOATS),
           IMN_ERR_LIMIT;
  float* U = nullptr;
  const int rc = imn::static_factor_workspace(&U);
  if (rc) return rc;
  // The factor kernel writes every entry of an active world's U before the solve
  // reads it, so nothing in the shared workspace has to start at zero.
  return imn_blocked_dense_factor_solve(plan, M, M_ld, y, U, x, active, nworld, rhs_count, 0, stream);
}
