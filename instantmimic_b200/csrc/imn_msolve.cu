// imn_msolve.cu -- factor + solve of inertia-like matrices (M and M - h qDeriv):
// the tree-structured L'DL and the blocked dense Cholesky.
//
// Tree L'DL (reference: tree_ldl.py:196-359, 419-433).  The reference generates
// straight-line source per model; imn_tree_jit.cu does the same with NVRTC.  The
// kernel here interprets the plan's instruction list instead (the fallback when no
// run-time compiler is installed, and the statement the generated code must match).  A block serves 32 worlds with one warp per group; lane l of
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
#include <atomic>

#include "imn_common.cuh"

namespace imn {

enum { OP_LOAD_M, OP_LOAD_Y, OP_ZERO, OP_INV, OP_UPD, OP_SCALE, OP_SUBMUL, OP_MUL, OP_ADD, OP_STORE_X, OP_MULSUB, OP_MULADD };

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
      case OP_MULSUB: col[dst * 32] = fmaf(col[a * 32], col[b * 32], -col[dst * 32]); break;
      case OP_MULADD: col[dst * 32] = fmaf(col[a * 32], col[b * 32], col[dst * 32]); break;
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
// One warp per world (or two worlds per warp, see dense_factor_carry), four warps per
// CTA.  Shared memory of a world:
//   A    (n + carry + 1) x ldu.  U[r][c] (r <= c) at A[r*ldu + c]; the value column c
//        starts from (M's column c above the diagonal, or right-hand side c - n) is
//        kept transposed at A[(c+1)*ldu + r], so a lane reads the 16 rows of its
//        column with four 128-bit loads.
//   dinv n, X n x rhs (right-hand sides, then solutions).
// The factorisation works on the nv x nv part only: with zero padding and a unit
// diagonal the padded rows of U are exactly the identity, which is what is stored.
// Up to `carry` right-hand sides ride through the factorisation as extra columns
// (that is the forward substitution); further ones, and mode 1, take the
// substitution with the stored factor.  Every value receives its terms in the same
// order as the plain row-by-row statement of the algorithm (ascending t).
static const int kDenseWarps = 4;

// LW lanes work on one world: 32 (a warp per world), or 16 for models whose n + carry
// columns fit three columns per lane of a half-warp (<= 48), where a whole warp would leave
// half its lanes without a column for most of the factorisation; a warp then factors two
// worlds at once.  `l` is the lane within the team, `base` the team's first lane (shuffle
// sources are base | lane-in-team).
template <int LW>
__device__ __forceinline__ void dense_factor_carry(float* A, float* dinv, const int n, const int nc, const int ldu,
                                                   const int l, const int base) {
#pragma unroll 1
  for (int b0 = 0; b0 < n; b0 += 16) {
    const int nr = min(16, n - b0);
    const int ng = (nr + 3) >> 2;
    float acc[3][16];
    int cc[3];
    bool act[3], valid[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const int c = b0 + l + LW * k;
      act[k] = b0 + LW * k < nc;  // uniform over the team (and over the warp: one model)
      valid[k] = c < nc;
      cc[k] = valid[k] ? c : nc - 1;
      if (act[k]) {
        const float* src = A + (cc[k] + 1) * ldu + b0;
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
    // terms of the rows above the block
#pragma unroll 2
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
    // the block's own rows, one by one; acc[k][0] is always the current row.  Row b0 + r's
    // column is held by lane r of the team (k = 0); the rows below it inside the block by
    // lanes r + 1 .. 15 (later sources wrap and feed slots that are never read).
#pragma unroll 1
    for (int r = 0; r < nr; ++r) {
      const float pv = __shfl_sync(IMN_FULL_MASK, acc[0][0], base | r);
      const float dg = sqrtf(pv);
      const float rinv = 1.0f / dg;
      float u[3];
      float* Ur = A + (b0 + r) * ldu;
#pragma unroll
      for (int k = 0; k < 3; ++k)
        if (act[k]) {
          u[k] = acc[k][0] * rinv;
          if (k == 0 && l == r) u[k] = dg;
          if (valid[k] && cc[k] >= b0 + r) Ur[cc[k]] = u[k];
        }
      if (l == 0) dinv[b0 + r] = rinv;
      float um[16];
#pragma unroll
      for (int j = 1; j < 16; ++j) um[j] = __shfl_sync(IMN_FULL_MASK, u[0], base | ((r + j) & (LW - 1)));
#pragma unroll
      for (int k = 0; k < 3; ++k)
        if (act[k]) {
#pragma unroll
          for (int j = 1; j < 16; ++j) acc[k][j - 1] = fmaf(-um[j], u[k], acc[k][j]);
          acc[k][15] = 0.0f;
        }
    }
    __syncwarp();
  }
}

template <int LW>
__global__ void __launch_bounds__(32 * kDenseWarps)
    blocked_dense_kernel(const int nv, const int pad, const int nM, const int* __restrict__ indices,
                         const float* __restrict__ identity, const float* __restrict__ M, const int64_t M_ld,
                         const float* __restrict__ y, float* __restrict__ Ug, float* __restrict__ x,
                         const int* __restrict__ active, const int rhs, const int mode, const int carry,
                         const int ldu, const int per_world, const int nworld) {
  extern __shared__ __align__(16) float sm[];
  constexpr int kPer = 32 / LW;  // worlds per warp
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int l = lane & (LW - 1), base = lane & ~(LW - 1), sub = lane / LW;
  const int first = (blockIdx.x * kDenseWarps + warp) * kPer;
  if (first >= nworld) return;
  const int wreal = first + sub;
  // a team without a world, or with an inactive one, runs along on the warp's first
  // world (the shuffles are full-warp) and stores nothing
  bool live = wreal < nworld;
  if (live && active && active[wreal] == 0) live = false;
  if (!__any_sync(IMN_FULL_MASK, live)) return;
  const int w = wreal < nworld ? wreal : first;
  const int n = nv, nc = n + carry;
  float* A = sm + (warp * kPer + sub) * per_world;
  float* dinv = A + (nc + 1) * ldu;
  float* X = dinv + ((n + 3) & ~3);
  float* Uw = Ug + (size_t)w * pad * pad;
  const int nblk = pad >> 4;
  const float* yw = y + (size_t)w * n * rhs;
  for (int q = l; q < n * rhs; q += LW) X[q] = yw[q];
  if (mode == 0) {
    // gather the blocks on and above the diagonal: table entry
    // ((kb*nblk + ib)*16 + r)*16 + c addresses M's value of (16 kb + r, 16 ib + c);
    // index nM is the extra zero slot
    const float* Mw = M + (size_t)w * M_ld;
    for (int kb = 0; kb < nblk; ++kb)
      for (int ib = kb; ib < nblk; ++ib) {
        const int* tab = indices + ((kb * nblk + ib) << 8);
#pragma unroll 4
        for (int q = l; q < 256; q += LW) {
          const int row = 16 * kb + (q >> 4), colm = 16 * ib + (q & 15);
          const int idx = __ldg(tab + q);
          if (row <= colm && colm < n) A[(colm + 1) * ldu + row] = idx < nM ? __ldg(Mw + idx) : 0.0f;
        }
      }
    __syncwarp();
    for (int e = l; e < n * carry; e += LW) {
      const int r = e / carry, q = e - r * carry;
      A[(n + q + 1) * ldu + r] = X[r * rhs + q];
    }
    __syncwarp();
    dense_factor_carry<LW>(A, dinv, n, nc, ldu, l, base);
    // the factor, padded: zeros below the diagonal, the padded diagonal's own root
    if (live) {
      for (int r = 0; r < n; ++r) {
        const float* Ar = A + r * ldu;
        float* Ur = Uw + r * pad;
#pragma unroll 3
        for (int c = l; c < pad; c += LW) Ur[c] = (c >= r && c < n) ? Ar[c] : 0.0f;
      }
      for (int r = n; r < pad; ++r) {
        const float dg = sqrtf(identity[((r & 15) << 4) | (r & 15)]);
        for (int c = l; c < pad; c += LW) Uw[r * pad + c] = c == r ? dg : 0.0f;
      }
    }
    for (int e = l; e < n * carry; e += LW) {
      const int r = e / carry, q = e - r * carry;
      X[r * rhs + q] = A[r * ldu + n + q];
    }
  } else {
    for (int r = 0; r < n; ++r)
      for (int c = r + l; c < n; c += LW) A[r * ldu + c] = Uw[r * pad + c];
    __syncwarp();
    for (int r = l; r < n; r += LW) dinv[r] = 1.0f / A[r * ldu + r];
  }
  __syncwarp();
  // forward substitution with the stored factor for the right-hand sides that did
  // not ride along: unknown r receives its terms in ascending order
  const int q0 = mode == 0 ? carry : 0;
  if (q0 < rhs) {
    const int nq = rhs - q0;
    for (int t = 0; t < n; ++t) {
      const float di = dinv[t];
      for (int q = l; q < nq; q += LW) X[t * rhs + q0 + q] = X[t * rhs + q0 + q] * di;
      __syncwarp();
      for (int e = l; e < (n - t - 1) * nq; e += LW) {
        const int r = t + 1 + e / nq, q = q0 + e % nq;
        X[r * rhs + q] = fmaf(-A[t * ldu + r], X[t * rhs + q], X[r * rhs + q]);
      }
      __syncwarp();
    }
  }
  // back substitution in 16-row blocks from the last: later blocks' columns first
  // (ascending), then the block's own columns from its last inwards; a team of 32 lanes
  // takes two right-hand sides at a time on its two halves, a team of 16 one
  constexpr int kRhsAtOnce = LW / 16;
  for (int qb = 0; qb < rhs; qb += kRhsAtOnce) {
    const int q = qb + (l >> 4), l16 = l & 15;
    const bool hasq = q < rhs;
    for (int b0 = ((n - 1) / 16) * 16; b0 >= 0; b0 -= 16) {
      const int b1 = min(b0 + 16, n);
      const int r = b0 + l16;
      const float* Ur = A + r * ldu;
      float acc = 0.0f, di = 0.0f;
      if (r < b1 && hasq) {
        acc = X[r * rhs + q];
        di = dinv[r];
#pragma unroll 2
        for (int c = b1; c < n; ++c) acc = fmaf(-Ur[c], X[c * rhs + q], acc);
      }
      for (int c = b1 - 1; c >= b0; --c) {
        const float xc = __shfl_sync(IMN_FULL_MASK, acc * di, (lane & ~15) | (c - b0));
        if (r < c && hasq) acc = fmaf(-Ur[c], xc, acc);
        if (l16 == 0 && hasq) X[c * rhs + q] = xc;
      }
      __syncwarp();
    }
  }
  if (live) {
    float* xw = x + (size_t)w * n * rhs;
    for (int q = l; q < n * rhs; q += LW) xw[q] = X[q];
  }
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
  const int n = plan->nv;
  if (n > 80) return imn::set_error("imn_blocked_dense_factor_solve: nv %d above 80", n), IMN_ERR_UNSUPPORTED;
  // right-hand sides that ride through the factorisation as extra columns
  const int carry = mode == 0 ? (rhs_count < 96 - n ? rhs_count : 96 - n) : 0;
  const int ldu = (n + carry + 3) & ~3;
  const int per_world = (n + carry + 1) * ldu + ((n + 3) & ~3) + ((n * rhs_count + 3) & ~3);
  // two worlds per warp when every column of the factorisation has a place on 16 lanes
  // and the batch is large enough to keep the GPU full that way
  const bool half = n + carry <= 48 && nworld >= 2048;
  const int per_cta = imn::kDenseWarps * (half ? 2 : 1);
  const size_t bytes = sizeof(float) * (size_t)per_world * per_cta;
  auto kernel = half ? imn::blocked_dense_kernel<16> : imn::blocked_dense_kernel<32>;
  if (bytes > 227 * 1024)
    return imn::set_error("imn_blocked_dense_factor_solve: %zu bytes of shared memory needed (max %d)", bytes,
                          227 * 1024),
           IMN_ERR_LIMIT;
  {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                         cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess && bytes > 48 * 1024)
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess)
      return imn::set_error("imn_blocked_dense_factor_solve: cudaFuncSetAttribute: %s", cudaGetErrorString(e)),
             IMN_ERR_LAUNCH;
  }
  kernel<<<(nworld + per_cta - 1) / per_cta, 32 * imn::kDenseWarps, bytes, (cudaStream_t)stream>>>(
      plan->nv, plan->pad, plan->nM, plan->indices, plan->identity, M, M_ld, y, U, x, active, rhs_count, mode, carry, ldu,
      per_world, nworld);
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
// once per device with that device current.  The slots are atomics: two host threads
// that make the first call on a device at the same time both look the address up and
// store the same value.  A cached address belongs to the device's primary context; it
// does not survive cudaDeviceReset (after a reset, reload the library).
static std::atomic<float*> g_static_factor_ptr[64];

static int static_factor_workspace(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error("static workspace: cudaGetDevice: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  if (dev < 0 || dev >= 64) return set_error("static workspace: device index %d out of range", dev), IMN_ERR_LIMIT;
  float* ptr = g_static_factor_ptr[dev].load(std::memory_order_acquire);
  if (!ptr) {
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_factor);
    if (e != cudaSuccess || !ptr)
      return set_error("static workspace: cudaGetSymbolAddress: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
    g_static_factor_ptr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
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
