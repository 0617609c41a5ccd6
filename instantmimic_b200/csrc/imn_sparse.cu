// imn_sparse.cu -- the sparse Hessian factor for the non-fused Newton iteration
// (reference: sparse_hessian_upstream_factor, sparse_hessian.py:849-894 with the
// generated body :651-679).  One warp per world gathers the dense H that the
// upstream assembly maintains into the pattern slots, factors it level by level
// and solves (mode 4), or reloads the stored factor and solves (mode 5).
// hfactor per world: [0, nfac) N = L D, [nfac, nfac + nv) 1/D.
#include <stdio.h>
#include <string.h>

#include "imn_sparse.cuh"

namespace imn {

__global__ void __launch_bounds__(32) sparse_nonfused_kernel(
    const ImnSparsePlan P, const uint8_t* __restrict__ done, const float* __restrict__ grad, int64_t grad_ld,
    const float* __restrict__ h, const int* __restrict__ quad_changed, const int* __restrict__ state_changed,
    float* __restrict__ hfactor, float* __restrict__ search, int64_t search_ld, float* __restrict__ search_dot,
    float* __restrict__ decrement, int skip_unchanged, int skip_noflip) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x, w = blockIdx.x;
  if (done && done[w]) return;
  if (skip_noflip && state_changed[w] == 0) return;
  const int mode = (skip_unchanged && quad_changed[w] == 0) ? 5 : 4;
  const int n = P.nv, nfac = P.nfac, P2 = P.nv_pad * P.nv_pad;
  float* N = sm;                        // nslots
  float* iD = N + ((P.nslots + 3) & ~3);  // nv
  float* g = iD + ((n + 3) & ~3);         // nv: grad staged in shared memory
  float* xs = g + ((n + 3) & ~3);         // nv: search
  float* Uf = hfactor + (size_t)w * P2;
  for (int i = lane; i < n; i += 32) g[i] = grad[(size_t)w * grad_ld + i];
  if (mode == 4) {
    const float* Hd = h + (size_t)w * P2;
    for (int s = lane; s < nfac; s += 32) N[s] = Hd[__ldg(P.gat + s)];
    __syncwarp();
    sp_load_rhs(P, N, g, lane);
    sp_factor_levels(P, N, iD, lane);
    for (int s = lane; s < nfac; s += 32) Uf[s] = N[s];
    for (int j = lane; j < n; j += 32) Uf[nfac + j] = iD[j];
  } else {
    for (int s = lane; s < nfac; s += 32) N[s] = Uf[s];
    for (int j = lane; j < n; j += 32) iD[j] = Uf[nfac + j];
    __syncwarp();
    sp_forward(P, N, iD, g, lane);
  }
  float s0, s1;
  sp_backward(P, N, iD, g, xs, P.block, lane, s0, s1);
  for (int i = lane; i < n; i += 32) search[(size_t)w * search_ld + i] = xs[i];
  if (lane == 0) {
    search_dot[w] = s0;
    decrement[w] = s1;
  }
}

}  // namespace imn

extern "C" int imn_sparse_factor_nonfused(const ImnSparsePlan* plan, const uint8_t* done, const float* grad,
                                          int64_t grad_ld, const float* h, const int32_t* quad_changed,
                                          const int32_t* state_changed, float* hfactor, float* search,
                                          int64_t search_ld, float* search_dot, float* decrement,
                                          int32_t nworld, int32_t skip_unchanged, int32_t skip_noflip,
                                          void* stream) {
  if (!plan || !grad || !h || !hfactor || !search || !search_dot || !decrement)
    return imn::set_error("imn_sparse_factor_nonfused: NULL argument"), IMN_ERR_NULL;
  if ((skip_unchanged && !quad_changed) || (skip_noflip && !state_changed))
    return imn::set_error("imn_sparse_factor_nonfused: a skip flag needs its counter array"), IMN_ERR_NULL;
  if (plan->nv <= 0 || plan->nfac <= 0 || plan->nslots != plan->nfac + plan->nv || plan->nlevels <= 0 ||
      plan->block % 32 != 0 || plan->block < 32 || plan->block > 128 ||
      plan->nfac + plan->nv > plan->nv_pad * plan->nv_pad)
    return imn::set_error("imn_sparse_factor_nonfused: malformed plan"), IMN_ERR_SHAPE;
  if (nworld < 0 || grad_ld < plan->nv || search_ld < plan->nv)
    return imn::set_error("imn_sparse_factor_nonfused: a stride is smaller than its extent"), IMN_ERR_SHAPE;
  if (!plan->gat || !plan->lvl_ptr || !plan->lvl_team || !plan->ent_slot || !plan->ent_col || !plan->run_ptr ||
      !plan->run_ab || !plan->run_kl || !plan->orig || !plan->b_lvl || !plan->b_slot || !plan->b_src ||
      !plan->b_dst || !plan->f_lvl || !plan->f_row || !plan->row_start || !plan->rk_ptr || !plan->rk)
    return imn::set_error("imn_sparse_factor_nonfused: a plan table is NULL"), IMN_ERR_NULL;
  if (nworld == 0) return IMN_OK;
  const int n4 = (plan->nv + 3) & ~3;
  const size_t bytes = sizeof(float) * (((plan->nslots + 3) & ~3) + 3 * (size_t)n4);
  if (bytes > 227 * 1024)
    return imn::set_error("imn_sparse_factor_nonfused: factor needs %zu bytes of shared memory", bytes), IMN_ERR_LIMIT;
  if (bytes > 48 * 1024) {
    cudaError_t e =
        cudaFuncSetAttribute(imn::sparse_nonfused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess)
      return imn::set_error("imn_sparse_factor_nonfused: cudaFuncSetAttribute: %s", cudaGetErrorString(e)),
             IMN_ERR_LAUNCH;
  }
  imn::sparse_nonfused_kernel<<<nworld, 32, bytes, (cudaStream_t)stream>>>(
      *plan, done, grad, grad_ld, h, quad_changed, state_changed, hfactor, search, search_ld, search_dot,
      decrement, skip_unchanged, skip_noflip);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return imn::set_error("imn_sparse_factor_nonfused: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}

// ---- plan upload ---------------------------------------------------------------
// The host builds the index tables once per model; this is the one place where the
// library allocates device memory: one slab that holds every table, freed by
// imn_sparse_plan_destroy.
namespace imn {

struct OwnedSparsePlan {
  ImnSparsePlan plan;  // first member: the pointer handed out is also the owner's
  void* slab;
};

}  // namespace imn

extern "C" int imn_sparse_plan_create(const ImnSparsePlan* host, ImnSparsePlan** out) {
  if (!host || !out) return imn::set_error("imn_sparse_plan_create: NULL argument"), IMN_ERR_NULL;
  *out = nullptr;
  if (host->nv <= 0 || host->nfac <= 0 || host->nlevels <= 0 || host->nentries <= 0 || host->nruns < 0 ||
      host->nback < 0 || host->nfsweep < 0 || host->nbsweep < 0 || !host->rk_ptr)
    return imn::set_error("imn_sparse_plan_create: malformed plan"), IMN_ERR_SHAPE;
  const int nv = host->nv, words = (nv + 31) / 32;
  const size_t nrk = host->rk_ptr[nv] > 0 ? host->rk_ptr[nv] : 1;
  struct Table {
    const void* src;
    size_t bytes;
    const void** dst;
  };
  imn::OwnedSparsePlan* owned = new imn::OwnedSparsePlan();
  owned->plan = *host;
  ImnSparsePlan& d = owned->plan;
#define TAB(field, count) {host->field, sizeof(*host->field) * (size_t)(count), (const void**)&d.field}
  const Table tabs[] = {
      TAB(lvl_ptr, host->nlevels + 1), TAB(lvl_team, host->nlevels), TAB(ent_slot, host->nentries),
      TAB(ent_col, host->nentries),    TAB(run_ptr, host->nentries + 1), TAB(run_ab, host->nruns > 0 ? host->nruns : 1),
      TAB(run_kl, host->nruns > 0 ? host->nruns : 1), TAB(orig, nv), TAB(b_lvl, host->nlevels + 1),
      TAB(b_slot, host->nback > 0 ? host->nback : 1), TAB(b_src, host->nback > 0 ? host->nback : 1),
      TAB(b_dst, host->nback > 0 ? host->nback : 1), TAB(pair, nv * nv), TAB(f_lvl, host->nlevels + 1),
      TAB(f_row, nv), TAB(row_start, nv), TAB(rk_ptr, nv + 1), TAB(rk, nrk), TAB(pmask, nv * words),
      TAB(s_a, host->nfac), TAB(s_b, host->nfac), TAB(s_m, host->nfac), TAB(gat, host->nfac),
      TAB(fsweep, (size_t)host->nfsweep * 128), TAB(bsweep, (size_t)host->nbsweep * 32),
  };
#undef TAB
  size_t total = 0;
  for (const Table& t : tabs) {
    if (t.bytes && !t.src) {
      delete owned;
      return imn::set_error("imn_sparse_plan_create: a table is NULL"), IMN_ERR_NULL;
    }
    total += (t.bytes + 15) & ~(size_t)15;
  }
  unsigned char* staging = new unsigned char[total]();
  cudaError_t e = cudaMalloc(&owned->slab, total);
  if (e != cudaSuccess) {
    delete[] staging;
    delete owned;
    return imn::set_error("imn_sparse_plan_create: cudaMalloc of %zu bytes: %s", total, cudaGetErrorString(e)),
           IMN_ERR_LAUNCH;
  }
  size_t off = 0;
  for (const Table& t : tabs) {
    if (t.bytes) {
      memcpy(staging + off, t.src, t.bytes);
      *t.dst = (const unsigned char*)owned->slab + off;
    } else {
      *t.dst = nullptr;
    }
    off += (t.bytes + 15) & ~(size_t)15;
  }
  e = cudaMemcpy(owned->slab, staging, total, cudaMemcpyHostToDevice);
  delete[] staging;
  if (e != cudaSuccess) {
    cudaFree(owned->slab);
    delete owned;
    return imn::set_error("imn_sparse_plan_create: upload: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  }
  *out = &owned->plan;
  return IMN_OK;
}

extern "C" void imn_sparse_plan_destroy(ImnSparsePlan* plan) {
  if (!plan) return;
  imn::OwnedSparsePlan* owned = reinterpret_cast<imn::OwnedSparsePlan*>(plan);
  cudaFree(owned->slab);
  delete owned;
}
