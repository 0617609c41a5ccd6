// imn_api.cu -- error text, ABI version and the two small per-dof kernels
// (rowless hand-off, M v).
#include <stdarg.h>
#include <stdio.h>

#include "imn_common.cuh"

namespace imn {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
}

// M v over the symmetric row tables, a bandwidth-bound pass: every CTA stages the
// (model-wide) tables in shared memory once and its eight warps then walk worlds
// with a grid stride.  A lane owns dofs lane, lane+32, ...; its loads of M and v
// are independent of one another, so many cache lines are in flight per warp; each
// line of a world's M row and v is fetched from HBM once and reused out of L1.
// Running sums are formed in table order (ascending stored entries), as the oracle.
__global__ void __launch_bounds__(256) mul_m_kernel(const int nv, const int* __restrict__ rowadr,
                                                    const int* __restrict__ col, const int* __restrict__ madr,
                                                    const float* __restrict__ M, const int64_t M_ld,
                                                    const float* __restrict__ v, const int64_t v_ld,
                                                    float* __restrict__ out, const int64_t out_ld,
                                                    float* __restrict__ copy_to, int* __restrict__ niter,
                                                    float* __restrict__ zero, const int nworld) {
  extern __shared__ uint32_t tab[];  // packed (col | madr << 16) entries, then nv + 1 row starts
  const int nnz = rowadr[nv];
  int* radr = reinterpret_cast<int*>(tab + nnz);
  for (int e = threadIdx.x; e < nnz; e += blockDim.x) tab[e] = (uint32_t)col[e] | ((uint32_t)madr[e] << 16);
  for (int i = threadIdx.x; i <= nv; i += blockDim.x) radr[i] = rowadr[i];
  __syncthreads();
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int w = blockIdx.x * warps + (threadIdx.x >> 5); w < nworld; w += gridDim.x * warps) {
    const float* Mw = M + (size_t)w * M_ld;
    const float* vw = v + (size_t)w * v_ld;
    for (int i = lane; i < nv; i += 32) {
      float s = 0.0f;
      const int k1 = radr[i + 1];
#pragma unroll 8
      for (int k = radr[i]; k < k1; ++k) {
        const uint32_t p = tab[k];
        s = fmaf(__ldg(Mw + (p >> 16)), __ldg(vw + (p & 0xFFFF)), s);
      }
      out[(size_t)w * out_ld + i] = s;
      if (copy_to) copy_to[(size_t)w * v_ld + i] = __ldg(vw + i);
      if (zero) zero[(size_t)w * v_ld + i] = 0.0f;
    }
    if (niter && lane == 0) niter[w] = 0;
  }
}

static int launch_mul_m(const ImnModel* m, const float* M, int64_t M_ld, const float* v, int64_t v_ld,
                        float* out, int64_t out_ld, float* copy_to, int* niter, float* zero, int nworld,
                        cudaStream_t stream) {
  if (nworld == 0) return IMN_OK;
  if (m->nM >= (1 << 16)) return set_error("mul_m: nM %d exceeds 16-bit indices", m->nM), IMN_ERR_LIMIT;
  // the symmetric tables list every stored entry at most twice
  const size_t bytes = ((size_t)2 * m->nM + m->nv + 1) * sizeof(uint32_t);
  if (bytes > 48 * 1024) return set_error("mul_m: nM %d too large", m->nM), IMN_ERR_LIMIT;
  const int warps = 8;
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int grid = min((nworld + warps - 1) / warps, sms * 8);
  mul_m_kernel<<<grid, warps * 32, bytes, stream>>>(m->nv, m->M_mulm_rowadr, m->M_mulm_col, m->M_mulm_madr, M, M_ld,
                                                    v, v_ld, out, out_ld, copy_to, niter, zero, nworld);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("mul_m: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}

}  // namespace imn

extern "C" const char* imn_last_error(void) { return imn::g_error; }
extern "C" int imn_abi_version(void) { return IMN_ABI_VERSION; }

extern "C" int imn_mul_m(const ImnModel* m, const float* M, int64_t M_ld, const float* v, int64_t v_ld,
                         float* out, int64_t out_ld, int32_t nworld, void* stream) {
  if (!m || !M || !v || !out || !m->M_mulm_rowadr || !m->M_mulm_col || !m->M_mulm_madr)
    return imn::set_error("imn_mul_m: NULL argument"), IMN_ERR_NULL;
  if (m->nv <= 0 || nworld < 0 || M_ld < m->nM || v_ld < m->nv || out_ld < m->nv)
    return imn::set_error("imn_mul_m: bad extent or stride"), IMN_ERR_SHAPE;
  return imn::launch_mul_m(m, M, M_ld, v, v_ld, out, out_ld, nullptr, nullptr, nullptr, nworld,
                           (cudaStream_t)stream);
}

extern "C" int imn_rowless_handoff(const ImnModel* m, const ImnData* d, void* stream) {
  if (!m || !d) return imn::set_error("imn_rowless_handoff: NULL struct"), IMN_ERR_NULL;
  if (!d->qacc_smooth || !d->qacc || !d->efc_Ma || !d->qfrc_constraint || !d->solver_niter || !d->M ||
      !m->M_mulm_rowadr || !m->M_mulm_col || !m->M_mulm_madr)
    return imn::set_error("imn_rowless_handoff: a required pointer is NULL"), IMN_ERR_NULL;
  if (m->nv <= 0 || d->nworld < 0 || d->dof_ld < m->nv || d->M_ld < m->nM)
    return imn::set_error("imn_rowless_handoff: bad extent or stride"), IMN_ERR_SHAPE;
  // qacc = qacc_smooth, Ma = M qacc, qfrc_constraint = 0, niter = 0
  return imn::launch_mul_m(m, d->M, d->M_ld, d->qacc_smooth, d->dof_ld, d->efc_Ma, d->dof_ld, d->qacc,
                           d->solver_niter, d->qfrc_constraint, d->nworld, (cudaStream_t)stream);
}

extern "C" int imn_copy_rows(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t width,
                             int32_t nworld, int32_t to_host, void* stream) {
  if (!dst || !src) return imn::set_error("imn_copy_rows: NULL buffer"), IMN_ERR_NULL;
  if (width < 0 || nworld < 0 || width > dst_pitch || width > src_pitch)
    return imn::set_error("imn_copy_rows: width %lld exceeds a pitch (%lld, %lld)", (long long)width,
                          (long long)dst_pitch, (long long)src_pitch),
           IMN_ERR_SHAPE;
  if (width == 0 || nworld == 0) return IMN_OK;
  const cudaError_t e = cudaMemcpy2DAsync(dst, (size_t)dst_pitch, src, (size_t)src_pitch, (size_t)width, (size_t)nworld,
                                          to_host ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice,
                                          (cudaStream_t)stream);
  if (e != cudaSuccess) return imn::set_error("imn_copy_rows: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}
