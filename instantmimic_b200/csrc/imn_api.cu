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

// The same product for large batches, tile by tile: a block takes 32 consecutive
// worlds, lane = world.  With one warp per world (above) a lane gathers M[madr] and
// v[col] from all over its world's row, every load instruction touches ~10 cache lines
// and the L1's one-line-per-cycle rate bounds the kernel at a sixth of the HBM rate.
// Here the tile -- 32 x nM floats of M, 32 x nv of v, both contiguous -- arrives in
// shared memory by two TMA bulk copies on one mbarrier (bounded wait; plain coalesced
// loads for a partial, strided or unaligned tile), the table entry is the same for all
// lanes (one broadcast read), a lane reads its own world's M and v from the tile
// (stride nM / nv between lanes: gcd(stride, 32)-way bank conflicts) and keeps a row's
// running sum in a register.  The warps of a block split the rows by stored entries.
// Results leave through the tile by one bulk store.  Sums are formed in table order,
// so the bits equal mul_m_kernel's.
static const int kTileWarps = 4;

__global__ void __launch_bounds__(32 * kTileWarps)
    mul_m_tile_kernel(const int nv, const int nM, const int* __restrict__ rowadr, const int* __restrict__ col,
                      const int* __restrict__ madr, const float* __restrict__ M, const int64_t M_ld,
                      const float* __restrict__ v, const int64_t v_ld, float* __restrict__ out, const int64_t out_ld,
                      float* __restrict__ copy_to, int* __restrict__ niter, float* __restrict__ zero, const int nworld,
                      const int bulk) {
  extern __shared__ __align__(16) float tile[];
  const int nnz = rowadr[nv];
  float* Mt = tile + 4;  // the first 16 bytes hold the mbarrier
  float* vt = Mt + ((32 * nM + 3) & ~3);
  float* ot = vt + ((32 * nv + 3) & ~3);
  uint32_t* tab = reinterpret_cast<uint32_t*>(ot + ((32 * nv + 3) & ~3));
  int* radr = reinterpret_cast<int*>(tab + nnz);
  const int lw = threadIdx.x & 31, part = threadIdx.x >> 5;
  const int w0 = blockIdx.x * 32;
  const bool whole = bulk && w0 + 32 <= nworld;
  const unsigned bar = (unsigned)__cvta_generic_to_shared(tile);
  if (whole && threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(128u * (unsigned)(nM + nv))
                 : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     (unsigned)__cvta_generic_to_shared(Mt)),
                 "l"(M + (size_t)w0 * nM), "r"(128u * (unsigned)nM), "r"(bar)
                 : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     (unsigned)__cvta_generic_to_shared(vt)),
                 "l"(v + (size_t)w0 * nv), "r"(128u * (unsigned)nv), "r"(bar)
                 : "memory");
  }
  for (int e = threadIdx.x; e < nnz; e += blockDim.x) tab[e] = (uint32_t)col[e] | ((uint32_t)madr[e] << 16);
  for (int i = threadIdx.x; i <= nv; i += blockDim.x) radr[i] = rowadr[i];
  __syncthreads();  // tables staged, barrier initialised
  bool arrived = false;
  if (whole) {
    // bounded wait; if it runs out the copies get one more bounded wait and the tile is
    // then loaded again with plain loads
#pragma unroll 1
    for (int round = 0; round < 2 && !arrived; ++round)
#pragma unroll 1
      for (int tries = 0; tries < (1 << 22) && !arrived; ++tries) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar)
                     : "memory");
        arrived = ok != 0;
      }
  }
  if (!__syncthreads_and(arrived)) {
    for (int e = threadIdx.x; e < 32 * nM; e += blockDim.x) {
      const int r = e / nM, c = e - r * nM;
      Mt[e] = M[(size_t)min(w0 + r, nworld - 1) * M_ld + c];
    }
    for (int e = threadIdx.x; e < 32 * nv; e += blockDim.x) {
      const int r = e / nv, c = e - r * nv;
      vt[e] = v[(size_t)min(w0 + r, nworld - 1) * v_ld + c];
    }
    __syncthreads();
  }
  // rows of this warp: the stored entries are cut into kTileWarps near-equal runs
  const float* Mw = Mt + lw * nM;
  const float* vw = vt + lw * nv;
  float* ow = ot + lw * nv;
  const int lo = (int)(((long long)nnz * part) / kTileWarps), hi = (int)(((long long)nnz * (part + 1)) / kTileWarps);
#pragma unroll 1
  for (int i = 0; i < nv; ++i) {
    const int k0 = radr[i], k1 = radr[i + 1];
    if (k0 < lo || k0 >= hi) continue;  // a row belongs to the warp its first entry falls to
    float s = 0.0f;
#pragma unroll 4
    for (int k = k0; k < k1; ++k) {
      const uint32_t p = tab[k];
      s = fmaf(Mw[p >> 16], vw[p & 0xFFFF], s);
    }
    ow[i] = s;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (whole && out_ld == nv) {
    if (threadIdx.x == 0) {
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(out + (size_t)w0 * nv),
                   "r"((unsigned)__cvta_generic_to_shared(ot)), "r"(128u * (unsigned)nv)
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  } else {
    for (int e = threadIdx.x; e < 32 * nv; e += blockDim.x) {
      const int r = e / nv, c = e - r * nv;
      if (w0 + r < nworld) out[(size_t)(w0 + r) * out_ld + c] = ot[e];
    }
  }
  if (copy_to || zero)
    for (int e = threadIdx.x; e < 32 * nv; e += blockDim.x) {
      const int r = e / nv, c = e - r * nv;
      if (w0 + r < nworld) {
        if (copy_to) copy_to[(size_t)(w0 + r) * v_ld + c] = vt[e];
        if (zero) zero[(size_t)(w0 + r) * v_ld + c] = 0.0f;
      }
    }
  if (niter && threadIdx.x < 32 && w0 + threadIdx.x < nworld) niter[w0 + threadIdx.x] = 0;
  // shared memory must stay valid until the bulk store has read it
  if (whole && out_ld == nv && threadIdx.x == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

static int launch_mul_m(const ImnModel* m, const float* M, int64_t M_ld, const float* v, int64_t v_ld,
                        float* out, int64_t out_ld, float* copy_to, int* niter, float* zero, int nworld,
                        cudaStream_t stream) {
  if (nworld == 0) return IMN_OK;
  if (m->nM >= (1 << 16)) return set_error("mul_m: nM %d exceeds 16-bit indices", m->nM), IMN_ERR_LIMIT;
  // the symmetric tables list every stored entry at most twice
  const size_t bytes = ((size_t)2 * m->nM + m->nv + 1) * sizeof(uint32_t);
  if (bytes > 48 * 1024) return set_error("mul_m: nM %d too large", m->nM), IMN_ERR_LIMIT;
  {
    // tiles of 32 worlds for batches that fill the GPU, when the lane stride nM does not
    // pile the lanes onto a few banks and four tiles fit an SM's shared memory
    int g = m->nM, b = 32;
    while (b) {
      const int t = g % b;
      g = b, b = t;
    }
    const size_t tile_bytes = 16 + sizeof(float) * ((size_t)((32 * m->nM + 3) & ~3) + 2 * (size_t)((32 * m->nv + 3) & ~3)) +
                              bytes;
    if (nworld >= 4096 && g < 8 && tile_bytes <= 56 * 1024) {
      const int bulk = M_ld == m->nM && v_ld == m->nv && (reinterpret_cast<uintptr_t>(M) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(v) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
      cudaError_t e = cudaFuncSetAttribute(mul_m_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_bytes);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(mul_m_tile_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
      if (e != cudaSuccess) return set_error("mul_m: cudaFuncSetAttribute: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
      mul_m_tile_kernel<<<(nworld + 31) / 32, 32 * kTileWarps, tile_bytes, stream>>>(
          m->nv, m->nM, m->M_mulm_rowadr, m->M_mulm_col, m->M_mulm_madr, M, M_ld, v, v_ld, out, out_ld, copy_to, niter,
          zero, nworld, bulk);
      e = cudaGetLastError();
      if (e != cudaSuccess) return set_error("mul_m: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
      return IMN_OK;
    }
  }
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

namespace imn {

// Rows of a sparse Jacobian (values + column indices + row starts, the layout of MuJoCo
// C's sparse mjData.efc_J) written out as dense rows: a warp clears its row, then
// scatters the row's entries.  An index outside [0, nv) is skipped.
template <typename Index>
__global__ void __launch_bounds__(256)
    expand_rows_kernel(const float* __restrict__ values, const Index* __restrict__ colind, const int* __restrict__ rowadr,
                       const int nrows, const int nv, float* __restrict__ dense, const int64_t ld_row) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= nrows) return;
  float* row = dense + (size_t)r * ld_row;
  for (int c = lane; c < nv; c += 32) row[c] = 0.0f;
  __syncwarp();
  const int k1 = rowadr[r + 1];
  for (int k = rowadr[r] + lane; k < k1; k += 32) {
    const int c = (int)colind[k];
    if (c >= 0 && c < nv) row[c] = values[k];
  }
}

// The per-row vectors of the live rows (one value per row, worlds back to back like the
// compact Jacobian) written into the padded (nworld, efc_ld) arrays the solver reads.
// Rows at or beyond a world's nefc are left alone: the solver never reads them.
__global__ void __launch_bounds__(256)
    expand_row_vectors_kernel(const float* __restrict__ cD, const float* __restrict__ cA, const float* __restrict__ cF,
                              const int64_t* __restrict__ first, const int64_t ld_row, const int* __restrict__ nefc,
                              const int njmax, float* __restrict__ D, float* __restrict__ A, float* __restrict__ F,
                              const int64_t efc_ld, const int nworld) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (int64_t)nworld * njmax) return;
  const int w = (int)(t / njmax), r = (int)(t - (int64_t)w * njmax);
  if (r >= min(nefc[w], njmax)) return;
  const int64_t src = first[w] / ld_row + r, dst = (int64_t)w * efc_ld + r;
  D[dst] = cD[src], A[dst] = cA[src], F[dst] = cF[src];
}

}  // namespace imn

extern "C" int imn_expand_row_vectors(const float* D_rows, const float* aref_rows, const float* frictionloss_rows,
                                      const int64_t* J_world_offset, int64_t J_ld_row, const int32_t* nefc,
                                      int32_t njmax, float* D, float* aref, float* frictionloss, int64_t efc_ld,
                                      int32_t nworld, void* stream) {
  if (!D_rows || !aref_rows || !frictionloss_rows || !J_world_offset || !nefc || !D || !aref || !frictionloss)
    return imn::set_error("imn_expand_row_vectors: NULL buffer"), IMN_ERR_NULL;
  if (nworld < 0 || njmax < 0 || J_ld_row <= 0 || efc_ld < njmax)
    return imn::set_error("imn_expand_row_vectors: bad extent or stride"), IMN_ERR_SHAPE;
  const int64_t threads = (int64_t)nworld * njmax;
  if (threads == 0) return IMN_OK;
  imn::expand_row_vectors_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      D_rows, aref_rows, frictionloss_rows, J_world_offset, J_ld_row, nefc, njmax, D, aref, frictionloss, efc_ld, nworld);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return imn::set_error("imn_expand_row_vectors: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
}

extern "C" int imn_expand_rows(const float* values, const void* colind, int32_t colind_bytes, const int32_t* rowadr,
                               int32_t nrows, int32_t nv, float* dense, int64_t ld_row, void* stream) {
  if (!values || !colind || !rowadr || !dense) return imn::set_error("imn_expand_rows: NULL buffer"), IMN_ERR_NULL;
  if (nrows < 0 || nv <= 0 || ld_row < nv) return imn::set_error("imn_expand_rows: bad extent or stride"), IMN_ERR_SHAPE;
  if (colind_bytes != 4 && colind_bytes != 1)
    return imn::set_error("imn_expand_rows: column indices are int32 (4) or uint8 (1), not %d bytes", colind_bytes),
           IMN_ERR_SHAPE;
  if (colind_bytes == 1 && nv > 256) return imn::set_error("imn_expand_rows: nv %d does not fit 8-bit indices", nv), IMN_ERR_LIMIT;
  if (nrows == 0) return IMN_OK;
  if (colind_bytes == 4)
    imn::expand_rows_kernel<int><<<(nrows + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
        values, static_cast<const int*>(colind), rowadr, nrows, nv, dense, ld_row);
  else
    imn::expand_rows_kernel<uint8_t><<<(nrows + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
        values, static_cast<const uint8_t*>(colind), rowadr, nrows, nv, dense, ld_row);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return imn::set_error("imn_expand_rows: launch failed: %s", cudaGetErrorString(e)), IMN_ERR_LAUNCH;
  return IMN_OK;
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
