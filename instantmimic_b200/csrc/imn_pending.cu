// Entry points whose kernels are not written yet: they refuse the call.
#include "imn_common.cuh"
extern "C" int imn_sparse_factor_nonfused(const ImnSparsePlan*, const uint8_t*, const float*, int64_t,
                                          const float*, const int32_t*, const int32_t*, float*, float*,
                                          int64_t, float*, float*, int32_t, int32_t, int32_t, void*) {
  return imn::set_error("imn_sparse_factor_nonfused: not implemented"), IMN_ERR_UNSUPPORTED;
}
