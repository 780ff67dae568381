#include "gemm_tcgen05.cuh"
int32_t ugb_tc_gemm_bf16(ugb_device *, void *, const void *, const void *, size_t, size_t, size_t,
                         size_t, long long, long long, bool) {
  return UGB_ERR_UNSUPPORTED;
}
void ugb_tc_state_free(ugb_device *) {}
