// Interface of the tcgen05 / TMEM bf16 GEMM translation unit.
#pragma once
#include "ugb_internal.h"

// C[b, m, n] (bf16, row-major) = A[b, m, k] (bf16, row-major) x B, fp32
// accumulation.  `b_is_nk`: B is [n, k] row-major (the matmul_t / weight
// layout), otherwise [k, n] row-major.  Batch strides in elements (0 = shared
// operand).  Returns UGB_ERR_UNSUPPORTED (without touching last_error) when
// the shape does not meet the kernel's alignment rules so that the caller can
// fall back to the strided kernel.
int32_t ugb_tc_gemm_bf16(ugb_device *dev, void *c, const void *a, const void *b_, size_t batch,
                         size_t m, size_t n, size_t k, long long a_batch, long long b_batch,
                         bool b_is_nk);
void ugb_tc_state_free(ugb_device *dev);
