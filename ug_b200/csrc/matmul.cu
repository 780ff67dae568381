// ug::Device::matmul for the B200 backend.
//
// The reference forwards every matmul to cublasGemmStridedBatchedEx after
// deriving transposition flags, leading dimensions and batch strides from the
// two operand layouts (ug-cuda/src/gemm.rs:8-83,292-332).  Here the same
// layout rules pick between
//   * the tcgen05 / TMEM tensor-core kernel (bf16 operands, fp32 accumulate),
//     declared in gemm_tcgen05.cuh, and
//   * a strided SIMT kernel with fp32 accumulation that covers every dtype
//     and every accepted layout (f32 model paths, tiny or odd shapes).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_tcgen05.cuh"
#include "ugb_internal.h"

namespace {

struct MatLayout {
  long long rs, cs;   // element strides of the last two dims
  long long batch;    // element stride between batch steps
  bool transposed;    // true when the minor stride is on the row index
};

// gemm.rs:18-43 (minor dims) and :59-74 (batch stride).  `rows`/`cols` are the
// logical extents of the last two dims (m,k for lhs; k,n for rhs).
int32_t parse_layout(ugb_device *dev, const char *which, int rank, const size_t *dims,
                     const size_t *strides, size_t rows, size_t cols, MatLayout *out) {
  UGB_REQUIRE(dev, rank >= 2 && rank <= 4, UGB_ERR_SHAPE, "matmul: %s rank %d not in 2..4", which, rank);
  const size_t m1 = strides[rank - 1], m2 = strides[rank - 2];
  if ((m1 == 1 || cols == 1) && (m2 == cols || rows == 1)) {
    out->rs = (long long)cols;
    out->cs = 1;
    out->transposed = false;
  } else if ((m1 == rows || cols == 1) && (m2 == 1 || rows == 1)) {
    out->rs = 1;
    out->cs = (long long)rows;
    out->transposed = true;
  } else {
    return ugb_fail(dev, UGB_ERR_SHAPE, "non contiguous matmul, %s strides (..., %zu, %zu) for %zux%zu",
                    which, m2, m1, rows, cols);
  }
  const int nb = rank - 2;
  if (nb == 0) {
    out->batch = (long long)(rows * cols);
  } else if (nb == 1) {
    out->batch = (long long)strides[0];
  } else {
    const size_t s1 = strides[0], s2 = strides[1];
    if (s1 == s2 * dims[1]) out->batch = (long long)s2;
    else if (dims[0] == 1) out->batch = (long long)s2;
    else if (dims[1] == 1) out->batch = (long long)s1;
    else
      return ugb_fail(dev, UGB_ERR_SHAPE, "non contiguous matmul, %s batch strides (%zu, %zu)", which, s1, s2);
  }
  return UGB_OK;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// 64x64 output tile, 16-deep k slices, 256 threads, 4x4 outputs per thread.
template <typename T>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(T *__restrict__ C, const T *__restrict__ A, const T *__restrict__ B, int m, int n,
                 int k, long long a_rs, long long a_cs, long long a_b, long long b_rs,
                 long long b_cs, long long b_b) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 1];
  __shared__ float Bs[BK][BN + 1];
  const int batch = blockIdx.z;
  const T *Ab = A + (long long)batch * a_b;
  const T *Bb = B + (long long)batch * b_b;
  T *Cb = C + (long long)batch * m * n;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += BK) {
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      // walk the contiguous direction of each operand with consecutive threads
      int i, p;
      if (a_cs == 1) { p = e % BK; i = e / BK; } else { i = e % BM; p = e / BM; }
      const int gi = m0 + i, gp = k0 + p;
      As[p][i] = (gi < m && gp < k) ? to_f32<T>(Ab[gi * a_rs + gp * a_cs]) : 0.f;
    }
    for (int e = threadIdx.x; e < BN * BK; e += 256) {
      int j, p;
      if (b_cs == 1) { j = e % BN; p = e / BN; } else { p = e % BK; j = e / BK; }
      const int gj = n0 + j, gp = k0 + p;
      Bs[p][j] = (gj < n && gp < k) ? to_f32<T>(Bb[gp * b_rs + gj * b_cs]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < BK; ++p) {
      float a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) a[u] = As[p][ty * 4 + u];
#pragma unroll
      for (int u = 0; u < 4; ++u) b[u] = Bs[p][tx * 4 + u];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] = fmaf(a[u], b[v], acc[u][v]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int gi = m0 + ty * 4 + u;
    if (gi >= m) continue;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int gj = n0 + tx * 4 + v;
      if (gj < n) Cb[(long long)gi * n + gj] = from_f32<T>(acc[u][v]);
    }
  }
}

template <typename T>
int32_t launch_simt(ugb_device *dev, void *dst, const void *lhs, const void *rhs, size_t b, size_t m,
                    size_t n, size_t k, const MatLayout &L, const MatLayout &R) {
  dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64), (unsigned)b);
  UGB_REQUIRE(dev, grid.y <= 65535 && grid.z <= 65535, UGB_ERR_UNSUPPORTED,
              "matmul: m or batch too large for the SIMT kernel");
  simt_gemm_kernel<T><<<grid, 256, 0, dev->stream>>>((T *)dst, (const T *)lhs, (const T *)rhs,
                                                     (int)m, (int)n, (int)k, L.rs, L.cs, L.batch,
                                                     R.rs, R.cs, R.batch);
  return ugb_after_launch(dev, "simt_gemm_kernel");
}

}  // namespace

extern "C" {

void ugb_gemm_state_free(ugb_device *dev) { ugb_tc_state_free(dev); }

int32_t ugb_matmul(ugb_device *dev, ugb_slice *dst, const ugb_slice *lhs, const ugb_slice *rhs,
                   size_t b, size_t m, size_t n, size_t k, int32_t rank, const size_t *lhs_dims,
                   const size_t *lhs_strides, size_t lhs_off, const size_t *rhs_dims,
                   const size_t *rhs_strides, size_t rhs_off) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, dst && lhs && rhs, UGB_ERR_INVALID, "matmul: null slice");
  UGB_REQUIRE(dev, lhs_dims && lhs_strides && rhs_dims && rhs_strides, UGB_ERR_INVALID,
              "matmul: null layout");
  // gemm.rs:301-331: the three dtypes must agree and be one of bf16/f16/f32.
  const int32_t dt = dst->dtype;
  UGB_REQUIRE(dev, dt == lhs->dtype && dt == rhs->dtype && (dt == UGB_BF16 || dt == UGB_F16 || dt == UGB_F32),
              UGB_ERR_DTYPE, "incorrect dtypes for matmul, dst: %s, lhs: %s, rhs: %s",
              ugb_dtype_name(dst->dtype), ugb_dtype_name(lhs->dtype), ugb_dtype_name(rhs->dtype));
  UGB_REQUIRE(dev, dst->dev == dev && lhs->dev == dev && rhs->dev == dev, UGB_ERR_INVALID,
              "matmul: slice belongs to another device");
  MatLayout L, R;
  int32_t rc = parse_layout(dev, "lhs", rank, lhs_dims, lhs_strides, m, k, &L);
  if (rc) return rc;
  rc = parse_layout(dev, "rhs", rank, rhs_dims, rhs_strides, k, n, &R);
  if (rc) return rc;
  UGB_REQUIRE(dev, m < (1u << 31) && n < (1u << 31) && k < (1u << 31), UGB_ERR_SHAPE, "matmul: extent too large");
  UGB_REQUIRE(dev, dst->len >= b * m * n, UGB_ERR_SHAPE, "matmul: dst holds %zu elements, %zu needed",
              dst->len, b * m * n);
  if (b == 0 || m == 0 || n == 0) return UGB_OK;
  // extent of each operand in elements, from its strides
  auto extent = [&](const MatLayout &X, size_t rows, size_t cols) {
    return (size_t)((long long)(b - 1) * X.batch + (long long)(rows - 1) * X.rs +
                    (long long)(cols - 1) * X.cs + 1);
  };
  if (k > 0) {
    UGB_REQUIRE(dev, lhs->len >= lhs_off + extent(L, m, k), UGB_ERR_SHAPE, "matmul: lhs slice too short");
    UGB_REQUIRE(dev, rhs->len >= rhs_off + extent(R, k, n), UGB_ERR_SHAPE, "matmul: rhs slice too short");
  }
  const size_t es = ugb_dtype_size(dt);
  const char *lp = (const char *)lhs->ptr + lhs_off * es;
  const char *rp = (const char *)rhs->ptr + rhs_off * es;

  // Tiny products do not fill a 128-row tensor-core tile; the strided kernel handles them.
  if (dt == UGB_BF16 && !L.transposed && m >= 16 && m * n >= 128 * 64) {
    // tensor-core path: A [m,k] row-major, B either [n,k] row-major ("TN",
    // matmul_t with a weight) or [k,n] row-major ("NN").
    int32_t trc = ugb_tc_gemm_bf16(dev, dst->ptr, lp, rp, b, m, n, k, L.batch, R.batch, R.transposed);
    if (trc != UGB_ERR_UNSUPPORTED) return trc;
  }
  switch (dt) {
    case UGB_F32: return launch_simt<float>(dev, dst->ptr, lp, rp, b, m, n, k, L, R);
    case UGB_BF16: return launch_simt<__nv_bfloat16>(dev, dst->ptr, lp, rp, b, m, n, k, L, R);
    default: return launch_simt<__half>(dev, dst->ptr, lp, rp, b, m, n, k, L, R);
  }
}

}  // extern "C"
