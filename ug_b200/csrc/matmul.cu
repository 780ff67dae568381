// ug::Device::matmul for the B200 backend.
//
// The reference forwards every matmul to cublasGemmStridedBatchedEx after
// deriving transposition flags, leading dimensions and batch strides from the
// two operand layouts (ug-cuda/src/gemm.rs:8-83,292-332).  Here the same
// layout rules pick between
//   * the tcgen05 / TMEM tensor-core kernel (bf16 operands, fp32 accumulate),
//     declared in gemm_tcgen05.cuh, and
//   * for f32 (the dtype ug-llama casts every weight to, model.rs:118,140,313) two FP32-pipe kernels: a
//     warp-per-column streaming kernel for the skinny products of a decode step and a 128 x 128 register-blocked
//     FFMA kernel for the rest, and
//   * a strided SIMT kernel with fp32 accumulation for bf16 / f16 shapes the tensor-core kernel does not take.
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

// ---- fp32 on the FP32 pipe (the reference's default for f32 is CUBLAS_COMPUTE_32F, gemm.rs:87-128: no reduced
// precision), two shapes -------------------------------------------------------------------------------------
// (1) Skinny products, m <= 16 rows against a [n, k] operand with k contiguous (Linear::fwd = matmul_t with a
// weight, model.rs:147-149, for the one new token of a decode step): HBM-bound on the weight.  One warp per output
// column: the lanes stream the column's k values with 128-bit loads, every value is used for all m rows, the
// partial dot products are summed by warp shuffles.
template <int MR>
__global__ void __launch_bounds__(256)
f32_skinny_kernel(float *__restrict__ C, const float *__restrict__ A, const float *__restrict__ B, int m, int n, int k,
                  long long a_b, long long b_b) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 8 + warp;
  if (col >= n) return;
  const int batch = blockIdx.y;
  const float4 *w = reinterpret_cast<const float4 *>(B + (long long)batch * b_b + (long long)col * k);
  const float *a = A + (long long)batch * a_b;
  float acc[MR];
#pragma unroll
  for (int r = 0; r < MR; ++r) acc[r] = 0.f;
  const int k4 = k >> 2;
#pragma unroll 4
  for (int c = lane; c < k4; c += 32) {
    const float4 wv = __ldcs(w + c);                 // streamed once
#pragma unroll
    for (int r = 0; r < MR; ++r) {
      if (r < m) {
        const float4 x = __ldg(reinterpret_cast<const float4 *>(a + (long long)r * k) + c);
        acc[r] = fmaf(x.x, wv.x, fmaf(x.y, wv.y, fmaf(x.z, wv.z, fmaf(x.w, wv.w, acc[r]))));
      }
    }
  }
#pragma unroll
  for (int r = 0; r < MR; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
    if (lane == 0 && r < m) C[(long long)batch * m * n + (long long)r * n + col] = acc[r];
  }
}

// (1b) Skinny products against a [k, n] operand with n contiguous (Attention::fwd's probabilities x values for the
// one new token, model.rs:243: [1, T] x [T, 64] per head): one CTA per (128-column chunk, batch step); its warps (32 for
// m <= 2, fewer for more rows) split k, a lane keeps 4 adjacent columns, so every k row of the chunk is one coalesced 512-byte read per warp and
// is used for all m rows; the partial sums meet in shared memory.  (The 128 x 128 tile kernel below needs 199 us
// for 32 heads x [1, 1024] x [1024, 64].)
template <int MR>
__global__ void __launch_bounds__(MR <= 2 ? 1024 : (MR <= 4 ? 512 : 256))
f32_skinny_n_kernel(float *__restrict__ C, const float *__restrict__ A, const float *__restrict__ B, int m, int n, int k,
                    long long a_rs, long long a_b, long long b_rs, long long b_b) {
  constexpr int WARPS = MR <= 2 ? 32 : (MR <= 4 ? 16 : 8);       // 32 KiB of partial sums at most
  __shared__ __align__(16) float red[WARPS][MR][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int batch = blockIdx.y, col = blockIdx.x * 128 + lane * 4;
  const float *a = A + (long long)batch * a_b;
  const float *bp = B + (long long)batch * b_b + col;
  float acc[MR][4];
#pragma unroll
  for (int r = 0; r < MR; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
  if (col < n) {                                       // n % 4 == 0: a lane's 4 columns are all in or all out
#pragma unroll 8
    for (int kk = warp; kk < k; kk += WARPS) {
      const float4 bv = __ldcs(reinterpret_cast<const float4 *>(bp + (long long)kk * b_rs));
#pragma unroll
      for (int r = 0; r < MR; ++r) {
        if (r < m) {
          const float x = __ldg(a + (long long)r * a_rs + kk);
          acc[r][0] = fmaf(x, bv.x, acc[r][0]); acc[r][1] = fmaf(x, bv.y, acc[r][1]);
          acc[r][2] = fmaf(x, bv.z, acc[r][2]); acc[r][3] = fmaf(x, bv.w, acc[r][3]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < MR; ++r)
    *reinterpret_cast<float4 *>(&red[warp][r][lane * 4]) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
  __syncthreads();
  for (int i = threadIdx.x; i < MR * 128; i += WARPS * 32) {
    const int r = i >> 7, c = i & 127, gc = blockIdx.x * 128 + c;
    if (r < m && gc < n) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) sum += red[w][r][c];
      C[(long long)batch * m * n + (long long)r * n + gc] = sum;
    }
  }
}

// (2) Everything else in f32: 128 x 128 output tile per CTA, k slices of 8, 256 threads with 8 x 8 outputs each in
// registers (64 FFMA per 16 shared-memory values read), global loads one slice ahead of the arithmetic, 128-bit
// global and shared accesses where the layout allows (VEC), zero fill at the m / n / k tails.
template <bool VEC>
__global__ void __launch_bounds__(256, 2)
f32_tile_kernel(float *__restrict__ C, const float *__restrict__ A, const float *__restrict__ B, int m, int n, int k,
                long long a_rs, long long a_cs, long long a_b, long long b_rs, long long b_cs, long long b_b) {
  constexpr int BM = 128, BN = 128, BK = 8;
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];
  const int batch = blockIdx.z, t = threadIdx.x;
  const float *Ab = A + (long long)batch * a_b;
  const float *Bb = B + (long long)batch * b_b;
  float *Cb = C + (long long)batch * m * n;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  // one 4-element piece of each tile per thread: along the operand's contiguous direction
  const bool a_kc = a_cs == 1, b_nc = b_cs == 1;       // A: k contiguous?  B: n contiguous?
  const int a_i = a_kc ? t >> 1 : (t & 31) * 4, a_p = a_kc ? (t & 1) * 4 : t >> 5;
  const int b_j = b_nc ? (t & 31) * 4 : t >> 1, b_p = b_nc ? t >> 5 : (t & 1) * 4;
  float ra[4], rb[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int gi = m0 + a_i + (a_kc ? 0 : e), gp = k0 + a_p + (a_kc ? e : 0);
      ra[e] = (gi < m && gp < k) ? __ldg(Ab + gi * a_rs + gp * a_cs) : 0.f;
      const int gj = n0 + b_j + (b_nc ? e : 0), gq = k0 + b_p + (b_nc ? 0 : e);
      rb[e] = (gj < n && gq < k) ? __ldg(Bb + gq * b_rs + gj * b_cs) : 0.f;
    }
  };
  auto fetch_vec = [&](int k0) {       // whole pieces inside the matrix, 16-byte aligned (checked by the host)
    const int gi = m0 + a_i, gp = k0 + a_p;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gi < m && gp < k) v = __ldg(reinterpret_cast<const float4 *>(Ab + gi * a_rs + gp * a_cs));
    ra[0] = v.x; ra[1] = v.y; ra[2] = v.z; ra[3] = v.w;
    const int gj = n0 + b_j, gq = k0 + b_p;
    v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gj < n && gq < k) v = __ldg(reinterpret_cast<const float4 *>(Bb + gq * b_rs + gj * b_cs));
    rb[0] = v.x; rb[1] = v.y; rb[2] = v.z; rb[3] = v.w;
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      As[buf][a_p + (a_kc ? e : 0)][a_i + (a_kc ? 0 : e)] = ra[e];
      Bs[buf][b_p + (b_nc ? 0 : e)][b_j + (b_nc ? e : 0)] = rb[e];
    }
  };
  const int tx = t & 15, ty = t >> 4;
  float acc[8][8];
#pragma unroll
  for (int u = 0; u < 8; ++u)
#pragma unroll
    for (int v = 0; v < 8; ++v) acc[u][v] = 0.f;
  if (VEC) fetch_vec(0); else fetch(0);
  stage(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < k; k0 += BK) {
    const bool more = k0 + BK < k;
    if (more) { if (VEC) fetch_vec(k0 + BK); else fetch(k0 + BK); }
#pragma unroll
    for (int p = 0; p < BK; ++p) {
      // rows ty*4 .. +3 and 64 + ty*4 .. +3, columns tx*4 .. +3 and 64 + tx*4 .. +3: conflict-free 128-bit reads
      const float4 a0 = *reinterpret_cast<const float4 *>(&As[buf][p][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4 *>(&As[buf][p][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[buf][p][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[buf][p][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int v = 0; v < 8; ++v) acc[u][v] = fmaf(a[u], b[v], acc[u][v]);
    }
    if (more) {
      stage(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int gi = m0 + (u < 4 ? ty * 4 + u : 64 + ty * 4 + (u - 4));
    if (gi >= m) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int gj = n0 + h * 64 + tx * 4;
      float *crow = Cb + (long long)gi * n + gj;
      if (VEC && gj + 3 < n) {
        *reinterpret_cast<float4 *>(crow) = make_float4(acc[u][4 * h], acc[u][4 * h + 1], acc[u][4 * h + 2], acc[u][4 * h + 3]);
      } else {
#pragma unroll
        for (int v = 0; v < 4; ++v)
          if (gj + v < n) crow[v] = acc[u][4 * h + v];
      }
    }
  }
}

inline bool al16(const void *p) { return ((uintptr_t)p & 15) == 0; }

int32_t launch_f32(ugb_device *dev, float *dst, const float *lhs, const float *rhs, size_t b, size_t m, size_t n, size_t k,
                   const MatLayout &L, const MatLayout &R) {
  if (k == 0) {
    UGB_CUDA(dev, cudaMemsetAsync(dst, 0, b * m * n * sizeof(float), dev->stream));
    return UGB_OK;
  }
  UGB_REQUIRE(dev, b <= 65535, UGB_ERR_UNSUPPORTED, "matmul: batch too large");
  const bool bases = al16(dst) && al16(lhs) && al16(rhs) && L.batch % 4 == 0 && R.batch % 4 == 0;
  if (m <= 16 && !L.transposed && R.transposed && k % 4 == 0 && bases) {
    const dim3 grid((unsigned)((n + 7) / 8), (unsigned)b);
#define UGB_SKINNY(MR) f32_skinny_kernel<MR><<<grid, 256, 0, dev->stream>>>(dst, lhs, rhs, (int)m, (int)n, (int)k, L.batch, R.batch)
    if (m <= 1) UGB_SKINNY(1); else if (m <= 2) UGB_SKINNY(2); else if (m <= 4) UGB_SKINNY(4); else if (m <= 8) UGB_SKINNY(8); else UGB_SKINNY(16);
#undef UGB_SKINNY
    return ugb_after_launch(dev, "f32_skinny_kernel");
  }
  // only the right operand is read in 128-bit pieces: the left rows may start anywhere (their length is the KV length)
  if (m <= 8 && !L.transposed && !R.transposed && (L.cs == 1 || k == 1) && (R.cs == 1 || n == 1) && n % 4 == 0 &&
      R.rs % 4 == 0 && R.batch % 4 == 0 && al16(rhs)) {
    const dim3 grid((unsigned)((n + 127) / 128), (unsigned)b);
#define UGB_SKINNY_N(MR) f32_skinny_n_kernel<MR><<<grid, (MR) <= 2 ? 1024 : ((MR) <= 4 ? 512 : 256), 0, dev->stream>>>(dst, lhs, rhs, (int)m, (int)n, (int)k, L.rs, L.batch, R.rs, R.batch)
    if (m <= 1) UGB_SKINNY_N(1); else if (m <= 2) UGB_SKINNY_N(2); else if (m <= 4) UGB_SKINNY_N(4); else UGB_SKINNY_N(8);
#undef UGB_SKINNY_N
    return ugb_after_launch(dev, "f32_skinny_n_kernel");
  }
  const dim3 grid((unsigned)((n + 127) / 128), (unsigned)((m + 127) / 128), (unsigned)b);
  UGB_REQUIRE(dev, grid.y <= 65535, UGB_ERR_UNSUPPORTED, "matmul: m too large for the f32 kernel");
  // 128-bit pieces: the contiguous extent and the leading stride of each operand in whole float4s
  const size_t a_c = L.transposed ? m : k, a_ld = (size_t)(L.transposed ? L.cs : L.rs);
  const size_t b_c = R.transposed ? k : n, b_ld = (size_t)(R.transposed ? R.cs : R.rs);
  const bool vec = bases && a_c % 4 == 0 && a_ld % 4 == 0 && b_c % 4 == 0 && b_ld % 4 == 0 && n % 4 == 0;
  if (vec) f32_tile_kernel<true><<<grid, 256, 0, dev->stream>>>(dst, lhs, rhs, (int)m, (int)n, (int)k, L.rs, L.cs, L.batch, R.rs, R.cs, R.batch);
  else f32_tile_kernel<false><<<grid, 256, 0, dev->stream>>>(dst, lhs, rhs, (int)m, (int)n, (int)k, L.rs, L.cs, L.batch, R.rs, R.cs, R.batch);
  return ugb_after_launch(dev, "f32_tile_kernel");
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
  if ((dt == UGB_BF16 || dt == UGB_F16) && !L.transposed && m >= 16 && m * n >= 128 * 64) {
    // tensor-core path (bf16 and f16 are the same tcgen05.mma.kind::f16 instruction with another format field, as
    // both go to cublasGemmStridedBatchedEx in the reference, gemm.rs:130-232): A [m,k] row-major, B either
    // [n,k] row-major ("TN", matmul_t with a weight) or [k,n] row-major ("NN").
    int32_t trc = ugb_tc_gemm_bf16(dev, dst->ptr, lp, rp, b, m, n, k, L.batch, R.batch, R.transposed, dt == UGB_F16);
    if (trc != UGB_ERR_UNSUPPORTED) return trc;
  }
  switch (dt) {
    case UGB_F32: return launch_f32(dev, (float *)dst->ptr, (const float *)lp, (const float *)rp, b, m, n, k, L, R);
    case UGB_BF16: return launch_simt<__nv_bfloat16>(dev, dst->ptr, lp, rp, b, m, n, k, L, R);
    default: return launch_simt<__half>(dev, dst->ptr, lp, rp, b, m, n, k, L, R);
  }
}

}  // extern "C"
