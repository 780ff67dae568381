// ug-llama's custom operators (rope, rope_i, cat, causal_mask) plus the
// elementwise / gather kernels the model needs (index_select, residual add,
// silu * up).  All are HBM-bound maps: 128-bit accesses whenever the shapes
// and pointers allow it, scalar otherwise; one thread never touches the same
// element twice.
//
// Results are bit-exact against the reference CPU operators: copies move bits,
// and the rotation uses separately rounded multiplies and adds (no fused
// multiply-add), which is what the reference's Rust arithmetic does
// (ug-llama/src/cpu_ops.rs:73-78,112-117).
#include <algorithm>

#include "ugb_internal.h"

namespace {

constexpr int THREADS = 256;

inline unsigned grid_for(ugb_device *dev, size_t work_items) {
  size_t ctas = (work_items + THREADS - 1) / THREADS;
  size_t cap = (size_t)dev->sm_count * 32;
  if (ctas < 1) ctas = 1;
  return (unsigned)(ctas < cap ? ctas : cap);
}

inline bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

// ---------------------------------------------------------------- rope -----
// src/dst [bh, t, d]; cos/sin [max_pos, d/2]; table row pos[0] + i_t.
// INTERLEAVED: pairs (2i, 2i+1) (cpu_ops.rs:58-89); otherwise (i, i + d/2)
// (cpu_ops.rs:91-127, rope.cu:5-35).
template <bool INTERLEAVED, bool VEC>
__global__ void __launch_bounds__(THREADS)
rope_kernel(const float *__restrict__ src, const float *__restrict__ cos_,
            const float *__restrict__ sin_, const int *__restrict__ pos, float *__restrict__ dst,
            size_t bh, int t, int d, size_t table_len, ugb_status_word *status) {
  const int half = d >> 1;
  // The position lives on the device: a stale or oversized value would index past the cos / sin tables
  // (the reference panics on the slice bound).  Nothing is read or written then; the status word is raised.
  if (pos[0] < 0 || ((size_t)pos[0] + (size_t)t) * half > table_len) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && atomicCAS(&status->code, 0u, (unsigned)UGB_ERR_INVALID) == 0u)
      status->detail = (unsigned)pos[0];
    return;
  }
  const size_t p0 = (size_t)pos[0] * half;
  constexpr int W = VEC ? 4 : 1;  // rotation pairs per thread
  const size_t pairs_per_bh = (size_t)t * half;
  const size_t n_items = bh * pairs_per_bh / W;
  for (size_t it = (size_t)blockIdx.x * THREADS + threadIdx.x; it < n_items;
       it += (size_t)gridDim.x * THREADS) {
    const size_t pair = it * W;              // first pair handled, flattened over (bh, t, d/2)
    const size_t i_bh = pair / pairs_per_bh;
    const size_t r = pair - i_bh * pairs_per_bh;  // = i_t * half + i_d  (the table index)
    const int i_t = (int)(r / half);
    const int i_d = (int)(r - (size_t)i_t * half);
    const size_t base = i_bh * (size_t)t * d + (size_t)i_t * d;
    if constexpr (VEC) {
      const float4 c = *reinterpret_cast<const float4 *>(cos_ + p0 + r);
      const float4 s = *reinterpret_cast<const float4 *>(sin_ + p0 + r);
      if constexpr (INTERLEAVED) {
        const float4 a = __ldcs(reinterpret_cast<const float4 *>(src + base + 2 * i_d));
        const float4 b = __ldcs(reinterpret_cast<const float4 *>(src + base + 2 * i_d + 4));
        float4 oa, ob;
        oa.x = __fsub_rn(__fmul_rn(a.x, c.x), __fmul_rn(a.y, s.x));
        oa.y = __fadd_rn(__fmul_rn(a.x, s.x), __fmul_rn(a.y, c.x));
        oa.z = __fsub_rn(__fmul_rn(a.z, c.y), __fmul_rn(a.w, s.y));
        oa.w = __fadd_rn(__fmul_rn(a.z, s.y), __fmul_rn(a.w, c.y));
        ob.x = __fsub_rn(__fmul_rn(b.x, c.z), __fmul_rn(b.y, s.z));
        ob.y = __fadd_rn(__fmul_rn(b.x, s.z), __fmul_rn(b.y, c.z));
        ob.z = __fsub_rn(__fmul_rn(b.z, c.w), __fmul_rn(b.w, s.w));
        ob.w = __fadd_rn(__fmul_rn(b.z, s.w), __fmul_rn(b.w, c.w));
        __stcs(reinterpret_cast<float4 *>(dst + base + 2 * i_d), oa);
        __stcs(reinterpret_cast<float4 *>(dst + base + 2 * i_d + 4), ob);
      } else {
        const float4 a = __ldcs(reinterpret_cast<const float4 *>(src + base + i_d));
        const float4 b = __ldcs(reinterpret_cast<const float4 *>(src + base + i_d + half));
        float4 oa, ob;
        oa.x = __fsub_rn(__fmul_rn(a.x, c.x), __fmul_rn(b.x, s.x));
        oa.y = __fsub_rn(__fmul_rn(a.y, c.y), __fmul_rn(b.y, s.y));
        oa.z = __fsub_rn(__fmul_rn(a.z, c.z), __fmul_rn(b.z, s.z));
        oa.w = __fsub_rn(__fmul_rn(a.w, c.w), __fmul_rn(b.w, s.w));
        ob.x = __fadd_rn(__fmul_rn(a.x, s.x), __fmul_rn(b.x, c.x));
        ob.y = __fadd_rn(__fmul_rn(a.y, s.y), __fmul_rn(b.y, c.y));
        ob.z = __fadd_rn(__fmul_rn(a.z, s.z), __fmul_rn(b.z, c.z));
        ob.w = __fadd_rn(__fmul_rn(a.w, s.w), __fmul_rn(b.w, c.w));
        __stcs(reinterpret_cast<float4 *>(dst + base + i_d), oa);
        __stcs(reinterpret_cast<float4 *>(dst + base + i_d + half), ob);
      }
    } else {
      const float c = cos_[p0 + r], s = sin_[p0 + r];
      const size_t i1 = INTERLEAVED ? base + 2 * (size_t)i_d : base + i_d;
      const size_t i2 = INTERLEAVED ? i1 + 1 : i1 + half;
      const float x1 = src[i1], x2 = src[i2];
      dst[i1] = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
      dst[i2] = __fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c));
    }
  }
}

// ----------------------------------------------------------------- cat -----
// dst [d1, d2_l + d2_r] = lhs [d1, d2_l] || rhs [d1, d2_r]   (cat.cu:5-36)
template <typename T>
__global__ void __launch_bounds__(THREADS)
cat_kernel(const T *__restrict__ lhs, const T *__restrict__ rhs, T *__restrict__ dst, size_t d1,
           size_t d2_l, size_t d2_r) {
  const size_t d2_lr = d2_l + d2_r;
  const size_t n = d1 * d2_lr;
  for (size_t i = (size_t)blockIdx.x * THREADS + threadIdx.x; i < n;
       i += (size_t)gridDim.x * THREADS) {
    const size_t row = i / d2_lr, col = i - row * d2_lr;
    dst[i] = col < d2_l ? lhs[row * d2_l + col] : rhs[row * d2_r + (col - d2_l)];
  }
}

// --------------------------------------------------------- causal mask -----
template <typename T, int W>
__global__ void __launch_bounds__(THREADS)
causal_mask_kernel(const T *__restrict__ src, T *__restrict__ dst, size_t n_items, int s1, int s2w) {
  // one item = W consecutive columns; s2w = s2 / W items per row
  for (size_t i = (size_t)blockIdx.x * THREADS + threadIdx.x; i < n_items;
       i += (size_t)gridDim.x * THREADS) {
    const size_t rowg = i / s2w;
    const int i2 = (int)(i - rowg * s2w) * W;
    const int i1 = (int)(rowg % s1);
    if constexpr (W == 1) {
      dst[i] = i2 <= i1 ? src[i] : -INFINITY;
    } else {
      float4 v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      if (i2 <= i1) {  // at least one kept column: read, then mask the tail
        v = __ldcs(reinterpret_cast<const float4 *>(src) + i);
        if (i2 + 1 > i1) v.y = -INFINITY;
        if (i2 + 2 > i1) v.z = -INFINITY;
        if (i2 + 3 > i1) v.w = -INFINITY;
      }
      __stcs(reinterpret_cast<float4 *>(dst) + i, v);
    }
  }
}

// -------------------------------------------------------- index_select -----
// Four rows per CTA and pass: the ids, then all four rows' loads, are requested before anything is stored, so a
// CTA has 4 rows in flight instead of one (a gather of 16384 rows of 8 KB: 5.4 -> 6.2 TB/s).
template <typename T>
__global__ void __launch_bounds__(THREADS)
index_select_kernel(const T *__restrict__ emb, const int *__restrict__ ids, T *__restrict__ dst,
                    size_t n_ids, size_t hw, int vocab, ugb_status_word *status) {
  // hw = row length in units of T
  constexpr int R = 4;
  for (size_t r0 = (size_t)blockIdx.x * R; r0 < n_ids; r0 += (size_t)gridDim.x * R) {
    const T *s[R];
    bool ok[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const size_t r = r0 + j;
      const int id = r < n_ids ? ids[r] : 0;
      ok[j] = r < n_ids && id >= 0 && id < vocab;
      if (r < n_ids && !ok[j] && threadIdx.x == 0) {
        atomicCAS(&status->code, 0u, (unsigned)UGB_ERR_INVALID);
        status->detail = (unsigned)r;
      }
      s[j] = emb + (size_t)(ok[j] ? id : 0) * hw;
    }
    for (size_t c = threadIdx.x; c < hw; c += THREADS) {
      T v[R];
#pragma unroll
      for (int j = 0; j < R; ++j)
        if (ok[j]) v[j] = s[j][c];
#pragma unroll
      for (int j = 0; j < R; ++j)
        if (ok[j]) dst[(r0 + j) * hw + c] = v[j];
    }
  }
}

// ---------------------------------------------------------- elementwise ----
enum MapOp { MAP_ADD = 0, MAP_SILU_MUL = 1 };
__device__ __forceinline__ float silu(float g) { return g / (expf(-g) + 1.0f); }
template <int OP>
__device__ __forceinline__ float map2(float a, float b) {
  return OP == MAP_ADD ? a + b : silu(a) * b;
}
template <int OP, bool VEC>
__global__ void __launch_bounds__(THREADS)
map2_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ y, size_t n) {
  if constexpr (VEC) {
    const size_t nv = n >> 2;
    for (size_t i = (size_t)blockIdx.x * THREADS + threadIdx.x; i < nv;
         i += (size_t)gridDim.x * THREADS) {
      const float4 u = __ldcs(reinterpret_cast<const float4 *>(a) + i);
      const float4 v = __ldcs(reinterpret_cast<const float4 *>(b) + i);
      __stcs(reinterpret_cast<float4 *>(y) + i,
             make_float4(map2<OP>(u.x, v.x), map2<OP>(u.y, v.y), map2<OP>(u.z, v.z), map2<OP>(u.w, v.w)));
    }
    // tail (n % 4 elements)
    const size_t t = (nv << 2) + (size_t)blockIdx.x * THREADS + threadIdx.x;
    if (t < n) y[t] = map2<OP>(a[t], b[t]);
  } else {
    for (size_t i = (size_t)blockIdx.x * THREADS + threadIdx.x; i < n;
         i += (size_t)gridDim.x * THREADS)
      y[i] = map2<OP>(a[i], b[i]);
  }
}

template <bool INTERLEAVED>
int32_t rope_impl(ugb_device *dev, const ugb_slice *src, const ugb_slice *cos,
                  const ugb_slice *sin, const ugb_slice *pos, ugb_slice *dst, size_t b, size_t h,
                  size_t t, size_t d) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, d % 2 == 0, UGB_ERR_SHAPE, "rope: head dim %zu is odd", d);
  UGB_REQUIRE(dev, t < (1u << 30) && d < (1u << 30), UGB_ERR_SHAPE, "rope: t or d too large");
  const size_t n = b * h * t * d;
  UGB_SLICE(dev, src, UGB_F32, n);
  UGB_SLICE(dev, dst, UGB_F32, n);
  UGB_SLICE(dev, cos, UGB_F32, t * d / 2);
  UGB_SLICE(dev, sin, UGB_F32, t * d / 2);
  UGB_SLICE(dev, pos, UGB_I32, 1);
  if (n == 0) return UGB_OK;
  // The table offset pos[0] * d/2 is only known on the device; vector access to
  // the tables needs d/2 % 4 == 0 so that every offset stays 16-byte aligned.
  const bool vec = (d % 8 == 0) && aligned16(src->ptr) && aligned16(dst->ptr) &&
                   aligned16(cos->ptr) && aligned16(sin->ptr);
  const size_t pairs = n / 2;
  if (vec)
    rope_kernel<INTERLEAVED, true><<<grid_for(dev, pairs / 4), THREADS, 0, dev->stream>>>(
        (const float *)src->ptr, (const float *)cos->ptr, (const float *)sin->ptr,
        (const int *)pos->ptr, (float *)dst->ptr, b * h, (int)t, (int)d, std::min(cos->len, sin->len), dev->status_dev);
  else
    rope_kernel<INTERLEAVED, false><<<grid_for(dev, pairs), THREADS, 0, dev->stream>>>(
        (const float *)src->ptr, (const float *)cos->ptr, (const float *)sin->ptr,
        (const int *)pos->ptr, (float *)dst->ptr, b * h, (int)t, (int)d, std::min(cos->len, sin->len), dev->status_dev);
  return ugb_after_launch(dev, "rope_kernel");
}

template <int OP>
int32_t map2_impl(ugb_device *dev, const ugb_slice *a, const ugb_slice *b, ugb_slice *dst, size_t n) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_SLICE(dev, a, UGB_F32, n);
  UGB_SLICE(dev, b, UGB_F32, n);
  UGB_SLICE(dev, dst, UGB_F32, n);
  if (n == 0) return UGB_OK;
  const bool vec = aligned16(a->ptr) && aligned16(b->ptr) && aligned16(dst->ptr) && n >= 4;
  if (vec)
    map2_kernel<OP, true><<<grid_for(dev, n / 4), THREADS, 0, dev->stream>>>(
        (const float *)a->ptr, (const float *)b->ptr, (float *)dst->ptr, n);
  else
    map2_kernel<OP, false><<<grid_for(dev, n), THREADS, 0, dev->stream>>>(
        (const float *)a->ptr, (const float *)b->ptr, (float *)dst->ptr, n);
  return ugb_after_launch(dev, "map2_kernel");
}

}  // namespace

extern "C" {

int32_t ugb_rope(ugb_device *dev, const ugb_slice *src, const ugb_slice *cos,
                 const ugb_slice *sin, const ugb_slice *pos, ugb_slice *dst, size_t b, size_t h,
                 size_t t, size_t d) {
  return rope_impl<false>(dev, src, cos, sin, pos, dst, b, h, t, d);
}

int32_t ugb_rope_i(ugb_device *dev, const ugb_slice *src, const ugb_slice *cos,
                   const ugb_slice *sin, const ugb_slice *pos, ugb_slice *dst, size_t b,
                   size_t h, size_t t, size_t d) {
  return rope_impl<true>(dev, src, cos, sin, pos, dst, b, h, t, d);
}

int32_t ugb_cat(ugb_device *dev, const ugb_slice *lhs, const ugb_slice *rhs, ugb_slice *dst,
                size_t d1, size_t d2_l, size_t d2_r) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_SLICE(dev, lhs, UGB_F32, d1 * d2_l);
  UGB_SLICE(dev, rhs, UGB_F32, d1 * d2_r);
  UGB_SLICE(dev, dst, UGB_F32, d1 * (d2_l + d2_r));
  const size_t n = d1 * (d2_l + d2_r);
  if (n == 0) return UGB_OK;
  const bool vec = d2_l % 4 == 0 && d2_r % 4 == 0 && (lhs->ptr == nullptr || aligned16(lhs->ptr)) &&
                   (rhs->ptr == nullptr || aligned16(rhs->ptr)) && aligned16(dst->ptr);
  if (vec)
    cat_kernel<float4><<<grid_for(dev, n / 4), THREADS, 0, dev->stream>>>(
        (const float4 *)lhs->ptr, (const float4 *)rhs->ptr, (float4 *)dst->ptr, d1, d2_l / 4, d2_r / 4);
  else
    cat_kernel<float><<<grid_for(dev, n), THREADS, 0, dev->stream>>>(
        (const float *)lhs->ptr, (const float *)rhs->ptr, (float *)dst->ptr, d1, d2_l, d2_r);
  return ugb_after_launch(dev, "cat_kernel");
}

int32_t ugb_causal_mask(ugb_device *dev, const ugb_slice *src, ugb_slice *dst, size_t bh,
                        size_t s1, size_t s2) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, s1 < (1u << 31) && s2 < (1u << 31), UGB_ERR_SHAPE, "causal_mask: s1/s2 too large");
  const size_t n = bh * s1 * s2;
  UGB_SLICE(dev, src, UGB_F32, n);
  UGB_SLICE(dev, dst, UGB_F32, n);
  if (n == 0) return UGB_OK;
  const bool vec = s2 % 4 == 0 && aligned16(src->ptr) && aligned16(dst->ptr);
  if (vec)
    causal_mask_kernel<float, 4><<<grid_for(dev, n / 4), THREADS, 0, dev->stream>>>(
        (const float *)src->ptr, (float *)dst->ptr, n / 4, (int)s1, (int)(s2 / 4));
  else
    causal_mask_kernel<float, 1><<<grid_for(dev, n), THREADS, 0, dev->stream>>>(
        (const float *)src->ptr, (float *)dst->ptr, n, (int)s1, (int)s2);
  return ugb_after_launch(dev, "causal_mask_kernel");
}

int32_t ugb_index_select(ugb_device *dev, const ugb_slice *emb, const ugb_slice *ids,
                         ugb_slice *dst, size_t n_ids, size_t h, size_t vocab) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, vocab < (1u << 31), UGB_ERR_SHAPE, "index_select: vocab too large");
  UGB_SLICE(dev, emb, UGB_F32, vocab * h);
  UGB_SLICE(dev, ids, UGB_I32, n_ids);
  UGB_SLICE(dev, dst, UGB_F32, n_ids * h);
  if (n_ids == 0 || h == 0) return UGB_OK;
  const size_t cap = (size_t)dev->sm_count * 16, groups = (n_ids + 3) / 4;     // 4 rows per CTA and pass
  const unsigned grid = (unsigned)(groups < cap ? groups : cap);
  if (h % 4 == 0 && aligned16(emb->ptr) && aligned16(dst->ptr))
    index_select_kernel<float4><<<grid, THREADS, 0, dev->stream>>>(
        (const float4 *)emb->ptr, (const int *)ids->ptr, (float4 *)dst->ptr, n_ids, h / 4,
        (int)vocab, dev->status_dev);
  else
    index_select_kernel<float><<<grid, THREADS, 0, dev->stream>>>(
        (const float *)emb->ptr, (const int *)ids->ptr, (float *)dst->ptr, n_ids, h, (int)vocab,
        dev->status_dev);
  return ugb_after_launch(dev, "index_select_kernel");
}

int32_t ugb_add(ugb_device *dev, const ugb_slice *a, const ugb_slice *b, ugb_slice *dst, size_t n) {
  return map2_impl<MAP_ADD>(dev, a, b, dst, n);
}

int32_t ugb_silu_mul(ugb_device *dev, const ugb_slice *gate, const ugb_slice *up, ugb_slice *dst,
                     size_t n) {
  return map2_impl<MAP_SILU_MUL>(dev, gate, up, dst, n);
}

}  // extern "C"
