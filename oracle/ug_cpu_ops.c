/* TEST INFRASTRUCTURE ONLY -- CPU oracle, never part of the shipped library.
 *
 * Restatement in C of the hand-written CPU operators of ug-llama
 * (ug-llama/src/cpu_ops.rs) plus a stand-in for the third-party `gemm` crate
 * that ug-core's CPU backend delegates matmul to (ug-core/src/cpu_runtime.rs:551-619).
 *
 * Arithmetic follows Rust semantics: strict IEEE f32, no reassociation, no
 * fused multiply-add contraction.  The build recipe therefore compiles this
 * file with -fno-fast-math -ffp-contract=off.  Rows are distributed over
 * threads the way rayon's par_chunks does; each row is computed by exactly
 * one thread so results do not depend on the thread count.
 *
 * Parity status: the reference holds no test for these operators
 * (ug-llama has no tests); they are cross-checked against independent
 * float64 numpy computations and, for softmax, against the 2x4 known-answer
 * vector of ug-core/tests/basic_tests.rs:41-116.  The GEMM stand-in is
 * "parity unpinned": the only reference test on that boundary is the
 * all-constant 4x2 . 2x3 product of ug-core/src/common_tests.rs:15-22.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Thread count of the row loops below (rayon uses every core by default;
 * launchers such as torchrun export OMP_NUM_THREADS=1, which would silently
 * serialise the oracle).  Returns the count now in force. */
int ug_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* ug-llama/src/cpu_ops.rs:6-31 -- custom_softmax: per row, running max with
 * f32::max, exp(x - max) written to dst, sequential sum of dst, divide. */
void ug_custom_softmax_f32(const float *src, float *dst, size_t n_rows, size_t n_cols) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t r = 0; r < (ptrdiff_t)n_rows; ++r) {
    const float *s = src + (size_t)r * n_cols;
    float *d = dst + (size_t)r * n_cols;
    float max = -INFINITY;
    for (size_t i = 0; i < n_cols; ++i) max = fmaxf(s[i], max);
    for (size_t i = 0; i < n_cols; ++i) d[i] = expf(s[i] - max);
    float sum_exp = 0.0f;
    for (size_t i = 0; i < n_cols; ++i) sum_exp += d[i];
    for (size_t i = 0; i < n_cols; ++i) d[i] /= sum_exp;
  }
}

/* ug-llama/src/cpu_ops.rs:33-56 -- causal_mask on [bh, s1, s2]: keep i2 <= i1,
 * -inf above the diagonal.  The query block is assumed to start at key 0. */
void ug_causal_mask_f32(const float *src, float *dst, size_t bh, size_t s1, size_t s2) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t b = 0; b < (ptrdiff_t)bh; ++b) {
    const float *s = src + (size_t)b * s1 * s2;
    float *d = dst + (size_t)b * s1 * s2;
    for (size_t i1 = 0; i1 < s1; ++i1) {
      for (size_t i2 = 0; i2 <= i1 && i2 < s2; ++i2) d[i1 * s2 + i2] = s[i1 * s2 + i2];
      for (size_t i2 = i1 + 1; i2 < s2; ++i2) d[i1 * s2 + i2] = -INFINITY;
    }
  }
}

/* ug-llama/src/cpu_ops.rs:91-127 -- rope (half rotation) on [b, h, t, d]:
 * pairs (i_d, i_d + d/2); the table row is pos[0] + i_t for every batch row. */
void ug_rope_f32(const float *src, const float *cos_, const float *sin_, const int32_t *pos,
                 float *dst, size_t b, size_t h, size_t t, size_t d) {
  const size_t p = (size_t)pos[0];
  const float *c = cos_ + p * d / 2;
  const float *s = sin_ + p * d / 2;
#pragma omp parallel for schedule(static)
  for (ptrdiff_t bh = 0; bh < (ptrdiff_t)(b * h); ++bh) {
    const float *x = src + (size_t)bh * t * d;
    float *y = dst + (size_t)bh * t * d;
    for (size_t i_t = 0; i_t < t; ++i_t) {
      for (size_t i_d = 0; i_d < d / 2; ++i_d) {
        size_t i1 = i_t * d + i_d, i2 = i1 + d / 2, i_cs = i_t * (d / 2) + i_d;
        float x1 = x[i1], x2 = x[i2];
        y[i1] = x1 * c[i_cs] - x2 * s[i_cs];
        y[i2] = x1 * s[i_cs] + x2 * c[i_cs];
      }
    }
  }
}

/* ug-llama/src/cpu_ops.rs:58-89 -- rope_i (interleaved) on [b, h, t, d]:
 * pairs (2i, 2i+1), table index i over the flattened (t, d/2) block. */
void ug_rope_i_f32(const float *src, const float *cos_, const float *sin_, const int32_t *pos,
                   float *dst, size_t b, size_t h, size_t t, size_t d) {
  const size_t p = (size_t)pos[0];
  const float *c = cos_ + p * d / 2;
  const float *s = sin_ + p * d / 2;
#pragma omp parallel for schedule(static)
  for (ptrdiff_t bh = 0; bh < (ptrdiff_t)(b * h); ++bh) {
    const float *x = src + (size_t)bh * t * d;
    float *y = dst + (size_t)bh * t * d;
    for (size_t i2 = 0; i2 < t * d / 2; ++i2) {
      size_t i = 2 * i2;
      float x1 = x[i], x2 = x[i + 1];
      y[i] = x1 * c[i2] - x2 * s[i2];
      y[i + 1] = x1 * s[i2] + x2 * c[i2];
    }
  }
}

/* ug-llama/src/cpu_ops.rs:129-167 -- cat along an axis, expressed on the
 * flattened (d1, d2_l) and (d1, d2_r) views; a pure copy. */
void ug_cat_f32(const float *lhs, const float *rhs, float *dst, size_t d1, size_t d2_l,
                size_t d2_r) {
  const size_t d2_lr = d2_l + d2_r;
  for (size_t i1 = 0; i1 < d1; ++i1) {
    memcpy(dst + i1 * d2_lr, lhs + i1 * d2_l, d2_l * sizeof(float));
    memcpy(dst + i1 * d2_lr + d2_l, rhs + i1 * d2_r, d2_r * sizeof(float));
  }
}

/* ug-llama/src/model.rs:32-63 -- index_select: dst[r, :] = emb[ids[r], :].
 * The reference's generated C reads the id through a float variable and
 * multiplies by h; for ids < 2^24 that equals integer indexing, which is what
 * is done here (ids outside [0, vocab) are a caller error in both). */
void ug_index_select_f32(const float *emb, const int32_t *ids, float *dst, size_t n_ids,
                         size_t h) {
  for (size_t r = 0; r < n_ids; ++r)
    memcpy(dst + r * h, emb + (size_t)ids[r] * h, h * sizeof(float));
}

/* Stand-in for crate `gemm` 0.18.0 as called at ug-core/src/cpu_runtime.rs:551-619:
 * dst[step] = lhs[step] . rhs[step] for `b` steps, operands addressed through
 * element strides (row stride rs, column stride cs) and a per-step skip,
 * dst row-major contiguous.  f32 accumulation, k innermost-ordered per
 * output element (the crate's own blocking order is not pinned by any
 * reference test).  Threads split the (step, row) space. */
void ug_gemm_f32(float *dst, const float *lhs, const float *rhs, size_t b, size_t m, size_t n,
                 size_t k, ptrdiff_t lhs_rs, ptrdiff_t lhs_cs, size_t a_skip, ptrdiff_t rhs_rs,
                 ptrdiff_t rhs_cs, size_t b_skip) {
#pragma omp parallel for schedule(static) collapse(2)
  for (ptrdiff_t step = 0; step < (ptrdiff_t)b; ++step) {
    for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
      const float *a = lhs + (size_t)step * a_skip + i * lhs_rs;
      const float *bm = rhs + (size_t)step * b_skip;
      float *c = dst + ((size_t)step * m + (size_t)i) * n;
      if (rhs_cs == 1) {
        /* rhs rows contiguous: accumulate rows of rhs scaled by lhs[i, p]. */
        for (size_t j = 0; j < n; ++j) c[j] = 0.0f;
        for (size_t p = 0; p < k; ++p) {
          const float av = a[(ptrdiff_t)p * lhs_cs];
          const float *br = bm + (ptrdiff_t)p * rhs_rs;
          for (size_t j = 0; j < n; ++j) c[j] += av * br[j];
        }
      } else {
        for (size_t j = 0; j < n; ++j) {
          const float *bc = bm + (ptrdiff_t)j * rhs_cs;
          float acc = 0.0f;
          for (size_t p = 0; p < k; ++p) acc += a[(ptrdiff_t)p * lhs_cs] * bc[(ptrdiff_t)p * rhs_rs];
          c[j] = acc;
        }
      }
    }
  }
}

/* half 2.3.1 bf16 <-> f32 conversions used by the loader's cast matrix
 * (ug-core/src/safetensors.rs:153-157): round to nearest even, NaN kept quiet. */
uint16_t ug_f32_to_bf16_bits(float v) {
  uint32_t x;
  memcpy(&x, &v, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x0040u);
  uint32_t round_bit = 0x00008000u;
  if ((x & round_bit) != 0 && (x & (3 * round_bit - 1)) != 0) return (uint16_t)((x >> 16) + 1);
  return (uint16_t)(x >> 16);
}
float ug_bf16_bits_to_f32(uint16_t h) {
  uint32_t x = (uint32_t)h << 16;
  float v;
  memcpy(&v, &x, 4);
  return v;
}
void ug_round_to_bf16_f32(const float *src, float *dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = ug_bf16_bits_to_f32(ug_f32_to_bf16_bits(src[i]));
}
void ug_f32_to_bf16(const float *src, uint16_t *dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = ug_f32_to_bf16_bits(src[i]);
}
