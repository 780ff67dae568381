/* TEST INFRASTRUCTURE ONLY -- CPU oracle, never part of the shipped library.
 *
 * The C that ug-core's CPU backend emits for the lazy-graph forms of the
 * row operators, written out by hand in the statement shape of
 * ug-core/src/cpu_code_gen.rs:68-186 (one typed local per SSA value, plain
 * `for (int v = lo; v < up; v += step)` loops, fmax/expf/sqrtf calls) with the
 * loop structure that ug-core/src/lower_op.rs:409-491 produces under the
 * default lowering options: every destination dimension is a sequential
 * loop and a reduction is an accumulator loop nested INSIDE the loop over
 * the reduced dimension (lower_op.rs:364-391), so a row operator costs
 * O(rows * cols^2).  Index arithmetic is 32-bit int (lower_op.rs:90-92).
 *
 * The build recipe compiles this file with exactly the reference's command
 * line (ug-core/src/cpu_runtime.rs:476-488):
 *   gcc -shared -lm -O3 -march=native -ffast-math -fomit-frame-pointer
 * The CPU backend is single threaded by construction (cpu_code_gen.rs:160-167).
 *
 * Each function takes [row_lo, row_hi) so that a timing run can cover a
 * stated subset of rows; the reference always runs all rows.
 *
 * Parity status: pinned by the 2x4 softmax known-answer vector of
 * ug-core/tests/basic_tests.rs:41-61 (same op::softmax graph, default
 * lowering); rms_norm / silu have no reference test and are cross-checked
 * against float64 numpy.
 */
#include <math.h>

/* ug-llama/src/model.rs:94-101 softmax, first scheduled kernel: `exp` has two
 * users so the scheduler materialises it (ug-core/src/schedule.rs:429-435).
 *   e[r, c] = exp(x[r, c] - max_k x[r, k])                                   */
void ug_gen_softmax_exp(float *__var0 /* x */, float *__var1 /* e */, int n_rows, int n_cols,
                        int row_lo, int row_hi) {
  (void)n_rows;
  for (int __var2 = row_lo; __var2 < row_hi; __var2 += 1) {
    for (int __var3 = 0; __var3 < n_cols; __var3 += 1) {
      int __var4 = __var2 * n_cols;
      int __var5 = __var3 + __var4;
      float __var6 = __var0[__var5];
      float __var7 = -1. / 0.;
      for (int __var8 = 0; __var8 < n_cols; __var8 += 1) {
        int __var9 = __var2 * n_cols;
        int __var10 = __var8 + __var9;
        float __var11 = __var0[__var10];
        float __var12 = fmax(__var7, __var11);
        __var7 = __var12;
      }
      float __var13 = __var6 - __var7;
      float __var14 = expf(__var13);
      __var1[__var5] = __var14;
    }
  }
}

/* Second scheduled kernel:  y[r, c] = e[r, c] / sum_k e[r, k]               */
void ug_gen_softmax_div(float *__var0 /* e */, float *__var1 /* y */, int n_rows, int n_cols,
                        int row_lo, int row_hi) {
  (void)n_rows;
  for (int __var2 = row_lo; __var2 < row_hi; __var2 += 1) {
    for (int __var3 = 0; __var3 < n_cols; __var3 += 1) {
      int __var4 = __var2 * n_cols;
      int __var5 = __var3 + __var4;
      float __var6 = __var0[__var5];
      float __var7 = 0.0;
      for (int __var8 = 0; __var8 < n_cols; __var8 += 1) {
        int __var9 = __var2 * n_cols;
        int __var10 = __var8 + __var9;
        float __var11 = __var0[__var10];
        float __var12 = __var7 + __var11;
        __var7 = __var12;
      }
      float __var13 = __var6 / __var7;
      __var1[__var5] = __var13;
    }
  }
}

/* ug-llama/src/model.rs:65-78 rms_norm as one fused kernel:
 *   y[r, c] = x[r, c] / sqrt(sum_k x[r, k]^2 * (1/d) + eps) * alpha[c]
 * `inv_d` is 1f32 / d as f32 rounded once on the host, as the graph builder
 * does when it creates the constant node.                                    */
void ug_gen_rms_norm(float *__var0 /* x */, float *__var1 /* alpha */, float *__var2 /* y */,
                     int n_rows, int n_cols, float inv_d, float eps, int row_lo, int row_hi) {
  (void)n_rows;
  for (int __var3 = row_lo; __var3 < row_hi; __var3 += 1) {
    for (int __var4 = 0; __var4 < n_cols; __var4 += 1) {
      int __var5 = __var3 * n_cols;
      int __var6 = __var4 + __var5;
      float __var7 = __var0[__var6];
      float __var8 = 0.0;
      for (int __var9 = 0; __var9 < n_cols; __var9 += 1) {
        int __var10 = __var3 * n_cols;
        int __var11 = __var9 + __var10;
        float __var12 = __var0[__var11];
        float __var13 = __var0[__var11];
        float __var14 = __var12 * __var13;
        float __var15 = __var8 + __var14;
        __var8 = __var15;
      }
      float __var16 = inv_d;
      float __var17 = __var8 * __var16;
      float __var18 = eps;
      float __var19 = __var17 + __var18;
      float __var20 = sqrtf(__var19);
      float __var21 = __var7 / __var20;
      float __var22 = __var1[__var4];
      float __var23 = __var21 * __var22;
      __var2[__var6] = __var23;
    }
  }
}

/* rms_norm(x) * alpha * silu(gate) as the single kernel the scheduler forms
 * for it (no node has two users, both inputs are realised buffers):
 * ug-llama/src/model.rs:65-78 and :103-109, silu(g) = g / (exp(-g) + 1).     */
void ug_gen_rms_norm_silu_gate(float *__var0 /* x */, float *__var1 /* alpha */,
                               float *__var2 /* gate */, float *__var3 /* y */, int n_rows,
                               int n_cols, float inv_d, float eps, int row_lo, int row_hi) {
  (void)n_rows;
  for (int __var4 = row_lo; __var4 < row_hi; __var4 += 1) {
    for (int __var5 = 0; __var5 < n_cols; __var5 += 1) {
      int __var6 = __var4 * n_cols;
      int __var7 = __var5 + __var6;
      float __var8 = __var0[__var7];
      float __var9 = 0.0;
      for (int __var10 = 0; __var10 < n_cols; __var10 += 1) {
        int __var11 = __var4 * n_cols;
        int __var12 = __var10 + __var11;
        float __var13 = __var0[__var12];
        float __var14 = __var0[__var12];
        float __var15 = __var13 * __var14;
        float __var16 = __var9 + __var15;
        __var9 = __var16;
      }
      float __var17 = inv_d;
      float __var18 = __var9 * __var17;
      float __var19 = eps;
      float __var20 = __var18 + __var19;
      float __var21 = sqrtf(__var20);
      float __var22 = __var8 / __var21;
      float __var23 = __var1[__var5];
      float __var24 = __var22 * __var23;
      float __var25 = __var2[__var7];
      float __var26 = __var2[__var7];
      float __var27 = -(__var26);
      float __var28 = expf(__var27);
      float __var29 = 1.0;
      float __var30 = __var28 + __var29;
      float __var31 = __var25 / __var30;
      float __var32 = __var24 * __var31;
      __var3[__var7] = __var32;
    }
  }
}

/* silu(gate) * up, ug-llama/src/model.rs:103-109,160-168: a pure map that
 * Kernel::optimize collapses to one dimension (lower_op.rs:493-535).        */
void ug_gen_silu_mul(float *__var0 /* gate */, float *__var1 /* up */, float *__var2 /* y */,
                     int n) {
  for (int __var3 = 0; __var3 < n; __var3 += 1) {
    float __var4 = __var0[__var3];
    float __var5 = __var0[__var3];
    float __var6 = -(__var5);
    float __var7 = expf(__var6);
    float __var8 = 1.0;
    float __var9 = __var7 + __var8;
    float __var10 = __var4 / __var9;
    float __var11 = __var1[__var3];
    float __var12 = __var10 * __var11;
    __var2[__var3] = __var12;
  }
}

/* Elementwise add (residual), ug-llama/src/model.rs:263,267.                */
void ug_gen_add(float *__var0, float *__var1, float *__var2, int n) {
  for (int __var3 = 0; __var3 < n; __var3 += 1) {
    float __var4 = __var0[__var3];
    float __var5 = __var1[__var3];
    float __var6 = __var4 + __var5;
    __var2[__var3] = __var6;
  }
}
