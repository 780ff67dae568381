// TEST INFRASTRUCTURE ONLY -- host launchers for the reference's own CUDA
// kernels (ug-llama/src/softmax.cu, rope.cu, cat.cu).  The kernel sources are
// NOT part of this repository: oracle/build_ref.py compiles this file with the
// reference's source directory on the include path, so the three #includes
// below pull the kernels in where they lie, and writes the result to
// oracle/_ref/.  Launch shapes follow ug-llama/src/cuda_ops.rs:
//   softmax_f32  grid n_rows, block (1, 32, 1)             (cuda_ops.rs:149-157)
//   rope_f32     LaunchConfig::for_num_elems(b*h*t*d / 2)  (cuda_ops.rs:60)
//   cat_f32      grid d1, block 32                          (cuda_ops.rs:118-122)
// ropei.cu is left out: it does not compile (it names undeclared variables).
// The reference builds these with NVRTC's use_fast_math; the recipe passes the
// same flag to nvcc.  Used by the tests as a second check of this backend's
// kernels and by the benchmark as the "reference kernel on the same box" figure.
#include <cuda_runtime.h>

#include "softmax.cu"
#include "rope.cu"
#include "cat.cu"

extern "C" {

int ugref_softmax_f32(const float *src, float *dst, int n_rows, int n_cols, void *stream) {
  if (n_rows <= 0) return 0;
  softmax_f32<<<dim3(n_rows, 1, 1), dim3(1, 32, 1), 0, (cudaStream_t)stream>>>(src, dst, n_cols);
  return (int)cudaGetLastError();
}

int ugref_rope_f32(const float *src, const float *cos, const float *sin, const int *pos, float *dst, unsigned b,
                   unsigned h, unsigned t, unsigned d, void *stream) {
  const unsigned n = b * h * t * d / 2;
  if (n == 0) return 0;
  // cudarc's LaunchConfig::for_num_elems: 1024 threads per block (ug-cuda re-exports cudarc's type)
  rope_f32<<<(n + 1023) / 1024, 1024, 0, (cudaStream_t)stream>>>(src, cos, sin, pos, dst, b * h, t * d, d);
  return (int)cudaGetLastError();
}

int ugref_cat_f32(const float *lhs, const float *rhs, float *dst, unsigned d1, unsigned d2_l, unsigned d2_r, void *stream) {
  if (d1 == 0) return 0;
  cat_f32<<<d1, 32, 0, (cudaStream_t)stream>>>(lhs, rhs, dst, d1, d2_l, d2_r, d2_l + d2_r);
  return (int)cudaGetLastError();
}

}  // extern "C"
