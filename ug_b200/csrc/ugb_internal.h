// Internal definitions shared by the translation units of libugb200.so.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/ugb200.h"

// Device-side status word layout (one per device handle, read at ugb_sync).
struct ugb_status_word {
  unsigned int code;           // 0 = ok, otherwise a ugb_status value
  unsigned int detail;         // kernel-specific (bad index, wait site, ...)
  unsigned int wait_limit_us;  // how long a device-side wait (mbarrier, peer flag, grid barrier) may last before it
                               // gives up with UGB_ERR_TIMEOUT; device option "wait_limit_us", default 2 s
  unsigned int pad;
};
constexpr unsigned int UGB_DEFAULT_WAIT_LIMIT_US = 2000000u;

struct ugb_device {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
  ugb_status_word *status_dev = nullptr;  // device memory
  int *sched_dev = nullptr;               // device memory: two work counters that persistent kernels leave at zero
  uint64_t launches = 0;
  int sm_count = 148;
  size_t smem_optin = 0;
  std::string last_error;
  void *gemm_state = nullptr;  // owned by the GEMM translation unit
  int gemm_pair = 1;           // option gemm_cta_pairs: tall bf16 GEMMs on pairs of CTAs (tcgen05 cta_group::2)
  cudaMemPool_t pool = nullptr;  // this handle's own stream-ordered pool (the process-wide default pool is left alone)
  unsigned wait_timeouts = 0;  // device-side waits that gave up, as seen by ugb_sync (tensor-parallel models refuse
                               // further steps once this has moved: their ranks may be out of step)
};

struct ugb_slice {
  ugb_device *dev = nullptr;
  void *ptr = nullptr;
  size_t len = 0;  // elements
  int32_t dtype = UGB_F32;
  bool owned = true;
};

static inline size_t ugb_dtype_size(int32_t dt) {
  switch (dt) {
    case UGB_BF16:
    case UGB_F16:
      return 2;
    case UGB_F32:
    case UGB_I32:
      return 4;
    case UGB_I64:
      return 8;
    default:
      return 0;
  }
}
static inline const char *ugb_dtype_name(int32_t dt) {
  switch (dt) {
    case UGB_BF16: return "BF16";
    case UGB_F16: return "F16";
    case UGB_F32: return "F32";
    case UGB_I32: return "I32";
    case UGB_I64: return "I64";
    default: return "?";
  }
}

// Stream-ordered allocation from the handle's own pool.
static inline cudaError_t ugb_malloc_async(ugb_device *dev, void **p, size_t bytes) {
  return dev->pool ? cudaMallocFromPoolAsync(p, bytes, dev->pool, dev->stream) : cudaMallocAsync(p, bytes, dev->stream);
}

// Records a formatted message on the device handle and returns `code`.
int32_t ugb_fail(ugb_device *dev, int32_t code, const char *fmt, ...);
// Checks the launch error of the kernel just enqueued and counts it.
int32_t ugb_after_launch(ugb_device *dev, const char *what);

#define UGB_CUDA(dev, call)                                                           \
  do {                                                                                \
    cudaError_t e__ = (call);                                                         \
    if (e__ != cudaSuccess)                                                           \
      return ugb_fail((dev), e__ == cudaErrorMemoryAllocation ? UGB_ERR_OOM : UGB_ERR_CUDA, \
                      "%s failed: %s", #call, cudaGetErrorString(e__));               \
  } while (0)

#define UGB_REQUIRE(dev, cond, code, ...) \
  do {                                    \
    if (!(cond)) return ugb_fail((dev), (code), __VA_ARGS__); \
  } while (0)

// Common argument checks for typed slices.
static inline int32_t ugb_check_slice(ugb_device *dev, const ugb_slice *s, int32_t dtype,
                                      size_t min_len, const char *name) {
  if (!s) return ugb_fail(dev, UGB_ERR_INVALID, "%s: null slice", name);
  if (s->dev != dev) return ugb_fail(dev, UGB_ERR_INVALID, "%s: slice belongs to another device", name);
  if (s->dtype != dtype)
    return ugb_fail(dev, UGB_ERR_DTYPE, "dtype mismatch for %s, expected %s, got %s", name,
                    ugb_dtype_name(dtype), ugb_dtype_name(s->dtype));
  if (s->len < min_len)
    return ugb_fail(dev, UGB_ERR_SHAPE, "%s: slice holds %zu elements, %zu needed", name, s->len,
                    min_len);
  return UGB_OK;
}
#define UGB_SLICE(dev, s, dtype, min_len)                                 \
  do {                                                                    \
    int32_t rc__ = ugb_check_slice((dev), (s), (dtype), (min_len), #s);   \
    if (rc__ != UGB_OK) return rc__;                                      \
  } while (0)

// ---- programmatic dependent launch ------------------------------------------
// A kernel launched with ugb_launch(..., pdl = true) may start while the kernel
// before it on the stream is still running.  It must execute ugb_pdl_wait()
// before it reads or writes anything an earlier kernel touches (the wait returns
// once the preceding kernel has completed and its writes are visible); what it
// does before that (barrier set-up, TMEM allocation, loads of weights that no
// kernel writes) overlaps the predecessor's tail.  ugb_pdl_trigger() lets the
// NEXT kernel on the stream begin its own preamble.  Both are no-ops in a
// kernel launched the ordinary way.
#ifdef __CUDACC__
__device__ __forceinline__ void ugb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ugb_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t ugb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              bool pdl, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// The same with thread-block clusters of `cluster` consecutive CTAs (1 = none); grid.x a multiple of it.
template <typename... KArgs, typename... Args>
inline cudaError_t ugb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                      bool pdl, int cluster, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif
