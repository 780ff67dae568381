// Stand-alone entry point of the grouped-query decode attention kernel
// (decode_kernels.cuh), the fused form of repeat + q.kT + scale + softmax + .v +
// head merge of ug-llama/src/model.rs:231-245 for one query position per
// sequence.  The kernel needs scratch memory for the per-slice partial results
// (m, l, O) and one completion counter per (sequence, KV head); this entry
// point takes it from the device's stream-ordered pool for the duration of the
// call.
#include "decode_kernels.cuh"

using namespace ugb_decode;

namespace {

int32_t check_attention_args(ugb_device *dev, const ugb_slice *q, const ugb_slice *k, const ugb_slice *v,
                             const ugb_slice *pos, ugb_slice *out, size_t b, size_t n_heads, size_t n_kv,
                             size_t t_max, int32_t n_slices) {
  UGB_REQUIRE(dev, n_kv > 0 && n_heads % n_kv == 0 && n_heads / n_kv <= (size_t)ATT_GROUP, UGB_ERR_UNSUPPORTED,
              "decode_attention: query heads per KV head must divide evenly and be <= %d", ATT_GROUP);
  UGB_REQUIRE(dev, t_max % ATT_SUB == 0, UGB_ERR_SHAPE, "decode_attention: cache positions (%zu) must be a multiple of %d",
              t_max, ATT_SUB);
  UGB_REQUIRE(dev, n_slices >= 1 && n_slices <= 8, UGB_ERR_INVALID, "decode_attention: n_slices %d outside 1..8", n_slices);
  UGB_REQUIRE(dev, b <= 65535 && n_kv <= 65535, UGB_ERR_SHAPE, "decode_attention: batch or KV heads exceed the grid limit");
  UGB_SLICE(dev, q, UGB_BF16, b * n_heads * ATT_HD);
  UGB_SLICE(dev, k, UGB_BF16, b * n_kv * t_max * ATT_HD);
  UGB_SLICE(dev, v, UGB_BF16, b * n_kv * t_max * ATT_HD);
  UGB_SLICE(dev, pos, UGB_I32, 1);
  UGB_SLICE(dev, out, UGB_BF16, b * n_heads * ATT_HD);
  return UGB_OK;
}

int32_t launch_attention(ugb_device *dev, const ugb_slice *q, const ugb_slice *k, const ugb_slice *v,
                         const ugb_slice *pos, ugb_slice *out, size_t b, size_t n_heads, size_t n_kv,
                         size_t t_max, int32_t n_slices, float *part_o, float *part_ml, unsigned int *counters) {
  static bool attr_set[64] = {};
  if (!attr_set[dev->ordinal & 63]) {
    UGB_CUDA(dev, cudaFuncSetAttribute(decode_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_RING_BYTES));
    attr_set[dev->ordinal & 63] = true;
  }
  dim3 grid((unsigned)n_slices, (unsigned)n_kv, (unsigned)b);
  AttRope front{};                       // q given, cache read only
  front.status = dev->status_dev;        // a position outside the cache is reported there
  decode_attention_kernel<<<grid, ATT_WARPS * 32, ATT_RING_BYTES, dev->stream>>>(
      (const __nv_bfloat16 *)q->ptr, (__nv_bfloat16 *)k->ptr, (__nv_bfloat16 *)v->ptr,
      (const int *)pos->ptr, part_o, part_ml, counters, (__nv_bfloat16 *)out->ptr, (int)n_heads, (int)n_kv,
      (int)(n_heads / n_kv), (int)t_max, 0.125f /* 64^-0.5, model.rs:236 */, front, CUtensorMap{}, CUtensorMap{} /* cp.async path */);
  return ugb_after_launch(dev, "decode_attention_kernel");
}

// ---- fixed scratch for callers that must not allocate ----------------------
// Room for NOALLOC_MAX_SLOTS (sequence, KV head, slice) partial results and as
// many completion counters.  Every GPU that loads this library carries the
// array (about 4.1 MiB) until the process exits.
constexpr size_t NOALLOC_MAX_SLOTS = 2048;
constexpr size_t NOALLOC_O_BYTES = NOALLOC_MAX_SLOTS * ATT_GROUP * ATT_HD * sizeof(float);
constexpr size_t NOALLOC_ML_BYTES = NOALLOC_MAX_SLOTS * ATT_GROUP * 2 * sizeof(float);
constexpr size_t NOALLOC_CNT_BYTES = NOALLOC_MAX_SLOTS * sizeof(unsigned int);
static __device__ __align__(256) unsigned char g_att_scratch[NOALLOC_O_BYTES + NOALLOC_ML_BYTES + NOALLOC_CNT_BYTES];

// DEVICE address of g_att_scratch on each device ordinal.  In host code the
// name g_att_scratch is only a handle for the runtime, never a pointer a
// kernel may be given: the address has to be asked for, per device.
constexpr int NOALLOC_MAX_DEVICES = 64;
static unsigned char *g_att_scratch_addr[NOALLOC_MAX_DEVICES] = {};

}  // namespace

extern "C" {

int32_t ugb_decode_attention_noalloc(ugb_device *dev, const ugb_slice *q, const ugb_slice *k,
                                     const ugb_slice *v, const ugb_slice *pos, ugb_slice *out, size_t b,
                                     size_t n_heads, size_t n_kv, size_t t_max, int32_t n_slices) {
  if (!dev) return UGB_ERR_INVALID;
  int32_t rc = check_attention_args(dev, q, k, v, pos, out, b, n_heads, n_kv, t_max, n_slices);
  if (rc) return rc;
  const size_t slots = b * n_kv * (size_t)n_slices;
  UGB_REQUIRE(dev, slots <= NOALLOC_MAX_SLOTS, UGB_ERR_SHAPE,
              "decode_attention_noalloc: batch * n_kv * n_slices = %zu exceeds the fixed scratch of %zu slots; "
              "use fewer slices or ugb_decode_attention", slots, NOALLOC_MAX_SLOTS);
  UGB_REQUIRE(dev, dev->ordinal >= 0 && dev->ordinal < NOALLOC_MAX_DEVICES, UGB_ERR_UNSUPPORTED,
              "decode_attention_noalloc: device ordinal %d beyond %d", dev->ordinal, NOALLOC_MAX_DEVICES);
  if (b == 0) return UGB_OK;
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  if (!g_att_scratch_addr[dev->ordinal]) {
    // one-time set-up on this device (it is the current device here)
    void *p = nullptr;
    UGB_CUDA(dev, cudaGetSymbolAddress(&p, g_att_scratch));
    g_att_scratch_addr[dev->ordinal] = (unsigned char *)p;
  }
  unsigned char *base = g_att_scratch_addr[dev->ordinal];
  float *part_o = (float *)base;
  float *part_ml = (float *)(base + NOALLOC_O_BYTES);
  unsigned int *counters = (unsigned int *)(base + NOALLOC_O_BYTES + NOALLOC_ML_BYTES);
  // The array keeps whatever the previous call left: the counters must start at
  // zero (the partial results are fully rewritten before they are read).
  UGB_CUDA(dev, cudaMemsetAsync(counters, 0, b * n_kv * sizeof(unsigned int), dev->stream));
  return launch_attention(dev, q, k, v, pos, out, b, n_heads, n_kv, t_max, n_slices, part_o, part_ml, counters);
}

int32_t ugb_decode_attention(ugb_device *dev, const ugb_slice *q, const ugb_slice *k, const ugb_slice *v,
                             const ugb_slice *pos, ugb_slice *out, size_t b, size_t n_heads, size_t n_kv,
                             size_t t_max, int32_t n_slices) {
  if (!dev) return UGB_ERR_INVALID;
  int32_t rc = check_attention_args(dev, q, k, v, pos, out, b, n_heads, n_kv, t_max, n_slices);
  if (rc) return rc;
  if (b == 0) return UGB_OK;
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  const size_t slots = b * n_kv * (size_t)n_slices;
  const size_t o_bytes = slots * ATT_GROUP * ATT_HD * sizeof(float);
  const size_t ml_bytes = slots * ATT_GROUP * 2 * sizeof(float);
  const size_t cnt_bytes = b * n_kv * sizeof(unsigned int);
  char *scratch = nullptr;
  UGB_CUDA(dev, ugb_malloc_async(dev, (void **)&scratch, o_bytes + ml_bytes + cnt_bytes));
  unsigned int *counters = (unsigned int *)(scratch + o_bytes + ml_bytes);
  cudaError_t e = cudaMemsetAsync(counters, 0, cnt_bytes, dev->stream);
  if (e == cudaSuccess)
    rc = launch_attention(dev, q, k, v, pos, out, b, n_heads, n_kv, t_max, n_slices, (float *)scratch,
                          (float *)(scratch + o_bytes), counters);
  else
    rc = ugb_fail(dev, UGB_ERR_CUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  cudaFreeAsync(scratch, dev->stream);
  return rc;
}

}  // extern "C"
