// Device, memory, copy and timing entry points of the ugb200 C ABI.
// Replaces ug-cuda/src/runtime.rs (Device::new, allocate_uninit, synchronize,
// Slice copies) with a stream-ordered allocator and a per-device status word.
#include <cstring>
#include <mutex>

#include "ugb_internal.h"

static std::mutex g_err_mu;
static std::string g_create_error;

int32_t ugb_fail(ugb_device *dev, int32_t code, const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (dev) {
    dev->last_error = buf;
  } else {
    std::lock_guard<std::mutex> g(g_err_mu);
    g_create_error = buf;
  }
  return code;
}

int32_t ugb_after_launch(ugb_device *dev, const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return ugb_fail(dev, UGB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  dev->launches++;
  return UGB_OK;
}

extern "C" {

int32_t ugb_device_create(int32_t ordinal, ugb_device **out) {
  if (!out) return ugb_fail(nullptr, UGB_ERR_INVALID, "ugb_device_create: null out pointer");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess)
    return ugb_fail(nullptr, UGB_ERR_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(e));
  if (ordinal < 0 || ordinal >= n)
    return ugb_fail(nullptr, UGB_ERR_INVALID, "device ordinal %d out of range (%d devices)", ordinal, n);
  cudaDeviceProp prop;
  if ((e = cudaGetDeviceProperties(&prop, ordinal)) != cudaSuccess)
    return ugb_fail(nullptr, UGB_ERR_CUDA, "cudaGetDeviceProperties failed: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return ugb_fail(nullptr, UGB_ERR_UNSUPPORTED,
                    "device %d is sm_%d%d; this library carries sm_100a code only", ordinal,
                    prop.major, prop.minor);
  if ((e = cudaSetDevice(ordinal)) != cudaSuccess)
    return ugb_fail(nullptr, UGB_ERR_CUDA, "cudaSetDevice failed: %s", cudaGetErrorString(e));
  ugb_device *d = new ugb_device();
  d->ordinal = ordinal;
  d->sm_count = prop.multiProcessorCount;
  d->smem_optin = prop.sharedMemPerBlockOptin;
  bool ok = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaEventCreate(&d->ev_begin) == cudaSuccess &&
            cudaEventCreate(&d->ev_end) == cudaSuccess &&
            cudaMalloc(&d->status_dev, sizeof(ugb_status_word)) == cudaSuccess &&
            cudaMalloc(&d->sched_dev, 2 * sizeof(int)) == cudaSuccess;
  if (ok) {
    // initial values go through the handle's own stream (a non-blocking stream is not ordered against the
    // legacy stream) and are complete before the handle is handed out
    const ugb_status_word w0 = {0u, 0u, UGB_DEFAULT_WAIT_LIMIT_US, 0u};
    ok = cudaMemcpyAsync(d->status_dev, &w0, sizeof(w0), cudaMemcpyHostToDevice, d->stream) == cudaSuccess &&
         cudaMemsetAsync(d->sched_dev, 0, 2 * sizeof(int), d->stream) == cudaSuccess &&
         cudaStreamSynchronize(d->stream) == cudaSuccess;
  }
  if (!ok) {
    e = cudaGetLastError();
    ugb_fail(nullptr, UGB_ERR_CUDA, "device set-up failed: %s", cudaGetErrorString(e));
    delete d;
    return UGB_ERR_CUDA;
  }
  // A pool of the handle's own, which keeps freed blocks instead of returning them to the driver at every
  // synchronisation (decode allocates per step); the default pool that other users of the process share is not touched.
  {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = ordinal;
    if (cudaMemPoolCreate(&d->pool, &props) == cudaSuccess) {
      uint64_t thresh = UINT64_MAX;
      cudaMemPoolSetAttribute(d->pool, cudaMemPoolAttrReleaseThreshold, &thresh);
    } else {
      d->pool = nullptr;            // fall back to the default pool with its default behaviour
      cudaGetLastError();
    }
  }
  *out = d;
  return UGB_OK;
}

void ugb_gemm_state_free(ugb_device *dev);

int32_t ugb_device_destroy(ugb_device *dev) {
  if (!dev) return UGB_ERR_INVALID;
  cudaSetDevice(dev->ordinal);
  cudaStreamSynchronize(dev->stream);
  ugb_gemm_state_free(dev);
  if (dev->pool) { cudaMemPoolDestroy(dev->pool); dev->pool = nullptr; }
  if (dev->status_dev) cudaFree(dev->status_dev);
  if (dev->sched_dev) cudaFree(dev->sched_dev);
  if (dev->ev_begin) cudaEventDestroy(dev->ev_begin);
  if (dev->ev_end) cudaEventDestroy(dev->ev_end);
  if (dev->stream) cudaStreamDestroy(dev->stream);
  delete dev;
  return UGB_OK;
}

const char *ugb_last_error(const ugb_device *dev) {
  if (dev) return dev->last_error.c_str();
  std::lock_guard<std::mutex> g(g_err_mu);
  return g_create_error.c_str();
}

int32_t ugb_sync(ugb_device *dev) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  ugb_status_word w;
  UGB_CUDA(dev, cudaMemcpyAsync(&w, dev->status_dev, sizeof(w), cudaMemcpyDeviceToHost, dev->stream));
  UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  if (w.code != 0) {
    cudaMemsetAsync(dev->status_dev, 0, 2 * sizeof(unsigned int), dev->stream);   // code and detail; the wait limit stays
    if (w.code == (unsigned)UGB_ERR_TIMEOUT) dev->wait_timeouts++;
    return ugb_fail(dev, (int32_t)w.code, "device-side status %u (detail %u) reported by a kernel",
                    w.code, w.detail);
  }
  return UGB_OK;
}

int32_t ugb_use_grid(void) { return 1; }
int32_t ugb_device_ordinal(const ugb_device *dev) { return dev ? dev->ordinal : -1; }
void *ugb_device_stream(const ugb_device *dev) { return dev ? (void *)dev->stream : nullptr; }
uint64_t ugb_launch_count(const ugb_device *dev) { return dev ? dev->launches : 0; }

int32_t ugb_device_set_option(ugb_device *dev, const char *name, int32_t value) {
  if (!dev || !name) return UGB_ERR_INVALID;
  if (strcmp(name, "gemm_cta_pairs") == 0) {
    UGB_REQUIRE(dev, value == 0 || value == 1, UGB_ERR_INVALID, "option gemm_cta_pairs: %d is not 0 or 1", value);
    dev->gemm_pair = value;
    return UGB_OK;
  }
  if (strcmp(name, "wait_limit_us") == 0) {
    UGB_REQUIRE(dev, value >= 100 && value <= 60000000, UGB_ERR_INVALID,
                "option wait_limit_us: %d outside 100..60000000", value);
    UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
    const unsigned int v = (unsigned int)value;
    UGB_CUDA(dev, cudaMemcpyAsync(&dev->status_dev->wait_limit_us, &v, sizeof(v), cudaMemcpyHostToDevice, dev->stream));
    UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
    return UGB_OK;
  }
  return ugb_fail(dev, UGB_ERR_INVALID, "unknown device option %s", name);
}

int32_t ugb_alloc(ugb_device *dev, int32_t dtype, size_t len, ugb_slice **out) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, out != nullptr, UGB_ERR_INVALID, "ugb_alloc: null out pointer");
  *out = nullptr;
  size_t es = ugb_dtype_size(dtype);
  UGB_REQUIRE(dev, es != 0, UGB_ERR_INVALID, "ugb_alloc: unknown dtype %d", dtype);
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  void *p = nullptr;
  if (len > 0) UGB_CUDA(dev, ugb_malloc_async(dev, &p, len * es));
  ugb_slice *s = new ugb_slice();
  s->dev = dev;
  s->ptr = p;
  s->len = len;
  s->dtype = dtype;
  s->owned = true;
  *out = s;
  return UGB_OK;
}

int32_t ugb_wrap(ugb_device *dev, void *device_ptr, int32_t dtype, size_t len, ugb_slice **out) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, out != nullptr, UGB_ERR_INVALID, "ugb_wrap: null out pointer");
  *out = nullptr;
  UGB_REQUIRE(dev, ugb_dtype_size(dtype) != 0, UGB_ERR_INVALID, "ugb_wrap: unknown dtype %d", dtype);
  UGB_REQUIRE(dev, device_ptr != nullptr || len == 0, UGB_ERR_INVALID, "ugb_wrap: null pointer");
  ugb_slice *s = new ugb_slice();
  s->dev = dev;
  s->ptr = device_ptr;
  s->len = len;
  s->dtype = dtype;
  s->owned = false;
  *out = s;
  return UGB_OK;
}

int32_t ugb_free(ugb_slice *s) {
  if (!s) return UGB_ERR_INVALID;
  ugb_device *dev = s->dev;
  int32_t rc = UGB_OK;
  if (s->owned && s->ptr) {
    cudaSetDevice(dev->ordinal);
    cudaError_t e = cudaFreeAsync(s->ptr, dev->stream);
    if (e != cudaSuccess) rc = ugb_fail(dev, UGB_ERR_CUDA, "cudaFreeAsync failed: %s", cudaGetErrorString(e));
  }
  delete s;
  return rc;
}

size_t ugb_slice_len(const ugb_slice *s) { return s ? s->len : 0; }
int32_t ugb_slice_dtype(const ugb_slice *s) { return s ? s->dtype : -1; }
void *ugb_slice_ptr(const ugb_slice *s) { return s ? s->ptr : nullptr; }

static int32_t copy_checks(ugb_device *dev, const ugb_slice *s, const void *host, size_t len,
                           int32_t dtype, const char *dir) {
  UGB_REQUIRE(dev, s->dtype == dtype, UGB_ERR_DTYPE, "%s dtype mismatch, slice %s, host %s", dir,
              ugb_dtype_name(s->dtype), ugb_dtype_name(dtype));
  UGB_REQUIRE(dev, s->len == len, UGB_ERR_SHAPE, "%s length mismatch, slice %zu, host %zu", dir,
              s->len, len);
  UGB_REQUIRE(dev, host != nullptr || len == 0, UGB_ERR_INVALID, "%s: null host pointer", dir);
  return UGB_OK;
}

int32_t ugb_h2d(ugb_slice *dst, const void *src, size_t len, int32_t dtype) {
  if (!dst) return UGB_ERR_INVALID;
  ugb_device *dev = dst->dev;
  int32_t rc = copy_checks(dev, dst, src, len, dtype, "htod");
  if (rc) return rc;
  if (len == 0) return UGB_OK;
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  UGB_CUDA(dev, cudaMemcpyAsync(dst->ptr, src, len * ugb_dtype_size(dtype), cudaMemcpyHostToDevice, dev->stream));
  UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return UGB_OK;
}

int32_t ugb_d2h(const ugb_slice *src, void *dst, size_t len, int32_t dtype) {
  if (!src) return UGB_ERR_INVALID;
  ugb_device *dev = src->dev;
  int32_t rc = copy_checks(dev, src, dst, len, dtype, "dtoh");
  if (rc) return rc;
  if (len == 0) return UGB_OK;
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  UGB_CUDA(dev, cudaMemcpyAsync(dst, src->ptr, len * ugb_dtype_size(dtype), cudaMemcpyDeviceToHost, dev->stream));
  UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return UGB_OK;
}

int32_t ugb_h2d_async(ugb_slice *dst, const void *src, size_t len, int32_t dtype) {
  if (!dst) return UGB_ERR_INVALID;
  ugb_device *dev = dst->dev;
  int32_t rc = copy_checks(dev, dst, src, len, dtype, "htod");
  if (rc) return rc;
  if (len == 0) return UGB_OK;
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  UGB_CUDA(dev, cudaMemcpyAsync(dst->ptr, src, len * ugb_dtype_size(dtype), cudaMemcpyHostToDevice, dev->stream));
  return UGB_OK;
}

int32_t ugb_d2h_async(const ugb_slice *src, void *dst, size_t len, int32_t dtype) {
  if (!src) return UGB_ERR_INVALID;
  ugb_device *dev = src->dev;
  int32_t rc = copy_checks(dev, src, dst, len, dtype, "dtoh");
  if (rc) return rc;
  if (len == 0) return UGB_OK;
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  UGB_CUDA(dev, cudaMemcpyAsync(dst, src->ptr, len * ugb_dtype_size(dtype), cudaMemcpyDeviceToHost, dev->stream));
  return UGB_OK;
}

int32_t ugb_host_alloc(size_t bytes, void **out) {
  if (!out) return UGB_ERR_INVALID;
  *out = nullptr;
  cudaError_t e = cudaMallocHost(out, bytes ? bytes : 1);
  if (e != cudaSuccess) return ugb_fail(nullptr, UGB_ERR_OOM, "cudaMallocHost failed: %s", cudaGetErrorString(e));
  return UGB_OK;
}

int32_t ugb_host_free(void *p) {
  if (!p) return UGB_ERR_INVALID;
  return cudaFreeHost(p) == cudaSuccess ? UGB_OK : UGB_ERR_CUDA;
}

int32_t ugb_timer_begin(ugb_device *dev) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_CUDA(dev, cudaEventRecord(dev->ev_begin, dev->stream));
  return UGB_OK;
}
int32_t ugb_timer_end(ugb_device *dev) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_CUDA(dev, cudaEventRecord(dev->ev_end, dev->stream));
  return UGB_OK;
}
int32_t ugb_timer_elapsed_ms(ugb_device *dev, float *ms) {
  if (!dev || !ms) return UGB_ERR_INVALID;
  UGB_CUDA(dev, cudaEventSynchronize(dev->ev_end));
  UGB_CUDA(dev, cudaEventElapsedTime(ms, dev->ev_begin, dev->ev_end));
  return UGB_OK;
}

}  // extern "C"
