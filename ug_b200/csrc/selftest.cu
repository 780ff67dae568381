// Self-test of the bounded device-side waits.
//
// Every wait a kernel of this library performs on something another agent has to produce -- an mbarrier
// that a TMA copy or an MMA completes, a flag that a peer GPU stores, a grid-wide barrier -- is limited
// to the device option "wait_limit_us"; a wait that runs out raises the device status word
// (UGB_ERR_TIMEOUT plus a site code), lets the kernel finish, and leaves the context usable.  This entry
// point drives exactly that path without any fault: one CTA waits on something nobody will ever
// complete, with the caller's (short) limit, gives up and returns.  It is how a deployment checks on a
// new machine that a lost peer or a lost copy ends in an error code and not in a hung GPU.
#include "tp_kernels.cuh"

using namespace ugb_decode;

namespace {

// which = 0: mbarrier that receives no arrival (the GEMM / attention pipelines' wait, ugb_tc::mbar_wait)
// which = 1: exchange flags of a two-rank tensor-parallel group whose second rank never signals
//            (tp_exchange_begin against two header blocks in this GPU's own memory)
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(int which, TpHeader *hdrs, ugb_status_word *status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (which == 0) {
    if (threadIdx.x == 0) {
      ugb_tc::mbar_init(ugb_tc::smem_u32(&bar), 1);
      abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (threadIdx.x == 0) ugb_tc::mbar_wait(ugb_tc::smem_u32(&bar), 0u, &abort_flag, status, 0x99u);
    return;
  }
  TpPeers tp{};
  tp.rank = 0;
  tp.size = 2;
  tp.hdr[0] = hdrs;
  tp.hdr[1] = hdrs + 1;
  tp_exchange_begin(tp, status, true);     // rank 1's flag never comes: thread 1 waits out the limit
  tp_exchange_end(tp);
}

}  // namespace

extern "C" int32_t ugb_selftest_bounded_wait(ugb_device *dev, int32_t which) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, which == 0 || which == 1, UGB_ERR_INVALID, "ugb_selftest_bounded_wait: which = %d is not 0 or 1", which);
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  TpHeader *hdrs = nullptr;
  UGB_CUDA(dev, ugb_malloc_async(dev, (void **)&hdrs, 2 * sizeof(TpHeader)));
  cudaError_t e = cudaMemsetAsync(hdrs, 0, 2 * sizeof(TpHeader), dev->stream);
  int32_t rc = UGB_OK;
  if (e != cudaSuccess) {
    rc = ugb_fail(dev, UGB_ERR_CUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  } else {
    bounded_wait_selftest_kernel<<<1, 32, 0, dev->stream>>>(which, hdrs, dev->status_dev);
    rc = ugb_after_launch(dev, "bounded_wait_selftest_kernel");
  }
  cudaFreeAsync(hdrs, dev->stream);
  return rc;
}
