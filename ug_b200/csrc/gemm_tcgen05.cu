// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// TMEM, operands staged in shared memory by TMA).  Replaces the
// cublasGemmStridedBatchedEx call of ug-cuda/src/gemm.rs:265-289 for bf16.
//
//   C[b, m, n] = A[b, m, k] . B         fp32 accumulate, bf16 output
//   A row-major (k contiguous).  B either [n, k] row-major (k contiguous, the
//   matmul_t / weight layout) or [k, n] row-major (n contiguous).
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer   (one elected lane issues cp.async.bulk.tensor)
//   warp 1      MMA issuer     (one elected lane issues tcgen05.mma / commit),
//               also owns the TMEM allocation
//   warps 2..5  epilogue       (tcgen05.ld -> bf16 -> global), one TMEM lane
//               quadrant each
// CTA tile 128 x 256, k slices of 64 bf16 (= one 128-byte swizzle row), a
// 4-stage shared-memory ring (48 KiB per stage) and two 256-column TMEM
// accumulators so that the epilogue of tile i overlaps the main loop of tile
// i+1.  No cluster launch and no multicast: every CTA fetches its own tiles.
//
// Every mbarrier wait is bounded by wall-clock time; a wait that gives up
// raises the device status word (UGB_ERR_TIMEOUT), flags the CTA as aborted so
// that all roles leave their loops, lets copies in flight land, frees TMEM and
// returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include "gemm_tcgen05.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4, ACC_STAGES = 2;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;          // 16 KiB
constexpr int B_BYTES = BN * BK * 2;          // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = ACC_STAGES * BN;    // 512 (all of TMEM)
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s per wait

struct Params {
  int M, N, K, batch;
  int tiles_m, tiles_n, k_blocks;
  int b_batched;          // 0: B shared by all batch steps
  int b_is_nk;            // 1: B [n,k] (k-major), 0: B [k,n] (n-major)
  long long c_batch;      // elements between batch steps of C
  __nv_bfloat16 *C;
  ugb_status_word *status;
};

// ----------------------------------------------------------------- PTX -----
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the CTA is (or becomes) aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          ugb_status_word *status, unsigned site) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = globaltimer();
  for (unsigned it = 1;; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (atomicCAS(&status->code, 0u, (unsigned)UGB_ERR_TIMEOUT) == 0u) status->detail = site;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1.
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4  bits 46-47 version   bits 61-63 layout (2 = SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor for kind::f16: D = f32, A = B = bf16, M x N tile.
//   bits 4-5 D format (1 = f32)   bits 7-9 A format (1 = bf16)   bits 10-12 B format
//   bit 15 A major (0 = K)        bit 16 B major (1 = MN)        bits 17-22 N >> 3   bits 24-28 M >> 4
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__global__ void __launch_bounds__(THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern repeats every 1024 bytes
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = (uint64_t *)(smem + STAGES * STAGE_BYTES);
  uint64_t *full = bars, *empty = bars + STAGES;
  uint64_t *acc_full = bars + 2 * STAGES, *acc_empty = bars + 2 * STAGES + ACC_STAGES;
  uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 2 * ACC_STAGES);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      mbar_init(smem_u32(&acc_full[s]), 1);
      mbar_init(smem_u32(&acc_empty[s]), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int n_tiles = tiles_per_batch * p.batch;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
        const int bi = tile / tiles_per_batch;
        const int r = tile - bi * tiles_per_batch;
        const int m0 = (r % p.tiles_m) * BM, n0 = (r / p.tiles_m) * BN;
        const int bz = p.b_batched ? bi : 0;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(smem_u32(&empty[stage]), phase ^ 1u, abort_flag, p.status, 1)) { alive = false; break; }
          const uint32_t bar = smem_u32(&full[stage]);
          mbar_expect_tx(bar, STAGE_BYTES);
          const uint32_t a_dst = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_dst = a_dst + A_BYTES;
          tma_load_3d(a_dst, &tmA, bar, kb * BK, m0, bi);
          if (p.b_is_nk) {
            tma_load_3d(b_dst, &tmB, bar, kb * BK, n0, bz);          // box {64 k, 256 n}
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)                         // 4 boxes {64 n, 64 k}
              tma_load_3d(b_dst + c * (64 * BK * 2), &tmB, bar, n0 + c * 64, kb * BK, bz);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, BN, !p.b_is_nk);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
        if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_phase ^ 1u, abort_flag, p.status, 2)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(smem_u32(&full[stage]), phase, abort_flag, p.status, 3)) { alive = false; break; }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            // A, and B when k-major: rows of 128 B, 8-row groups 1024 B apart; a
            // k step of 16 bf16 moves 32 B inside the swizzled row.
            const uint64_t a_desc = make_smem_desc(a_addr + j * (UMMA_K * 2), 0, 1024);
            // B n-major: 64-wide n chunks 8 KiB apart (LBO), 8-k groups 1024 B
            // apart (SBO); a k step of 16 moves 16 rows of 128 B.
            const uint64_t b_desc = p.b_is_nk ? make_smem_desc(b_addr + j * (UMMA_K * 2), 0, 1024)
                                              : make_smem_desc(b_addr + j * (UMMA_K * 128), 64 * BK * 2, 1024);
            umma_bf16(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty[stage]));      // frees the smem stage when the MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        umma_commit(smem_u32(&acc_full[acc]));       // accumulator complete
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue --
    const int quad = warp & 3;                        // TMEM lane quadrant of this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      const int bi = tile / tiles_per_batch;
      const int r = tile - bi * tiles_per_batch;
      const int m0 = (r % p.tiles_m) * BM, n0 = (r / p.tiles_m) * BN;
      if (!mbar_wait(smem_u32(&acc_full[acc]), acc_phase, abort_flag, p.status, 4)) break;
      tcgen05_fence_after();
      const int row = m0 + quad * 32 + lane;
      __nv_bfloat16 *crow = p.C + (long long)bi * p.c_batch + (long long)row * p.N + n0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + c * 32), v);
        tmem_ld_wait();
        if (row < p.M) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int col = n0 + c * 32 + q * 8;
            if (col < p.N) {                          // N % 8 == 0: a chunk of 8 is all in or all out
              uint4 o;
              __nv_bfloat162 t;
              t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1])); o.x = *(uint32_t *)&t;
              t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3])); o.y = *(uint32_t *)&t;
              t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5])); o.z = *(uint32_t *)&t;
              t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7])); o.w = *(uint32_t *)&t;
              *reinterpret_cast<uint4 *>(crow + c * 32 + q * 8) = o;
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ------------------------------------------------------------- teardown --
  __syncwarp();
  if (*abort_flag) {
    // give copies and MMAs in flight time to land before shared memory and TMEM go away
    const unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ----------------------------------------------------------------- host ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

struct TcState {
  EncodeTiledFn encode = nullptr;
  bool attr_set = false;
};

TcState *state_of(ugb_device *dev) {
  if (!dev->gemm_state) dev->gemm_state = new TcState();
  return (TcState *)dev->gemm_state;
}

// rank-3 bf16 tensor map: dims {d0 (contiguous), d1, d2}, strides in elements for d1, d2.
int32_t encode_map(ugb_device *dev, TcState *st, CUtensorMap *map, const void *base, uint64_t d0,
                   uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t box0, uint32_t box1) {
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1 * 2, s2 * 2};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = st->encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides,
                          box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return ugb_fail(dev, UGB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return UGB_OK;
}

}  // namespace

int32_t ugb_tc_gemm_bf16(ugb_device *dev, void *c, const void *a, const void *b_, size_t batch, size_t m,
                         size_t n, size_t k, long long a_batch, long long b_batch, bool b_is_nk) {
  // TMA: 16-byte aligned bases, row strides that are multiples of 16 bytes.
  if (k == 0 || k % 8 != 0 || n % 8 != 0) return UGB_ERR_UNSUPPORTED;
  if (((uintptr_t)a | (uintptr_t)b_ | (uintptr_t)c) & 15) return UGB_ERR_UNSUPPORTED;
  if ((a_batch % 8) != 0 || (b_batch % 8) != 0 || a_batch < 0 || b_batch < 0) return UGB_ERR_UNSUPPORTED;
  if (batch > 1 && a_batch == 0) return UGB_ERR_UNSUPPORTED;
  if (m > (1u << 30) || n > (1u << 30) || k > (1u << 30) || batch > 65535) return UGB_ERR_UNSUPPORTED;
  // Tiny products do not fill a 128 x 256 tile; the strided kernel handles them.
  if (m * n < 128 * 64 || m < 16) return UGB_ERR_UNSUPPORTED;

  TcState *st = state_of(dev);
  if (!st->encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return ugb_fail(dev, UGB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    st->encode = (EncodeTiledFn)fn;
  }
  if (!st->attr_set) {
    UGB_CUDA(dev, cudaFuncSetAttribute(tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    st->attr_set = true;
  }
  // A shared B with densely stacked A batches is one tall GEMM.
  if (batch > 1 && b_batch == 0 && a_batch == (long long)(m * k)) {
    m *= batch;
    batch = 1;
  }
  Params p;
  p.M = (int)m; p.N = (int)n; p.K = (int)k; p.batch = (int)batch;
  p.tiles_m = (int)((m + BM - 1) / BM);
  p.tiles_n = (int)((n + BN - 1) / BN);
  p.k_blocks = (int)((k + BK - 1) / BK);
  p.b_batched = (batch > 1 && b_batch != 0) ? 1 : 0;
  p.b_is_nk = b_is_nk ? 1 : 0;
  p.c_batch = (long long)(m * n);
  p.C = (__nv_bfloat16 *)c;
  p.status = dev->status_dev;

  CUtensorMap tmA, tmB;
  int32_t rc = encode_map(dev, st, &tmA, a, k, m, batch, k, batch > 1 ? (uint64_t)a_batch : m * k, BK, BM);
  if (rc) return rc;
  const uint64_t nb = p.b_batched ? batch : 1;
  const uint64_t bs = p.b_batched ? (uint64_t)b_batch : n * k;
  if (b_is_nk) rc = encode_map(dev, st, &tmB, b_, k, n, nb, k, bs, BK, BN);
  else rc = encode_map(dev, st, &tmB, b_, n, k, nb, n, bs, 64, BK);
  if (rc) return rc;

  const long long n_tiles = (long long)p.tiles_m * p.tiles_n * p.batch;
  const unsigned grid = (unsigned)(n_tiles < dev->sm_count ? n_tiles : dev->sm_count);
  tc_gemm_kernel<<<grid, THREADS, SMEM_BYTES, dev->stream>>>(tmA, tmB, p);
  return ugb_after_launch(dev, "tc_gemm_kernel");
}

void ugb_tc_state_free(ugb_device *dev) {
  if (dev->gemm_state) {
    delete (TcState *)dev->gemm_state;
    dev->gemm_state = nullptr;
  }
}
