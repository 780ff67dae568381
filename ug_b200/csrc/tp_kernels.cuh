// Tensor-parallel exchange for the Llama engine: the row-parallel projections
// (o_proj, down_proj) of every rank leave fp32 partial sums in that rank's own
// memory; the consumer kernel of each rank then reads all ranks' partials over
// NVLink (plain peer loads) and fuses the cross-rank sum with the residual add
// and the next RMSNorm -- the all-reduce is never a kernel of its own.
//
// Synchronisation: one flag word per (rank, peer) in each rank's exchange block.
// A kernel that needs its peers' data (1) makes sure its own producer kernel
// has completed (stream order / griddepcontrol.wait), (2) stores the current
// epoch into its slot of every peer's flag array (st.release.sys), (3) waits
// until its own flag array shows that epoch for every peer (ld.acquire.sys).
// Data is only ever *read* remotely; remote stores carry flags only.  Waits
// are bounded (device option "wait_limit_us", 2 s of %globaltimer by default;
// the limit also has to cover the host-side skew between the ranks' launches):
// on expiry the kernel raises the status word, marks the exchange as failed
// and carries on with whatever the buffers hold, so that no rank can hang
// another.  While the mark is set every later exchange skips its wait AND
// raises the status word again, so no step after a failed one passes for good;
// the engine refuses further steps once ugb_sync has reported the timeout.
//
// Buffer reuse needs no second barrier: a partial buffer is rewritten two
// exchanges later, and its owner passes the exchange in between only after
// every peer has signalled it, which a peer does after its own reading kernel
// has completed.
#pragma once
#include "decode_kernels.cuh"

namespace ugb_decode {

constexpr int TP_MAX = 8;

// Layout of the per-rank exchange block header (device memory shared with the peers).
struct TpHeader {
  unsigned int flags[TP_MAX];   // flags[r]: last epoch rank r has signalled to this rank
  unsigned int epoch;           // exchanges completed by this rank
  unsigned int done;            // CTAs of the running exchange kernel that have finished
  unsigned int failed;          // sticky: a wait gave up
  unsigned int pad[5];
};

struct TpPeers {
  const float *part[TP_MAX];    // this exchange's partial buffer on every rank (own included)
  TpHeader *hdr[TP_MAX];        // every rank's header (own included)
  int rank, size;
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long tp_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Called by every CTA of an exchange kernel after its producer has completed.
// CTA 0 signals the peers; every CTA waits for all of them.  Ends in a CTA barrier.
__device__ __forceinline__ void tp_exchange_begin(const TpPeers &tp, ugb_status_word *status, bool first_cta) {
  TpHeader *mine = tp.hdr[tp.rank];
  const unsigned int e = *reinterpret_cast<volatile unsigned int *>(&mine->epoch) + 1u;
  if (threadIdx.x < (unsigned)tp.size) {
    const int r = threadIdx.x;
    if (first_cta) {
      __threadfence_system();
      st_release_sys(&tp.hdr[r]->flags[tp.rank], e);           // own slot too: uniform wait below
    }
    if (!*reinterpret_cast<volatile unsigned int *>(&mine->failed)) {
      const unsigned long long limit = 1000ull * *reinterpret_cast<volatile unsigned int *>(&status->wait_limit_us);
      const unsigned long long t0 = tp_globaltimer();
      unsigned int it = 0;
      while ((int)(ld_acquire_sys(&mine->flags[r]) - e) < 0) {
        if ((++it & 63u) == 0u && tp_globaltimer() - t0 > limit) {
          mine->failed = 1u;
          if (atomicCAS(&status->code, 0u, (unsigned)UGB_ERR_TIMEOUT) == 0u) status->detail = 0x7000u + r;
          break;
        }
      }
    } else if (r == 0 && atomicCAS(&status->code, 0u, (unsigned)UGB_ERR_TIMEOUT) == 0u) {
      status->detail = 0x70ffu;       // an earlier exchange of this model gave up: its ranks are out of step
    }
  }
  __syncthreads();
}

// Called by every CTA when it no longer needs the peers' buffers: the last one advances the epoch.
__device__ __forceinline__ void tp_exchange_end(const TpPeers &tp) {
  __syncthreads();
  if (threadIdx.x == 0) {
    TpHeader *mine = tp.hdr[tp.rank];
    __threadfence();
    const unsigned int n = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(&mine->done, 1u) == n - 1u) {
      mine->done = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int *>(&mine->epoch) = *reinterpret_cast<volatile unsigned int *>(&mine->epoch) + 1u;
    }
  }
}

// x[b, :] += sum over ranks r (ascending) of sum over split-K partials s of part_r[s][b][:]
// then xn = bf16(x / sqrt(mean(x^2) + eps) * alpha)            (Layer::fwd's residual add + RmsNorm::fwd,
// ug-llama/src/model.rs:65-78,259-269, with the tensor-parallel all-reduce folded in).
// Every rank adds the same numbers in the same order, so the replicas of x stay bit-identical.
// One CTA of 512 threads per row; hidden <= 8192, hidden % 4 == 0.
constexpr int TP_RED_THREADS = 512;
template <int VPT>
__global__ void __launch_bounds__(TP_RED_THREADS)
tp_reduce_rmsnorm_kernel(float *__restrict__ x, TpPeers tp, int n_part, size_t part_stride,
                         const float *__restrict__ alpha, __nv_bfloat16 *__restrict__ xn, int hidden,
                         float inv_d, float eps, ugb_status_word *status) {
  __shared__ float sm[TP_RED_THREADS / 32];
  ugb_pdl_trigger();
  ugb_pdl_wait();
  tp_exchange_begin(tp, status, blockIdx.x == 0);
  const int b = blockIdx.x;
  const int nvec = hidden >> 2;
  float4 *xr = reinterpret_cast<float4 *>(x + (size_t)b * hidden);
  float4 v[VPT];
  float ss = 0.f;
  const int n_loads = tp.size * n_part;        // (rank, partial) pairs, rank-major = the order of the sum
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * TP_RED_THREADS;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < nvec) {
      v[i] = xr[c];
      // Peer loads cross NVLink (microseconds each): up to 16 are requested before the first is used, so a
      // thread waits once per batch instead of once per partial.  ld.cv: never served from this SM's L1,
      // whose lines may be from the buffer's previous use.
      for (int j0 = 0; j0 < n_loads; j0 += 16) {
        float4 p[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int j = j0 + u;
          if (j < n_loads) {
            const int r = j / n_part, sp = j - r * n_part;
            p[u] = __ldcv(reinterpret_cast<const float4 *>(tp.part[r] + (size_t)sp * part_stride + (size_t)b * hidden) + c);
          } else {
            p[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int u = 0; u < 16; ++u)
          if (j0 + u < n_loads) { v[i].x += p[u].x; v[i].y += p[u].y; v[i].z += p[u].z; v[i].w += p[u].w; }
      }
      xr[c] = v[i];
      ss += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
  }
  tp_exchange_end(tp);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = (threadIdx.x & 31) < TP_RED_THREADS / 32 ? sm[threadIdx.x & 31] : 0.f;
  tot = warp_sum(tot);
  const float m = sqrtf(tot * inv_d + eps);
  uint2 *out = reinterpret_cast<uint2 *>(xn + (size_t)b * hidden);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * TP_RED_THREADS;
    if (c < nvec) {
      const float4 w = __ldg(reinterpret_cast<const float4 *>(alpha) + c);
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[i].x / m * w.x, v[i].y / m * w.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(v[i].z / m * w.z, v[i].w / m * w.w);
      out[c] = make_uint2(*(uint32_t *)&lo, *(uint32_t *)&hi);
    }
  }
}

// Vocab-parallel greedy choice.  Stage 1 (per rank): best (value, global id) of the rank's logit
// slice for every row -> pairs[b] in the rank's own exchange block.  One CTA of 1024 threads per row.
static __global__ void __launch_bounds__(1024)
tp_argmax_local_kernel(const float *__restrict__ logits, int vocab_local, int vocab_offset, float2 *__restrict__ pairs) {
  __shared__ float sv[32];
  __shared__ int si[32];
  ugb_pdl_trigger();
  ugb_pdl_wait();
  const int b = blockIdx.x;
  const float4 *row = reinterpret_cast<const float4 *>(logits + (size_t)b * vocab_local);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  auto upd = [&](float v, int j) { if (v > best || (v == best && j < bi)) { best = v; bi = j; } };
  for (int j = threadIdx.x; j < vocab_local / 4; j += blockDim.x) {
    const float4 v = __ldcs(row + j);
    upd(v.x, 4 * j); upd(v.y, 4 * j + 1); upd(v.z, 4 * j + 2); upd(v.w, 4 * j + 3);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    upd(ov, oi);
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      upd(ov, oi);
    }
    if (threadIdx.x == 0) pairs[b] = make_float2(best, __int_as_float(bi == 0x7fffffff ? 0 : bi + vocab_offset));
  }
}

// Stage 2: after the exchange, every rank picks the best pair over the ranks (ties -> lowest id,
// as a single-rank argmax over the whole vocabulary would) and advances the position.  One CTA.
static __global__ void __launch_bounds__(128)
tp_argmax_final_kernel(TpPeers tp, int batch, int *__restrict__ next, int *pos_p, ugb_status_word *status) {
  ugb_pdl_trigger();
  ugb_pdl_wait();
  tp_exchange_begin(tp, status, true);
  for (int b = threadIdx.x; b < batch; b += blockDim.x) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < tp.size; ++r) {
      const float2 p = __ldcv(reinterpret_cast<const float2 *>(tp.part[r]) + b);
      const int j = __float_as_int(p.y);
      if (p.x > best || (p.x == best && j < bi)) { best = p.x; bi = j; }
    }
    next[b] = bi == 0x7fffffff ? 0 : bi;
  }
  if (threadIdx.x == 0) *pos_p = *pos_p + 1;
  tp_exchange_end(tp);
}

}  // namespace ugb_decode
