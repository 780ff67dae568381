// Device kernels of the fused Llama decode step (one new token per sequence).
//
// They restate, fused and in bf16 storage / fp32 arithmetic, the operator
// chain of ug-llama/src/model.rs:203-269 between the matmuls:
//   embed_gather        index_select (model.rs:32-63)
//   reduce_rmsnorm      residual add (model.rs:263,267) + rms_norm (model.rs:65-78)
//   rope_append         split/transpose + rope (cpu_ops.rs:58-127) + cat into the KV cache (model.rs:226-230)
//   decode_attention    repeat + q.kT + scale + softmax + .v + head merge (model.rs:231-245)
//   argmax_rows         greedy pick (the reference samples on the host, main.rs:151-152)
// All of them are HBM- or latency-bound; the attention kernel streams the KV
// cache once with 16-byte cp.async copies and does its two small contractions
// on mma.sync tiles (m16n8k16, 8 query heads of one KV group padded to 16).
#pragma once
#include <cuda_bf16.h>

#include "ugb_internal.h"
#include "tc_ptx.cuh"

namespace ugb_decode {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// x[r, :] = float(embed[id(r), :]) for row r = (sequence s, step i) = (r / t, r % t),
// id(r) = tok[s * tok_stride + tok_off + i] (decode: t = 1, tok_stride = 1, tok_off = 0).
// One CTA per row; ids outside the table raise the status word and leave the row
// untouched.
static __global__ void __launch_bounds__(256)
embed_gather_kernel(const __nv_bfloat16 *__restrict__ embed, const int *__restrict__ tok,
                    float *__restrict__ x, int hidden, int vocab, ugb_status_word *status,
                    int t, int tok_stride, int tok_off) {
  ugb_pdl_trigger();
  ugb_pdl_wait();
  const int b = blockIdx.x;
  const int id = tok[(size_t)(b / t) * tok_stride + tok_off + b % t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && atomicCAS(&status->code, 0u, (unsigned)UGB_ERR_INVALID) == 0u) status->detail = b;
    return;
  }
  const uint4 *src = reinterpret_cast<const uint4 *>(embed + (size_t)id * hidden);
  float4 *dst = reinterpret_cast<float4 *>(x + (size_t)b * hidden);
  for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
    const uint4 v = __ldg(src + c);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
    const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
    const float2 f2 = __bfloat1622float2(h[2]), f3 = __bfloat1622float2(h[3]);
    dst[2 * c] = make_float4(f0.x, f0.y, f1.x, f1.y);
    dst[2 * c + 1] = make_float4(f2.x, f2.y, f3.x, f3.y);
  }
}

// x[b, :] += sum_s part[s][b][:]   (split-K partials of the previous projection,
// summed in a fixed order), then xn = bf16(x / sqrt(mean(x^2) + eps) * alpha).
// One CTA of 256 threads per row; hidden <= 8192, hidden % 4 == 0.
template <int VPT>
__global__ void __launch_bounds__(256)
reduce_rmsnorm_kernel(float *__restrict__ x, const float *__restrict__ part, int n_part,
                      size_t part_stride, const float *__restrict__ alpha,
                      __nv_bfloat16 *__restrict__ xn, int hidden, float inv_d, float eps, int early) {
  __shared__ float sm[8];
  ugb_pdl_trigger();
  // `early`: x was last written two or more kernels back (the previous residual add), so its row and the
  // norm gains are fetched before waiting for the preceding kernel, whose partials are all that is new.
  if (!early) ugb_pdl_wait();
  const int b = blockIdx.x;
  const int nvec = hidden >> 2;
  float4 *xr = reinterpret_cast<float4 *>(x + (size_t)b * hidden);
  float4 v[VPT], w[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    w[i] = v[i];
    if (c < nvec) {
      v[i] = xr[c];
      w[i] = __ldg(reinterpret_cast<const float4 *>(alpha) + c);
    }
  }
  if (early) ugb_pdl_wait();
  if (n_part == 1) {
    // one partial (the tall, unsplit products of a prefill chunk): every load of the row is in flight before
    // the first addition -- the general loop below issues them one round trip at a time
    float4 q[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * 256;
      q[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < nvec) q[i] = __ldcs(reinterpret_cast<const float4 *>(part + (size_t)b * hidden) + c);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * 256;
      if (c < nvec) {
        v[i].x += q[i].x; v[i].y += q[i].y; v[i].z += q[i].z; v[i].w += q[i].w;
        xr[c] = v[i];
        ss += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
      }
    }
  } else
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      for (int s = 0; s < n_part; ++s) {
        const float4 p = __ldcs(reinterpret_cast<const float4 *>(part + s * part_stride + (size_t)b * hidden) + c);
        v[i].x += p.x; v[i].y += p.y; v[i].z += p.z; v[i].w += p.w;
      }
      if (n_part > 0) xr[c] = v[i];
      ss += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = (threadIdx.x & 31) < 8 ? sm[threadIdx.x & 31] : 0.f;
  tot = warp_sum(tot);
  const float m = sqrtf(tot * inv_d + eps);
  uint2 *out = reinterpret_cast<uint2 *>(xn + (size_t)b * hidden);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[i].x / m * w[i].x, v[i].y / m * w[i].y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(v[i].z / m * w[i].z, v[i].w / m * w[i].w);
      out[c] = make_uint2(*(uint32_t *)&lo, *(uint32_t *)&hi);
    }
  }
}

// Row r = (sequence b, step i) = (r / t, r % t) of a block of t new positions per
// sequence (decode: t = 1).  qkv[r, :] = sum_s part[s][r][:]  (fp32), then
//   q  -> rope -> bf16 q_out[r][head][d]
//   k  -> rope -> bf16 K cache [b][kvh][pos][d]
//   v  ->         bf16 V cache [b][kvh][pos][d]
// with pos = *pos_p + pos_off + i: the base position is read from device memory
// (every sequence of the batch sits at the same position, the reference's pos[0]
// convention, cpu_ops.rs:67-71).  grid = (rows, ceil(items / 256)): one thread
// per FOUR rotation pairs or four v elements -- 128-bit loads of the fp32
// sums and of the cos / sin rows, 64- or 128-bit bf16 stores -- so that all of a
// thread's loads are independent and issued at once.  hd % 8 == 0.
static __global__ void __launch_bounds__(256)
rope_append_kernel(const float *__restrict__ part, int n_part, size_t part_stride,
                   const float *__restrict__ cos_, const float *__restrict__ sin_,
                   const int *__restrict__ pos_p, __nv_bfloat16 *__restrict__ q_out,
                   __nv_bfloat16 *__restrict__ kcache, __nv_bfloat16 *__restrict__ vcache,
                   int n_heads, int n_kv, int hd, int t_max, int interleaved, int t, int pos_off) {
  ugb_pdl_trigger();
  ugb_pdl_wait();
  const int r = blockIdx.x, b = r / t;
  const int it = blockIdx.y * blockDim.x + threadIdx.x;
  const int half = hd >> 1, quads = half >> 2;          // groups of 4 rotation pairs per head
  const int n_rot = (n_heads + n_kv) * quads;
  const int qkv_dim = (n_heads + 2 * n_kv) * hd;
  const float *row = part + (size_t)r * qkv_dim;
  const int pos = *pos_p + pos_off + r % t;
  auto sum4 = [&](int col) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n_part; ++s) {
      const float4 p = *reinterpret_cast<const float4 *>(row + s * part_stride + col);
      a.x += p.x; a.y += p.y; a.z += p.z; a.w += p.w;
    }
    return a;
  };
  auto pack2 = [](float lo, float hi) { __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t *>(&v); };
  if (it < n_rot) {
    const int head = it / quads, i = (it - head * quads) * 4;          // pairs i .. i + 3 of this head
    const float4 c = *reinterpret_cast<const float4 *>(cos_ + (size_t)pos * half + i);
    const float4 sn = *reinterpret_cast<const float4 *>(sin_ + (size_t)pos * half + i);
    __nv_bfloat16 *dst = head < n_heads
        ? q_out + ((size_t)r * n_heads + head) * hd
        : kcache + (((size_t)b * n_kv + (head - n_heads)) * t_max + pos) * hd;
    // dst[i1] = x1 c - x2 s, dst[i2] = x1 s + x2 c, each product and sum rounded separately (cpu_ops.rs:73-78)
    if (interleaved) {                                                  // pairs (2i, 2i + 1): 8 contiguous values
      const float4 u = sum4(head * hd + 2 * i), w = sum4(head * hd + 2 * i + 4);
      uint4 o;
      o.x = pack2(__fsub_rn(__fmul_rn(u.x, c.x), __fmul_rn(u.y, sn.x)), __fadd_rn(__fmul_rn(u.x, sn.x), __fmul_rn(u.y, c.x)));
      o.y = pack2(__fsub_rn(__fmul_rn(u.z, c.y), __fmul_rn(u.w, sn.y)), __fadd_rn(__fmul_rn(u.z, sn.y), __fmul_rn(u.w, c.y)));
      o.z = pack2(__fsub_rn(__fmul_rn(w.x, c.z), __fmul_rn(w.y, sn.z)), __fadd_rn(__fmul_rn(w.x, sn.z), __fmul_rn(w.y, c.z)));
      o.w = pack2(__fsub_rn(__fmul_rn(w.z, c.w), __fmul_rn(w.w, sn.w)), __fadd_rn(__fmul_rn(w.z, sn.w), __fmul_rn(w.w, c.w)));
      *reinterpret_cast<uint4 *>(dst + 2 * i) = o;
    } else {                                                            // pairs (i, i + hd / 2)
      const float4 x1 = sum4(head * hd + i), x2 = sum4(head * hd + i + half);
      uint2 lo, hi;
      lo.x = pack2(__fsub_rn(__fmul_rn(x1.x, c.x), __fmul_rn(x2.x, sn.x)), __fsub_rn(__fmul_rn(x1.y, c.y), __fmul_rn(x2.y, sn.y)));
      lo.y = pack2(__fsub_rn(__fmul_rn(x1.z, c.z), __fmul_rn(x2.z, sn.z)), __fsub_rn(__fmul_rn(x1.w, c.w), __fmul_rn(x2.w, sn.w)));
      hi.x = pack2(__fadd_rn(__fmul_rn(x1.x, sn.x), __fmul_rn(x2.x, c.x)), __fadd_rn(__fmul_rn(x1.y, sn.y), __fmul_rn(x2.y, c.y)));
      hi.y = pack2(__fadd_rn(__fmul_rn(x1.z, sn.z), __fmul_rn(x2.z, c.z)), __fadd_rn(__fmul_rn(x1.w, sn.w), __fmul_rn(x2.w, c.w)));
      *reinterpret_cast<uint2 *>(dst + i) = lo;
      *reinterpret_cast<uint2 *>(dst + i + half) = hi;
    }
  } else if (it < n_rot + n_kv * (hd >> 2)) {
    const int e = (it - n_rot) * 4;                                     // 4 contiguous v values
    const int head = e / hd, i = e - head * hd;
    const float4 x = sum4((n_heads + n_kv) * hd + e);
    uint2 o;
    o.x = pack2(x.x, x.y);
    o.y = pack2(x.z, x.w);
    *reinterpret_cast<uint2 *>(vcache + (((size_t)b * n_kv + head) * t_max + pos) * hd + i) = o;
  }
}

// ------------------------------------------------------------- attention ---
__device__ __forceinline__ void mma_bf16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                 uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t smem, const void *gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {      // addr: a shared::cluster address (mapa)
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *(uint32_t *)&t;
}

constexpr int ATT_WARPS = 4;
constexpr int ATT_STAGES = 3;          // 16-key sub-tiles in flight per warp (default ring depth)
constexpr int ATT_SUB = 16;            // keys per sub-tile
constexpr int ATT_HD = 64;             // head dim (compile-time: fragment layout)
constexpr int ATT_GROUP = 8;           // query heads per KV head (<= 8, padded to the 16-row tile)
constexpr int ATT_SUB_BYTES = ATT_SUB * ATT_HD * 2;   // 2 KiB per K or V sub-tile
constexpr int att_ring_bytes(int stages) { return ATT_WARPS * stages * 2 * ATT_SUB_BYTES; }   // dynamic shared memory
constexpr int ATT_RING_BYTES = att_ring_bytes(ATT_STAGES);

// Flash-decode for one new query position per sequence, grouped-query heads.
//   grid = (n_split, n_kv, batch), 128 threads.
// CTA (sp, kvh, b) covers the sp-th slice of the T = pos + 1 cached positions of
// sequence b, KV head kvh, for the `group` query heads that share it.  Each warp
// walks its own 16-key sub-tiles (a private cp.async ring, no CTA barrier in the
// loop) with a private online-softmax state; the four states are merged through
// shared memory, written as a partial (m, l, O) and the last CTA of a (b, kvh)
// to finish combines the partials of all slices into the bf16 output
//   out[b][head][d]   (= the transposed + merged layout o_proj consumes).
// K frags use a permuted k index (dims 16t+4s.. for lane t, step s) so that a
// lane's operands are two contiguous 16-byte pieces of a row; Q uses the same
// permutation.  V frags come from ldmatrix.trans on the staged sub-tile.
// Fused front end (the engine's decode step): with `rope.part` set, q / k / v of the new position are
// taken from the fp32 split-K partials of the qkv projection ([s][b][(n_heads + 2 n_kv) * 64]) instead
// of `q`: the CTA sums the partials in order, applies the rotation (each product and sum rounded
// separately, as ug-llama/src/cpu_ops.rs:73-78), rounds to bf16 (q once per CTA, 64 threads with 8 independent
// loads each, handed to the warps' fragments through shared memory: 2.4 us against 4.8 when every warp
// fetched and rotated all of q for itself), and -- the CTA whose slice holds the
// new position, when `rope.append` -- writes the K / V rows of position pos into the cache before it
// reads them back with the rest of its slice.  Same arithmetic as rope_append_kernel.
struct AttRope {
  const float *part;
  int n_part;
  size_t part_stride;
  const float *cos_, *sin_;
  int interleaved, append;
  int early;                     // 1: the ring may be filled before griddepcontrol.wait (see the kernel)
  int cluster;                   // 1: the launch groups the KV slices of a (sequence, KV head) pair into one thread-block
                                 // cluster (cluster dims = (n_split, 1, 1)): the slices are combined through
                                 // distributed shared memory instead of scratch, fence, counter and a last CTA
  ugb_status_word *status;       // where a position outside the cache, or (TMA variant) a wait that gave up, is reported
};

// TMA variant (TMA = true): the K / V sub-tiles arrive by cp.async.bulk.tensor through rank-3 maps over the
// caches (dims {64, t_max, sequences x KV heads}, box {64, 16, 1}, 128-byte swizzle = the XOR pattern the
// cp.async path applies by hand); one lane issues the two copies of a sub-tile and the warp waits on the
// stage's mbarrier (bounded: 2^22 polls, then the status word is raised and the warp goes on).
constexpr int att_dyn_smem(int stages, bool tma) {
  return att_ring_bytes(stages) + (tma ? 1024 + ATT_WARPS * stages * 8 : 0);
}

template <int NSTAGE, bool TMA = false>
__global__ void __launch_bounds__(ATT_WARPS * 32)
decode_attention_kernel_t(const __nv_bfloat16 *__restrict__ q, __nv_bfloat16 *__restrict__ kcache,
                        __nv_bfloat16 *__restrict__ vcache, const int *__restrict__ pos_p,
                        float *__restrict__ part_o, float *__restrict__ part_ml,
                        unsigned int *__restrict__ counters, __nv_bfloat16 *__restrict__ out,
                        int n_heads, int n_kv, int group, int t_max, float scale, AttRope rope,
                        const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
  extern __shared__ __align__(128) uint8_t att_smem_raw[];                 // the K / V ring
  // the swizzle atoms of the TMA variant are 1024 bytes: align the ring by hand
  uint8_t *att_smem = TMA ? (uint8_t *)(((uintptr_t)att_smem_raw + 1023) & ~(uintptr_t)1023) : att_smem_raw;
  uint8_t (*ring)[NSTAGE][2][ATT_SUB_BYTES] =
      reinterpret_cast<uint8_t (*)[NSTAGE][2][ATT_SUB_BYTES]>(att_smem);
  uint64_t *bars = reinterpret_cast<uint64_t *>(att_smem + att_ring_bytes(NSTAGE));   // [warp][stage], TMA only
  __shared__ float merge_o[ATT_WARPS][ATT_GROUP][ATT_HD];
  __shared__ float merge_ml[ATT_WARPS][ATT_GROUP][2];
  __shared__ float cl_o[ATT_GROUP][ATT_HD], cl_ml[ATT_GROUP][2];   // this CTA's slice result, read by the cluster's rank 0
  __shared__ int is_last;

  if (TMA) {
    if (threadIdx.x == 0) {
      for (int i = 0; i < ATT_WARPS * NSTAGE; ++i) ugb_tc::mbar_init(ugb_tc::smem_u32(&bars[i]), 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmK) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmV) : "memory");
    }
    __syncthreads();
  }
  // With rope.early the ring is filled before waiting for the preceding kernel (the qkv projection), whose
  // output only the rotation of q and the new cache row need: the cached rows of earlier positions were
  // written a step ago.  The caller sets it only where the position counter, too, is certainly up to date
  // (not for the first layer of a step, which follows the previous step's argmax closely).
  ugb_pdl_trigger();
  bool dep_ready = false;
  if (rope.part == nullptr || !rope.early) { ugb_pdl_wait(); dep_ready = true; }
  const int sp = blockIdx.x, n_split = gridDim.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int T = *pos_p + 1;
  // The position lives on the device: a stale or oversized value would walk (and, when appending, write) past
  // the cache, where the reference panics on a slice bound.  Nothing is touched then; the status word is raised.
  if (T < 1 || T > t_max) {
    if (!dep_ready) ugb_pdl_wait();
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && rope.status != nullptr &&
        atomicCAS(&rope.status->code, 0u, (unsigned)UGB_ERR_INVALID) == 0u)
      rope.status->detail = (unsigned)(T - 1);
    return;
  }
  const int n_sub = (T + ATT_SUB - 1) / ATT_SUB;
  const int sub_per_split = (n_sub + n_split - 1) / n_split;
  const int sub_lo = sp * sub_per_split;
  const int sub_hi = min(n_sub, sub_lo + sub_per_split);

  const __nv_bfloat16 *kbase = kcache + ((size_t)b * n_kv + kvh) * (size_t)t_max * ATT_HD;
  const __nv_bfloat16 *vbase = vcache + ((size_t)b * n_kv + kvh) * (size_t)t_max * ATT_HD;

  // Q fragments (rows >= group are zero padding): lane (g, t) holds dims 16t .. 16t + 15 of query head g.
  // With the fused front end they are computed after the ring has been filled (below).
  uint32_t qa[8];
  if (rope.part == nullptr) {
    uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
    if (g < group) {
      const uint4 *qp = reinterpret_cast<const uint4 *>(q + ((size_t)b * n_heads + kvh * group + g) * ATT_HD + 16 * t);
      lo = __ldg(qp);
      hi = __ldg(qp + 1);
    }
    qa[0] = lo.x; qa[1] = lo.y; qa[2] = lo.z; qa[3] = lo.w;
    qa[4] = hi.x; qa[5] = hi.y; qa[6] = hi.z; qa[7] = hi.w;
  }
  const int half = ATT_HD / 2;
  const float *rope_row = rope.part ? rope.part + (size_t)b * ((n_heads + 2 * n_kv) * ATT_HD) : nullptr;
  auto sum4 = [&](int col) {       // all partials requested before the first is used (at most 8 of them)
    float4 p[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
      p[s] = s < rope.n_part ? __ldcg(reinterpret_cast<const float4 *>(rope_row + s * rope.part_stride + col))
                             : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 8; ++s)
      if (s < rope.n_part) { a.x += p[s].x; a.y += p[s].y; a.z += p[s].z; a.w += p[s].w; }
    return a;
  };
  // K / V rows of the new position: written by the warp that will fetch the sub-tile holding them, so
  // that no CTA barrier is needed -- before the ring is filled when that sub-tile is part of the fill,
  // otherwise after, with the fill's loads in flight.
  auto append_kv = [&]() {
    const int pos = T - 1;
    const int kcol = (n_heads + kvh) * ATT_HD, vcol = (n_heads + n_kv + kvh) * ATT_HD;
    __nv_bfloat16 *kd = kcache + (((size_t)b * n_kv + kvh) * t_max + pos) * ATT_HD;
    __nv_bfloat16 *vd = vcache + (((size_t)b * n_kv + kvh) * t_max + pos) * ATT_HD;
    if (lane < 8) {                                      // 4 rotation pairs per lane
      const int i = lane * 4;
      const float4 c = *reinterpret_cast<const float4 *>(rope.cos_ + (size_t)pos * half + i);
      const float4 sn = *reinterpret_cast<const float4 *>(rope.sin_ + (size_t)pos * half + i);
      if (rope.interleaved) {
        const float4 u = sum4(kcol + 2 * i), w = sum4(kcol + 2 * i + 4);
        uint4 o;
        o.x = pack_bf16(__fsub_rn(__fmul_rn(u.x, c.x), __fmul_rn(u.y, sn.x)), __fadd_rn(__fmul_rn(u.x, sn.x), __fmul_rn(u.y, c.x)));
        o.y = pack_bf16(__fsub_rn(__fmul_rn(u.z, c.y), __fmul_rn(u.w, sn.y)), __fadd_rn(__fmul_rn(u.z, sn.y), __fmul_rn(u.w, c.y)));
        o.z = pack_bf16(__fsub_rn(__fmul_rn(w.x, c.z), __fmul_rn(w.y, sn.z)), __fadd_rn(__fmul_rn(w.x, sn.z), __fmul_rn(w.y, c.z)));
        o.w = pack_bf16(__fsub_rn(__fmul_rn(w.z, c.w), __fmul_rn(w.w, sn.w)), __fadd_rn(__fmul_rn(w.z, sn.w), __fmul_rn(w.w, c.w)));
        *reinterpret_cast<uint4 *>(kd + 2 * i) = o;
      } else {
        const float4 x1 = sum4(kcol + i), x2 = sum4(kcol + i + half);
        uint2 lo, hi;
        lo.x = pack_bf16(__fsub_rn(__fmul_rn(x1.x, c.x), __fmul_rn(x2.x, sn.x)), __fsub_rn(__fmul_rn(x1.y, c.y), __fmul_rn(x2.y, sn.y)));
        lo.y = pack_bf16(__fsub_rn(__fmul_rn(x1.z, c.z), __fmul_rn(x2.z, sn.z)), __fsub_rn(__fmul_rn(x1.w, c.w), __fmul_rn(x2.w, sn.w)));
        hi.x = pack_bf16(__fadd_rn(__fmul_rn(x1.x, sn.x), __fmul_rn(x2.x, c.x)), __fadd_rn(__fmul_rn(x1.y, sn.y), __fmul_rn(x2.y, c.y)));
        hi.y = pack_bf16(__fadd_rn(__fmul_rn(x1.z, sn.z), __fmul_rn(x2.z, c.z)), __fadd_rn(__fmul_rn(x1.w, sn.w), __fmul_rn(x2.w, c.w)));
        *reinterpret_cast<uint2 *>(kd + i) = lo;
        *reinterpret_cast<uint2 *>(kd + i + half) = hi;
      }
    } else if (lane < 24) {                              // 4 v values per lane
      const int i = (lane - 8) * 4;
      const float4 x = sum4(vcol + i);
      *reinterpret_cast<uint2 *>(vd + i) = make_uint2(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w));
    }
    __threadfence();                                     // in L2 before this warp's cp.async fetches the row
    if (TMA) asm volatile("fence.proxy.async;" ::: "memory");   // ... or before the TMA engine reads it
    __syncwarp();
  };
  const int sub_pos = (T - 1) / ATT_SUB;                 // sub-tile of the new position
  const bool appender = rope.part != nullptr && rope.append && sub_pos >= sub_lo && sub_pos < sub_hi &&
                        ((sub_pos - sub_lo) & (ATT_WARPS - 1)) == warp;

  auto issue = [&](int sub, int stage) {
    // 16 keys x 128 B for K and for V: 4 + 4 chunks of 16 B per lane, XOR-swizzled rows
    const uint32_t ks = (uint32_t)__cvta_generic_to_shared(&ring[warp][stage][0][0]);
    const uint32_t vs = (uint32_t)__cvta_generic_to_shared(&ring[warp][stage][1][0]);
    if (TMA) {
      if (lane == 0) {
        const uint32_t bar = ugb_tc::smem_u32(&bars[warp * NSTAGE + stage]);
        ugb_tc::mbar_expect_tx(bar, 2 * ATT_SUB_BYTES);
        ugb_tc::tma_load_3d(ks, &tmK, bar, 0, sub * ATT_SUB, b * n_kv + kvh);
        ugb_tc::tma_load_3d(vs, &tmV, bar, 0, sub * ATT_SUB, b * n_kv + kvh);
      }
      return;
    }
    const char *kg = reinterpret_cast<const char *>(kbase + (size_t)sub * ATT_SUB * ATT_HD);
    const char *vg = reinterpret_cast<const char *>(vbase + (size_t)sub * ATT_SUB * ATT_HD);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = lane + 32 * i, key = c >> 3, ch = c & 7;
      const uint32_t so = key * 128 + ((ch ^ (key & 7)) << 4);
      cp_async16(ks + so, kg + c * 16);
      cp_async16(vs + so, vg + c * 16);
    }
  };

  float m_run = -INFINITY, l_run = 0.f;   // row g (this lane's query head)
  float o[8][4];
#pragma unroll
  for (int d = 0; d < 8; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

  // prologue: fill the ring
  const int first = sub_lo + warp;
  const bool append_first = appender && sub_pos < first + (NSTAGE - 1) * ATT_WARPS;
  if (!dep_ready && append_first) { ugb_pdl_wait(); dep_ready = true; }   // the new row comes first
  if (append_first) append_kv();
#pragma unroll
  for (int s = 0; s < NSTAGE - 1; ++s) {
    const int sub = first + s * ATT_WARPS;
    if (sub < sub_hi) issue(sub, s);
    cp_async_commit();
  }
  if (!dep_ready) ugb_pdl_wait();
  if (appender && !append_first) append_kv();
  if (rope.part != nullptr) {
    // ---- q of the 8 heads, rotated: computed once per CTA (threads 0..63: one head and 8 of its dims each, all
    // of a thread's loads requested before the first is used), rounded to bf16 and handed to the four warps
    // through shared memory, each lane picking up the 16 dims of its fragment --------------------------------
    __shared__ __align__(16) uint32_t q_sh[ATT_GROUP][ATT_HD / 2];
    if (threadIdx.x < 64) {
      const int h = threadIdx.x >> 3, c = threadIdx.x & 7;
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      if (h < group) {
        const int pos = T - 1, qcol = (kvh * group + h) * ATT_HD;
        const float4 cs = *reinterpret_cast<const float4 *>(rope.cos_ + (size_t)pos * half + 4 * c);
        const float4 sn = *reinterpret_cast<const float4 *>(rope.sin_ + (size_t)pos * half + 4 * c);
        if (rope.interleaved) {                              // pairs (2i, 2i + 1), i = 4c .. 4c + 3: dims 8c .. 8c + 7
          const float4 u = sum4(qcol + 8 * c), w = sum4(qcol + 8 * c + 4);
          lo.x = pack_bf16(__fsub_rn(__fmul_rn(u.x, cs.x), __fmul_rn(u.y, sn.x)), __fadd_rn(__fmul_rn(u.x, sn.x), __fmul_rn(u.y, cs.x)));
          lo.y = pack_bf16(__fsub_rn(__fmul_rn(u.z, cs.y), __fmul_rn(u.w, sn.y)), __fadd_rn(__fmul_rn(u.z, sn.y), __fmul_rn(u.w, cs.y)));
          lo.z = pack_bf16(__fsub_rn(__fmul_rn(w.x, cs.z), __fmul_rn(w.y, sn.z)), __fadd_rn(__fmul_rn(w.x, sn.z), __fmul_rn(w.y, cs.z)));
          lo.w = pack_bf16(__fsub_rn(__fmul_rn(w.z, cs.w), __fmul_rn(w.w, sn.w)), __fadd_rn(__fmul_rn(w.z, sn.w), __fmul_rn(w.w, cs.w)));
          *reinterpret_cast<uint4 *>(&q_sh[h][4 * c]) = lo;
        } else {                                             // pairs (i, i + 32), i = 4c .. 4c + 3
          const float4 x1 = sum4(qcol + 4 * c), x2 = sum4(qcol + half + 4 * c);
          lo.x = pack_bf16(__fsub_rn(__fmul_rn(x1.x, cs.x), __fmul_rn(x2.x, sn.x)), __fsub_rn(__fmul_rn(x1.y, cs.y), __fmul_rn(x2.y, sn.y)));
          lo.y = pack_bf16(__fsub_rn(__fmul_rn(x1.z, cs.z), __fmul_rn(x2.z, sn.z)), __fsub_rn(__fmul_rn(x1.w, cs.w), __fmul_rn(x2.w, sn.w)));
          hi.x = pack_bf16(__fadd_rn(__fmul_rn(x1.x, sn.x), __fmul_rn(x2.x, cs.x)), __fadd_rn(__fmul_rn(x1.y, sn.y), __fmul_rn(x2.y, cs.y)));
          hi.y = pack_bf16(__fadd_rn(__fmul_rn(x1.z, sn.z), __fmul_rn(x2.z, cs.z)), __fadd_rn(__fmul_rn(x1.w, sn.w), __fmul_rn(x2.w, cs.w)));
          *reinterpret_cast<uint2 *>(&q_sh[h][2 * c]) = make_uint2(lo.x, lo.y);
          *reinterpret_cast<uint2 *>(&q_sh[h][16 + 2 * c]) = make_uint2(hi.x, hi.y);
        }
      } else if (rope.interleaved) {
        *reinterpret_cast<uint4 *>(&q_sh[h][4 * c]) = lo;    // zero padding rows
      } else {
        *reinterpret_cast<uint2 *>(&q_sh[h][2 * c]) = make_uint2(0u, 0u);
        *reinterpret_cast<uint2 *>(&q_sh[h][16 + 2 * c]) = make_uint2(0u, 0u);
      }
    }
    __syncthreads();
    {
      const uint4 lo = *reinterpret_cast<const uint4 *>(&q_sh[g][8 * t]);
      const uint4 hi = *reinterpret_cast<const uint4 *>(&q_sh[g][8 * t + 4]);
      qa[0] = lo.x; qa[1] = lo.y; qa[2] = lo.z; qa[3] = lo.w;
      qa[4] = hi.x; qa[5] = hi.y; qa[6] = hi.z; qa[7] = hi.w;
    }
  }
  int stage = 0;
  uint32_t phases = 0;                                   // TMA: parity of the next completion of every stage
  for (int sub = first; sub < sub_hi; sub += ATT_WARPS) {
    {
      const int nxt = sub + (NSTAGE - 1) * ATT_WARPS;
      const int nstage = (stage + NSTAGE - 1) % NSTAGE;
      if (nxt < sub_hi) issue(nxt, nstage);
      cp_async_commit();
    }
    if (TMA) {
      const uint32_t bar = ugb_tc::smem_u32(&bars[warp * NSTAGE + stage]);
      const uint32_t par = (phases >> stage) & 1u;
      unsigned polls = 0;
      while (!ugb_tc::mbar_try(bar, par)) {
        if (++polls > (1u << 22)) {                      // the copy never landed: report, do not hang
          if (lane == 0 && atomicCAS(&rope.status->code, 0u, (unsigned)UGB_ERR_TIMEOUT) == 0u) rope.status->detail = 0x51u;
          break;
        }
      }
      phases ^= 1u << stage;
    } else {
      cp_async_wait<NSTAGE - 1>();
    }
    __syncwarp();
    const uint8_t *ks = &ring[warp][stage][0][0];
    const uint32_t vs = (uint32_t)__cvta_generic_to_shared(&ring[warp][stage][1][0]);

    // S = Q . K^T for 16 keys: two n-tiles of 8 keys
    float s_acc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.f;
      const int key = 8 * j + g;
      const uint4 k0 = *reinterpret_cast<const uint4 *>(ks + key * 128 + (((2 * t) ^ (key & 7)) << 4));
      const uint4 k1 = *reinterpret_cast<const uint4 *>(ks + key * 128 + (((2 * t + 1) ^ (key & 7)) << 4));
      mma_bf16_16x8x16(s_acc[j], qa[0], 0u, qa[1], 0u, k0.x, k0.y);
      mma_bf16_16x8x16(s_acc[j], qa[2], 0u, qa[3], 0u, k0.z, k0.w);
      mma_bf16_16x8x16(s_acc[j], qa[4], 0u, qa[5], 0u, k1.x, k1.y);
      mma_bf16_16x8x16(s_acc[j], qa[6], 0u, qa[7], 0u, k1.z, k1.w);
    }
    // scale, mask keys >= T, online softmax on row g (values [j][0], [j][1])
    const int key0 = sub * ATT_SUB;
    float sv[4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + 8 * j + 2 * t + e;
        sv[2 * j + e] = key < T ? s_acc[j][e] * scale : -INFINITY;
      }
    float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);             // finite: key0 < T for every sub-tile visited
    const float alpha = __expf(m_run - m_new);
    float p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) p[e] = __expf(sv[e] - m_new);
    l_run = l_run * alpha + ((p[0] + p[1]) + (p[2] + p[3]));
    m_run = m_new;
#pragma unroll
    for (int d = 0; d < 8; ++d) { o[d][0] *= alpha; o[d][1] *= alpha; }
    const uint32_t pa0 = pack_bf16(p[0], p[1]), pa2 = pack_bf16(p[2], p[3]);

    // O += P . V : 8 n-tiles of 8 dims, k = 16 keys; B frags by ldmatrix.trans
#pragma unroll
    for (int d = 0; d < 8; d += 2) {
      const int mi = lane >> 3, ri = lane & 7;
      const int key = ri + 8 * (mi & 1), ch = d + (mi >> 1);
      const uint32_t addr = vs + key * 128 + ((ch ^ (key & 7)) << 4);
      uint32_t r0, r1, r2, r3;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
      mma_bf16_16x8x16(o[d], pa0, 0u, pa2, 0u, r0, r1);
      mma_bf16_16x8x16(o[d + 1], pa0, 0u, pa2, 0u, r2, r3);
    }
    __syncwarp();
    stage = (stage + 1) % NSTAGE;
  }
  cp_async_wait<0>();

  // l is a per-lane partial over this lane's key columns: finish the row sum
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

  // ---- merge the four warps of this CTA -----------------------------------
  if (g < ATT_GROUP) {
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      merge_o[warp][g][8 * d + 2 * t] = o[d][0];
      merge_o[warp][g][8 * d + 2 * t + 1] = o[d][1];
    }
    if (t == 0) { merge_ml[warp][g][0] = m_run; merge_ml[warp][g][1] = l_run; }
  }
  __syncthreads();
  const size_t slot = ((size_t)b * n_kv + kvh) * n_split + sp;
  for (int idx = threadIdx.x; idx < ATT_GROUP * ATT_HD; idx += blockDim.x) {
    const int h = idx / ATT_HD, dd = idx - h * ATT_HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, merge_ml[w][h][0]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float f = merge_ml[w][h][0] == -INFINITY ? 0.f : __expf(merge_ml[w][h][0] - mm);
      acc += merge_o[w][h][dd] * f;
      ll += merge_ml[w][h][1] * f;
    }
    if (n_split == 1) {      // the only slice: no partials, no counter
      if (h < group) out[((size_t)b * n_heads + kvh * group + h) * ATT_HD + dd] = __float2bfloat16_rn(acc / ll);
      continue;
    }
    if (rope.cluster) {
      cl_o[h][dd] = acc;
      if (dd == 0) { cl_ml[h][0] = mm; cl_ml[h][1] = ll; }
      continue;
    }
    part_o[(slot * ATT_GROUP + h) * ATT_HD + dd] = acc;
    if (dd == 0) { part_ml[(slot * ATT_GROUP + h) * 2] = mm; part_ml[(slot * ATT_GROUP + h) * 2 + 1] = ll; }
  }
  if (n_split == 1) return;
  if (rope.cluster) {
    // ---- the slices of this (b, kvh) are the CTAs of one cluster (rank = slice): rank 0 combines them in slice
    // order, the same sums as the scratch path below, reading the peers' shared memory -------------------------
    ugb_tc::cluster_sync_all();                     // every slice's result is in its CTA's shared memory
    if (sp == 0) {
      for (int idx = threadIdx.x; idx < group * ATT_HD; idx += blockDim.x) {
        const int h = idx / ATT_HD, dd = idx - h * ATT_HD;
        const uint32_t a_ml = ugb_tc::smem_u32(&cl_ml[h][0]), a_o = ugb_tc::smem_u32(&cl_o[h][dd]);
        float ms[8], ls[8], os[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          const bool on = s < n_split;
          const uint32_t r = (uint32_t)(on ? s : 0);
          ms[s] = on ? ld_cluster_f32(ugb_tc::mapa_u32(a_ml, r)) : -INFINITY;
          ls[s] = on ? ld_cluster_f32(ugb_tc::mapa_u32(a_ml + 4, r)) : 0.f;
          os[s] = on ? ld_cluster_f32(ugb_tc::mapa_u32(a_o, r)) : 0.f;
        }
        float mm = -INFINITY;
#pragma unroll
        for (int s = 0; s < 8; ++s) mm = fmaxf(mm, ms[s]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if (s < n_split) {
            const float f = ms[s] == -INFINITY ? 0.f : __expf(ms[s] - mm);
            acc += os[s] * f;
            ll += ls[s] * f;
          }
        }
        out[((size_t)b * n_heads + kvh * group + h) * ATT_HD + dd] = __float2bfloat16_rn(acc / ll);
      }
    }
    ugb_tc::cluster_sync_all();                     // no CTA leaves while rank 0 may still read its shared memory
    return;
  }
  // ---- last CTA of this (b, kvh) combines the slices ------------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&counters[(size_t)b * n_kv + kvh], 1u);
    is_last = (prev == (unsigned)n_split - 1u);
    if (is_last) counters[(size_t)b * n_kv + kvh] = 0u;   // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const size_t slot0 = ((size_t)b * n_kv + kvh) * n_split;
  // at most 8 slices (the launcher's limit): every partial of an output element is requested before the first
  // is used, so the combine costs one round trip to L2 instead of one per slice
  for (int idx = threadIdx.x; idx < group * ATT_HD; idx += blockDim.x) {
    const int h = idx / ATT_HD, dd = idx - h * ATT_HD;
    float ms[8], ls[8], os[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const bool on = s < n_split;
      const size_t sl = (slot0 + (on ? s : 0)) * ATT_GROUP + h;
      ms[s] = on ? __ldcg(&part_ml[sl * 2]) : -INFINITY;
      ls[s] = on ? __ldcg(&part_ml[sl * 2 + 1]) : 0.f;
      os[s] = on ? __ldcg(&part_o[sl * ATT_HD + dd]) : 0.f;
    }
    float mm = -INFINITY;
#pragma unroll
    for (int s = 0; s < 8; ++s) mm = fmaxf(mm, ms[s]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < n_split) {
        const float f = ms[s] == -INFINITY ? 0.f : __expf(ms[s] - mm);
        acc += os[s] * f;
        ll += ls[s] * f;
      }
    }
    out[((size_t)b * n_heads + kvh * group + h) * ATT_HD + dd] = __float2bfloat16_rn(acc / ll);
  }
}

#define decode_attention_kernel decode_attention_kernel_t<ATT_STAGES>

// next[b] = argmax_j logits[b, j] (ties -> lowest index); thread 0 of CTA 0 also
// advances the shared position counter.  One CTA of 1024 threads per row,
// 128-bit loads (vocab % 4 == 0).
static __global__ void __launch_bounds__(1024)
argmax_rows_kernel(const float *__restrict__ logits, int vocab, int *__restrict__ next, int *pos_p) {
  __shared__ float sv[32];
  __shared__ int si[32];
  ugb_pdl_trigger();
  ugb_pdl_wait();
  const int b = blockIdx.x;
  const float4 *row = reinterpret_cast<const float4 *>(logits + (size_t)b * vocab);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  auto upd = [&](float v, int j) { if (v > best || (v == best && j < bi)) { best = v; bi = j; } };
  for (int j = threadIdx.x; j < vocab / 4; j += blockDim.x) {
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
    if (threadIdx.x == 0) {
      next[b] = bi == 0x7fffffff ? 0 : bi;
      if (b == 0) *pos_p = *pos_p + 1;
    }
  }
}

// cos/sin tables [max_pos, hd/2]: angle = float(pos) * inv_freq[i] as one f32
// product (the [max,1].[1,d/2] matmul of model.rs:291), then precise cosf/sinf.
static __global__ void rope_table_kernel(const float *__restrict__ inv_freq, float *__restrict__ cos_,
                                  float *__restrict__ sin_, int max_pos, int half) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= max_pos * half) return;
  const float ang = __fmul_rn((float)(i / half), inv_freq[i % half]);
  cos_[i] = cosf(ang);
  sin_[i] = sinf(ang);
}

}  // namespace ugb_decode

namespace ugb_decode {

// ------------------------------------------------------ prefill attention ---
// Causal grouped-query attention for a block of `t` new positions per sequence
// (Attention::fwd with seq_len > 1: repeat + q.kT + scale + causal_mask + softmax
// + .v + head merge, ug-llama/src/model.rs:231-245, without materialising the
// [b, h, t, T] score tensor).  Query i attends the cached positions
// 0 .. pos0 + i (the reference's causal_mask assumes pos0 == 0,
// ug-llama/src/cpu_ops.rs:33-56; a non-empty cache is the natural extension).
//   q    bf16 [b, t, n_heads, 64]          (rope already applied)
//   k, v bf16 [b, n_kv, t_max, 64]         (positions < pos0 + t are valid)
//   out  bf16 [b, t, n_heads * 64]
// grid (ceil(t / 64), n_heads, b), 128 threads: a CTA owns 64 queries of one
// head, a warp 16 of them; K / V tiles of 64 keys are staged by cp.async in a
// two-deep shared-memory ring; both contractions run on mma.sync m16n8k16 bf16
// tiles with an online softmax in fp32 registers.
constexpr int PF_BQ = 64, PF_BKV = 64;

static __global__ void __launch_bounds__(128, 4)
prefill_attention_kernel(const __nv_bfloat16 *__restrict__ q, const __nv_bfloat16 *__restrict__ kcache,
                         const __nv_bfloat16 *__restrict__ vcache, __nv_bfloat16 *__restrict__ out, int t, int pos0,
                         int n_heads, int n_kv, int t_max, float scale) {
  __shared__ __align__(128) uint8_t ks[2][PF_BKV * 128];
  __shared__ __align__(128) uint8_t vs[2][PF_BKV * 128];
  const int q0 = blockIdx.x * PF_BQ, head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / (n_heads / n_kv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const __nv_bfloat16 *kbase = kcache + ((size_t)b * n_kv + kvh) * (size_t)t_max * ATT_HD;
  const __nv_bfloat16 *vbase = vcache + ((size_t)b * n_kv + kvh) * (size_t)t_max * ATT_HD;

  // rows of this lane: r_lo = q0 + 16*warp + g, r_hi = r_lo + 8 (query indexes inside the block of t)
  const int r_lo = q0 + 16 * warp + g, r_hi = r_lo + 8;
  uint32_t qa[4][4];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const int c = 16 * s + 2 * tq;
    auto ld = [&](int row, int col) -> uint32_t {
      if (row >= t) return 0u;
      return *reinterpret_cast<const uint32_t *>(q + (((size_t)b * t + row) * n_heads + head) * ATT_HD + col);
    };
    qa[s][0] = ld(r_lo, c);
    qa[s][1] = ld(r_hi, c);
    qa[s][2] = ld(r_lo, c + 8);
    qa[s][3] = ld(r_hi, c + 8);
  }

  const int last_q = min(q0 + PF_BQ, t) - 1;                 // last query of this CTA
  const int n_keys = pos0 + last_q + 1;                       // keys any query of this CTA may attend
  const int n_tiles = (n_keys + PF_BKV - 1) / PF_BKV;

  auto issue = [&](int tile, int stage) {
    const uint32_t kd = (uint32_t)__cvta_generic_to_shared(&ks[stage][0]);
    const uint32_t vd = (uint32_t)__cvta_generic_to_shared(&vs[stage][0]);
    const char *kg = reinterpret_cast<const char *>(kbase + (size_t)tile * PF_BKV * ATT_HD);
    const char *vg = reinterpret_cast<const char *>(vbase + (size_t)tile * PF_BKV * ATT_HD);
#pragma unroll
    for (int i = 0; i < 4; ++i) {                              // 64 keys x 8 chunks of 16 B = 512 chunks, 4 per thread
      const int c = threadIdx.x + 128 * i, key = c >> 3, ch = c & 7;
      const uint32_t so = key * 128 + ((ch ^ (key & 7)) << 4);
      if (tile * PF_BKV + key < t_max) {
        cp_async16(kd + so, kg + c * 16);
        cp_async16(vd + so, vg + c * 16);
      } else {                                                 // past the end of the cache: zeros, masked below
        *reinterpret_cast<uint4 *>(&ks[stage][so]) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4 *>(&vs[stage][so]) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    cp_async_commit();
  };

  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[8][4];
#pragma unroll
  for (int d = 0; d < 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  if (n_tiles > 0) issue(0, 0);
  for (int j = 0; j < n_tiles; ++j) {
    cp_async_wait<0>();
    __syncthreads();                                           // tile j landed; everyone is done with tile j-1
    if (j + 1 < n_tiles) issue(j + 1, (j + 1) & 1);
    const uint32_t kd = (uint32_t)__cvta_generic_to_shared(&ks[j & 1][0]);
    const uint32_t vd = (uint32_t)__cvta_generic_to_shared(&vs[j & 1][0]);

    // S = Q K^T : 8 n-tiles of 8 keys
    float s_acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f;
#pragma unroll
      for (int sp = 0; sp < 2; ++sp) {                         // two k-steps per ldmatrix.x4
        const int mi = lane >> 3, ri = lane & 7;
        const int key = 8 * n + ri, ch = 4 * sp + mi;          // matrices: dim chunks 4sp .. 4sp+3 of keys 8n..8n+7
        uint32_t r0, r1, r2, r3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(kd + key * 128 + ((ch ^ (key & 7)) << 4)));
        mma_bf16_16x8x16(s_acc[n], qa[2 * sp][0], qa[2 * sp][1], qa[2 * sp][2], qa[2 * sp][3], r0, r1);
        mma_bf16_16x8x16(s_acc[n], qa[2 * sp + 1][0], qa[2 * sp + 1][1], qa[2 * sp + 1][2], qa[2 * sp + 1][3], r2, r3);
      }
    }
    // scale + causal mask (key <= pos0 + query), online softmax for the two rows of this lane
    const int key0 = j * PF_BKV;
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + 8 * n + 2 * tq + e;
        s_acc[n][e] = key <= pos0 + r_lo ? s_acc[n][e] * scale : -INFINITY;
        s_acc[n][2 + e] = key <= pos0 + r_hi ? s_acc[n][2 + e] * scale : -INFINITY;
        mx_lo = fmaxf(mx_lo, s_acc[n][e]);
        mx_hi = fmaxf(mx_hi, s_acc[n][2 + e]);
      }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    // a row with nothing to attend yet in this tile keeps max = -inf: use 0 as the reference point
    const float ref_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
    const float a_lo = __expf(m_lo - ref_lo), a_hi = __expf(m_hi - ref_hi);
    float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      s_acc[n][0] = __expf(s_acc[n][0] - ref_lo); s_acc[n][1] = __expf(s_acc[n][1] - ref_lo);
      s_acc[n][2] = __expf(s_acc[n][2] - ref_hi); s_acc[n][3] = __expf(s_acc[n][3] - ref_hi);
      sum_lo += s_acc[n][0] + s_acc[n][1];
      sum_hi += s_acc[n][2] + s_acc[n][3];
    }
    l_lo = l_lo * a_lo + sum_lo; l_hi = l_hi * a_hi + sum_hi;
    m_lo = mn_lo; m_hi = mn_hi;
#pragma unroll
    for (int d = 0; d < 8; ++d) { o[d][0] *= a_lo; o[d][1] *= a_lo; o[d][2] *= a_hi; o[d][3] *= a_hi; }

    // O += P V : k = 64 keys in 4 steps of 16, 8 n-tiles of 8 dims
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t pa0 = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]), pa1 = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
      const uint32_t pa2 = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]), pa3 = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
      for (int d = 0; d < 8; d += 2) {
        const int mi = lane >> 3, ri = lane & 7;
        const int key = 16 * kk + ri + 8 * (mi & 1), ch = d + (mi >> 1);
        uint32_t r0, r1, r2, r3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(vd + key * 128 + ((ch ^ (key & 7)) << 4)));
        mma_bf16_16x8x16(o[d], pa0, pa1, pa2, pa3, r0, r1);
        mma_bf16_16x8x16(o[d + 1], pa0, pa1, pa2, pa3, r2, r3);
      }
    }
  }
  cp_async_wait<0>();
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
  for (int d = 0; d < 8; ++d) {
    const int col = head * ATT_HD + 8 * d + 2 * tq;
    if (r_lo < t)
      *reinterpret_cast<uint32_t *>(out + ((size_t)b * t + r_lo) * ((size_t)n_heads * ATT_HD) + col) = pack_bf16(o[d][0] * inv_lo, o[d][1] * inv_lo);
    if (r_hi < t)
      *reinterpret_cast<uint32_t *>(out + ((size_t)b * t + r_hi) * ((size_t)n_heads * ATT_HD) + col) = pack_bf16(o[d][2] * inv_hi, o[d][3] * inv_hi);
  }
}

}  // namespace ugb_decode
