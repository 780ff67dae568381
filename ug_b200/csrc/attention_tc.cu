// Causal grouped-query attention for a block of new positions on the 5th-generation tensor cores
// (Attention::fwd with seq_len > 1, ug-llama/src/model.rs:231-245: repeat + q.kT + scale + causal_mask +
// softmax + .v + head merge, without the [b, h, t, T] score tensor).
//
//   grid (ceil(t / 128), n_heads, batch), 192 threads, two CTAs per SM (80 KiB of shared memory and 256 TMEM
//   columns each: while one CTA's softmax warps work, the other's products run):
//     warp 0      TMA producer: the 128 x 64 query tile once, then 64-key K and V tiles into two-deep rings
//     warp 1      MMA issuer:   S = Q K^T  (tcgen05.mma M128 N64 K16 x 4, both operands K-major) into one of two
//                               TMEM score buffers; O_j = P V (M128 N64 K16 x 4, V consumed MN-major as it lies
//                               in the cache) into one of two TMEM output buffers
//     warps 2..5  softmax:      one query row per thread (= one TMEM lane): scale, causal mask, running max and
//                               sum without any shuffle, P rounded to bf16 into swizzled shared memory for the
//                               second product; the rescaled sum of the O_j lives in registers
//   S(j+1) is issued before the softmax of tile j has finished, and O_(j-1) is folded in after the softmax of
//   tile j, so that the tensor pipe and the exp pipe overlap.  Every mbarrier wait is bounded (2 s): on expiry
//   the status word is raised, all roles drain, TMEM is freed and the kernel returns.
#include "attention_tc.cuh"

#include "gemm_tcgen05.cuh"
#include "tc_ptx.cuh"

namespace {

using namespace ugb_tc;

constexpr int BQ = 128, BKV = 64, HD = 64;
constexpr int THREADS = 192;
constexpr int Q_BYTES = BQ * HD * 2;          // 16 KiB
constexpr int KV_BYTES = BKV * HD * 2;        // 8 KiB per K or V tile
constexpr int P_BYTES = BQ * BKV * 2;         // 16 KiB: 128 rows x 128 B (64 keys)
constexpr int SMEM_BYTES = Q_BYTES + 4 * KV_BYTES + 2 * P_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 256;                // S: 2 x 64 columns, O: 2 x 64 columns
constexpr int O_COL = 128;
static_assert(BKV == 64 && HD == 64, "one 128-byte swizzle atom per P row and per K / V row");

struct Params {
  int t, pos0, n_heads, n_kv;
  float scale;
  __nv_bfloat16 *out;
  ugb_status_word *status;
};

// 64 consecutive TMEM columns of this thread's lane: both loads in flight, one wait
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&f)[64]) {
  uint32_t r0[32], r1[32];
  tmem_ld_32x32b_x32(taddr, r0);
  tmem_ld_32x32b_x32(taddr + 32, r1);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) { f[i] = __uint_as_float(r0[i]); f[32 + i] = __uint_as_float(r1[i]); }
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(THREADS, 2)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *q_s = smem, *k_s = q_s + Q_BYTES, *v_s = k_s + 2 * KV_BYTES, *p_s = v_s + 2 * KV_BYTES;
  uint64_t *bars = (uint64_t *)(p_s + 2 * P_BYTES);
  uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = bars + 3, *v_full = bars + 5, *v_empty = bars + 7;
  uint64_t *s_full = bars + 9, *p_full = bars + 11, *o_full = bars + 13;
  uint32_t *tmem_slot = (uint32_t *)(bars + 15);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // query tiles in descending order: the CTAs with the most key tiles (causal) start first
  const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * BQ, head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / (p.n_heads / p.n_kv);
  const int last_q = min(q0 + BQ, p.t) - 1;                        // last query row of this CTA
  const int n_tiles = (p.pos0 + last_q + 1 + BKV - 1) / BKV;       // key tiles any of its rows attends

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&p_full[s]), 4);                          // one arrival per softmax warp
      mbar_init(smem_u32(&o_full[s]), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmQ) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmK) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmV) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer --
    if (lane == 0) {
      mbar_expect_tx(smem_u32(q_full), Q_BYTES);
      tma_load_4d(smem_u32(q_s), &tmQ, smem_u32(q_full), 0, head, q0, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!mbar_wait(smem_u32(&k_empty[s]), ph ^ 1u, abort_flag, p.status, 0x41)) break;
        mbar_expect_tx(smem_u32(&k_full[s]), KV_BYTES);
        tma_load_3d(smem_u32(k_s + s * KV_BYTES), &tmK, smem_u32(&k_full[s]), 0, j * BKV, b * p.n_kv + kvh);
        if (!mbar_wait(smem_u32(&v_empty[s]), ph ^ 1u, abort_flag, p.status, 0x42)) break;
        mbar_expect_tx(smem_u32(&v_full[s]), KV_BYTES);
        tma_load_3d(smem_u32(v_s + s * KV_BYTES), &tmV, smem_u32(&v_full[s]), 0, j * BKV, b * p.n_kv + kvh);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer --
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BQ, BKV, false);          // Q and K both K-major (rows of 64 dims)
      const uint32_t idesc_o = make_idesc(BQ, HD, true);            // P K-major, V MN-major ([key][dim] rows)
      bool alive = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status, 0x43);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        if (!mbar_wait(smem_u32(&k_full[s]), (uint32_t)(j >> 1) & 1u, abort_flag, p.status, 0x44)) { alive = false; return; }
        tcgen05_fence_after();
        const uint32_t qa = smem_u32(q_s), kb = smem_u32(k_s + s * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / UMMA_K; ++kk)
          umma_bf16(tmem + (uint32_t)(s * BKV), make_smem_desc(qa + kk * (UMMA_K * 2), 0, 1024),
                    make_smem_desc(kb + kk * (UMMA_K * 2), 0, 1024), idesc_s, kk > 0 ? 1u : 0u);
        umma_commit(smem_u32(&k_empty[s]));                         // K stage free once the products retire
        umma_commit(smem_u32(&s_full[s]));                          // scores ready for the softmax warps
      };
      auto issue_pv = [&](int j) {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!mbar_wait(smem_u32(&p_full[s]), ph, abort_flag, p.status, 0x45)) { alive = false; return; }
        if (!mbar_wait(smem_u32(&v_full[s]), ph, abort_flag, p.status, 0x46)) { alive = false; return; }
        tcgen05_fence_after();
        const uint32_t pa = smem_u32(p_s + s * P_BYTES), vb = smem_u32(v_s + s * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < BKV / UMMA_K; ++kk) {
          // P: 128 rows x 128 B, a step of 16 keys moves 32 B inside the swizzled row.
          // V: rows of 128 B per key, 8-key groups 1024 B apart; a step of 16 keys moves 16 rows.
          const uint64_t ad = make_smem_desc(pa + kk * (UMMA_K * 2), 0, 1024);
          const uint64_t bd = make_smem_desc(vb + kk * (UMMA_K * 128), BKV * 128, 1024);
          umma_bf16(tmem + (uint32_t)(O_COL + s * HD), ad, bd, idesc_o, kk > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&v_empty[s]));
        umma_commit(smem_u32(&o_full[s]));
      };
      if (alive && n_tiles > 0) issue_s(0);
      if (alive && n_tiles > 1) issue_s(1);
      for (int j = 0; j < n_tiles && alive; ++j) {
        issue_pv(j);
        if (alive && j + 2 < n_tiles) issue_s(j + 2);
      }
    }
  } else {
    // -------------------------------------------------------------- softmax warps --
    const int quad = warp & 3;                                      // TMEM lane quadrant this warp may read
    const int row = quad * 32 + lane;                               // query row of the tile = TMEM lane
    const int qi = q0 + row;
    const int reach = p.pos0 + qi;                                  // last key this query attends
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    // running maximum kept in the exponent's own unit: scores are multiplied by scale * log2(e) once and the
    // probabilities are 2^(s - m), one FFMA and one ex2.approx each
    const float sc = p.scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;
    float o[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) o[d] = 0.f;
    bool alive = true;
    auto fold = [&](int j, float alpha) {                           // o = o * alpha + O_j
      const int s = j & 1;
      // .aligned TMEM loads follow: the whole warp leaves together or not at all
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&o_full[s]), (uint32_t)(j >> 1) & 1u, abort_flag, p.status, 0x47))) { alive = false; return; }
      tcgen05_fence_after();
      float f[HD];
      tmem_ld64(lane_base + (uint32_t)(O_COL + s * HD), f);
#pragma unroll
      for (int i = 0; i < HD; ++i) o[i] = o[i] * alpha + f[i];
    };
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int s = j & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_full[s]), (uint32_t)(j >> 1) & 1u, abort_flag, p.status, 0x48))) { alive = false; break; }
      tcgen05_fence_after();
      const int key0 = j * BKV;
      float f[BKV];
      tmem_ld64(lane_base + (uint32_t)(s * BKV), f);
      // four interleaved chains for the maximum and for the sum: a single one is 64 dependent operations.
      // The maximum is taken over the raw scores (sc > 0) and scaled once; 2^(s sc - m) is one FFMA + ex2.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (key0 + BKV - 1 > reach) {                                 // the diagonal crosses this tile: causal mask
#pragma unroll
        for (int i = 0; i < BKV; ++i)
          if (key0 + i > reach) f[i] = -INFINITY;
      }
#pragma unroll
      for (int i = 0; i < BKV; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], f[i]);
      const float m_new = fmaxf(m_run, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc);   // finite: key 0 is attended by every row
      const float alpha = ex2(m_run - m_new);
      const float neg_m = -m_new;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < BKV; ++i) {
        f[i] = ex2(fmaf(f[i], sc, neg_m));
        l4[i & 3] += f[i];
      }
      l_run = l_run * alpha + ((l4[0] + l4[1]) + (l4[2] + l4[3]));
      m_run = m_new;
      // probabilities rounded to bf16 into the swizzled A tile of the second product
      uint8_t *prow = p_s + s * P_BYTES + row * 128;
#pragma unroll
      for (int ch = 0; ch < BKV / 8; ++ch) {                        // 8 keys = 16 bytes per chunk
        uint4 v;
        __nv_bfloat162 t;
        t = __floats2bfloat162_rn(f[ch * 8 + 0], f[ch * 8 + 1]); v.x = *(uint32_t *)&t;
        t = __floats2bfloat162_rn(f[ch * 8 + 2], f[ch * 8 + 3]); v.y = *(uint32_t *)&t;
        t = __floats2bfloat162_rn(f[ch * 8 + 4], f[ch * 8 + 5]); v.z = *(uint32_t *)&t;
        t = __floats2bfloat162_rn(f[ch * 8 + 6], f[ch * 8 + 7]); v.w = *(uint32_t *)&t;
        *reinterpret_cast<uint4 *>(prow + ((ch ^ (row & 7)) << 4)) = v;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P visible to the tensor core's reads
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[s]));
      if (j > 0) fold(j - 1, alpha_prev);
      alpha_prev = alpha;
    }
    if (alive && n_tiles > 0) fold(n_tiles - 1, alpha_prev);
    if (alive && qi < p.t) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16 *dst = p.out + ((size_t)b * p.t + qi) * ((size_t)p.n_heads * HD) + (size_t)head * HD;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        uint4 v;
        __nv_bfloat162 t;
        t = __floats2bfloat162_rn(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv); v.x = *(uint32_t *)&t;
        t = __floats2bfloat162_rn(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv); v.y = *(uint32_t *)&t;
        t = __floats2bfloat162_rn(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv); v.z = *(uint32_t *)&t;
        t = __floats2bfloat162_rn(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv); v.w = *(uint32_t *)&t;
        *reinterpret_cast<uint4 *>(dst + c * 8) = v;
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace

int32_t ugb_prefill_attention_tc(ugb_device *dev, const __nv_bfloat16 *q, const __nv_bfloat16 *kcache,
                                 const __nv_bfloat16 *vcache, __nv_bfloat16 *out, int batch, int t, int pos0,
                                 int n_heads, int n_kv, int t_max, float scale) {
  if (batch == 0 || t == 0) return UGB_OK;
  static bool attr_set[64] = {};
  if (!attr_set[dev->ordinal & 63]) {
    UGB_CUDA(dev, cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    attr_set[dev->ordinal & 63] = true;
  }
  CUtensorMap tmQ, tmK, tmV;
  int32_t rc;
  {   // q [batch, t, n_heads, 64]: dims {d, head, position, sequence}, a box is 128 positions of one head
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)n_heads, (uint64_t)t, (uint64_t)batch};
    const uint64_t strides[3] = {(uint64_t)HD, (uint64_t)n_heads * HD, (uint64_t)t * n_heads * HD};
    const uint32_t box[4] = {(uint32_t)HD, 1, (uint32_t)BQ, 1};
    if ((rc = ugb_tc_encode_bf16(dev, &tmQ, q, 4, dims, strides, box))) return rc;
  }
  {   // caches [batch, n_kv, t_max, 64]: dims {d, position, sequence x kv head}
    const uint64_t dims[3] = {(uint64_t)HD, (uint64_t)t_max, (uint64_t)batch * n_kv};
    const uint64_t strides[2] = {(uint64_t)HD, (uint64_t)t_max * HD};
    const uint32_t box[3] = {(uint32_t)HD, (uint32_t)BKV, 1};
    if ((rc = ugb_tc_encode_bf16(dev, &tmK, kcache, 3, dims, strides, box))) return rc;
    if ((rc = ugb_tc_encode_bf16(dev, &tmV, vcache, 3, dims, strides, box))) return rc;
  }
  Params p;
  p.t = t; p.pos0 = pos0; p.n_heads = n_heads; p.n_kv = n_kv; p.scale = scale; p.out = out; p.status = dev->status_dev;
  dim3 grid((unsigned)((t + BQ - 1) / BQ), (unsigned)n_heads, (unsigned)batch);
  prefill_attention_tc_kernel<<<grid, THREADS, SMEM_BYTES, dev->stream>>>(tmQ, tmK, tmV, p);
  return ugb_after_launch(dev, "prefill_attention_tc_kernel");
}
