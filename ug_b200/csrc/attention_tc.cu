// Causal grouped-query attention for a block of new positions on the 5th-generation tensor cores
// (Attention::fwd with seq_len > 1, ug-llama/src/model.rs:231-245: repeat + q.kT + scale + causal_mask +
// softmax + .v + head merge, without the [b, h, t, T] score tensor).
//
//   persistent grid of at most 2 x SMs CTAs over the (query tile, head, sequence) work items, 192 threads,
//   two CTAs per SM (80 KiB of shared memory and 256 TMEM columns each: while one CTA's softmax warps work,
//   the other's products run):
//     warp 0      TMA producer: draws the work item, loads its 128 x 64 query tile, then 64-key K and V tiles
//                               into two-deep rings
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
  int t, pos0, n_heads, n_kv, batch;
  float scale;
  __nv_bfloat16 *out;
  ugb_status_word *status;
  int *sched;   // {next item, CTAs done}: both zero between launches; null = items dealt round-robin
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

// One work item = one 128-query tile of one head of one sequence.  Items are numbered with the query
// tiles in descending order (the tiles with the most key tiles first).  A CTA's first item is its block
// index; the later ones come from a global counter (longest-first list scheduling: a CTA that drew short
// items draws more of them), or round-robin when no counter is given.  The producer draws the item and
// publishes it to the other roles through a four-deep ring of shared-memory slots (item_full barriers,
// -1 = no more work).  A CTA keeps its TMEM, barriers and tensor maps across its items, and the producer
// and MMA roles run ahead into the next item while the softmax warps finish the current one.  The K / V /
// S / P / O rings are indexed by a tile counter `g` that runs on across items (stage g & 1, phase
// (g >> 1) & 1), the query buffer by the item counter.  The producer cannot be more than two items ahead
// of the softmax warps (the query buffer of item n + 1 is released by products that need the probabilities
// of item n), so a slot is never overwritten before every role has read it.
struct Item {
  int q0, head, b, kvh, n_tiles;
};
__device__ __forceinline__ Item item_of(int idx, const Params &p, int q_tiles) {
  Item it;
  const int per_q = p.n_heads * p.batch;
  const int qt = q_tiles - 1 - idx / per_q;                         // descending query tile
  const int r = idx - (idx / per_q) * per_q;
  it.b = r / p.n_heads;
  it.head = r - it.b * p.n_heads;
  it.q0 = qt * BQ;
  it.kvh = it.head / (p.n_heads / p.n_kv);
  const int last_q = min(it.q0 + BQ, p.t) - 1;                       // last query row of the tile
  it.n_tiles = (p.pos0 + last_q + 1 + BKV - 1) / BKV;                // key tiles any of its rows attends
  return it;
}

__global__ void __launch_bounds__(THREADS, 2)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *q_s = smem, *k_s = q_s + Q_BYTES, *v_s = k_s + 2 * KV_BYTES, *p_s = v_s + 2 * KV_BYTES;
  uint64_t *bars = (uint64_t *)(p_s + 2 * P_BYTES);
  uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = bars + 3, *v_full = bars + 5, *v_empty = bars + 7;
  uint64_t *s_full = bars + 9, *p_full = bars + 11, *o_full = bars + 13, *q_empty = bars + 15, *item_full = bars + 16;
  uint32_t *tmem_slot = (uint32_t *)(bars + 20);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
  volatile int *item_slot = (volatile int *)(tmem_slot + 2);       // four entries

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (p.t + BQ - 1) / BQ;
  const int n_items = q_tiles * p.n_heads * p.batch;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 1);
    mbar_init(smem_u32(q_empty), 1);
    for (int s = 0; s < 4; ++s) mbar_init(smem_u32(&item_full[s]), 1);
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
      int g = 0;
      bool alive = true;
      int idx = blockIdx.x;
      for (int n_it = 0; alive; ++n_it) {
        // the query buffer is free once every S product of the previous item has retired
        if (!mbar_wait(smem_u32(q_empty), ((uint32_t)n_it & 1u) ^ 1u, abort_flag, p.status, 0x40)) break;
        const bool more = idx < n_items;
        item_slot[n_it & 3] = more ? idx : -1;
        mbar_arrive(smem_u32(&item_full[n_it & 3]));                // release: the slot is visible to the waiters
        if (!more) break;
        const Item it = item_of(idx, p, q_tiles);
        mbar_expect_tx(smem_u32(q_full), Q_BYTES);
        tma_load_4d(smem_u32(q_s), &tmQ, smem_u32(q_full), 0, it.head, it.q0, it.b);
        // the next item is drawn now, its latency hidden behind this item's tiles
        idx = p.sched ? (int)gridDim.x + atomicAdd(p.sched, 1) : idx + (int)gridDim.x;
        for (int j = 0; j < it.n_tiles; ++j, ++g) {
          const int s = g & 1;
          const uint32_t ph = (uint32_t)(g >> 1) & 1u;
          if (!mbar_wait(smem_u32(&k_empty[s]), ph ^ 1u, abort_flag, p.status, 0x41)) { alive = false; break; }
          mbar_expect_tx(smem_u32(&k_full[s]), KV_BYTES);
          tma_load_3d(smem_u32(k_s + s * KV_BYTES), &tmK, smem_u32(&k_full[s]), 0, j * BKV, it.b * p.n_kv + it.kvh);
          if (!mbar_wait(smem_u32(&v_empty[s]), ph ^ 1u, abort_flag, p.status, 0x42)) { alive = false; break; }
          mbar_expect_tx(smem_u32(&v_full[s]), KV_BYTES);
          tma_load_3d(smem_u32(v_s + s * KV_BYTES), &tmV, smem_u32(&v_full[s]), 0, j * BKV, it.b * p.n_kv + it.kvh);
        }
      }
      if (p.sched) {
        // every producer passes here exactly once, after its last draw: the last one re-arms the counters
        __threadfence();
        if (atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) {
          p.sched[0] = 0;
          p.sched[1] = 0;
          __threadfence();
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer --
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BQ, BKV, false);          // Q and K both K-major (rows of 64 dims)
      const uint32_t idesc_o = make_idesc(BQ, HD, true);            // P K-major, V MN-major ([key][dim] rows)
      bool alive = true;
      auto issue_s = [&](int g) {
        const int s = g & 1;
        if (!mbar_wait(smem_u32(&k_full[s]), (uint32_t)(g >> 1) & 1u, abort_flag, p.status, 0x44)) { alive = false; return; }
        tcgen05_fence_after();
        const uint32_t qa = smem_u32(q_s), kb = smem_u32(k_s + s * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / UMMA_K; ++kk)
          umma_bf16(tmem + (uint32_t)(s * BKV), make_smem_desc(qa + kk * (UMMA_K * 2), 0, 1024),
                    make_smem_desc(kb + kk * (UMMA_K * 2), 0, 1024), idesc_s, kk > 0 ? 1u : 0u);
        umma_commit(smem_u32(&k_empty[s]));                         // K stage free once the products retire
        umma_commit(smem_u32(&s_full[s]));                          // scores ready for the softmax warps
      };
      auto issue_pv = [&](int g) {
        const int s = g & 1;
        const uint32_t ph = (uint32_t)(g >> 1) & 1u;
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
      int g0 = 0;
      for (int n_it = 0; alive; ++n_it) {
        if (!mbar_wait(smem_u32(&item_full[n_it & 3]), (uint32_t)(n_it >> 2) & 1u, abort_flag, p.status, 0x49)) break;
        const int idx = item_slot[n_it & 3];
        if (idx < 0) break;
        const Item it = item_of(idx, p, q_tiles);
        if (!mbar_wait(smem_u32(q_full), (uint32_t)n_it & 1u, abort_flag, p.status, 0x43)) break;
        // S(0), S(1), then PV(j) followed by S(j + 2): the score buffer of tile j + 2 is the one the softmax
        // warps released before PV(j) could be issued
        if (alive && it.n_tiles > 0) issue_s(g0);
        if (alive && it.n_tiles > 1) issue_s(g0 + 1);
        if (alive && it.n_tiles <= 2) umma_commit(smem_u32(q_empty));          // no more products read Q
        for (int j = 0; j < it.n_tiles && alive; ++j) {
          issue_pv(g0 + j);
          if (alive && j + 2 < it.n_tiles) {
            issue_s(g0 + j + 2);
            if (alive && j + 3 == it.n_tiles) umma_commit(smem_u32(q_empty));  // that was the item's last S
          }
        }
        g0 += it.n_tiles;
      }
    }
  } else {
    // -------------------------------------------------------------- softmax warps --
    const int quad = warp & 3;                                      // TMEM lane quadrant this warp may read
    const int row = quad * 32 + lane;                               // query row of the tile = TMEM lane
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    // running maximum kept in the exponent's own unit: scores are multiplied by scale * log2(e) once and the
    // probabilities are 2^(s - m), one FFMA and one ex2.approx each
    const float sc = p.scale * 1.4426950408889634f;
    bool alive = true;
    int g0 = 0;
    for (int n_it = 0; alive; ++n_it) {
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&item_full[n_it & 3]), (uint32_t)(n_it >> 2) & 1u, abort_flag, p.status, 0x4a))) break;
      const int idx = item_slot[n_it & 3];
      if (idx < 0) break;
      const Item it = item_of(idx, p, q_tiles);
      const int qi = it.q0 + row;
      const int reach = p.pos0 + qi;                                // last key this query attends
      float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;
      float o[HD];
#pragma unroll
      for (int d = 0; d < HD; ++d) o[d] = 0.f;
      auto fold = [&](int g, float alpha) {                         // o = o * alpha + O_g
        const int s = g & 1;
        // .aligned TMEM loads follow: the whole warp leaves together or not at all
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&o_full[s]), (uint32_t)(g >> 1) & 1u, abort_flag, p.status, 0x47))) { alive = false; return; }
        tcgen05_fence_after();
        float f[HD];
        tmem_ld64(lane_base + (uint32_t)(O_COL + s * HD), f);
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] = o[i] * alpha + f[i];
      };
      for (int j = 0; j < it.n_tiles && alive; ++j) {
        const int g = g0 + j, s = g & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_full[s]), (uint32_t)(g >> 1) & 1u, abort_flag, p.status, 0x48))) { alive = false; break; }
        tcgen05_fence_after();
        const int key0 = j * BKV;
        float f[BKV];
        tmem_ld64(lane_base + (uint32_t)(s * BKV), f);
        // four interleaved chains for the maximum and for the sum: a single one is 64 dependent operations.
        // The maximum is taken over the raw scores (sc > 0) and scaled once; 2^(s sc - m) is one FFMA + ex2.
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (key0 + BKV - 1 > reach) {                               // the diagonal crosses this tile: causal mask
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
        for (int ch = 0; ch < BKV / 8; ++ch) {                      // 8 keys = 16 bytes per chunk
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
        if (j > 0) fold(g - 1, alpha_prev);
        alpha_prev = alpha;
      }
      if (alive && it.n_tiles > 0) fold(g0 + it.n_tiles - 1, alpha_prev);
      if (alive && qi < p.t) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16 *dst = p.out + ((size_t)it.b * p.t + qi) * ((size_t)p.n_heads * HD) + (size_t)it.head * HD;
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
      g0 += it.n_tiles;
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
                                 int n_heads, int n_kv, int t_max, float scale, int dynamic) {
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
  p.t = t; p.pos0 = pos0; p.n_heads = n_heads; p.n_kv = n_kv; p.batch = batch; p.scale = scale; p.out = out;
  p.status = dev->status_dev;
  p.sched = dynamic ? dev->sched_dev : nullptr;
  const long long n_items = (long long)((t + BQ - 1) / BQ) * n_heads * batch;
  const long long slots = 2LL * dev->sm_count;                     // two CTAs per SM
  dim3 grid((unsigned)(n_items < slots ? n_items : slots));
  prefill_attention_tc_kernel<<<grid, THREADS, SMEM_BYTES, dev->stream>>>(tmQ, tmK, tmV, p);
  return ugb_after_launch(dev, "prefill_attention_tc_kernel");
}

extern "C" int32_t ugb_causal_attention(ugb_device *dev, const ugb_slice *q, const ugb_slice *k, const ugb_slice *v,
                                        ugb_slice *out, size_t b, size_t t, size_t pos0, size_t n_heads,
                                        size_t n_kv, size_t t_max) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, n_kv > 0 && n_heads > 0 && n_heads % n_kv == 0, UGB_ERR_UNSUPPORTED,
              "causal_attention: %zu query heads do not divide over %zu KV heads", n_heads, n_kv);
  UGB_REQUIRE(dev, pos0 + t <= t_max, UGB_ERR_SHAPE, "causal_attention: positions %zu..%zu exceed the cache depth %zu",
              pos0, pos0 + t, t_max);
  UGB_REQUIRE(dev, b <= 65535 && n_heads <= 65535 && t_max <= (1u << 30) && b * n_kv <= (1u << 30) &&
                       ((t + BQ - 1) / BQ) * n_heads * b <= (size_t)INT32_MAX,
              UGB_ERR_SHAPE, "causal_attention: a dimension exceeds the kernel's index range");
  UGB_SLICE(dev, q, UGB_BF16, b * t * n_heads * HD);
  UGB_SLICE(dev, k, UGB_BF16, b * n_kv * t_max * HD);
  UGB_SLICE(dev, v, UGB_BF16, b * n_kv * t_max * HD);
  UGB_SLICE(dev, out, UGB_BF16, b * t * n_heads * HD);
  if (b == 0 || t == 0) return UGB_OK;
  UGB_REQUIRE(dev, (((uintptr_t)q->ptr | (uintptr_t)k->ptr | (uintptr_t)v->ptr | (uintptr_t)out->ptr) & 15) == 0,
              UGB_ERR_UNSUPPORTED, "causal_attention: buffers must be 16-byte aligned");
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  return ugb_prefill_attention_tc(dev, (const __nv_bfloat16 *)q->ptr, (const __nv_bfloat16 *)k->ptr,
                                  (const __nv_bfloat16 *)v->ptr, (__nv_bfloat16 *)out->ptr, (int)b, (int)t, (int)pos0,
                                  (int)n_heads, (int)n_kv, (int)t_max, 0.125f /* 64^-0.5, model.rs:236 */, 1);
}
