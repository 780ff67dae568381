// Persistent decode step: all layers of one Llama decode step (one new token per sequence,
// ug-llama/src/model.rs:203-269,365-373 with seq_len == 1) in ONE kernel launch.
//
// Why: as separate kernels the step is a chain of 7 dependent launches per layer, and every
// weight-streaming projection pays its own start-up (launch, tensor-map fetch, TMEM allocation, first
// bytes from HBM) before it streams a few microseconds' worth of weights.  Here the grid stays resident
// (one CTA per SM), the phases of a layer are separated by grid-wide barriers, and the weight stream
// never stops: a dedicated producer thread per CTA runs through the weight tiles of ALL phases and
// layers in order, limited only by its shared-memory ring, so the weights of the next projection arrive
// while the current phase computes and while the barrier is pending.
//
// CTA = 384 threads:
//   warp 0      weight producer: cp.async.bulk.tensor (TMA) of [bn x 64] weight tiles into a ring of 16 KiB stages
//   warp 1      MMA issuer: tcgen05.mma (M = 64, N = bn, K = 16) into two TMEM accumulator stages; owns TMEM
//   warp 2      activation producer: TMA of [64 rows x 64] activation tiles, after the barrier that completes them
//   warps 4..11 everything else: GEMM epilogues (tcgen05.ld -> fp32 split-K partials / silu(gate) * up),
//               residual add + RMSNorm rows, rope + KV append + grouped-query flash-decode attention, and the
//               grid barriers
// Phases of a layer (a grid barrier after each):
//   rows      x += sum of the previous projection's partials;  xn = bf16(rmsnorm(x) * gain)   (first layer: x = embedding)
//   GEMM      q|k|v partials = xn . Wqkv^T
//   attention per (sequence, KV head): sum partials, rope(q, k), append k / v to the cache, flash-decode over
//             the cache; the 16-key sub-tiles of all (sequence, KV head) pairs are dealt to the CTAs in equal
//             contiguous shares, pairs cut by a share boundary are merged by their last finisher
//   GEMM      o partials = att . Wo^T
//   rows      x += o partials;  xn = rmsnorm(x)
//   GEMM      h = silu(gate) * up of xn . Wgu^T (gate / up rows interleaved)
//   GEMM      down partials = h . Wdown^T
// and after the last layer the final norm; the tied lm_head and the greedy choice stay separate kernels.
//
// Every wait (mbarrier, grid barrier, hand-over between roles) is bounded by the device's wait limit; a wait
// that gives up raises the status word, sets a grid-wide abort flag that every other wait polls, and all
// roles leave their loops, let copies in flight land, free TMEM and return.
#include <cuda.h>
#include <cuda_bf16.h>

#include "decode_kernels.cuh"
#include "decode_step.cuh"
#include "gemm_tcgen05.cuh"
#include "tc_ptx.cuh"

namespace {

using namespace ugb_tc;
using ugb_decode::cp_async16;
using ugb_decode::cp_async_commit;
using ugb_decode::cp_async_wait;
using ugb_decode::mma_bf16_16x8x16;
using ugb_decode::pack_bf16;
using ugb_decode::warp_sum;

constexpr int BK = 64;
constexpr int NB = 7;                       // weight ring stages
constexpr int NA = 12;                      // activation ring stages
constexpr int B_STAGE = 16384;              // up to 128 weight rows x 64 k bf16
constexpr int A_STAGE = 8192;               // 64 activation rows x 64 k bf16
constexpr int ACC_STRIDE = 128;             // TMEM columns between the two accumulator stages
constexpr int TMEM_COLS = 256;
constexpr int THREADS = 384;
constexpr int EPI_WARP0 = 4;                // warps 4..11: TMEM lane quadrant = warp & 3
constexpr int EPI_WARPS = 8;
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int ATT_ST = 3;                   // 16-key sub-tiles per warp in the ring (8 warps x 3 x 4 KiB = the activation ring)
constexpr int ATT_PF = 4;                   // L2 prefetch distance, in sub-tiles of the same warp
constexpr int ATT_SUB = 16, ATT_HD = 64, ATT_GROUP = 8;
constexpr int ATT_SUB_BYTES = ATT_SUB * ATT_HD * 2;
constexpr int MAX_PART = 9;                 // split-K partials a row phase sums at most
constexpr int SYNCS_PER_LAYER = 7;

static_assert(NA * A_STAGE == EPI_WARPS * ATT_ST * 2 * ATT_SUB_BYTES, "the attention ring aliases the activation ring");

struct Smem {
  uint8_t b_ring[NB][B_STAGE];
  uint8_t a_ring[NA][A_STAGE];              // during the attention phase: [warp][stage][K | V][2 KiB]
  float merge_o[EPI_WARPS][ATT_GROUP][ATT_HD];
  float merge_ml[EPI_WARPS][ATT_GROUP][2];
  float red[8];
  uint64_t full_b[NB], empty_b[NB], full_a[NA], empty_a[NA], acc_full[2], acc_empty[2];
  uint32_t tmem_slot;
  int abort_flag;
  int sync_count;                           // grid barriers this CTA has passed (written by the barrier thread)
  int is_last;
};

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_cta_shared(const int *p) {
  int v;
  asm volatile("ld.acquire.cta.shared.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta_shared(int *p, int v) {
  asm volatile("st.release.cta.shared.s32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void l2_prefetch(const void *p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// What every bounded wait of this kernel shares: the CTA's abort flag, the grid's abort word, the status word.
struct Waiter {
  volatile int *abort_s;
  unsigned *abort_g;
  ugb_status_word *status;
  __device__ __forceinline__ bool aborted() const {
    if (*abort_s) return true;
    if (*reinterpret_cast<volatile unsigned *>(abort_g)) { *abort_s = 1; return true; }
    return false;
  }
  __device__ __forceinline__ void give_up(unsigned site) const {
    *abort_s = 1;
    atomicExch(abort_g, 1u);
    if (atomicCAS(&status->code, 0u, (unsigned)UGB_ERR_TIMEOUT) == 0u) status->detail = site;
  }
  __device__ __forceinline__ unsigned long long limit_ns() const {
    return 1000ull * *reinterpret_cast<volatile unsigned int *>(&status->wait_limit_us);
  }
  int backoff_ns = 0;
  __device__ __forceinline__ bool mbar(uint32_t bar, uint32_t parity, unsigned site) const {
    if (mbar_try(bar, parity)) return true;
    const unsigned long long t0 = globaltimer();
    for (unsigned it = 1;; ++it) {
      if (mbar_try(bar, parity)) return true;
      if (backoff_ns) __nanosleep(backoff_ns);
      if ((it & 255u) == 0) {
        if (aborted()) return false;
        if (globaltimer() - t0 > limit_ns()) { give_up(site); return false; }
      }
    }
  }
};

struct Item { int tile, kb0, kb1; };
__device__ __forceinline__ Item item_of(const ugb_step_gemm &g, int item) {
  Item it;
  const int sp = item / g.tiles;
  it.tile = item - sp * g.tiles;
  it.kb0 = sp * g.kb_per;
  it.kb1 = min(g.kb, it.kb0 + g.kb_per);
  return it;
}

// ---------------------------------------------------------------------------------------------------------
// rows phase: x[r] (+)= sum of partials (or the embedding row), xn[r] = bf16(x / sqrt(mean(x^2) + eps) * gain)
// (Layer::fwd's residual add + RmsNorm::fwd, model.rs:65-78,259-269).  256 threads per row.
__device__ void rows_phase(const ugb_step_params &p, Smem &s, int et, int cta, int grid, const float *part, int n_part,
                           size_t part_stride, const float *__restrict__ gain, bool from_embed) {
  const int H = p.hidden, nvec = H >> 2;
  for (int r = cta; r < p.batch; r += grid) {
    float4 *xr = reinterpret_cast<float4 *>(p.x + (size_t)r * H);
    const uint2 *er = nullptr;
    if (from_embed) {
      const int id = p.tok[r];
      if (id < 0 || id >= p.vocab) {        // as embed_gather: report, leave the row alone
        if (et == 0 && atomicCAS(&p.status->code, 0u, (unsigned)UGB_ERR_INVALID) == 0u) p.status->detail = r;
        continue;
      }
      er = reinterpret_cast<const uint2 *>(p.embed + (size_t)id * H);
    }
    float ss = 0.f;
    // The row's first 1024 float4 (all of them when hidden <= 4096) are fetched with every load -- x and all partials
    // -- in flight before the first addition, and stay in registers for the second pass.
    constexpr int KEEP = 4;
    float4 keep[KEEP];
    if (from_embed) {
#pragma unroll
      for (int i = 0; i < KEEP; ++i) {
        const int c = et + i * EPI_THREADS;
        keep[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < nvec) {
          const uint2 e = __ldg(er + c);
          const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&e.x));
          const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&e.y));
          keep[i] = make_float4(lo.x, lo.y, hi.x, hi.y);
        }
      }
    } else {
      float4 q[2][MAX_PART];
#pragma unroll
      for (int h = 0; h < KEEP; h += 2) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int c = et + (h + i) * EPI_THREADS;
          keep[h + i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (c < nvec) keep[h + i] = __ldcg(xr + c);
#pragma unroll
          for (int sp = 0; sp < MAX_PART; ++sp)
            q[i][sp] = (c < nvec && sp < n_part) ? __ldcg(reinterpret_cast<const float4 *>(part + sp * part_stride + (size_t)r * H) + c)
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int sp = 0; sp < MAX_PART; ++sp)
            if (sp < n_part) { keep[h + i].x += q[i][sp].x; keep[h + i].y += q[i][sp].y; keep[h + i].z += q[i][sp].z; keep[h + i].w += q[i][sp].w; }
      }
    }
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
      const int c = et + i * EPI_THREADS;
      if (c < nvec) {
        if (from_embed || n_part > 0) xr[c] = keep[i];
        ss += (keep[i].x * keep[i].x + keep[i].y * keep[i].y) + (keep[i].z * keep[i].z + keep[i].w * keep[i].w);
      }
    }
    for (int c = et + KEEP * EPI_THREADS; c < nvec; c += EPI_THREADS) {      // hidden > 4096: the rest of the row, one float4 at a time
      float4 v;
      if (from_embed) {
        const uint2 e = __ldg(er + c);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&e.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&e.y));
        v = make_float4(lo.x, lo.y, hi.x, hi.y);
      } else {
        v = __ldcg(xr + c);
        for (int sp = 0; sp < n_part; ++sp) {
          const float4 qv = __ldcg(reinterpret_cast<const float4 *>(part + sp * part_stride + (size_t)r * H) + c);
          v.x += qv.x; v.y += qv.y; v.z += qv.z; v.w += qv.w;
        }
      }
      if (from_embed || n_part > 0) xr[c] = v;
      ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
    ss = warp_sum(ss);
    epi_bar();                               // s.red is free again (previous row)
    if ((et & 31) == 0) s.red[et >> 5] = ss;
    epi_bar();
    const float tot = ((s.red[0] + s.red[1]) + (s.red[2] + s.red[3])) + ((s.red[4] + s.red[5]) + (s.red[6] + s.red[7]));
    const float m = sqrtf(tot * p.inv_d + p.eps);
    uint2 *out = reinterpret_cast<uint2 *>(p.xn + (size_t)r * H);
    auto emit = [&](int c, const float4 &v) {
      const float4 gw = __ldg(reinterpret_cast<const float4 *>(gain) + c);
      out[c] = make_uint2(pack_bf16(v.x / m * gw.x, v.y / m * gw.y), pack_bf16(v.z / m * gw.z, v.w / m * gw.w));
    };
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
      const int c = et + i * EPI_THREADS;
      if (c < nvec) emit(c, keep[i]);
    }
    for (int c = et + KEEP * EPI_THREADS; c < nvec; c += EPI_THREADS) emit(c, xr[c]);
  }
}

// ---------------------------------------------------------------------------------------------------------
// GEMM epilogue of one phase: drains this CTA's accumulators.  64 accumulator rows: rows 16q .. 16q + 15 sit on
// lanes 0 .. 15 of TMEM lane quadrant q; warps q and q + 4 share quadrant q and take alternate 32-column chunks.
__device__ bool gemm_epilogue(const ugb_step_params &p, Smem &s, const Waiter &w, const ugb_step_gemm &g, int phase,
                              uint32_t tmem_base, int ew, int lane, int cta, int grid, int &acc, uint32_t &acc_phase) {
  for (int item = cta; item < g.items; item += grid) {
    const Item it = item_of(g, item);
    const int sp = item / g.tiles, n0 = it.tile * g.bn;
    if (!w.mbar(smem_u32(&s.acc_full[acc]), acc_phase, 0x104u)) return false;
    tcgen05_fence_after();
    const int quad = ew & 3;
    const int row = quad * 16 + lane;
    const bool live = lane < 16 && row < p.batch;
    for (int c = ew >> 2; c * 32 < g.bn; c += 2) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * ACC_STRIDE + c * 32), v);
      tmem_ld_wait();
      if (!live) continue;
      const int col0 = n0 + c * 32;
      if (phase != UGB_STEP_GATE_UP) {
        float *crow = p.part + (size_t)sp * p.batch * g.n + (size_t)row * g.n + col0;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (c * 32 + q * 4 < g.bn && col0 + q * 4 < g.n)
            *reinterpret_cast<uint4 *>(crow + q * 4) = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      } else {                               // columns are (gate, up) pairs: h[row][col / 2] = silu(gate) * up
        __nv_bfloat16 *crow = p.h + (size_t)row * (g.n / 2) + col0 / 2;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (c * 32 + q * 16 < g.bn && col0 + q * 16 < g.n) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float g0 = __uint_as_float(v[q * 16 + e * 4 + 0]), u0 = __uint_as_float(v[q * 16 + e * 4 + 1]);
              const float g1 = __uint_as_float(v[q * 16 + e * 4 + 2]), u1 = __uint_as_float(v[q * 16 + e * 4 + 3]);
              o[e] = pack_bf16(__fdividef(g0, __expf(-g0) + 1.0f) * u0, __fdividef(g1, __expf(-g1) + 1.0f) * u1);
            }
            *reinterpret_cast<uint4 *>(crow + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    }
    tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&s.acc_empty[acc]));
    if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
  }
  return true;
}

// ---------------------------------------------------------------------------------------------------------
// attention phase (model.rs:203-245 between the projections, for one query position per sequence): the CTA's
// share [f_lo, f_hi) of the flattened (pair, 16-key sub-tile) list; warp w of the eight takes sub-tiles
// f_lo + w, f_lo + w + 8, ...  with a private cp.async ring (plus L2 prefetches further ahead) and a private
// online-softmax state.
__device__ void attention_phase(const ugb_step_params &p, Smem &s, int layer, int T, int ew, int lane, int et, int cta,
                                int grid) {
  const int n_kv = p.n_kv, n_heads = p.n_heads, group = p.group, t_max = p.t_max;
  const int n_sub = (T + ATT_SUB - 1) / ATT_SUB, n_pairs = p.batch * n_kv;
  const long long S = (long long)n_pairs * n_sub;
  const long long per = (S + grid - 1) / grid;
  const long long f_lo = (long long)cta * per, f_hi = min(S, f_lo + per);
  if (f_lo >= f_hi) return;                                   // CTA-uniform: nothing dealt to this CTA
  __nv_bfloat16 *kcache = p.layer[layer].kcache, *vcache = p.layer[layer].vcache;
  if (p.tune & 8) {   // measurement aid: read this CTA's share of K and V with plain 128-bit loads, nothing else
    float sink = 0.f;
    for (int which = 0; which < 2; ++which) {
      const int pair0 = (int)(f_lo / n_sub), sub0 = (int)(f_lo - (long long)pair0 * n_sub);
      const uint4 *src = reinterpret_cast<const uint4 *>((which ? vcache : kcache) + ((size_t)pair0 * t_max + (size_t)sub0 * ATT_SUB) * ATT_HD);
      const long long n16 = (f_hi - f_lo) * (ATT_SUB_BYTES / 16);     // (ignores the gaps between pairs: a bandwidth probe)
      for (long long i = et; i < n16; i += 8 * EPI_THREADS) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = i + u * EPI_THREADS < n16 ? __ldcs(src + i + u * EPI_THREADS) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 8; ++u) sink += __uint_as_float(v[u].x ^ v[u].w);
      }
    }
    if (sink == 123.456f) p.att_pml[0] = sink;
    return;
  }
  uint8_t (*ring)[ATT_ST][2][ATT_SUB_BYTES] = reinterpret_cast<uint8_t (*)[ATT_ST][2][ATT_SUB_BYTES]>(&s.a_ring[0][0]);   // [warp][stage][K | V]
  const int g = lane >> 2, t = lane & 3;
  const int half = ATT_HD / 2, pos = T - 1, sub_pos = pos / ATT_SUB;
  const int n_part = p.g[UGB_STEP_QKV].splits;
  const size_t part_stride = (size_t)p.batch * p.qkv_dim;
  const float scale = p.scale;

  auto sum4 = [&](const float *row, int col) {                // all partials requested before the first is used
    float4 q[8];
#pragma unroll
    for (int sp = 0; sp < 8; ++sp)
      q[sp] = sp < n_part ? __ldcg(reinterpret_cast<const float4 *>(row + sp * part_stride + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int sp = 0; sp < 8; ++sp)
      if (sp < n_part) { a.x += q[sp].x; a.y += q[sp].y; a.z += q[sp].z; a.w += q[sp].w; }
    return a;
  };
  // K / V rows of the new position (rope on k: products and sums rounded separately, cpu_ops.rs:73-78), written by
  // the warp that is about to fetch the sub-tile holding them.
  auto append_kv = [&](int pair) {
    const int b = pair / n_kv, kvh = pair - b * n_kv;
    const float *row = p.part + (size_t)b * p.qkv_dim;
    const int kcol = (n_heads + kvh) * ATT_HD, vcol = (n_heads + n_kv + kvh) * ATT_HD;
    __nv_bfloat16 *kd = kcache + ((size_t)pair * t_max + pos) * ATT_HD;
    __nv_bfloat16 *vd = vcache + ((size_t)pair * t_max + pos) * ATT_HD;
    if (lane < 8) {
      const int i = lane * 4;
      const float4 c = *reinterpret_cast<const float4 *>(p.cos_ + (size_t)pos * half + i);
      const float4 sn = *reinterpret_cast<const float4 *>(p.sin_ + (size_t)pos * half + i);
      if (p.interleaved) {
        const float4 u = sum4(row, kcol + 2 * i), w = sum4(row, kcol + 2 * i + 4);
        uint4 o;
        o.x = pack_bf16(__fsub_rn(__fmul_rn(u.x, c.x), __fmul_rn(u.y, sn.x)), __fadd_rn(__fmul_rn(u.x, sn.x), __fmul_rn(u.y, c.x)));
        o.y = pack_bf16(__fsub_rn(__fmul_rn(u.z, c.y), __fmul_rn(u.w, sn.y)), __fadd_rn(__fmul_rn(u.z, sn.y), __fmul_rn(u.w, c.y)));
        o.z = pack_bf16(__fsub_rn(__fmul_rn(w.x, c.z), __fmul_rn(w.y, sn.z)), __fadd_rn(__fmul_rn(w.x, sn.z), __fmul_rn(w.y, c.z)));
        o.w = pack_bf16(__fsub_rn(__fmul_rn(w.z, c.w), __fmul_rn(w.w, sn.w)), __fadd_rn(__fmul_rn(w.z, sn.w), __fmul_rn(w.w, c.w)));
        *reinterpret_cast<uint4 *>(kd + 2 * i) = o;
      } else {
        const float4 x1 = sum4(row, kcol + i), x2 = sum4(row, kcol + i + half);
        uint2 lo, hi;
        lo.x = pack_bf16(__fsub_rn(__fmul_rn(x1.x, c.x), __fmul_rn(x2.x, sn.x)), __fsub_rn(__fmul_rn(x1.y, c.y), __fmul_rn(x2.y, sn.y)));
        lo.y = pack_bf16(__fsub_rn(__fmul_rn(x1.z, c.z), __fmul_rn(x2.z, sn.z)), __fsub_rn(__fmul_rn(x1.w, c.w), __fmul_rn(x2.w, sn.w)));
        hi.x = pack_bf16(__fadd_rn(__fmul_rn(x1.x, sn.x), __fmul_rn(x2.x, c.x)), __fadd_rn(__fmul_rn(x1.y, sn.y), __fmul_rn(x2.y, c.y)));
        hi.y = pack_bf16(__fadd_rn(__fmul_rn(x1.z, sn.z), __fmul_rn(x2.z, c.z)), __fadd_rn(__fmul_rn(x1.w, sn.w), __fmul_rn(x2.w, c.w)));
        *reinterpret_cast<uint2 *>(kd + i) = lo;
        *reinterpret_cast<uint2 *>(kd + i + half) = hi;
      }
    } else if (lane < 24) {
      const int i = (lane - 8) * 4;
      const float4 x = sum4(row, vcol + i);
      *reinterpret_cast<uint2 *>(vd + i) = make_uint2(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w));
    }
    __threadfence();                                          // in L2 before this warp's cp.async fetches the row
    __syncwarp();
  };
  auto issue = [&](long long f, int stage) {
    const int pair = (int)(f / n_sub), sub = (int)(f - (long long)pair * n_sub);
    if (sub == sub_pos) append_kv(pair);
    {   // the sub-tile this warp will fetch ATT_PF iterations from now: on its way from HBM to L2 already
      const long long fp = f + (long long)ATT_PF * EPI_WARPS;
      if (fp < f_hi && lane < 2 && !(p.tune & 2)) {
        const int pp = (int)(fp / n_sub), sp2 = (int)(fp - (long long)pp * n_sub);
        const __nv_bfloat16 *base = lane == 0 ? kcache : vcache;
        l2_prefetch(base + ((size_t)pp * t_max + (size_t)sp2 * ATT_SUB) * ATT_HD, ATT_SUB_BYTES);
      }
    }
    const uint32_t ks = smem_u32(&ring[ew][stage][0][0]), vs = smem_u32(&ring[ew][stage][1][0]);
    const char *kg = reinterpret_cast<const char *>(kcache + ((size_t)pair * t_max + (size_t)sub * ATT_SUB) * ATT_HD);
    const char *vg = reinterpret_cast<const char *>(vcache + ((size_t)pair * t_max + (size_t)sub * ATT_SUB) * ATT_HD);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = lane + 32 * i, key = c >> 3, ch = c & 7;
      const uint32_t so = key * 128 + ((ch ^ (key & 7)) << 4);
      cp_async16(ks + so, kg + c * 16);
      cp_async16(vs + so, vg + c * 16);
    }
  };

  uint32_t qa[8];
  float m_run, l_run, o[8][4];
  // Q fragments of a pair: lane (g, t) holds dims 16t .. 16t + 15 of query head g of the group, rotated.
  auto begin_pair = [&](int pair) {
    m_run = -INFINITY;
    l_run = 0.f;
#pragma unroll
    for (int d = 0; d < 8; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    const int b = pair / n_kv, kvh = pair - b * n_kv;
    const float *row = p.part + (size_t)b * p.qkv_dim;
    float y[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) y[e] = 0.f;
    if (g < group) {
      const int qcol = (kvh * group + g) * ATT_HD, d0 = 16 * t;
      float xa[16];
#pragma unroll
      for (int v4 = 0; v4 < 4; ++v4) {
        const float4 a = sum4(row, qcol + d0 + 4 * v4);
        xa[4 * v4] = a.x; xa[4 * v4 + 1] = a.y; xa[4 * v4 + 2] = a.z; xa[4 * v4 + 3] = a.w;
      }
      if (p.interleaved) {
        float cs[8], sn[8];
#pragma unroll
        for (int v4 = 0; v4 < 2; ++v4) {
          const float4 c4 = *reinterpret_cast<const float4 *>(p.cos_ + (size_t)pos * half + 8 * t + 4 * v4);
          const float4 s4 = *reinterpret_cast<const float4 *>(p.sin_ + (size_t)pos * half + 8 * t + 4 * v4);
          cs[4 * v4] = c4.x; cs[4 * v4 + 1] = c4.y; cs[4 * v4 + 2] = c4.z; cs[4 * v4 + 3] = c4.w;
          sn[4 * v4] = s4.x; sn[4 * v4 + 1] = s4.y; sn[4 * v4 + 2] = s4.z; sn[4 * v4 + 3] = s4.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          y[2 * i] = __fsub_rn(__fmul_rn(xa[2 * i], cs[i]), __fmul_rn(xa[2 * i + 1], sn[i]));
          y[2 * i + 1] = __fadd_rn(__fmul_rn(xa[2 * i], sn[i]), __fmul_rn(xa[2 * i + 1], cs[i]));
        }
      } else {
        const int i0 = d0 & (half - 1);
        float xb[16], cs[16], sn[16];
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const float4 a = sum4(row, qcol + (d0 ^ half) + 4 * v4);
          const float4 c4 = *reinterpret_cast<const float4 *>(p.cos_ + (size_t)pos * half + i0 + 4 * v4);
          const float4 s4 = *reinterpret_cast<const float4 *>(p.sin_ + (size_t)pos * half + i0 + 4 * v4);
          xb[4 * v4] = a.x; xb[4 * v4 + 1] = a.y; xb[4 * v4 + 2] = a.z; xb[4 * v4 + 3] = a.w;
          cs[4 * v4] = c4.x; cs[4 * v4 + 1] = c4.y; cs[4 * v4 + 2] = c4.z; cs[4 * v4 + 3] = c4.w;
          sn[4 * v4] = s4.x; sn[4 * v4 + 1] = s4.y; sn[4 * v4 + 2] = s4.z; sn[4 * v4 + 3] = s4.w;
        }
#pragma unroll
        for (int e = 0; e < 16; ++e)
          y[e] = d0 < half ? __fsub_rn(__fmul_rn(xa[e], cs[e]), __fmul_rn(xb[e], sn[e]))
                           : __fadd_rn(__fmul_rn(xb[e], sn[e]), __fmul_rn(xa[e], cs[e]));
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) qa[e] = pack_bf16(y[2 * e], y[2 * e + 1]);
  };
  // Merge of the four warps' states for `pair`, then either the output rows (the pair lies inside this CTA's
  // share) or a partial result; the last CTA to deliver a partial of the pair combines them.
  auto end_pair = [&](int pair) {
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      s.merge_o[ew][g][8 * d + 2 * t] = o[d][0];
      s.merge_o[ew][g][8 * d + 2 * t + 1] = o[d][1];
    }
    if (t == 0) { s.merge_ml[ew][g][0] = m_run; s.merge_ml[ew][g][1] = l_run; }
    epi_bar();
    const int b = pair / n_kv, kvh = pair - b * n_kv;
    const long long p0 = (long long)pair * n_sub;
    const int c_first = (int)(p0 / per), c_last = (int)((p0 + n_sub - 1) / per);
    const int n_seg = c_last - c_first + 1;
    for (int idx = et; idx < ATT_GROUP * ATT_HD; idx += EPI_THREADS) {
      const int h = idx / ATT_HD, dd = idx - h * ATT_HD;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < EPI_WARPS; ++w) mm = fmaxf(mm, s.merge_ml[w][h][0]);
      float acc = 0.f, ll = 0.f;
#pragma unroll
      for (int w = 0; w < EPI_WARPS; ++w) {
        const float f = s.merge_ml[w][h][0] == -INFINITY ? 0.f : __expf(s.merge_ml[w][h][0] - mm);
        acc += s.merge_o[w][h][dd] * f;
        ll += s.merge_ml[w][h][1] * f;
      }
      if (n_seg == 1) {
        if (h < group) p.att[((size_t)b * n_heads + kvh * group + h) * ATT_HD + dd] = __float2bfloat16_rn(acc / ll);
      } else {
        const size_t slot = (size_t)pair + cta;               // unique: pair and CTA index both grow along the list
        p.att_po[(slot * ATT_GROUP + h) * ATT_HD + dd] = acc;
        if (dd == 0) { p.att_pml[(slot * ATT_GROUP + h) * 2] = mm; p.att_pml[(slot * ATT_GROUP + h) * 2 + 1] = ll; }
      }
    }
    if (n_seg > 1) {
      __threadfence();
      epi_bar();
      if (et == 0) {
        const unsigned prev = atomicAdd(&p.att_cnt[pair], 1u);
        s.is_last = (prev == (unsigned)n_seg - 1u);
        if (s.is_last) p.att_cnt[pair] = 0u;                   // ready for the next layer
      }
      epi_bar();
      if (s.is_last) {
        __threadfence();
        for (int idx = et; idx < group * ATT_HD; idx += EPI_THREADS) {
          const int h = idx / ATT_HD, dd = idx - h * ATT_HD;
          float mm = -INFINITY;
          for (int c = c_first; c <= c_last; ++c) mm = fmaxf(mm, __ldcg(&p.att_pml[(((size_t)pair + c) * ATT_GROUP + h) * 2]));
          float acc = 0.f, ll = 0.f;
          for (int c = c_first; c <= c_last; ++c) {
            const size_t slot = (size_t)pair + c;
            const float ms = __ldcg(&p.att_pml[(slot * ATT_GROUP + h) * 2]);
            const float f = ms == -INFINITY ? 0.f : __expf(ms - mm);
            acc += __ldcg(&p.att_po[(slot * ATT_GROUP + h) * ATT_HD + dd]) * f;
            ll += __ldcg(&p.att_pml[(slot * ATT_GROUP + h) * 2 + 1]) * f;
          }
          p.att[((size_t)b * n_heads + kvh * group + h) * ATT_HD + dd] = __float2bfloat16_rn(acc / ll);
        }
      }
    }
    epi_bar();                                                 // merge buffers and is_last are free again
  };

  int cur_pair = (int)(f_lo / n_sub);
  const int last_pair = (int)((f_hi - 1) / n_sub);
#pragma unroll
  for (int st = 0; st < ATT_ST - 1; ++st) {
    const long long f = f_lo + ew + EPI_WARPS * st;
    if (f < f_hi) issue(f, st);
    cp_async_commit();
  }
  begin_pair(cur_pair);
  int stage = 0;
  for (long long f = f_lo + ew;; f += EPI_WARPS) {
    bool done = false;
    while (f >= f_hi || (int)(f / n_sub) > cur_pair) {         // this warp is through with cur_pair
      end_pair(cur_pair);
      if (++cur_pair > last_pair) { done = true; break; }
      begin_pair(cur_pair);
    }
    if (done) break;
    {
      const long long nxt = f + (ATT_ST - 1) * EPI_WARPS;
      if (nxt < f_hi) issue(nxt, (stage + ATT_ST - 1) % ATT_ST);
      cp_async_commit();
    }
    cp_async_wait<ATT_ST - 1>();
    __syncwarp();
    const int sub = (int)(f - (long long)cur_pair * n_sub);
    if (p.tune & 1) { __syncwarp(); stage = (stage + 1) % ATT_ST; continue; }
    const uint8_t *ks = &ring[ew][stage][0][0];
    const uint32_t vs = smem_u32(&ring[ew][stage][1][0]);
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
    const float m_new = fmaxf(m_run, mx);                     // finite: key0 < T for every sub-tile of the list
    const float alpha = __expf(m_run - m_new);
    float pr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) pr[e] = __expf(sv[e] - m_new);
    l_run = l_run * alpha + ((pr[0] + pr[1]) + (pr[2] + pr[3]));
    m_run = m_new;
#pragma unroll
    for (int d = 0; d < 8; ++d) { o[d][0] *= alpha; o[d][1] *= alpha; }
    const uint32_t pa0 = pack_bf16(pr[0], pr[1]), pa2 = pack_bf16(pr[2], pr[3]);
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
    stage = (stage + 1) % ATT_ST;
  }
  cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 1) decode_step_kernel(const __grid_constant__ ugb_step_params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem &s = *reinterpret_cast<Smem *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, grid = gridDim.x;
  const Waiter w{&s.abort_flag, p.sync + 2, p.status, (p.tune & 4) ? 200 : 0};
  const int L = p.layers;
  const CUtensorMap *act_maps = p.maps + (size_t)L * 4;        // xn, att, h

  if (threadIdx.x == 0) {
    for (int i = 0; i < NB; ++i) { mbar_init(smem_u32(&s.full_b[i]), 1); mbar_init(smem_u32(&s.empty_b[i]), 1); }
    for (int i = 0; i < NA; ++i) { mbar_init(smem_u32(&s.full_a[i]), 1); mbar_init(smem_u32(&s.empty_a[i]), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&s.acc_full[i]), 1); mbar_init(smem_u32(&s.acc_empty[i]), EPI_WARPS); }
    s.abort_flag = 0;
    s.sync_count = 0;
    s.is_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = s.tmem_slot;
  if (threadIdx.x == 0) ugb_pdl_trigger();

  if (warp == 0) {
    // ---------------------------------------------------------------- weight producer --
    if (lane == 0) {
      int sb = 0;
      uint32_t ph_b = 0;
      bool alive = true;
      for (int l = 0; l < L && alive; ++l)
        for (int ph = 0; ph < 4 && alive; ++ph) {
          const ugb_step_gemm &g = p.g[ph];
          const CUtensorMap *map = p.maps + (size_t)l * 4 + ph;
          const uint32_t tx = (uint32_t)g.bn * (BK * 2);
          for (int item = cta; item < g.items && alive; item += grid) {
            const Item it = item_of(g, item);
            for (int kb = it.kb0; kb < it.kb1; ++kb) {
              if (!w.mbar(smem_u32(&s.empty_b[sb]), ph_b ^ 1u, 0x101u)) { alive = false; break; }
              const uint32_t bar = smem_u32(&s.full_b[sb]);
              mbar_expect_tx(bar, tx);
              tma_load_3d(smem_u32(&s.b_ring[sb][0]), map, bar, kb * BK, it.tile * g.bn, 0);
              if (++sb == NB) { sb = 0; ph_b ^= 1u; }
            }
          }
        }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      int sa = 0, sb = 0, acc = 0;
      uint32_t ph_a = 0, ph_b = 0, acc_phase = 0;
      bool alive = true;
      for (int l = 0; l < L && alive; ++l)
        for (int ph = 0; ph < 4 && alive; ++ph) {
          const ugb_step_gemm &g = p.g[ph];
          const uint32_t idesc = make_idesc(64, g.bn, false);
          for (int item = cta; item < g.items && alive; item += grid) {
            const Item it = item_of(g, item);
            if (!w.mbar(smem_u32(&s.acc_empty[acc]), acc_phase ^ 1u, 0x102u)) { alive = false; break; }
            tcgen05_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(acc * ACC_STRIDE);
            for (int kb = it.kb0; kb < it.kb1; ++kb) {
              if (!w.mbar(smem_u32(&s.full_a[sa]), ph_a, 0x103u) || !w.mbar(smem_u32(&s.full_b[sb]), ph_b, 0x105u)) { alive = false; break; }
              tcgen05_fence_after();
              const uint32_t a_addr = smem_u32(&s.a_ring[sa][0]), b_addr = smem_u32(&s.b_ring[sb][0]);
#pragma unroll
              for (int j = 0; j < BK / UMMA_K; ++j)
                umma_bf16(d_tmem, make_smem_desc(a_addr + j * (UMMA_K * 2), 0, 1024),
                          make_smem_desc(b_addr + j * (UMMA_K * 2), 0, 1024), idesc, (kb > it.kb0 || j > 0) ? 1u : 0u);
              umma_commit(smem_u32(&s.empty_a[sa]));
              umma_commit(smem_u32(&s.empty_b[sb]));
              if (++sa == NA) { sa = 0; ph_a ^= 1u; }
              if (++sb == NB) { sb = 0; ph_b ^= 1u; }
            }
            if (!alive) break;
            umma_commit(smem_u32(&s.acc_full[acc]));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
          }
        }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ activation producer --
    if (lane == 0) {
      int sa = 0;
      uint32_t ph_a = 0;
      bool alive = true;
      for (int l = 0; l < L && alive; ++l)
        for (int ph = 0; ph < 4 && alive; ++ph) {
          const ugb_step_gemm &g = p.g[ph];
          if (cta >= g.items) continue;
          // barriers that complete this phase's input: rows | qkv | attention | o | rows | gate-up | down
          const int need = SYNCS_PER_LAYER * l + (ph == UGB_STEP_QKV ? 1 : ph == UGB_STEP_O ? 3 : ph == UGB_STEP_GATE_UP ? 5 : 6);
          {
            const unsigned long long t0 = globaltimer();
            unsigned itn = 0;
            while (ld_acquire_cta_shared(&s.sync_count) < need) {
              if (p.tune & 4) __nanosleep(200);
              if ((++itn & 63u) == 0) {
                if (w.aborted()) { alive = false; break; }
                if (globaltimer() - t0 > w.limit_ns()) { w.give_up(0x106u); alive = false; break; }
              }
            }
            if (!alive) break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");      // other CTAs' generic stores -> this thread's TMA reads
          const CUtensorMap *map = act_maps + (ph == UGB_STEP_O ? 1 : ph == UGB_STEP_DOWN ? 2 : 0);
          for (int item = cta; item < g.items && alive; item += grid) {
            const Item it = item_of(g, item);
            for (int kb = it.kb0; kb < it.kb1; ++kb) {
              if (!w.mbar(smem_u32(&s.empty_a[sa]), ph_a ^ 1u, 0x107u)) { alive = false; break; }
              const uint32_t bar = smem_u32(&s.full_a[sa]);
              mbar_expect_tx(bar, (uint32_t)A_STAGE);
              tma_load_3d(smem_u32(&s.a_ring[sa][0]), map, bar, kb * BK, 0, 0);
              if (++sa == NA) { sa = 0; ph_a ^= 1u; }
            }
          }
        }
    }
  } else if (warp >= EPI_WARP0) {
    // --------------------------------------------- epilogues, row phases, attention, barriers --
    const int ew = warp - EPI_WARP0, et = threadIdx.x - EPI_WARP0 * 32;   // 0..7, 0..255
    ugb_pdl_wait();                                            // position, tokens and the barrier words are the predecessor's
    const unsigned base = *reinterpret_cast<volatile unsigned *>(p.sync + 1);
    const int T = *p.pos + 1;
    int n_sync = 0, acc = 0;
    uint32_t acc_phase = 0;
    bool alive = T >= 1 && T <= p.t_max;
    if (!alive && et == 0 && cta == 0 && atomicCAS(&p.status->code, 0u, (unsigned)UGB_ERR_INVALID) == 0u) p.status->detail = (unsigned)(T - 1);
    if (!alive && et == 0) s.abort_flag = 1;     // every CTA reads the same position: each one bails out by itself
    // Grid barrier: the CTA's epilogue threads meet, one of them announces the CTA and waits for all CTAs.
    unsigned long long *prof = (p.prof != nullptr && cta % 37 == 0 && cta / 37 < 4) ? p.prof + (size_t)(cta / 37) * UGB_STEP_PROF_SLOTS : nullptr;
    if (prof && et == 0) prof[0] = globaltimer();
    auto grid_sync = [&]() -> bool {
      epi_bar();
      ++n_sync;
      if (et == 0) {
        if (prof && 2 * n_sync < UGB_STEP_PROF_SLOTS) prof[2 * n_sync - 1] = globaltimer();
        __threadfence();
        atomicAdd(p.sync, 1u);
        const unsigned target = base + (unsigned)n_sync * (unsigned)grid;
        const unsigned long long t0 = globaltimer();
        unsigned itn = 0;
        while ((int)(ld_acquire_gpu(p.sync) - target) < 0) {
          if ((++itn & 31u) == 0) {
            if (w.aborted()) break;
            if (globaltimer() - t0 > w.limit_ns()) { w.give_up(0x108u); break; }
          }
        }
        st_release_cta_shared(&s.sync_count, n_sync);
        if (prof && 2 * n_sync < UGB_STEP_PROF_SLOTS) prof[2 * n_sync] = globaltimer();
      }
      epi_bar();
      return !*reinterpret_cast<volatile int *>(&s.abort_flag);
    };
    const size_t stride_qkv = (size_t)p.batch * p.qkv_dim, stride_h = (size_t)p.batch * p.hidden;
    for (int l = 0; l < L && alive; ++l) {
      const ugb_step_layer &ly = p.layer[l];
      rows_phase(p, s, et, cta, grid, p.part, l == 0 ? 0 : p.g[UGB_STEP_DOWN].splits, stride_h, ly.rms1, l == 0);
      if (!(alive = grid_sync())) break;
      if (!(alive = gemm_epilogue(p, s, w, p.g[UGB_STEP_QKV], UGB_STEP_QKV, tmem_base, ew, lane, cta, grid, acc, acc_phase))) break;
      if (!(alive = grid_sync())) break;
      attention_phase(p, s, l, T, ew, lane, et, cta, grid);
      if (!(alive = grid_sync())) break;
      if (!(alive = gemm_epilogue(p, s, w, p.g[UGB_STEP_O], UGB_STEP_O, tmem_base, ew, lane, cta, grid, acc, acc_phase))) break;
      if (!(alive = grid_sync())) break;
      rows_phase(p, s, et, cta, grid, p.part, p.g[UGB_STEP_O].splits, stride_h, ly.rms2, false);
      if (!(alive = grid_sync())) break;
      if (!(alive = gemm_epilogue(p, s, w, p.g[UGB_STEP_GATE_UP], UGB_STEP_GATE_UP, tmem_base, ew, lane, cta, grid, acc, acc_phase))) break;
      if (!(alive = grid_sync())) break;
      if (!(alive = gemm_epilogue(p, s, w, p.g[UGB_STEP_DOWN], UGB_STEP_DOWN, tmem_base, ew, lane, cta, grid, acc, acc_phase))) break;
      if (!(alive = grid_sync())) break;
    }
    (void)stride_qkv;
    if (alive) {
      rows_phase(p, s, et, cta, grid, p.part, p.g[UGB_STEP_DOWN].splits, stride_h, p.ln_f, false);
      // every CTA has arrived at the last barrier: the arrival count is final, the next launch starts from it
      if (cta == 0 && et == 0) *reinterpret_cast<volatile unsigned *>(p.sync + 1) = base + (unsigned)n_sync * (unsigned)grid;
    }
  }

  // ------------------------------------------------------------------------------ teardown --
  __syncwarp();
  if (*reinterpret_cast<volatile int *>(&s.abort_flag)) {
    const unsigned long long t0 = globaltimer();               // copies and MMAs in flight land before smem / TMEM go away
    while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------- host ----
size_t ugb_decode_step_smem() { return sizeof(Smem) + 1024; }

// Tile width and k split of a projection for `grid` CTAs: the choice that leaves the busiest CTA the fewest
// weight bytes (rounds x k blocks x tile rows); ties go to fewer partials, then wider tiles.
static void plan_one(ugb_step_gemm &g, int n, int k, int grid, bool may_split, int max_splits) {
  g.n = n;
  g.k = k;
  g.kb = (k + BK - 1) / BK;
  long long best = -1;
  for (int bn = 128; bn >= 64; bn -= 16) {
    const int tiles = (n + bn - 1) / bn;
    for (int sp = 1; sp <= (may_split ? max_splits : 1); ++sp) {
      if (sp > g.kb) break;
      const int kb_per = (g.kb + sp - 1) / sp;
      const int splits = (g.kb + kb_per - 1) / kb_per;
      if (splits != sp) continue;
      const int items = tiles * splits;
      const long long rounds = (items + grid - 1) / grid;
      const long long cost = rounds * kb_per * bn * 1000 + splits;      // bytes first, partials second
      if (best < 0 || cost < best) {
        best = cost;
        g.bn = bn; g.tiles = tiles; g.splits = splits; g.kb_per = kb_per; g.items = items;
      }
    }
  }
}

int ugb_decode_step_plan(ugb_step_params &p, int grid) {
  plan_one(p.g[UGB_STEP_QKV], p.qkv_dim, p.hidden, grid, true, 8);          // the attention front end sums at most 8
  plan_one(p.g[UGB_STEP_O], p.hidden, p.att_width, grid, true, MAX_PART);
  plan_one(p.g[UGB_STEP_GATE_UP], 2 * p.ffn, p.hidden, grid, false, 1);
  plan_one(p.g[UGB_STEP_DOWN], p.hidden, p.ffn, grid, true, MAX_PART);
  int most = 1;
  for (int i = 0; i < 4; ++i) most = p.g[i].splits > most ? p.g[i].splits : most;
  return most;
}

int32_t ugb_decode_step_launch(ugb_device *dev, const ugb_step_params &p, int grid, bool pdl) {
  static bool attr_set[64] = {};
  const size_t smem = ugb_decode_step_smem();
  if (!attr_set[dev->ordinal & 63]) {
    UGB_CUDA(dev, cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[dev->ordinal & 63] = true;
  }
  cudaError_t e = ugb_launch(decode_step_kernel, dim3((unsigned)grid), dim3(THREADS), smem, dev->stream, pdl, p);
  if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "launch of decode_step_kernel failed: %s", cudaGetErrorString(e));
  return ugb_after_launch(dev, "decode_step_kernel");
}
