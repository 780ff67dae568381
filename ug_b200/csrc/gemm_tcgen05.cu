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
// i+1.  Products with more than 128 rows run on pairs of CTAs (template flag
// PAIR, a cluster of two): one 256 x 256 tile per pair with
// tcgen05.mma.cta_group::2 issued by the even CTA; each CTA stages its own 128
// rows of A and its own half of B's n range (32 KiB per stage, 6 stages) and
// drains its own 128 accumulator rows.  No multicast loads: every CTA fetches
// its own tiles.
//
// Every mbarrier wait is bounded by wall-clock time; a wait that gives up
// raises the device status word (UGB_ERR_TIMEOUT), flags the CTA as aborted so
// that all roles leave their loops, lets copies in flight land, frees TMEM and
// returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_tcgen05.cuh"
#include "tc_ptx.cuh"

namespace {

constexpr int BK = 64;
constexpr int ACC_STAGES = 2;
constexpr int THREADS = 192;

// Tile shapes.  BM = 128 (one accumulator row per TMEM lane) for tall products;
// BM = 64 when m <= 64 (decode: the activation tile is half the size, so the
// shared-memory ring holds more stages and more weight bytes are in flight per
// SM; the 64 accumulator rows then sit on 16 lanes of each TMEM lane quadrant).
// BN = 256 for compute-bound products, 64 / 128 for weight streaming.  The ring
// takes as many stages as fit in 220 KiB (at most 12).
// PAIR: two CTAs of a cluster work on one 256 x BN tile (tcgen05 cta_group::2): each stages its own 128
// rows of A and its own half of B's n range, so a CTA's ring stage is BM x 64 of A plus BN/2 x 64 of B.
template <int BM, int BN, bool PAIR = false> struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int BN_CTA = PAIR ? BN / 2 : BN;           // B rows (n) this CTA stages
  static constexpr int B_BYTES = BN_CTA * BK * 2;
  static constexpr int TILE_M = PAIR ? 2 * BM : BM;           // rows of C per tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int FIT = (220 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = FIT > 12 ? 12 : FIT;
  // TMEM columns between the accumulator stages (a power of two >= BN) and columns allocated
  static constexpr int ACC_STRIDE = BN <= 64 ? 64 : (BN <= 128 ? 128 : 256);
  static constexpr int TMEM_COLS = ACC_STAGES * ACC_STRIDE;   // 512, 256 or 128 (powers of two)
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 512 /*barriers*/;
  // pair_k (two CTAs split k and exchange sums): f32 [64][BN / 2] behind the barriers, where it fits
  static constexpr int PARK_BYTES = 64 * (BN / 2) * 4;
  static constexpr bool PAIR_K_OK = BM == 64 && !PAIR && BN % 32 == 0 && SMEM_BYTES + PARK_BYTES <= 227 * 1024;
};

struct Params {
  int M, N, K, batch;
  int tiles_m, tiles_n, k_blocks;
  int splits, kb_per_split;   // split-K: split s covers k blocks [s*kb_per_split, ...)
  int b_batched;          // 0: B shared by all batch steps
  int b_is_nk;            // 1: B [n,k] (k-major), 0: B [k,n] (n-major)
  int epi;                // UGB_EPI_*
  int stage_tx;           // bytes one pipeline stage receives (A box + B box)
  int n_fast;             // tile order: 1 = n-tiles vary fastest (a wave re-reads B, the smaller operand)
  int b_static;           // 1: no kernel on the stream writes B (weights): it may be fetched before ugb_pdl_wait
  int stages;             // depth of the shared-memory ring in use (2 .. Cfg::STAGES)
  int f16;                // operands and 16-bit output are IEEE f16 (0: bf16)
  unsigned long long *prof;   // measurement aid (or null): %globaltimer stamps of CTA 0, see UGB_TC_PROF_* in the header
  int pair_k;             // 1: CTAs 2c and 2c + 1 are a cluster and take the two k halves of tile c (BM = 64,
                          // UGB_EPI_SILU_MUL_BF16): rank 1 hands its sums to rank 0 through shared memory
  long long c_batch;      // output elements between batch steps
  long long c_split;      // output elements between split-K partials
  void *C;
  ugb_status_word *status;
  ugb_tc_rope_epilogue rope;
};

using namespace ugb_tc;

// Measurement aid: CTA 0 of a launch with p.prof set records when it passed the points UGB_TC_PROF_* name.
#define UGB_TC_STAMP(i)                                                      \
  do {                                                                       \
    if (p.prof != nullptr && blockIdx.x == 0 && (i) < UGB_TC_PROF_SLOTS) p.prof[(i)] = globaltimer(); \
  } while (0)

template <int BM, int BN, bool PAIR = false>
__global__ void __launch_bounds__(THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  using C_ = Cfg<BM, BN, PAIR>;
  const int STAGES = p.stages;
  constexpr int STAGE_BYTES = C_::STAGE_BYTES;
  constexpr int A_BYTES = C_::A_BYTES;
  constexpr int TMEM_COLS = C_::TMEM_COLS;
  constexpr int TILE_M = C_::TILE_M;
  constexpr int BN_CTA = C_::BN_CTA;
  // PAIR: CTAs 2c and 2c + 1 form cluster c; rank 0 (the leader) owns the full / accumulator-empty barriers
  // and issues the MMAs, each CTA loads and stores its own rows.  Tiles are dealt to clusters.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int cta0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_ctas = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern repeats every 1024 bytes
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = (uint64_t *)(smem + STAGES * STAGE_BYTES);
  uint64_t *full = bars, *empty = bars + STAGES;
  uint64_t *acc_full = bars + 2 * STAGES, *acc_empty = bars + 2 * STAGES + ACC_STAGES;
  uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 2 * ACC_STAGES);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) UGB_TC_STAMP(UGB_TC_PROF_START);
  bool pair_ready = false;           // pair_k: this epilogue thread saw its accumulator complete
  int pair_m0 = 0, pair_n0 = 0;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int tiles_per_split = tiles_per_batch * p.batch;
  const int n_tiles = tiles_per_split * p.splits;
  // tile number -> (k split, tile inside the split); with pair_k the two k halves of a tile are neighbours
  auto split_of = [&](int tile, int &sp, int &ts) {
    if (p.pair_k) { sp = tile & 1; ts = tile >> 1; }
    else { sp = tile / tiles_per_split; ts = tile - sp * tiles_per_split; }
  };
  // `bar`: this CTA's barrier, or for PAIR the leader's (a shared::cluster address)
  auto load3 = [&](uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y, int z) {
    if constexpr (PAIR) tma_load_3d_pair(dst, map, bar, x, y, z);
    else tma_load_3d(dst, map, bar, x, y, z);
  };
  auto issue_b = [&](uint32_t b_dst, uint32_t bar, int kb, int n0, int bz) {
    n0 += (int)rank * BN_CTA;                                     // PAIR: this CTA's half of the n range
    if (p.b_is_nk) {
      load3(b_dst, &tmB, bar, kb * BK, n0, bz);                   // box {64 k, BN_CTA n}
    } else {
#pragma unroll
      for (int c = 0; c < BN_CTA / 64; ++c)                       // boxes {64 n, 64 k}
        load3(b_dst + c * (64 * BK * 2), &tmB, bar, n0 + c * 64, kb * BK, bz);
    }
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      mbar_init(smem_u32(&acc_full[s]), 1);
      mbar_init(smem_u32(&acc_empty[s]), PAIR ? 8 : 4);  // one arrival per epilogue warp (of both CTAs)
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    // Preamble: the B operand of the first tile (weights in the decode step) is written by no kernel of
    // the stream, so its first stages are requested right here -- before the TMEM allocation, the CTA
    // barrier and the wait for the preceding kernel; A follows once that kernel is done.
    if (!PAIR && p.b_static) {
      const int tile = blockIdx.x;
      int sp, ts;
      split_of(tile, sp, ts);
      const int bi = ts / tiles_per_batch;
      const int r = ts - bi * tiles_per_batch;
      const int n0 = (p.n_fast ? r % p.tiles_n : r / p.tiles_m) * BN;
      const int bz = p.b_batched ? bi : 0;
      const int kb0 = sp * p.kb_per_split;
      const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
      const int pre = min(STAGES, kb1 - kb0);
      for (int i = 0; i < pre; ++i) {
        const uint32_t bar = smem_u32(&full[i]);
        mbar_expect_tx(bar, (uint32_t)p.stage_tx);
        issue_b(smem_u32(smem + i * STAGE_BYTES) + A_BYTES, bar, kb0 + i, n0, bz);
      }
    }
  }
  if (warp == 1) {
    if constexpr (PAIR) {   // collective: one warp of each CTA of the pair
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();    // both CTAs' barriers exist before either signals the other's
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) ugb_pdl_trigger();   // the next kernel on the stream may begin its preamble

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      // The B halves of the first `pre` stages were requested in the preamble above; on CTA pairs they are
      // requested here, now that the cluster barrier has made both CTAs' barriers visible -- still before the
      // wait for the preceding kernel.
      int pre = 0;
      {
        const int tile = cta0;
        int sp, ts;
        split_of(tile, sp, ts);
        const int bi = ts / tiles_per_batch;
        const int r = ts - bi * tiles_per_batch;
        const int m0 = (p.n_fast ? r / p.tiles_n : r % p.tiles_m) * TILE_M + (int)rank * BM;
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        pre = p.b_static ? min(STAGES, kb1 - kb0) : 0;
        if constexpr (PAIR) {
          const int n0 = (p.n_fast ? r % p.tiles_n : r / p.tiles_m) * BN;
          const int bz = p.b_batched ? bi : 0;
          for (int i = 0; i < pre; ++i) {
            if (rank == 0) mbar_expect_tx(smem_u32(&full[i]), (uint32_t)p.stage_tx);
            issue_b(smem_u32(smem + i * STAGE_BYTES) + A_BYTES, mapa_u32(smem_u32(&full[i]), 0), kb0 + i, n0, bz);
          }
        }
        ugb_pdl_wait();
        UGB_TC_STAMP(UGB_TC_PROF_DEP);
        for (int i = 0; i < pre; ++i)
          load3(smem_u32(smem + i * STAGE_BYTES), &tmA, PAIR ? mapa_u32(smem_u32(&full[i]), 0) : smem_u32(&full[i]),
                (kb0 + i) * BK, m0, bi);
        stage = pre % STAGES;
        phase = pre == STAGES ? 1u : 0u;
      }
      for (int tile = cta0; tile < n_tiles && alive; tile += n_ctas) {
        int sp, ts;
        split_of(tile, sp, ts);
        const int bi = ts / tiles_per_batch;
        const int r = ts - bi * tiles_per_batch;
        const int m0 = (p.n_fast ? r / p.tiles_n : r % p.tiles_m) * TILE_M + (int)rank * BM;
        const int n0 = (p.n_fast ? r % p.tiles_n : r / p.tiles_m) * BN;
        const int bz = p.b_batched ? bi : 0;
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0 + (tile == cta0 ? pre : 0); kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&empty[stage]), phase ^ 1u, abort_flag, p.status, 1)) { alive = false; break; }
          // PAIR: the leader's barrier counts the bytes of both CTAs' loads (stage_tx is their sum); the leader
          // alone posts the expectation -- bytes of the other CTA that land first are held against it
          const uint32_t bar = PAIR ? mapa_u32(smem_u32(&full[stage]), 0) : smem_u32(&full[stage]);
          if (rank == 0) mbar_expect_tx(smem_u32(&full[stage]), (uint32_t)p.stage_tx);
          const uint32_t a_dst = smem_u32(smem + stage * STAGE_BYTES);
          load3(a_dst, &tmA, bar, kb * BK, m0, bi);
          issue_b(a_dst + A_BYTES, bar, kb, n0, bz);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc(TILE_M, BN, !p.b_is_nk, p.f16 != 0);
      auto mma = [&](uint32_t d, uint64_t a_desc, uint64_t b_desc, uint32_t acc_in) {
        if constexpr (PAIR) umma_bf16_pair(d, a_desc, b_desc, idesc, acc_in);
        else umma_bf16(d, a_desc, b_desc, idesc, acc_in);
      };
      auto commit = [&](uint32_t bar) {           // PAIR: the barrier at this offset in both CTAs
        if constexpr (PAIR) umma_commit_pair(bar);
        else umma_commit(bar);
      };
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool alive = true;
      for (int tile = cta0; tile < n_tiles && alive; tile += n_ctas) {
        int sp, ts_unused;
        split_of(tile, sp, ts_unused);
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_phase ^ 1u, abort_flag, p.status, 2)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * C_::ACC_STRIDE);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&full[stage]), phase, abort_flag, p.status, 3)) { alive = false; break; }
          if (tile == cta0) UGB_TC_STAMP(UGB_TC_PROF_KBLOCK0 + (kb - kb0));
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
            mma(d_tmem, a_desc, b_desc, (kb > kb0 || j > 0) ? 1u : 0u);
          }
          commit(smem_u32(&empty[stage]));           // frees the smem stage when the MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        commit(smem_u32(&acc_full[acc]));            // accumulator complete
        if (tile == cta0) UGB_TC_STAMP(UGB_TC_PROF_LAST_MMA);
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue --
    const int quad = warp & 3;                        // TMEM lane quadrant of this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    auto release_acc = [&](int a) {                   // this warp is done with accumulator stage a
      if constexpr (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[a]), 0));
      else mbar_arrive(smem_u32(&acc_empty[a]));
    };
    for (int tile = cta0; tile < n_tiles; tile += n_ctas) {
      int sp, ts;
      split_of(tile, sp, ts);
      const int bi = ts / tiles_per_batch;
      const int r = ts - bi * tiles_per_batch;
      const int m0 = (p.n_fast ? r / p.tiles_n : r % p.tiles_m) * TILE_M + (int)rank * BM;
      const int n0 = (p.n_fast ? r % p.tiles_n : r / p.tiles_m) * BN;
      if (!mbar_wait(smem_u32(&acc_full[acc]), acc_phase, abort_flag, p.status, 4)) break;
      if (warp == 2 && lane == 0 && tile == cta0) UGB_TC_STAMP(UGB_TC_PROF_ACC_SEEN);
      tcgen05_fence_after();
      // BM = 128: accumulator row = TMEM lane.  BM = 64: rows 16q..16q+15 sit on lanes 0..15 of quadrant q.
      const bool row_lane = BM == 128 || lane < 16;
      const int row = BM == 128 ? m0 + quad * 32 + lane : m0 + quad * 16 + lane;
      const long long out_off = (long long)sp * p.c_split + (long long)bi * p.c_batch;
      if constexpr (BM == 64 && !PAIR) {
        if (p.pair_k) {
          // This half's sums of the columns the OTHER half finishes go straight into the other CTA's parking area
          // (f32 [64][BN / 2] behind the barriers: nothing else ever touches it, so no barrier is needed first);
          // remote stores are not waited for one by one the way remote loads are.  Its own columns stay in TMEM.
          if constexpr (BN % 32 == 0) {
            constexpr int GROUPS = BN / 16;
            const int half = sp;
            auto mine = [&](int g) { return (g >= GROUPS / 2 ? 1 : 0) == half; };
            const uint32_t park = mapa_u32(smem_u32(smem + STAGES * STAGE_BYTES + 512), (uint32_t)(half ^ 1)) +
                                  (uint32_t)((quad * 16 + (lane & 15)) * (BN / 2) * 4);
            const int col_base = (half ^ 1) * (BN / 2);            // first column of the peer's half
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              if (mine(2 * c) && mine(2 * c + 1)) continue;         // warp-uniform: nothing of this chunk goes to the peer
              uint32_t v[32];
              tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C_::ACC_STRIDE + c * 32), v);
              tmem_ld_wait();
              if (row_lane) {                                       // lanes 16..31 of a BM = 64 warp hold no rows
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  if (!mine(2 * c + q / 4))
                    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};"
                                 ::"r"(park + (uint32_t)((c * 32 + q * 4 - col_base) * 4)), "r"(v[q * 4]), "r"(v[q * 4 + 1]),
                                   "r"(v[q * 4 + 2]), "r"(v[q * 4 + 3])
                                 : "memory");
              }
            }
          }
          pair_ready = true;
          pair_m0 = m0; pair_n0 = n0;
          break;
        }
      }
      if constexpr (BM == 128) {
        if (p.epi == UGB_EPI_ROPE_QKV) {
          // One head (64 columns) at a time: both halves of every rotation pair (i, i + 32) -- or the 32
          // adjacent pairs of the interleaved form -- are columns of this thread's row.
          const ugb_tc_rope_epilogue &R = p.rope;
          const bool live = row < p.M;
          const int rr = live ? row : 0;
          const int seq = rr / R.t, pos = *R.pos_p + R.pos_off + (rr - seq * R.t);
          // the row's 32 cosines and 32 sines, fetched once and used for every head of the tile (they depend on the
          // position only): 16 loads per row instead of 16 per row and head
          float4 cq[8], sq[8];
          {
            const float4 *cs4 = reinterpret_cast<const float4 *>(R.cos_ + (size_t)pos * 32);
            const float4 *sn4 = reinterpret_cast<const float4 *>(R.sin_ + (size_t)pos * 32);
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) { cq[q4] = __ldg(cs4 + q4); sq[q4] = __ldg(sn4 + q4); }
          }
#pragma unroll 1
          for (int hc = 0; hc < BN / 64; ++hc) {
            const int head = (n0 >> 6) + hc;                  // warp-uniform
            if (head * 64 >= p.N) break;
            uint32_t v0[32], v1[32];
            tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C_::ACC_STRIDE + hc * 64), v0);
            tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C_::ACC_STRIDE + hc * 64 + 32), v1);
            tmem_ld_wait();
            if (!live) continue;
            __nv_bfloat16 *dst;
            if (head < R.n_heads) dst = R.q_out + ((size_t)row * R.n_heads + head) * 64;
            else if (head < R.n_heads + R.n_kv) dst = R.kcache + (((size_t)seq * R.n_kv + (head - R.n_heads)) * R.t_max + pos) * 64;
            else dst = R.vcache + (((size_t)seq * R.n_kv + (head - R.n_heads - R.n_kv)) * R.t_max + pos) * 64;
            uint32_t o[32];                                   // 64 bf16
            if (head >= R.n_heads + R.n_kv) {                 // value head: rounded as it is
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                __nv_bfloat162 a = __floats2bfloat162_rn(__uint_as_float(v0[2 * e]), __uint_as_float(v0[2 * e + 1]));
                __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v1[2 * e]), __uint_as_float(v1[2 * e + 1]));
                o[e] = *(uint32_t *)&a; o[16 + e] = *(uint32_t *)&b2;
              }
            } else if (R.interleaved) {                       // pairs (2i, 2i + 1): y0 = x0 c - x1 s, y1 = x0 s + x1 c
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) {
                const float4 c = cq[q4], sn = sq[q4];
                const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int i = q4 * 4 + e;                   // pair index 0..31: columns 2i, 2i + 1
                  const float x0 = __uint_as_float(i < 16 ? v0[2 * i] : v1[2 * i - 32]);
                  const float x1 = __uint_as_float(i < 16 ? v0[2 * i + 1] : v1[2 * i - 31]);
                  __nv_bfloat162 y = __floats2bfloat162_rn(__fsub_rn(__fmul_rn(x0, cc[e]), __fmul_rn(x1, ss[e])),
                                                           __fadd_rn(__fmul_rn(x0, ss[e]), __fmul_rn(x1, cc[e])));
                  o[i] = *(uint32_t *)&y;
                }
              }
            } else {                                          // pairs (i, i + 32): v0 holds x1, v1 holds x2
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) {
                const float4 c = cq[q4], sn = sq[q4];
                const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int e = 0; e < 4; e += 2) {
                  const int i = q4 * 4 + e;
                  const float a0 = __uint_as_float(v0[i]), a1 = __uint_as_float(v0[i + 1]);
                  const float b0 = __uint_as_float(v1[i]), b1 = __uint_as_float(v1[i + 1]);
                  __nv_bfloat162 lo = __floats2bfloat162_rn(__fsub_rn(__fmul_rn(a0, cc[e]), __fmul_rn(b0, ss[e])),
                                                            __fsub_rn(__fmul_rn(a1, cc[e + 1]), __fmul_rn(b1, ss[e + 1])));
                  __nv_bfloat162 hi = __floats2bfloat162_rn(__fadd_rn(__fmul_rn(a0, ss[e]), __fmul_rn(b0, cc[e])),
                                                            __fadd_rn(__fmul_rn(a1, ss[e + 1]), __fmul_rn(b1, cc[e + 1])));
                  o[i >> 1] = *(uint32_t *)&lo;
                  o[16 + (i >> 1)] = *(uint32_t *)&hi;
                }
              }
            }
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4 *>(dst + q * 8) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
          }
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) release_acc(acc);
          if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
          continue;
        }
      }
#pragma unroll 1
      for (int c = 0; c < (BN + 31) / 32; ++c) {      // a tile width that is not a multiple of 32 ends in a partly used chunk
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C_::ACC_STRIDE + c * 32), v);
        tmem_ld_wait();
        if (row_lane && row < p.M) {
          const int col0 = n0 + c * 32;
          if (p.epi == UGB_EPI_BF16) {
            __nv_bfloat16 *crow = (__nv_bfloat16 *)p.C + out_off + (long long)row * p.N + col0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (c * 32 + q * 8 < BN && col0 + q * 8 < p.N) {   // BN % 8 == N % 8 == 0: a chunk of 8 is all in or all out
                uint4 o;
                if (p.f16) {
                  __half2 t;
                  t = __floats2half2_rn(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1])); o.x = *(uint32_t *)&t;
                  t = __floats2half2_rn(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3])); o.y = *(uint32_t *)&t;
                  t = __floats2half2_rn(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5])); o.z = *(uint32_t *)&t;
                  t = __floats2half2_rn(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7])); o.w = *(uint32_t *)&t;
                } else {
                  __nv_bfloat162 t;
                  t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1])); o.x = *(uint32_t *)&t;
                  t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3])); o.y = *(uint32_t *)&t;
                  t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5])); o.z = *(uint32_t *)&t;
                  t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7])); o.w = *(uint32_t *)&t;
                }
                *reinterpret_cast<uint4 *>(crow + q * 8) = o;
              }
            }
          } else if (p.epi == UGB_EPI_F32) {
            float *crow = (float *)p.C + out_off + (long long)row * p.N + col0;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (c * 32 + q * 4 < BN && col0 + q * 4 < p.N)
                *reinterpret_cast<uint4 *>(crow + q * 4) = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
          } else {
            // UGB_EPI_SILU_MUL_BF16: columns come in (gate, up) pairs; out [M, N/2] bf16
            __nv_bfloat16 *crow = (__nv_bfloat16 *)p.C + out_off + (long long)row * (p.N / 2) + col0 / 2;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              if (c * 32 + q * 16 < BN && col0 + q * 16 < p.N) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float g0 = __uint_as_float(v[q * 16 + e * 4 + 0]), u0 = __uint_as_float(v[q * 16 + e * 4 + 1]);
                  const float g1 = __uint_as_float(v[q * 16 + e * 4 + 2]), u1 = __uint_as_float(v[q * 16 + e * 4 + 3]);
                  // ex2.approx-based exp and approximate division: ~1e-6 relative, far below the bf16 output step
                  __nv_bfloat162 t = __floats2bfloat162_rn(__fdividef(g0, __expf(-g0) + 1.0f) * u0,
                                                           __fdividef(g1, __expf(-g1) + 1.0f) * u1);
                  o[e] = *(uint32_t *)&t;
                }
                *reinterpret_cast<uint4 *>(crow + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) release_acc(acc);
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------------------------------- pair_k: the two k halves meet --
  // Each half finishes one half of the tile's columns (groups of 16 = 8 (gate, up) pairs: half h owns the groups
  // g with g / (groups / 2) == h).  The epilogue warps have already sent the other half's columns over (above);
  // after one cluster barrier the peer's sums are in this CTA's parking area, and each half adds its own and
  // applies the epilogue to its groups.
  if constexpr (BM == 64 && !PAIR && BN % 32 == 0) {
    if (p.pair_k) {
      constexpr int GROUPS = BN / 16;
      const int half = (int)(blockIdx.x & 1);
      const int quad = warp & 3;
      const bool row_lane = lane < 16;
      const bool work = warp >= 2 && pair_ready && !*abort_flag;
      auto mine = [&](int g) { return (g >= GROUPS / 2 ? 1 : 0) == half; };
      __syncwarp();
      cluster_sync_all();
      if (work) {
        const int row = pair_m0 + quad * 16 + lane;
        const float *park = reinterpret_cast<const float *>(smem + STAGES * STAGE_BYTES + 512) +
                            (size_t)(quad * 16 + (lane & 15)) * (BN / 2) - half * (BN / 2);   // indexed by tile column
        tcgen05_fence_after();
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (!mine(2 * c) && !mine(2 * c + 1)) continue;
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), v);
          tmem_ld_wait();
          if (row_lane && row < p.M) {
            const int col0 = pair_n0 + c * 32;
            // out [M, N/2] bf16 = silu(gate) * up over the summed (gate, up) column pairs
            __nv_bfloat16 *crow = (__nv_bfloat16 *)p.C + (long long)row * (p.N / 2) + col0 / 2;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              if (mine(2 * c + q) && col0 + q * 16 < p.N) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float4 w = *reinterpret_cast<const float4 *>(park + c * 32 + q * 16 + e * 4);
                  const float g0 = __uint_as_float(v[q * 16 + e * 4 + 0]) + w.x, u0 = __uint_as_float(v[q * 16 + e * 4 + 1]) + w.y;
                  const float g1 = __uint_as_float(v[q * 16 + e * 4 + 2]) + w.z, u1 = __uint_as_float(v[q * 16 + e * 4 + 3]) + w.w;
                  __nv_bfloat162 t = __floats2bfloat162_rn(__fdividef(g0, __expf(-g0) + 1.0f) * u0,
                                                           __fdividef(g1, __expf(-g1) + 1.0f) * u1);
                  o[e] = *(uint32_t *)&t;
                }
                *reinterpret_cast<uint4 *>(crow + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
        tcgen05_fence_before();
      }
    }
  }

  // ------------------------------------------------------------- teardown --
  if (warp == 2 && lane == 0) UGB_TC_STAMP(UGB_TC_PROF_EPILOGUE_DONE);
  __syncwarp();
  if (*abort_flag) {
    // give copies and MMAs in flight time to land before shared memory and TMEM go away
    const unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // neither CTA's shared memory, barriers or TMEM go away under the other
  if (warp == 1) {
    tcgen05_fence_after();
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    if (lane == 0) UGB_TC_STAMP(UGB_TC_PROF_END);
  }
}

// ----------------------------------------------------------------- host ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

struct TcState {
  EncodeTiledFn encode = nullptr;
  bool attr_set[10] = {false, false, false, false, false, false, false, false, false, false};
};

TcState *state_of(ugb_device *dev) {
  if (!dev->gemm_state) dev->gemm_state = new TcState();
  return (TcState *)dev->gemm_state;
}

int32_t ensure_encode(ugb_device *dev, TcState *st) {
  if (st->encode) return UGB_OK;
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
    return ugb_fail(dev, UGB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  st->encode = (EncodeTiledFn)fn;
  return UGB_OK;
}

// rank-3 bf16 tensor map: dims {d0 (contiguous), d1, d2}, strides in elements for d1, d2.
int32_t encode_map(ugb_device *dev, TcState *st, CUtensorMap *map, const void *base, uint64_t d0,
                   uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t box0, uint32_t box1, bool f16 = false) {
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1 * 2, s2 * 2};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = st->encode(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides,
                          box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return ugb_fail(dev, UGB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return UGB_OK;
}

template <int BM, int BN, bool PAIR = false>
int32_t launch_tc(ugb_device *dev, TcState *st, const ugb_tc_gemm_args &g, size_t batch, size_t m) {
  using C_ = Cfg<BM, BN, PAIR>;
  const size_t n = g.n, k = g.k;
  constexpr int slot = PAIR ? 8 : BN == 160 ? 9 : BN == 80 ? 6 : BN == 96 ? 7 : (BN == 256 ? 2 : (BN == 128 ? 1 : 0)) + (BM == 64 ? 3 : 0);
  if (!st->attr_set[slot]) {
    UGB_CUDA(dev, cudaFuncSetAttribute(tc_gemm_kernel<BM, BN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       C_::SMEM_BYTES + (C_::PAIR_K_OK ? C_::PARK_BYTES : 0)));

    st->attr_set[slot] = true;
  }
  Params p;
  p.M = (int)m; p.N = (int)n; p.K = (int)k; p.batch = (int)batch;
  p.tiles_m = (int)((m + C_::TILE_M - 1) / C_::TILE_M);
  p.tiles_n = (int)((n + BN - 1) / BN);
  p.k_blocks = (int)((k + BK - 1) / BK);
  int splits = g.splits < 1 ? 1 : g.splits;
  if (splits > p.k_blocks) splits = p.k_blocks;
  p.kb_per_split = (p.k_blocks + splits - 1) / splits;
  p.splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;   // no empty split
  p.b_batched = (batch > 1 && g.b_batch != 0) ? 1 : 0;
  p.b_is_nk = g.b_is_nk ? 1 : 0;
  p.epi = g.epi;
  p.b_static = g.b_static ? 1 : 0;
  p.f16 = g.f16 ? 1 : 0;
  p.prof = g.prof;
  p.pair_k = 0;
  if (g.pair_k) {
    // two CTAs (a cluster) per tile, each over half of k
    if (!C_::PAIR_K_OK || g.epi != UGB_EPI_SILU_MUL_BF16 || batch != 1 || p.k_blocks < 2 ||
        2 * (long long)p.tiles_m * p.tiles_n > dev->sm_count)
      return UGB_ERR_UNSUPPORTED;
    p.pair_k = 1;
    p.kb_per_split = (p.k_blocks + 1) / 2;
    p.splits = 2;
  }
  // Consecutive tiles run in the same wave.  The operand that is walked completely by every wave is read
  // from L2 again and again, so it should be the smaller one: B (n x k) when n <= m, otherwise A.
  p.n_fast = n <= m ? 1 : 0;
  const long long out_cols = g.epi == UGB_EPI_SILU_MUL_BF16 ? (long long)n / 2 : (long long)n;
  p.c_batch = g.c_batch ? g.c_batch : (long long)m * out_cols;
  p.c_split = (long long)batch * m * out_cols;
  p.C = g.out;
  p.status = dev->status_dev;
  p.rope = g.rope;

  CUtensorMap tmA, tmB;
  p.stage_tx = C_::STAGE_BYTES * (PAIR ? 2 : 1);      // PAIR: one barrier counts both CTAs' stage
  int32_t rc = encode_map(dev, st, &tmA, g.a, k, m, batch, k, batch > 1 ? (uint64_t)g.a_batch : m * k, BK, BM, g.f16);
  if (rc) return rc;
  const uint64_t nb = p.b_batched ? batch : 1;
  const uint64_t bs = p.b_batched ? (uint64_t)g.b_batch : n * k;
  if (g.b_is_nk) rc = encode_map(dev, st, &tmB, g.b, k, n, nb, k, bs, BK, C_::BN_CTA, g.f16);
  else rc = encode_map(dev, st, &tmB, g.b, n, k, nb, n, bs, 64, BK, g.f16);
  if (rc) return rc;

  const long long n_tiles = (long long)p.tiles_m * p.tiles_n * p.batch * p.splits;
  const long long slots = PAIR ? dev->sm_count / 2 : dev->sm_count;      // PAIR: one tile per cluster of two SMs
  const unsigned grid = (unsigned)(n_tiles < slots ? n_tiles : slots) * (PAIR ? 2u : 1u);
  // A shallower ring (smem_kib) leaves room for a second CTA per SM: with programmatic dependent launch
  // the next kernel's CTAs then become resident, and fetch their weights, while this kernel still runs.
  int stages = C_::STAGES;
  if (g.smem_kib > 0) {
    const int fit = (g.smem_kib * 1024 - 1536) / C_::STAGE_BYTES;
    stages = fit < 2 ? 2 : (fit > stages ? stages : fit);
  }
  p.stages = stages;
  // pair_k: behind the barriers, the parking area the other k half writes its sums into (f32 [64][BN / 2])
  const size_t smem = (size_t)stages * C_::STAGE_BYTES + 1536 + (p.pair_k ? (size_t)C_::PARK_BYTES : 0);
  if (g.query_grid || g.query_ctas_per_sm) {
    int occ = 0;
    UGB_CUDA(dev, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, tc_gemm_kernel<BM, BN, PAIR>, THREADS, smem));
    if (g.query_grid) *g.query_grid = (int)grid;
    if (g.query_ctas_per_sm) *g.query_ctas_per_sm = occ;
    return UGB_OK;
  }
  cudaError_t le = ugb_launch_cluster(tc_gemm_kernel<BM, BN, PAIR>, dim3(grid), dim3(THREADS), smem, dev->stream,
                                      g.pdl, (PAIR || p.pair_k) ? 2 : 1, tmA, tmB, p);
  if (le != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "launch of tc_gemm_kernel failed: %s", cudaGetErrorString(le));
  return ugb_after_launch(dev, "tc_gemm_kernel");
}

}  // namespace

int32_t ugb_tc_encode_bf16(ugb_device *dev, CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                           const uint64_t *strides_elems, const uint32_t *box) {
  TcState *st = state_of(dev);
  if (int32_t rc = ensure_encode(dev, st)) return rc;
  cuuint64_t d[5], sb[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) sb[i] = strides_elems[i] * 2;
  CUresult r = st->encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void *>(base), d, sb, bx, es,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ugb_fail(dev, UGB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return UGB_OK;
}

int ugb_tc_gemm_effective_splits(size_t k, int splits) {
  const int k_blocks = (int)((k + BK - 1) / BK);
  if (splits < 1) splits = 1;
  if (splits > k_blocks) splits = k_blocks;
  const int per = (k_blocks + splits - 1) / splits;
  return (k_blocks + per - 1) / per;
}

int32_t ugb_tc_gemm(ugb_device *dev, const ugb_tc_gemm_args &g) {
  size_t batch = g.batch, m = g.m;
  const size_t n = g.n, k = g.k;
  // TMA: 16-byte aligned bases, row strides that are multiples of 16 bytes.
  if (k == 0 || k % 8 != 0 || n % 8 != 0) return UGB_ERR_UNSUPPORTED;
  if (((uintptr_t)g.a | (uintptr_t)g.b | (uintptr_t)g.out) & 15) return UGB_ERR_UNSUPPORTED;
  if ((g.a_batch % 8) != 0 || (g.b_batch % 8) != 0 || g.a_batch < 0 || g.b_batch < 0) return UGB_ERR_UNSUPPORTED;
  if (batch > 1 && g.a_batch == 0) return UGB_ERR_UNSUPPORTED;
  if (m > (1u << 30) || n > (1u << 30) || k > (1u << 30) || batch > 65535) return UGB_ERR_UNSUPPORTED;
  if (g.epi == UGB_EPI_SILU_MUL_BF16 && n % 16 != 0) return UGB_ERR_UNSUPPORTED;
  if (g.splits > 1 && g.epi != UGB_EPI_F32) return UGB_ERR_UNSUPPORTED;
  if (g.f16 && g.epi != UGB_EPI_BF16 && g.epi != UGB_EPI_F32) return UGB_ERR_UNSUPPORTED;   // the fused epilogues write bf16
  if (g.epi == UGB_EPI_ROPE_QKV && (m <= 64 || batch != 1 || !g.b_is_nk || n % 64 != 0 || g.rope.t < 1)) return UGB_ERR_UNSUPPORTED;
  if (m == 0 || n == 0) return UGB_ERR_UNSUPPORTED;

  TcState *st = state_of(dev);
  if (int32_t rc = ensure_encode(dev, st)) return rc;
  // A shared B with densely stacked A batches is one tall GEMM.
  const long long dense_c = (long long)m * (long long)(g.epi == UGB_EPI_SILU_MUL_BF16 ? n / 2 : n);
  if (batch > 1 && g.b_batch == 0 && g.a_batch == (long long)(m * k) && (g.c_batch == 0 || g.c_batch == dense_c)) {
    m *= batch;
    batch = 1;
  }
  int bn = g.bn;
  if (bn == 0) bn = (m <= 128) ? 64 : 256;
  if (!g.b_is_nk && (bn == 80 || bn == 96)) bn = 128;                  // n-major B is boxed in 64-column pieces
  if (m <= 64) {
    if (bn == 64) return launch_tc<64, 64>(dev, st, g, batch, m);
    if (bn == 80) return launch_tc<64, 80>(dev, st, g, batch, m);      // widths that split n into close to one
    if (bn == 96) return launch_tc<64, 96>(dev, st, g, batch, m);      // tile per SM where 64 / 128 do not
    if (bn == 128) return launch_tc<64, 128>(dev, st, g, batch, m);
    if (bn == 160) return launch_tc<64, 160>(dev, st, g, batch, m);
    return launch_tc<64, 256>(dev, st, g, batch, m);
  }
  if (bn == 80 || bn == 96) bn = 128;                                  // BM = 128 needs n % 16 == 0 tiles: keep the three sizes
  // CTA pairs: 256 x 256 tiles over two SMs; every SM fetches half as much of B per flop
  const bool pair = g.pair < 0 ? dev->gemm_pair != 0 : g.pair != 0;
  if (pair && bn == 256 && m > 128 && g.splits <= 1 && dev->sm_count >= 2) return launch_tc<128, 256, true>(dev, st, g, batch, m);
  if (bn == 64) return launch_tc<128, 64>(dev, st, g, batch, m);
  if (bn == 128) return launch_tc<128, 128>(dev, st, g, batch, m);
  return launch_tc<128, 256>(dev, st, g, batch, m);
}

int32_t ugb_tc_gemm_bf16(ugb_device *dev, void *c, const void *a, const void *b_, size_t batch, size_t m,
                         size_t n, size_t k, long long a_batch, long long b_batch, bool b_is_nk, bool f16) {
  ugb_tc_gemm_args g;
  g.f16 = f16;
  g.out = c; g.a = a; g.b = b_;
  g.batch = batch; g.m = m; g.n = n; g.k = k;
  g.a_batch = a_batch; g.b_batch = b_batch; g.b_is_nk = b_is_nk;
  g.epi = UGB_EPI_BF16; g.splits = 1; g.bn = 0; g.b_static = false; g.pdl = false;
  return ugb_tc_gemm(dev, g);
}

void ugb_tc_state_free(ugb_device *dev) {
  if (dev->gemm_state) {
    delete (TcState *)dev->gemm_state;
    dev->gemm_state = nullptr;
  }
}
