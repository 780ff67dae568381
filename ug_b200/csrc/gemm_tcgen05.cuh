// Interface of the tcgen05 / TMEM bf16 GEMM translation unit.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "ugb_internal.h"

// Epilogues applied to the fp32 accumulators.
enum {
  UGB_EPI_BF16 = 0,           // out [b, m, n] in the operands' 16-bit type (bf16, or f16 with args.f16)
  UGB_EPI_F32 = 1,            // out f32 [splits, b, m, n]  (split-K partials when splits > 1)
  UGB_EPI_SILU_MUL_BF16 = 2,  // columns are (gate, up) pairs: out bf16 [b, m, n/2] = silu(gate) * up
  UGB_EPI_ROPE_QKV = 3        // columns are [q heads | k heads | v heads] of 64: rope + KV append (see ugb_tc_rope_epilogue)
};

// Epilogue UGB_EPI_ROPE_QKV (m > 64, b_is_nk, batch 1, no split-K): row r of the product is position
// pos = *pos_p + pos_off + r % t of sequence r / t.  Query heads are rotated and written as bf16 to
// q_out[r][head][64]; key heads are rotated and written to kcache[b][kvh][pos][64]; value heads are
// written to vcache likewise -- what rope_append_kernel does with the fp32 product, without the round trip.
struct ugb_tc_rope_epilogue {
  const float *cos_, *sin_;       // [max_pos, 32]
  const int *pos_p;
  int pos_off, t, n_heads, n_kv, t_max, interleaved;
  __nv_bfloat16 *q_out, *kcache, *vcache;
};

// Measurement aid: with ugb_tc_gemm_args::prof set (device memory, UGB_TC_PROF_SLOTS values, zeroed by the caller),
// CTA 0 records %globaltimer when it starts, when the wait for the preceding kernel returns, when its MMA thread
// finds every k block of its first tile complete in shared memory, when it has issued the last MMA, when the
// epilogue sees the accumulator, when the epilogue (and, with pair_k, the exchange) is done, and after the TMEM release.
enum { UGB_TC_PROF_START = 0, UGB_TC_PROF_DEP = 1, UGB_TC_PROF_LAST_MMA = 2, UGB_TC_PROF_ACC_SEEN = 3,
       UGB_TC_PROF_EPILOGUE_DONE = 4, UGB_TC_PROF_END = 5, UGB_TC_PROF_KBLOCK0 = 8, UGB_TC_PROF_SLOTS = 64 };

struct ugb_tc_gemm_args {
  void *out;
  const void *a;        // bf16 [b, m, k] row-major
  const void *b;        // bf16 [n, k] row-major when b_is_nk, else [k, n] row-major
  size_t batch, m, n, k;
  long long a_batch, b_batch;   // elements between batch steps (b_batch 0 = shared operand)
  long long c_batch = 0;        // output elements between batch steps; 0 = dense (m * output columns)
  bool b_is_nk;
  int epi;              // UGB_EPI_*
  int splits;           // split-K factor (only with UGB_EPI_F32); the kernel may use fewer
  int bn;               // tile width: 64, 128, 256 (80, 96, 160 too when m <= 64 and b_is_nk), or 0 = choose from m
  bool b_static;        // no kernel on the stream writes b (weights): fetch it before waiting for the predecessor
  bool pdl;             // launch with programmatic stream serialization (see ugb_launch)
  int smem_kib = 0;     // cap on the shared memory of a CTA (ring depth follows); 0 = as deep as fits in 220 KiB
  bool f16 = false;     // operands (and the UGB_EPI_BF16 output) are IEEE f16 instead of bf16: same instruction, other format field
  bool pair_k = false;  // m <= 64, UGB_EPI_SILU_MUL_BF16: two CTAs (a thread-block cluster) per tile, each over half of k; the
                        // second hands its sums to the first through distributed shared memory.  UGB_ERR_UNSUPPORTED when
                        // twice the tiles exceed the SMs
  unsigned long long *prof = nullptr;   // measurement aid, see UGB_TC_PROF_*
  int pair = -1;        // 256 x 256 tiles on pairs of CTAs (cta_group::2) where the shape allows: 1 / 0, -1 = the device's setting
  ugb_tc_rope_epilogue rope = {};   // UGB_EPI_ROPE_QKV only
  // Query instead of launch: when set, ugb_tc_gemm launches nothing and reports the grid it would launch and how many
  // CTAs of that kernel (with its dynamic shared memory) the hardware keeps resident per SM.
  int *query_grid = nullptr, *query_ctas_per_sm = nullptr;
};

// Returns UGB_ERR_UNSUPPORTED (without touching last_error) when the shape
// does not meet the kernel's alignment rules so that the caller can fall back
// to the strided kernel.
int32_t ugb_tc_gemm(ugb_device *dev, const ugb_tc_gemm_args &args);
// Number of partials ugb_tc_gemm writes for a requested split factor.
int ugb_tc_gemm_effective_splits(size_t k, int splits);
// C[b, m, n] = A . B with the default epilogue, all three bf16 (f16 = false) or IEEE f16.
int32_t ugb_tc_gemm_bf16(ugb_device *dev, void *c, const void *a, const void *b_, size_t batch,
                         size_t m, size_t n, size_t k, long long a_batch, long long b_batch,
                         bool b_is_nk, bool f16 = false);
// bf16 tensor map with the 128-byte swizzle: dims / box of `rank` entries (dims[0] contiguous), strides in
// elements for dims 1 .. rank-1 (multiples of 8).
int32_t ugb_tc_encode_bf16(ugb_device *dev, CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                           const uint64_t *strides_elems, const uint32_t *box);
void ugb_tc_state_free(ugb_device *dev);
