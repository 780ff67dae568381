// Interface of the persistent decode-step kernel (decode_step.cu): one launch runs all layers of a
// decode step of the Llama engine (ug-llama/src/model.rs:203-269,365-373 for seq_len == 1).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "ugb_internal.h"

// One weight-streaming projection of a layer: out[batch, n] = a[batch, k] . w[n, k]^T, cut into
// `tiles` column tiles of `bn` and `splits` k ranges of `kb_per` 64-wide k blocks: items = tiles * splits
// work items, one per CTA and round.
struct ugb_step_gemm {
  int n, k, bn, tiles, splits, kb, kb_per, items;
};

struct ugb_step_layer {
  const float *rms1, *rms2;              // norm gains [hidden]
  __nv_bfloat16 *kcache, *vcache;        // [batch][n_kv][t_max][64]
};

enum { UGB_STEP_QKV = 0, UGB_STEP_O = 1, UGB_STEP_GATE_UP = 2, UGB_STEP_DOWN = 3 };

struct ugb_step_params {
  int batch, hidden, qkv_dim, att_width, ffn, layers, n_heads, n_kv, group, t_max, vocab, interleaved;
  float eps, inv_d, scale;
  ugb_step_gemm g[4];                    // UGB_STEP_*
  const CUtensorMap *maps;               // device memory: [layers][4] weight maps (box {64 k, bn n}), then the
                                         // activation maps of xn, att, h (box {64 k, 64 rows})
  const ugb_step_layer *layer;           // device memory: [layers]
  const __nv_bfloat16 *embed;            // [vocab, hidden]
  const int *tok;                        // [batch] input ids
  const float *ln_f;                     // final norm gains
  const float *cos_, *sin_;              // rope tables [max_pos, 32]
  const int *pos;                        // device-side position (number of cached positions)
  float *x;                              // residual stream f32 [batch, hidden]
  __nv_bfloat16 *xn, *att, *h;           // normalised rows, attention output, silu(gate) * up
  float *part;                           // split-K partials of the projection in flight: [splits][batch][n]
  float *att_po, *att_pml;               // attention partial results: (batch * n_kv + grid) slots of [8][64] and [8][2]
  unsigned int *att_cnt;                 // [batch * n_kv] completion counters, left at zero
  unsigned int *sync;                    // [0] barrier arrivals, [1] arrivals at the start of this launch, [2] abort
  ugb_status_word *status;
  int tune;                              // measurement aid: bit 0 leaves the attention arithmetic out (results are garbage),
                                         // bit 1 leaves the L2 prefetches out
  unsigned long long *prof;              // measurement aid (or null): %globaltimer of CTAs 0, 37, 74, 111 at the start,
                                         // and at the arrival at / the completion of every grid barrier: [4][UGB_STEP_PROF_SLOTS]
};
constexpr int UGB_STEP_PROF_SLOTS = 512;

// Chooses tile widths and k splits for `grid` CTAs; returns the largest number of partials any projection writes.
int ugb_decode_step_plan(ugb_step_params &p, int grid);
// Shared memory the kernel needs and the grid it wants on this device.
size_t ugb_decode_step_smem();
int32_t ugb_decode_step_launch(ugb_device *dev, const ugb_step_params &p, int grid, bool pdl);
