// Fused Llama engine: the Model::fwd call sites of ug-llama (ug-llama/src/model.rs:298-374) as fixed
// sequences of hand-written kernels.
//
// Decode (one new token per sequence), per layer (model.rs:203-269) 7 launches, captured in a CUDA graph:
//   reduce_rmsnorm   residual += previous down-proj partials; rms1 -> bf16
//   tcgen05 GEMM     fused q|k|v projection, split-K fp32 partials
//   decode_attention sums the partials, rope(q), rope(k), writes k/v into the KV cache, then
//                    grouped-query flash-decode over the cache (+ slice merge)
//   tcgen05 GEMM     o_proj, split-K partials
//   reduce_rmsnorm   residual += o_proj partials; rms2 -> bf16
//   tcgen05 GEMM     gate|up projection (rows interleaved), epilogue silu(gate)*up -> bf16
//   tcgen05 GEMM     down projection, split-K partials
// then the final norm, the tied lm_head GEMM (fp32 logits) and a row argmax that also advances the
// position.  Prefill (a block of positions per sequence, in chunks of rows): the same chain with m = rows;
// the qkv GEMM's epilogue rotates q / k and appends K / V, attention is the causal tcgen05 kernel of
// attention_tc.cu.  Tensor parallel: a rank keeps its share of heads / FFN columns / vocabulary and the
// norm kernel sums all ranks' partials over peer memory (tp_kernels.cuh).
// Weights and the KV cache are bf16, the residual stream and every reduction are fp32.  Batch rows are
// independent sequences that share one position (the reference's pos[0] convention).
//
// HBM layout per model: weights [layer]{wqkv [(h+2kv)*d, hidden], wo [hidden, h*d], wgu [2*ffn, hidden]
// (gate row j at 2j, up row j at 2j+1), wdown [hidden, ffn]}, embedding [vocab, hidden]; KV cache K and V
// each [layer][batch][kv_head][t_max][head_dim] bf16 (t_max rounded up to 16).
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "decode_kernels.cuh"
#include "gemm_tcgen05.cuh"
#include "tp_kernels.cuh"
#include "attention_tc.cuh"
#include "decode_step.cuh"

using namespace ugb_decode;

struct LayerW {
  __nv_bfloat16 *wqkv = nullptr, *wo = nullptr, *wgu = nullptr, *wdown = nullptr;
  float *rms1 = nullptr, *rms2 = nullptr;
};

struct ugb_llama {
  ugb_device *dev = nullptr;
  ugb_llama_config cfg{};         // the whole model (weight shapes, vocabulary range)
  ugb_llama_config lc{};          // this rank's share: n_heads, n_kv_heads and ffn are the local counts
  int batch = 0, t_max = 0;       // t_max padded to a multiple of 16
  // tensor parallelism: rank tp_rank of tp_size owns query heads [q0, q0 + lc.n_heads), KV heads
  // [kv0, kv0 + lc.n_kv_heads) (a KV head is replicated when tp_size > n_kv_heads), FFN columns
  // [tp_rank * lc.ffn, ...) and logit columns [tp_rank * vl, ...).  tp == false: one rank, plain kernels.
  bool tp = false;
  int tp_rank = 0, tp_size = 1, q0 = 0, kv0 = 0, vl = 0;
  void *tp_block = nullptr;       // exchange block of this rank (header, o / down partials, argmax pairs)
  size_t tp_off_o = 0, tp_off_down = 0, tp_off_pairs = 0, tp_block_bytes = 0, tp_part_rows = 0;
  void *tp_peer[TP_MAX] = {};     // every rank's exchange block as mapped here (own included)
  bool tp_ready = false;
  unsigned timeouts_at_create = 0;   // dev->wait_timeouts when the model was created (see tp_in_step)
  int qkv_dim = 0;
  std::vector<LayerW> layers;
  __nv_bfloat16 *embed = nullptr;
  float *ln_f = nullptr;
  float *cos = nullptr, *sin = nullptr;
  __nv_bfloat16 *kcache = nullptr, *vcache = nullptr;
  size_t kv_layer_stride = 0;     // elements per layer of one cache
  // activations / scratch
  float *x = nullptr, *part = nullptr, *logits = nullptr;
  __nv_bfloat16 *xn = nullptr, *q = nullptr, *att = nullptr, *h = nullptr;
  float *att_po = nullptr, *att_pml = nullptr;
  unsigned int *att_cnt = nullptr;
  int *tok = nullptr, *next = nullptr, *pos = nullptr;
  int host_pos = 0;
  // tuning
  int splits_qkv = 5, splits_o = 8, splits_down = 8, att_splits = 1, att_stages = 5;
  int pdl = 1;                    // programmatic dependent launch between the kernels of a step
  int gemm_smem_kib = 144;        // shared-memory cap of the decode GEMM CTAs (0 = deepest ring); measured best
  int skip = 0;                   // measurement aid: bit mask of kernel types left out of the step
  int bn_qkv = 128, bn_o = 128, bn_gate_up = 128, bn_down = 128, bn_lm_head = 256;   // GEMM tile widths
  size_t part_elems = 0;
  // graph of one step that reads `next` as its input tokens
  cudaGraphExec_t graph = nullptr;
  int graph_nodes = 0;
  bool warmed = false;
  std::vector<void *> allocs;
  size_t loaded = 0;
  // prefill workspace, allocated by the first ugb_llama_prefill: activations of one chunk of
  // pf_rows = batch * pf_chunk rows (pf_chunk positions of every sequence)
  // persistent decode-step kernel (decode_step.cu): option step_kernel
  int step_kernel = 0;            // 1: a decode step is one launch of decode_step_kernel + lm_head + argmax
  bool step_ready = false;
  int step_grid = 0;
  ugb_step_params step{};
  unsigned step_timeouts = 0;     // dev->wait_timeouts when the barrier words were last cleared
  int att_early = 1;              // option att_early: kernels may fetch old data before griddepcontrol.wait when that is provably safe
  bool early_ok = false;          // ... and it is, for the current shapes and options (set by enqueue_step)
  unsigned long long *gemm_prof = nullptr;   // option gemm_profile: [5 projections][UGB_TC_PROF_SLOTS] stamps of the decode GEMMs
  int gate_up_pair = 1;           // option gate_up_pair: decode gate|up on pairs of CTAs that split k (see gemm_rows)
  int att_cluster = 1;            // option att_cluster: the KV slices of a (sequence, KV head) pair run as one cluster and
                                  // are combined through distributed shared memory
  int att_tma = 0;                // option att_tma: decode attention fetches K / V by TMA (1) or cp.async (0)
  std::vector<CUtensorMap> att_kmap, att_vmap;   // per layer, for the TMA variant
  int pf_att_tc = 1;              // option prefill_attention_tc: 1 = tcgen05 / TMEM attention kernel drawing its
                                  // work items from a counter, 2 = the same dealt round-robin, 0 = mma.sync kernel
  int pf_rows_max = 8192;         // option prefill_rows: upper bound on rows per chunk
  int pf_rows = 0, pf_chunk = 0;
  float *pf_x = nullptr, *pf_f32 = nullptr;            // residual stream; f32 GEMM output (qkv, o, down)
  __nv_bfloat16 *pf_xn = nullptr, *pf_q = nullptr, *pf_att = nullptr, *pf_h = nullptr;
  int *pf_tok = nullptr;
  size_t pf_tok_cap = 0;
  float *pf_logits = nullptr;     // [batch, pf_logits_t, vocab] when all-position logits were requested
  int pf_logits_t = 0;
  size_t pf_logits_cap = 0;
};

namespace {

template <typename T>
int32_t dmalloc(ugb_llama *m, T **p, size_t n, bool zero = false) {
  ugb_device *dev = m->dev;
  void *v = nullptr;
  UGB_CUDA(dev, cudaMalloc(&v, n * sizeof(T) ? n * sizeof(T) : 16));
  if (zero) UGB_CUDA(dev, cudaMemsetAsync(v, 0, n * sizeof(T), dev->stream));
  m->allocs.push_back(v);
  *p = (T *)v;
  return UGB_OK;
}

__global__ void f32_to_bf16_kernel(const float *__restrict__ s, __nv_bfloat16 *__restrict__ d, size_t n,
                                   size_t row_len, size_t dst_pitch, size_t src_pitch) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    d[(i / row_len) * dst_pitch + i % row_len] = __float2bfloat16_rn(s[(i / row_len) * src_pitch + i % row_len]);
}

// Copies rows [row0, row0 + nrows) x columns [col0, col0 + ncols) of a [rows, cols] matrix (bf16, or f32
// rounded to bf16) into `dst` with a destination row pitch in elements (interleaving gate/up uses
// pitch 2 * hidden).  The shape check is on the whole tensor, as Linear::new does it (model.rs:142-144);
// a tensor-parallel rank keeps its slice only.
int32_t put_sub(ugb_llama *m, const ugb_slice *w, __nv_bfloat16 *dst, size_t rows, size_t cols, size_t row0,
                size_t nrows, size_t col0, size_t ncols, size_t dst_pitch, const char *name) {
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, w->len == rows * cols, UGB_ERR_SHAPE, "unexpected shape for %s: %zu elements, expected (%zu, %zu)",
              name, w->len, rows, cols);
  const size_t off = row0 * cols + col0;
  if (w->dtype == UGB_BF16) {
    UGB_CUDA(dev, cudaMemcpy2DAsync(dst, dst_pitch * 2, (const __nv_bfloat16 *)w->ptr + off, cols * 2, ncols * 2, nrows,
                                    cudaMemcpyDeviceToDevice, dev->stream));
  } else if (w->dtype == UGB_F32) {
    f32_to_bf16_kernel<<<dev->sm_count * 8, 256, 0, dev->stream>>>((const float *)w->ptr + off, dst, nrows * ncols, ncols,
                                                                    dst_pitch, cols);
    return ugb_after_launch(dev, "f32_to_bf16_kernel");
  } else {
    return ugb_fail(dev, UGB_ERR_DTYPE, "%s: weights must be BF16 or F32", name);
  }
  return UGB_OK;
}

int32_t put_matrix(ugb_llama *m, const ugb_slice *w, __nv_bfloat16 *dst, size_t rows, size_t cols,
                   size_t dst_pitch, const char *name) {
  return put_sub(m, w, dst, rows, cols, 0, rows, 0, cols, dst_pitch, name);
}

int32_t put_vector(ugb_llama *m, const ugb_slice *w, float *dst, size_t n, const char *name) {
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, w->len == n, UGB_ERR_SHAPE, "unexpected shape for %s: %zu elements, expected %zu", name, w->len, n);
  UGB_REQUIRE(dev, w->dtype == UGB_F32, UGB_ERR_DTYPE, "%s: norm weights must be F32", name);
  UGB_CUDA(dev, cudaMemcpyAsync(dst, w->ptr, n * 4, cudaMemcpyDeviceToDevice, dev->stream));
  return UGB_OK;
}

// out[rows, n] = a[rows, k] . w[n, k]^T on the tensor-core kernel (weights are the static operand).
int32_t gemm_rows(ugb_llama *m, size_t rows, void *out, const __nv_bfloat16 *a, const __nv_bfloat16 *w, size_t n,
                  size_t k, int epi, int splits, int bn, const ugb_tc_rope_epilogue *rope = nullptr, int *query_grid = nullptr,
                  int *query_occ = nullptr) {
  ugb_tc_gemm_args g;
  g.query_grid = query_grid;
  g.query_ctas_per_sm = query_occ;
  if (rope) g.rope = *rope;
  g.out = out; g.a = a; g.b = w;
  g.batch = 1; g.m = rows; g.n = n; g.k = k;
  g.a_batch = 0; g.b_batch = 0; g.b_is_nk = true;
  g.epi = epi; g.splits = splits; g.bn = bn; g.b_static = true; g.pdl = m->pdl != 0;
  g.smem_kib = rows <= 64 ? m->gemm_smem_kib : 0;
  if (m->gemm_prof && rows <= 64) {     // qkv, o, gate|up, down, lm_head
    const int kind = epi == UGB_EPI_SILU_MUL_BF16 ? 2 : n == (size_t)m->qkv_dim ? 0 : n == (size_t)m->vl ? 4 : k == (size_t)m->lc.ffn ? 3 : 1;
    g.prof = m->gemm_prof + (size_t)kind * UGB_TC_PROF_SLOTS;
  }
  if (epi == UGB_EPI_SILU_MUL_BF16 && rows <= 64 && m->gate_up_pair && (n + 159) / 160 * 2 <= (size_t)m->dev->sm_count) {
    // gate|up of a decode step: 160-wide tiles, the two k halves of a tile on a pair of CTAs (the k loop of a CTA,
    // not the weight stream, is what bounds the narrow-tile kernel)
    g.bn = 160;
    g.pair_k = true;
    const int32_t rc2 = ugb_tc_gemm(m->dev, g);
    if (rc2 != UGB_ERR_UNSUPPORTED) return rc2;
    g.bn = bn;
    g.pair_k = false;
  }
  int32_t rc = ugb_tc_gemm(m->dev, g);
  if (rc == UGB_ERR_UNSUPPORTED)
    return ugb_fail(m->dev, rc, "GEMM m=%zu n=%zu k=%zu does not meet the tensor-core kernel's shape rules", rows, n, k);
  return rc;
}

int32_t gemm(ugb_llama *m, void *out, const __nv_bfloat16 *a, const __nv_bfloat16 *w, size_t n, size_t k,
             int epi, int splits, int bn) {
  return gemm_rows(m, (size_t)m->batch, out, a, w, n, k, epi, splits, bn);
}

int32_t launch_reduce_rmsnorm_rows(ugb_llama *m, int rows, float *x, __nv_bfloat16 *xn, const float *part, int n_part,
                                   const float *alpha, int early = 0) {
  const int hidden = m->cfg.hidden;
  const int nvec = hidden / 4;
  const size_t stride = (size_t)rows * hidden;
  const float inv_d = 1.0f / (float)hidden, eps = m->cfg.rms_eps;
  dim3 grid(rows);
  cudaStream_t st = m->dev->stream;
  const bool pdl = m->pdl != 0;
  cudaError_t e;
  if (nvec <= 256) e = ugb_launch(reduce_rmsnorm_kernel<1>, grid, dim3(256), 0, st, pdl, x, part, n_part, stride, alpha, xn, hidden, inv_d, eps, early);
  else if (nvec <= 512) e = ugb_launch(reduce_rmsnorm_kernel<2>, grid, dim3(256), 0, st, pdl, x, part, n_part, stride, alpha, xn, hidden, inv_d, eps, early);
  else if (nvec <= 1024) e = ugb_launch(reduce_rmsnorm_kernel<4>, grid, dim3(256), 0, st, pdl, x, part, n_part, stride, alpha, xn, hidden, inv_d, eps, early);
  else e = ugb_launch(reduce_rmsnorm_kernel<8>, grid, dim3(256), 0, st, pdl, x, part, n_part, stride, alpha, xn, hidden, inv_d, eps, early);
  if (e != cudaSuccess) return ugb_fail(m->dev, UGB_ERR_CUDA, "launch of reduce_rmsnorm_kernel failed: %s", cudaGetErrorString(e));
  return ugb_after_launch(m->dev, "reduce_rmsnorm_kernel");
}

int32_t launch_reduce_rmsnorm(ugb_llama *m, const float *part, int n_part, const float *alpha) {
  return launch_reduce_rmsnorm_rows(m, m->batch, m->x, m->xn, part, n_part, alpha);
}

// Where the row-parallel projections leave their fp32 partials: in the exchange block when peers read them.
enum { RED_NONE = 0, RED_O = 1, RED_DOWN = 2 };
float *o_out(ugb_llama *m, float *local) { return m->tp ? (float *)((char *)m->tp_block + m->tp_off_o) : local; }
float *down_out(ugb_llama *m, float *local) { return m->tp ? (float *)((char *)m->tp_block + m->tp_off_down) : local; }

TpPeers tp_peers(const ugb_llama *m, size_t offset) {
  TpPeers t{};
  t.rank = m->tp_rank;
  t.size = m->tp_size;
  for (int r = 0; r < m->tp_size; ++r) {
    t.hdr[r] = (TpHeader *)m->tp_peer[r];
    t.part[r] = (const float *)((const char *)m->tp_peer[r] + offset);
  }
  return t;
}

// x += (sum of the partials of projection `which`), xn = rmsnorm(x) for `rows` rows.  Single rank: the
// split-K partials in `local`; tensor parallel: every rank's partials, read in place over NVLink.
int32_t launch_reduce(ugb_llama *m, int rows, float *x, __nv_bfloat16 *xn, int which, const float *local, int n_part,
                      const float *alpha, int early = 0) {
  if (!m->tp || which == RED_NONE || n_part == 0) return launch_reduce_rmsnorm_rows(m, rows, x, xn, local, n_part, alpha, early);
  if (!m->tp_ready) return ugb_fail(m->dev, UGB_ERR_INVALID, "tensor-parallel model: peers not connected (ugb_llama_tp_connect)");
  const int hidden = m->cfg.hidden, nvec = hidden / 4;
  const size_t stride = (size_t)rows * hidden;
  const float inv_d = 1.0f / (float)hidden, eps = m->cfg.rms_eps;
  const TpPeers tp = tp_peers(m, which == RED_O ? m->tp_off_o : m->tp_off_down);
  cudaStream_t st = m->dev->stream;
  const bool pdl = m->pdl != 0;
  ugb_status_word *status = m->dev->status_dev;
  cudaError_t e;
  const dim3 blk(TP_RED_THREADS);
  if (nvec <= TP_RED_THREADS) e = ugb_launch(tp_reduce_rmsnorm_kernel<1>, dim3(rows), blk, 0, st, pdl, x, tp, n_part, stride, alpha, xn, hidden, inv_d, eps, status);
  else if (nvec <= 2 * TP_RED_THREADS) e = ugb_launch(tp_reduce_rmsnorm_kernel<2>, dim3(rows), blk, 0, st, pdl, x, tp, n_part, stride, alpha, xn, hidden, inv_d, eps, status);
  else e = ugb_launch(tp_reduce_rmsnorm_kernel<4>, dim3(rows), blk, 0, st, pdl, x, tp, n_part, stride, alpha, xn, hidden, inv_d, eps, status);
  if (e != cudaSuccess) return ugb_fail(m->dev, UGB_ERR_CUDA, "launch of tp_reduce_rmsnorm_kernel failed: %s", cudaGetErrorString(e));
  return ugb_after_launch(m->dev, "tp_reduce_rmsnorm_kernel");
}

// logits[rows, vl] = xn . embed[rank's vocabulary slice]^T (tied lm_head, vocab-parallel), then the greedy
// choice: plain argmax on one rank, (value, id) pairs exchanged between the ranks otherwise.
int32_t launch_lm_head_argmax(ugb_llama *m, bool pdl_first) {
  ugb_device *dev = m->dev;
  const ugb_llama_config &c = m->lc;
  int32_t rc;
  const __nv_bfloat16 *w = m->embed + (size_t)m->tp_rank * m->vl * c.hidden;
  if (!(m->skip & 128) && (rc = gemm(m, m->logits, m->xn, w, (size_t)m->vl, c.hidden, UGB_EPI_F32, 1, m->bn_lm_head))) return rc;
  cudaStream_t st = dev->stream;
  const bool pdl = pdl_first && m->pdl != 0;
  cudaError_t e;
  if (!m->tp) {
    e = ugb_launch(argmax_rows_kernel, dim3(m->batch), dim3(1024), 0, st, pdl, m->logits, m->vl, m->next, m->pos);
    if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "launch of argmax_rows_kernel failed: %s", cudaGetErrorString(e));
    return ugb_after_launch(dev, "argmax_rows_kernel");
  }
  if (!m->tp_ready) return ugb_fail(dev, UGB_ERR_INVALID, "tensor-parallel model: peers not connected (ugb_llama_tp_connect)");
  float2 *pairs = (float2 *)((char *)m->tp_block + m->tp_off_pairs);
  e = ugb_launch(tp_argmax_local_kernel, dim3(m->batch), dim3(1024), 0, st, pdl, m->logits, m->vl, m->tp_rank * m->vl, pairs);
  if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "launch of tp_argmax_local_kernel failed: %s", cudaGetErrorString(e));
  if ((rc = ugb_after_launch(dev, "tp_argmax_local_kernel"))) return rc;
  const TpPeers tp = tp_peers(m, m->tp_off_pairs);
  e = ugb_launch(tp_argmax_final_kernel, dim3(1), dim3(128), 0, st, m->pdl != 0, tp, m->batch, m->next, m->pos, dev->status_dev);
  if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "launch of tp_argmax_final_kernel failed: %s", cudaGetErrorString(e));
  return ugb_after_launch(dev, "tp_argmax_final_kernel");
}

// Rope of q and k, append of the new K / V rows and attention over the cache, one kernel per layer.
// `append` false (kernel timing): the cache is left untouched.
bool tma_requested(const ugb_llama *m) { return m->att_tma != 0 && !m->att_kmap.empty(); }

int32_t launch_attention(ugb_llama *m, int layer, float scale, int n_part, bool append) {
  const ugb_llama_config &c = m->lc;
  __nv_bfloat16 *kc = m->kcache + (size_t)layer * m->kv_layer_stride;
  __nv_bfloat16 *vc = m->vcache + (size_t)layer * m->kv_layer_stride;
  dim3 grid(m->att_splits, c.n_kv_heads, m->batch);
  cudaStream_t st = m->dev->stream;
  AttRope rope;
  rope.part = m->part; rope.n_part = n_part; rope.part_stride = (size_t)m->batch * m->qkv_dim;
  rope.cos_ = m->cos; rope.sin_ = m->sin; rope.interleaved = c.rope_interleaved; rope.append = append ? 1 : 0;
  rope.status = m->dev->status_dev;
  rope.early = (layer > 0 && append && m->early_ok && !tma_requested(m)) ? 1 : 0;
  const int cluster = (m->att_cluster && m->att_splits > 1) ? m->att_splits : 1;
  rope.cluster = cluster > 1 ? 1 : 0;
  const bool tma = m->att_tma != 0 && !m->att_kmap.empty();
  const CUtensorMap none{};
  const CUtensorMap &mk = tma ? m->att_kmap[layer] : none, &mv = tma ? m->att_vmap[layer] : none;
  cudaError_t e = cudaSuccess;
#define UGB_ATT_LAUNCH(NS)                                                                                   \
  e = tma ? ugb_launch_cluster(decode_attention_kernel_t<NS, true>, grid, dim3(ATT_WARPS * 32), att_dyn_smem(NS, true), st,       \
                       m->pdl != 0, cluster, (const __nv_bfloat16 *)nullptr, kc, vc, (const int *)m->pos, m->att_po, m->att_pml,   \
                       m->att_cnt, m->att, c.n_heads, c.n_kv_heads, c.n_heads / c.n_kv_heads, m->t_max, scale, rope, mk, mv) \
          : ugb_launch_cluster(decode_attention_kernel_t<NS, false>, grid, dim3(ATT_WARPS * 32), att_dyn_smem(NS, false), st,     \
                       m->pdl != 0, cluster, (const __nv_bfloat16 *)nullptr, kc, vc, (const int *)m->pos, m->att_po, m->att_pml,   \
                       m->att_cnt, m->att, c.n_heads, c.n_kv_heads, c.n_heads / c.n_kv_heads, m->t_max, scale, rope, mk, mv)
  switch (m->att_stages) {
    case 2: UGB_ATT_LAUNCH(2); break;
    case 4: UGB_ATT_LAUNCH(4); break;
    case 5: UGB_ATT_LAUNCH(5); break;
    case 3: UGB_ATT_LAUNCH(3); break;
    case 6: UGB_ATT_LAUNCH(6); break;
    default: UGB_ATT_LAUNCH(5); break;
  }
#undef UGB_ATT_LAUNCH
  if (e != cudaSuccess) return ugb_fail(m->dev, UGB_ERR_CUDA, "launch of decode_attention_kernel failed: %s", cudaGetErrorString(e));
  return ugb_after_launch(m->dev, "decode_attention_kernel");
}

// Everything the persistent decode-step kernel needs besides the model's own buffers: the plan (tile widths and
// k splits for this device's SM count), tensor maps over the weights and the activation buffers, partial and
// attention scratch sized for the plan, the barrier words.  Allocated once, freed with the model.
bool step_kernel_applies(const ugb_llama *m) { return m->step_kernel && !m->tp && m->batch <= 64 && m->skip == 0; }

int32_t ensure_step_kernel(ugb_llama *m) {
  if (m->step_ready) return UGB_OK;
  ugb_device *dev = m->dev;
  const ugb_llama_config &c = m->lc;
  ugb_step_params &p = m->step;
  p = ugb_step_params{};
  p.batch = m->batch; p.hidden = c.hidden; p.qkv_dim = m->qkv_dim; p.att_width = c.n_heads * c.head_dim;
  p.ffn = c.ffn; p.layers = c.layers; p.n_heads = c.n_heads; p.n_kv = c.n_kv_heads; p.group = c.n_heads / c.n_kv_heads;
  p.t_max = m->t_max; p.vocab = c.vocab; p.interleaved = c.rope_interleaved;
  p.eps = c.rms_eps; p.inv_d = 1.0f / (float)c.hidden; p.scale = powf((float)c.head_dim, -0.5f);   // model.rs:236
  m->step_grid = dev->sm_count;
  const int most = ugb_decode_step_plan(p, m->step_grid);
  UGB_REQUIRE(dev, c.hidden % 64 == 0 && c.ffn % 8 == 0, UGB_ERR_UNSUPPORTED, "step_kernel: hidden must be a multiple of 64");
  int32_t rc;
  // partials of the widest projection
  size_t part = 0;
  for (int i = 0; i < 4; ++i)
    if (i != UGB_STEP_GATE_UP) part = std::max(part, (size_t)p.g[i].splits * m->batch * p.g[i].n);
  (void)most;
  float *partials = nullptr, *po = nullptr, *pml = nullptr;
  unsigned *cnt = nullptr, *sync = nullptr;
  const size_t slots = (size_t)m->batch * c.n_kv_heads + (size_t)m->step_grid;
  if ((rc = dmalloc(m, &partials, part))) return rc;
  if ((rc = dmalloc(m, &po, slots * ATT_GROUP * ATT_HD))) return rc;
  if ((rc = dmalloc(m, &pml, slots * ATT_GROUP * 2))) return rc;
  if ((rc = dmalloc(m, &cnt, (size_t)m->batch * c.n_kv_heads, true))) return rc;
  if ((rc = dmalloc(m, &sync, 4, true))) return rc;
  // tensor maps: per layer qkv / o / gate-up / down weights with the plan's tile width, then xn / att / h
  std::vector<CUtensorMap> maps((size_t)c.layers * 4 + 3);
  auto weight_map = [&](CUtensorMap *map, const __nv_bfloat16 *w, const ugb_step_gemm &g) {
    const uint64_t dims[3] = {(uint64_t)g.k, (uint64_t)g.n, 1};
    const uint64_t strides[2] = {(uint64_t)g.k, (uint64_t)g.n * g.k};
    const uint32_t box[3] = {64, (uint32_t)g.bn, 1};
    return ugb_tc_encode_bf16(dev, map, w, 3, dims, strides, box);
  };
  auto act_map = [&](CUtensorMap *map, const __nv_bfloat16 *a, size_t k) {
    const uint64_t dims[3] = {(uint64_t)k, (uint64_t)m->batch, 1};
    const uint64_t strides[2] = {(uint64_t)k, (uint64_t)m->batch * k};
    const uint32_t box[3] = {64, 64, 1};
    return ugb_tc_encode_bf16(dev, map, a, 3, dims, strides, box);
  };
  std::vector<ugb_step_layer> layers(c.layers);
  for (int l = 0; l < c.layers; ++l) {
    const LayerW &w = m->layers[l];
    if ((rc = weight_map(&maps[(size_t)l * 4 + UGB_STEP_QKV], w.wqkv, p.g[UGB_STEP_QKV]))) return rc;
    if ((rc = weight_map(&maps[(size_t)l * 4 + UGB_STEP_O], w.wo, p.g[UGB_STEP_O]))) return rc;
    if ((rc = weight_map(&maps[(size_t)l * 4 + UGB_STEP_GATE_UP], w.wgu, p.g[UGB_STEP_GATE_UP]))) return rc;
    if ((rc = weight_map(&maps[(size_t)l * 4 + UGB_STEP_DOWN], w.wdown, p.g[UGB_STEP_DOWN]))) return rc;
    layers[l].rms1 = w.rms1; layers[l].rms2 = w.rms2;
    layers[l].kcache = m->kcache + (size_t)l * m->kv_layer_stride;
    layers[l].vcache = m->vcache + (size_t)l * m->kv_layer_stride;
  }
  if ((rc = act_map(&maps[(size_t)c.layers * 4 + 0], m->xn, c.hidden))) return rc;
  if ((rc = act_map(&maps[(size_t)c.layers * 4 + 1], m->att, (size_t)c.n_heads * c.head_dim))) return rc;
  if ((rc = act_map(&maps[(size_t)c.layers * 4 + 2], m->h, c.ffn))) return rc;
  CUtensorMap *maps_dev = nullptr;
  ugb_step_layer *layers_dev = nullptr;
  if ((rc = dmalloc(m, &maps_dev, maps.size()))) return rc;
  if ((rc = dmalloc(m, &layers_dev, layers.size()))) return rc;
  UGB_CUDA(dev, cudaMemcpyAsync(maps_dev, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice, dev->stream));
  UGB_CUDA(dev, cudaMemcpyAsync(layers_dev, layers.data(), layers.size() * sizeof(ugb_step_layer), cudaMemcpyHostToDevice, dev->stream));
  UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));         // the host vectors go away
  p.maps = maps_dev; p.layer = layers_dev;
  p.embed = m->embed; p.ln_f = m->ln_f; p.cos_ = m->cos; p.sin_ = m->sin; p.pos = m->pos;
  p.x = m->x; p.xn = m->xn; p.att = m->att; p.h = m->h; p.part = partials;
  p.att_po = po; p.att_pml = pml; p.att_cnt = cnt; p.sync = sync; p.status = dev->status_dev;
  m->step_timeouts = dev->wait_timeouts;
  m->step_ready = true;
  return UGB_OK;
}

// A tensor-parallel model whose device has reported a wait that gave up since the model was created may have
// ranks that are no longer in step (a rank that stopped waiting summed partials its peers had not finished):
// it takes no further steps.
int32_t tp_in_step(ugb_llama *m) {
  if (m->tp && m->tp_size > 1 && m->dev->wait_timeouts != m->timeouts_at_create)
    return ugb_fail(m->dev, UGB_ERR_TIMEOUT, "tensor-parallel model: a wait on a peer gave up earlier (UGB_ERR_TIMEOUT was "
                    "reported by ugb_sync); the ranks may be out of step -- destroy and recreate the model on every rank");
  return UGB_OK;
}

// Enqueues one decode step on the device stream; `tok` holds the input ids.
int32_t enqueue_step(ugb_llama *m, const int *tok) {
  ugb_device *dev = m->dev;
  const ugb_llama_config &c = m->lc;         // this rank's share of heads and FFN columns
  cudaStream_t st = dev->stream;
  const int B = m->batch, H = c.hidden, AW = c.n_heads * c.head_dim;
  int32_t rc;
  const bool pdl = m->pdl != 0;
  if (step_kernel_applies(m) && m->step_ready) {
    // one persistent kernel for the embedding, all layers and the final norm; then the tied lm_head and the choice
    m->step.tok = tok;
    if ((rc = ugb_decode_step_launch(dev, m->step, m->step_grid, pdl))) return rc;
    return launch_lm_head_argmax(m, true);
  }
  cudaError_t e = ugb_launch(embed_gather_kernel, dim3(B), dim3(256), 0, st, pdl, m->embed, tok, m->x, H, c.vocab, dev->status_dev, 1, 1, 0);
  if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "launch of embed_gather_kernel failed: %s", cudaGetErrorString(e));
  if ((rc = ugb_after_launch(dev, "embed_gather_kernel"))) return rc;
  const int s_qkv = ugb_tc_gemm_effective_splits(H, m->splits_qkv);
  const int s_o = ugb_tc_gemm_effective_splits(AW, m->splits_o);
  const int s_down = ugb_tc_gemm_effective_splits(c.ffn, m->splits_down);
  const float scale = powf((float)c.head_dim, -0.5f);   // model.rs:236
  float *po = o_out(m, m->part), *pd = down_out(m, m->part);
  // Work done before griddepcontrol.wait (the attention kernel's K/V ring, the norm kernel's residual row)
  // reads data written two or more kernels back.  That is safe when the two projections around the
  // writer's successor cannot be resident together: if at most ONE CTA of each projection fits on an SM and
  // neither grid exceeds the SM count, then once all CTAs of the later GEMM have started (which is what lets
  // the reading kernel launch) fewer than sm_count - ctas(later) CTAs of the earlier one can still be there;
  // with ctas(earlier) + ctas(later) > sm_count at least one has left, hence passed its own wait, hence
  // everything before it -- the writer included -- has completed.  Both facts are taken from the launches
  // themselves (the grid each projection gets, the residency the occupancy calculator gives its kernel with
  // its shared memory), not from the tuning options, so a retune that breaks the argument switches this off.
  const int sms = dev->sm_count;
  int c_qkv = 0, c_o = 0, c_gu = 0, c_down = 0, o_qkv = 0, o_o = 0, o_gu = 0, o_down = 0;
  bool early = m->att_early && m->pdl && m->skip == 0;
  if (early) {
    const LayerW &w0 = m->layers[0];
    if (gemm_rows(m, B, m->part, m->xn, w0.wqkv, m->qkv_dim, H, UGB_EPI_F32, m->splits_qkv, m->bn_qkv, nullptr, &c_qkv, &o_qkv) ||
        gemm_rows(m, B, po, m->att, w0.wo, H, AW, UGB_EPI_F32, m->splits_o, m->bn_o, nullptr, &c_o, &o_o) ||
        gemm_rows(m, B, m->h, m->xn, w0.wgu, 2 * (size_t)c.ffn, H, UGB_EPI_SILU_MUL_BF16, 1, m->bn_gate_up, nullptr, &c_gu, &o_gu) ||
        gemm_rows(m, B, pd, m->h, w0.wdown, H, c.ffn, UGB_EPI_F32, m->splits_down, m->bn_down, nullptr, &c_down, &o_down))
      early = false;
  }
  m->early_ok = early && o_qkv == 1 && o_o == 1 && o_gu == 1 && o_down == 1 && c_qkv <= sms && c_o <= sms && c_gu <= sms &&
                c_down <= sms && c_qkv + c_o > sms && c_gu + c_down > sms && c_down + c_qkv > sms;
  const int early_i = m->early_ok ? 1 : 0;
  for (int l = 0; l < c.layers; ++l) {
    const LayerW &w = m->layers[l];
    if (!(m->skip & 1) && (rc = launch_reduce(m, B, m->x, m->xn, l == 0 ? RED_NONE : RED_DOWN, pd, l == 0 ? 0 : s_down, w.rms1, l > 0 ? early_i : 0))) return rc;
    if (!(m->skip & 2) && (rc = gemm(m, m->part, m->xn, w.wqkv, m->qkv_dim, H, UGB_EPI_F32, m->splits_qkv, m->bn_qkv))) return rc;
    __nv_bfloat16 *kc = m->kcache + (size_t)l * m->kv_layer_stride;
    __nv_bfloat16 *vc = m->vcache + (size_t)l * m->kv_layer_stride;
    if (!(m->skip & 8) && (rc = launch_attention(m, l, scale, s_qkv, true))) return rc;   // rope + append + attention
    if (!(m->skip & 16) && (rc = gemm(m, po, m->att, w.wo, H, AW, UGB_EPI_F32, m->splits_o, m->bn_o))) return rc;
    if (!(m->skip & 1) && (rc = launch_reduce(m, B, m->x, m->xn, RED_O, po, s_o, w.rms2, early_i))) return rc;
    if (!(m->skip & 32) && (rc = gemm(m, m->h, m->xn, w.wgu, 2 * (size_t)c.ffn, H, UGB_EPI_SILU_MUL_BF16, 1, m->bn_gate_up))) return rc;
    if (!(m->skip & 64) && (rc = gemm(m, pd, m->h, w.wdown, H, c.ffn, UGB_EPI_F32, m->splits_down, m->bn_down))) return rc;
  }
  if ((rc = launch_reduce(m, B, m->x, m->xn, RED_DOWN, pd, s_down, m->ln_f, early_i))) return rc;
  return launch_lm_head_argmax(m, true);
}

// Activations for one prefill chunk; allocated once, freed with the model.
int32_t ensure_prefill_workspace(ugb_llama *m) {
  if (m->pf_rows) return UGB_OK;
  const ugb_llama_config &c = m->lc;
  int rows_max = m->pf_rows_max;
  if (m->tp && (size_t)rows_max > m->tp_part_rows) rows_max = (int)m->tp_part_rows;   // the exchange block was sized at creation
  int chunk = rows_max / m->batch;
  if (chunk < 1) chunk = 1;
  if (chunk >= PF_BQ) chunk -= chunk % PF_BQ;     // whole query tiles per chunk
  const size_t rows = (size_t)m->batch * chunk, H = c.hidden, F = c.ffn;
  int32_t rc;
  if ((rc = dmalloc(m, &m->pf_x, rows * H))) return rc;
  if ((rc = dmalloc(m, &m->pf_f32, rows * std::max<size_t>(m->qkv_dim, H)))) return rc;
  if ((rc = dmalloc(m, &m->pf_xn, rows * H))) return rc;
  if ((rc = dmalloc(m, &m->pf_q, rows * H))) return rc;
  if ((rc = dmalloc(m, &m->pf_att, rows * H))) return rc;
  if ((rc = dmalloc(m, &m->pf_h, rows * F))) return rc;
  m->pf_chunk = chunk;
  m->pf_rows = (int)rows;
  return UGB_OK;
}

// One chunk of a prefill: positions c0 .. c0 + tc - 1 of a block of t per sequence, cache positions
// host_pos + c0 onwards.  Rows are ordered (sequence, position).
int32_t enqueue_prefill_chunk(ugb_llama *m, const int *tok, int t, int c0, int tc, bool all_logits) {
  ugb_device *dev = m->dev;
  const ugb_llama_config &c = m->lc;
  cudaStream_t st = dev->stream;
  const int B = m->batch, H = c.hidden, rows = B * tc, AW = c.n_heads * c.head_dim;
  const bool pdl = m->pdl != 0;
  const float scale = powf((float)c.head_dim, -0.5f);   // model.rs:236
  int32_t rc;
  cudaError_t e = ugb_launch(embed_gather_kernel, dim3(rows), dim3(256), 0, st, pdl, m->embed, tok, m->pf_x, H, c.vocab,
                             dev->status_dev, tc, t, c0);
  if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "launch of embed_gather_kernel failed: %s", cudaGetErrorString(e));
  if ((rc = ugb_after_launch(dev, "embed_gather_kernel"))) return rc;
  const int rope_items = ((c.n_heads + c.n_kv_heads) * c.head_dim / 2 + c.n_kv_heads * c.head_dim) / 4;   // 4 pairs / values per thread
  float *po = o_out(m, m->pf_f32), *pd = down_out(m, m->pf_f32);
  for (int l = 0; l < c.layers; ++l) {
    const LayerW &w = m->layers[l];
    __nv_bfloat16 *kc = m->kcache + (size_t)l * m->kv_layer_stride;
    __nv_bfloat16 *vc = m->vcache + (size_t)l * m->kv_layer_stride;
    if ((rc = launch_reduce(m, rows, m->pf_x, m->pf_xn, l == 0 ? RED_NONE : RED_DOWN, pd, l == 0 ? 0 : 1, w.rms1))) return rc;
    if (rows > 64) {
      // qkv projection with the rotation and the cache append in its epilogue: no fp32 round trip, no rope kernel
      ugb_tc_rope_epilogue re;
      re.cos_ = m->cos; re.sin_ = m->sin; re.pos_p = m->pos; re.pos_off = c0; re.t = tc;
      re.n_heads = c.n_heads; re.n_kv = c.n_kv_heads; re.t_max = m->t_max; re.interleaved = c.rope_interleaved;
      re.q_out = m->pf_q; re.kcache = kc; re.vcache = vc;
      if ((rc = gemm_rows(m, rows, m->pf_f32, m->pf_xn, w.wqkv, m->qkv_dim, H, UGB_EPI_ROPE_QKV, 1, 0, &re))) return rc;
    } else {
      if ((rc = gemm_rows(m, rows, m->pf_f32, m->pf_xn, w.wqkv, m->qkv_dim, H, UGB_EPI_F32, 1, 0))) return rc;
      e = ugb_launch(rope_append_kernel, dim3(rows, (rope_items + 255) / 256), dim3(256), 0, st, pdl, m->pf_f32, 1,
                     (size_t)0, m->cos, m->sin, m->pos, m->pf_q, kc, vc, c.n_heads, c.n_kv_heads, c.head_dim, m->t_max,
                     c.rope_interleaved, tc, c0);
      if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "launch of rope_append_kernel failed: %s", cudaGetErrorString(e));
      if ((rc = ugb_after_launch(dev, "rope_append_kernel"))) return rc;
    }
    if (m->pf_att_tc) {
      if ((rc = ugb_prefill_attention_tc(dev, m->pf_q, kc, vc, m->pf_att, B, tc, m->host_pos + c0, c.n_heads, c.n_kv_heads,
                                         m->t_max, scale, m->pf_att_tc == 1))) return rc;
    } else {
      prefill_attention_kernel<<<dim3((tc + PF_BQ - 1) / PF_BQ, c.n_heads, B), 128, 0, st>>>(
          m->pf_q, kc, vc, m->pf_att, tc, m->host_pos + c0, c.n_heads, c.n_kv_heads, m->t_max, scale);
      if ((rc = ugb_after_launch(dev, "prefill_attention_kernel"))) return rc;
    }
    if ((rc = gemm_rows(m, rows, po, m->pf_att, w.wo, H, AW, UGB_EPI_F32, 1, 0))) return rc;
    if ((rc = launch_reduce(m, rows, m->pf_x, m->pf_xn, RED_O, po, 1, w.rms2))) return rc;
    if ((rc = gemm_rows(m, rows, m->pf_h, m->pf_xn, w.wgu, 2 * (size_t)c.ffn, H, UGB_EPI_SILU_MUL_BF16, 1, 0))) return rc;
    if ((rc = gemm_rows(m, rows, pd, m->pf_h, w.wdown, H, c.ffn, UGB_EPI_F32, 1, 0))) return rc;
  }
  // The last down_proj output is folded into the residual stream here (every rank's partial under tensor
  // parallelism), so that what follows -- all-position logits, the last-position step -- sees the final x.
  if ((rc = launch_reduce(m, rows, m->pf_x, m->pf_xn, RED_DOWN, pd, 1, m->ln_f))) return rc;
  if (all_logits) {
    // logits[b, c0 + i, rank's vocabulary slice] for the chunk as one GEMM batched over sequences
    ugb_tc_gemm_args g;
    g.out = m->pf_logits + (size_t)c0 * m->vl; g.a = m->pf_xn; g.b = m->embed + (size_t)m->tp_rank * m->vl * H;
    g.batch = (size_t)B; g.m = (size_t)tc; g.n = (size_t)m->vl; g.k = (size_t)H;
    g.a_batch = (long long)tc * H; g.b_batch = 0; g.c_batch = (long long)t * m->vl; g.b_is_nk = true;
    g.epi = UGB_EPI_F32; g.splits = 1; g.bn = 0; g.b_static = true; g.pdl = pdl;
    rc = ugb_tc_gemm(dev, g);
    if (rc == UGB_ERR_UNSUPPORTED) return ugb_fail(dev, rc, "prefill lm_head GEMM does not meet the tensor-core kernel's shape rules");
    if (rc) return rc;
  }
  return UGB_OK;
}

bool ends_with(const std::string &s, const char *suffix) {
  const size_t n = strlen(suffix);
  return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

}  // namespace

extern "C" {

int32_t ugb_llama_create(ugb_device *dev, const ugb_llama_config *cfg, int32_t batch, int32_t t_max,
                         ugb_llama **out) {
  return ugb_llama_create_tp(dev, cfg, batch, t_max, 0, 0, out);
}

int32_t ugb_llama_create_tp(ugb_device *dev, const ugb_llama_config *cfg, int32_t batch, int32_t t_max,
                            int32_t tp_rank, int32_t tp_size, ugb_llama **out) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, cfg && out, UGB_ERR_INVALID, "ugb_llama_create: null argument");
  *out = nullptr;
  const ugb_llama_config &g = *cfg;
  const bool tp = tp_size >= 1;          // tp_size 0: single rank on the plain kernels
  const int n_rank = tp ? tp_size : 1;
  UGB_REQUIRE(dev, n_rank <= TP_MAX && tp_rank >= 0 && tp_rank < n_rank, UGB_ERR_INVALID,
              "tensor-parallel rank %d of %d (at most %d ranks)", tp_rank, n_rank, TP_MAX);
  UGB_REQUIRE(dev, g.n_heads > 0 && g.n_kv_heads > 0 && g.ffn > 0 && g.vocab > 0, UGB_ERR_INVALID,
              "ugb_llama_create: non-positive dimension");
  UGB_REQUIRE(dev, g.n_heads % n_rank == 0 && (g.n_kv_heads % n_rank == 0 || n_rank % g.n_kv_heads == 0) &&
                   g.ffn % (8 * n_rank) == 0 && g.vocab % (8 * n_rank) == 0, UGB_ERR_UNSUPPORTED,
              "%d ranks do not divide heads %d / KV heads %d / ffn %d / vocab %d evenly", n_rank, g.n_heads,
              g.n_kv_heads, g.ffn, g.vocab);
  ugb_llama_config c = g;                // local share
  c.n_heads = g.n_heads / n_rank;
  c.n_kv_heads = g.n_kv_heads >= n_rank ? g.n_kv_heads / n_rank : 1;
  c.ffn = g.ffn / n_rank;
  c.hidden = g.hidden;
  UGB_REQUIRE(dev, c.hidden > 0 && c.layers > 0 && c.n_heads > 0 && c.n_kv_heads > 0 && c.ffn > 0 && c.vocab > 0,
              UGB_ERR_INVALID, "ugb_llama_create: non-positive dimension");
  UGB_REQUIRE(dev, c.head_dim == ATT_HD, UGB_ERR_UNSUPPORTED, "head_dim %d: the decode attention kernel is built for 64", c.head_dim);
  UGB_REQUIRE(dev, g.n_heads * g.head_dim == g.hidden, UGB_ERR_SHAPE, "n_heads * head_dim != hidden");
  UGB_REQUIRE(dev, c.n_heads % c.n_kv_heads == 0 && c.n_heads / c.n_kv_heads <= ATT_GROUP, UGB_ERR_UNSUPPORTED,
              "query heads per KV head must divide evenly and be <= %d", ATT_GROUP);
  UGB_REQUIRE(dev, c.hidden % 8 == 0 && c.hidden <= 8192 && c.ffn % 8 == 0 && c.vocab % 8 == 0, UGB_ERR_UNSUPPORTED,
              "hidden, ffn and vocab must be multiples of 8 (hidden <= 8192)");
  UGB_REQUIRE(dev, batch >= 1 && batch <= 128, UGB_ERR_UNSUPPORTED, "batch %d: the decode kernels take 1..128 sequences", batch);
  UGB_REQUIRE(dev, t_max >= 1 && t_max <= c.max_pos, UGB_ERR_INVALID, "t_max %d outside 1..max_pos %d", t_max, c.max_pos);
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));

  ugb_llama *m = new ugb_llama();
  m->dev = dev;
  m->cfg = g;
  m->lc = c;
  m->tp = tp;
  m->tp_rank = tp_rank;
  m->tp_size = n_rank;
  m->timeouts_at_create = dev->wait_timeouts;
  m->q0 = tp_rank * c.n_heads;
  m->kv0 = tp_rank * g.n_kv_heads / n_rank;
  m->vl = g.vocab / n_rank;
  m->batch = batch;
  m->t_max = (t_max + 15) / 16 * 16;
  m->qkv_dim = (c.n_heads + 2 * c.n_kv_heads) * c.head_dim;
  m->layers.resize(c.layers);
  const size_t H = c.hidden, F = c.ffn, B = batch;
  int32_t rc = UGB_OK;
#define TRY(e) do { if ((rc = (e)) != UGB_OK) { ugb_llama_destroy(m); return rc; } } while (0)
  for (auto &w : m->layers) {
    TRY(dmalloc(m, &w.wqkv, (size_t)m->qkv_dim * H));
    TRY(dmalloc(m, &w.wo, H * (size_t)c.n_heads * c.head_dim));
    TRY(dmalloc(m, &w.wgu, 2 * F * H));
    TRY(dmalloc(m, &w.wdown, H * F));
    TRY(dmalloc(m, &w.rms1, H));
    TRY(dmalloc(m, &w.rms2, H));
  }
  TRY(dmalloc(m, &m->embed, (size_t)g.vocab * H));
  TRY(dmalloc(m, &m->ln_f, H));
  const size_t half = c.head_dim / 2;
  TRY(dmalloc(m, &m->cos, (size_t)c.max_pos * half));
  TRY(dmalloc(m, &m->sin, (size_t)c.max_pos * half));
  m->kv_layer_stride = B * c.n_kv_heads * (size_t)m->t_max * c.head_dim;
  TRY(dmalloc(m, &m->kcache, m->kv_layer_stride * c.layers, true));
  TRY(dmalloc(m, &m->vcache, m->kv_layer_stride * c.layers, true));
  TRY(dmalloc(m, &m->x, B * H));
  TRY(dmalloc(m, &m->xn, B * H));
  TRY(dmalloc(m, &m->q, B * H));
  TRY(dmalloc(m, &m->att, B * H));
  TRY(dmalloc(m, &m->h, B * F));
  const size_t widest = std::max<size_t>(m->qkv_dim, H);
  m->part_elems = 8 * B * widest;    // up to 8 split-K partials
  TRY(dmalloc(m, &m->part, m->part_elems));
  TRY(dmalloc(m, &m->logits, B * (size_t)m->vl));
  const size_t slots = B * c.n_kv_heads * 8;   // up to 8 attention slices
  TRY(dmalloc(m, &m->att_po, slots * ATT_GROUP * ATT_HD));
  TRY(dmalloc(m, &m->att_pml, slots * ATT_GROUP * 2));
  TRY(dmalloc(m, &m->att_cnt, B * c.n_kv_heads, true));
  TRY(dmalloc(m, &m->tok, B, true));
  TRY(dmalloc(m, &m->next, B, true));
  TRY(dmalloc(m, &m->pos, 1, true));
  {
    // A (sequence, KV head) pair is one attention CTA per KV slice; with few sequences (a rank's share of a batch that
    // is split over several GPUs) the cache is cut into slices so that up to about 256 CTAs stream it, as at batch 64.
    // Measured at 2048+ positions (step time in ms, slices 1 / 2 / 4 / 8): 32 sequences 1.47 / 1.35 / 1.45 / -,
    // 16 sequences - / 1.29 / 1.21 / 1.42, 8 sequences - / 1.29 / 1.17 / 1.19: more than 4 slices cost more in
    // start-up and merging than they gain.  The ring holds 5 sub-tiles per warp (80 KiB per CTA, two CTAs per SM):
    // step time at 64 sequences with 3 / 4 / 5 / 6 of them 1.535 / 1.529 / 1.521 / 1.531 ms; 8 of them for a
    // grid of one CTA per SM (8 sequences) 1.166 against 1.140 ms with 5.
    const int pairs = batch * c.n_kv_heads;
    int splits = (256 + pairs - 1) / pairs;
    m->att_splits = splits < 1 ? 1 : (splits > 4 ? 4 : splits);
  }
  if (tp) {
    // exchange block: header | o_proj partials | down_proj partials | argmax pairs.  Partial buffers hold
    // up to 8 split-K partials of a decode step or one partial of a prefill chunk, whichever is larger.
    m->tp_part_rows = std::max<size_t>(8 * B, (size_t)m->pf_rows_max);
    const size_t part_bytes = m->tp_part_rows * H * sizeof(float);
    m->tp_off_o = 256;
    m->tp_off_down = m->tp_off_o + part_bytes;
    m->tp_off_pairs = m->tp_off_down + part_bytes;
    m->tp_block_bytes = m->tp_off_pairs + ((B * sizeof(float2) + 255) / 256) * 256;
    unsigned char *blk = nullptr;
    TRY(dmalloc(m, &blk, m->tp_block_bytes));
    if (cudaMemsetAsync(blk, 0, m->tp_block_bytes, dev->stream) != cudaSuccess) {
      ugb_fail(dev, UGB_ERR_CUDA, "clearing the exchange block failed");
      ugb_llama_destroy(m);
      return UGB_ERR_CUDA;
    }
    m->tp_block = blk;
    m->tp_peer[tp_rank] = blk;
    m->tp_ready = n_rank == 1;
    if (n_rank > 1) {
      // a rank's projections are 1 / n_rank of the work: fewer split-K partials to fetch from the peers (the KV
      // slices above already follow the rank's own number of (sequence, KV head) pairs)
      m->splits_qkv = 7;
      m->splits_o = 2;
      m->splits_down = 2;
      m->bn_qkv = 64;
      m->bn_o = 64;
    }
  }
  // rope tables, model.rs:278-295: theta_i = 1 / theta^(i/d) in f32 on the host
  {
    std::vector<float> inv(half);
    for (size_t i = 0; i < half; ++i) inv[i] = 1.0f / powf(c.rope_theta, (float)(2 * i) / (float)c.head_dim);
    float *inv_d = nullptr;
    TRY(dmalloc(m, &inv_d, half));
    if (cudaMemcpyAsync(inv_d, inv.data(), half * 4, cudaMemcpyHostToDevice, dev->stream) != cudaSuccess ||
        cudaStreamSynchronize(dev->stream) != cudaSuccess) {
      ugb_fail(dev, UGB_ERR_CUDA, "rope table upload failed");
      ugb_llama_destroy(m);
      return UGB_ERR_CUDA;
    }
    const int n = c.max_pos * (int)half;
    rope_table_kernel<<<(n + 255) / 256, 256, 0, dev->stream>>>(inv_d, m->cos, m->sin, c.max_pos, (int)half);
    TRY(ugb_after_launch(dev, "rope_table_kernel"));
  }
  if (cudaFuncSetAttribute(decode_attention_kernel_t<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_ring_bytes(2)) != cudaSuccess ||
      cudaFuncSetAttribute(decode_attention_kernel_t<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_ring_bytes(3)) != cudaSuccess ||
      cudaFuncSetAttribute(decode_attention_kernel_t<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_ring_bytes(4)) != cudaSuccess ||
      cudaFuncSetAttribute(decode_attention_kernel_t<5>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_ring_bytes(5)) != cudaSuccess ||
      cudaFuncSetAttribute(decode_attention_kernel_t<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_ring_bytes(6)) != cudaSuccess) {
    ugb_fail(dev, UGB_ERR_CUDA, "cudaFuncSetAttribute(decode_attention_kernel) failed");
    ugb_llama_destroy(m);
    return UGB_ERR_CUDA;
  }
  if (cudaFuncSetAttribute(decode_attention_kernel_t<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_dyn_smem(2, true)) != cudaSuccess ||
      cudaFuncSetAttribute(decode_attention_kernel_t<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_dyn_smem(3, true)) != cudaSuccess ||
      cudaFuncSetAttribute(decode_attention_kernel_t<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_dyn_smem(4, true)) != cudaSuccess ||
      cudaFuncSetAttribute(decode_attention_kernel_t<5, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_dyn_smem(5, true)) != cudaSuccess ||
      cudaFuncSetAttribute(decode_attention_kernel_t<6, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, att_dyn_smem(6, true)) != cudaSuccess) {
    ugb_fail(dev, UGB_ERR_CUDA, "cudaFuncSetAttribute(decode_attention_kernel, TMA) failed");
    ugb_llama_destroy(m);
    return UGB_ERR_CUDA;
  }
  {   // per-layer maps over the caches for the TMA variant: dims {d, position, sequence x kv head}, box 16 positions
    const uint64_t dims[3] = {(uint64_t)c.head_dim, (uint64_t)m->t_max, (uint64_t)B * c.n_kv_heads};
    const uint64_t strides[2] = {(uint64_t)c.head_dim, (uint64_t)m->t_max * c.head_dim};
    const uint32_t box[3] = {(uint32_t)c.head_dim, (uint32_t)ATT_SUB, 1};
    m->att_kmap.resize(c.layers);
    m->att_vmap.resize(c.layers);
    for (int l = 0; l < c.layers; ++l) {
      TRY(ugb_tc_encode_bf16(dev, &m->att_kmap[l], m->kcache + (size_t)l * m->kv_layer_stride, 3, dims, strides, box));
      TRY(ugb_tc_encode_bf16(dev, &m->att_vmap[l], m->vcache + (size_t)l * m->kv_layer_stride, 3, dims, strides, box));
    }
  }
#undef TRY
  *out = m;
  return UGB_OK;
}

int32_t ugb_llama_destroy(ugb_llama *m) {
  if (!m) return UGB_ERR_INVALID;
  cudaSetDevice(m->dev->ordinal);
  cudaStreamSynchronize(m->dev->stream);
  if (m->graph) cudaGraphExecDestroy(m->graph);
  for (int r = 0; r < m->tp_size; ++r)
    if (r != m->tp_rank && m->tp_peer[r]) cudaIpcCloseMemHandle(m->tp_peer[r]);
  for (void *p : m->allocs) cudaFree(p);
  if (m->pf_logits) cudaFree(m->pf_logits);
  delete m;
  return UGB_OK;
}

int32_t ugb_llama_load_weight(ugb_llama *m, const char *name, const ugb_slice *w) {
  if (!m) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, name && w, UGB_ERR_INVALID, "ugb_llama_load_weight: null argument");
  UGB_REQUIRE(dev, w->dev == dev, UGB_ERR_INVALID, "%s: slice belongs to another device", name);
  const ugb_llama_config &c = m->cfg;
  const ugb_llama_config &lc = m->lc;
  const size_t H = c.hidden, F = c.ffn, KV = (size_t)c.n_kv_heads * c.head_dim, D = c.head_dim;
  const size_t QL = (size_t)lc.n_heads * D, KVL = (size_t)lc.n_kv_heads * D, FL = lc.ffn;   // this rank's widths
  const size_t q_row0 = (size_t)m->q0 * D, kv_row0 = (size_t)m->kv0 * D, f0 = (size_t)m->tp_rank * FL;
  const std::string s(name);
  m->loaded++;
  if (s == "model.embed_tokens.weight") return put_matrix(m, w, m->embed, c.vocab, H, H, name);
  if (s == "model.norm.weight") return put_vector(m, w, m->ln_f, H, name);
  const std::string pre = "model.layers.";
  if (s.compare(0, pre.size(), pre) == 0) {
    const size_t dot = s.find('.', pre.size());
    if (dot != std::string::npos) {
      const int l = atoi(s.substr(pre.size(), dot - pre.size()).c_str());
      UGB_REQUIRE(dev, l >= 0 && l < c.layers, UGB_ERR_INVALID, "%s: layer index out of range", name);
      LayerW &L = m->layers[l];
      if (ends_with(s, ".input_layernorm.weight")) return put_vector(m, w, L.rms1, H, name);
      if (ends_with(s, ".post_attention_layernorm.weight")) return put_vector(m, w, L.rms2, H, name);
      // column-parallel: rows of q/k/v/gate/up; row-parallel: columns of o/down
      if (ends_with(s, ".self_attn.q_proj.weight")) return put_sub(m, w, L.wqkv, H, H, q_row0, QL, 0, H, H, name);
      if (ends_with(s, ".self_attn.k_proj.weight")) return put_sub(m, w, L.wqkv + QL * H, KV, H, kv_row0, KVL, 0, H, H, name);
      if (ends_with(s, ".self_attn.v_proj.weight")) return put_sub(m, w, L.wqkv + (QL + KVL) * H, KV, H, kv_row0, KVL, 0, H, H, name);
      if (ends_with(s, ".self_attn.o_proj.weight")) return put_sub(m, w, L.wo, H, H, 0, H, q_row0, QL, QL, name);
      if (ends_with(s, ".mlp.gate_proj.weight")) return put_sub(m, w, L.wgu, F, H, f0, FL, 0, H, 2 * H, name);
      if (ends_with(s, ".mlp.up_proj.weight")) return put_sub(m, w, L.wgu + H, F, H, f0, FL, 0, H, 2 * H, name);
      if (ends_with(s, ".mlp.down_proj.weight")) return put_sub(m, w, L.wdown, H, F, 0, H, f0, FL, FL, name);
    }
  }
  m->loaded--;
  return ugb_fail(dev, UGB_ERR_INVALID, "unknown weight name %s", name);
}

int32_t ugb_llama_set_option(ugb_llama *m, const char *key, int32_t value) {
  if (!m || !key) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  const std::string k(key);
  if (k == "measure_skip_mask") {   // measurement aid: results of a step are meaningless while it is non-zero
    m->skip = value;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return UGB_OK;
  }
  if (k == "pdl") {
    m->pdl = value != 0;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return UGB_OK;
  }
  if (k == "gemm_smem_kib") {
    UGB_REQUIRE(dev, value == 0 || (value >= 32 && value <= 220), UGB_ERR_INVALID, "option gemm_smem_kib: %d outside 32..220 (0 = no cap)", value);
    m->gemm_smem_kib = value;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return UGB_OK;
  }
  if (k == "step_kernel") {
    UGB_REQUIRE(dev, value == 0 || value == 1, UGB_ERR_INVALID, "option step_kernel: %d is not 0 or 1", value);
    m->step_kernel = value;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    m->warmed = false;            // the kernel's attributes are set by its first, eager launch
    if (value && !m->tp && m->batch <= 64) return ensure_step_kernel(m);
    return UGB_OK;
  }
  if (k == "step_tune") {         // measurement aid of the persistent step kernel; non-zero values give wrong results
    m->step.tune = value;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return UGB_OK;
  }
  if (k == "step_profile") {      // measurement aid: barrier time stamps of the persistent step kernel (UGB_LLAMA_STEP_PROFILE)
    UGB_REQUIRE(dev, m->step_ready, UGB_ERR_INVALID, "option step_profile: set step_kernel first");
    if (value && !m->step.prof) {
      unsigned long long *buf = nullptr;
      if (int32_t rc = dmalloc(m, &buf, (size_t)4 * UGB_STEP_PROF_SLOTS, true)) return rc;
      m->step.prof = buf;
    }
    if (!value) m->step.prof = nullptr;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return UGB_OK;
  }
  if (k == "att_early") {
    m->att_early = value != 0;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return UGB_OK;
  }
  if (k == "gemm_profile") {      // measurement aid: time stamps inside the decode projections (UGB_LLAMA_GEMM_PROFILE)
    if (value && !m->gemm_prof) {
      unsigned long long *buf = nullptr;
      if (int32_t rc = dmalloc(m, &buf, (size_t)5 * UGB_TC_PROF_SLOTS, true)) return rc;
      m->gemm_prof = buf;
    }
    if (!value) m->gemm_prof = nullptr;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return UGB_OK;
  }
  if (k == "gate_up_pair") {
    m->gate_up_pair = value != 0;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    m->warmed = false;
    return UGB_OK;
  }
  if (k == "att_cluster") {
    m->att_cluster = value != 0;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return UGB_OK;
  }
  if (k == "att_tma") {
    m->att_tma = value != 0;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return UGB_OK;
  }
  if (k == "prefill_attention_tc") {
    UGB_REQUIRE(dev, value >= 0 && value <= 2, UGB_ERR_INVALID, "option prefill_attention_tc: %d outside 0..2", value);
    m->pf_att_tc = value;
    return UGB_OK;
  }
  if (k == "prefill_rows") {
    UGB_REQUIRE(dev, value >= 64 && value <= 65536, UGB_ERR_INVALID, "option prefill_rows: %d outside 64..65536", value);
    UGB_REQUIRE(dev, m->pf_rows == 0, UGB_ERR_INVALID, "option prefill_rows must be set before the first prefill");
    m->pf_rows_max = value;
    return UGB_OK;
  }
  if (k.compare(0, 3, "bn_") == 0) {
    UGB_REQUIRE(dev, value == 64 || value == 80 || value == 96 || value == 128 || value == 160 || value == 256, UGB_ERR_INVALID,
                "option %s: tile width must be 64, 80, 96, 128, 160 or 256", key);
    if (k == "bn_qkv") m->bn_qkv = value;
    else if (k == "bn_o") m->bn_o = value;
    else if (k == "bn_gate_up") m->bn_gate_up = value;
    else if (k == "bn_down") m->bn_down = value;
    else if (k == "bn_lm_head") m->bn_lm_head = value;
    else return ugb_fail(dev, UGB_ERR_INVALID, "unknown option %s", key);
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    m->warmed = false;   // a tile width used for the first time sets a kernel attribute: run one step eagerly
    return UGB_OK;
  }
  UGB_REQUIRE(dev, value >= 1 && value <= 8, UGB_ERR_INVALID, "option %s: value %d outside 1..8", key, value);
  if (k == "splits_qkv") m->splits_qkv = value;
  else if (k == "splits_o") m->splits_o = value;
  else if (k == "splits_down") m->splits_down = value;
  else if (k == "att_splits") m->att_splits = value;
  else if (k == "att_stages") m->att_stages = value < 2 ? 2 : (value > 6 ? 6 : value);
  else return ugb_fail(dev, UGB_ERR_INVALID, "unknown option %s", key);
  if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
  return UGB_OK;
}

int32_t ugb_llama_reset(ugb_llama *m, int32_t pos) {
  if (!m) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, pos >= 0 && pos < m->t_max, UGB_ERR_INVALID, "reset position %d outside 0..%d", pos, m->t_max - 1);
  UGB_CUDA(dev, cudaMemcpyAsync(m->pos, &pos, 4, cudaMemcpyHostToDevice, dev->stream));
  UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  m->host_pos = pos;
  return UGB_OK;
}

int32_t ugb_llama_position(const ugb_llama *m) { return m ? m->host_pos : -1; }

int32_t ugb_llama_decode(ugb_llama *m, const ugb_slice *tokens, int32_t n_steps) {
  if (!m) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, n_steps >= 1, UGB_ERR_INVALID, "n_steps must be >= 1");
  UGB_REQUIRE(dev, tokens == nullptr || n_steps == 1, UGB_ERR_INVALID, "explicit tokens feed exactly one step");
  UGB_REQUIRE(dev, m->host_pos + n_steps <= m->t_max && m->host_pos + n_steps <= m->cfg.max_pos, UGB_ERR_SHAPE,
              "decode of %d steps from position %d exceeds the KV cache (%d positions)", n_steps, m->host_pos, m->t_max);
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  if (int32_t in_step = tp_in_step(m)) return in_step;
  if (m->step_ready && m->step_timeouts != dev->wait_timeouts) {
    // a wait gave up since the barrier words were last known good (an aborted step leaves them half counted)
    UGB_CUDA(dev, cudaMemsetAsync(m->step.sync, 0, 4 * sizeof(unsigned), dev->stream));
    m->step_timeouts = dev->wait_timeouts;
  }
  if (tokens) {
    UGB_SLICE(dev, tokens, UGB_I32, (size_t)m->batch);
    UGB_CUDA(dev, cudaMemcpyAsync(m->next, tokens->ptr, (size_t)m->batch * 4, cudaMemcpyDeviceToDevice, dev->stream));
  }
  int32_t rc;
  for (int s = 0; s < n_steps; ++s) {
    if (!m->warmed) {
      // first step runs eagerly: it sets kernel attributes, which must not happen inside a capture
      if ((rc = enqueue_step(m, m->next))) return rc;
      m->warmed = true;
    } else {
      if (!m->graph) {
        cudaGraph_t g = nullptr;
        const uint64_t before = dev->launches;
        UGB_CUDA(dev, cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
        rc = enqueue_step(m, m->next);
        cudaError_t e = cudaStreamEndCapture(dev->stream, &g);
        m->graph_nodes = (int)(dev->launches - before);
        dev->launches = before;
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "stream capture failed: %s", cudaGetErrorString(e));
        e = cudaGraphInstantiate(&m->graph, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
      }
      UGB_CUDA(dev, cudaGraphLaunch(m->graph, dev->stream));
      dev->launches += (uint64_t)m->graph_nodes;
    }
    m->host_pos++;
  }
  return UGB_OK;
}

int32_t ugb_llama_prefill(ugb_llama *m, const ugb_slice *tokens, int32_t t, int32_t all_logits) {
  if (!m) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, t >= 1, UGB_ERR_INVALID, "prefill of %d positions", t);
  UGB_REQUIRE(dev, tokens != nullptr, UGB_ERR_INVALID, "ugb_llama_prefill: null tokens");
  UGB_SLICE(dev, tokens, UGB_I32, (size_t)m->batch * t);
  UGB_REQUIRE(dev, m->host_pos + t <= m->t_max && m->host_pos + t <= m->cfg.max_pos, UGB_ERR_SHAPE,
              "prefill of %d positions from position %d exceeds the KV cache (%d positions)", t, m->host_pos, m->t_max);
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  if (int32_t in_step = tp_in_step(m)) return in_step;
  const ugb_llama_config &c = m->cfg;
  const size_t H = c.hidden;
  int32_t rc;
  if ((rc = ensure_prefill_workspace(m))) return rc;
  if (all_logits) {
    const size_t need = (size_t)m->batch * t * m->vl;
    if (need > m->pf_logits_cap) {
      UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
      if (m->pf_logits) { cudaFree(m->pf_logits); m->pf_logits = nullptr; m->pf_logits_cap = 0; }
      void *v = nullptr;
      UGB_CUDA(dev, cudaMalloc(&v, need * sizeof(float)));
      m->pf_logits = (float *)v;
      m->pf_logits_cap = need;
    }
    m->pf_logits_t = t;
  }
  const int *tok = (const int *)tokens->ptr;
  int tc = 0;
  for (int c0 = 0; c0 < t; c0 += tc) {
    tc = std::min(m->pf_chunk, t - c0);
    if ((rc = enqueue_prefill_chunk(m, tok, t, c0, tc, all_logits != 0))) return rc;
  }
  // Last position of every sequence -> the decode-shaped buffers (x already holds the last down_proj
  // output), final norm, lm_head, greedy choice.
  UGB_CUDA(dev, cudaMemcpy2DAsync(m->x, H * 4, m->pf_x + (size_t)(tc - 1) * H, (size_t)tc * H * 4, H * 4, m->batch,
                                  cudaMemcpyDeviceToDevice, dev->stream));
  if ((rc = launch_reduce(m, m->batch, m->x, m->xn, RED_NONE, m->part, 0, m->ln_f))) return rc;
  const int last = m->host_pos + t - 1;     // the argmax kernel advances the device-side position by one
  UGB_CUDA(dev, cudaMemcpyAsync(m->pos, &last, 4, cudaMemcpyHostToDevice, dev->stream));
  if ((rc = launch_lm_head_argmax(m, false))) return rc;
  m->host_pos += t;
  return UGB_OK;
}

int32_t ugb_llama_read(ugb_llama *m, int32_t what, void *host_dst, size_t len) {
  if (!m) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, host_dst != nullptr, UGB_ERR_INVALID, "ugb_llama_read: null destination");
  const void *src = nullptr;
  size_t n = 0, es = 4;
  switch (what) {
    case UGB_LLAMA_LOGITS: src = m->logits; n = (size_t)m->batch * m->vl; break;
    case UGB_LLAMA_NEXT_TOKENS: src = m->next; n = (size_t)m->batch; break;
    case UGB_LLAMA_HIDDEN: src = m->x; n = (size_t)m->batch * m->cfg.hidden; break;
    case UGB_LLAMA_PREFILL_LOGITS:
      UGB_REQUIRE(dev, m->pf_logits && m->pf_logits_t > 0, UGB_ERR_INVALID, "no all-position logits: run ugb_llama_prefill with all_logits first");
      src = m->pf_logits; n = (size_t)m->batch * m->pf_logits_t * m->vl; break;
    case UGB_LLAMA_STEP_PROFILE: {
      UGB_REQUIRE(dev, m->step_ready && m->step.prof, UGB_ERR_INVALID, "no step profile: set options step_kernel and step_profile first");
      n = (size_t)4 * UGB_STEP_PROF_SLOTS;
      UGB_REQUIRE(dev, len == n, UGB_ERR_SHAPE, "ugb_llama_read: destination holds %zu elements, %zu expected", len, n);
      std::vector<unsigned long long> raw(n);
      UGB_CUDA(dev, cudaMemcpyAsync(raw.data(), m->step.prof, n * 8, cudaMemcpyDeviceToHost, dev->stream));
      UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
      float *out = (float *)host_dst;                 // microseconds since CTA 0's first stamp; 0 where nothing was recorded
      for (size_t i = 0; i < n; ++i) out[i] = raw[i] ? (float)((double)(raw[i] - raw[0]) * 1e-3) : 0.f;
      return UGB_OK;
    }
    case UGB_LLAMA_GEMM_PROFILE: {
      UGB_REQUIRE(dev, m->gemm_prof, UGB_ERR_INVALID, "no projection profile: set option gemm_profile first");
      n = (size_t)5 * UGB_TC_PROF_SLOTS;
      UGB_REQUIRE(dev, len == n, UGB_ERR_SHAPE, "ugb_llama_read: destination holds %zu elements, %zu expected", len, n);
      std::vector<unsigned long long> raw(n);
      UGB_CUDA(dev, cudaMemcpyAsync(raw.data(), m->gemm_prof, n * 8, cudaMemcpyDeviceToHost, dev->stream));
      UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
      float *out = (float *)host_dst;   // microseconds after the projection's own dependency wait returned; 0 where nothing was recorded
      for (size_t i = 0; i < n; ++i) {
        const unsigned long long dep = raw[i / UGB_TC_PROF_SLOTS * UGB_TC_PROF_SLOTS + UGB_TC_PROF_DEP];
        out[i] = raw[i] ? (float)(((double)raw[i] - (double)dep) * 1e-3) : 0.f;
      }
      return UGB_OK;
    }
    default: return ugb_fail(dev, UGB_ERR_INVALID, "ugb_llama_read: unknown selector %d", what);
  }
  UGB_REQUIRE(dev, len == n, UGB_ERR_SHAPE, "ugb_llama_read: destination holds %zu elements, %zu expected", len, n);
  UGB_CUDA(dev, cudaMemcpyAsync(host_dst, src, n * es, cudaMemcpyDeviceToHost, dev->stream));
  UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return UGB_OK;
}

int32_t ugb_llama_read_kv(ugb_llama *m, int32_t layer, int32_t which, void *host_dst, size_t len) {
  if (!m) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, layer >= 0 && layer < m->cfg.layers && (which == 0 || which == 1) && host_dst, UGB_ERR_INVALID,
              "ugb_llama_read_kv: bad argument");
  UGB_REQUIRE(dev, len == m->kv_layer_stride, UGB_ERR_SHAPE, "ugb_llama_read_kv: destination holds %zu elements, %zu expected",
              len, m->kv_layer_stride);
  const __nv_bfloat16 *src = (which == 0 ? m->kcache : m->vcache) + (size_t)layer * m->kv_layer_stride;
  UGB_CUDA(dev, cudaMemcpyAsync(host_dst, src, len * 2, cudaMemcpyDeviceToHost, dev->stream));
  UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return UGB_OK;
}

int32_t ugb_llama_time_kernel(ugb_llama *m, int32_t which, int32_t iters, float *ms_per_pass) {
  if (!m) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, ms_per_pass && iters >= 1, UGB_ERR_INVALID, "ugb_llama_time_kernel: bad argument");
  UGB_REQUIRE(dev, m->host_pos >= 1, UGB_ERR_INVALID, "ugb_llama_time_kernel: the cache is empty");
  const ugb_llama_config &c = m->lc;
  const int H = c.hidden, AW = c.n_heads * c.head_dim;
  const float scale = powf((float)c.head_dim, -0.5f);
  int32_t rc = UGB_OK;
  // the kernels read the device-side position; during timing it must name the last cached position
  const int last = m->host_pos - 1;
  UGB_CUDA(dev, cudaMemcpyAsync(m->pos, &last, 4, cudaMemcpyHostToDevice, dev->stream));
  for (int it = -1; it < iters && rc == UGB_OK; ++it) {    // it == -1: untimed warm-up pass
    if (it == 0) UGB_CUDA(dev, cudaEventRecord(dev->ev_begin, dev->stream));
    for (int l = 0; l < c.layers && rc == UGB_OK; ++l) {
      const LayerW &w = m->layers[(m->skip & 256) ? 0 : l];   // bit 8: reuse layer 0 (weights stay in L2)
      switch (which) {
        case UGB_LLAMA_K_QKV: rc = gemm(m, m->part, m->xn, w.wqkv, m->qkv_dim, H, UGB_EPI_F32, m->splits_qkv, m->bn_qkv); break;
        case UGB_LLAMA_K_ATTENTION: {
          rc = launch_attention(m, l, scale, ugb_tc_gemm_effective_splits(H, m->splits_qkv), false);
          break;
        }
        case UGB_LLAMA_K_O: rc = gemm(m, m->part, m->att, w.wo, H, AW, UGB_EPI_F32, m->splits_o, m->bn_o); break;
        case UGB_LLAMA_K_GATE_UP: rc = gemm(m, m->h, m->xn, w.wgu, 2 * (size_t)c.ffn, H, UGB_EPI_SILU_MUL_BF16, 1, m->bn_gate_up); break;
        case UGB_LLAMA_K_DOWN: rc = gemm(m, m->part, m->h, w.wdown, H, c.ffn, UGB_EPI_F32, m->splits_down, m->bn_down); break;
        case UGB_LLAMA_K_LM_HEAD:
          if (l == 0) rc = gemm(m, m->logits, m->xn, m->embed + (size_t)m->tp_rank * m->vl * H, (size_t)m->vl, H, UGB_EPI_F32, 1, m->bn_lm_head);
          break;
        default: rc = ugb_fail(dev, UGB_ERR_INVALID, "ugb_llama_time_kernel: unknown kernel %d", which);
      }
    }
  }
  const int cur = m->host_pos;
  cudaMemcpyAsync(m->pos, &cur, 4, cudaMemcpyHostToDevice, dev->stream);
  if (rc) return rc;
  UGB_CUDA(dev, cudaEventRecord(dev->ev_end, dev->stream));
  UGB_CUDA(dev, cudaEventSynchronize(dev->ev_end));
  float ms = 0.f;
  UGB_CUDA(dev, cudaEventElapsedTime(&ms, dev->ev_begin, dev->ev_end));
  *ms_per_pass = ms / (float)iters;
  return UGB_OK;
}

int32_t ugb_llama_kv_positions(const ugb_llama *m) { return m ? m->t_max : -1; }

int32_t ugb_llama_tp_info(const ugb_llama *m, int32_t *tp_rank, int32_t *tp_size, int32_t *vocab_local,
                          int32_t *vocab_offset, int32_t *kv_heads_local) {
  if (!m) return UGB_ERR_INVALID;
  if (tp_rank) *tp_rank = m->tp_rank;
  if (tp_size) *tp_size = m->tp_size;
  if (vocab_local) *vocab_local = m->vl;
  if (vocab_offset) *vocab_offset = m->tp_rank * m->vl;
  if (kv_heads_local) *kv_heads_local = m->lc.n_kv_heads;
  return UGB_OK;
}

int32_t ugb_llama_tp_export(ugb_llama *m, void *handle_out, size_t handle_bytes) {
  if (!m) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, m->tp && m->tp_block, UGB_ERR_INVALID, "ugb_llama_tp_export: not a tensor-parallel model");
  UGB_REQUIRE(dev, handle_out && handle_bytes == sizeof(cudaIpcMemHandle_t), UGB_ERR_INVALID,
              "ugb_llama_tp_export: the handle buffer must hold %zu bytes", sizeof(cudaIpcMemHandle_t));
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  UGB_CUDA(dev, cudaStreamSynchronize(dev->stream));      // the block has been cleared before anyone maps it
  cudaIpcMemHandle_t h;
  UGB_CUDA(dev, cudaIpcGetMemHandle(&h, m->tp_block));
  memcpy(handle_out, &h, sizeof(h));
  return UGB_OK;
}

int32_t ugb_llama_tp_connect(ugb_llama *m, const void *handles, size_t handle_bytes, int32_t n_ranks) {
  if (!m) return UGB_ERR_INVALID;
  ugb_device *dev = m->dev;
  UGB_REQUIRE(dev, m->tp, UGB_ERR_INVALID, "ugb_llama_tp_connect: not a tensor-parallel model");
  UGB_REQUIRE(dev, handles && handle_bytes == sizeof(cudaIpcMemHandle_t) && n_ranks == m->tp_size, UGB_ERR_INVALID,
              "ugb_llama_tp_connect: expected %d handles of %zu bytes", m->tp_size, sizeof(cudaIpcMemHandle_t));
  UGB_REQUIRE(dev, !m->tp_ready || m->tp_size == 1, UGB_ERR_INVALID, "ugb_llama_tp_connect: already connected");
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  for (int r = 0; r < m->tp_size; ++r) {
    if (r == m->tp_rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char *)handles + (size_t)r * handle_bytes, sizeof(h));
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return ugb_fail(dev, UGB_ERR_CUDA, "mapping the exchange block of rank %d failed: %s", r, cudaGetErrorString(e));
    m->tp_peer[r] = p;
  }
  m->tp_ready = true;
  if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
  return UGB_OK;
}

}  // extern "C"
