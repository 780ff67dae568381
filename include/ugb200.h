/* ugb200 -- C ABI of the B200 (sm_100a) execution backend for ug.
 *
 * Every entry point is plain C: opaque handles, raw pointers and sizes, an
 * int32 status as the return value (0 = success).  Nothing here throws or
 * aborts across the boundary; the text of the last failure on a device is
 * kept per device and read with ugb_last_error().  A Rust `impl ug::Device`
 * binds exactly these symbols.
 *
 * Threading model (ug-cuda/src/runtime.rs:80-85,163-169): one stream per
 * device handle, launches are asynchronous and ordered on that stream, only
 * device->host copies and ugb_sync block.  Calls on ONE device handle must be
 * serialised by the caller; different handles are independent.
 *
 * There is no CPU fallback: every compute entry point launches a CUDA kernel
 * or fails with a status.
 */
#ifndef UGB200_H
#define UGB200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define UGB_API __attribute__((visibility("default")))
#else
#define UGB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ugb_device ugb_device;
typedef struct ugb_slice ugb_slice;
typedef struct ugb_func ugb_func;

/* ug::DType, same order as ug-core/src/dtype.rs:4-11. */
typedef enum {
  UGB_BF16 = 0,
  UGB_F16 = 1,
  UGB_F32 = 2,
  UGB_I32 = 3,
  UGB_I64 = 4
} ugb_dtype;

typedef enum {
  UGB_OK = 0,
  UGB_ERR_INVALID = 1,     /* null handle, bad enum value, bad argument          */
  UGB_ERR_DTYPE = 2,       /* dtype mismatch (runtime.rs:113-117,376,390)        */
  UGB_ERR_SHAPE = 3,       /* length / layout mismatch (gemm.rs:32,42,65,73)     */
  UGB_ERR_CUDA = 4,        /* a CUDA runtime/driver call failed                  */
  UGB_ERR_OOM = 5,         /* device allocation failed                           */
  UGB_ERR_UNSUPPORTED = 6, /* valid request this backend does not cover          */
  UGB_ERR_TIMEOUT = 7,     /* a bounded device-side wait gave up                 */
  UGB_ERR_COMPILE = 8      /* run-time compilation of an SSA kernel failed       */
} ugb_status;

/* ------------------------------------------------------------------ device */

/* ug_cuda::Device::new (ug-cuda/src/runtime.rs:163-169): binds device
 * `ordinal`, creates its stream.  On failure *out is NULL and
 * ugb_last_error(NULL) holds the message. */
UGB_API int32_t ugb_device_create(int32_t ordinal, ugb_device **out);
UGB_API int32_t ugb_device_destroy(ugb_device *dev);
/* Message of the last failed call on `dev` (or of the last failed
 * ugb_device_create when dev is NULL).  Valid until the next call on it. */
UGB_API const char *ugb_last_error(const ugb_device *dev);
/* ug::Device::synchronize (ug-core/src/lib.rs:55; runtime.rs:204-207).  Also
 * reads the device-side status word and reports UGB_ERR_TIMEOUT if a kernel
 * gave up on a bounded wait since the previous sync. */
UGB_API int32_t ugb_sync(ugb_device *dev);
/* ug::Device::use_grid (lib.rs:72; runtime.rs:346-348): always 1. */
UGB_API int32_t ugb_use_grid(void);
UGB_API int32_t ugb_device_ordinal(const ugb_device *dev);
/* The CUDA stream (cudaStream_t) all work of this device is ordered on;
 * ug_cuda::Device::cudarc_stream (runtime.rs:171-173). */
UGB_API void *ugb_device_stream(const ugb_device *dev);
/* Number of kernels this library has launched on `dev` since creation. */
UGB_API uint64_t ugb_launch_count(const ugb_device *dev);
/* Tuning switches of a device handle (no counterpart in the reference).
 *   "gemm_cta_pairs"  1 (default) / 0: bf16 GEMMs with more than 128 rows run
 *                     256 x 256 tiles on pairs of CTAs (tcgen05 cta_group::2, a
 *                     cluster of two SMs sharing the B operand) instead of
 *                     128 x 256 tiles on single CTAs.  Same results bit for bit.
 *   "wait_limit_us"   100 .. 60000000 (default 2000000): how long a device-side
 *                     wait on something another agent completes (an mbarrier fed
 *                     by TMA / MMA, a peer GPU's flag, a grid-wide barrier) may
 *                     last before the kernel gives up, raises UGB_ERR_TIMEOUT in
 *                     the status word (read by ugb_sync) and returns.  For the
 *                     tensor-parallel engine the limit must also cover the skew
 *                     between the ranks' host threads (a slow first launch on
 *                     one rank counts against the others' waits).
 * Unknown names and out-of-range values are UGB_ERR_INVALID. */
UGB_API int32_t ugb_device_set_option(ugb_device *dev, const char *name, int32_t value);

/* Self-test of the bounded waits (no counterpart in the reference, which has no
 * device-side waits): enqueues one CTA that waits on something nobody completes
 * -- which = 0: an mbarrier without arrivals (site code 0x99); which = 1: the
 * flag of a tensor-parallel peer that never signals (site code 0x7001) -- with
 * the current "wait_limit_us".  The wait gives up, the kernel returns, and the
 * NEXT ugb_sync reports UGB_ERR_TIMEOUT with that site code in its message;
 * after that the device handle works as before.  Nothing faults or hangs. */
UGB_API int32_t ugb_selftest_bounded_wait(ugb_device *dev, int32_t which);

/* ------------------------------------------------------------------ memory */

/* ug::Device::allocate_uninit (lib.rs:53; runtime.rs:216-241): `len` ELEMENTS
 * of `dtype`, contents undefined.  len == 0 is legal (the KV cache starts as
 * a 0-element buffer, ug-llama/src/model.rs:192-193). */
UGB_API int32_t ugb_alloc(ugb_device *dev, int32_t dtype, size_t len, ugb_slice **out);
/* Drop of a Slice (stream-ordered free). */
UGB_API int32_t ugb_free(ugb_slice *s);
/* Wraps device memory owned by the caller (never freed by this library). */
UGB_API int32_t ugb_wrap(ugb_device *dev, void *device_ptr, int32_t dtype, size_t len, ugb_slice **out);
/* ug::Slice::len / dtype (lib.rs:33-34), device_ptr (runtime.rs:137-161). */
UGB_API size_t ugb_slice_len(const ugb_slice *s);
UGB_API int32_t ugb_slice_dtype(const ugb_slice *s);
UGB_API void *ugb_slice_ptr(const ugb_slice *s);
/* ug::Slice::copy_host_to_device (lib.rs:35; runtime.rs:367-379): `dtype` is
 * the host element type and must equal the slice's, `len` must equal the
 * slice length.  Blocks until the host buffer may be reused. */
UGB_API int32_t ugb_h2d(ugb_slice *dst, const void *src, size_t len, int32_t dtype);
/* ug::Slice::copy_device_to_host (lib.rs:36; runtime.rs:381-393): blocks
 * until the data is in `dst`. */
UGB_API int32_t ugb_d2h(const ugb_slice *src, void *dst, size_t len, int32_t dtype);
/* Asynchronous variants for pinned host memory: ordered on the device stream,
 * return without waiting.  The host buffer must stay valid until ugb_sync. */
UGB_API int32_t ugb_h2d_async(ugb_slice *dst, const void *pinned_src, size_t len, int32_t dtype);
UGB_API int32_t ugb_d2h_async(const ugb_slice *src, void *pinned_dst, size_t len, int32_t dtype);
/* Page-locked host buffers for the asynchronous copies. */
UGB_API int32_t ugb_host_alloc(size_t bytes, void **out);
UGB_API int32_t ugb_host_free(void *p);

/* ------------------------------------------------------------------ timing */

/* CUDA-event stopwatch on the device's own stream (the stream every kernel
 * of this library runs on).  begin/end record events; elapsed waits for the
 * end event and returns milliseconds. */
UGB_API int32_t ugb_timer_begin(ugb_device *dev);
UGB_API int32_t ugb_timer_end(ugb_device *dev);
UGB_API int32_t ugb_timer_elapsed_ms(ugb_device *dev, float *ms);

/* --------------------------------------------- ug-llama Device trait (ops) */
/* trait ug_llama::Device (ug-llama/src/main.rs:22-28).  Argument order is the
 * order the reference's custom-op closures receive their slices in: inputs in
 * call order, destination last (ug-llama/src/cuda_ops.rs:26-28,128,165). All
 * slices are F32 except `pos` (I32). */

/* custom_softmax (cuda_ops.rs:149-174, cpu_ops.rs:6-31): max-subtracted
 * softmax over rows of `n_cols`.  src may equal dst. */
UGB_API int32_t ugb_softmax(ugb_device *dev, const ugb_slice *src, ugb_slice *dst, size_t n_rows,
                    size_t n_cols);
/* causal_mask (cpu_ops.rs:33-56; the reference CUDA backend bails,
 * cuda_ops.rs:176-178): [bh, s1, s2], keeps i2 <= i1, writes -inf above. */
UGB_API int32_t ugb_causal_mask(ugb_device *dev, const ugb_slice *src, ugb_slice *dst, size_t bh,
                        size_t s1, size_t s2);
/* rope (cuda_ops.rs:58-96, cpu_ops.rs:91-127): half rotation on [b,h,t,d];
 * table row pos[0] + i_t; cos/sin are [max_pos, d/2]. */
UGB_API int32_t ugb_rope(ugb_device *dev, const ugb_slice *src, const ugb_slice *cos,
                 const ugb_slice *sin, const ugb_slice *pos, ugb_slice *dst, size_t b, size_t h,
                 size_t t, size_t d);
/* rope_i (cpu_ops.rs:58-89; the reference's ropei.cu does not compile):
 * interleaved pairs (2i, 2i+1). */
UGB_API int32_t ugb_rope_i(ugb_device *dev, const ugb_slice *src, const ugb_slice *cos,
                   const ugb_slice *sin, const ugb_slice *pos, ugb_slice *dst, size_t b,
                   size_t h, size_t t, size_t d);
/* cat (cuda_ops.rs:98-147, cpu_ops.rs:129-167) on the flattened views
 * lhs [d1, d2_l], rhs [d1, d2_r] -> dst [d1, d2_l + d2_r].  Bit-exact copy. */
UGB_API int32_t ugb_cat(ugb_device *dev, const ugb_slice *lhs, const ugb_slice *rhs, ugb_slice *dst,
                size_t d1, size_t d2_l, size_t d2_r);

/* ---------------------------------------------- ug::Device::compile / run */
/* The SSA kernel IR crosses the boundary verbatim: one ugb_ssa_instr per
 * ssa::Instr (ug-core/src/lang.rs:690-709), a variable being the line number
 * of the instruction that defines it (lang.rs:611-636). */
typedef enum {
  UGB_SSA_DEFINE_ACC = 0,   /* cst                                   DefineAcc(Const)            */
  UGB_SSA_DEFINE_GLOBAL,    /* index, dtype                          DefineGlobal{index,dtype}   */
  UGB_SSA_DEFINE_LOCAL,     /* index = size, dtype                   DefineLocal{size,dtype}     */
  UGB_SSA_SPECIAL,          /* op = UGB_SSA_THREAD_IDX | BLOCK_IDX   Special                     */
  UGB_SSA_CONST,            /* cst                                   Const(Const)                */
  UGB_SSA_UNARY,            /* op = UGB_UNARY_*, a0, dtype           Unary{op,arg,dtype}         */
  UGB_SSA_BINARY,           /* op = UGB_BINARY_*, a0, a1, dtype      Binary{op,lhs,rhs,dtype}    */
  UGB_SSA_RANGE,            /* a0 = lo, a1 = up, index = step, v0    Range{lo,up,step,end_idx}   */
  UGB_SSA_LOAD,             /* v0 = src, a0 = offset, dtype          Load{src,offset,dtype}      */
  UGB_SSA_ASSIGN,           /* v0 = dst, a0 = src                    Assign{dst,src}             */
  UGB_SSA_END_RANGE,        /* v0 = start_idx                        EndRange{start_idx}         */
  UGB_SSA_IF,               /* a0 = cond, v0 = end_idx               If{cond,end_idx}            */
  UGB_SSA_END_IF,           /*                                       EndIf                       */
  UGB_SSA_STORE,            /* v0 = dst, a0 = offset, a1 = value     Store{dst,offset,value,..}  */
  UGB_SSA_BARRIER,          /*                                       Barrier                     */
  UGB_SSA_REDUCE_LOCAL      /* op = UGB_REDUCE_*, a0, dtype          ReduceLocal{op,arg,dtype}   */
} ugb_ssa_kind;
enum { UGB_SSA_THREAD_IDX = 0, UGB_SSA_BLOCK_IDX = 1 };
enum { UGB_UNARY_ID = 0, UGB_UNARY_EXP, UGB_UNARY_SIN, UGB_UNARY_COS, UGB_UNARY_NEG, UGB_UNARY_SQRT, UGB_UNARY_CAST };
enum { UGB_BINARY_ADD = 0, UGB_BINARY_SUB, UGB_BINARY_MUL, UGB_BINARY_DIV, UGB_BINARY_MOD, UGB_BINARY_MIN, UGB_BINARY_MAX };
enum { UGB_REDUCE_SUM = 0, UGB_REDUCE_MAX, UGB_REDUCE_MIN };

/* ssa::A (lang.rs:642-646): a variable, or an inline constant whose bit
 * pattern sits in the low bits of `value` (f32: 32 bits, bf16/f16: 16 bits). */
typedef struct {
  int32_t is_var;
  int32_t dtype;  /* constants only */
  int64_t value;  /* variable id, or constant bits */
} ugb_ssa_arg;

typedef struct {
  int32_t kind;   /* ugb_ssa_kind */
  int32_t dtype;
  int32_t op;
  int32_t reserved;
  int64_t index;
  int64_t v0;
  ugb_ssa_arg a0, a1;
  ugb_ssa_arg cst;
} ugb_ssa_instr;

/* ug::Device::compile (lib.rs:56; ug-cuda/src/runtime.rs:247-264) with the
 * kernel's LaunchConfig (lang.rs:34-45).  The kernel's pointer arguments are
 * its DefineGlobal instructions in index order.  Loads and stores of global AND
 * of DefineLocal (shared-memory) buffers are checked against the buffer's length
 * and raise the status word (UGB_ERR_INVALID at the next ugb_sync) instead of
 * touching memory outside it.  Barrier and ReduceLocal are block-wide: they must
 * be reached by every thread of the block (not under an If, nor inside a Range
 * whose bounds depend on the thread index); anything else is undefined, as for
 * __syncthreads.  Errors in the IR or in the
 * run-time compilation are UGB_ERR_COMPILE with the compiler log in the
 * message. */
UGB_API int32_t ugb_compile(ugb_device *dev, const ugb_ssa_instr *instrs, size_t n_instrs,
                            uint32_t grid_dim, uint32_t block_dim, uint32_t shared_mem,
                            const char *name, ugb_func **out);
/* ug_cuda::Device::compile_cu / compile_ptx (ug-cuda/src/runtime.rs:179-193): a
 * kernel written by the caller, CUDA C compiled at run time with
 * use_fast_math as the reference does, or PTX handed to the driver.  Its
 * parameters must be device pointers only: ugb_run passes the slices' pointers
 * in order and nothing else (no lengths, no status word), with the launch
 * shape given here.  Bounds are the author's responsibility. */
UGB_API int32_t ugb_compile_cu(ugb_device *dev, const char *cu_code, const char *func_name,
                               uint32_t grid_dim, uint32_t block_dim, uint32_t shared_mem,
                               ugb_func **out);
UGB_API int32_t ugb_compile_ptx(ugb_device *dev, const char *ptx_code, const char *func_name,
                                uint32_t grid_dim, uint32_t block_dim, uint32_t shared_mem,
                                ugb_func **out);
/* The shape-polymorphic compile cache of the host layer (ug-core/src/cache.rs:8-101 keys on shapes, so every
 * kernel whose shape follows the KV length is recompiled each token, ug-llama/src/main.rs:140-149) works on the
 * CUDA C this library generates from SSA: ugb_ssa_source returns that text for an entry-point name of the
 * caller's choice without compiling it (the kernel's parameters are its pointers, one length per pointer, the
 * status word), together with the dtypes of the pointer arguments; ugb_compile_generated compiles a text of that
 * form whose parameter list ends in n_dyn extra `const long long` values; ugb_run_dyn launches a function with a
 * grid size and those values chosen per call (n_dyn == 0 and the compiled grid make it ugb_run). */
UGB_API int32_t ugb_ssa_source(ugb_device *dev, const ugb_ssa_instr *instrs, size_t n_instrs, const char *entry_name,
                               char *buf, size_t buf_len, int32_t *arg_dtypes, size_t max_args, size_t *n_args);
UGB_API int32_t ugb_compile_generated(ugb_device *dev, const char *cu_code, const char *entry_name,
                                      const int32_t *arg_dtypes, size_t n_args, int32_t n_dyn, uint32_t grid_dim,
                                      uint32_t block_dim, uint32_t shared_mem, ugb_func **out);
UGB_API int32_t ugb_run_dyn(ugb_device *dev, ugb_func *f, ugb_slice *const *args, size_t n_args, uint32_t grid_dim,
                            const int64_t *dyn, size_t n_dyn);
UGB_API int32_t ugb_func_free(ugb_func *f);
/* The CUDA C this backend generated for the kernel (inspection, tests). */
UGB_API const char *ugb_func_source(const ugb_func *f);
/* ug::Device::run (lib.rs:60; runtime.rs:266-332): launches asynchronously on
 * the device stream.  One slice per pointer argument, any number of them (the
 * reference accepts 1 to 5); dtypes are checked; a zero grid or block
 * dimension is a no-op (runtime.rs:269-277).  Loads and stores that fall
 * outside the slice they address are skipped and reported as UGB_ERR_SHAPE
 * by the next ugb_sync. */
UGB_API int32_t ugb_run(ugb_device *dev, ugb_func *f, ugb_slice *const *args, size_t n_args);

/* ------------------------------------------ ug::safetensors::MmapedSafetensors */
/* Memory-mapped .safetensors files (ug-core/src/safetensors.rs:10-318; container
 * format of crate safetensors 0.4.5).  Files stay mapped until ugb_st_close; a
 * tensor name present in several files resolves to the last file (safetensors.rs:40). */
typedef struct ugb_safetensors ugb_safetensors;
/* MmapedSafetensors::new (one path) / ::multi (several).  Errors (unreadable
 * file, malformed or inconsistent header) are UGB_ERR_INVALID with the path in
 * the message, on `dev`. */
UGB_API int32_t ugb_st_open(ugb_device *dev, const char *const *paths, size_t n_paths,
                            ugb_safetensors **out);
UGB_API int32_t ugb_st_close(ugb_safetensors *st);
/* MmapedSafetensors::tensors: names in file order of their data. */
UGB_API size_t ugb_st_count(const ugb_safetensors *st);
UGB_API const char *ugb_st_name(const ugb_safetensors *st, size_t i);
/* MmapedSafetensors::get: dtype (ugb_dtype, or -1 for a safetensors dtype that ug
 * has no DType for), rank and up to dims_cap dimensions. */
UGB_API int32_t ugb_st_info(ugb_device *dev, const ugb_safetensors *st, const char *name,
                            int32_t *dtype, int32_t *rank, size_t *dims, size_t dims_cap);
/* load_slice (safetensors.rs:83-118): a new slice of the tensor's dtype holding
 * its elements.  Dtypes other than BF16/F16/F32/I32/I64 are UGB_ERR_DTYPE. */
UGB_API int32_t ugb_st_load_slice(ugb_device *dev, const ugb_safetensors *st, const char *name,
                                  ugb_slice **out);
/* load_slice_with_cast (safetensors.rs:120-271): converted on the host, element
 * by element, through f32 for the float types (round to nearest even into
 * bf16 / f16), float -> int saturating, i64 -> i32 wrapping.  BF16 / F16 -> I64
 * fail with the dtype mismatch the reference's own copy raises there. */
UGB_API int32_t ugb_st_load_slice_with_cast(ugb_device *dev, const ugb_safetensors *st,
                                            const char *name, int32_t dst_dtype, ugb_slice **out);

/* ------------------------------------------------------- ug::Device::matmul */

/* ug::Device::matmul (ug-core/src/lib.rs:61-69; ug-cuda/src/gemm.rs:292-332):
 * dst[b, m, n] = lhs[b, m, k] . rhs[b, k, n], dst row-major contiguous.  The
 * operand layouts are passed the way ug::Layout holds them: `rank` dims and
 * element strides plus an element offset.  The same layout rules as
 * gemm_config (gemm.rs:8-83) apply: each operand's last two dims must be
 * row-major or its transpose, the leading dims must collapse to one batch
 * stride (0 is allowed: a shared operand); anything else is UGB_ERR_SHAPE
 * ("non contiguous matmul").  dst, lhs and rhs must share one dtype out of
 * BF16 / F16 / F32 (UGB_ERR_DTYPE otherwise); accumulation is fp32.  bf16
 * operands with a row-major lhs run on the tcgen05 tensor-core kernel. */
UGB_API int32_t ugb_matmul(ugb_device *dev, ugb_slice *dst, const ugb_slice *lhs,
                           const ugb_slice *rhs, size_t b, size_t m, size_t n, size_t k,
                           int32_t rank, const size_t *lhs_dims, const size_t *lhs_strides,
                           size_t lhs_off, const size_t *rhs_dims, const size_t *rhs_strides,
                           size_t rhs_off);

/* ------------------------------------------------- fused row operators (new) */
/* The reference reaches these through generated kernels; the new backend
 * gives them one fused launch each (single read, single write). */

/* rms_norm (ug-llama/src/model.rs:65-78): y = x / sqrt(mean(x^2) + eps) * alpha,
 * rows of n_cols, alpha [n_cols]. */
UGB_API int32_t ugb_rms_norm(ugb_device *dev, const ugb_slice *x, const ugb_slice *alpha, ugb_slice *dst,
                     size_t n_rows, size_t n_cols, float eps);
/* rms_norm(x) * alpha * silu(gate) (model.rs:65-78 and :103-109). */
UGB_API int32_t ugb_rms_norm_silu_gate(ugb_device *dev, const ugb_slice *x, const ugb_slice *alpha,
                               const ugb_slice *gate, ugb_slice *dst, size_t n_rows,
                               size_t n_cols, float eps);
/* silu(gate) * up (model.rs:103-109,160-168), n elements. */
UGB_API int32_t ugb_silu_mul(ugb_device *dev, const ugb_slice *gate, const ugb_slice *up, ugb_slice *dst,
                     size_t n);
/* elementwise a + b (residual adds, model.rs:263,267), n elements. */
UGB_API int32_t ugb_add(ugb_device *dev, const ugb_slice *a, const ugb_slice *b, ugb_slice *dst,
                size_t n);
/* index_select (model.rs:32-63): dst[r, :] = emb[ids[r], :], emb [vocab, h]
 * F32, ids I32 [n_ids].  Ids outside [0, vocab) are reported as
 * UGB_ERR_INVALID at the next ugb_sync and their rows are left untouched. */
UGB_API int32_t ugb_index_select(ugb_device *dev, const ugb_slice *emb, const ugb_slice *ids,
                         ugb_slice *dst, size_t n_ids, size_t h, size_t vocab);


/* Grouped-query attention for ONE new query position per sequence: the fused
 * form of repeat + q.kT + scale (head_dim^-0.5) + softmax + .v + transpose/merge
 * of Attention::fwd (ug-llama/src/model.rs:231-245) over a preallocated bf16 KV
 * cache.  q bf16 [b, n_heads, 64]; k, v bf16 [b, n_kv, t_max, 64] of which the
 * first pos[0] + 1 positions are attended (pos I32 [1], read on the device);
 * out bf16 [b, n_heads * 64].  head_dim is 64, n_heads / n_kv <= 8, t_max a
 * multiple of 16, n_slices (1..8) KV slices per (sequence, KV head) run as
 * separate CTAs.  Cache rows at positions > pos[0] must hold finite values.
 * Scratch for the per-slice partial results comes from the device's
 * stream-ordered pool for the duration of the call. */
UGB_API int32_t ugb_decode_attention(ugb_device *dev, const ugb_slice *q, const ugb_slice *k,
                                     const ugb_slice *v, const ugb_slice *pos, ugb_slice *out,
                                     size_t b, size_t n_heads, size_t n_kv, size_t t_max,
                                     int32_t n_slices);

/* ugb_decode_attention for callers that cannot allocate device memory.  It has
 * no counterpart in the reference.  Some hosts of this library give every byte
 * of the GPU to their own pool when they start (an inference server with a
 * pre-sized KV arena, a framework's caching allocator), so a driver allocation
 * made later fails or fragments their arena; others call from a
 * latency-critical thread where an allocator call may take a lock or
 * synchronise the device.  This variant takes its scratch (per-slice partial
 * results and completion counters) from a fixed array inside the library
 * instead: it calls no cudaMalloc / cudaFree and no allocating routine.
 * Arguments, results and errors are those of ugb_decode_attention, plus:
 *  - limit: b * n_kv * n_slices <= 2048, otherwise UGB_ERR_SHAPE (the array is
 *    about 4.1 MiB and every GPU that loads the library holds it until exit);
 *  - the first call on each device looks the array's device address up
 *    (one-time set-up); make that call before starting any stream capture;
 *  - all calls on a device share the one array, which keeps the previous
 *    call's contents; each call clears the counters it needs.  Two calls that
 *    overlap on the GPU (different streams or device handles of one GPU) race
 *    on it: serialise them. */
UGB_API int32_t ugb_decode_attention_noalloc(ugb_device *dev, const ugb_slice *q,
                                             const ugb_slice *k, const ugb_slice *v,
                                             const ugb_slice *pos, ugb_slice *out, size_t b,
                                             size_t n_heads, size_t n_kv, size_t t_max,
                                             int32_t n_slices);

/* Causal grouped-query attention for a block of t NEW positions per sequence:
 * the fused form of Attention::fwd with seq_len > 1 (ug-llama/src/model.rs:231-245:
 * repeat + q.kT + scale (head_dim^-0.5) + causal mask + softmax + .v +
 * transpose/merge) over a preallocated bf16 KV cache, without the
 * [b, h, t, pos0 + t] score tensor.  q bf16 [b, t, n_heads, 64] (rotation
 * applied); k, v bf16 [b, n_kv, t_max, 64] already holding the keys / values of
 * positions 0 .. pos0 + t - 1 (the block's own included); query i of the block
 * attends positions 0 .. pos0 + i; out bf16 [b, t, n_heads * 64].  head_dim is
 * 64, n_heads a multiple of n_kv, pos0 + t <= t_max, all buffers 16-byte
 * aligned.  Cache rows between pos0 + t and the next multiple of 64 must hold
 * finite values (they are loaded with their 64-key tile and weighted by zero).
 * Runs on the tcgen05 / TMEM kernel; allocates nothing. */
UGB_API int32_t ugb_causal_attention(ugb_device *dev, const ugb_slice *q, const ugb_slice *k,
                                     const ugb_slice *v, ugb_slice *out, size_t b, size_t t,
                                     size_t pos0, size_t n_heads, size_t n_kv, size_t t_max);

/* ------------------------------------------- ug-llama Model::fwd (decode step) */
/* The reference builds one lazy graph per token from Model::fwd
 * (ug-llama/src/model.rs:298-374) and runs ~27 launches per layer; this entry
 * point family runs the same operator chain for one new token per sequence as
 * a fixed, fused kernel sequence captured in a CUDA graph.  Weights and the KV
 * cache are bf16, reductions and the residual stream fp32.  Batch rows are
 * independent sequences that share one position (the reference reads pos[0]
 * for every row, ug-llama/src/cpu_ops.rs:67-71). */
typedef struct ugb_llama ugb_llama;

/* ug_llama::model::Config (ug-llama/src/model.rs:10-30). */
typedef struct {
  int32_t hidden;           /* hidden_size                  */
  int32_t layers;           /* num_hidden_layers            */
  int32_t n_heads;          /* num_attention_heads          */
  int32_t n_kv_heads;       /* num_key_value_heads          */
  int32_t head_dim;         /* hidden_size / n_heads        */
  int32_t ffn;              /* intermediate_size            */
  int32_t vocab;            /* vocab_size                   */
  int32_t max_pos;          /* max_position_embeddings      */
  float rope_theta;
  float rms_eps;
  int32_t rope_interleaved; /* rope_interleaved (0 / 1)     */
} ugb_llama_config;

enum { UGB_LLAMA_LOGITS = 0, UGB_LLAMA_NEXT_TOKENS = 1, UGB_LLAMA_HIDDEN = 2, UGB_LLAMA_PREFILL_LOGITS = 3,
       UGB_LLAMA_STEP_PROFILE = 4 /* measurement aid, see option "step_profile" */,
       UGB_LLAMA_GEMM_PROFILE = 5 /* measurement aid, see option "gemm_profile" */ };

/* Model::new + Cache::new (model.rs:183-198,298-363): allocates weights, the
 * RoPE tables (model.rs:278-295) and a KV cache for `batch` sequences of up to
 * `t_max` positions.  tie_word_embeddings is assumed, as in model.rs:315-319. */
UGB_API int32_t ugb_llama_create(ugb_device *dev, const ugb_llama_config *cfg, int32_t batch,
                                 int32_t t_max, ugb_llama **out);
UGB_API int32_t ugb_llama_destroy(ugb_llama *m);
/* Tensor-parallel variant (no counterpart in the reference, which runs on one
 * device): rank `tp_rank` of `tp_size` (1..8) keeps the query heads, KV heads
 * (replicated when tp_size > n_kv_heads), FFN columns and vocabulary slice it
 * owns; q/k/v/gate/up are column-parallel, o_proj/down_proj row-parallel.  All
 * ranks are fed the same tokens and hold the same residual stream.  The sums
 * over ranks are not separate collectives: every rank leaves its fp32 partials
 * in an exchange block that the peers map (ugb_llama_tp_export ->
 * ugb_llama_tp_connect, CUDA IPC, one process per GPU), and the kernel that
 * adds the residual and applies the next RMSNorm reads all ranks' partials
 * over NVLink in rank order, so the replicas stay bit-identical.  Logits are
 * vocab-parallel: ugb_llama_read returns this rank's columns
 * [vocab_offset, vocab_offset + vocab_local) and the greedy choice is made over
 * (value, id) pairs exchanged the same way.  Waits on peers are bounded (device
 * option "wait_limit_us", then UGB_ERR_TIMEOUT at the next ugb_sync, after which
 * ugb_llama_decode / ugb_llama_prefill of this model refuse further steps: the
 * ranks may be out of step and the model has to be recreated); ranks must issue
 * the same calls.
 * ugb_llama_load_weight takes whole tensors and keeps the rank's slice. */
UGB_API int32_t ugb_llama_create_tp(ugb_device *dev, const ugb_llama_config *cfg, int32_t batch,
                                    int32_t t_max, int32_t tp_rank, int32_t tp_size, ugb_llama **out);
/* 64-byte CUDA IPC handle of this rank's exchange block. */
UGB_API int32_t ugb_llama_tp_export(ugb_llama *m, void *handle_out, size_t handle_bytes);
/* `handles`: tp_size handles in rank order (own entry ignored).  Every rank must
 * have exported before any rank connects, and connected before any rank steps. */
UGB_API int32_t ugb_llama_tp_connect(ugb_llama *m, const void *handles, size_t handle_bytes,
                                     int32_t n_ranks);
UGB_API int32_t ugb_llama_tp_info(const ugb_llama *m, int32_t *tp_rank, int32_t *tp_size,
                                  int32_t *vocab_local, int32_t *vocab_offset,
                                  int32_t *kv_heads_local);

/* One tensor by its safetensors name (model.rs:313-346), e.g.
 * "model.layers.3.self_attn.q_proj.weight".  Matrices: BF16, or F32 rounded to
 * bf16 (round to nearest even).  Norm weights: F32.  Shapes are checked like
 * Linear::new / RmsNorm::new do (model.rs:120-122,142-144). */
UGB_API int32_t ugb_llama_load_weight(ugb_llama *m, const char *name, const ugb_slice *w);
/* Tuning knobs: "splits_qkv", "splits_o", "splits_down" (split-K factors of the
 * projections) and "att_splits" (KV slices per sequence and KV head), 1..8;
 * "bn_qkv", "bn_o", "bn_gate_up", "bn_down", "bn_lm_head" (GEMM tile width:
 * 64, 80, 96, 128, 160 or 256); "gemm_smem_kib" (shared-memory cap of a decode GEMM
 * CTA, 32..220, 0 = none); "att_stages" (2..6); "att_early", "att_tma",
 * "att_cluster" (the KV slices of a pair run as one thread-block cluster),
 * "gate_up_pair" (decode gate|up on pairs of CTAs that split k),
 * "prefill_attention_tc", "pdl" (0 / 1); "prefill_rows" (64..65536, see
 * ugb_llama_prefill); "step_kernel" (0 / 1): a decode step of up to 64
 * sequences runs all its layers in ONE persistent kernel launch (grid-wide
 * barriers between the phases, the weight stream running ahead of them)
 * followed by the lm_head and the greedy choice, instead of seven launches per
 * layer; "step_profile" (0 / 1, measurement aid): that kernel records
 * %globaltimer at every grid barrier, read with UGB_LLAMA_STEP_PROFILE;
 * "gemm_profile" (0 / 1, measurement aid): CTA 0 of every decode projection
 * records %globaltimer at its start, when the wait for the preceding kernel
 * returns, at its last MMA, when the epilogue sees the accumulator, when the
 * epilogue is done, at its end (values 0..5 of a projection) and at every k
 * block of its main loop (values 8..); UGB_LLAMA_GEMM_PROFILE reads 5 x 64
 * floats (qkv, o, gate|up, down, lm_head of the last launches), microseconds
 * after the projection's own wait returned, 0 = not recorded. */
UGB_API int32_t ugb_llama_set_option(ugb_llama *m, const char *key, int32_t value);
/* Sets the number of cached positions (0 = empty cache); cache contents at
 * positions >= pos are ignored by later steps. */
UGB_API int32_t ugb_llama_reset(ugb_llama *m, int32_t pos);
UGB_API int32_t ugb_llama_position(const ugb_llama *m);
UGB_API int32_t ugb_llama_kv_positions(const ugb_llama *m);
/* Model::fwd for seq_len == 1, n_steps times.  With `tokens` (I32 [batch],
 * n_steps must be 1) the step consumes those ids; with NULL each step
 * consumes the argmax of the previous step's logits (greedy decoding, ties to
 * the lowest id).  Asynchronous; results are read with ugb_llama_read. */
UGB_API int32_t ugb_llama_decode(ugb_llama *m, const ugb_slice *tokens, int32_t n_steps);
/* Model::fwd for seq_len == t > 1 (model.rs:365-374 with the causal mask of
 * Attention::fwd, model.rs:231-245): consumes `tokens` (I32 [batch, t]), appends
 * t positions to the KV cache of every sequence and leaves the logits of the
 * LAST position in the place ugb_llama_decode leaves them, so that
 * ugb_llama_decode(m, NULL, n) continues greedily from there.  The block is
 * processed in chunks of positions bounded by option "prefill_rows" (rows =
 * batch * positions per chunk, default 8192; set it before the first call);
 * the projections run on the same tensor-core GEMM as decode with m = rows,
 * attention is a causal flash kernel over the cache.  With all_logits != 0 the
 * logits of every position are kept too (f32 [batch, t, vocab], the tensor
 * Model::fwd returns) and read with UGB_LLAMA_PREFILL_LOGITS.  Asynchronous. */
UGB_API int32_t ugb_llama_prefill(ugb_llama *m, const ugb_slice *tokens, int32_t t,
                                  int32_t all_logits);
/* Blocking read of the last step's logits (f32 [batch, vocab]), next tokens
 * (i32 [batch]), final residual stream (f32 [batch, hidden]) or the logits of
 * the last all_logits prefill (f32 [batch, t, vocab]); len in elements. */
UGB_API int32_t ugb_llama_read(ugb_llama *m, int32_t what, void *host_dst, size_t len);
/* Blocking read of one layer's K (which = 0) or V (1) cache, bf16
 * [batch, n_kv_heads, ugb_llama_kv_positions, head_dim]. */
UGB_API int32_t ugb_llama_read_kv(ugb_llama *m, int32_t layer, int32_t which, void *host_dst,
                                  size_t len);

/* Measurement aid: runs ONE kernel type of the decode step over all layers
 * (the cache must hold at least one position), `iters` passes after one
 * warm-up pass, timed with CUDA events on the device stream; returns
 * milliseconds per pass (= per decode step's worth of that kernel; the
 * lm_head GEMM runs once per pass).  Activations are scratch afterwards; the
 * KV cache and the position are left as they were. */
enum {
  UGB_LLAMA_K_QKV = 0, UGB_LLAMA_K_ATTENTION = 1, UGB_LLAMA_K_O = 2, UGB_LLAMA_K_GATE_UP = 3,
  UGB_LLAMA_K_DOWN = 4, UGB_LLAMA_K_LM_HEAD = 5
};
UGB_API int32_t ugb_llama_time_kernel(ugb_llama *m, int32_t which, int32_t iters,
                                      float *ms_per_pass);

#ifdef __cplusplus
}
#endif
#endif /* UGB200_H */
