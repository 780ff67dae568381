/* ughost -- C ABI of the host side above the backend boundary: ug-core's lazy
 * graph, scheduler and lowering (ug-core/src/lazy_buffer.rs, schedule.rs,
 * lower_op.rs, cache.rs) restated in C++ (ug_b200/csrc/host/) and driven
 * through opaque handles.  The reference is Rust and generic over its Device
 * trait; here a device is a handle that is either the B200 backend
 * (ugh_device_b200, over include/ugb200.h) or any other implementation of the
 * C++ ug::Device interface handed in by pointer (ugh_device_adopt -- the test
 * suite plugs the CPU oracle in that way).
 *
 * Every function returns an int32 status (0 = ok) unless it returns a handle
 * (NULL = failure); ugh_last_error() gives the message of the calling
 * thread's last failure.  Handles are reference-like: free each one exactly
 * once; freeing a buffer handle does not free the graph node while other
 * nodes still use it. */
#ifndef UGHOST_H
#define UGHOST_H
#include <stddef.h>
#include <stdint.h>

#include "ugb200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ugh_device ugh_device;
typedef struct ugh_lb ugh_lb;              /* LazyBuffer<D>                      */
typedef struct ugh_schedule ugh_schedule;  /* Schedule<D>                        */
typedef struct ugh_compiled ugh_compiled;  /* CompiledSchedule<D>                */
typedef struct ugh_cache ugh_cache;        /* cache::CompilationCache<D>         */
typedef struct ugh_slice ugh_slice;        /* a D::Slice seen by a custom op     */

UGB_API const char *ugh_last_error(void);

/* ---- devices */
UGB_API ugh_device *ugh_device_b200(ugb_device *dev);   /* does not take ownership of `dev` */
/* launch_policy: 0 = reference heuristic (ug-core/src/schedule.rs:162-188), 1 = this backend's */
UGB_API int32_t ugh_device_set_launch_policy(ugh_device *dev, int32_t policy);
UGB_API ugh_device *ugh_device_adopt(void *cpp_ug_device);   /* takes ownership of a ug::Device* */
UGB_API void ugh_device_free(ugh_device *dev);
UGB_API int32_t ugh_device_synchronize(ugh_device *dev);
UGB_API ugb_slice *ugh_slice_b200(ugh_slice *s);          /* NULL unless the slice is a B200 slice */
UGB_API size_t ugh_slice_len(const ugh_slice *s);
UGB_API int32_t ugh_slice_dtype(const ugh_slice *s);

/* ---- LazyBuffer builders (lazy_buffer.rs:229-765).  dims: `rank` extents; dim arguments may be
 * negative (D::Minus1 = -1).  dtype / op codes are those of include/ugb200.h. */
UGB_API ugh_lb *ugh_lb_cst_f32(float v, const size_t *dims, size_t rank, ugh_device *dev);
UGB_API ugh_lb *ugh_lb_cst_i32(int32_t v, const size_t *dims, size_t rank, ugh_device *dev);
UGB_API ugh_lb *ugh_lb_copy(const void *data, size_t len, int32_t dtype, const size_t *dims, size_t rank, ugh_device *dev);
UGB_API ugh_lb *ugh_lb_alloc_uninit(int32_t dtype, const size_t *dims, size_t rank, ugh_device *dev);
UGB_API ugh_lb *ugh_lb_unary(ugh_lb *a, int32_t op);
UGB_API ugh_lb *ugh_lb_cast(ugh_lb *a, int32_t dtype);
UGB_API ugh_lb *ugh_lb_binary(ugh_lb *a, int32_t op, ugh_lb *b);
UGB_API ugh_lb *ugh_lb_reduce(ugh_lb *a, int32_t op, int64_t dim);
UGB_API ugh_lb *ugh_lb_matmul(ugh_lb *a, ugh_lb *b, int32_t transpose_rhs);
UGB_API ugh_lb *ugh_lb_broadcast(ugh_lb *a, const size_t *dims, size_t rank);
UGB_API ugh_lb *ugh_lb_reshape(ugh_lb *a, const size_t *dims, size_t rank);
UGB_API ugh_lb *ugh_lb_transpose(ugh_lb *a, int64_t dim1, int64_t dim2);
UGB_API ugh_lb *ugh_lb_split_dim(ugh_lb *a, int64_t dim, size_t size1, size_t size2);
UGB_API ugh_lb *ugh_lb_merge_dims(ugh_lb *a, int64_t dim);
UGB_API ugh_lb *ugh_lb_narrow(ugh_lb *a, int64_t dim, size_t offset, size_t length);
UGB_API ugh_lb *ugh_lb_squeeze(ugh_lb *a, int64_t dim);
UGB_API ugh_lb *ugh_lb_unsqueeze(ugh_lb *a, int64_t dim);
UGB_API ugh_lb *ugh_lb_set(ugh_lb *dst, ugh_lb *values);
UGB_API ugh_lb *ugh_lb_set_l(ugh_lb *dst, ugh_lb *values, const size_t *dims, const size_t *strides, size_t rank, size_t offset);
UGB_API ugh_lb *ugh_lb_cat(ugh_lb *const *args, size_t n, int64_t dim);
/* LazyBuffer::custom / custom_ip: `fn` receives the argument slices in call order, the destination (or the
 * in-place source) last (ug-llama/src/cuda_ops.rs:26-28); a non-zero return aborts the run with an error. */
typedef int32_t (*ugh_custom_fn)(void *user, ugh_slice *const *slices, size_t n);
UGB_API ugh_lb *ugh_lb_custom(ugh_custom_fn fn, void *user, ugh_lb *const *args, size_t n, const size_t *dims, size_t rank,
                              int32_t dtype, ugh_device *dev);
UGB_API ugh_lb *ugh_lb_custom_ip(ugh_lb *src, ugh_custom_fn fn, void *user, ugh_lb *const *args, size_t n);
/* LazyBuffer::ssa: a hand-built SSA kernel (launch config 1x1 as ssa::Kernel::from_instrs, lang.rs:739-753) */
UGB_API ugh_lb *ugh_lb_ssa(const ugb_ssa_instr *instrs, size_t n_instrs, ugh_lb *const *args, size_t n, const size_t *dims,
                           size_t rank, int32_t dtype, ugh_device *dev);
UGB_API void ugh_lb_free(ugh_lb *a);

UGB_API size_t ugh_lb_rank(const ugh_lb *a);
UGB_API int32_t ugh_lb_dims(const ugh_lb *a, size_t *dims_out);
UGB_API int32_t ugh_lb_dtype(const ugh_lb *a);
UGB_API int32_t ugh_lb_realized(const ugh_lb *a);
UGB_API int32_t ugh_lb_realize(ugh_lb *a);
/* LazyBuffer::data_vec: realize, then copy to the host (`len` elements of `dtype`) */
UGB_API int32_t ugh_lb_data(ugh_lb *a, void *dst, size_t len, int32_t dtype);
/* overwrite the realized storage of a buffer from the host (what the reference's tests do through data()) */
UGB_API int32_t ugh_lb_write(ugh_lb *a, const void *src, size_t len, int32_t dtype);

/* ---- Schedule (schedule.rs:62-306) */
UGB_API ugh_schedule *ugh_schedule_create(ugh_lb *const *buffers, size_t n);
UGB_API void ugh_schedule_free(ugh_schedule *s);
UGB_API size_t ugh_schedule_n_items(const ugh_schedule *s);
/* 0 = Kernel, 1 = MatMul, 2 = Custom, 3 = Ssa */
UGB_API int32_t ugh_schedule_item_kind(const ugh_schedule *s, size_t i);
/* the SSA of a Kernel item: policy -1 = default Opts (all dims sequential), 0 = reference grid heuristic,
 * 1 = this backend's.  Writes a NUL-terminated listing (one line per instruction) into buf. */
UGB_API int32_t ugh_schedule_item_ssa_text(const ugh_schedule *s, size_t i, int32_t policy, char *buf, size_t buf_len);
/* CUDA C this backend generates for a Kernel item that is a row-reduce + map or a pure map (128-bit accesses,
 * the row in registers); an empty string when the item is not of those shapes and takes the SSA path.  The first
 * line is a comment naming the shape, the entry point and the launch dimensions. */
UGB_API int32_t ugh_schedule_item_fast_source(const ugh_schedule *s, size_t i, char *buf, size_t buf_len);
UGB_API ugh_cache *ugh_cache_create(void);
UGB_API void ugh_cache_free(ugh_cache *c);
UGB_API size_t ugh_cache_hits(const ugh_cache *c);
UGB_API size_t ugh_cache_misses(const ugh_cache *c);
/* Hits served by a shape-generic function (a kernel seen before at another size; part of ugh_cache_hits), and the
 * switch for that reuse (default on; off = the reference's per-shape behaviour, ug-core/src/cache.rs:8-12). */
UGB_API size_t ugh_cache_poly_hits(const ugh_cache *c);
UGB_API void ugh_cache_set_polymorphic(ugh_cache *c, int32_t on);
UGB_API ugh_compiled *ugh_schedule_compile(const ugh_schedule *s, ugh_cache *cache_or_null);
UGB_API void ugh_compiled_free(ugh_compiled *c);
UGB_API int32_t ugh_compiled_run(const ugh_compiled *c);
UGB_API size_t ugh_compiled_n_funcs(const ugh_compiled *c);
/* What function i of a compiled schedule runs on: "matmul", "custom", "ssa" (per-instruction code from the SSA),
 * "row_vec4" / "warp_row_vec4" / "map_vec4" (generated 128-bit row / map code). */
UGB_API int32_t ugh_compiled_func_origin(const ugh_compiled *c, size_t i, char *buf, size_t buf_len);

#ifdef __cplusplus
}
#endif
#endif /* UGHOST_H */
