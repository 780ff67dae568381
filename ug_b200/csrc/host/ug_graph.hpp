// The backend contract and the lazy graph above it: restatement of
// ug-core/src/lib.rs:29-73 (Slice / Device), lazy_buffer.rs (LazyBuffer, Op),
// schedule.rs (Schedule, ScheduleItem, CompiledSchedule) and cache.rs.
#pragma once
#include "ug_lower.hpp"

namespace ug {

// ug::Slice (lib.rs:29-47)
struct Slice {
  virtual ~Slice() = default;
  virtual DType dtype() const = 0;
  virtual size_t len() const = 0;
  virtual void copy_host_to_device(const void *src, size_t len, DType dtype) = 0;
  virtual void copy_device_to_host(void *dst, size_t len, DType dtype) const = 0;
  bool is_empty() const { return len() == 0; }
};

struct Func {
  virtual ~Func() = default;
  std::string origin = "ssa";   // which generator produced the code: "ssa" (per-instruction code of the SSA path) or one
                                // of the vectorised shapes of fast_kernel() ("row_vec4", "warp_row_vec4", "map_vec4")
};

// A kernel as CUDA C source with its launch shape (see fast_kernel in ug_fast.cpp).
struct FastKernel {
  std::string source, func_name, origin;
  LaunchConfig launch;
  // origin "index_select": no source; the device runs its row-gather operator on (table, ids, dst) with
  // n_ids rows of h elements (the table's row count comes from the slice at run time)
  size_t n_ids = 0, h = 0;
};

// CUDA C generated from an SSA kernel, with the dtypes of its pointer arguments.
struct GeneratedSource {
  std::string text;
  std::vector<DType> arg_dtypes;
};

// How Schedule::compile picks the launch shape of a fused kernel.
enum class LaunchPolicy {
  Sequential,     // use_grid() == false: default Opts, every dim a sequential loop (the CPU backend)
  ReferenceGrid,  // schedule.rs:162-188 as written
  B200            // reduce-aware shapes of this backend (see choose_opts in ug_graph.cpp)
};

// ug::Device (lib.rs:49-73)
struct Device {
  virtual ~Device() = default;
  virtual std::unique_ptr<Slice> allocate_uninit(DType dtype, size_t len) = 0;
  virtual void synchronize() = 0;
  virtual std::shared_ptr<Func> compile(const ssa::Kernel &kernel, const std::string *name) = 0;
  virtual void run(Func &f, std::vector<Slice *> &args) = 0;
  virtual void matmul(Slice &dst, const Slice &lhs, const Slice &rhs, size_t b, size_t m, size_t n, size_t k,
                      const Layout &lhs_l, const Layout &rhs_l) = 0;
  virtual bool use_grid() const = 0;
  // Compiles caller-generated CUDA C whose parameters are the kernel's arguments (device pointers) in order;
  // a device without run-time compilation of source returns null and the SSA path is taken.
  virtual std::shared_ptr<Func> compile_cu(const FastKernel &) { return nullptr; }
  // The pieces the shape-polymorphic cache (ug_poly.cpp) needs from a backend that generates source from SSA:
  // the text for an entry name, compilation of a text of that form with `n_dyn` trailing value parameters, and a
  // launch with the grid and those values chosen per call.  A backend without them keeps the per-shape cache.
  virtual bool ssa_source(const ssa::Kernel &, const std::string & /*entry*/, GeneratedSource &) { return false; }
  virtual std::shared_ptr<Func> compile_generated(const GeneratedSource &, const std::string & /*entry*/, int /*n_dyn*/,
                                                  const LaunchConfig &) { return nullptr; }
  virtual void run_dyn(Func &, std::vector<Slice *> &, uint32_t /*grid*/, const std::vector<int64_t> &) { bail("run_dyn: not supported by this device"); }
  virtual LaunchPolicy launch_policy() const { return use_grid() ? LaunchPolicy::ReferenceGrid : LaunchPolicy::Sequential; }
};

using CustomF = std::function<void(std::vector<Slice *> &)>;

struct LazyBufferInner;
// LazyBuffer<D> (lazy_buffer.rs:86-112): a shared handle on a node of the op DAG.
struct LazyBuffer {
  std::shared_ptr<LazyBufferInner> p;
  LazyBufferInner *operator->() const { return p.get(); }
  explicit operator bool() const { return (bool)p; }

  // builders, lazy_buffer.rs:229-765
  LazyBuffer unary(UnaryOp op) const;
  LazyBuffer cast(DType dtype) const;
  LazyBuffer binary(BinaryOp op, const LazyBuffer &rhs) const;
  LazyBuffer reduce(ReduceOp op, long dim) const;
  LazyBuffer matmul(const LazyBuffer &rhs) const { return matmul_(rhs, false); }
  LazyBuffer matmul_t(const LazyBuffer &rhs) const { return matmul_(rhs, true); }
  LazyBuffer matmul_(const LazyBuffer &rhs, bool transpose) const;
  LazyBuffer split_dim(long dim, size_t size1, size_t size2) const;
  LazyBuffer merge_dims(long dim) const;
  LazyBuffer squeeze(long dim) const;
  LazyBuffer unsqueeze(long dim) const;
  LazyBuffer reshape(const Shape &s) const;
  LazyBuffer narrow(long dim, size_t offset, size_t length) const;
  LazyBuffer broadcast(const Shape &s) const;
  LazyBuffer transpose(long dim1, long dim2) const;
  LazyBuffer custom_ip(CustomF f, std::vector<LazyBuffer> args) const;
  LazyBuffer set(const LazyBuffer &values) const;
  LazyBuffer set_l(const LazyBuffer &values, const Layout &dst_layout) const;

  static LazyBuffer alloc_uninit(DType dtype, const Shape &s, Device *dev);
  static LazyBuffer cst(Const c, const Shape &s, Device *dev);
  static LazyBuffer copy(const void *data, size_t len, DType dtype, const Shape &s, Device *dev);
  static LazyBuffer from_slice(std::unique_ptr<Slice> data, const Shape &s, Device *dev);
  static LazyBuffer custom(CustomF f, std::vector<LazyBuffer> args, const Shape &s, DType dtype, Device *dev);
  static LazyBuffer ssa(ssa::Kernel k, std::vector<LazyBuffer> args, const Shape &s, DType dtype, Device *dev);
  static LazyBuffer cat(const std::vector<LazyBuffer> &args, long dim);

  bool in_place_op() const;
  bool realized() const;
  void realize() const;
  void maybe_allocate_uninit() const;
  void data_vec(void *dst, size_t len, DType dtype) const;
};

// The storage cell shared by clones and by in-place ops (Arc<RefCell<Option<Slice>>>).
struct DataCell {
  std::unique_ptr<Slice> slice;
};

// lazy_buffer.rs:51-83
struct Op {
  enum Kind { Unary, Binary, MatMul, Reduce, Const, Value, Layout, Reshape, Custom, CustomIp, Ssa, Set } kind = Value;
  UnaryOp uop;
  BinaryOp bop = BinaryOp::Add;
  ReduceOp rop = ReduceOp::Sum;
  size_t reduce_dim = 0;
  ug::Const cst;
  op::LayoutOp lop;
  size_t b = 0, m = 0, n = 0, k = 0;
  bool transpose = false;
  CustomF f;
  ssa::Kernel ssa_kernel;
  ug::Layout dst_layout;
  LazyBuffer a0, a1;                // operand(s): arg | lhs, rhs | src, values
  std::vector<LazyBuffer> args;     // Custom / CustomIp / Ssa
};

struct LazyBufferInner {
  size_t id;
  std::shared_ptr<DataCell> data;
  Op op;
  DType dtype;
  Shape shape;
  Device *device;
  size_t rank() const { return shape.size(); }
};

// ------------------------------------------------------------- schedule ----
using Args = std::vector<std::pair<ArgId, LazyBuffer>>;

struct ScheduleItem {  // schedule.rs:42-60
  enum Kind { Kernel, MatMul, Custom, Ssa } kind = Kernel;
  // Kernel
  op::AstP ast;
  std::pair<ArgId, LazyBuffer> dst;
  bool has_dst_layout = false;
  Layout dst_layout;
  // MatMul
  LazyBuffer mm_dst, lhs, rhs;
  size_t b = 0, m = 0, n = 0, k = 0;
  bool transpose = false;
  // Custom / Ssa
  CustomF f;
  ssa::Kernel ssa_kernel;
  Args args;

  op::Kernel kernel() const;  // schedule.rs:23-39
};

// ---- shape-polymorphic reuse (ug_poly.cpp) ----
// A generated text split into what stays and what moves: `skeleton` is the text with every decimal integer
// literal's digits replaced by POLY_MARK, `ints` the literal values in order of appearance.
constexpr char POLY_MARK = '\x01';
struct PolyText {
  std::string skeleton;
  size_t text_len = 0;                // skeleton[0, text_len) is the program text; a caller may append a key suffix
  std::vector<long long> ints;
};
struct PolyGeneric {                  // one generic function: literal number i of the text is b[i] + a[i] * t
  std::shared_ptr<Func> func;
  std::vector<long long> a, b;
};
struct PolyEntry {                    // everything known about one skeleton
  bool failed = false, have_pending = false;
  std::vector<long long> pending;     // the literals of a sighting that no generic function covers yet
  std::vector<PolyGeneric> generics;  // several when the same text moves along more than one line of sizes
};
PolyText poly_scan(const std::string &text);
bool poly_generalize(const PolyEntry &e, const PolyText &second, PolyGeneric &out, std::string &generic_text);
bool poly_match(const PolyGeneric &e, const std::vector<long long> &ints, long long &t);

struct CompilationCache {  // cache.rs:73-101
  std::map<NormalizedKernel, std::shared_ptr<Func>> op_cache;
  std::map<std::vector<ssa::Instr>, std::shared_ptr<Func>> ssa_cache;
  std::unordered_map<std::string, PolyEntry> poly;   // by skeleton of the generated text (+ block size, shared memory)
  bool polymorphic = true;                 // B200 launch policy only
  size_t hits = 0, misses = 0, poly_hits = 0;
};

struct CompiledFunc {  // schedule.rs:209-227
  enum Kind { Kernel, MatMul, Custom } kind = Kernel;
  std::shared_ptr<Func> func;
  Args args;
  LazyBuffer dst, lhs, rhs;
  size_t b = 0, m = 0, n = 0, k = 0;
  bool transpose = false;
  CustomF f;
  bool dyn = false;         // func is a shape-generic kernel: launched with this grid and this value of t
  uint32_t dyn_grid = 0;
  int64_t dyn_t = 0;
};

struct CompiledSchedule {
  std::vector<CompiledFunc> funcs;
  Device *device = nullptr;
  void run() const;  // schedule.rs:233-306
};

struct Schedule {
  std::vector<ScheduleItem> items;
  std::map<ArgId, LazyBuffer> per_arg_id;
  Device *device = nullptr;

  static Schedule create(const std::vector<LazyBuffer> &buffers);  // schedule.rs:78-101
  static Schedule create_one(const LazyBuffer &b) { return create({b}); }
  CompiledSchedule compile() const { CompilationCache c; return compile_with_cache(c); }
  CompiledSchedule compile_with_cache(CompilationCache &cache) const;  // schedule.rs:115-207
};

// Vectorised CUDA C for row-reduce + map and pure-map kernels (ug_fast.cpp); false = not one of those shapes.
bool fast_kernel(const op::Kernel &optimized, const std::string &name, FastKernel &out);
// Hand-built SSA the model feeds through LB::ssa that has a dedicated kernel: ug-llama's index_select
// (ug-llama/src/model.rs:32-63, two nested loops run by a single thread in the reference).
bool fast_ssa_kernel(const ssa::Kernel &k, FastKernel &out);

// Launch shapes: the reference's heuristic and this backend's.
Opts reference_opts(const op::Kernel &optimized);
Opts b200_opts(const op::Kernel &optimized);

}  // namespace ug
