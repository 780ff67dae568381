// C ABI of the host layer (include/ughost.h) and the adapter that makes the
// B200 library (include/ugb200.h) a ug::Device.
#include <cstdio>

#include "../../../include/ughost.h"
#include "ug_graph.hpp"

using namespace ug;

static thread_local std::string g_err;

struct ugh_device { std::unique_ptr<Device> dev; };
struct ugh_lb { LazyBuffer lb; };
struct ugh_schedule { Schedule s; };
struct ugh_compiled { CompiledSchedule c; };
struct ugh_cache { CompilationCache c; };
struct ugh_slice;  // = ug::Slice

namespace {

// ---------------------------------------------------------- B200 device ----
struct B200Slice : Slice {
  ugb_slice *h = nullptr;
  ~B200Slice() override { if (h) ugb_free(h); }
  DType dtype() const override { return (DType)ugb_slice_dtype(h); }
  size_t len() const override { return ugb_slice_len(h); }
  void copy_host_to_device(const void *src, size_t len, DType dt) override;
  void copy_device_to_host(void *dst, size_t len, DType dt) const override;
  ugb_device *dev = nullptr;
};
struct B200Func : Func {
  ugb_func *h = nullptr;       // a compiled kernel, or null for an operator of the library:
  size_t gather_ids = 0, gather_h = 0;   // ugb_index_select over (table, ids, dst)
  bool empty = false;                    // a store of zero elements: nothing to launch
  ~B200Func() override { if (h) ugb_func_free(h); }
};
void check(ugb_device *d, int32_t rc) {
  if (rc != 0) bail("[ugb status ", rc, "] ", ugb_last_error(d));
}
void B200Slice::copy_host_to_device(const void *src, size_t len, DType dt) { check(dev, ugb_h2d(h, src, len, (int32_t)dt)); }
void B200Slice::copy_device_to_host(void *dst, size_t len, DType dt) const { check(dev, ugb_d2h(h, dst, len, (int32_t)dt)); }

ugb_ssa_arg to_c(const ssa::A &a) {
  ugb_ssa_arg o{};
  o.is_var = a.is_var ? 1 : 0;
  if (a.is_var) { o.value = (int64_t)a.var; return o; }
  o.dtype = (int32_t)a.cst.dtype;
  switch (a.cst.dtype) {
    case DType::F32: { uint32_t b; std::memcpy(&b, &a.cst.f32, 4); o.value = b; break; }
    case DType::I32: o.value = a.cst.i32; break;
    case DType::I64: o.value = a.cst.i64; break;
    default: o.value = a.cst.h; break;
  }
  return o;
}
ssa::A from_c(const ugb_ssa_arg &a) {
  if (a.is_var) return ssa::A::v((size_t)a.value);
  Const c = Const::zero((DType)a.dtype);
  switch ((DType)a.dtype) {
    case DType::F32: { uint32_t b = (uint32_t)a.value; std::memcpy(&c.f32, &b, 4); break; }
    case DType::I32: c.i32 = (int32_t)a.value; break;
    case DType::I64: c.i64 = a.value; break;
    default: c.h = (uint16_t)a.value; break;
  }
  return ssa::A::c(c);
}
// ssa::Instr <-> ugb_ssa_instr.  The enum orders match (checked by static_asserts below).
static_assert((int)ssa::K::DefineAcc == UGB_SSA_DEFINE_ACC && (int)ssa::K::ReduceLocal == UGB_SSA_REDUCE_LOCAL &&
              (int)ssa::K::Store == UGB_SSA_STORE && (int)ssa::K::Range == UGB_SSA_RANGE, "instruction kinds out of sync");
ugb_ssa_instr to_c(const ssa::Instr &i) {
  ugb_ssa_instr o{};
  o.kind = (int32_t)i.kind;
  o.dtype = (int32_t)i.dtype;
  o.index = (int64_t)i.index;
  o.v0 = (int64_t)i.v0;
  o.a0 = to_c(i.a0);
  o.a1 = to_c(i.a1);
  o.cst = to_c(ssa::A::c(i.cst));
  switch (i.kind) {
    case ssa::K::Special: o.op = (int32_t)i.special; break;
    case ssa::K::Unary: o.op = (int32_t)i.uop.kind; if (i.uop.kind == UnaryKind::Cast) o.dtype = (int32_t)i.uop.cast_to; break;
    case ssa::K::Binary: o.op = (int32_t)i.bop; break;
    case ssa::K::ReduceLocal: o.op = (int32_t)i.rop; break;
    default: break;
  }
  return o;
}
ssa::Instr from_c(const ugb_ssa_instr &c) {
  ssa::Instr i;
  i.kind = (ssa::K)c.kind;
  i.dtype = (DType)c.dtype;
  i.index = (size_t)c.index;
  i.v0 = (size_t)c.v0;
  i.a0 = from_c(c.a0);
  i.a1 = from_c(c.a1);
  if (!c.cst.is_var) i.cst = from_c(c.cst).cst;
  switch (i.kind) {
    case ssa::K::Special: i.special = (ssa::Special)c.op; break;
    case ssa::K::Unary: i.uop = UnaryOp{(UnaryKind)c.op, (DType)c.dtype}; break;
    case ssa::K::Binary: i.bop = (BinaryOp)c.op; break;
    case ssa::K::ReduceLocal: i.rop = (ReduceOp)c.op; break;
    default: break;
  }
  return i;
}

struct B200Device : Device {
  ugb_device *d = nullptr;
  LaunchPolicy policy = LaunchPolicy::B200;
  std::unique_ptr<Slice> allocate_uninit(DType dtype, size_t len) override {
    auto s = std::make_unique<B200Slice>();
    s->dev = d;
    check(d, ugb_alloc(d, (int32_t)dtype, len, &s->h));
    return s;
  }
  void synchronize() override { check(d, ugb_sync(d)); }
  std::shared_ptr<Func> compile(const ssa::Kernel &k, const std::string *name) override {
    std::vector<ugb_ssa_instr> ins;
    ins.reserve(k.instrs.size());
    for (auto &i : k.instrs) ins.push_back(to_c(i));
    auto f = std::make_shared<B200Func>();
    check(d, ugb_compile(d, ins.data(), ins.size(), k.launch_config.grid_dim, k.launch_config.block_dim,
                         k.launch_config.shared_mem, name ? name->c_str() : nullptr, &f->h));
    return f;
  }
  std::shared_ptr<Func> compile_cu(const FastKernel &fk) override {
    auto f = std::make_shared<B200Func>();
    if (fk.origin == "index_select") { f->gather_ids = fk.n_ids; f->gather_h = fk.h; return f; }
    if (fk.origin == "empty") { f->empty = true; return f; }
    check(d, ugb_compile_cu(d, fk.source.c_str(), fk.func_name.c_str(), fk.launch.grid_dim, fk.launch.block_dim,
                            fk.launch.shared_mem, &f->h));
    return f;
  }
  bool ssa_source(const ssa::Kernel &k, const std::string &entry, GeneratedSource &out) override {
    std::vector<ugb_ssa_instr> ins;
    ins.reserve(k.instrs.size());
    for (auto &i : k.instrs) ins.push_back(to_c(i));
    std::vector<char> buf(1 << 18);
    int32_t dts[32];
    size_t n_args = 0;
    if (ugb_ssa_source(d, ins.data(), ins.size(), entry.c_str(), buf.data(), buf.size(), dts, 32, &n_args) != 0) return false;
    out.text = buf.data();
    out.arg_dtypes.clear();
    for (size_t i = 0; i < n_args; ++i) out.arg_dtypes.push_back((DType)dts[i]);
    return true;
  }
  std::shared_ptr<Func> compile_generated(const GeneratedSource &g, const std::string &entry, int n_dyn, const LaunchConfig &lc) override {
    std::vector<int32_t> dts;
    for (DType t : g.arg_dtypes) dts.push_back((int32_t)t);
    auto f = std::make_shared<B200Func>();
    check(d, ugb_compile_generated(d, g.text.c_str(), entry.c_str(), dts.data(), dts.size(), n_dyn, lc.grid_dim, lc.block_dim,
                                   lc.shared_mem, &f->h));
    return f;
  }
  void run_dyn(Func &f, std::vector<Slice *> &args, uint32_t grid, const std::vector<int64_t> &dyn) override {
    std::vector<ugb_slice *> hs;
    for (Slice *s : args) {
      auto *b = dynamic_cast<B200Slice *>(s);
      if (!b) bail("run: slice of another device");
      hs.push_back(b->h);
    }
    check(d, ugb_run_dyn(d, static_cast<B200Func &>(f).h, hs.data(), hs.size(), grid, dyn.data(), dyn.size()));
  }
  void run(Func &f, std::vector<Slice *> &args) override {
    std::vector<ugb_slice *> hs;
    for (Slice *s : args) {
      auto *b = dynamic_cast<B200Slice *>(s);
      if (!b) bail("run: slice of another device");
      hs.push_back(b->h);
    }
    auto &bf = static_cast<B200Func &>(f);
    if (bf.empty) return;
    if (!bf.h) {   // the library's row gather: bad ids raise the status word instead of reading out of bounds
      if (hs.size() != 3 || bf.gather_h == 0) bail("index_select takes (table, ids, dst)");
      check(d, ugb_index_select(d, hs[0], hs[1], hs[2], bf.gather_ids, bf.gather_h, ugb_slice_len(hs[0]) / bf.gather_h));
      return;
    }
    check(d, ugb_run(d, bf.h, hs.data(), hs.size()));
  }
  void matmul(Slice &dst, const Slice &lhs, const Slice &rhs, size_t b, size_t m, size_t n, size_t k, const Layout &ll,
              const Layout &rl) override {
    if (ll.rank() != rl.rank()) bail("matmul: operand ranks differ");
    check(d, ugb_matmul(d, static_cast<B200Slice &>(dst).h, static_cast<const B200Slice &>(lhs).h,
                        static_cast<const B200Slice &>(rhs).h, b, m, n, k, (int32_t)ll.rank(), ll.shape.data(),
                        ll.strides.data(), ll.offset, rl.shape.data(), rl.strides.data(), rl.offset));
  }
  bool use_grid() const override { return ugb_use_grid() != 0; }
  LaunchPolicy launch_policy() const override { return policy; }
};

Shape shape_of(const size_t *dims, size_t rank) { return Shape(dims, dims + rank); }

template <typename F> auto guard_ptr(F &&f) -> decltype(f()) {
  try {
    return f();
  } catch (const std::exception &e) {
    g_err = e.what();
    return nullptr;
  }
}
template <typename F> int32_t guard(F &&f) {
  try {
    f();
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}
ugh_lb *wrap(LazyBuffer lb) { return new ugh_lb{std::move(lb)}; }

CustomF make_custom(ugh_custom_fn fn, void *user) {
  return [fn, user](std::vector<Slice *> &slices) {
    std::vector<ugh_slice *> hs;
    for (Slice *s : slices) hs.push_back(reinterpret_cast<ugh_slice *>(s));
    int32_t rc = fn(user, hs.data(), hs.size());
    if (rc != 0) bail("custom op failed with status ", rc);
  };
}
std::vector<LazyBuffer> lbs(ugh_lb *const *args, size_t n) {
  std::vector<LazyBuffer> v;
  for (size_t i = 0; i < n; ++i) v.push_back(args[i]->lb);
  return v;
}
}  // namespace

extern "C" {

const char *ugh_last_error(void) { return g_err.c_str(); }

ugh_device *ugh_device_b200(ugb_device *dev) {
  return guard_ptr([&]() -> ugh_device * {
    if (!dev) bail("ugh_device_b200: null device");
    auto d = std::make_unique<B200Device>();
    d->d = dev;
    return new ugh_device{std::move(d)};
  });
}
int32_t ugh_device_set_launch_policy(ugh_device *dev, int32_t policy) {
  return guard([&] {
    auto *b = dynamic_cast<B200Device *>(dev->dev.get());
    if (!b) bail("launch policy applies to the B200 device only");
    b->policy = policy == 0 ? LaunchPolicy::ReferenceGrid : LaunchPolicy::B200;
  });
}
ugh_device *ugh_device_adopt(void *p) {
  if (!p) { g_err = "ugh_device_adopt: null"; return nullptr; }
  return new ugh_device{std::unique_ptr<Device>(static_cast<Device *>(p))};
}
void ugh_device_free(ugh_device *dev) { delete dev; }
int32_t ugh_device_synchronize(ugh_device *dev) { return guard([&] { dev->dev->synchronize(); }); }
ugb_slice *ugh_slice_b200(ugh_slice *s) {
  auto *b = dynamic_cast<B200Slice *>(reinterpret_cast<Slice *>(s));
  return b ? b->h : nullptr;
}
size_t ugh_slice_len(const ugh_slice *s) { return reinterpret_cast<const Slice *>(s)->len(); }
int32_t ugh_slice_dtype(const ugh_slice *s) { return (int32_t) reinterpret_cast<const Slice *>(s)->dtype(); }

ugh_lb *ugh_lb_cst_f32(float v, const size_t *dims, size_t rank, ugh_device *dev) {
  return guard_ptr([&] { return wrap(LazyBuffer::cst(Const::from_f32(v), shape_of(dims, rank), dev->dev.get())); });
}
ugh_lb *ugh_lb_cst_i32(int32_t v, const size_t *dims, size_t rank, ugh_device *dev) {
  return guard_ptr([&] { return wrap(LazyBuffer::cst(Const::from_i32(v), shape_of(dims, rank), dev->dev.get())); });
}
ugh_lb *ugh_lb_copy(const void *data, size_t len, int32_t dtype, const size_t *dims, size_t rank, ugh_device *dev) {
  return guard_ptr([&] { return wrap(LazyBuffer::copy(data, len, (DType)dtype, shape_of(dims, rank), dev->dev.get())); });
}
ugh_lb *ugh_lb_alloc_uninit(int32_t dtype, const size_t *dims, size_t rank, ugh_device *dev) {
  return guard_ptr([&] { return wrap(LazyBuffer::alloc_uninit((DType)dtype, shape_of(dims, rank), dev->dev.get())); });
}
ugh_lb *ugh_lb_unary(ugh_lb *a, int32_t op) {
  return guard_ptr([&] { return wrap(a->lb.unary(UnaryOp{(UnaryKind)op, DType::F32})); });
}
ugh_lb *ugh_lb_cast(ugh_lb *a, int32_t dtype) { return guard_ptr([&] { return wrap(a->lb.cast((DType)dtype)); }); }
ugh_lb *ugh_lb_binary(ugh_lb *a, int32_t op, ugh_lb *b) {
  return guard_ptr([&] { return wrap(a->lb.binary((BinaryOp)op, b->lb)); });
}
ugh_lb *ugh_lb_reduce(ugh_lb *a, int32_t op, int64_t dim) {
  return guard_ptr([&] { return wrap(a->lb.reduce((ReduceOp)op, (long)dim)); });
}
ugh_lb *ugh_lb_matmul(ugh_lb *a, ugh_lb *b, int32_t t) { return guard_ptr([&] { return wrap(a->lb.matmul_(b->lb, t != 0)); }); }
ugh_lb *ugh_lb_broadcast(ugh_lb *a, const size_t *dims, size_t rank) {
  return guard_ptr([&] { return wrap(a->lb.broadcast(shape_of(dims, rank))); });
}
ugh_lb *ugh_lb_reshape(ugh_lb *a, const size_t *dims, size_t rank) {
  return guard_ptr([&] { return wrap(a->lb.reshape(shape_of(dims, rank))); });
}
ugh_lb *ugh_lb_transpose(ugh_lb *a, int64_t d1, int64_t d2) { return guard_ptr([&] { return wrap(a->lb.transpose((long)d1, (long)d2)); }); }
ugh_lb *ugh_lb_split_dim(ugh_lb *a, int64_t dim, size_t s1, size_t s2) {
  return guard_ptr([&] { return wrap(a->lb.split_dim((long)dim, s1, s2)); });
}
ugh_lb *ugh_lb_merge_dims(ugh_lb *a, int64_t dim) { return guard_ptr([&] { return wrap(a->lb.merge_dims((long)dim)); }); }
ugh_lb *ugh_lb_narrow(ugh_lb *a, int64_t dim, size_t off, size_t len) {
  return guard_ptr([&] { return wrap(a->lb.narrow((long)dim, off, len)); });
}
ugh_lb *ugh_lb_squeeze(ugh_lb *a, int64_t dim) { return guard_ptr([&] { return wrap(a->lb.squeeze((long)dim)); }); }
ugh_lb *ugh_lb_unsqueeze(ugh_lb *a, int64_t dim) { return guard_ptr([&] { return wrap(a->lb.unsqueeze((long)dim)); }); }
ugh_lb *ugh_lb_set(ugh_lb *dst, ugh_lb *values) { return guard_ptr([&] { return wrap(dst->lb.set(values->lb)); }); }
ugh_lb *ugh_lb_set_l(ugh_lb *dst, ugh_lb *values, const size_t *dims, const size_t *strides, size_t rank, size_t offset) {
  return guard_ptr([&] {
    Layout l;
    l.shape = shape_of(dims, rank);
    l.strides.assign(strides, strides + rank);
    l.offset = offset;
    return wrap(dst->lb.set_l(values->lb, l));
  });
}
ugh_lb *ugh_lb_cat(ugh_lb *const *args, size_t n, int64_t dim) {
  return guard_ptr([&] { return wrap(LazyBuffer::cat(lbs(args, n), (long)dim)); });
}
ugh_lb *ugh_lb_custom(ugh_custom_fn fn, void *user, ugh_lb *const *args, size_t n, const size_t *dims, size_t rank,
                      int32_t dtype, ugh_device *dev) {
  return guard_ptr([&] {
    return wrap(LazyBuffer::custom(make_custom(fn, user), lbs(args, n), shape_of(dims, rank), (DType)dtype, dev->dev.get()));
  });
}
ugh_lb *ugh_lb_custom_ip(ugh_lb *src, ugh_custom_fn fn, void *user, ugh_lb *const *args, size_t n) {
  return guard_ptr([&] { return wrap(src->lb.custom_ip(make_custom(fn, user), lbs(args, n))); });
}
ugh_lb *ugh_lb_ssa(const ugb_ssa_instr *instrs, size_t n_instrs, ugh_lb *const *args, size_t n, const size_t *dims,
                   size_t rank, int32_t dtype, ugh_device *dev) {
  return guard_ptr([&] {
    std::vector<ssa::Instr> ins;
    for (size_t i = 0; i < n_instrs; ++i) ins.push_back(from_c(instrs[i]));
    return wrap(LazyBuffer::ssa(ssa::Kernel::from_instrs(std::move(ins)), lbs(args, n), shape_of(dims, rank), (DType)dtype,
                                dev->dev.get()));
  });
}
void ugh_lb_free(ugh_lb *a) { delete a; }

size_t ugh_lb_rank(const ugh_lb *a) { return a->lb->rank(); }
int32_t ugh_lb_dims(const ugh_lb *a, size_t *out) {
  for (size_t i = 0; i < a->lb->rank(); ++i) out[i] = a->lb->shape[i];
  return 0;
}
int32_t ugh_lb_dtype(const ugh_lb *a) { return (int32_t)a->lb->dtype; }
int32_t ugh_lb_realized(const ugh_lb *a) { return a->lb.realized() ? 1 : 0; }
int32_t ugh_lb_realize(ugh_lb *a) { return guard([&] { a->lb.realize(); }); }
int32_t ugh_lb_data(ugh_lb *a, void *dst, size_t len, int32_t dtype) {
  return guard([&] { a->lb.data_vec(dst, len, (DType)dtype); });
}
int32_t ugh_lb_write(ugh_lb *a, const void *src, size_t len, int32_t dtype) {
  return guard([&] {
    if (!a->lb->data->slice) bail("buffer has no storage yet");
    a->lb->data->slice->copy_host_to_device(src, len, (DType)dtype);
  });
}

ugh_schedule *ugh_schedule_create(ugh_lb *const *buffers, size_t n) {
  return guard_ptr([&] { return new ugh_schedule{Schedule::create(lbs(buffers, n))}; });
}
void ugh_schedule_free(ugh_schedule *s) { delete s; }
size_t ugh_schedule_n_items(const ugh_schedule *s) { return s->s.items.size(); }
int32_t ugh_schedule_item_kind(const ugh_schedule *s, size_t i) { return i < s->s.items.size() ? (int32_t)s->s.items[i].kind : -1; }
int32_t ugh_schedule_item_ssa_text(const ugh_schedule *s, size_t i, int32_t policy, char *buf, size_t buf_len) {
  return guard([&] {
    if (i >= s->s.items.size() || s->s.items[i].kind != ScheduleItem::Kernel) bail("item ", i, " is not a kernel");
    op::Kernel k = s->s.items[i].kernel();
    Opts o;
    if (policy >= 0) {
      k = optimize(std::move(k));
      o = policy == 0 ? reference_opts(k) : b200_opts(k);
    }
    std::string t = ssa::to_text(lower(k, o));
    if (t.size() + 1 > buf_len) bail("buffer too small: ", t.size() + 1, " bytes needed");
    std::memcpy(buf, t.c_str(), t.size() + 1);
  });
}
int32_t ugh_schedule_item_fast_source(const ugh_schedule *s, size_t i, char *buf, size_t buf_len) {
  return guard([&] {
    if (i >= s->s.items.size() || s->s.items[i].kind != ScheduleItem::Kernel) bail("item ", i, " is not a kernel");
    op::Kernel k = optimize(s->s.items[i].kernel());
    FastKernel fk;
    std::string t;
    if (fast_kernel(k, "k", fk) && !fk.source.empty())
      t = "// " + fk.origin + " " + fk.func_name + " grid " + std::to_string(fk.launch.grid_dim) + " block " +
          std::to_string(fk.launch.block_dim) + "\n" + fk.source;
    if (t.size() + 1 > buf_len) bail("buffer too small: ", t.size() + 1, " bytes needed");
    std::memcpy(buf, t.c_str(), t.size() + 1);
  });
}
ugh_cache *ugh_cache_create(void) { return new ugh_cache(); }
void ugh_cache_free(ugh_cache *c) { delete c; }
size_t ugh_cache_hits(const ugh_cache *c) { return c->c.hits; }
size_t ugh_cache_misses(const ugh_cache *c) { return c->c.misses; }
size_t ugh_cache_poly_hits(const ugh_cache *c) { return c->c.poly_hits; }
void ugh_cache_set_polymorphic(ugh_cache *c, int32_t on) { c->c.polymorphic = on != 0; }
ugh_compiled *ugh_schedule_compile(const ugh_schedule *s, ugh_cache *cache) {
  return guard_ptr([&] {
    if (cache) return new ugh_compiled{s->s.compile_with_cache(cache->c)};
    return new ugh_compiled{s->s.compile()};
  });
}
void ugh_compiled_free(ugh_compiled *c) { delete c; }
int32_t ugh_compiled_run(const ugh_compiled *c) { return guard([&] { c->c.run(); }); }
size_t ugh_compiled_n_funcs(const ugh_compiled *c) { return c->c.funcs.size(); }
int32_t ugh_compiled_func_origin(const ugh_compiled *c, size_t i, char *buf, size_t buf_len) {
  return guard([&] {
    if (i >= c->c.funcs.size()) bail("no function ", i);
    const CompiledFunc &f = c->c.funcs[i];
    const std::string t = f.kind == CompiledFunc::MatMul ? "matmul" : f.kind == CompiledFunc::Custom ? "custom" : (f.func ? f.func->origin : "?");
    if (t.size() + 1 > buf_len) bail("buffer too small");
    std::memcpy(buf, t.c_str(), t.size() + 1);
  });
}

}  // extern "C"
