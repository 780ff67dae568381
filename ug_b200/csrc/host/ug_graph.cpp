// See ug_graph.hpp.  File:line references name ug-core/src/lazy_buffer.rs and
// ug-core/src/schedule.rs.
#include "ug_graph.hpp"

#include <unordered_set>

#include <algorithm>

namespace ug {

namespace {
size_t fresh_lb_id() {
  static std::atomic<size_t> counter{1};
  return counter.fetch_add(1);
}
LazyBuffer make(Op op, DType dtype, Shape shape, Device *dev, std::shared_ptr<DataCell> data = nullptr) {
  auto in = std::make_shared<LazyBufferInner>();
  in->id = fresh_lb_id();
  in->data = data ? std::move(data) : std::make_shared<DataCell>();
  in->op = std::move(op);
  in->dtype = dtype;
  in->shape = std::move(shape);
  in->device = dev;
  return LazyBuffer{in};
}
}  // namespace

// ---------------------------------------------------------- LazyBuffer ----
bool LazyBuffer::in_place_op() const { return p->op.kind == Op::CustomIp || p->op.kind == Op::Set; }  // lazy_buffer.rs:130-144
bool LazyBuffer::realized() const { return !in_place_op() && p->data->slice != nullptr; }              // :146-154
void LazyBuffer::maybe_allocate_uninit() const {                                                        // :114-124
  if (!p->data->slice) p->data->slice = p->device->allocate_uninit(p->dtype, num_elements(p->shape));
}
void LazyBuffer::realize() const {  // :156-164
  if (realized()) return;
  Schedule::create_one(*this).compile().run();
}
void LazyBuffer::data_vec(void *dst, size_t len, DType dtype) const {  // :170-183
  realize();
  if (!p->data->slice) bail("no data");
  if (len != num_elements(p->shape)) bail("data_vec: destination holds ", len, " elements, buffer has ", num_elements(p->shape));
  p->data->slice->copy_device_to_host(dst, len, dtype);
}

LazyBuffer LazyBuffer::unary(UnaryOp op) const {
  Op o; o.kind = Op::Unary; o.uop = op; o.a0 = *this;
  return make(std::move(o), p->dtype, p->shape, p->device);
}
LazyBuffer LazyBuffer::cast(DType dtype) const {
  if (p->dtype == dtype) return *this;
  Op o; o.kind = Op::Unary; o.uop = UnaryOp{UnaryKind::Cast, dtype}; o.a0 = *this;
  return make(std::move(o), dtype, p->shape, p->device);
}
LazyBuffer LazyBuffer::binary(BinaryOp op, const LazyBuffer &rhs) const {
  if (p->shape != rhs->shape) bail("shape mismatch in binary op, ", shape_str(p->shape), " vs ", shape_str(rhs->shape));
  if (p->dtype != rhs->dtype) bail("dtype mismatch in binary op, ", dtype_str(p->dtype), " vs ", dtype_str(rhs->dtype));
  Op o; o.kind = Op::Binary; o.bop = op; o.a0 = *this; o.a1 = rhs;
  return make(std::move(o), p->dtype, p->shape, p->device);
}
LazyBuffer LazyBuffer::reduce(ReduceOp op, long dim) const {  // the graph-level shape keeps the reduced dim (:455,463)
  Op o; o.kind = Op::Reduce; o.rop = op; o.reduce_dim = to_index(dim, p->shape, "reduce"); o.a0 = *this;
  return make(std::move(o), p->dtype, p->shape, p->device);
}
LazyBuffer LazyBuffer::matmul_(const LazyBuffer &rhs, bool transpose) const {  // :414-451
  const Shape &l = p->shape, &r = rhs->shape;
  const size_t dim = l.size(), rdim = r.size();
  if (dim < 2 || rdim < 2) bail("shape mismatch in matmul ", shape_str(l), " ", shape_str(r));
  const size_t m = l[dim - 2], k = l[dim - 1];
  const size_t k2 = transpose ? r[rdim - 1] : r[rdim - 2], n = transpose ? r[rdim - 2] : r[rdim - 1];
  size_t lb = 1, rb = 1;
  for (size_t i = 0; i + 2 < dim; ++i) lb *= l[i];
  for (size_t i = 0; i + 2 < rdim; ++i) rb *= r[i];
  if (k != k2 || lb != rb) bail("shape mismatch in matmul ", shape_str(l), " ", shape_str(r));
  Shape shape(l.begin(), l.end() - 2);
  shape.push_back(m);
  shape.push_back(n);
  Op o; o.kind = Op::MatMul; o.a0 = *this; o.a1 = rhs; o.b = lb; o.m = m; o.n = n; o.k = k; o.transpose = transpose;
  return make(std::move(o), p->dtype, shape, p->device);
}
LazyBuffer LazyBuffer::split_dim(long dim_, size_t size1, size_t size2) const {  // :473-493
  const size_t dim = to_index(dim_, p->shape, "split_dim");
  Shape dims = p->shape;
  const size_t size = dims[dim];
  if (size1 * size2 != size) bail("unexpected target sizes for split_dim ", dim, ", ", size1, "x", size2, " != ", size);
  dims.erase(dims.begin() + (long)dim);
  dims.insert(dims.begin() + (long)dim, size2);
  dims.insert(dims.begin() + (long)dim, size1);
  Op o; o.kind = Op::Layout; o.lop.kind = op::LayoutOp::SplitDim; o.lop.dim = dim; o.lop.d1 = dim; o.lop.d2 = dim + 1; o.a0 = *this;
  return make(std::move(o), p->dtype, dims, p->device);
}
LazyBuffer LazyBuffer::merge_dims(long dim_) const {  // :496-515
  const size_t dim = to_index(dim_, p->shape, "merge_dims");
  if (dim + 1 >= p->rank()) bail("unexpected dim for merge_dims ", dim, " ", shape_str(p->shape));
  Shape dims = p->shape;
  const size_t sp = dims[dim + 1];
  dims.erase(dims.begin() + (long)dim + 1);
  dims[dim] *= sp;
  Op o; o.kind = Op::Layout; o.lop.kind = op::LayoutOp::MergeDims; o.lop.dim = dim; o.lop.d1 = dim; o.lop.d2 = dim + 1; o.a0 = *this;
  return make(std::move(o), p->dtype, dims, p->device);
}
LazyBuffer LazyBuffer::squeeze(long dim_) const {  // :519-527, errors unless the dim has size 1
  const size_t dim = to_index(dim_, p->shape, "squeeze");
  Shape dims = p->shape;
  if (dims[dim] != 1) bail("cannot squeeze on dim ", dim, " for shape ", shape_str(dims));
  dims.erase(dims.begin() + (long)dim);
  return reshape(dims);
}
LazyBuffer LazyBuffer::unsqueeze(long dim_) const {  // :539-544
  const long r = (long)p->rank();
  long d = dim_ < 0 ? r + 1 + dim_ : dim_;
  if (d < 0 || d > r) bail("dim out of range in 'unsqueeze', dim: ", dim_, ", shape: ", shape_str(p->shape));
  Shape dims = p->shape;
  dims.insert(dims.begin() + d, 1);
  return reshape(dims);
}
LazyBuffer LazyBuffer::reshape(const Shape &s) const {  // :546-567
  if (num_elements(s) != num_elements(p->shape))
    bail("cannot reshape between ", shape_str(p->shape), " (", num_elements(p->shape), " elts) and ", shape_str(s), " (", num_elements(s), " elts)");
  Op o; o.kind = Op::Reshape; o.a0 = *this;
  return make(std::move(o), p->dtype, s, p->device);
}
LazyBuffer LazyBuffer::narrow(long dim_, size_t offset, size_t length) const {  // :569-590
  const size_t dim = to_index(dim_, p->shape, "narrow");
  const size_t size = p->shape[dim];
  if (offset + length > size) bail("cannot narrow, offset ", offset, " + length ", length, " > size ", size);
  if (offset == 0 && length == size) return *this;
  Shape dims = p->shape;
  dims[dim] = length;
  Op o; o.kind = Op::Layout; o.lop.kind = op::LayoutOp::Narrow; o.lop.dim = dim; o.lop.offset = offset; o.a0 = *this;
  return make(std::move(o), p->dtype, dims, p->device);
}
LazyBuffer LazyBuffer::broadcast(const Shape &s) const {  // :592-623
  if (p->rank() > s.size()) bail("target shape ", shape_str(s), " has less dimensions than original shape ", shape_str(p->shape));
  Op o; o.kind = Op::Layout; o.lop.kind = op::LayoutOp::Broadcast; o.a0 = *this;
  o.lop.inserted_dims = s.size() - p->rank();
  for (size_t i = 0; i < o.lop.inserted_dims; ++i) o.lop.broadcasted_dims.push_back(i);
  for (size_t i = 0; i < p->rank(); ++i) {
    const size_t di = i + o.lop.inserted_dims;
    if (s[di] != p->shape[i]) {
      if (p->shape[i] == 1) o.lop.broadcasted_dims.push_back(di);
      else bail("cannot broadcast from ", shape_str(p->shape), " to ", shape_str(s));
    }
  }
  return make(std::move(o), p->dtype, s, p->device);
}
LazyBuffer LazyBuffer::transpose(long dim1_, long dim2_) const {  // :625-644
  const size_t d1 = to_index(dim1_, p->shape, "transpose"), d2 = to_index(dim2_, p->shape, "transpose");
  if (d1 == d2) return *this;
  Shape dims = p->shape;
  std::swap(dims[d1], dims[d2]);
  Op o; o.kind = Op::Layout; o.lop.kind = op::LayoutOp::Transpose; o.lop.d1 = d1; o.lop.d2 = d2; o.a0 = *this;
  return make(std::move(o), p->dtype, dims, p->device);
}
LazyBuffer LazyBuffer::custom_ip(CustomF f, std::vector<LazyBuffer> args) const {  // :313-330, shares the storage cell
  Op o; o.kind = Op::CustomIp; o.f = std::move(f); o.args = std::move(args); o.a0 = *this;
  return make(std::move(o), p->dtype, p->shape, p->device, p->data);
}
LazyBuffer LazyBuffer::set(const LazyBuffer &values) const {  // :333-351
  if (p->shape != values->shape) bail("shape mismatch in set, ", shape_str(p->shape), " vs ", shape_str(values->shape));
  if (p->dtype != values->dtype) bail("dtype mismatch in set, ", dtype_str(p->dtype), " vs ", dtype_str(values->dtype));
  Op o; o.kind = Op::Set; o.a0 = *this; o.a1 = values; o.dst_layout = Layout::from_shape(p->shape);
  return make(std::move(o), p->dtype, p->shape, p->device, p->data);
}
LazyBuffer LazyBuffer::set_l(const LazyBuffer &values, const Layout &dst_layout) const {  // :353-388
  size_t max_off = dst_layout.offset;
  for (size_t i = 0; i < dst_layout.rank(); ++i) max_off += (dst_layout.shape[i] ? dst_layout.shape[i] - 1 : 0) * dst_layout.strides[i];
  if (max_off >= num_elements(p->shape)) bail("set_l out of bounds, dst shape ", shape_str(p->shape), ", max off ", max_off);
  if (dst_layout.num_elements() != num_elements(values->shape)) bail("set_l mismatch between the values shape ", shape_str(values->shape), " and layout");
  if (p->dtype != values->dtype) bail("dtype mismatch in set, ", dtype_str(p->dtype), " vs ", dtype_str(values->dtype));
  Op o; o.kind = Op::Set; o.a0 = *this; o.a1 = values; o.dst_layout = dst_layout;
  return make(std::move(o), p->dtype, p->shape, p->device, p->data);
}
LazyBuffer LazyBuffer::alloc_uninit(DType dtype, const Shape &s, Device *dev) {
  Op o; o.kind = Op::Value;
  return make(std::move(o), dtype, s, dev);
}
LazyBuffer LazyBuffer::cst(Const c, const Shape &s, Device *dev) {  // :646-668
  Op o; o.kind = Op::Const; o.cst = c;
  return make(std::move(o), c.dtype, s, dev);
}
LazyBuffer LazyBuffer::from_slice(std::unique_ptr<Slice> data, const Shape &s, Device *dev) {  // :670-691
  if (num_elements(s) != data->len()) bail("unexpected number of elements ", data->len(), " for shape ", shape_str(s));
  Op o; o.kind = Op::Value;
  DType dt = data->dtype();
  auto cell = std::make_shared<DataCell>();
  cell->slice = std::move(data);
  return make(std::move(o), dt, s, dev, cell);
}
LazyBuffer LazyBuffer::copy(const void *data, size_t len, DType dtype, const Shape &s, Device *dev) {  // :693-728
  if (num_elements(s) != len) bail("unexpected number of elements ", len, " for shape ", shape_str(s));
  auto slice = dev->allocate_uninit(dtype, len);
  slice->copy_host_to_device(data, len, dtype);
  return from_slice(std::move(slice), s, dev);
}
LazyBuffer LazyBuffer::custom(CustomF f, std::vector<LazyBuffer> args, const Shape &s, DType dtype, Device *dev) {  // :292-310
  Op o; o.kind = Op::Custom; o.f = std::move(f); o.args = std::move(args);
  return make(std::move(o), dtype, s, dev);
}
LazyBuffer LazyBuffer::ssa(ssa::Kernel k, std::vector<LazyBuffer> args, const Shape &s, DType dtype, Device *dev) {  // :390-408
  Op o; o.kind = Op::Ssa; o.ssa_kernel = std::move(k); o.args = std::move(args);
  return make(std::move(o), dtype, s, dev);
}
// :730-765.  Each piece is written with a contiguous layout of its own shape at
// an element offset, which is only a concatenation for the outermost axis (the
// reference's test pins that behaviour, ug-core/src/common_tests.rs:31-33).
LazyBuffer LazyBuffer::cat(const std::vector<LazyBuffer> &args, long dim_) {
  if (args.empty()) bail("empty list in cat");
  const LazyBuffer &a0 = args[0];
  if (args.size() == 1) return a0;
  const size_t dim = to_index(dim_, a0->shape, "cat");
  Shape dims = a0->shape;
  dims[dim] = 0;
  for (size_t i = 0; i < args.size(); ++i) {
    const LazyBuffer &a = args[i];
    if (a->dtype != a0->dtype) bail("mismatch between dtypes in cat");
    if (a->rank() != a0->rank()) bail("mismatch between ranks in cat");
    dims[dim] += a->shape[dim];
    for (size_t d = 0; d < dims.size(); ++d)
      if (d != dim && dims[d] != a->shape[d]) bail("mismatch between shapes in cat on dim ", dim, ", arg0: ", shape_str(a0->shape), ", arg", i, ": ", shape_str(a->shape));
  }
  size_t stride = 1;
  for (size_t d = dim + 1; d < dims.size(); ++d) stride *= dims[d];
  size_t offset = 0;
  LazyBuffer vs = alloc_uninit(a0->dtype, dims, a0->device);
  for (const LazyBuffer &a : args) {
    Layout l = Layout::from_shape(a->shape);
    l.offset = offset * stride;
    vs = vs.set_l(a, l);
    offset += a->shape[dim];
  }
  return vs;
}

// ------------------------------------------------------------- schedule ----
op::Kernel ScheduleItem::kernel() const {
  op::Kernel k;
  for (auto &[id, lb] : args) k.args.push_back(Arg{id, lb->dtype});
  Layout l = has_dst_layout ? dst_layout : Layout::from_shape(dst.second->shape);
  k.ops.push_back(op::Store{dst.first, l, ast});
  k.name = "realize_" + std::to_string(dst.second->id);
  return k;
}

namespace {
// schedule.rs:480-520: 1 = used once, 2 = used twice or more; realized nodes stop the walk.
void id_cnts(const LazyBuffer &b, std::unordered_map<size_t, size_t> &cnts) {
  if (b.realized()) return;
  size_t &c = cnts[b->id];
  c += 1;
  if (c > 1) return;
  const Op &o = b->op;
  switch (o.kind) {
    case Op::Value: case Op::Const: break;
    case Op::Reshape: case Op::Layout: case Op::Reduce: case Op::Unary: id_cnts(o.a0, cnts); break;
    case Op::Set: case Op::MatMul: case Op::Binary: id_cnts(o.a0, cnts); id_cnts(o.a1, cnts); break;
    case Op::CustomIp:
      for (auto &a : o.args) id_cnts(a, cnts);
      id_cnts(o.a0, cnts);
      break;
    case Op::Ssa: case Op::Custom:
      for (auto &a : o.args) id_cnts(a, cnts);
      break;
  }
}

bool fusable(const Op &o) {
  return o.kind == Op::Unary || o.kind == Op::Binary || o.kind == Op::Reduce || o.kind == Op::Layout || o.kind == Op::Const;
}

struct Context {  // schedule.rs:308-475
  // This backend's addition to the cut rule of schedule.rs:429-435 (a node with several users gets a kernel of
  // its own): when ALL users of such a node end up inside one and the same fused kernel, materialising it would
  // only buy an HBM round trip -- `exp(x - max)` of model.rs:98-100 feeds the sum and the division of the same
  // softmax row -- so the node is evaluated in place (twice, from registers) and the row is read and written once.
  bool fuse_private = false;
  std::unordered_set<size_t> inlined;
  // number of edges into every node reached from `b` without crossing a cut
  void region_edges(const LazyBuffer &b, bool root, std::unordered_map<size_t, size_t> &seen, std::unordered_set<size_t> &multi) const {
    if (b.realized()) return;
    if (!root) {
      size_t &c = seen[b->id];
      c += 1;
      if (c > 1) return;
      auto it = cnts.find(b->id);
      if (it != cnts.end() && it->second > 1 && !inlined.count(b->id)) { multi.insert(b->id); return; }   // a cut (so far)
    }
    const Op &o = b->op;
    if (!fusable(o)) return;
    if (o.a0) region_edges(o.a0, false, seen, multi);
    if (o.kind == Op::Binary && o.a1) region_edges(o.a1, false, seen, multi);
  }
  void find_private(const LazyBuffer &root) {
    if (!fuse_private || root.realized() || !fusable(root->op)) return;
    for (int round = 0; round < 8; ++round) {
      std::unordered_map<size_t, size_t> seen;
      std::unordered_set<size_t> multi;
      region_edges(root, true, seen, multi);
      bool changed = false;
      for (size_t id : multi)
        if (seen[id] == cnts[id] && inlined.size() < 64) { inlined.insert(id); changed = true; }
      if (!changed) break;
    }
  }
  std::vector<ScheduleItem> items;
  std::map<ArgId, LazyBuffer> per_arg_id;
  std::unordered_map<size_t, op::AstP> ast_cache;
  std::unordered_map<size_t, size_t> cnts;

  const LazyBuffer &get_arg(ArgId id) const {
    auto it = per_arg_id.find(id);
    if (it == per_arg_id.end()) bail("no arg for id ", id.v);
    return it->second;
  }

  ArgId push_kernel(const LazyBuffer &buffer, op::AstP ast, const Layout *dst_layout) {
    if (ast->kind == op::AstNode::Load) {
      // load x -> store x is a no-op (schedule.rs:446-453)
      if (get_arg(ast->load_src)->data.get() == buffer->data.get()) return ast->load_src;
    }
    ArgId dst_id = ArgId::fresh();
    per_arg_id[dst_id] = buffer;
    std::set<ArgId> ids;
    op::arg_ids(ast, ids);
    ids.insert(dst_id);
    ScheduleItem si;
    si.kind = ScheduleItem::Kernel;
    for (ArgId id : ids) si.args.push_back({id, get_arg(id)});   // ascending ArgId (schedule.rs:457-465)
    si.ast = std::move(ast);
    si.dst = {dst_id, buffer};
    if (dst_layout) { si.has_dst_layout = true; si.dst_layout = *dst_layout; }
    items.push_back(std::move(si));
    return dst_id;
  }
  ArgId push_schedule_item(const LazyBuffer &b) {
    find_private(b);
    return push_kernel(b, walk(b), nullptr);
  }

  op::AstP load_of(ArgId id, const LazyBuffer &b) { return op::load(id, Layout::from_shape(b->shape), b->dtype); }

  op::AstP walk(const LazyBuffer &b) {
    auto cached = ast_cache.find(b->id);
    if (cached != ast_cache.end()) return cached->second;
    op::AstP ast;
    if (b.realized()) {
      ArgId id = ArgId::fresh();
      per_arg_id[id] = b;
      ast = load_of(id, b);
    } else {
      const Op &o = b->op;
      switch (o.kind) {
        case Op::Unary: ast = op::unary(o.uop, walk(o.a0)); break;
        case Op::Binary: { auto l = walk(o.a0); auto r = walk(o.a1); ast = op::binary(o.bop, l, r); break; }
        case Op::MatMul: {  // never fused (schedule.rs:352-367)
          push_schedule_item(o.a0);
          push_schedule_item(o.a1);
          ArgId dst = ArgId::fresh();
          per_arg_id[dst] = b;
          ScheduleItem si;
          si.kind = ScheduleItem::MatMul;
          si.mm_dst = b; si.lhs = o.a0; si.rhs = o.a1; si.b = o.b; si.m = o.m; si.n = o.n; si.k = o.k; si.transpose = o.transpose;
          items.push_back(std::move(si));
          ast = load_of(dst, b);
          break;
        }
        case Op::Reduce: ast = op::reduce(o.rop, walk(o.a0), o.reduce_dim); break;
        case Op::Const: ast = op::cst(o.cst); break;
        case Op::Value: { ArgId id = ArgId::fresh(); per_arg_id[id] = b; ast = load_of(id, b); break; }
        case Op::Reshape: { ArgId id = push_schedule_item(o.a0); ast = load_of(id, b); break; }
        case Op::Layout: ast = op::layout(o.lop, walk(o.a0), b->shape); break;
        case Op::Ssa: {
          ScheduleItem si;
          si.kind = ScheduleItem::Ssa;
          for (auto &a : o.args) si.args.push_back({push_schedule_item(a), a});
          ArgId dst = ArgId::fresh();
          per_arg_id[dst] = b;
          si.args.push_back({dst, b});
          si.ssa_kernel = o.ssa_kernel;
          items.push_back(std::move(si));
          ast = load_of(dst, b);
          break;
        }
        case Op::Set: {
          ArgId id = push_schedule_item(o.a0);
          op::AstP values = walk(o.a1);
          push_kernel(o.a0, values, &o.dst_layout);
          ast = load_of(id, b);
          break;
        }
        case Op::CustomIp: {
          ScheduleItem si;
          si.kind = ScheduleItem::Custom;
          for (auto &a : o.args) si.args.push_back({push_schedule_item(a), a});
          ArgId id = push_schedule_item(o.a0);
          si.args.push_back({id, o.a0});
          si.f = o.f;
          items.push_back(std::move(si));
          ast = load_of(id, b);
          break;
        }
        case Op::Custom: {
          ScheduleItem si;
          si.kind = ScheduleItem::Custom;
          for (auto &a : o.args) si.args.push_back({push_schedule_item(a), a});
          ArgId dst = ArgId::fresh();
          per_arg_id[dst] = b;
          si.args.push_back({dst, b});
          si.f = o.f;
          items.push_back(std::move(si));
          ast = load_of(dst, b);
          break;
        }
      }
    }
    // a subtree with more than one user gets a kernel of its own (schedule.rs:429-435)
    auto c = cnts.find(b->id);
    if (c != cnts.end() && c->second > 1 && !inlined.count(b->id)) {
      ArgId dst = push_kernel(b, ast, nullptr);
      ast = load_of(dst, b);
    }
    ast_cache[b->id] = ast;
    return ast;
  }
};
}  // namespace

Schedule Schedule::create(const std::vector<LazyBuffer> &buffers) {
  if (buffers.empty()) bail("no buffers provided");
  Context ctx;
  ctx.fuse_private = buffers[0]->device->launch_policy() == LaunchPolicy::B200;
  for (auto &b : buffers) id_cnts(b, ctx.cnts);
  for (auto &b : buffers) ctx.push_schedule_item(b);
  Schedule s;
  s.items = std::move(ctx.items);
  s.per_arg_id = std::move(ctx.per_arg_id);
  s.device = buffers[0]->device;
  return s;
}

// schedule.rs:162-188 as written: block axis = the largest dim, 32 threads on the
// second largest; a kernel with a single non-unit dim gets a global axis only when it
// has more than one dim; everything else (in particular a pure map that optimize()
// collapsed to one dim) runs as one thread.
Opts reference_opts(const op::Kernel &k) {
  if (!(k.ops.size() == 1 && k.ops[0].layout.rank() >= 1 && k.ops[0].layout.num_elements() >= 1)) return Opts{};
  std::vector<std::pair<size_t, size_t>> dims;
  for (size_t i = 0; i < k.ops[0].layout.rank(); ++i) dims.push_back({i, k.ops[0].layout.shape[i]});
  std::stable_sort(dims.begin(), dims.end(), [](auto &a, auto &b) { return a.second > b.second; });
  if (dims.size() >= 2 && dims[1].second > 1) return Opts{}.with_block_axis(dims[0].first).with_thread_block(dims[1].first, 32);
  if (dims.size() > 1 && dims[0].second > 1) return Opts{}.with_global_axis(dims[0].first, 32);
  return Opts{};
}

namespace {
void collect_reduce_dims(const op::AstP &a, std::set<size_t> &dims) {
  switch (a->kind) {
    case op::AstNode::Reduce: dims.insert(a->reduce_dim); collect_reduce_dims(a->arg, dims); break;
    case op::AstNode::Unary: case op::AstNode::Layout: collect_reduce_dims(a->arg, dims); break;
    case op::AstNode::Binary: collect_reduce_dims(a->arg, dims); collect_reduce_dims(a->rhs, dims); break;
    default: break;
  }
}
}  // namespace

// Launch shapes of this backend.
//  * a pure map collapsed to one dim: one thread per element, 256-thread blocks
//    (the reference runs it as a single thread);
//  * reductions over the last dim only (softmax, rms_norm rows): one block per index
//    of the largest other dim, 256 threads striding the reduced dim, each reduction
//    evaluated once per row before the loop over the row (Opts::hoist_row_reduces) and
//    finished by a block-wide ReduceLocal -- O(rows * cols) work, coalesced accesses;
//  * anything else: the reference shape with 256 instead of 32 threads.
Opts b200_opts(const op::Kernel &k) {
  if (!(k.ops.size() == 1 && k.ops[0].layout.rank() >= 1 && k.ops[0].layout.num_elements() >= 1)) return Opts{};
  const Layout &l = k.ops[0].layout;
  if (l.rank() == 1) return l.shape[0] > 1 ? Opts{}.with_global_axis(0, 256) : Opts{};
  std::set<size_t> rdims;
  collect_reduce_dims(k.ops[0].value, rdims);
  const size_t last = l.rank() - 1;
  if (rdims.size() == 1 && *rdims.begin() == last && l.shape[last] > 1) {
    size_t best = 0, best_len = 0;
    for (size_t i = 0; i < last; ++i)
      if (l.shape[i] > best_len) { best = i; best_len = l.shape[i]; }
    Opts o = Opts{}.with_block_axis(best).with_thread_block(last, 256);
    o.hoist_row_reduces = true;
    return o;
  }
  if (!rdims.empty()) return reference_opts(k);
  std::vector<std::pair<size_t, size_t>> dims;
  for (size_t i = 0; i < l.rank(); ++i) dims.push_back({i, l.shape[i]});
  std::stable_sort(dims.begin(), dims.end(), [](auto &a, auto &b) { return a.second > b.second; });
  if (dims.size() >= 2 && dims[1].second > 1) return Opts{}.with_block_axis(dims[0].first).with_thread_block(dims[1].first, 256);
  if (dims[0].second > 1) return Opts{}.with_global_axis(dims[0].first, 256);
  return Opts{};
}

CompiledSchedule Schedule::compile_with_cache(CompilationCache &cache) const {
  CompiledSchedule out;
  out.device = device;
  for (const ScheduleItem &item : items) {
    CompiledFunc cf;
    switch (item.kind) {
      case ScheduleItem::MatMul:
        cf.kind = CompiledFunc::MatMul;
        cf.dst = item.mm_dst; cf.lhs = item.lhs; cf.rhs = item.rhs;
        cf.b = item.b; cf.m = item.m; cf.n = item.n; cf.k = item.k; cf.transpose = item.transpose;
        break;
      case ScheduleItem::Custom:
        cf.kind = CompiledFunc::Custom;
        cf.f = item.f;
        cf.args = item.args;
        break;
      case ScheduleItem::Ssa: {
        cf.kind = CompiledFunc::Kernel;
        cf.args = item.args;
        auto it = cache.ssa_cache.find(item.ssa_kernel.instrs);
        if (it != cache.ssa_cache.end()) { cf.func = it->second; cache.hits++; }
        else {
          FastKernel fk;
          if (device->launch_policy() == LaunchPolicy::B200 && fast_ssa_kernel(item.ssa_kernel, fk)) {
            cf.func = device->compile_cu(fk);
            if (cf.func) cf.func->origin = fk.origin;
          }
          if (!cf.func) cf.func = device->compile(item.ssa_kernel, nullptr);
          cache.ssa_cache[item.ssa_kernel.instrs] = cf.func;
          cache.misses++;
        }
        break;
      }
      case ScheduleItem::Kernel: {
        cf.kind = CompiledFunc::Kernel;
        op::Kernel kernel = item.kernel();
        NormalizedKernel norm(kernel);
        for (const Arg &a : kernel.args) {
          auto it = per_arg_id.find(a.id);
          if (it == per_arg_id.end()) bail("no arg for id ", a.id.v);
          cf.args.push_back({a.id, it->second});
        }
        auto it = cache.op_cache.find(norm);
        if (it != cache.op_cache.end()) { cf.func = it->second; cache.hits++; break; }
        const std::string name = kernel.ops.empty() ? std::string() : kernel.ops[0].name();
        kernel = optimize(std::move(kernel));
        if (device->launch_policy() == LaunchPolicy::B200 && cache.polymorphic) {
          // the same kernel at another size (see ug_poly.cpp): reuse, or build, the function that takes the size at run time
          const ssa::Kernel poly_k = lower(kernel, b200_opts(kernel));
          GeneratedSource gs;
          if (device->ssa_source(poly_k, "ug_poly_kernel", gs)) {
            PolyText txt = poly_scan(gs.text);
            const uint32_t grid = poly_k.launch_config.grid_dim;
            // the map key: the skeleton followed by the launch shape (no marks in the suffix; text_len says where it starts)
            std::string &key = txt.skeleton;
            key += '|'; key += std::to_string(poly_k.launch_config.block_dim);
            key += '|'; key += std::to_string(poly_k.launch_config.shared_mem);
            auto pit = cache.poly.find(key);
            if (pit == cache.poly.end()) pit = cache.poly.emplace(key, PolyEntry{}).first;
            PolyEntry &pe = pit->second;
            long long t = 0;
            bool served = false;
            for (const PolyGeneric &g : pe.generics)
              if (poly_match(g, txt.ints, t)) {
                cf.func = g.func; cf.dyn = true; cf.dyn_grid = grid; cf.dyn_t = t;
                cache.hits++; cache.poly_hits++;
                served = true;
                break;
              }
            if (served) break;
            if (!pe.failed && pe.have_pending && pe.generics.size() < 8) {
              std::string generic;
              PolyGeneric g;
              bool ok = poly_generalize(pe, txt, g, generic);
              const std::string sig = "ugb_status_word* ugb_status) {";
              const size_t at = ok ? generic.find(sig) : std::string::npos;
              ok = ok && at != std::string::npos;
              if (ok) {
                generic.replace(at, sig.size(), "ugb_status_word* ugb_status, const long long ugp_t) {");
                GeneratedSource g2{generic, gs.arg_dtypes};
                try { g.func = device->compile_generated(g2, "ug_poly_kernel", 1, poly_k.launch_config); }
                catch (const Error &) { g.func = nullptr; }   // a literal the compiler needs as a constant: per-shape kernels
                ok = (bool)g.func;
              }
              if (ok) {
                g.func->origin = "ssa_generic";
                cf.func = g.func; cf.dyn = true; cf.dyn_grid = grid; cf.dyn_t = 1;
                pe.generics.push_back(std::move(g));
                pe.pending.clear();
                pe.have_pending = false;
                cache.misses++;
                break;
              }
              pe.failed = true;
            }
            if (!pe.have_pending) { pe.pending = std::move(txt.ints); pe.have_pending = true; }
          }
        }
        if (device->launch_policy() == LaunchPolicy::B200) {
          // row-reduce + map and pure-map kernels run on generated 128-bit code; everything else on the SSA path
          FastKernel fk;
          if (fast_kernel(kernel, name.empty() ? "k" : name, fk)) {
            cf.func = device->compile_cu(fk);
            if (cf.func) {
              cf.func->origin = fk.origin;
              cache.op_cache.emplace(std::move(norm), cf.func);
              cache.misses++;
              break;
            }
          }
        }
        Opts opts;
        switch (device->launch_policy()) {
          case LaunchPolicy::Sequential: break;
          case LaunchPolicy::ReferenceGrid: opts = reference_opts(kernel); break;
          case LaunchPolicy::B200: opts = b200_opts(kernel); break;
        }
        ssa::Kernel ssa_k = lower(kernel, opts);
        cf.func = device->compile(ssa_k, name.empty() ? nullptr : &name);
        cache.op_cache.emplace(std::move(norm), cf.func);
        cache.misses++;
        break;
      }
    }
    out.funcs.push_back(std::move(cf));
  }
  return out;
}

void CompiledSchedule::run() const {
  for (const CompiledFunc &f : funcs) {
    switch (f.kind) {
      case CompiledFunc::Kernel: {
        std::vector<Slice *> bs;
        for (auto &[id, lb] : f.args) { lb.maybe_allocate_uninit(); bs.push_back(lb->data->slice.get()); }
        if (f.dyn) device->run_dyn(*f.func, bs, f.dyn_grid, {f.dyn_t});
        else device->run(*f.func, bs);
        break;
      }
      case CompiledFunc::MatMul: {  // schedule.rs:256-288: operand layouts come from the shapes, padded with leading 1s
        Shape ld = f.lhs->shape, rd = f.rhs->shape;
        while (ld.size() < rd.size()) ld.insert(ld.begin(), 1);
        while (rd.size() < ld.size()) rd.insert(rd.begin(), 1);
        Layout ll = Layout::from_shape(ld), rl = Layout::from_shape(rd);
        if (f.transpose) rl = rl.transpose();
        f.dst.maybe_allocate_uninit();
        f.lhs.maybe_allocate_uninit();
        f.rhs.maybe_allocate_uninit();
        device->matmul(*f.dst->data->slice, *f.lhs->data->slice, *f.rhs->data->slice, f.b, f.m, f.n, f.k, ll, rl);
        break;
      }
      case CompiledFunc::Custom: {
        std::vector<Slice *> bs;
        for (auto &[id, lb] : f.args) { lb.maybe_allocate_uninit(); bs.push_back(lb->data->slice.get()); }
        f.f(bs);
        break;
      }
    }
  }
}

}  // namespace ug
