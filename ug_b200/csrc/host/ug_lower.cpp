// See ug_lower.hpp.  File:line references are to ug-core/src/lower_op.rs unless
// stated otherwise.
#include "ug_lower.hpp"

#include <algorithm>

namespace ug {

using block::Block;
using ssa::A;
using ssa::Instr;
using ssa::K;

// ------------------------------------------------------ index formulas ----
// :51-124.  A tree giving the index on one dimension of the data being read as
// a function of the loop variables of the enclosing store.
namespace {
struct IndexFormula;
using IF = std::shared_ptr<const IndexFormula>;
struct IndexFormula {
  enum Kind { Id, Const, Add, Mul, Div, Mod } kind = Const;
  block::Id id = 0;
  size_t c = 0;
  IF lhs, rhs;
};
IF f_id(block::Id id) { auto f = std::make_shared<IndexFormula>(); f->kind = IndexFormula::Id; f->id = id; return f; }
IF f_const(size_t c) { auto f = std::make_shared<IndexFormula>(); f->kind = IndexFormula::Const; f->c = c; return f; }
IF f_add(IF l, IF r) { auto f = std::make_shared<IndexFormula>(); f->kind = IndexFormula::Add; f->lhs = l; f->rhs = r; return f; }
IF f_bin(IndexFormula::Kind k, IF l, size_t c) { auto f = std::make_shared<IndexFormula>(); f->kind = k; f->lhs = l; f->c = c; return f; }

// :90-123, indexes are i32.
block::Id eval(const IF &f, Block &b) {
  switch (f->kind) {
    case IndexFormula::Id: return f->id;
    case IndexFormula::Const: return b.cst_i32((int32_t)f->c);
    case IndexFormula::Add: {
      block::Id l = eval(f->lhs, b), r = eval(f->rhs, b);
      return b.binary(BinaryOp::Add, A::v(l), A::v(r), DType::I32);
    }
    case IndexFormula::Mul: return b.mul(eval(f->lhs, b), (int32_t)f->c);
    case IndexFormula::Div:
      if (f->c == 1) return eval(f->lhs, b);
      return b.binary(BinaryOp::Div, A::v(eval(f->lhs, b)), A::i32((int32_t)f->c), DType::I32);
    case IndexFormula::Mod:
      if (f->c == 1) return b.cst_i32(0);
      return b.binary(BinaryOp::Mod, A::v(eval(f->lhs, b)), A::i32((int32_t)f->c), DType::I32);
  }
  return 0;
}

using Indexes = std::vector<IF>;

// :131-200
Indexes layout_op(const Indexes &in, const op::LayoutOp &op, const Shape &shape, const Shape &arg_shape) {
  Indexes idxs = in;
  using L = op::LayoutOp;
  switch (op.kind) {
    case L::Broadcast:
      for (size_t d : op.broadcasted_dims) {
        if (d >= idxs.size()) bail("unexpected dim for broadcast, ", d, " ", shape_str(shape));
        idxs[d] = f_const(0);
      }
      idxs.erase(idxs.begin(), idxs.begin() + (long)op.inserted_dims);
      break;
    case L::Narrow:
      if (op.dim >= idxs.size()) bail("unexpected dim for narrow, ", op.dim, " ", shape_str(shape));
      idxs[op.dim] = f_add(idxs[op.dim], f_const(op.offset));
      break;
    case L::Transpose:
      if (op.d1 >= idxs.size() || op.d2 >= idxs.size()) bail("unexpected dims for transpose ", op.d1, " ", op.d2);
      std::swap(idxs[op.d1], idxs[op.d2]);
      break;
    case L::SplitDim: {
      const size_t lhs = op.d1, rhs = op.d2;
      if (op.dim >= arg_shape.size()) bail("unexpected split dim ", op.dim);
      if (lhs >= shape.size() || rhs >= shape.size() || lhs == rhs) bail("unexpected split dims ", lhs, "x", rhs);
      IF l, r;
      if (lhs < rhs) { r = idxs[rhs]; idxs.erase(idxs.begin() + (long)rhs); l = idxs[lhs]; idxs.erase(idxs.begin() + (long)lhs); }
      else { l = idxs[lhs]; idxs.erase(idxs.begin() + (long)lhs); r = idxs[rhs]; idxs.erase(idxs.begin() + (long)rhs); }
      idxs.insert(idxs.begin() + (long)op.dim, f_add(f_bin(IndexFormula::Mul, l, shape[rhs]), r));
      break;
    }
    case L::MergeDims: {
      const size_t lhs = op.d1, rhs = op.d2;
      if (op.dim >= shape.size()) bail("unexpected merge dim ", op.dim);
      if (lhs >= arg_shape.size() || rhs >= arg_shape.size() || lhs == rhs) bail("unexpected merge dims ", lhs, "x", rhs);
      IF idx = idxs[op.dim];
      idxs.erase(idxs.begin() + (long)op.dim);
      // C layout: lhs is the outer of the two merged dims
      IF lhs_idx = arg_shape[lhs] <= 1 ? f_const(0) : f_bin(IndexFormula::Div, idx, arg_shape[rhs]);
      IF rhs_idx = arg_shape[rhs] <= 1 ? f_const(0) : f_bin(IndexFormula::Mod, idx, arg_shape[rhs]);
      if (lhs < rhs) { idxs.insert(idxs.begin() + (long)lhs, lhs_idx); idxs.insert(idxs.begin() + (long)rhs, rhs_idx); }
      else { idxs.insert(idxs.begin() + (long)rhs, rhs_idx); idxs.insert(idxs.begin() + (long)lhs, lhs_idx); }
      break;
    }
  }
  return idxs;
}

// :205-232: offset = sum idx * stride (+ layout offset), `* 1` elided.
std::pair<block::Id, Block> lower_layout(const Layout &l, const Indexes &idxs) {
  if (idxs.size() != l.strides.size()) bail("len mismatch between strides and idxs");
  Block b;
  bool have = false;
  block::Id acc = 0;
  if (l.offset != 0) { acc = b.cst_i32((int32_t)l.offset); have = true; }
  for (size_t i = 0; i < idxs.size(); ++i) {
    block::Id d = eval(idxs[i], b);
    d = b.mul(d, (int32_t)l.strides[i]);
    if (have) d = b.binary(BinaryOp::Add, A::v(d), A::v(acc), DType::I32);
    acc = d;
    have = true;
  }
  if (!have) acc = b.cst_i32(0);
  return {acc, std::move(b)};
}

Const reduce_init(ReduceOp op, DType dt) {  // :234-242
  switch (op) {
    case ReduceOp::Sum: return Const::zero(dt);
    case ReduceOp::Min: return Const::max_value(dt);
    case ReduceOp::Max: return Const::min_value(dt);
  }
  return Const::zero(dt);
}
BinaryOp reduce_fold(ReduceOp op) {  // :243-249
  return op == ReduceOp::Sum ? BinaryOp::Add : (op == ReduceOp::Max ? BinaryOp::Max : BinaryOp::Min);
}

// :251-298: reductions over `dim` nested inside `ast` do not depend on the index on
// that dim; they are pulled out so that the enclosing reduce loop evaluates them once.
op::AstP extract_const(const op::AstP &ast, size_t dim, std::vector<std::pair<block::Id, op::AstP>> &accs) {
  using N = op::AstNode;
  switch (ast->kind) {
    case N::Id: case N::Load: case N::Const: return ast;
    case N::Reduce:
      if (ast->reduce_dim == dim) {
        block::Id src = block::fresh_id();
        accs.push_back({src, ast});
        return op::id_node(src, ast->dtype, ast->shape);
      }
      return op::reduce(ast->rop, extract_const(ast->arg, dim, accs), ast->reduce_dim);
    case N::Unary: return op::unary(ast->uop, extract_const(ast->arg, dim, accs));
    case N::Binary: {
      auto l = extract_const(ast->arg, dim, accs);
      auto r = extract_const(ast->rhs, dim, accs);
      return op::binary(ast->bop, l, r);
    }
    case N::Layout: return op::layout(ast->lop, extract_const(ast->arg, dim, accs), ast->shape);
  }
  return ast;
}

using PerArg = std::map<ArgId, ssa::VarId>;
thread_local block::Id g_tid = 0;   // the ThreadIdx value of the kernel being lowered (set by lower_b)

// :300-406
std::pair<block::Id, Block> lower_ast(const op::AstP &ast, const Indexes &idxs, const Opts &opts, const PerArg &per_arg) {
  using N = op::AstNode;
  const DType dtype = ast->dtype;
  switch (ast->kind) {
    case N::Load: {
      auto it = per_arg.find(ast->load_src);
      if (it == per_arg.end()) bail("unknown arg ", ast->load_src.v);
      auto [off, b] = lower_layout(ast->load_layout, idxs);
      Instr ld; ld.kind = K::Load; ld.v0 = it->second; ld.dtype = dtype; ld.a0 = A::v(off);
      block::Id dst = b.push(ld);
      return {dst, std::move(b)};
    }
    case N::Layout: return lower_ast(ast->arg, layout_op(idxs, ast->lop, ast->shape, ast->arg->shape), opts, per_arg);
    case N::Const: {
      Block b;
      Instr c; c.kind = K::Const; c.cst = ast->cst; c.dtype = ast->cst.dtype;
      block::Id dst = b.push(c);
      return {dst, std::move(b)};
    }
    case N::Unary: {
      auto [a, b] = lower_ast(ast->arg, idxs, opts, per_arg);
      Instr u; u.kind = K::Unary; u.uop = ast->uop; u.a0 = A::v(a); u.dtype = dtype;
      block::Id dst = b.push(u);
      return {dst, std::move(b)};
    }
    case N::Reduce: {
      const size_t dim = ast->reduce_dim;
      const block::Id dst = block::fresh_id();
      Block b;
      std::vector<std::pair<block::Id, op::AstP>> const_bits;
      op::AstP arg = extract_const(ast->arg, dim, const_bits);
      for (auto &cb : const_bits) {
        auto [cid, cblock] = lower_ast(cb.second, idxs, opts, per_arg);
        b.extend(cblock);
        Instr u; u.kind = K::Unary; u.uop = UnaryOp{UnaryKind::Id, DType::F32}; u.a0 = A::v(cid); u.dtype = cb.second->dtype;
        b.push_with(cb.first, u);
      }
      if (opts.has_thread_block && opts.thread_block.dim == dim && !(opts.has_block_axis && opts.block_axis == dim)) {
        const size_t reduce_len = dim < arg->shape.size() ? arg->shape[dim] : 0;
        if (!opts.hoist_row_reduces || reduce_len == opts.thread_block.block_dim) {
          // the reduced dim is spread over the threads of the block: one block-wide reduction (:358-363)
          auto [a, ab] = lower_ast(arg, idxs, opts, per_arg);
          b.extend(ab);
          Instr r; r.kind = K::ReduceLocal; r.rop = ast->rop; r.a0 = A::v(a); r.dtype = dtype;
          b.push_with(dst, r);
        } else {
          // row longer (or shorter) than the block: every thread folds the elements tid, tid + block_dim, ...
          // into a private accumulator that starts at the identity, then the block reduces the accumulators
          Instr acc; acc.kind = K::DefineAcc; acc.cst = reduce_init(ast->rop, dtype); acc.dtype = dtype;
          const block::Id acc_id = b.push(acc);
          block::Range r = b.range(A::v(g_tid), A::i32((int32_t)reduce_len), opts.thread_block.block_dim);
          Indexes ridx = idxs;
          ridx[dim] = f_id(r.range_id);
          auto [a, ab] = lower_ast(arg, ridx, opts, per_arg);
          b.extend(ab);
          block::Id folded = b.binary(reduce_fold(ast->rop), A::v(acc_id), A::v(a), dtype);
          Instr as; as.kind = K::Assign; as.v0 = acc_id; as.a0 = A::v(folded);
          b.push(as);
          b.end_range(r);
          Instr rl; rl.kind = K::ReduceLocal; rl.rop = ast->rop; rl.a0 = A::v(acc_id); rl.dtype = dtype;
          b.push_with(dst, rl);
        }
      } else {
        Instr acc; acc.kind = K::DefineAcc; acc.cst = reduce_init(ast->rop, dtype); acc.dtype = dtype;
        b.push_with(dst, acc);
        if (dim >= arg->shape.size()) bail("unexpected dim for reduce, ", dim, " ", shape_str(ast->shape));
        const size_t reduce_len = arg->shape[dim];
        block::Range r = b.range(A::i32(0), A::i32((int32_t)reduce_len), 1);
        Indexes ridx = idxs;
        ridx[dim] = f_id(r.range_id);
        auto [a, ab] = lower_ast(arg, ridx, opts, per_arg);
        b.extend(ab);
        block::Id folded = b.binary(reduce_fold(ast->rop), A::v(dst), A::v(a), dtype);
        Instr as; as.kind = K::Assign; as.v0 = dst; as.a0 = A::v(folded);
        b.push(as);
        b.end_range(r);
      }
      return {dst, std::move(b)};
    }
    case N::Binary: {
      auto [l, lb] = lower_ast(ast->arg, idxs, opts, per_arg);
      auto [r, rb] = lower_ast(ast->rhs, idxs, opts, per_arg);
      lb.extend(rb);
      block::Id dst = lb.binary(ast->bop, A::v(l), A::v(r), dtype);
      return {dst, std::move(lb)};
    }
    case N::Id: return {ast->id_src, Block{}};
  }
  bail("unreachable ast kind");
}

// :409-491
Block lower_b(const op::Kernel &k, const Opts &opts) {
  Block block;
  PerArg per_arg;
  for (size_t index = 0; index < k.args.size(); ++index) {
    Instr g; g.kind = K::DefineGlobal; g.index = index; g.dtype = k.args[index].dtype;
    per_arg[k.args[index].id] = block.push(g);
  }
  bool has_bid = opts.has_block_axis, has_tid = opts.has_thread_block;
  block::Id bid = 0, tid = 0;
  if (has_bid) { Instr s; s.kind = K::Special; s.special = ssa::Special::BlockIdx; s.dtype = DType::I32; bid = block.push(s); }
  if (has_tid) { Instr s; s.kind = K::Special; s.special = ssa::Special::ThreadIdx; s.dtype = DType::I32; tid = block.push(s); }
  g_tid = tid;
  for (const op::Store &st : k.ops) {
    auto it = per_arg.find(st.dst);
    if (it == per_arg.end()) bail("unknown arg ", st.dst.v);
    std::vector<block::Range> ranges;
    Indexes idxs;
    op::AstP value = st.value;
    for (size_t d = 0; d < st.layout.rank(); ++d) {
      const size_t len = st.layout.shape[d];
      if (opts.hoist_row_reduces && has_tid && opts.thread_block.dim == d && d + 1 == st.layout.rank()) {
        // every index but the last is known here: reductions over the last dim do not depend on the
        // position inside the row, so they are computed now, once per row
        std::vector<std::pair<block::Id, op::AstP>> hoisted;
        value = extract_const(value, d, hoisted);
        Indexes hidx = idxs;
        // position inside the row = the thread id: used as is when the row is exactly one block wide
        // (ReduceLocal of one element per thread); longer rows substitute their own strided loop variable
        hidx.push_back(f_id(tid));
        for (auto &h : hoisted) {
          auto [hid, hb] = lower_ast(h.second, hidx, opts, per_arg);
          block.extend(hb);
          Instr u; u.kind = K::Unary; u.uop = UnaryOp{UnaryKind::Id, DType::F32}; u.a0 = A::v(hid); u.dtype = h.second->dtype;
          block.push_with(h.first, u);
        }
      }
      block::Id id;
      const bool is_b = has_bid && opts.block_axis == d, is_t = has_tid && opts.thread_block.dim == d;
      if (is_b && is_t) {
        // global index bid * block_dim + tid; the range acts as an `if (idx < len)`
        block::Id g = block.mul(bid, (int32_t)opts.thread_block.block_dim);
        g = block.binary(BinaryOp::Add, A::v(g), A::v(tid), DType::I32);
        block::Range r = block.range(A::v(g), A::i32((int32_t)len), len);
        id = r.range_id;
        ranges.push_back(r);
      } else if (is_b) {
        id = bid;
      } else if (is_t) {
        if (len == opts.thread_block.block_dim) {
          id = tid;
        } else {
          block::Range r = block.range(A::v(tid), A::i32((int32_t)len), opts.thread_block.block_dim);
          id = r.range_id;
          ranges.push_back(r);
        }
      } else {
        block::Range r = block.range(A::i32(0), A::i32((int32_t)len), 1);
        id = r.range_id;
        ranges.push_back(r);
      }
      idxs.push_back(f_id(id));
    }
    auto [off, offb] = lower_layout(st.layout, idxs);
    block.extend(offb);
    auto [src, srcb] = lower_ast(value, idxs, opts, per_arg);
    block.extend(srcb);
    Instr s; s.kind = K::Store; s.v0 = it->second; s.a0 = A::v(off); s.a1 = A::v(src); s.dtype = st.value->dtype;
    block.push(s);
    for (size_t i = ranges.size(); i-- > 0;) block.end_range(ranges[i]);
  }
  return block;
}

op::AstP optimize_walk(const op::AstP &v) {  // :494-526
  using N = op::AstNode;
  switch (v->kind) {
    case N::Unary: return op::unary(v->uop, optimize_walk(v->arg));
    case N::Binary: { auto l = optimize_walk(v->arg); auto r = optimize_walk(v->rhs); return op::binary(v->bop, l, r); }
    case N::Load: return op::load(v->load_src, v->load_layout.compress_all(), v->dtype);
    case N::Reduce: bail("unexpected result in optimize step");
    case N::Layout:
      if (v->lop.kind != op::LayoutOp::Broadcast) bail("unexpected layout op in optimize step");
      return op::broadcast(optimize_walk(v->arg), Shape{num_elements(v->shape)});  // all dims are broadcast here
    default: return v;
  }
}
}  // namespace

op::Kernel optimize(op::Kernel k) {
  for (op::Store &st : k.ops) {
    if (st.can_merge_all()) {
      st.layout = st.layout.compress_all();
      st.value = optimize_walk(st.value);
    }
  }
  return k;
}

ssa::Kernel lower(const op::Kernel &k, const Opts &opts) {
  Block b = lower_b(k, opts);
  ssa::Kernel out;
  out.instrs = b.relocate();
  for (size_t i = 0; i < k.args.size(); ++i) out.args.push_back({k.args[i], i});
  uint32_t grid = 1;
  if (opts.has_block_axis && !k.ops.empty()) {
    uint32_t local = (opts.has_thread_block && opts.thread_block.dim == opts.block_axis) ? (uint32_t)opts.thread_block.block_dim : 1;
    const Shape &dims = k.ops[0].layout.shape;
    uint32_t len = opts.block_axis < dims.size() ? (uint32_t)dims[opts.block_axis] : 1;
    grid = (len + local - 1) / local;
  }
  out.launch_config.grid_dim = grid;
  out.launch_config.block_dim = opts.has_thread_block ? (uint32_t)opts.thread_block.block_dim : 1;
  out.launch_config.shared_mem = 0;
  return out;
}

// ------------------------------------------------------------- op::Store ----
namespace op {
std::string Store::name() const {
  std::string out;
  std::function<void(const AstP &)> walk = [&](const AstP &a) {
    switch (a->kind) {
      case AstNode::Unary: {
        static const char c[] = {'i', 'e', 's', 'c', 'n', 's', 'a'};
        out += 'U'; out += c[(int)a->uop.kind]; out += '_';
        walk(a->arg);
        break;
      }
      case AstNode::Binary: {
        static const char c[] = {'a', 's', 'm', 'd', 'o', 'n', 'x'};
        out += 'B'; out += c[(int)a->bop]; out += '_';
        walk(a->arg); out += '_'; walk(a->rhs);
        break;
      }
      case AstNode::Load: out += 'O'; break;
      case AstNode::Reduce: {
        static const char c[] = {'s', 'x', 'n'};
        out += 'R'; out += c[(int)a->rop]; out += '_';
        walk(a->arg);
        break;
      }
      case AstNode::Layout: {
        static const char c[] = {'b', 'n', 't', 's', 'm'};
        out += 'L'; out += c[(int)a->lop.kind]; out += '_';
        walk(a->arg);
        break;
      }
      case AstNode::Const: out += 'C'; break;
      case AstNode::Id: out += 'I'; break;
    }
  };
  walk(value);
  return out.substr(0, 40);
}

bool Store::can_merge_all() const {
  std::function<bool(const AstP &)> walk = [&](const AstP &a) -> bool {
    switch (a->kind) {
      case AstNode::Unary: return walk(a->arg);
      case AstNode::Binary: return walk(a->arg) && walk(a->rhs);
      case AstNode::Load: return a->load_layout.can_be_compressed();
      case AstNode::Reduce: return false;
      case AstNode::Layout: return a->lop.kind == LayoutOp::Broadcast && a->lop.broadcasted_dims.size() >= a->shape.size();
      default: return true;
    }
  };
  if (!layout.can_be_compressed()) return false;
  return walk(value);
}

int compare(const AstP &a, const AstP &b) {
  if (a.get() == b.get()) return 0;
  auto cmp = [](auto x, auto y) { return x < y ? -1 : (y < x ? 1 : 0); };
  if (int c = cmp((int)a->kind, (int)b->kind)) return c;
  if (int c = cmp((int)a->dtype, (int)b->dtype)) return c;
  if (int c = cmp(a->shape, b->shape)) return c;
  switch (a->kind) {
    case AstNode::Id: return cmp(a->id_src, b->id_src);
    case AstNode::Load:
      if (int c = cmp(a->load_src, b->load_src)) return c;
      return cmp(a->load_layout, b->load_layout);
    case AstNode::Reduce:
      if (int c = cmp((int)a->rop, (int)b->rop)) return c;
      if (int c = cmp(a->reduce_dim, b->reduce_dim)) return c;
      return compare(a->arg, b->arg);
    case AstNode::Unary:
      if (int c = cmp(a->uop, b->uop)) return c;
      return compare(a->arg, b->arg);
    case AstNode::Binary:
      if (int c = cmp((int)a->bop, (int)b->bop)) return c;
      if (int c = compare(a->arg, b->arg)) return c;
      return compare(a->rhs, b->rhs);
    case AstNode::Const: return cmp(a->cst, b->cst);
    case AstNode::Layout:
      if (int c = cmp(a->lop, b->lop)) return c;
      return compare(a->arg, b->arg);
  }
  return 0;
}
}  // namespace op

// ------------------------------------------------------------- cache key ----
namespace {
op::AstP renumber(const op::AstP &a, const std::map<ArgId, ArgId> &m) {
  using N = op::AstNode;
  switch (a->kind) {
    case N::Id: bail("unexpected id node");
    case N::Load: {
      auto it = m.find(a->load_src);
      if (it == m.end()) bail("BUG: missing arg id ", a->load_src.v);
      return op::load(it->second, a->load_layout, a->dtype);
    }
    case N::Unary: return op::unary(a->uop, renumber(a->arg, m));
    case N::Binary: { auto l = renumber(a->arg, m); auto r = renumber(a->rhs, m); return op::binary(a->bop, l, r); }
    case N::Const: return op::cst(a->cst);
    case N::Reduce: return op::reduce(a->rop, renumber(a->arg, m), a->reduce_dim);
    case N::Layout: return op::layout(a->lop, renumber(a->arg, m), a->shape);
  }
  return a;
}
}  // namespace

NormalizedKernel::NormalizedKernel(const op::Kernel &k) {
  std::map<ArgId, ArgId> m;
  for (size_t i = 0; i < k.args.size(); ++i) {
    m[k.args[i].id] = ArgId{i};
    args.push_back(Arg{ArgId{i}, k.args[i].dtype});
  }
  for (const op::Store &st : k.ops) {
    auto it = m.find(st.dst);
    if (it == m.end()) bail("BUG: missing arg id ", st.dst.v);
    ops.push_back(op::Store{it->second, st.layout, renumber(st.value, m)});
  }
}

bool NormalizedKernel::operator<(const NormalizedKernel &o) const {
  if (args.size() != o.args.size()) return args.size() < o.args.size();
  for (size_t i = 0; i < args.size(); ++i)
    if (!(args[i] == o.args[i])) return std::tie(args[i].id, args[i].dtype) < std::tie(o.args[i].id, o.args[i].dtype);
  if (ops.size() != o.ops.size()) return ops.size() < o.ops.size();
  for (size_t i = 0; i < ops.size(); ++i) {
    if (!(ops[i].dst == o.ops[i].dst)) return ops[i].dst < o.ops[i].dst;
    if (!(ops[i].layout == o.ops[i].layout)) return ops[i].layout < o.ops[i].layout;
    if (int c = op::compare(ops[i].value, o.ops[i].value)) return c < 0;
  }
  return false;
}

// ---------------------------------------------------------------- block ----
std::vector<Instr> block::Block::relocate() const {
  std::unordered_map<Id, size_t> line;
  for (size_t i = 0; i < v.size(); ++i) line[v[i].first] = i;
  auto id = [&](ssa::VarId x) {
    auto it = line.find(x);
    if (it == line.end()) bail("id not found ", x);
    return it->second;
  };
  auto fix = [&](A a) { if (a.is_var) a.var = id(a.var); return a; };
  std::vector<Instr> out;
  out.reserve(v.size());
  for (auto &[_, in] : v) {
    Instr i = in;
    switch (i.kind) {
      case K::Store: i.v0 = id(i.v0); i.a0 = fix(i.a0); i.a1 = fix(i.a1); break;
      case K::If: i.a0 = fix(i.a0); i.v0 = id(i.v0); break;
      case K::Range: i.a0 = fix(i.a0); i.a1 = fix(i.a1); i.v0 = id(i.v0); break;
      case K::Load: i.v0 = id(i.v0); i.a0 = fix(i.a0); break;
      case K::Binary: i.a0 = fix(i.a0); i.a1 = fix(i.a1); break;
      case K::Unary: case K::ReduceLocal: i.a0 = fix(i.a0); break;
      case K::Assign: i.v0 = id(i.v0); i.a0 = fix(i.a0); break;
      case K::EndRange: i.v0 = id(i.v0); break;
      default: break;
    }
    out.push_back(i);
  }
  return out;
}

// ------------------------------------------------------------- ssa text ----
namespace ssa {
static std::string a_str(const A &a) {
  std::ostringstream os;
  if (a.is_var) { os << "%" << a.var; return os.str(); }
  switch (a.cst.dtype) {
    case DType::F32: os << a.cst.f32 << "f32"; break;
    case DType::I32: os << a.cst.i32 << "i32"; break;
    case DType::I64: os << a.cst.i64 << "i64"; break;
    default: os << "0x" << std::hex << a.cst.h << dtype_str(a.cst.dtype); break;
  }
  return os.str();
}
std::string to_text(const Kernel &k) {
  static const char *un[] = {"id", "exp", "sin", "cos", "neg", "sqrt", "cast"};
  static const char *bn[] = {"add", "sub", "mul", "div", "mod", "min", "max"};
  static const char *rn[] = {"sum", "max", "min"};
  std::ostringstream os;
  os << "launch grid=" << k.launch_config.grid_dim << " block=" << k.launch_config.block_dim << "\n";
  for (size_t l = 0; l < k.instrs.size(); ++l) {
    const Instr &i = k.instrs[l];
    os << l << ": ";
    switch (i.kind) {
      case K::DefineAcc: os << "acc " << a_str(A::c(i.cst)); break;
      case K::DefineGlobal: os << "global " << i.index << " " << dtype_str(i.dtype); break;
      case K::DefineLocal: os << "local " << i.index << " " << dtype_str(i.dtype); break;
      case K::Special: os << (i.special == Special::ThreadIdx ? "thread_idx" : "block_idx"); break;
      case K::Const: os << "const " << a_str(A::c(i.cst)); break;
      case K::Unary: os << un[(int)i.uop.kind] << "." << dtype_str(i.dtype) << " " << a_str(i.a0); break;
      case K::Binary: os << bn[(int)i.bop] << "." << dtype_str(i.dtype) << " " << a_str(i.a0) << " " << a_str(i.a1); break;
      case K::Range: os << "range " << a_str(i.a0) << " " << a_str(i.a1) << " step " << i.index << " end %" << i.v0; break;
      case K::Load: os << "load." << dtype_str(i.dtype) << " %" << i.v0 << "[" << a_str(i.a0) << "]"; break;
      case K::Assign: os << "assign %" << i.v0 << " = " << a_str(i.a0); break;
      case K::EndRange: os << "end_range %" << i.v0; break;
      case K::If: os << "if " << a_str(i.a0) << " end %" << i.v0; break;
      case K::EndIf: os << "end_if"; break;
      case K::Store: os << "store." << dtype_str(i.dtype) << " %" << i.v0 << "[" << a_str(i.a0) << "] = " << a_str(i.a1); break;
      case K::Barrier: os << "barrier"; break;
      case K::ReduceLocal: os << "reduce_local." << rn[(int)i.rop] << "." << dtype_str(i.dtype) << " " << a_str(i.a0); break;
    }
    os << "\n";
  }
  return os.str();
}
}  // namespace ssa

}  // namespace ug
