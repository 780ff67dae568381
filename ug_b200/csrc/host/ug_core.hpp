// Host-side restatement of ug-core's data model in C++17: dtypes and constants
// (ug-core/src/dtype.rs, const.rs), shapes and layouts (layout.rs), the tensor
// level op::Ast and the flat ssa::Instr IR (lang.rs), and the Block builder
// (block.rs).  Pure data: nothing here touches a device.  Errors are C++
// exceptions of type ug::Error (the counterpart of ug::Error / bail!), caught
// at the C boundary.
#pragma once
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <variant>
#include <vector>

namespace ug {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
template <typename... A> [[noreturn]] inline void bail(A &&...a) {
  std::ostringstream os;
  (os << ... << a);
  throw Error(os.str());
}

// ---------------------------------------------------------------- dtype ----
// ug-core/src/dtype.rs:4-11, same order.
enum class DType : int32_t { BF16 = 0, F16 = 1, F32 = 2, I32 = 3, I64 = 4 };
inline size_t size_in_bytes(DType d) {
  switch (d) {
    case DType::BF16: case DType::F16: return 2;
    case DType::F32: case DType::I32: return 4;
    case DType::I64: return 8;
  }
  return 0;
}
inline const char *dtype_str(DType d) {
  switch (d) {
    case DType::BF16: return "bf16";
    case DType::F16: return "f16";
    case DType::F32: return "f32";
    case DType::I32: return "i32";
    case DType::I64: return "i64";
  }
  return "?";
}

inline uint16_t f32_to_bf16_bits(float v) {
  uint32_t x;
  std::memcpy(&x, &v, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x0040u);
  return (uint16_t)((x + 0x7fffu + ((x >> 16) & 1u)) >> 16);
}
inline float bf16_bits_to_f32(uint16_t h) {
  uint32_t x = (uint32_t)h << 16;
  float v;
  std::memcpy(&v, &x, 4);
  return v;
}

// ---------------------------------------------------------------- const ----
// ug-core/src/const.rs:83-174: NaN-free scalar constants, hashable / ordered.
struct Const {
  DType dtype = DType::F32;
  union {
    float f32;
    int32_t i32;
    int64_t i64;
    uint16_t h;  // bf16 / f16 bit pattern
  };
  Const() : i64(0) {}
  static Const from_f32(float v) {
    if (std::isnan(v)) bail("unable to create const for NaN");
    Const c; c.dtype = DType::F32; c.i64 = 0; c.f32 = v; return c;
  }
  static Const from_i32(int32_t v) { Const c; c.dtype = DType::I32; c.i64 = 0; c.i32 = v; return c; }
  static Const from_i64(int64_t v) { Const c; c.dtype = DType::I64; c.i64 = v; return c; }
  static Const from_bf16(float v) {
    if (std::isnan(v)) bail("unable to create const for NaN");
    Const c; c.dtype = DType::BF16; c.i64 = 0; c.h = f32_to_bf16_bits(v); return c;
  }
  static Const zero(DType d) {
    Const c; c.dtype = d; c.i64 = 0; return c;
  }
  static Const min_value(DType d) {  // const.rs:155-163
    switch (d) {
      case DType::F32: return from_f32(-INFINITY);
      case DType::BF16: { Const c = zero(d); c.h = 0xff80; return c; }
      case DType::F16: { Const c = zero(d); c.h = 0xfc00; return c; }
      case DType::I32: return from_i32(INT32_MIN);
      case DType::I64: return from_i64(INT64_MIN);
    }
    return zero(d);
  }
  static Const max_value(DType d) {  // const.rs:165-173
    switch (d) {
      case DType::F32: return from_f32(INFINITY);
      case DType::BF16: { Const c = zero(d); c.h = 0x7f80; return c; }
      case DType::F16: { Const c = zero(d); c.h = 0x7c00; return c; }
      case DType::I32: return from_i32(INT32_MAX);
      case DType::I64: return from_i64(INT64_MAX);
    }
    return zero(d);
  }
  int64_t bits() const { return dtype == DType::I64 ? i64 : (dtype == DType::F32 || dtype == DType::I32 ? (int64_t)i32 : (int64_t)h); }
  bool operator==(const Const &o) const { return dtype == o.dtype && bits() == o.bits(); }
  bool operator<(const Const &o) const { return dtype != o.dtype ? dtype < o.dtype : bits() < o.bits(); }
};

// --------------------------------------------------------------- layout ----
using Shape = std::vector<size_t>;
inline size_t num_elements(const Shape &s) {
  size_t n = 1;
  for (size_t d : s) n *= d;
  return n;
}
inline std::string shape_str(const Shape &s) {
  std::ostringstream os;
  os << "[";
  for (size_t i = 0; i < s.size(); ++i) os << (i ? ", " : "") << s[i];
  os << "]";
  return os.str();
}
// Dim / D::Minus1 resolution (layout.rs:226-307): negative indexes count from the end.
inline size_t to_index(long dim, const Shape &shape, const char *op) {
  long r = (long)shape.size();
  long d = dim < 0 ? r + dim : dim;
  if (d < 0 || d >= r) bail("dim out of range in '", op, "', dim: ", dim, ", shape: ", shape_str(shape));
  return (size_t)d;
}

// ug-core/src/layout.rs:576-674
struct Layout {
  Shape shape;
  std::vector<size_t> strides;
  size_t offset = 0;

  static Layout from_shape(const Shape &s) {
    Layout l;
    l.shape = s;
    l.strides.assign(s.size(), 1);
    size_t st = 1;
    for (size_t i = s.size(); i-- > 0;) { l.strides[i] = st; st *= s[i]; }
    return l;
  }
  size_t rank() const { return shape.size(); }
  const Shape &dims() const { return shape; }
  size_t num_elements() const { return ug::num_elements(shape); }
  bool can_be_compressed() const {  // layout.rs:585-597
    if (shape.size() <= 1) return false;
    for (size_t i = 0; i + 1 < shape.size(); ++i)
      if (strides[i] != strides[i + 1] * shape[i + 1]) return false;
    return true;
  }
  Layout compress_all() const {  // layout.rs:599-610
    for (size_t i = 0; i + 1 < shape.size(); ++i)
      if (strides[i] != strides[i + 1] * shape[i + 1]) bail("cannot collapse dims");
    Layout l;
    l.shape = {num_elements()};
    l.strides = {strides.empty() ? 1 : strides.back()};
    l.offset = offset;
    return l;
  }
  Layout transpose() const {  // layout.rs:624-634 (last two dims)
    Layout l = *this;
    size_t r = rank();
    if (r < 2) return l;
    std::swap(l.shape[r - 2], l.shape[r - 1]);
    std::swap(l.strides[r - 2], l.strides[r - 1]);
    return l;
  }
  bool c_contiguous() const {
    size_t prod = 1;
    for (size_t i = shape.size(); i-- > 0;) {
      if (strides[i] != prod) return false;
      prod *= shape[i];
    }
    return true;
  }
  bool operator==(const Layout &o) const { return shape == o.shape && strides == o.strides && offset == o.offset; }
  bool operator<(const Layout &o) const {
    return std::tie(shape, strides, offset) < std::tie(o.shape, o.strides, o.offset);
  }
};

// ----------------------------------------------------------------- lang ----
enum class ReduceOp : int32_t { Sum = 0, Max = 1, Min = 2 };
enum class UnaryKind : int32_t { Id = 0, Exp = 1, Sin = 2, Cos = 3, Neg = 4, Sqrt = 5, Cast = 6 };
struct UnaryOp {
  UnaryKind kind = UnaryKind::Id;
  DType cast_to = DType::F32;  // only for Cast
  bool operator==(const UnaryOp &o) const { return kind == o.kind && (kind != UnaryKind::Cast || cast_to == o.cast_to); }
  bool operator<(const UnaryOp &o) const { return kind != o.kind ? kind < o.kind : (kind == UnaryKind::Cast && cast_to < o.cast_to); }
};
enum class BinaryOp : int32_t { Add = 0, Sub = 1, Mul = 2, Div = 3, Mod = 4, Min = 5, Max = 6 };

// lang.rs:98-116: process-unique argument ids.
struct ArgId {
  size_t v = 0;
  static ArgId fresh() {
    static std::atomic<size_t> counter{1};
    return ArgId{counter.fetch_add(1)};
  }
  bool operator==(const ArgId &o) const { return v == o.v; }
  bool operator<(const ArgId &o) const { return v < o.v; }
};
struct Arg {  // pointer arguments only (lower_op.rs:415-418 rejects value arguments)
  ArgId id;
  DType dtype;
  bool operator==(const Arg &o) const { return id == o.id && dtype == o.dtype; }
  bool operator<(const Arg &o) const { return id < o.id; }
};

struct LaunchConfig {  // lang.rs:34-45
  uint32_t grid_dim = 1, block_dim = 1, shared_mem = 0;
};



namespace ssa {
// Variable ids are line numbers once a block is relocated (lang.rs:617-636).
using VarId = size_t;
struct A {  // lang.rs:642-646
  bool is_var = true;
  VarId var = 0;
  Const cst;
  static A v(VarId id) { A a; a.is_var = true; a.var = id; return a; }
  static A c(Const c_) { A a; a.is_var = false; a.cst = c_; return a; }
  static A i32(int32_t x) { return c(Const::from_i32(x)); }
  bool operator==(const A &o) const { return is_var == o.is_var && (is_var ? var == o.var : cst == o.cst); }
  bool operator<(const A &o) const {
    if (is_var != o.is_var) return is_var < o.is_var;
    return is_var ? var < o.var : cst < o.cst;
  }
};
enum class Special : int32_t { ThreadIdx = 0, BlockIdx = 1 };
// lang.rs:690-709, one tagged struct instead of a Rust enum.
enum class K : int32_t {
  DefineAcc = 0, DefineGlobal, DefineLocal, Special, Const, Unary, Binary, Range, Load, Assign, EndRange, If,
  EndIf, Store, Barrier, ReduceLocal
};
struct Instr {
  K kind = K::Barrier;
  DType dtype = DType::F32;
  Const cst;                 // DefineAcc, Const
  size_t index = 0;          // DefineGlobal.index, DefineLocal.size, Range.step
  ssa::Special special = ssa::Special::ThreadIdx;
  UnaryOp uop;
  BinaryOp bop = BinaryOp::Add;
  ReduceOp rop = ReduceOp::Sum;
  A a0, a1, a2;              // Unary.arg | Binary.lhs,rhs | Range.lo,up | Load.offset | Assign.src | If.cond |
                             // Store.offset,value | ReduceLocal.arg
  VarId v0 = 0;              // Range.end_idx | Load.src | Assign.dst | EndRange.start_idx | If.end_idx | Store.dst

  bool operator==(const Instr &o) const {
    return kind == o.kind && dtype == o.dtype && cst == o.cst && index == o.index && special == o.special &&
           uop == o.uop && bop == o.bop && rop == o.rop && a0 == o.a0 && a1 == o.a1 && a2 == o.a2 && v0 == o.v0;
  }
  bool operator<(const Instr &o) const {
    auto key = [](const Instr &i) {
      return std::tie(i.kind, i.dtype, i.cst, i.index, i.special, i.uop, i.bop, i.rop, i.a0, i.a1, i.a2, i.v0);
    };
    return key(*this) < key(o);
  }
};
struct Kernel {  // lang.rs:711-753
  std::vector<Instr> instrs;
  std::vector<std::pair<Arg, size_t>> args;  // (arg, line of its DefineGlobal)
  LaunchConfig launch_config;

  static Kernel from_instrs(std::vector<Instr> instrs) {
    Kernel k;
    for (size_t line = 0; line < instrs.size(); ++line) {
      const Instr &i = instrs[line];
      if (i.kind == K::DefineGlobal) {
        if (i.index != k.args.size()) bail("unexpected order for arguments in kernel");
        k.args.push_back({Arg{ArgId::fresh(), i.dtype}, line});
      }
    }
    k.instrs = std::move(instrs);
    return k;
  }
};
std::string to_text(const Kernel &k);  // one line per instruction, for inspection and golden tests
}  // namespace ssa

// ------------------------------------------------------------ op (AST) ----
namespace op {
// lang.rs:425-432
struct LayoutOp {
  enum Kind : int32_t { Broadcast = 0, Narrow, Transpose, SplitDim, MergeDims } kind = Broadcast;
  size_t inserted_dims = 0;
  std::vector<size_t> broadcasted_dims;
  size_t dim = 0, offset = 0;     // Narrow {dim, offset}; SplitDim/MergeDims {dim}
  size_t d1 = 0, d2 = 0;          // Transpose {dim1, dim2}; SplitDim/MergeDims {lhs, rhs}
  bool operator==(const LayoutOp &o) const {
    return kind == o.kind && inserted_dims == o.inserted_dims && broadcasted_dims == o.broadcasted_dims &&
           dim == o.dim && offset == o.offset && d1 == o.d1 && d2 == o.d2;
  }
  bool operator<(const LayoutOp &o) const {
    return std::tie(kind, inserted_dims, broadcasted_dims, dim, offset, d1, d2) <
           std::tie(o.kind, o.inserted_dims, o.broadcasted_dims, o.dim, o.offset, o.d1, o.d2);
  }
};

struct AstNode;
using AstP = std::shared_ptr<const AstNode>;
// lang.rs:417-447.  `Id` nodes name a value that an enclosing lowering step has already computed.
struct AstNode {
  enum Kind : int32_t { Id = 0, Load, Reduce, Unary, Binary, Const, Layout } kind = Const;
  DType dtype = DType::F32;
  Shape shape;
  size_t id_src = 0;        // Id: block id
  ArgId load_src;           // Load
  ug::Layout load_layout;   // Load
  ReduceOp rop = ReduceOp::Sum;
  size_t reduce_dim = 0;
  UnaryOp uop;
  BinaryOp bop = BinaryOp::Add;
  ug::Const cst;
  LayoutOp lop;
  AstP arg, rhs;            // arg (= lhs for Binary), rhs
};

inline AstP load(ArgId src, const ug::Layout &layout, DType dtype) {
  auto n = std::make_shared<AstNode>();
  n->kind = AstNode::Load; n->dtype = dtype; n->shape = layout.shape; n->load_src = src; n->load_layout = layout;
  return n;
}
inline AstP layout(const LayoutOp &op, AstP arg, const Shape &shape) {
  auto n = std::make_shared<AstNode>();
  n->kind = AstNode::Layout; n->dtype = arg->dtype; n->shape = shape; n->lop = op; n->arg = std::move(arg);
  return n;
}
inline AstP broadcast(AstP arg, const Shape &shape) {  // lang.rs:455-482
  if (arg->shape.size() > shape.size())
    bail("target shape ", shape_str(shape), " has less dimensions than original shape ", shape_str(arg->shape));
  LayoutOp op;
  op.kind = LayoutOp::Broadcast;
  op.inserted_dims = shape.size() - arg->shape.size();
  for (size_t i = 0; i < op.inserted_dims; ++i) op.broadcasted_dims.push_back(i);
  for (size_t i = 0; i < arg->shape.size(); ++i) {
    size_t di = i + op.inserted_dims;
    if (shape[di] != arg->shape[i]) {
      if (arg->shape[i] == 1) op.broadcasted_dims.push_back(di);
      else bail("cannot broadcast from ", shape_str(arg->shape), " to ", shape_str(shape));
    }
  }
  return layout(op, std::move(arg), shape);
}
inline AstP unary(UnaryOp op, AstP arg) {
  auto n = std::make_shared<AstNode>();
  n->kind = AstNode::Unary; n->dtype = op.kind == UnaryKind::Cast ? op.cast_to : arg->dtype; n->shape = arg->shape;
  n->uop = op; n->arg = std::move(arg);
  return n;
}
inline AstP reduce(ReduceOp op, AstP arg, size_t dim) {  // keepdim: the reduced dim becomes 1 (lang.rs:496-505)
  if (dim >= arg->shape.size()) bail("no dim ", dim, " in shape ", shape_str(arg->shape));
  auto n = std::make_shared<AstNode>();
  n->kind = AstNode::Reduce; n->dtype = arg->dtype; n->shape = arg->shape; n->shape[dim] = 1;
  n->rop = op; n->reduce_dim = dim; n->arg = std::move(arg);
  return n;
}
inline AstP binary(BinaryOp op, AstP lhs, AstP rhs) {  // lang.rs:507-520
  if (lhs->dtype != rhs->dtype) bail("dtype mismatch in binary op, lhs: ", dtype_str(lhs->dtype), ", rhs: ", dtype_str(rhs->dtype));
  if (lhs->shape != rhs->shape && !lhs->shape.empty() && !rhs->shape.empty())
    bail("shape mismatch in binary op, lhs: ", shape_str(lhs->shape), ", rhs: ", shape_str(rhs->shape));
  auto n = std::make_shared<AstNode>();
  n->kind = AstNode::Binary; n->dtype = lhs->dtype; n->shape = lhs->shape; n->bop = op;
  n->arg = std::move(lhs); n->rhs = std::move(rhs);
  return n;
}
inline AstP cst(ug::Const c) {  // rank 0 (lang.rs:529-537)
  auto n = std::make_shared<AstNode>();
  n->kind = AstNode::Const; n->dtype = c.dtype; n->cst = c;
  return n;
}
inline AstP id_node(size_t src, DType dtype, const Shape &shape) {
  auto n = std::make_shared<AstNode>();
  n->kind = AstNode::Id; n->dtype = dtype; n->shape = shape; n->id_src = src;
  return n;
}
inline void arg_ids(const AstP &a, std::set<ArgId> &ids) {  // ordered, lang.rs:549-570
  switch (a->kind) {
    case AstNode::Layout: case AstNode::Reduce: case AstNode::Unary: arg_ids(a->arg, ids); break;
    case AstNode::Binary: arg_ids(a->arg, ids); arg_ids(a->rhs, ids); break;
    case AstNode::Load: ids.insert(a->load_src); break;
    default: break;
  }
}
// Structural comparison (the derived Eq / Ord of the Rust types); Id nodes never reach a cache key.
int compare(const AstP &a, const AstP &b);

struct Store {  // lang.rs:573-588
  ArgId dst;
  ug::Layout layout;
  AstP value;
  std::string name() const;          // lower_op.rs:559-633
  bool can_merge_all() const;        // lower_op.rs:635-664
};
struct Kernel {  // lang.rs:590-605
  std::string name;
  std::vector<Arg> args;
  std::vector<Store> ops;
};
}  // namespace op

// ---------------------------------------------------------------- block ----
// block.rs: instructions with explicit process-unique destination ids, turned into
// line-numbered SSA by relocate().
namespace block {
using Id = size_t;
inline Id fresh_id() {
  static std::atomic<size_t> counter{1};
  return counter.fetch_add(1);
}
struct Range { Id range_id, erange_id; };
struct Block {
  std::vector<std::pair<Id, ssa::Instr>> v;

  Id push(ssa::Instr i) { Id id = fresh_id(); v.push_back({id, std::move(i)}); return id; }
  void push_with(Id id, ssa::Instr i) { v.push_back({id, std::move(i)}); }
  void extend(const Block &o) { v.insert(v.end(), o.v.begin(), o.v.end()); }
  Range range(ssa::A lo, ssa::A up, size_t step) {
    Range r{fresh_id(), fresh_id()};
    ssa::Instr i; i.kind = ssa::K::Range; i.a0 = lo; i.a1 = up; i.index = step; i.v0 = r.erange_id;
    v.push_back({r.range_id, i});
    return r;
  }
  void end_range(const Range &r) {
    ssa::Instr i; i.kind = ssa::K::EndRange; i.v0 = r.range_id;
    v.push_back({r.erange_id, i});
  }
  Id cst_i32(int32_t c) { ssa::Instr i; i.kind = ssa::K::Const; i.cst = Const::from_i32(c); i.dtype = DType::I32; return push(i); }
  Id binary(BinaryOp op, ssa::A lhs, ssa::A rhs, DType dt) {
    ssa::Instr i; i.kind = ssa::K::Binary; i.bop = op; i.a0 = lhs; i.a1 = rhs; i.dtype = dt;
    return push(i);
  }
  Id mul(Id src, int32_t c) { return c == 1 ? src : binary(BinaryOp::Mul, ssa::A::v(src), ssa::A::i32(c), DType::I32); }  // block.rs:86-102
  Id add(Id src, int32_t c) { return c == 0 ? src : binary(BinaryOp::Add, ssa::A::v(src), ssa::A::i32(c), DType::I32); }
  std::vector<ssa::Instr> relocate() const;  // block.rs:143-222
};
}  // namespace block

}  // namespace ug
