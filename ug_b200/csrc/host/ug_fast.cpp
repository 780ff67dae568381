// Vectorised code generation for the two kernel shapes that carry ug-llama's elementwise and row work:
//   * row kernels   -- a store into a contiguous [rows.., cols] buffer whose value reduces over the last
//                      dim only (rms_norm, softmax, x * gain, scale, ...): one CTA (or one warp for short
//                      rows) per row, the row's operands held in registers as float4, every reduction a
//                      pass over those registers finished by a warp-shuffle / shared-memory block reduce,
//                      one 128-bit read per operand element and one 128-bit write per result element;
//   * map kernels   -- a 1-D store of a pure map (silu(gate) * up, residual add, ...): 4096 elements per
//                      CTA, 128-bit accesses.
// Rows whose length or bases rule 128-bit accesses out get the same kernels with one element per access (coalesced).
// This replaces, for these shapes, the per-instruction scalar code the SSA path generates
// (ug-cuda/src/code_gen.rs:68-186 in the reference: one 4-byte access per statement) and the launch shapes
// of ug-core/src/schedule.rs:162-188.  Anything the analysis below does not understand (non-affine
// indexes from merge_dims, reductions over other dims, dtypes other than f32, unaligned bases) returns
// "not applicable" and takes the SSA path.
//
// Every load address is reduced to the form  offset + f(leading indexes) + cc * column  over the loop indexes
// of the store (ug-core/src/lower_op.rs:131-232 folds the same layout ops into index formulas); the
// coefficient cc of the last index decides how the operand is fetched: 1 = float4 row segment kept in
// registers, 0 = one scalar per row, anything else = scalar gathers.
#include <algorithm>
#include <cctype>
#include <cinttypes>
#include <cstdio>

#include "ug_graph.hpp"

namespace ug {

namespace {

// One index (or address) as a function of the store's loop indexes:
//   column part + row part + off
// The column part is cc * col, or -- after a merge_dims of the store's last dim, e.g. the head merge
// [.., heads, 64] -> [.., heads * 64] of model.rs:243 -- ch * (col / cd) + cl * (col % cd).  The row part is any
// integer expression of the leading indexes i0, i1, ... (kept as C text) known to be a multiple of `rm`.
struct Affine {
  long cc = 0;
  long cd = 0, ch = 0, cl = 0;   // cd != 0: split column
  std::string re;
  long rm = 0;
  long off = 0;
  bool col_free() const { return cc == 0 && (cd == 0 || (ch == 0 && cl == 0)); }
};
using Idx = std::vector<Affine>;

struct NotApplicable {};

long gcd_l(long a, long b) { a = a < 0 ? -a : a; b = b < 0 ? -b : b; while (b) { long t = a % b; a = b; b = t; } return a; }
Affine aff_const(long c) { Affine a; a.off = c; return a; }
Affine aff_add(const Affine &x, const Affine &y) {
  Affine a;
  a.off = x.off + y.off;
  if (x.cd == 0 && y.cd == 0) a.cc = x.cc + y.cc;
  else if (x.cd != 0 && y.cd != 0 && x.cd == y.cd) { a.cd = x.cd; a.ch = x.ch + y.ch; a.cl = x.cl + y.cl; }
  else if (x.cd != 0 && y.cd == 0 && y.cc == 0) { a.cd = x.cd; a.ch = x.ch; a.cl = x.cl; }
  else if (y.cd != 0 && x.cd == 0 && x.cc == 0) { a.cd = y.cd; a.ch = y.ch; a.cl = y.cl; }
  else throw NotApplicable{};
  if (x.re.empty()) { a.re = y.re; a.rm = y.rm; }
  else if (y.re.empty()) { a.re = x.re; a.rm = x.rm; }
  else { a.re = "(" + x.re + " + " + y.re + ")"; a.rm = gcd_l(x.rm, y.rm); }
  return a;
}
Affine aff_scale(const Affine &x, long s) {
  Affine a = x;
  a.cc *= s; a.ch *= s; a.cl *= s;
  a.off *= s;
  if (s == 0) { a.re.clear(); a.rm = 0; a.cd = 0; }
  else if (!a.re.empty() && s != 1) { a.re = "(" + a.re + " * " + std::to_string(s) + "L)"; a.rm *= s; }
  return a;
}
// idx / n and idx % n
Affine aff_divmod(const Affine &x, long n, bool mod) {
  Affine a;
  if (x.col_free()) {
    if (x.re.empty()) { a.off = mod ? x.off % n : x.off / n; return a; }
    a.re = "((" + x.re + " + " + std::to_string(x.off) + "L) " + (mod ? "% " : "/ ") + std::to_string(n) + "L)";
    a.rm = 1;
    return a;
  }
  if (x.cd == 0 && x.cc == 1 && x.re.empty() && x.off == 0) {   // the column itself
    a.cd = n;
    (mod ? a.cl : a.ch) = 1;
    return a;
  }
  throw NotApplicable{};
}

// lower_op.rs:131-200 on these indexes
Idx layout_op(const Idx &in, const op::LayoutOp &op, const Shape &shape, const Shape &arg_shape) {
  Idx idxs = in;
  using L = op::LayoutOp;
  switch (op.kind) {
    case L::Broadcast:
      for (size_t d : op.broadcasted_dims) {
        if (d >= idxs.size()) throw NotApplicable{};
        idxs[d] = aff_const(0);
      }
      idxs.erase(idxs.begin(), idxs.begin() + (long)op.inserted_dims);
      break;
    case L::Narrow:
      if (op.dim >= idxs.size()) throw NotApplicable{};
      idxs[op.dim].off += (long)op.offset;
      break;
    case L::Transpose:
      if (op.d1 >= idxs.size() || op.d2 >= idxs.size()) throw NotApplicable{};
      std::swap(idxs[op.d1], idxs[op.d2]);
      break;
    case L::SplitDim: {
      const size_t lhs = op.d1, rhs = op.d2;
      if (lhs >= shape.size() || rhs >= shape.size() || lhs == rhs || op.dim >= arg_shape.size()) throw NotApplicable{};
      Affine l, r;
      if (lhs < rhs) { r = idxs[rhs]; idxs.erase(idxs.begin() + (long)rhs); l = idxs[lhs]; idxs.erase(idxs.begin() + (long)lhs); }
      else { l = idxs[lhs]; idxs.erase(idxs.begin() + (long)lhs); r = idxs[rhs]; idxs.erase(idxs.begin() + (long)rhs); }
      idxs.insert(idxs.begin() + (long)op.dim, aff_add(aff_scale(l, (long)shape[rhs]), r));
      break;
    }
    case L::MergeDims: {
      const size_t lhs = op.d1, rhs = op.d2;
      if (op.dim >= shape.size() || lhs >= arg_shape.size() || rhs >= arg_shape.size() || lhs == rhs) throw NotApplicable{};
      Affine idx = idxs[op.dim];
      idxs.erase(idxs.begin() + (long)op.dim);
      Affine lhs_idx, rhs_idx;
      if (arg_shape[lhs] <= 1) { lhs_idx = aff_const(0); rhs_idx = arg_shape[rhs] <= 1 ? aff_const(0) : idx; }
      else if (arg_shape[rhs] <= 1) { lhs_idx = idx; rhs_idx = aff_const(0); }
      else { lhs_idx = aff_divmod(idx, (long)arg_shape[rhs], false); rhs_idx = aff_divmod(idx, (long)arg_shape[rhs], true); }
      if (lhs < rhs) { idxs.insert(idxs.begin() + (long)lhs, lhs_idx); idxs.insert(idxs.begin() + (long)rhs, rhs_idx); }
      else { idxs.insert(idxs.begin() + (long)rhs, rhs_idx); idxs.insert(idxs.begin() + (long)lhs, lhs_idx); }
      break;
    }
  }
  return idxs;
}

std::string f32_literal(float v) {
  if (std::isinf(v)) return v > 0 ? "__int_as_float(0x7f800000)" : "__int_as_float(0xff800000)";
  char buf[64];
  snprintf(buf, sizeof buf, "%.9gf", (double)v);
  std::string s(buf);
  if (s.find('.') == std::string::npos && s.find('e') == std::string::npos && s.find("inf") == std::string::npos)
    s.insert(s.size() - 1, ".0");
  return s;
}

struct LoadSite {
  size_t arg = 0;            // position in kernel.args
  Affine addr;               // element address as a function of the store's indexes
  enum Kind { Vec, Scalar, Gather } kind = Gather;
};
struct Pass {
  const op::AstNode *node = nullptr;
  ReduceOp rop = ReduceOp::Sum;
  std::string body;          // value of the reduced expression at element J / column COL
};

struct Gen {
  const op::Kernel &k;
  size_t n = 0;              // rank of the store
  size_t cols = 0;
  int W = 4;                 // elements per access: 4 (128-bit) or 1
  bool chunked = false;      // 1-D map cut into chunks (the element index is row * chunk + column)
  std::vector<LoadSite> loads;
  std::vector<Pass> passes;

  Gen(const op::Kernel &k_, int w) : k(k_), W(w) {}

  size_t arg_pos(ArgId id) const {
    for (size_t i = 0; i < k.args.size(); ++i) if (k.args[i].id == id) return i;
    throw NotApplicable{};
  }
  size_t load_site(size_t arg, const Affine &addr) {
    for (size_t i = 0; i < loads.size(); ++i) {
      const Affine &o = loads[i].addr;
      if (loads[i].arg == arg && o.cc == addr.cc && o.cd == addr.cd && o.ch == addr.ch && o.cl == addr.cl && o.re == addr.re && o.off == addr.off) return i;
    }
    LoadSite s;
    s.arg = arg;
    s.addr = addr;
    const bool aligned = W == 1 || (addr.off % 4 == 0 && (addr.re.empty() || addr.rm % 4 == 0));
    if (addr.col_free()) s.kind = LoadSite::Scalar;
    else if (addr.cd == 0) s.kind = (addr.cc == 1 && aligned) ? LoadSite::Vec : LoadSite::Gather;
    else s.kind = (addr.cl == 1 && aligned && (W == 1 || (addr.cd % 4 == 0 && addr.ch % 4 == 0))) ? LoadSite::Vec : LoadSite::Gather;
    if (chunked && s.kind == LoadSite::Gather) throw NotApplicable{};
    if (chunked && addr.cd != 0) throw NotApplicable{};
    loads.push_back(s);
    return loads.size() - 1;
  }
  // element offset of column `col` (a C expression) from the load's row base
  static std::string col_offset(const Affine &a, const std::string &col) {
    if (a.cd == 0) return std::to_string(a.cc) + "L * (" + col + ")";
    return "(" + std::to_string(a.ch) + "L * ((" + col + ") / " + std::to_string(a.cd) + "L) + " + std::to_string(a.cl) + "L * ((" + col + ") % " +
           std::to_string(a.cd) + "L))";
  }

  // C expression of `a` at element J (register index) / column COL of the current row
  std::string emit(const op::AstP &a, const Idx &idx) {
    using N = op::AstNode;
    if (a->dtype != DType::F32) throw NotApplicable{};
    switch (a->kind) {
      case N::Id: throw NotApplicable{};
      case N::Const: return "(" + f32_literal(a->cst.f32) + ")";
      case N::Load: {
        const Layout &l = a->load_layout;
        if (idx.size() != l.strides.size()) throw NotApplicable{};
        Affine addr = aff_const((long)l.offset);
        for (size_t d = 0; d < idx.size(); ++d) addr = aff_add(addr, aff_scale(idx[d], (long)l.strides[d]));
        const size_t s = load_site(arg_pos(a->load_src), addr);
        switch (loads[s].kind) {
          case LoadSite::Vec: return "L" + std::to_string(s) + "[J]";
          case LoadSite::Scalar: return "S" + std::to_string(s);
          case LoadSite::Gather: return "__ldg(a" + std::to_string(loads[s].arg) + " + B" + std::to_string(s) + " + " + col_offset(loads[s].addr, "COL") + ")";
        }
        throw NotApplicable{};
      }
      case N::Layout: return emit(a->arg, layout_op(idx, a->lop, a->shape, a->arg->shape));
      case N::Unary: {
        const std::string x = emit(a->arg, idx);
        switch (a->uop.kind) {
          case UnaryKind::Id: return x;
          case UnaryKind::Exp: return "expf(" + x + ")";
          case UnaryKind::Sin: return "sinf(" + x + ")";
          case UnaryKind::Cos: return "cosf(" + x + ")";
          case UnaryKind::Neg: return "(-" + x + ")";
          case UnaryKind::Sqrt: return "sqrtf(" + x + ")";
          case UnaryKind::Cast:
            if (a->uop.cast_to != DType::F32 || a->arg->dtype != DType::F32) throw NotApplicable{};
            return x;
        }
        throw NotApplicable{};
      }
      case N::Binary: {
        const std::string l = emit(a->arg, idx), r = emit(a->rhs, idx);
        switch (a->bop) {
          case BinaryOp::Add: return "(" + l + " + " + r + ")";
          case BinaryOp::Sub: return "(" + l + " - " + r + ")";
          case BinaryOp::Mul: return "(" + l + " * " + r + ")";
          case BinaryOp::Div: return "(" + l + " / " + r + ")";
          case BinaryOp::Min: return "fminf(" + l + ", " + r + ")";
          case BinaryOp::Max: return "fmaxf(" + l + ", " + r + ")";
          case BinaryOp::Mod: throw NotApplicable{};
        }
        throw NotApplicable{};
      }
      case N::Reduce: {
        if (chunked) throw NotApplicable{};
        const size_t dim = a->reduce_dim;
        if (dim >= a->arg->shape.size() || a->arg->shape[dim] != cols) throw NotApplicable{};
        for (size_t i = 0; i < passes.size(); ++i)
          if (passes[i].node == a.get()) return "R" + std::to_string(i);
        // inside the reduction the index on `dim` is the position in the row; every other index must not
        // depend on it, or the result would differ from column to column
        Idx inner = idx;
        if (dim >= inner.size()) throw NotApplicable{};
        inner[dim] = aff_const(0);
        inner[dim].cc = 1;
        for (size_t d = 0; d < inner.size(); ++d)
          if (d != dim && !inner[d].col_free()) throw NotApplicable{};
        Pass p;
        p.node = a.get();
        p.rop = a->rop;
        p.body = emit(a->arg, inner);          // registers inner passes first
        passes.push_back(p);
        return "R" + std::to_string(passes.size() - 1);
      }
    }
    throw NotApplicable{};
  }
};

const char *PRELUDE = R"(
__device__ __forceinline__ float ugf_fold0(float a, float b) { return a + b; }
__device__ __forceinline__ float ugf_fold1(float a, float b) { return fmaxf(a, b); }
__device__ __forceinline__ float ugf_fold2(float a, float b) { return fminf(a, b); }
#define UGF_WARP_RED(FOLD, v, W) \
  for (int o_ = (W) / 2; o_ > 0; o_ >>= 1) v = FOLD(v, __shfl_xor_sync(0xffffffffu, v, o_));
)";

bool generate(const op::Kernel &k, const std::string &name, int W, FastKernel &out) {
  try {
    const op::Store &st = k.ops[0];
    const Layout &dl = st.layout;
    Gen g(k, W);
    g.n = dl.rank();
    const size_t total = dl.num_elements();
    const size_t CHUNK = 1024 * (size_t)W;
    size_t rows;
    if (dl.rank() == 1) {
      g.chunked = true;
      g.cols = CHUNK;
      rows = (total + CHUNK - 1) / CHUNK;
      if (total % W != 0) return false;
    } else {
      g.cols = dl.shape.back();
      rows = total / g.cols;
      if (g.cols % W != 0) return false;
    }
    if (W == 4 && dl.offset % 4 != 0) return false;
    Idx idx;
    for (size_t d = 0; d < g.n; ++d) {
      Affine a;
      if (d + 1 == g.n) a.cc = 1;          // chunked 1-D maps: the element index is row * CHUNK + column
      else { a.re = "i" + std::to_string(d); a.rm = 1; }
      idx.push_back(a);
    }
    const std::string value = g.emit(st.value, idx);
    const size_t dst_arg = g.arg_pos(st.dst);
    const size_t cw = g.cols / W;          // accesses per row
    // lanes per row: part of a warp for short rows (several rows per warp), a whole CTA of 256 .. 1024 threads otherwise
    const bool warp_mode = !g.chunked && cw <= 256;
    int threads = 256;
    if (warp_mode) threads = cw <= 8 ? 8 : (cw <= 16 ? 16 : 32);
    else if (!g.chunked) while (threads < 1024 && (cw + threads - 1) / threads > 8) threads *= 2;
    const int block = warp_mode ? 256 : threads;
    const size_t vpt = (cw + threads - 1) / threads;
    size_t cached = 0;
    for (auto &l : g.loads) if (l.kind == LoadSite::Vec) cached += vpt * W;
    if (vpt > 8 || cached > 96) return false;
    for (auto &l : g.loads)      // a store into one of its own operands needs the element-wise order of the SSA path
      if (l.arg == dst_arg) return false;

    const std::string ws = std::to_string(W);
    std::string s = PRELUDE;
    char buf[512];
    const std::string fn = "ugf_" + std::string(g.chunked ? "map" : (warp_mode ? "wrow" : "row")) + "_" + name;
    std::string fname;
    for (char c : fn) fname += (isalnum((unsigned char)c) ? c : '_');
    s += "extern \"C\" __global__ void __launch_bounds__(" + std::to_string(block) + ") " + fname + "(";
    for (size_t i = 0; i < k.args.size(); ++i) {
      if (k.args[i].dtype != DType::F32) return false;
      s += std::string(i ? ", " : "") + (i == dst_arg ? "float *__restrict__ a" : "const float *__restrict__ a") + std::to_string(i);
    }
    s += ") {\n";
    snprintf(buf, sizeof buf, "  constexpr int T = %d, VPT = %zu, W = %d, CW = %zu;\n  const long ROWS = %zuL, TOTAL = %zuL;\n", threads, vpt, W, cw, rows, total);
    s += buf;
    if (warp_mode) s += "  const int tid = threadIdx.x % T;\n  const long row = (long)blockIdx.x * (256 / T) + threadIdx.x / T;\n  const bool live_row = row < ROWS;\n";
    else s += "  const int tid = threadIdx.x;\n  const long row = blockIdx.x;\n  const bool live_row = true;\n  __shared__ float ugf_sm[2][T / 32];\n";
    s += "  (void)TOTAL; (void)ROWS;\n";
    // indexes of the row on the leading dims of the store
    if (!g.chunked) {
      s += "  long rem_ = row;\n";
      for (size_t d = g.n - 1; d-- > 0;) {
        snprintf(buf, sizeof buf, "  const long i%zu = rem_ %% %zuL; rem_ /= %zuL;\n", d, dl.shape[d], dl.shape[d]);
        s += buf;
      }
    }
    auto base_expr = [&](const Affine &a) {
      std::string e = std::to_string(a.off) + "L";
      if (g.chunked) {        // the only index is the element index: row * CHUNK + column
        if (a.cc != 0) e += " + " + std::to_string(a.cc * (long)CHUNK) + "L * row";
      } else if (!a.re.empty()) {
        e += " + " + a.re;
      }
      return e;
    };
    const std::string live = g.chunked ? "(row * CW + c_ < TOTAL / W)" : "(live_row && c_ < CW)";
    const std::string vty = W == 4 ? "float4" : "float";
    for (size_t i = 0; i < g.loads.size(); ++i) {
      const LoadSite &l = g.loads[i];
      const std::string id = std::to_string(i), arg = "a" + std::to_string(l.arg);
      s += "  const long B" + id + " = " + base_expr(l.addr) + ";\n";
      if (l.kind == LoadSite::Scalar) s += "  const float S" + id + " = live_row ? __ldg(" + arg + " + B" + id + ") : 0.f;\n";
      if (l.kind == LoadSite::Vec) {
        const std::string ld = (l.addr.re.empty() && !g.chunked) ? "__ldg" : "__ldcs";    // shared by all rows: keep it cached
        const std::string at = arg + " + B" + id + " + " + Gen::col_offset(l.addr, ws + "L * c_");
        s += "  float L" + id + "[VPT * W];\n#pragma unroll\n  for (int v_ = 0; v_ < VPT; ++v_) {\n    const int c_ = tid + v_ * T;\n";
        if (W == 4)
          s += "    float4 t_ = make_float4(0.f, 0.f, 0.f, 0.f);\n    if " + live + " t_ = " + ld + "(reinterpret_cast<const float4 *>(" + at + "));\n"
               "    L" + id + "[4 * v_] = t_.x; L" + id + "[4 * v_ + 1] = t_.y; L" + id + "[4 * v_ + 2] = t_.z; L" + id + "[4 * v_ + 3] = t_.w;\n  }\n";
        else
          s += "    L" + id + "[v_] = " + live + " ? " + ld + "(" + at + ") : 0.f;\n  }\n";
      }
    }
    for (size_t i = 0; i < g.passes.size(); ++i) {
      const Pass &p = g.passes[i];
      const std::string id = std::to_string(i), fold = "ugf_fold" + std::to_string((int)p.rop);
      const std::string init = p.rop == ReduceOp::Sum ? "0.f" : (p.rop == ReduceOp::Max ? "__int_as_float(0xff800000)" : "__int_as_float(0x7f800000)");
      s += "  float R" + id + ";\n  {\n    float acc_ = " + init + ";\n#pragma unroll\n    for (int v_ = 0; v_ < VPT; ++v_) {\n      const int c_ = tid + v_ * T;\n      if (live_row && c_ < CW) {\n#pragma unroll\n"
           "        for (int e_ = 0; e_ < W; ++e_) {\n          const int J = W * v_ + e_; const long COL = (long)W * c_ + e_; (void)J; (void)COL;\n"
           "          acc_ = " + fold + "(acc_, " + p.body + ");\n        }\n      }\n    }\n    UGF_WARP_RED(" + fold + ", acc_, T < 32 ? T : 32)\n";
      if (!warp_mode) {
        const std::string b = std::to_string(i & 1);
        s += "    if ((tid & 31) == 0) ugf_sm[" + b + "][tid >> 5] = acc_;\n    __syncthreads();\n    acc_ = ugf_sm[" + b + "][0];\n#pragma unroll\n"
             "    for (int w_ = 1; w_ < T / 32; ++w_) acc_ = " + fold + "(acc_, ugf_sm[" + b + "][w_]);\n";
      }
      s += "    R" + id + " = acc_;\n  }\n";
    }
    {
      const std::string dst = "a" + std::to_string(dst_arg);
      snprintf(buf, sizeof buf, "%zuL + row * %zuL", dl.offset, g.cols);
      s += "  float *out_ = " + dst + " + " + buf + ";\n#pragma unroll\n  for (int v_ = 0; v_ < VPT; ++v_) {\n    const int c_ = tid + v_ * T;\n    if " + live + " {\n      float o_[W];\n#pragma unroll\n"
           "      for (int e_ = 0; e_ < W; ++e_) {\n        const int J = W * v_ + e_; const long COL = (long)W * c_ + e_; (void)J; (void)COL;\n        o_[e_] = " + value + ";\n      }\n";
      if (W == 4) s += "      __stcs(reinterpret_cast<float4 *>(out_) + c_, make_float4(o_[0], o_[1], o_[2], o_[3]));\n";
      else s += "      __stcs(out_ + c_, o_[0]);\n";
      s += "    }\n  }\n}\n";
    }
    out.source = std::move(s);
    out.func_name = fname;
    const size_t rows_per_cta = warp_mode ? 256 / threads : 1;
    out.launch.grid_dim = (uint32_t)((rows + rows_per_cta - 1) / rows_per_cta);
    out.launch.block_dim = (uint32_t)block;
    out.launch.shared_mem = 0;
    const std::string w = W == 4 ? "vec4" : "scalar";
    out.origin = (g.chunked ? "map_" : (warp_mode ? "warp_row_" : "row_")) + w;
    return true;
  } catch (const NotApplicable &) {
    return false;
  }
}

}  // namespace

// Returns true and fills `out` when `k` (already through optimize()) is one of the shapes above: 128-bit accesses
// where the row length and every base allow them, otherwise the same kernel with one element per access.  A store of
// zero elements (the empty KV cache of model.rs:192-193) needs no code at all: origin "empty".
bool fast_kernel(const op::Kernel &k, const std::string &name, FastKernel &out) {
  if (k.ops.size() != 1) return false;
  const op::Store &st = k.ops[0];
  const Layout &dl = st.layout;
  if (dl.rank() >= 1 && dl.num_elements() == 0) {
    out = FastKernel{};
    out.origin = "empty";
    return true;
  }
  if (st.value->dtype != DType::F32 || dl.rank() == 0) return false;
  if (!dl.c_contiguous() || dl.num_elements() >= (1ull << 31)) return false;
  return generate(k, name, 4, out) || generate(k, name, 1, out);
}

// ug-llama/src/model.rs:32-63 as instructions: globals src (f32), ids (i32), dst (f32); for r in 0..n: the id is
// loaded (with an f32 tag, as the reference writes it), multiplied by h; for c in 0..h: dst[r * h + c] = src[id * h + c].
bool fast_ssa_kernel(const ssa::Kernel &k, FastKernel &out) {
  using ssa::K;
  const auto &in = k.instrs;
  if (in.size() != 14 || k.args.size() != 3) return false;
  const K kinds[14] = {K::DefineGlobal, K::DefineGlobal, K::DefineGlobal, K::Range, K::Load, K::Binary, K::Binary,
                       K::Range, K::Binary, K::Binary, K::Load, K::Store, K::EndRange, K::EndRange};
  for (int i = 0; i < 14; ++i) if (in[i].kind != kinds[i]) return false;
  auto is_i32 = [](const ssa::A &a, long &v) { if (a.is_var || a.cst.dtype != DType::I32) return false; v = a.cst.i32; return true; };
  auto is_var = [](const ssa::A &a, size_t v) { return a.is_var && a.var == v; };
  long lo1, n, lo2, h, h5, h6;
  if (in[0].dtype != DType::F32 || in[1].dtype != DType::I32 || in[2].dtype != DType::F32) return false;
  if (!is_i32(in[3].a0, lo1) || !is_i32(in[3].a1, n) || lo1 != 0 || in[3].index != 1) return false;
  if (in[4].v0 != 1 || !is_var(in[4].a0, 3)) return false;                                   // ids[r]
  if (in[5].bop != BinaryOp::Mul || !is_var(in[5].a0, 4) || !is_i32(in[5].a1, h5)) return false;
  if (in[6].bop != BinaryOp::Mul || !is_var(in[6].a0, 3) || !is_i32(in[6].a1, h6)) return false;
  if (!is_i32(in[7].a0, lo2) || !is_i32(in[7].a1, h) || lo2 != 0 || in[7].index != 1 || h5 != h || h6 != h) return false;
  if (in[8].bop != BinaryOp::Add || !is_var(in[8].a0, 5) || !is_var(in[8].a1, 7)) return false;
  if (in[9].bop != BinaryOp::Add || !is_var(in[9].a0, 6) || !is_var(in[9].a1, 7)) return false;
  if (in[10].v0 != 0 || !is_var(in[10].a0, 8) || in[10].dtype != DType::F32) return false;   // src[id * h + c]
  if (in[11].v0 != 2 || !is_var(in[11].a0, 9) || !is_var(in[11].a1, 10)) return false;       // dst[r * h + c]
  if (n <= 0 || h <= 0) return false;
  out = FastKernel{};
  out.origin = "index_select";
  out.n_ids = (size_t)n;
  out.h = (size_t)h;
  return true;
}

}  // namespace ug
