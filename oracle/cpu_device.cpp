// TEST INFRASTRUCTURE ONLY -- ug-core's CPU backend as an implementation of the
// C++ ug::Device interface (ug_b200/csrc/host/ug_graph.hpp), so that the same
// lazy graphs can run on the CPU oracle and on the B200 backend in the tests.
//
// Restates ug-core/src/cpu_code_gen.rs:68-186 (SSA -> C text, one statement per
// instruction, `__var{line}` names, ThreadIdx / BlockIdx / ReduceLocal rejected)
// and ug-core/src/cpu_runtime.rs: the C is written to a temporary file, built with
// exactly `gcc <c> -shared -lm -O3 -march=native -ffast-math -fomit-frame-pointer`
// (cpu_runtime.rs:476-488), dlopen-ed and called with 0..8 pointers
// (cpu_runtime.rs:274-334); matmul goes to the f32 GEMM stand-in of
// ug_cpu_ops.c (crate gemm 0.18.0 is not part of the reference tree) and, like
// the reference (cpu_runtime.rs:345-356,561-564), exists for F32 only here.
// Never linked into the shipped library.
#include <dlfcn.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>

#include "../ug_b200/csrc/host/ug_graph.hpp"

extern "C" void ug_gemm_f32(float *dst, const float *lhs, const float *rhs, size_t b, size_t m, size_t n, size_t k,
                            ptrdiff_t lhs_rs, ptrdiff_t lhs_cs, size_t a_skip, ptrdiff_t rhs_rs, ptrdiff_t rhs_cs,
                            size_t b_skip);

using namespace ug;

namespace {

struct CpuSlice : Slice {
  DType dt;
  size_t n;
  std::vector<uint8_t> bytes;
  CpuSlice(DType d, size_t len) : dt(d), n(len), bytes(len * size_in_bytes(d) + 8) {}
  DType dtype() const override { return dt; }
  size_t len() const override { return n; }
  void copy_host_to_device(const void *src, size_t len, DType dtype) override {  // cpu_runtime.rs:380-392
    if (dtype != dt) bail("htod dtype mismatch, dst ", dtype_str(dt), ", src ", dtype_str(dtype));
    if (len != n) bail("htod length mismatch, dst ", n, ", src ", len);
    std::memcpy(bytes.data(), src, len * size_in_bytes(dt));
  }
  void copy_device_to_host(void *dst, size_t len, DType dtype) const override {
    if (dtype != dt) bail("dtoh dtype mismatch, dst ", dtype_str(dtype), ", src ", dtype_str(dt));
    if (len != n) bail("dtoh length mismatch, dst ", len, ", src ", n);
    std::memcpy(dst, bytes.data(), len * size_in_bytes(dt));
  }
};

struct CpuFunc : Func {
  void *lib = nullptr;
  void *sym = nullptr;
  size_t n_args = 0;
  std::string c_code;
  ~CpuFunc() override { if (lib) dlclose(lib); }
};

const char *c_type(DType d) {  // cpu_code_gen.rs:55-66
  switch (d) {
    case DType::BF16: return "__bf16";
    case DType::F16: return "_Float16";
    case DType::F32: return "float";
    case DType::I32: return "int";
    case DType::I64: return "long long";
  }
  return "?";
}
std::string fmt_f32(float v) {  // cpu_code_gen.rs:14-28
  if (std::isnan(v)) return "0. / 0.";
  if (std::isinf(v)) return v > 0 ? "1. / 0." : "-1. / 0.";
  char buf[64];
  snprintf(buf, sizeof buf, "%.9g", (double)v);
  std::string s = buf;
  if (s.find_first_of(".einf") == std::string::npos) s += ".0";   // a float literal, as Rust's {:?} prints one
  return s;
}
std::string fmt_const(const Const &c) {
  switch (c.dtype) {
    case DType::F32: return fmt_f32(c.f32);
    case DType::BF16: return fmt_f32(bf16_bits_to_f32(c.h));
    case DType::F16: bail("f16 constants are not covered by the oracle");
    case DType::I32: return std::to_string(c.i32);
    case DType::I64: return std::to_string(c.i64);
  }
  return "0";
}
std::string fmt_a(const ssa::A &a) { return a.is_var ? "__var" + std::to_string(a.var) : fmt_const(a.cst); }

// cpu_code_gen.rs:68-186
std::string gen_c(const std::string &name, const ssa::Kernel &k) {
  using ssa::K;
  for (auto &i : k.instrs)
    if (i.kind == K::ReduceLocal) bail("TODO: add the reduce code if needed");
  std::ostringstream w;
  w << "#include<math.h>\nvoid " << name << "(\n";
  for (size_t a = 0; a < k.args.size(); ++a)
    w << "  " << c_type(k.args[a].first.dtype) << "* __var" << k.args[a].second << (a + 1 == k.args.size() ? "" : ",") << "\n";
  w << ") {\n";
  size_t depth = 0;
  for (size_t l = 0; l < k.instrs.size(); ++l) {
    const ssa::Instr &i = k.instrs[l];
    const std::string v = "__var" + std::to_string(l);
    std::string ind(2 * depth + 2, ' ');
    switch (i.kind) {
      case K::DefineGlobal: break;
      case K::DefineLocal: w << ind << "__shared__ " << c_type(i.dtype) << " " << v << "[" << i.index << "];\n"; break;
      case K::DefineAcc: case K::Const: w << ind << c_type(i.cst.dtype) << " " << v << " = " << fmt_const(i.cst) << ";\n"; break;
      case K::If: w << ind << "if (" << fmt_a(i.a0) << ") {\n"; depth++; break;
      case K::Range:
        w << ind << "for (int " << v << " = " << fmt_a(i.a0) << "; " << v << " < " << fmt_a(i.a1) << "; " << v << "+=" << i.index << ") {\n";
        depth++;
        break;
      case K::EndIf: case K::EndRange:
        if (depth == 0) bail("unmatched EndRange");
        depth--;
        w << std::string(2 * depth + 2, ' ') << "}\n";
        break;
      case K::Load: w << ind << c_type(i.dtype) << " " << v << " = __var" << i.v0 << "[" << fmt_a(i.a0) << "];\n"; break;
      case K::Assign: w << ind << "__var" << i.v0 << " = " << fmt_a(i.a0) << ";\n"; break;
      case K::Store: w << ind << "__var" << i.v0 << "[" << fmt_a(i.a0) << "] = " << fmt_a(i.a1) << ";\n"; break;
      case K::Binary: {
        const std::string a = fmt_a(i.a0), b = fmt_a(i.a1);
        std::string e;
        switch (i.bop) {
          case BinaryOp::Add: e = a + " + " + b; break;
          case BinaryOp::Mul: e = a + " * " + b; break;
          case BinaryOp::Sub: e = a + " - " + b; break;
          case BinaryOp::Div: e = a + " / " + b; break;
          case BinaryOp::Min: e = "fmin(" + a + ", " + b + ")"; break;
          case BinaryOp::Max: e = "fmax(" + a + ", " + b + ")"; break;
          case BinaryOp::Mod: e = a + " % " + b; break;
        }
        w << ind << c_type(i.dtype) << " " << v << " = " << e << ";\n";
        break;
      }
      case K::Unary: {
        std::string f;
        switch (i.uop.kind) {
          case UnaryKind::Sqrt: f = "sqrtf"; break;
          case UnaryKind::Exp: f = "expf"; break;
          case UnaryKind::Sin: f = "sinf"; break;
          case UnaryKind::Cos: f = "cosf"; break;
          case UnaryKind::Neg: f = "-"; break;
          case UnaryKind::Id: f = ""; break;
          case UnaryKind::Cast: f = std::string("(") + c_type(i.dtype) + ")"; break;
        }
        w << ind << c_type(i.dtype) << " " << v << " = " << f << "(" << fmt_a(i.a0) << ");\n";
        break;
      }
      case K::Special:
        bail(i.special == ssa::Special::ThreadIdx ? "thread-id is currently not supported in the cpu backend"
                                                 : "block-id is currently not supported in the cpu backend");
      case K::Barrier: break;
      case K::ReduceLocal: break;
    }
  }
  w << "}\n";
  if (depth > 0) bail("unmatched Range");
  return w.str();
}

struct CpuDevice : Device {
  std::unique_ptr<Slice> allocate_uninit(DType dtype, size_t len) override { return std::make_unique<CpuSlice>(dtype, len); }
  void synchronize() override {}
  std::shared_ptr<Func> compile(const ssa::Kernel &k, const std::string *name) override {
    static std::atomic<size_t> counter{1};
    const size_t id = counter.fetch_add(1);
    const std::string fn = std::string("ugc_") + (name ? *name : std::string("kernel")) + "_" + std::to_string(getpid()) + "_" + std::to_string(id);
    std::string safe;
    for (char c : fn) safe += (isalnum((unsigned char)c) || c == '_') ? c : '_';
    auto f = std::make_shared<CpuFunc>();
    f->c_code = gen_c(safe, k);
    f->n_args = k.args.size();
    const char *tmp = getenv("TMPDIR");
    const std::string dir = tmp ? tmp : "/tmp";
    const std::string c_path = dir + "/" + safe + ".c", so_path = dir + "/" + safe + ".so";
    { std::ofstream o(c_path); o << f->c_code; }
    const std::string cmd = "gcc " + c_path + " -shared -lm -O3 -march=native -ffast-math -fomit-frame-pointer -o " + so_path + " 2>" + c_path + ".log";
    const int rc = std::system(cmd.c_str());
    if (rc != 0) {
      std::ifstream lg(c_path + ".log");
      std::stringstream ss; ss << lg.rdbuf();
      bail("compilation failed\nstderr:\n", ss.str().substr(0, 2000), "\n--- source ---\n", f->c_code.substr(0, 3000));
    }
    f->lib = dlopen(so_path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!getenv("UG_KEEP_TMP")) { unlink(c_path.c_str()); unlink(so_path.c_str()); unlink((c_path + ".log").c_str()); }   // utils.rs:3-12
    if (!f->lib) bail("dlopen failed: ", dlerror());
    f->sym = dlsym(f->lib, safe.c_str());
    if (!f->sym) bail("symbol not found: ", safe);
    return f;
  }
  void run(Func &fb, std::vector<Slice *> &args) override {
    auto &f = static_cast<CpuFunc &>(fb);
    if (args.size() != f.n_args) bail("unsupported number of args for kernel ", args.size());
    void *p[8] = {};
    if (args.size() > 8) bail("unsupported number of args for kernel ", args.size());
    for (size_t i = 0; i < args.size(); ++i) p[i] = static_cast<CpuSlice *>(args[i])->bytes.data();
    using F8 = void (*)(void *, void *, void *, void *, void *, void *, void *, void *);
    // extra trailing pointer arguments are ignored by the SysV x86-64 calling convention
    ((F8)f.sym)(p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7]);
  }
  void matmul(Slice &dst, const Slice &lhs, const Slice &rhs, size_t b, size_t m, size_t n, size_t k, const Layout &ll,
              const Layout &rl) override {  // cpu_runtime.rs:513-619
    if (dst.dtype() != DType::F32 || lhs.dtype() != DType::F32 || rhs.dtype() != DType::F32) bail("unsupported dtype for gemm");
    auto skip = [&](const Layout &l, size_t dflt, const char *msg) -> size_t {
      const size_t r = l.rank();
      if (r == 2) return dflt;
      if (r == 3) return l.strides[0];
      if (r == 4) {
        if (l.strides[0] == l.strides[1] * l.shape[1]) return l.strides[1];
        if (l.shape[0] == 1) return l.strides[1];
        if (l.shape[1] == 1) return l.strides[0];
      }
      bail(msg);
    };
    const size_t a_skip = skip(ll, m * k, "non-contiguous lhs"), b_skip = skip(rl, n * k, "non-contiguous rhs");
    const size_t r = ll.rank();
    auto &d = static_cast<CpuSlice &>(dst);
    auto &l = static_cast<const CpuSlice &>(lhs);
    auto &rr = static_cast<const CpuSlice &>(rhs);
    ug_gemm_f32((float *)d.bytes.data(), (const float *)l.bytes.data() + ll.offset, (const float *)rr.bytes.data() + rl.offset, b, m,
                n, k, (ptrdiff_t)ll.strides[r - 2], (ptrdiff_t)ll.strides[r - 1], a_skip, (ptrdiff_t)rl.strides[r - 2],
                (ptrdiff_t)rl.strides[r - 1], b_skip);
  }
  bool use_grid() const override { return false; }  // cpu_runtime.rs:270-272
};

}  // namespace

extern "C" {
// A heap-allocated ug::Device* for ugh_device_adopt.
__attribute__((visibility("default"))) void *oracle_cpu_device_new() { return static_cast<Device *>(new CpuDevice()); }
// Host pointer of a CPU slice (custom ops of the CPU device work on host memory directly).
__attribute__((visibility("default"))) void *oracle_cpu_slice_ptr(void *slice) {
  auto *s = dynamic_cast<CpuSlice *>(reinterpret_cast<Slice *>(slice));
  return s ? s->bytes.data() : nullptr;
}
// The C text the CPU backend emits for a hand-built SSA kernel made of `n` instructions in the wire format.
}
