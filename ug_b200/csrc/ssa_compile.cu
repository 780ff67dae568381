// ug::Device::compile / run for raw SSA kernels (ug-core/src/lib.rs:56-60).
//
// The reference turns an ssa::Kernel into CUDA C, one statement per
// instruction, and compiles it with NVRTC under use_fast_math
// (ug-cuda/src/code_gen.rs:68-186, runtime.rs:179-186,247-264).  This file is
// the counterpart for this backend, written from the instruction semantics
// (ug-core/src/lang.rs:690-709, ug-core/src/interpreter.rs):
//   * accurate expf / sinf / cosf / IEEE division (results are checked against
//     ug's CPU backend, not against the fast-math CUDA one);
//   * every Load / Store is bounds-checked against the length of the slice it
//     addresses (lengths travel as extra kernel parameters); an out-of-range
//     access is skipped and raises the device status word instead of faulting;
//   * ReduceLocal is a block-wide reduction that works for any block size;
//   * compiled for sm_100a straight to a cubin.
// NVRTC and the few driver entry points needed to load a cubin are resolved at
// run time (dlopen / cudaGetDriverEntryPoint), so the library still loads on a
// machine without them and fails with a message at the first compile.
#include <cuda.h>
#include <dlfcn.h>

#include <atomic>
#include <cctype>
#include <cstdlib>
#include <mutex>
#include <cstring>
#include <sstream>
#include <string>
#include <vector>

#include "ugb_internal.h"

struct ugb_func {
  ugb_device *dev = nullptr;
  CUmodule module = nullptr;
  CUfunction fn = nullptr;
  unsigned grid = 1, block = 1, smem = 0;
  std::vector<int32_t> arg_dtypes;
  std::string source, name;
  bool raw = false;     // user-supplied CUDA C / PTX: pointer arguments only, no length or status parameters
  int n_dyn = 0;        // trailing `long long` value parameters that ugb_run_dyn supplies
};

namespace {

// ---- dynamically resolved NVRTC and driver entry points ---------------------
typedef int nvrtcResult_t;
struct Nvrtc {
  void *lib = nullptr;
  nvrtcResult_t (*create)(void **, const char *, const char *, int, const char *const *, const char *const *) = nullptr;
  nvrtcResult_t (*compile)(void *, int, const char *const *) = nullptr;
  nvrtcResult_t (*log_size)(void *, size_t *) = nullptr;
  nvrtcResult_t (*get_log)(void *, char *) = nullptr;
  nvrtcResult_t (*cubin_size)(void *, size_t *) = nullptr;
  nvrtcResult_t (*get_cubin)(void *, char *) = nullptr;
  nvrtcResult_t (*destroy)(void **) = nullptr;
  std::string error;
};
Nvrtc &nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char *names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so"};
    for (const char *nm : names)
      if ((n.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL))) break;
    if (!n.lib) { n.error = "libnvrtc not found (tried libnvrtc.so.12 and /usr/local/cuda/lib64)"; return; }
#define SYM(field, name) *(void **)(&n.field) = dlsym(n.lib, name); if (!n.field) { n.error = std::string("missing symbol ") + name; return; }
    SYM(create, "nvrtcCreateProgram") SYM(compile, "nvrtcCompileProgram") SYM(log_size, "nvrtcGetProgramLogSize")
    SYM(get_log, "nvrtcGetProgramLog") SYM(cubin_size, "nvrtcGetCUBINSize") SYM(get_cubin, "nvrtcGetCUBIN")
    SYM(destroy, "nvrtcDestroyProgram")
#undef SYM
  });
  return n;
}

struct Driver {
  CUresult (*module_load_data)(CUmodule *, const void *) = nullptr;
  CUresult (*module_get_function)(CUfunction *, CUmodule, const char *) = nullptr;
  CUresult (*module_unload)(CUmodule) = nullptr;
  CUresult (*launch_kernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                            void **, void **) = nullptr;
  std::string error;
};
Driver &driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [&](const char *name, void **out) {
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !*out)
        d.error = std::string("driver entry point not available: ") + name;
    };
    get("cuModuleLoadData", (void **)&d.module_load_data);
    get("cuModuleGetFunction", (void **)&d.module_get_function);
    get("cuModuleUnload", (void **)&d.module_unload);
    get("cuLaunchKernel", (void **)&d.launch_kernel);
  });
  return d;
}

// ---- code generation ----------------------------------------------------------
const char *c_type(int32_t dt) {
  switch (dt) {
    case UGB_BF16: return "__nv_bfloat16";
    case UGB_F16: return "__half";
    case UGB_F32: return "float";
    case UGB_I32: return "int";
    case UGB_I64: return "long long";
  }
  return nullptr;
}
bool is_float(int32_t dt) { return dt == UGB_BF16 || dt == UGB_F16 || dt == UGB_F32; }

std::string const_str(const ugb_ssa_arg &a) {
  std::ostringstream os;
  switch (a.dtype) {
    case UGB_F32: {
      uint32_t bits = (uint32_t)a.value;
      os << "__uint_as_float(0x" << std::hex << bits << "u)";   // exact, covers +-inf
      break;
    }
    case UGB_BF16: os << "__ushort_as_bfloat16((unsigned short)0x" << std::hex << (uint16_t)a.value << ")"; break;
    case UGB_F16: os << "__ushort_as_half((unsigned short)0x" << std::hex << (uint16_t)a.value << ")"; break;
    case UGB_I32: os << "(int)" << (int32_t)a.value; break;
    case UGB_I64: os << (long long)a.value << "ll"; break;
  }
  return os.str();
}
std::string arg_str(const ugb_ssa_arg &a) { return a.is_var ? "v" + std::to_string((long long)a.value) : const_str(a); }

const char *PRELUDE = R"(
#include <cuda_bf16.h>
#include <cuda_fp16.h>
struct ugb_status_word { unsigned int code; unsigned int detail; };
__device__ __forceinline__ void ugb_oob(ugb_status_word* s, unsigned int line) {
  if (atomicCAS(&s->code, 0u, 3u) == 0u) s->detail = line;
}
template <typename T> struct UgbSum { __device__ T operator()(T a, T b) const { return a + b; } };
template <typename T> struct UgbMax { __device__ T operator()(T a, T b) const { return a > b ? a : b; } };
template <typename T> struct UgbMin { __device__ T operator()(T a, T b) const { return a < b ? a : b; } };
template <> struct UgbMax<float> { __device__ float operator()(float a, float b) const { return fmaxf(a, b); } };
template <> struct UgbMin<float> { __device__ float operator()(float a, float b) const { return fminf(a, b); } };
// Block-wide reduction for any blockDim.x <= 1024; every thread of the block must call it.
template <typename T, typename Op> __device__ T ugb_block_reduce(T v, Op op) {
  __shared__ T sm[1024];
  const unsigned tid = threadIdx.x, n = blockDim.x;
  sm[tid] = v;
  __syncthreads();
  unsigned s = 1;
  while (s < n) s <<= 1;
  for (s >>= 1; s > 0; s >>= 1) {
    if (tid < s && tid + s < n) sm[tid] = op(sm[tid], sm[tid + s]);
    __syncthreads();
  }
  const T r = sm[0];
  __syncthreads();
  return r;
}
__device__ __forceinline__ float ugb_f(float v) { return v; }
__device__ __forceinline__ float ugb_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float ugb_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float ugb_f(int v) { return (float)v; }
__device__ __forceinline__ float ugb_f(long long v) { return (float)v; }
template <typename T> __device__ __forceinline__ T ugb_from_f(float v);
template <> __device__ __forceinline__ float ugb_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 ugb_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half ugb_from_f<__half>(float v) { return __float2half_rn(v); }
template <typename T, typename S> __device__ __forceinline__ T ugb_cast(S v) { return (T)v; }
template <> __device__ __forceinline__ __nv_bfloat16 ugb_cast<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half ugb_cast<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float ugb_cast<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float ugb_cast<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ __nv_bfloat16 ugb_cast<__nv_bfloat16, int>(int v) { return __float2bfloat16_rn((float)v); }
template <> __device__ __forceinline__ __half ugb_cast<__half, int>(int v) { return __float2half_rn((float)v); }
template <> __device__ __forceinline__ int ugb_cast<int, __nv_bfloat16>(__nv_bfloat16 v) { return (int)__bfloat162float(v); }
template <> __device__ __forceinline__ int ugb_cast<int, __half>(__half v) { return (int)__half2float(v); }
template <> __device__ __forceinline__ __nv_bfloat16 ugb_cast<__nv_bfloat16, __half>(__half v) { return __float2bfloat16_rn(__half2float(v)); }
template <> __device__ __forceinline__ __half ugb_cast<__half, __nv_bfloat16>(__nv_bfloat16 v) { return __float2half_rn(__bfloat162float(v)); }
)";

// One statement per instruction; variable n is `v<n>` (a line number, lang.rs:611-636).
int32_t generate(ugb_device *dev, const ugb_ssa_instr *ins, size_t n, const std::string &fname, std::string *out,
                 std::vector<int32_t> *arg_dtypes) {
  std::ostringstream os;
  os << PRELUDE << "\nextern \"C\" __global__ void " << fname << "(";
  // arguments: DefineGlobal instructions, in index order
  std::vector<std::pair<size_t, int32_t>> args;   // (line, dtype)
  for (size_t l = 0; l < n; ++l)
    if (ins[l].kind == UGB_SSA_DEFINE_GLOBAL) {
      UGB_REQUIRE(dev, (size_t)ins[l].index == args.size(), UGB_ERR_COMPILE, "unexpected order for arguments in kernel (line %zu)", l);
      UGB_REQUIRE(dev, c_type(ins[l].dtype) != nullptr, UGB_ERR_COMPILE, "line %zu: unknown dtype %d", l, ins[l].dtype);
      args.push_back({l, ins[l].dtype});
    }
  for (size_t i = 0; i < args.size(); ++i) os << c_type(args[i].second) << "* __restrict__ v" << args[i].first << ", ";
  for (size_t i = 0; i < args.size(); ++i) os << "unsigned long long n" << args[i].first << ", ";
  os << "ugb_status_word* ugb_status) {\n";
  // dtype of every defined value, for casts and typed helpers
  std::vector<int32_t> vtype(n, -1);
  int depth = 0;
  auto type_of = [&](const ugb_ssa_arg &a) -> int32_t { return a.is_var ? ((size_t)a.value < n ? vtype[(size_t)a.value] : -1) : a.dtype; };
  for (size_t l = 0; l < n; ++l) {
    const ugb_ssa_instr &i = ins[l];
    const std::string ind(2 * (size_t)depth + 2, ' ');
    const char *ty = c_type(i.dtype);
    auto need_type = [&]() -> int32_t {
      if (!ty) return ugb_fail(dev, UGB_ERR_COMPILE, "line %zu: unknown dtype %d", l, i.dtype);
      return UGB_OK;
    };
    auto need_var = [&](long long v) -> int32_t {
      if (v < 0 || (size_t)v >= n) return ugb_fail(dev, UGB_ERR_COMPILE, "line %zu: variable %lld out of range", l, v);
      return UGB_OK;
    };
    int32_t rc = UGB_OK;
    switch (i.kind) {
      case UGB_SSA_DEFINE_GLOBAL: vtype[l] = i.dtype; break;
      case UGB_SSA_DEFINE_LOCAL:
        if ((rc = need_type())) return rc;
        os << ind << "__shared__ " << ty << " v" << l << "[" << i.index << "];\n";
        vtype[l] = i.dtype;
        break;
      case UGB_SSA_DEFINE_ACC:
      case UGB_SSA_CONST: {
        const char *cty = c_type(i.cst.dtype);
        UGB_REQUIRE(dev, cty != nullptr && !i.cst.is_var, UGB_ERR_COMPILE, "line %zu: bad constant", l);
        os << ind << cty << " v" << l << " = " << const_str(i.cst) << ";\n";
        vtype[l] = i.cst.dtype;
        break;
      }
      case UGB_SSA_SPECIAL:
        os << ind << "int v" << l << " = " << (i.op == UGB_SSA_THREAD_IDX ? "(int)threadIdx.x" : "(int)blockIdx.x") << ";\n";
        vtype[l] = UGB_I32;
        break;
      case UGB_SSA_UNARY: {
        if ((rc = need_type())) return rc;
        const std::string a = arg_str(i.a0);
        const int32_t st = type_of(i.a0);
        std::string e;
        const bool f = is_float(i.dtype);
        auto fwrap = [&](const char *fn) {   // float math in f32, rounded back to the value dtype
          return std::string("ugb_from_f<") + ty + ">(" + fn + "(ugb_f(" + a + ")))";
        };
        switch (i.op) {
          case UGB_UNARY_ID: e = a; break;
          case UGB_UNARY_EXP: e = fwrap("expf"); break;
          case UGB_UNARY_SIN: e = fwrap("sinf"); break;
          case UGB_UNARY_COS: e = fwrap("cosf"); break;
          case UGB_UNARY_SQRT: e = fwrap("sqrtf"); break;
          case UGB_UNARY_NEG: e = f && i.dtype != UGB_F32 ? fwrap("-") : "-(" + a + ")"; break;
          case UGB_UNARY_CAST: {
            const char *sty = c_type(st);
            UGB_REQUIRE(dev, sty != nullptr, UGB_ERR_COMPILE, "line %zu: cast of a value of unknown type", l);
            e = std::string("ugb_cast<") + ty + ", " + sty + ">(" + a + ")";
            break;
          }
          default: return ugb_fail(dev, UGB_ERR_COMPILE, "line %zu: unknown unary op %d", l, i.op);
        }
        if ((i.op == UGB_UNARY_EXP || i.op == UGB_UNARY_SIN || i.op == UGB_UNARY_COS || i.op == UGB_UNARY_SQRT) && !f)
          return ugb_fail(dev, UGB_ERR_COMPILE, "line %zu: transcendental on an integer value", l);
        os << ind << ty << " v" << l << " = " << e << ";\n";
        vtype[l] = i.dtype;
        break;
      }
      case UGB_SSA_BINARY: {
        if ((rc = need_type())) return rc;
        const std::string a = arg_str(i.a0), b = arg_str(i.a1);
        std::string e;
        const bool half = i.dtype == UGB_BF16 || i.dtype == UGB_F16;
        auto arith = [&](const char *op) {
          if (half) return std::string("ugb_from_f<") + ty + ">(ugb_f(" + a + ") " + op + " ugb_f(" + b + "))";
          return "(" + a + ") " + op + " (" + b + ")";
        };
        switch (i.op) {
          case UGB_BINARY_ADD: e = arith("+"); break;
          case UGB_BINARY_SUB: e = arith("-"); break;
          case UGB_BINARY_MUL: e = arith("*"); break;
          case UGB_BINARY_DIV: e = arith("/"); break;
          case UGB_BINARY_MOD:
            e = is_float(i.dtype) ? std::string("ugb_from_f<") + ty + ">(fmodf(ugb_f(" + a + "), ugb_f(" + b + ")))" : arith("%");
            break;
          case UGB_BINARY_MIN:
          case UGB_BINARY_MAX: {
            const char *fn = i.op == UGB_BINARY_MIN ? (is_float(i.dtype) ? "fminf" : "min") : (is_float(i.dtype) ? "fmaxf" : "max");
            e = is_float(i.dtype) ? std::string("ugb_from_f<") + ty + ">(" + fn + "(ugb_f(" + a + "), ugb_f(" + b + ")))"
                                  : std::string(fn) + "((" + ty + ")(" + a + "), (" + ty + ")(" + b + "))";
            break;
          }
          default: return ugb_fail(dev, UGB_ERR_COMPILE, "line %zu: unknown binary op %d", l, i.op);
        }
        os << ind << ty << " v" << l << " = " << e << ";\n";
        vtype[l] = i.dtype;
        break;
      }
      case UGB_SSA_RANGE:
        os << ind << "for (int v" << l << " = " << arg_str(i.a0) << "; v" << l << " < " << arg_str(i.a1) << "; v" << l << " += "
           << (i.index > 0 ? i.index : 1) << ") {\n";
        vtype[l] = UGB_I32;
        depth++;
        break;
      case UGB_SSA_IF:
        os << ind << "if (" << arg_str(i.a0) << ") {\n";
        depth++;
        break;
      case UGB_SSA_END_RANGE:
      case UGB_SSA_END_IF:
        UGB_REQUIRE(dev, depth > 0, UGB_ERR_COMPILE, "line %zu: unmatched end of range / if", l);
        depth--;
        os << std::string(2 * (size_t)depth + 2, ' ') << "}\n";
        break;
      case UGB_SSA_LOAD: {
        if ((rc = need_type()) || (rc = need_var(i.v0))) return rc;
        const bool global = ins[i.v0].kind == UGB_SSA_DEFINE_GLOBAL;
        UGB_REQUIRE(dev, global || ins[i.v0].kind == UGB_SSA_DEFINE_LOCAL, UGB_ERR_COMPILE, "line %zu: load from a non-buffer", l);
        const char *bty = c_type(ins[i.v0].dtype);
        // a load may name another dtype than the buffer's (ug-llama/src/model.rs:49 reads i32 ids as f32): convert
        const std::string elem = std::string("ugb_cast<") + ty + ", " + bty + ">(v" + std::to_string(i.v0) + "[o" + std::to_string(l) + "])";
        os << ind << "const long long o" << l << " = (long long)(" << arg_str(i.a0) << ");\n";
        // every access is checked against the buffer's length -- the slice length for an argument, the declared size for
        // shared memory -- and raises the status word instead of touching memory outside it
        os << ind << ty << " v" << l << " = (" << ty << ")0;\n";
        if (global) os << ind << "if ((unsigned long long)o" << l << " < n" << i.v0 << ") v" << l << " = " << elem << "; else ugb_oob(ugb_status, " << l << "u);\n";
        else os << ind << "if ((unsigned long long)o" << l << " < " << ins[i.v0].index << "ull) v" << l << " = " << elem << "; else ugb_oob(ugb_status, " << l << "u);\n";
        vtype[l] = i.dtype;
        break;
      }
      case UGB_SSA_STORE: {
        if ((rc = need_var(i.v0))) return rc;
        const bool global = ins[i.v0].kind == UGB_SSA_DEFINE_GLOBAL;
        UGB_REQUIRE(dev, global || ins[i.v0].kind == UGB_SSA_DEFINE_LOCAL, UGB_ERR_COMPILE, "line %zu: store to a non-buffer", l);
        const char *bty = c_type(ins[i.v0].dtype);
        const int32_t st = type_of(i.a1);
        const char *sty = c_type(st);
        UGB_REQUIRE(dev, sty != nullptr, UGB_ERR_COMPILE, "line %zu: store of a value of unknown type", l);
        const std::string val = std::string("ugb_cast<") + bty + ", " + sty + ">(" + arg_str(i.a1) + ")";
        os << ind << "{ const long long o = (long long)(" << arg_str(i.a0) << "); ";
        if (global) os << "if ((unsigned long long)o < n" << i.v0 << ") v" << i.v0 << "[o] = " << val << "; else ugb_oob(ugb_status, " << l << "u); }\n";
        else os << "if ((unsigned long long)o < " << ins[i.v0].index << "ull) v" << i.v0 << "[o] = " << val << "; else ugb_oob(ugb_status, " << l << "u); }\n";
        break;
      }
      case UGB_SSA_ASSIGN:
        if ((rc = need_var(i.v0))) return rc;
        os << ind << "v" << i.v0 << " = " << arg_str(i.a0) << ";\n";
        break;
      case UGB_SSA_BARRIER: os << ind << "__syncthreads();\n"; break;
      case UGB_SSA_REDUCE_LOCAL: {
        if ((rc = need_type())) return rc;
        const char *opn = i.op == UGB_REDUCE_SUM ? "UgbSum" : (i.op == UGB_REDUCE_MAX ? "UgbMax" : "UgbMin");
        if (i.dtype == UGB_BF16 || i.dtype == UGB_F16)
          os << ind << ty << " v" << l << " = ugb_from_f<" << ty << ">(ugb_block_reduce(ugb_f(" << arg_str(i.a0) << "), " << opn << "<float>()));\n";
        else
          os << ind << ty << " v" << l << " = ugb_block_reduce((" << ty << ")(" << arg_str(i.a0) << "), " << opn << "<" << ty << ">());\n";
        vtype[l] = i.dtype;
        break;
      }
      default: return ugb_fail(dev, UGB_ERR_COMPILE, "line %zu: unknown instruction kind %d", l, i.kind);
    }
  }
  UGB_REQUIRE(dev, depth == 0, UGB_ERR_COMPILE, "unmatched Range / If");
  os << "}\n";
  *out = os.str();
  for (auto &a : args) arg_dtypes->push_back(a.second);
  return UGB_OK;
}

// NVRTC (unless `is_ptx`) -> module -> function.  `fast_math`: the reference compiles user CUDA C with
// use_fast_math (ug-cuda/src/runtime.rs:179-186); generated kernels are compiled without it.
int32_t compile_and_load(ugb_device *dev, const std::string &src, const std::string &unit, const std::string &entry,
                         bool fast_math, bool is_ptx, ugb_func **out) {
  Driver &drv = driver();
  UGB_REQUIRE(dev, drv.error.empty(), UGB_ERR_COMPILE, "%s", drv.error.c_str());
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  std::vector<char> image;
  if (is_ptx) {
    image.assign(src.begin(), src.end());
    image.push_back('\0');
  } else {
    Nvrtc &nv = nvrtc();
    UGB_REQUIRE(dev, nv.error.empty(), UGB_ERR_COMPILE, "NVRTC unavailable: %s", nv.error.c_str());
    void *prog = nullptr;
    if (nv.create(&prog, src.c_str(), (unit + ".cu").c_str(), 0, nullptr, nullptr) != 0)
      return ugb_fail(dev, UGB_ERR_COMPILE, "nvrtcCreateProgram failed");
    const char *cuda_home = getenv("CUDA_HOME");
    const std::string inc = std::string("--include-path=") + (cuda_home ? cuda_home : "/usr/local/cuda") + "/include";
    const char *opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", inc.c_str(), "--use_fast_math"};
    const nvrtcResult_t cr = nv.compile(prog, fast_math ? 4 : 3, opts);
    if (cr != 0) {
      size_t ls = 0;
      nv.log_size(prog, &ls);
      std::string log(ls, '\0');
      if (ls) nv.get_log(prog, &log[0]);
      nv.destroy(&prog);
      return ugb_fail(dev, UGB_ERR_COMPILE, "NVRTC failed for %s: %.700s", unit.c_str(), log.c_str());
    }
    size_t cs = 0;
    nv.cubin_size(prog, &cs);
    image.resize(cs);
    nv.get_cubin(prog, image.data());
    nv.destroy(&prog);
  }
  ugb_func *f = new ugb_func();
  f->dev = dev;
  f->source = src;
  f->name = entry;
  CUresult r = drv.module_load_data(&f->module, image.data());
  if (r == CUDA_SUCCESS) r = drv.module_get_function(&f->fn, f->module, entry.c_str());
  if (r != CUDA_SUCCESS) {
    if (f->module) drv.module_unload(f->module);
    delete f;
    return ugb_fail(dev, UGB_ERR_COMPILE, "loading kernel %s failed with CUresult %d", entry.c_str(), (int)r);
  }
  *out = f;
  return UGB_OK;
}

}  // namespace

extern "C" {

int32_t ugb_compile(ugb_device *dev, const ugb_ssa_instr *instrs, size_t n_instrs, uint32_t grid_dim, uint32_t block_dim,
                    uint32_t shared_mem, const char *name, ugb_func **out) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, out != nullptr && (instrs != nullptr || n_instrs == 0), UGB_ERR_INVALID, "ugb_compile: null argument");
  *out = nullptr;
  UGB_REQUIRE(dev, block_dim <= 1024, UGB_ERR_INVALID, "ugb_compile: block_dim %u exceeds 1024", block_dim);
  static std::atomic<unsigned> kernel_id{1};
  std::string fname = "ug_";
  if (name) for (const char *c = name; *c; ++c) fname += (isalnum((unsigned char)*c) ? *c : '_');
  fname += "_" + std::to_string(kernel_id.fetch_add(1));
  std::string src;
  std::vector<int32_t> arg_dtypes;
  int32_t rc = generate(dev, instrs, n_instrs, fname, &src, &arg_dtypes);
  if (rc) return rc;

  ugb_func *f = nullptr;
  rc = compile_and_load(dev, src, fname, fname, false, false, &f);
  if (rc) return rc;
  f->grid = grid_dim; f->block = block_dim; f->smem = shared_mem;
  f->arg_dtypes = arg_dtypes;
  *out = f;
  return UGB_OK;
}

int32_t ugb_compile_cu(ugb_device *dev, const char *cu_code, const char *func_name, uint32_t grid_dim,
                       uint32_t block_dim, uint32_t shared_mem, ugb_func **out) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, cu_code && func_name && out, UGB_ERR_INVALID, "ugb_compile_cu: null argument");
  *out = nullptr;
  ugb_func *f = nullptr;
  const int32_t rc = compile_and_load(dev, cu_code, func_name, func_name, true, false, &f);
  if (rc) return rc;
  f->grid = grid_dim; f->block = block_dim; f->smem = shared_mem;
  f->raw = true;
  *out = f;
  return UGB_OK;
}

int32_t ugb_compile_ptx(ugb_device *dev, const char *ptx_code, const char *func_name, uint32_t grid_dim,
                        uint32_t block_dim, uint32_t shared_mem, ugb_func **out) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, ptx_code && func_name && out, UGB_ERR_INVALID, "ugb_compile_ptx: null argument");
  *out = nullptr;
  ugb_func *f = nullptr;
  const int32_t rc = compile_and_load(dev, ptx_code, func_name, func_name, false, true, &f);
  if (rc) return rc;
  f->grid = grid_dim; f->block = block_dim; f->smem = shared_mem;
  f->raw = true;
  *out = f;
  return UGB_OK;
}

int32_t ugb_func_free(ugb_func *f) {
  if (!f) return UGB_ERR_INVALID;
  if (f->module && driver().module_unload) {
    cudaSetDevice(f->dev->ordinal);
    cudaStreamSynchronize(f->dev->stream);
    driver().module_unload(f->module);
  }
  delete f;
  return UGB_OK;
}

const char *ugb_func_source(const ugb_func *f) { return f ? f->source.c_str() : nullptr; }

static int32_t run_impl(ugb_device *dev, ugb_func *f, ugb_slice *const *args, size_t n_args, unsigned grid,
                        const long long *dyn, size_t n_dyn) {
  UGB_REQUIRE(dev, f != nullptr && f->dev == dev, UGB_ERR_INVALID, "ugb_run: function belongs to another device");
  UGB_REQUIRE(dev, (size_t)f->n_dyn == n_dyn, UGB_ERR_INVALID, "kernel %s takes %d run-time values, %zu given", f->name.c_str(), f->n_dyn, n_dyn);
  // a zero launch dimension is a no-op (ug-cuda/src/runtime.rs:269-277)
  if (grid == 0 || f->block == 0) return UGB_OK;
  std::vector<long long> dv(dyn, dyn + n_dyn);
  if (f->raw) {
    // user-supplied kernel: its parameters are the slices' device pointers in order, nothing else.  Bounds
    // are the kernel author's business, as with Func::launch in the reference (ug-pyo3/src/lib.rs:27-50).
    std::vector<void *> p(n_args), pp;
    for (size_t i = 0; i < n_args; ++i) {
      UGB_REQUIRE(dev, args[i] != nullptr && args[i]->dev == dev, UGB_ERR_INVALID, "ugb_run: argument %zu is null or on another device", i);
      p[i] = args[i]->ptr;
    }
    for (size_t i = 0; i < n_args; ++i) pp.push_back(&p[i]);
    for (size_t i = 0; i < n_dyn; ++i) pp.push_back(&dv[i]);
    UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
    CUresult rr = driver().launch_kernel(f->fn, grid, 1, 1, f->block, 1, 1, f->smem, (CUstream)dev->stream, pp.data(), nullptr);
    if (rr != CUDA_SUCCESS) return ugb_fail(dev, UGB_ERR_CUDA, "launch of %s failed with CUresult %d", f->name.c_str(), (int)rr);
    dev->launches++;
    return UGB_OK;
  }
  UGB_REQUIRE(dev, n_args == f->arg_dtypes.size(), UGB_ERR_INVALID, "unsupported number of args for kernel %zu, it takes %zu",
              n_args, f->arg_dtypes.size());
  std::vector<void *> ptrs(n_args);
  std::vector<unsigned long long> lens(n_args);
  std::vector<void *> params;
  for (size_t i = 0; i < n_args; ++i) {
    const ugb_slice *s = args[i];
    UGB_REQUIRE(dev, s != nullptr && s->dev == dev, UGB_ERR_INVALID, "ugb_run: argument %zu is null or on another device", i);
    UGB_REQUIRE(dev, s->dtype == f->arg_dtypes[i], UGB_ERR_DTYPE, "dtype mismatch for kernel argument %zu, expected %s, got %s", i,
                ugb_dtype_name(f->arg_dtypes[i]), ugb_dtype_name(s->dtype));
    ptrs[i] = s->ptr;
    lens[i] = s->len;
  }
  for (size_t i = 0; i < n_args; ++i) params.push_back(&ptrs[i]);
  for (size_t i = 0; i < n_args; ++i) params.push_back(&lens[i]);
  void *status = dev->status_dev;
  params.push_back(&status);
  for (size_t i = 0; i < n_dyn; ++i) params.push_back(&dv[i]);
  UGB_CUDA(dev, cudaSetDevice(dev->ordinal));
  CUresult r = driver().launch_kernel(f->fn, grid, 1, 1, f->block, 1, 1, f->smem, (CUstream)dev->stream, params.data(), nullptr);
  if (r != CUDA_SUCCESS) return ugb_fail(dev, UGB_ERR_CUDA, "launch of %s failed with CUresult %d", f->name.c_str(), (int)r);
  dev->launches++;
  return UGB_OK;
}

int32_t ugb_run(ugb_device *dev, ugb_func *f, ugb_slice *const *args, size_t n_args) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, f != nullptr, UGB_ERR_INVALID, "ugb_run: null function");
  return run_impl(dev, f, args, n_args, f->grid, nullptr, 0);
}

int32_t ugb_run_dyn(ugb_device *dev, ugb_func *f, ugb_slice *const *args, size_t n_args, uint32_t grid_dim,
                    const int64_t *dyn, size_t n_dyn) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, f != nullptr && (dyn != nullptr || n_dyn == 0) && n_dyn <= 8, UGB_ERR_INVALID, "ugb_run_dyn: bad argument");
  long long v[8];
  for (size_t i = 0; i < n_dyn; ++i) v[i] = (long long)dyn[i];
  return run_impl(dev, f, args, n_args, grid_dim, v, n_dyn);
}

int32_t ugb_ssa_source(ugb_device *dev, const ugb_ssa_instr *instrs, size_t n_instrs, const char *entry_name, char *buf,
                       size_t buf_len, int32_t *arg_dtypes, size_t max_args, size_t *n_args) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, entry_name && buf && arg_dtypes && n_args && (instrs || n_instrs == 0), UGB_ERR_INVALID, "ugb_ssa_source: null argument");
  std::string src;
  std::vector<int32_t> dts;
  int32_t rc = generate(dev, instrs, n_instrs, entry_name, &src, &dts);
  if (rc) return rc;
  UGB_REQUIRE(dev, src.size() + 1 <= buf_len && dts.size() <= max_args, UGB_ERR_SHAPE, "ugb_ssa_source: %zu bytes and %zu arguments needed",
              src.size() + 1, dts.size());
  memcpy(buf, src.c_str(), src.size() + 1);
  for (size_t i = 0; i < dts.size(); ++i) arg_dtypes[i] = dts[i];
  *n_args = dts.size();
  return UGB_OK;
}

int32_t ugb_compile_generated(ugb_device *dev, const char *cu_code, const char *entry_name, const int32_t *arg_dtypes,
                              size_t n_args, int32_t n_dyn, uint32_t grid_dim, uint32_t block_dim, uint32_t shared_mem,
                              ugb_func **out) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, cu_code && entry_name && out && (arg_dtypes || n_args == 0) && n_dyn >= 0 && n_dyn <= 8, UGB_ERR_INVALID,
              "ugb_compile_generated: bad argument");
  *out = nullptr;
  UGB_REQUIRE(dev, block_dim <= 1024, UGB_ERR_INVALID, "ugb_compile_generated: block_dim %u exceeds 1024", block_dim);
  ugb_func *f = nullptr;
  const int32_t rc = compile_and_load(dev, cu_code, entry_name, entry_name, false, false, &f);
  if (rc) return rc;
  f->grid = grid_dim; f->block = block_dim; f->smem = shared_mem;
  f->arg_dtypes.assign(arg_dtypes, arg_dtypes + n_args);
  f->n_dyn = n_dyn;
  *out = f;
  return UGB_OK;
}

}  // extern "C"
