// ug::safetensors::MmapedSafetensors (ug-core/src/safetensors.rs:10-318) behind the C ABI: memory-mapped
// .safetensors files, tensors looked up by name and copied into device slices, optionally cast on the host.
//
// The container format is that of the `safetensors` crate the reference depends on (0.4.5, Cargo.toml:43;
// the crate is not part of the reference tree): an 8-byte little-endian header length N, N bytes of JSON
//   { "<name>": {"dtype": "F32", "shape": [..], "data_offsets": [begin, end]}, ..., "__metadata__": {..} }
// and the tensor bytes; offsets are relative to the end of the header.  As the crate does, the reader
// rejects headers above 100 MB, tensors whose byte length is not shape-product x element size, and
// offset tables that are not a gap-free cover of the data section.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cmath>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ugb_internal.h"

namespace {

struct StFile {
  int fd = -1;
  void *map = nullptr;
  size_t size = 0;
  const uint8_t *data = nullptr;   // first byte after the header
  size_t data_len = 0;
};

struct StTensor {
  std::string name, dtype_name;
  int dtype = -1;                  // ugb_dtype, or -1: a safetensors dtype ug has no DType for
  std::vector<size_t> shape;
  size_t begin = 0, end = 0;
  int file = 0;
};

// ---- a JSON reader for exactly the header's shape --------------------------------------------
struct Json {
  const char *p, *e;
  std::string err;
  bool fail(const char *m) { if (err.empty()) err = m; return false; }
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool lit(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  bool string(std::string &out) {
    ws();
    if (p >= e || *p != '"') return fail("expected a string");
    ++p;
    out.clear();
    while (p < e && *p != '"') {
      if (*p == '\\') {
        if (++p >= e) return fail("unterminated escape");
        switch (*p) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {
            if (e - p < 5) return fail("short \\u escape");
            unsigned v = 0;
            for (int i = 1; i <= 4; ++i) {
              const char c = p[i];
              v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : (c | 32) >= 'a' && (c | 32) <= 'f' ? (c | 32) - 'a' + 10 : 99);
            }
            if (v < 0x80) out += (char)v;
            else if (v < 0x800) { out += (char)(0xC0 | (v >> 6)); out += (char)(0x80 | (v & 63)); }
            else { out += (char)(0xE0 | (v >> 12)); out += (char)(0x80 | ((v >> 6) & 63)); out += (char)(0x80 | (v & 63)); }
            p += 4;
            break;
          }
          default: out += *p;      // \" \\ \/
        }
        ++p;
      } else {
        out += *p++;
      }
    }
    if (p >= e) return fail("unterminated string");
    ++p;
    return true;
  }
  bool number(size_t &out) {
    ws();
    if (p >= e || *p < '0' || *p > '9') return fail("expected a non-negative integer");
    out = 0;
    while (p < e && *p >= '0' && *p <= '9') {
      if (out > (SIZE_MAX - 9) / 10) return fail("integer overflow");
      out = out * 10 + (size_t)(*p++ - '0');
    }
    return true;
  }
  bool numbers(std::vector<size_t> &out) {
    out.clear();
    if (!lit('[')) return fail("expected an array");
    if (lit(']')) return true;
    do { size_t v; if (!number(v)) return false; out.push_back(v); } while (lit(','));
    return lit(']') || fail("unterminated array");
  }
  bool skip_value() {              // __metadata__: an object of strings
    ws();
    if (p < e && *p == '"') { std::string s; return string(s); }
    if (lit('{')) {
      if (lit('}')) return true;
      do { std::string k; if (!string(k) || !lit(':') || !skip_value()) return fail("bad metadata object"); } while (lit(','));
      return lit('}') || fail("unterminated object");
    }
    return fail("unexpected value in __metadata__");
  }
};

int dtype_of(const std::string &s, size_t *bytes) {
  struct { const char *n; int d; size_t b; } t[] = {
      {"BF16", UGB_BF16, 2}, {"F16", UGB_F16, 2}, {"F32", UGB_F32, 4}, {"I32", UGB_I32, 4}, {"I64", UGB_I64, 8},
      {"F64", -1, 8}, {"U64", -1, 8}, {"U32", -1, 4}, {"I16", -1, 2}, {"U16", -1, 2}, {"I8", -1, 1}, {"U8", -1, 1},
      {"BOOL", -1, 1}, {"F8_E4M3", -1, 1}, {"F8_E5M2", -1, 1}};
  for (auto &e : t)
    if (s == e.n) { *bytes = e.b; return e.d; }
  *bytes = 0;
  return -2;
}

}  // namespace

struct ugb_safetensors {
  std::vector<StFile> files;
  std::vector<StTensor> tensors;
  std::unordered_map<std::string, size_t> index;   // a name in several files: the last file wins (safetensors.rs:40)
  ~ugb_safetensors() {
    for (auto &f : files) {
      if (f.map && f.map != MAP_FAILED) munmap(f.map, f.size);
      if (f.fd >= 0) close(f.fd);
    }
  }
};

namespace {

int32_t open_one(ugb_device *dev, ugb_safetensors *st, const char *path) {
  StFile f;
  f.fd = open(path, O_RDONLY);
  UGB_REQUIRE(dev, f.fd >= 0, UGB_ERR_INVALID, "%s: cannot open (%s)", path, strerror(errno));
  struct stat sb;
  if (fstat(f.fd, &sb) != 0 || sb.st_size < 8) {
    close(f.fd);
    return ugb_fail(dev, UGB_ERR_INVALID, "%s: header too small", path);
  }
  f.size = (size_t)sb.st_size;
  f.map = mmap(nullptr, f.size, PROT_READ, MAP_PRIVATE, f.fd, 0);
  if (f.map == MAP_FAILED) {
    close(f.fd);
    return ugb_fail(dev, UGB_ERR_INVALID, "%s: mmap failed (%s)", path, strerror(errno));
  }
  const int file_index = (int)st->files.size();
  st->files.push_back(f);          // owned from here on: the destructor unmaps
  const uint8_t *base = (const uint8_t *)f.map;
  uint64_t n = 0;
  for (int i = 7; i >= 0; --i) n = (n << 8) | base[i];
  UGB_REQUIRE(dev, n <= 100000000ull, UGB_ERR_INVALID, "%s: header too large (%llu bytes)", path, (unsigned long long)n);
  UGB_REQUIRE(dev, n <= f.size - 8, UGB_ERR_INVALID, "%s: invalid header length %llu for a file of %zu bytes", path,
              (unsigned long long)n, f.size);
  StFile &sf = st->files.back();
  sf.data = base + 8 + n;
  sf.data_len = f.size - 8 - (size_t)n;
  Json j{(const char *)base + 8, (const char *)base + 8 + n, {}};
  UGB_REQUIRE(dev, j.lit('{'), UGB_ERR_INVALID, "%s: invalid header start", path);
  std::vector<StTensor> found;
  if (!j.lit('}')) {
    do {
      StTensor t;
      t.file = file_index;
      if (!j.string(t.name)) break;
      if (!j.lit(':')) { j.fail("expected ':'"); break; }
      if (t.name == "__metadata__") { if (!j.skip_value()) break; continue; }
      if (!j.lit('{')) { j.fail("expected a tensor description"); break; }
      bool have_d = false, have_s = false, have_o = false;
      do {
        std::string k;
        if (!j.string(k)) break;
        if (!j.lit(':')) { j.fail("expected ':'"); break; }
        if (k == "dtype") { have_d = j.string(t.dtype_name); }
        else if (k == "shape") { have_s = j.numbers(t.shape); }
        else if (k == "data_offsets") {
          std::vector<size_t> o;
          have_o = j.numbers(o) && o.size() == 2;
          if (have_o) { t.begin = o[0]; t.end = o[1]; }
        } else { j.fail("unknown key in a tensor description"); }
      } while (j.err.empty() && j.lit(','));
      if (!j.err.empty() || !j.lit('}') || !have_d || !have_s || !have_o) { j.fail("incomplete tensor description"); break; }
      found.push_back(std::move(t));
    } while (j.lit(','));
    if (j.err.empty() && !j.lit('}')) j.fail("unterminated header object");
  }
  UGB_REQUIRE(dev, j.err.empty(), UGB_ERR_INVALID, "%s: invalid header: %s", path, j.err.c_str());
  // the crate's validation: byte length = shape product x element size, and a gap-free cover of the data
  std::sort(found.begin(), found.end(), [](const StTensor &a, const StTensor &b) { return a.begin < b.begin; });
  size_t cursor = 0;
  for (StTensor &t : found) {
    size_t es = 0;
    t.dtype = dtype_of(t.dtype_name, &es);
    UGB_REQUIRE(dev, t.dtype != -2, UGB_ERR_INVALID, "%s: unknown dtype %s for %s", path, t.dtype_name.c_str(), t.name.c_str());
    size_t n_el = 1;
    for (size_t d : t.shape) {
      UGB_REQUIRE(dev, d == 0 || n_el <= SIZE_MAX / d, UGB_ERR_INVALID, "%s: shape of %s overflows", path, t.name.c_str());
      n_el *= d;
    }
    UGB_REQUIRE(dev, t.begin == cursor && t.end >= t.begin, UGB_ERR_INVALID, "%s: invalid offset for tensor %s", path, t.name.c_str());
    UGB_REQUIRE(dev, t.end - t.begin == n_el * es, UGB_ERR_INVALID, "%s: tensor %s: %zu bytes for %zu elements of %s", path,
                t.name.c_str(), t.end - t.begin, n_el, t.dtype_name.c_str());
    cursor = t.end;
  }
  UGB_REQUIRE(dev, cursor == sf.data_len, UGB_ERR_INVALID, "%s: metadata covers %zu of %zu data bytes", path, cursor, sf.data_len);
  for (StTensor &t : found) {
    auto it = st->index.find(t.name);
    if (it != st->index.end()) { st->tensors[it->second] = std::move(t); }
    else { st->index[t.name] = st->tensors.size(); st->tensors.push_back(std::move(t)); }
  }
  return UGB_OK;
}

const StTensor *find(ugb_device *dev, const ugb_safetensors *st, const char *name) {
  auto it = st->index.find(name);
  if (it == st->index.end()) { ugb_fail(dev, UGB_ERR_INVALID, "cannot find tensor %s", name); return nullptr; }
  return &st->tensors[it->second];
}

// ---- host-side element conversions (what `half` and Rust's `as` do) -----------------------------
inline float load_as_f32(const uint8_t *p, int dtype, size_t i) {
  switch (dtype) {
    case UGB_BF16: { uint16_t b; memcpy(&b, p + 2 * i, 2); uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
    case UGB_F16: { __half h; memcpy(&h, p + 2 * i, 2); return __half2float(h); }
    case UGB_F32: { float f; memcpy(&f, p + 4 * i, 4); return f; }
    default: return 0.f;
  }
}
inline int32_t sat_i32(float v) {       // Rust `as i32`: saturating, NaN -> 0
  if (std::isnan(v)) return 0;
  if (v >= 2147483648.0f) return INT32_MAX;
  if (v <= -2147483648.0f) return INT32_MIN;
  return (int32_t)v;
}
inline int64_t sat_i64(float v) {
  if (std::isnan(v)) return 0;
  if (v >= 9223372036854775808.0f) return INT64_MAX;
  if (v <= -9223372036854775808.0f) return INT64_MIN;
  return (int64_t)v;
}
// f32 -> bf16 / f16 as crate half 2.3.1 does them in software (Cargo.toml:28): round to nearest even; a NaN
// keeps its sign and upper payload bits and gets the quiet bit (the GPU's own converters return 0x7FFF).
inline uint16_t bf16_from_f32(float v) {
  uint32_t x;
  memcpy(&x, &v, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);
  const uint32_t round_bit = 0x8000u;
  if ((x & round_bit) != 0 && (x & (3 * round_bit - 1)) != 0) return (uint16_t)((x >> 16) + 1);
  return (uint16_t)(x >> 16);
}
inline uint16_t f16_from_f32(float v) {
  uint32_t x;
  memcpy(&x, &v, 4);
  const uint32_t sign = (x >> 16) & 0x8000u, exp = x & 0x7F800000u, man = x & 0x007FFFFFu;
  if (exp == 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (man ? 0x0200u : 0u) | (man >> 13));
  const int half_exp = (int)(exp >> 23) - 127 + 15;
  if (half_exp >= 0x1F) return (uint16_t)(sign | 0x7C00u);
  if (half_exp <= 0) {
    if (14 - half_exp > 24) return (uint16_t)sign;
    const uint32_t m = man | 0x00800000u;
    uint32_t hm = m >> (14 - half_exp);
    const uint32_t round_bit = 1u << (13 - half_exp);
    if ((m & round_bit) != 0 && (m & (3 * round_bit - 1)) != 0) hm += 1;
    return (uint16_t)(sign | hm);
  }
  const uint32_t he = (uint32_t)half_exp << 10, hm = man >> 13, round_bit = 0x1000u;
  if ((man & round_bit) != 0 && (man & (3 * round_bit - 1)) != 0) return (uint16_t)((sign | he | hm) + 1);
  return (uint16_t)(sign | he | hm);
}
inline void store_from_f32(uint8_t *p, int dtype, size_t i, float v) {
  switch (dtype) {
    case UGB_BF16: { const uint16_t b = bf16_from_f32(v); memcpy(p + 2 * i, &b, 2); break; }
    case UGB_F16: { const uint16_t h = f16_from_f32(v); memcpy(p + 2 * i, &h, 2); break; }
    case UGB_F32: memcpy(p + 4 * i, &v, 4); break;
    default: break;
  }
}

}  // namespace

extern "C" {

int32_t ugb_st_open(ugb_device *dev, const char *const *paths, size_t n_paths, ugb_safetensors **out) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, paths && out && n_paths >= 1, UGB_ERR_INVALID, "ugb_st_open: null argument or no path");
  *out = nullptr;
  ugb_safetensors *st = new ugb_safetensors();
  for (size_t i = 0; i < n_paths; ++i) {
    const int32_t rc = paths[i] ? open_one(dev, st, paths[i]) : ugb_fail(dev, UGB_ERR_INVALID, "ugb_st_open: null path");
    if (rc) { delete st; return rc; }
  }
  *out = st;
  return UGB_OK;
}

int32_t ugb_st_close(ugb_safetensors *st) {
  if (!st) return UGB_ERR_INVALID;
  delete st;
  return UGB_OK;
}

size_t ugb_st_count(const ugb_safetensors *st) { return st ? st->tensors.size() : 0; }

const char *ugb_st_name(const ugb_safetensors *st, size_t i) {
  return st && i < st->tensors.size() ? st->tensors[i].name.c_str() : nullptr;
}

int32_t ugb_st_info(ugb_device *dev, const ugb_safetensors *st, const char *name, int32_t *dtype, int32_t *rank,
                    size_t *dims, size_t dims_cap) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, st && name, UGB_ERR_INVALID, "ugb_st_info: null argument");
  const StTensor *t = find(dev, st, name);
  if (!t) return UGB_ERR_INVALID;
  if (dtype) *dtype = t->dtype;
  if (rank) *rank = (int32_t)t->shape.size();
  if (dims)
    for (size_t i = 0; i < t->shape.size() && i < dims_cap; ++i) dims[i] = t->shape[i];
  return UGB_OK;
}

int32_t ugb_st_load_slice_with_cast(ugb_device *dev, const ugb_safetensors *st, const char *name, int32_t dst_dtype,
                                    ugb_slice **out) {
  if (!dev) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, st && name && out, UGB_ERR_INVALID, "ugb_st_load_slice: null argument");
  *out = nullptr;
  const StTensor *t = find(dev, st, name);
  if (!t) return UGB_ERR_INVALID;
  UGB_REQUIRE(dev, t->dtype >= 0, UGB_ERR_DTYPE, "unsupported dtype for %s: %s", name, t->dtype_name.c_str());   // safetensors.rs:92
  const int src = t->dtype, dst = dst_dtype < 0 ? src : dst_dtype;
  UGB_REQUIRE(dev, dst >= UGB_BF16 && dst <= UGB_I64, UGB_ERR_INVALID, "ugb_st_load_slice: unknown target dtype %d", dst);
  size_t n = 1;
  for (size_t d : t->shape) n *= d;
  const uint8_t *bytes = st->files[t->file].data + t->begin;
  // The reference builds a Vec<i32> for BF16 -> I64 and F16 -> I64 and hands it to an I64 slice
  // (safetensors.rs:163-166,188-191): the copy then fails its dtype check.  Same outcome here.
  UGB_REQUIRE(dev, !((src == UGB_BF16 || src == UGB_F16) && dst == UGB_I64), UGB_ERR_DTYPE,
              "dtype mismatch, slice: I64, host data: I32 (%s)", name);
  ugb_slice *s = nullptr;
  int32_t rc = ugb_alloc(dev, dst, n, &s);
  if (rc) return rc;
  if (src == dst) {
    rc = ugb_h2d(s, bytes, n, dst);        // the mapping is copied as it lies (alignment is the copy engine's business)
  } else {
    static const size_t es[] = {2, 2, 4, 4, 8};
    std::vector<uint8_t> tmp(n * es[dst]);
    const bool src_f = src <= UGB_F32, dst_f = dst <= UGB_F32;
    for (size_t i = 0; i < n; ++i) {
      if (src_f && dst_f) {
        store_from_f32(tmp.data(), dst, i, load_as_f32(bytes, src, i));
      } else if (src_f) {                  // float -> int: through f32, saturating
        const float v = load_as_f32(bytes, src, i);
        if (dst == UGB_I32) { const int32_t o = sat_i32(v); memcpy(tmp.data() + 4 * i, &o, 4); }
        else { const int64_t o = sat_i64(v); memcpy(tmp.data() + 8 * i, &o, 8); }
      } else {                             // int source
        int64_t v;
        if (src == UGB_I32) { int32_t a; memcpy(&a, bytes + 4 * i, 4); v = a; } else { memcpy(&v, bytes + 8 * i, 8); }
        if (dst_f) store_from_f32(tmp.data(), dst, i, (float)v);
        else if (dst == UGB_I32) { const int32_t o = (int32_t)v; memcpy(tmp.data() + 4 * i, &o, 4); }   // `as i32` wraps
        else { memcpy(tmp.data() + 8 * i, &v, 8); }
      }
    }
    rc = ugb_h2d(s, tmp.data(), n, dst);
  }
  if (rc) { ugb_free(s); return rc; }
  *out = s;
  return UGB_OK;
}

int32_t ugb_st_load_slice(ugb_device *dev, const ugb_safetensors *st, const char *name, ugb_slice **out) {
  return ugb_st_load_slice_with_cast(dev, st, name, -1, out);
}

}  // extern "C"
