// Shape-polymorphic kernel reuse.
//
// ug-core keys its compilation cache on the kernel INCLUDING every shape, stride and offset
// (ug-core/src/cache.rs:8-12, lang.rs:415-420), so in a decode loop every fused kernel whose shape follows
// the KV length (the GQA repeat copies, the scale / softmax rows of ug-llama/src/model.rs:80-101,231-241) is a
// cache miss and a run-time compilation per token (main.rs:140-149 times it as `comp`).  Here a second
// sighting of "the same kernel at another size" produces ONE kernel that takes the size at run time:
//
//   * the unit of comparison is the CUDA C the backend generates from the kernel's SSA.  Two texts whose
//     tokens are equal except for decimal integer literals are the same kernel at two sizes;
//   * the first sighting is compiled as it is and its literals are remembered.  On the second one every
//     literal that differs becomes  b + a * t  with t = 0 for the first text and t = 1 for the second, t being
//     a `long long` value parameter of the kernel, and that text is compiled once;
//   * any later kernel is generated as text again (cheap: no compiler involved; one pass over the text splits it
//     into the skeleton, which is the cache key, and the list of literals), and if every literal matches the
//     template for one common integer t -- constants exactly, the others as b + a * t -- the generic function
//     runs with that t and with the grid of the kernel it replaces.  By construction it then executes exactly
//     the statements the specialised text would have; anything that does not fit (a size that enters
//     non-affinely, a literal inside a float constant) simply fails to match or to compile and is compiled per
//     shape as before.
#include "ug_graph.hpp"

namespace ug {

namespace {
inline bool is_digit(unsigned char c) { return c >= '0' && c <= '9'; }
inline bool is_word(unsigned char c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || c == '_' || is_digit(c); }
}  // namespace

// One pass: identifiers and punctuation go to the skeleton as they are; a token that starts with a digit is a
// number (digits, letters, '.', and a sign after an exponent letter unless it is hexadecimal), and when it is a
// plain decimal integer with an optional u / l suffix its digits become POLY_MARK and its value joins `ints`.
PolyText poly_scan(const std::string &s) {
  PolyText out;
  const size_t n = s.size();
  out.skeleton.reserve(n + 24);
  out.ints.reserve(64);
  size_t i = 0;
  while (i < n) {
    const unsigned char c = (unsigned char)s[i];
    if (is_digit(c)) {
      const size_t b = i;
      const bool hex = c == '0' && i + 1 < n && (s[i + 1] == 'x' || s[i + 1] == 'X');
      while (i < n) {
        const unsigned char d = (unsigned char)s[i];
        if (is_word(d) || d == '.') { ++i; continue; }
        if ((d == '+' || d == '-') && (s[i - 1] == 'e' || s[i - 1] == 'E') && !hex) { ++i; continue; }
        break;
      }
      size_t j = b;
      long long v = 0;
      while (j < i && is_digit((unsigned char)s[j]) && j - b < 19) { v = v * 10 + (s[j] - '0'); ++j; }
      bool plain = j - b <= 18;
      for (size_t q = j; q < i && plain; ++q) plain = s[q] == 'u' || s[q] == 'U' || s[q] == 'l' || s[q] == 'L';
      if (plain) {
        out.ints.push_back(v);
        out.skeleton.push_back(POLY_MARK);
        out.skeleton.append(s, j, i - j);
      } else {
        out.skeleton.append(s, b, i - b);
      }
    } else if (is_word(c)) {
      const size_t b = i;
      while (i < n && is_word((unsigned char)s[i])) ++i;
      out.skeleton.append(s, b, i - b);
    } else {
      out.skeleton.push_back((char)c);
      ++i;
    }
  }
  out.text_len = out.skeleton.size();
  return out;
}

// Template from two sightings of one skeleton (t = 0: the pending literals, t = 1: `second`).
bool poly_generalize(const PolyEntry &pe, const PolyText &second, PolyGeneric &e, std::string &generic_text) {
  const std::vector<long long> &first = pe.pending;
  if (first.size() != second.ints.size()) return false;
  e = PolyGeneric{};
  e.b = first;
  e.a.resize(first.size());
  generic_text.clear();
  generic_text.reserve(second.text_len + 32 * first.size());
  size_t k = 0;
  for (size_t i = 0; i < second.text_len; ++i) {
    const char c = second.skeleton[i];
    if (c != POLY_MARK) { generic_text.push_back(c); continue; }
    if (k >= first.size()) return false;
    const long long a = second.ints[k] - first[k];
    e.a[k] = a;
    if (a == 0) {
      generic_text += std::to_string(first[k]);
    } else {
      // a moving literal loses its suffix: the expression is a long long whatever the literal was
      generic_text += "(" + std::to_string(first[k]) + "LL + " + std::to_string(a) + "LL * ugp_t)";
      while (i + 1 < second.text_len && (second.skeleton[i + 1] == 'u' || second.skeleton[i + 1] == 'U' ||
                                         second.skeleton[i + 1] == 'l' || second.skeleton[i + 1] == 'L')) ++i;
    }
    ++k;
  }
  if (k != first.size()) return false;
  return true;
}

// Do `ints` (literals of a text with the template's skeleton) instantiate the template for one integer t?
// The grid is not part of the template: every launch of a generic function uses the grid of the kernel it stands
// in for (ceil(elements / block) for a one-dimensional map, which is not affine in the size).
bool poly_match(const PolyGeneric &e, const std::vector<long long> &ints, long long &t_out) {
  if (ints.size() != e.b.size()) return false;
  bool have_t = false;
  long long t = 0;
  auto solve = [&](long long q, long long a, long long b) {
    if (a == 0) return q == b;
    if ((q - b) % a != 0) return false;
    const long long tt = (q - b) / a;
    if (have_t) return tt == t;
    have_t = true;
    t = tt;
    return true;
  };
  for (size_t i = 0; i < ints.size(); ++i)
    if (!solve(ints[i], e.a[i], e.b[i])) return false;
  t_out = t;
  return true;
}

}  // namespace ug
