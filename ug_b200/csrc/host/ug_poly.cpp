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
//   * the first sighting is compiled as it is and remembered (tokens + launch grid).  On the second one every
//     literal that differs becomes  b + a * t  with t = 0 for the first text and t = 1 for the second, t being
//     a `long long` value parameter of the kernel, and that text is compiled once;
//   * any later kernel is generated as text again (cheap: no compiler involved), and if every token matches
//     the template for one common integer t -- constants exactly, literals as b + a * t, the grid likewise --
//     the generic function runs with that t.  By construction it then executes exactly the statements the
//     specialised text would have; anything that does not fit (a size that enters non-affinely, a literal
//     inside a float constant) simply fails to match or to compile and is compiled per shape as before.
#include <cctype>

#include "ug_graph.hpp"

namespace ug {

std::vector<PolyToken> poly_tokenize(const std::string &s) {
  std::vector<PolyToken> out;
  size_t i = 0;
  const size_t n = s.size();
  while (i < n) {
    PolyToken t;
    const size_t w0 = i;
    while (i < n && isspace((unsigned char)s[i])) ++i;
    t.ws = s.substr(w0, i - w0);
    if (i >= n) { if (!t.ws.empty()) out.push_back(t); break; }
    const size_t b = i;
    const unsigned char c = (unsigned char)s[i];
    if (isalpha(c) || c == '_') {
      while (i < n && (isalnum((unsigned char)s[i]) || s[i] == '_')) ++i;
    } else if (isdigit(c)) {
      while (i < n) {
        const unsigned char d = (unsigned char)s[i];
        if (isalnum(d) || d == '_' || d == '.') { ++i; continue; }
        if ((d == '+' || d == '-') && (s[i - 1] == 'e' || s[i - 1] == 'E') && s.compare(b, 2, "0x") != 0) { ++i; continue; }
        break;
      }
      // a plain decimal integer with an optional u / l suffix?
      size_t j = b;
      while (j < i && isdigit((unsigned char)s[j])) ++j;
      bool suffix_ok = true;
      for (size_t q = j; q < i; ++q) suffix_ok = suffix_ok && (s[q] == 'u' || s[q] == 'U' || s[q] == 'l' || s[q] == 'L');
      if (suffix_ok && j - b <= 18) { t.is_int = true; t.value = std::stoll(s.substr(b, j - b)); }
    } else {
      ++i;
    }
    t.text = s.substr(b, i - b);
    out.push_back(std::move(t));
  }
  return out;
}

std::string poly_skeleton(const std::vector<PolyToken> &toks) {
  std::string k;
  for (const PolyToken &t : toks) {
    if (t.is_int) k += '#';
    else k += t.text;
    k += ' ';
  }
  return k;
}

// Template from two sightings (t = 0: `first`, t = 1: `second`); false when they are not the same text modulo integers.
bool poly_generalize(const PolyEntry &pe, const std::vector<PolyToken> &second, uint32_t second_grid, PolyGeneric &e,
                     std::string &generic_text) {
  const std::vector<PolyToken> &first = pe.pending;
  if (first.size() != second.size()) return false;
  e = PolyGeneric{};
  generic_text.clear();
  for (size_t i = 0; i < first.size(); ++i) {
    const PolyToken &p = first[i], &c = second[i];
    generic_text += p.ws;
    if (p.is_int != c.is_int) return false;
    if (p.is_int && p.value != c.value) {
      e.slots.push_back(PolySlot{i, c.value - p.value, p.value});
      generic_text += "(" + std::to_string(p.value) + "LL + " + std::to_string(c.value - p.value) + "LL * ugp_t)";
    } else {
      if (p.text != c.text) return false;
      generic_text += p.text;
    }
  }
  e.grid_b = (long long)pe.pending_grid;
  e.grid_a = (long long)second_grid - (long long)pe.pending_grid;
  e.tmpl = first;
  return true;
}

// Does `toks` instantiate the template for one integer t?
bool poly_match(const PolyGeneric &e, const std::vector<PolyToken> &toks, uint32_t grid, long long &t_out) {
  if (toks.size() != e.tmpl.size()) return false;
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
  if (!solve((long long)grid, e.grid_a, e.grid_b)) return false;
  size_t s = 0;
  for (size_t i = 0; i < toks.size(); ++i) {
    if (s < e.slots.size() && e.slots[s].token == i) {
      if (!toks[i].is_int || !solve(toks[i].value, e.slots[s].a, e.slots[s].b)) return false;
      ++s;
    } else if (toks[i].text != e.tmpl[i].text) {
      return false;
    }
  }
  t_out = t;
  return true;
}

}  // namespace ug
