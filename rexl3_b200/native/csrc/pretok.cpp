// Pre-tokenizer of byte-level BPE vocabularies in C++: the split that the tokenizer files express as a regular expression, as a hand-written
// scanner over UTF-8 (role of the reference server's C tokenizer, crates/server/csrc/toks: the whole encode path without the interpreter).
//
// Three patterns cover the families served here; alternatives are tried in order at every position, exactly as the regex engine does
// (first alternative that matches wins, greedy inside with the backtracking the pattern implies):
//   kind 0  GPT-2          's|'t|'re|'ve|'m|'ll|'d | ?\p{L}+ | ?\p{N}+ | ?[^\s\p{L}\p{N}]+ |\s+(?!\S)|\s+
//   kind 1  cl100k / Llama-3   (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
//   kind 2  Qwen2 / Qwen3      as kind 1 with \p{N} (one digit per piece)
// The Unicode classes come from generated range tables (unicode_tables.inc) so that they agree with the Python oracle code point by code point.
#include <cstdint>
#include <cstring>
#include <vector>

#include "unicode_tables.inc"

namespace {

inline bool in_ranges(const uint32_t (*t)[2], int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) >> 1;
    if (cp < t[mid][0]) hi = mid - 1;
    else if (cp > t[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}

struct Cp {
  uint32_t cp;
  uint32_t off;     // byte offset of the code point
  uint8_t cls;      // bit 0 letter, bit 1 number, bit 2 whitespace
};
enum : uint8_t { C_L = 1, C_N = 2, C_S = 4 };

inline uint8_t classify(uint32_t cp) {
  if (cp < 128) {
    if ((cp >= 'a' && cp <= 'z') || (cp >= 'A' && cp <= 'Z')) return C_L;
    if (cp >= '0' && cp <= '9') return C_N;
    if (cp == ' ' || (cp >= 9 && cp <= 13)) return C_S;
    return 0;
  }
  uint8_t c = 0;
  if (in_ranges(RX_UNI_L, RX_UNI_L_N, cp)) c |= C_L;
  else if (in_ranges(RX_UNI_N, RX_UNI_N_N, cp)) c |= C_N;
  else if (in_ranges(RX_UNI_S, RX_UNI_S_N, cp)) c |= C_S;
  return c;
}

// UTF-8 -> code points (the input comes from str.encode(): well formed; a stray byte is taken as one code point of its own value)
void decode(const uint8_t* s, int64_t n, std::vector<Cp>& out) {
  out.clear();
  out.reserve((size_t)n + 1);
  int64_t i = 0;
  while (i < n) {
    const uint8_t b = s[i];
    uint32_t cp = b;
    int len = 1;
    if (b >= 0xF0 && i + 3 < n) { cp = ((b & 7u) << 18) | ((s[i + 1] & 63u) << 12) | ((s[i + 2] & 63u) << 6) | (s[i + 3] & 63u); len = 4; }
    else if (b >= 0xE0 && i + 2 < n) { cp = ((b & 15u) << 12) | ((s[i + 1] & 63u) << 6) | (s[i + 2] & 63u); len = 3; }
    else if (b >= 0xC0 && i + 1 < n) { cp = ((b & 31u) << 6) | (s[i + 1] & 63u); len = 2; }
    out.push_back(Cp{cp, (uint32_t)i, classify(cp)});
    i += len;
  }
  out.push_back(Cp{0, (uint32_t)n, 0});     // sentinel: end of text (class 0, never matched by a run)
}

inline bool is_crlf(uint32_t cp) { return cp == '\r' || cp == '\n'; }

// length (in code points) of a contraction at i, 0 if none.  ci: case-insensitive (the long s folds to s, as in the regex engine).
inline int contraction(const std::vector<Cp>& v, size_t i, size_t n, bool ci) {
  if (v[i].cp != '\'' || i + 1 >= n) return 0;
  auto low = [&](uint32_t c) -> uint32_t {
    if (!ci) return c;
    if (c >= 'A' && c <= 'Z') return c + 32;
    if (c == 0x17F) return 's';
    if (c == 0x212A) return 'k';
    return c;
  };
  const uint32_t a = low(v[i + 1].cp), b = i + 2 < n ? low(v[i + 2].cp) : 0;
  // order of the alternation: 's 't 're 've 'm 'll 'd
  if (a == 's' || a == 't') return 2;
  if (a == 'r' && b == 'e') return 3;
  if (a == 'v' && b == 'e') return 3;
  if (a == 'm') return 2;
  if (a == 'l' && b == 'l') return 3;
  if (a == 'd') return 2;
  return 0;
}

// Splits v[0 .. n) (n code points; v[n] is the sentinel) into pieces; appends the START offset of every piece to `cuts`.
void split(const std::vector<Cp>& v, int kind, std::vector<int64_t>& cuts) {
  const size_t n = v.size() - 1;
  size_t i = 0;
  auto run = [&](size_t from, uint8_t mask) { size_t j = from; while (j < n && (v[j].cls & mask)) ++j; return j; };
  auto run_other = [&](size_t from) { size_t j = from; while (j < n && v[j].cls == 0) ++j; return j; };      // not space, letter or number
  while (i < n) {
    cuts.push_back(v[i].off);
    size_t end = 0;
    const int cl = contraction(v, i, n, kind != 0);
    if (cl) { i += cl; continue; }
    if (kind == 0) {
      const size_t s = (v[i].cp == ' ' && i + 1 < n) ? i + 1 : i;          // the optional leading space
      if (s < n && (v[s].cls & C_L)) end = run(s, C_L);
      else if (s < n && (v[s].cls & C_N)) end = run(s, C_N);
      else if (s < n && v[s].cls == 0) end = run_other(s);
      if (end == 0 && s != i) {                                              // the space could not lead anything: try without it
        if (v[i].cls & C_L) end = run(i, C_L);                               // (a space is none of these: falls to the whitespace rules)
      }
    } else {
      // [^\r\n\p{L}\p{N}]?\p{L}+
      if (v[i].cls & C_L) end = run(i, C_L);
      else if (!is_crlf(v[i].cp) && !(v[i].cls & C_N) && i + 1 < n && (v[i + 1].cls & C_L)) end = run(i + 1, C_L);
      // \p{N}{1,3} (kind 1) / \p{N} (kind 2)
      if (end == 0 && (v[i].cls & C_N)) {
        end = i + 1;
        if (kind == 1) while (end < n && end < i + 3 && (v[end].cls & C_N)) ++end;
      }
      //  ?[^\s\p{L}\p{N}]+[\r\n]*
      if (end == 0) {
        const size_t s = (v[i].cp == ' ' && i + 1 < n && v[i + 1].cls == 0) ? i + 1 : i;
        if (v[s].cls == 0 && s < n) {
          end = run_other(s);
          while (end < n && is_crlf(v[end].cp)) ++end;
        }
      }
      // \s*[\r\n]+ : the whitespace run up to and including its last line break
      if (end == 0 && (v[i].cls & C_S)) {
        const size_t e = run(i, C_S);
        size_t last = 0;
        bool found = false;
        for (size_t j = i; j < e; ++j)
          if (is_crlf(v[j].cp)) { last = j; found = true; }
        if (found) end = last + 1;
      }
    }
    if (end == 0 && (v[i].cls & C_S)) {
      // \s+(?!\S) : the run if the text ends after it, else the run without its last character (if anything is left); then \s+
      const size_t e = run(i, C_S);
      if (e == n) end = e;
      else if (e - i >= 2) end = e - 1;
      else end = e;
    }
    if (end == 0) end = i + 1;          // cannot happen for these patterns (every character is in some class); never loop forever
    i = end;
  }
}

}  // namespace

extern "C" {

// Piece boundaries of `text` (UTF-8, n bytes) under pattern `kind`: writes the start offset of every piece and, last, n into `offsets`
// (at most cap values); returns how many values the split has (pieces + 1), or -1 on bad arguments.
int64_t rx_pretok_split(int kind, const uint8_t* text, int64_t n, int64_t* offsets, int64_t cap) {
  if (kind < 0 || kind > 2 || n < 0 || (n > 0 && text == nullptr)) return -1;
  std::vector<Cp> v;
  decode(text, n, v);
  std::vector<int64_t> cuts;
  cuts.reserve(v.size() / 3 + 4);
  split(v, kind, cuts);
  cuts.push_back(n);
  for (size_t i = 0; i < cuts.size() && (int64_t)i < cap; ++i) offsets[i] = cuts[i];
  return (int64_t)cuts.size();
}

int64_t rx_bpe_encode(void* h, const uint8_t* bytes, const int64_t* offsets, int n_pieces, int32_t* out, int64_t cap);      // bpe.cpp

// Split + merge in one call: token ids of `text` under pattern `kind` with the merges of BPE handle `h`.  Returns the id count (retry with a
// larger `cap` if it exceeds it), -1 on bad arguments.
int64_t rx_bpe_encode_text(void* h, int kind, const uint8_t* text, int64_t n, int32_t* out, int64_t cap) {
  if (h == nullptr || kind < 0 || kind > 2 || n < 0) return -1;
  if (n == 0) return 0;
  std::vector<Cp> v;
  decode(text, n, v);
  std::vector<int64_t> cuts;
  split(v, kind, cuts);
  cuts.push_back(n);
  if (cuts.size() - 1 > (size_t)INT32_MAX) return -1;
  return rx_bpe_encode(h, text, cuts.data(), (int)(cuts.size() - 1), out, cap);
}

}  // extern "C"
