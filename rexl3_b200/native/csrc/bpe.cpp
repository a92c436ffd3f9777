// Byte-level BPE merge core: the hot loop of the tokenizer (role of the reference server's C tokenizer fast path,
// crates/server/csrc/toks).  Pre-tokenization (the regex split) stays with the caller; this takes the pieces as byte ranges and
// applies the ranked merges on token ids: a piece starts as one token per byte, and the adjacent pair with the lowest merge rank
// (leftmost on ties) is replaced by its merged token until no pair has a rank.
#include <cstdint>
#include <unordered_map>
#include <vector>

namespace {

struct Bpe {
  int32_t byte_id[256];
  std::unordered_map<uint64_t, uint64_t> pairs;    // (left << 32 | right) -> (rank << 32 | merged)
};

inline uint64_t key(int32_t a, int32_t b) { return ((uint64_t)(uint32_t)a << 32) | (uint32_t)b; }

}  // namespace

extern "C" {

// byte_ids: int32 [256], the token of each byte (-1: none).  merges: int32 [n][3] = (left id, right id, merged id) in rank order.
void* rx_bpe_new(const int32_t* byte_ids, const int32_t* merges, int n) {
  Bpe* b = new Bpe();
  for (int i = 0; i < 256; ++i) b->byte_id[i] = byte_ids[i];
  b->pairs.reserve((size_t)n * 2);
  for (int r = 0; r < n; ++r) {
    const int32_t l = merges[3 * r], rt = merges[3 * r + 1], m = merges[3 * r + 2];
    if (l < 0 || rt < 0 || m < 0) continue;
    b->pairs.emplace(key(l, rt), ((uint64_t)(uint32_t)r << 32) | (uint32_t)m);   // the first (lowest) rank of a pair wins
  }
  return b;
}

void rx_bpe_free(void* h) { delete static_cast<Bpe*>(h); }

// bytes: the concatenated pieces; offsets: int64 [n_pieces + 1].  Writes at most `cap` ids to out; returns the number of ids the text
// encodes to (if that exceeds cap the caller retries with a larger buffer), or -1 on bad arguments.
int64_t rx_bpe_encode(void* h, const uint8_t* bytes, const int64_t* offsets, int n_pieces, int32_t* out, int64_t cap) {
  if (h == nullptr || n_pieces < 0) return -1;
  const Bpe& b = *static_cast<Bpe*>(h);
  std::vector<int32_t> sym;
  int64_t count = 0;
  for (int p = 0; p < n_pieces; ++p) {
    sym.clear();
    for (int64_t i = offsets[p]; i < offsets[p + 1]; ++i) sym.push_back(b.byte_id[bytes[i]]);
    while (sym.size() > 1) {
      uint32_t best = UINT32_MAX;
      size_t bi = 0;
      int32_t merged = -1;
      for (size_t i = 0; i + 1 < sym.size(); ++i) {
        if (sym[i] < 0 || sym[i + 1] < 0) continue;
        auto it = b.pairs.find(key(sym[i], sym[i + 1]));
        if (it == b.pairs.end()) continue;
        const uint32_t rank = (uint32_t)(it->second >> 32);
        if (rank < best) best = rank, bi = i, merged = (int32_t)(uint32_t)it->second;
      }
      if (merged < 0) break;
      sym[bi] = merged;
      sym.erase(sym.begin() + (long)bi + 1);
    }
    for (int32_t s : sym) {
      if (s < 0) continue;                       // a byte the vocabulary has no token for
      if (count < cap) out[count] = s;
      ++count;
    }
  }
  return count;
}

}  // extern "C"
