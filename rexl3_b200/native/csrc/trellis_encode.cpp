// EXL3 trellis encoder (host): tail-biting Viterbi over the 65,536 sixteen-bit states of one 16x16 tile.
//
// A tile is a ring of 256*bits bits; value p is the 16-bit window ending at E(p), so consecutive states overlap:
// s_p = ((s_{p-1} << nb_p) & 0xFFFF) | fresh, nb_p = E(p) - E(p-1) fresh bits (2 or 3 alternating for 2.5 bpw, etc.).
// The best cost of reaching s_p depends only on its top 16 - nb_p bits (the bits it shares with s_{p-1}), so a step is
// "min over the 2^nb predecessors per shared prefix" (65,536 compares) plus one add per state, not 65,536 * 2^nb.
// Tail-biting: a first pass over the sequence rotated by half a tile finds the state at the seam; the second pass is
// constrained to start and end on that seam's overlap bits, so the emitted ring decodes back to exactly the chosen states.
// What it must produce is what the reference's encoder contract asks for (crates/quant/src/exl3_trellis.rs:6-24):
// a bit ring whose decoded values minimise the squared error to the tile; the search organisation here is new.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

struct Plan {
  int twice;
  int ends[256];
  int nb[256];   // fresh bits of value p
};

Plan make_plan(int twice) {
  Plan pl;
  pl.twice = twice;
  int prev = 0;
  for (int p = 0; p < 256; ++p) {
    const int p1 = p + 1;
    const int e = (twice % 2 == 0) ? p1 * (twice / 2) : (p1 * twice - (p1 & 1)) / 2;
    pl.ends[p] = e;
    pl.nb[p] = e - prev;
    prev = e;
  }
  return pl;
}

struct Scratch {
  std::vector<float> cost, next, best;
  std::vector<uint8_t> back;   // [256][65536 >> nbmin] argmin of the predecessor's top bits
  Scratch() : cost(65536), next(65536), best(65536), back((size_t)256 * 32768) {}
};

// One Viterbi pass over values w[order[i]], i = 0..255 (order = rotation).  If seam >= 0 the first state's shared prefix and
// the last state's low bits are forced to `seam` (the overlap of the ring's closing window).  Returns the states in `order`
// positions and the total cost.
float viterbi(const Plan& pl, const float* w, const float* table, int rot, int seam, Scratch& sc, uint16_t* states) {
  const float INF = std::numeric_limits<float>::infinity();
  float* cost = sc.cost.data();
  float* next = sc.next.data();
  {
    const int p = rot % 256;
    const int nb = pl.nb[p];
    const float x = w[p];
    for (int s = 0; s < 65536; ++s) {
      const float d = x - table[s];
      cost[s] = (seam >= 0 && (s >> nb) != seam) ? INF : d * d;
    }
  }
  for (int i = 1; i < 256; ++i) {
    const int p = (rot + i) % 256;
    const int nb = pl.nb[p];
    const int npre = 65536 >> nb;          // shared prefixes
    const int fan = 1 << nb;               // predecessors per prefix
    float* best = sc.best.data();
    uint8_t* bk = sc.back.data() + (size_t)i * 32768;
    for (int u = 0; u < npre; ++u) {
      float b = cost[u];
      int arg = 0;
      for (int t = 1; t < fan; ++t) {
        const float c = cost[(t << (16 - nb)) | u];
        if (c < b) { b = c; arg = t; }
      }
      best[u] = b;
      bk[u] = (uint8_t)arg;
    }
    const float x = w[p];
    for (int s = 0; s < 65536; ++s) {
      const float d = x - table[s];
      next[s] = best[s >> nb] + d * d;
    }
    std::swap(cost, next);
  }
  // final state
  int last = -1;
  float bestc = INF;
  const int p_first = rot % 256;
  const int mask = (1 << (16 - pl.nb[p_first])) - 1;
  for (int s = 0; s < 65536; ++s) {
    if (seam >= 0 && (s & mask) != seam) continue;
    if (cost[s] < bestc) { bestc = cost[s]; last = s; }
  }
  if (last < 0) return INF;
  int s = last;
  for (int i = 255; i >= 0; --i) {
    states[(rot + i) % 256] = (uint16_t)s;
    if (i == 0) break;
    const int p = (rot + i) % 256;
    const int nb = pl.nb[p];
    const int u = s >> nb;
    const int t = sc.back[(size_t)i * 32768 + u];
    s = (t << (16 - nb)) | u;
  }
  return bestc;
}

void pack(const Plan& pl, const uint16_t* states, int16_t* out) {
  const int nbits = 128 * pl.twice;
  std::vector<uint8_t> ring(nbits, 0);
  int start = 0;
  for (int p = 0; p < 256; ++p) {
    const int nb = pl.nb[p];
    for (int b = 0; b < nb; ++b) ring[start + b] = (states[p] >> (nb - 1 - b)) & 1;
    start += nb;
  }
  const int nw = nbits / 32;
  for (int i = 0; i < nw; ++i) {
    uint32_t v = 0;
    for (int b = 0; b < 32; ++b) v = (v << 1) | ring[i * 32 + b];
    out[2 * i] = (int16_t)(v & 0xFFFF);
    out[2 * i + 1] = (int16_t)(v >> 16);
  }
}

}  // namespace

extern "C" {

// tiles: float [T][256] in stream order (already divided by the layer scale); table: float [65536] codebook values.
// out: int16 [T][16*bits]; err: float [T] squared error of each tile (may be null).  Returns 0, or 1 on bad arguments.
int rx_trellis_encode(const float* tiles, int T, int twice, const float* table, int16_t* out, float* err, int threads) {
  static const int ok_twice[] = {2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16};
  if (std::find(std::begin(ok_twice), std::end(ok_twice), twice) == std::end(ok_twice) || T < 0) return 1;
  const Plan pl = make_plan(twice);
  const int words = 8 * twice;
  std::atomic<int> next_tile(0);
  int nthreads = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
  nthreads = std::max(1, std::min(nthreads, std::max(T, 1)));
  auto work = [&]() {
    Scratch sc;
    uint16_t st[256];
    for (;;) {
      const int t = next_tile.fetch_add(1);
      if (t >= T) break;
      const float* w = tiles + (size_t)t * 256;
      // pass 1: free ends, sequence rotated by half a tile, so the true seam (between value 255 and value 0) is mid-path
      viterbi(pl, w, table, 128, -1, sc, st);
      const int seam = st[0] >> pl.nb[0];   // the bits value 0 shares with value 255
      const float c = viterbi(pl, w, table, 0, seam, sc, st);
      pack(pl, st, out + (size_t)t * words);
      if (err != nullptr) err[t] = c;
    }
  };
  std::vector<std::thread> pool;
  for (int i = 1; i < nthreads; ++i) pool.emplace_back(work);
  work();
  for (auto& th : pool) th.join();
  return 0;
}

}  // extern "C"
