// Host-side EXL3 codec: the bit-exact trellis decoder (tile bit ring -> 16-bit states -> codebook fp16 bits) and the effective
// dense weight (both Hadamard rotations and the sign / scale vectors applied), multi-threaded over tile rows.
//
// Format facts (behaviour parity: reference crates/exl3/src/lib.rs:64-154): a 16x16 tile is a circular, MSB-first ring of 256*bits
// bits stored as int16 words, two per 32-bit ring word (low half first); value p is the 16-bit window that ends at bit E(p); stream
// position p sits at row 2*(lane%4) + (j&1) + 8*((j>>1)&1), column lane/4 + 8*(j>>2) of the tile, with lane = p/8, j = p%8.
// The Python module `rexl3_b200.format.exl3` is the oracle these functions are tested against.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

struct TilePlan {
  int nw;            // 32-bit ring words per tile
  int i0[256], i1[256], sh[256];
  int row[256], col[256];
};

TilePlan make_tile_plan(int twice) {
  TilePlan pl;
  pl.nw = 4 * twice;
  const long ring = 32L * pl.nw;
  for (int p = 0; p < 256; ++p) {
    const long p1 = p + 1;
    const long end = (twice % 2 == 0) ? p1 * (twice / 2) : (p1 * twice - (p1 % 2)) / 2;
    const long first = end + ring - 16;
    pl.i0[p] = (int)((first / 32) % pl.nw);
    pl.i1[p] = (pl.i0[p] + 1) % pl.nw;
    pl.sh[p] = 48 - (int)(first % 32);
    const int lane = p / 8, j = p % 8;
    pl.row[p] = 2 * (lane % 4) + (j & 1) + 8 * ((j >> 1) & 1);
    pl.col[p] = lane / 4 + 8 * (j >> 2);
  }
  return pl;
}

inline void tile_states(const TilePlan& pl, const int16_t* tile, uint16_t* st) {
  uint64_t words[64];
  const uint16_t* u = reinterpret_cast<const uint16_t*>(tile);
  for (int i = 0; i < pl.nw; ++i) words[i] = (uint64_t)u[2 * i] | ((uint64_t)u[2 * i + 1] << 16);
  for (int p = 0; p < 256; ++p) {
    const uint64_t pair = (words[pl.i0[p]] << 32) | words[pl.i1[p]];
    st[p] = (uint16_t)((pair >> pl.sh[p]) & 0xFFFF);
  }
}

inline float half_bits_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF, out;
  if (exp == 0) {
    if (man == 0) {
      out = sign;
    } else {                       // subnormal: renormalise
      int e = -1;
      do { ++e; man <<= 1; } while ((man & 0x400) == 0);
      out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) {
    out = sign | 0x7F800000u | (man << 13);
  } else {
    out = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

// in-place unnormalised Walsh-Hadamard transform of 128 values (Sylvester order), then / sqrt(128)
inline void fwht128(double* v) {
  for (int h = 1; h < 128; h <<= 1)
    for (int i = 0; i < 128; i += h << 1)
      for (int j = i; j < i + h; ++j) {
        const double a = v[j], b = v[j + h];
        v[j] = a + b;
        v[j + h] = a - b;
      }
  const double s = 1.0 / std::sqrt(128.0);
  for (int i = 0; i < 128; ++i) v[i] *= s;
}

template <class F>
void parallel_for(int n, int threads, F&& body) {
  int nt = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
  nt = std::max(1, std::min(nt, std::max(n, 1)));
  std::atomic<int> next(0);
  auto work = [&]() {
    for (;;) {
      const int i = next.fetch_add(1);
      if (i >= n) break;
      body(i);
    }
  };
  std::vector<std::thread> pool;
  for (int i = 1; i < nt; ++i) pool.emplace_back(work);
  work();
  for (auto& th : pool) th.join();
}

bool width_ok(int twice) {
  static const int ok[] = {2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16};
  return std::find(std::begin(ok), std::end(ok), twice) != std::end(ok);
}

}  // namespace

extern "C" {

// trellis int16 [kt][nt][8*twice] -> states uint16 [kt][nt][256] (stream order).  Returns 0, or 1 on bad arguments.
int rx_exl3_states_host(const int16_t* trellis, int kt, int nt, int twice, uint16_t* out, int threads) {
  if (!width_ok(twice) || kt < 0 || nt < 0) return 1;
  const TilePlan pl = make_tile_plan(twice);
  const int words = 8 * twice;
  parallel_for(kt, threads, [&](int r) {
    for (int c = 0; c < nt; ++c) tile_states(pl, trellis + ((size_t)r * nt + c) * words, out + ((size_t)r * nt + c) * 256);
  });
  return 0;
}

// trellis -> W_q as fp16 bit patterns, uint16 [kt*16][nt*16]; table: uint16 [65536] codebook (fp16 bits of every state).
int rx_exl3_unpack_host(const int16_t* trellis, int kt, int nt, int twice, const uint16_t* table, uint16_t* out, int threads) {
  if (!width_ok(twice) || kt < 0 || nt < 0) return 1;
  const TilePlan pl = make_tile_plan(twice);
  const int words = 8 * twice;
  const size_t N = (size_t)nt * 16;
  parallel_for(kt, threads, [&](int r) {
    uint16_t st[256];
    for (int c = 0; c < nt; ++c) {
      tile_states(pl, trellis + ((size_t)r * nt + c) * words, st);
      uint16_t* base = out + (size_t)r * 16 * N + (size_t)c * 16;
      for (int p = 0; p < 256; ++p) base[(size_t)pl.row[p] * N + pl.col[p]] = table[st[p]];
    }
  });
  return 0;
}

// The effective dense weight W [K][N] (float64) with layer(x) == x @ W:  W = diag(suh) Had_K W_q Had_N diag(svh), Had block-diagonal
// 128 wide.  suh [K], svh [N] as float64 (null = ones).  Summation order inside a transform is the butterfly's; results agree with the
// matrix form to rounding, not bit for bit.
int rx_exl3_decode_weight_host(const int16_t* trellis, int kt, int nt, int twice, const uint16_t* table, const double* suh, const double* svh,
                               double* out, int threads) {
  if (!width_ok(twice) || kt % 8 || nt % 8 || kt < 0 || nt < 0) return 1;
  const TilePlan pl = make_tile_plan(twice);
  const int words = 8 * twice;
  const size_t K = (size_t)kt * 16, N = (size_t)nt * 16;
  // pass 1: decode, one 16-row tile row at a time
  parallel_for(kt, threads, [&](int r) {
    uint16_t st[256];
    for (int c = 0; c < nt; ++c) {
      tile_states(pl, trellis + ((size_t)r * nt + c) * words, st);
      double* base = out + (size_t)r * 16 * N + (size_t)c * 16;
      for (int p = 0; p < 256; ++p) base[(size_t)pl.row[p] * N + pl.col[p]] = (double)half_bits_to_float(table[st[p]]);
    }
  });
  // pass 2: Had_K down the columns, per 128-row block and column strip (16 columns at a time for locality)
  const int kb = (int)(K / 128), strips = (int)(N / 16);
  parallel_for(kb * strips, threads, [&](int job) {
    const int b = job / strips, s = job % strips;
    double col[128];
    for (int c = 0; c < 16; ++c) {
      const size_t n = (size_t)s * 16 + c;
      for (int i = 0; i < 128; ++i) col[i] = out[((size_t)b * 128 + i) * N + n];
      fwht128(col);
      for (int i = 0; i < 128; ++i) out[((size_t)b * 128 + i) * N + n] = col[i] * (suh ? suh[(size_t)b * 128 + i] : 1.0);
    }
  });
  // pass 3: Had_N along each row, then svh
  parallel_for((int)K, threads, [&](int k) {
    double* row = out + (size_t)k * N;
    for (size_t n0 = 0; n0 < N; n0 += 128) {
      fwht128(row + n0);
      if (svh)
        for (int i = 0; i < 128; ++i) row[n0 + i] *= svh[n0 + i];
    }
  });
  return 0;
}

}  // extern "C"
