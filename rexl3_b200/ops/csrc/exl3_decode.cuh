// EXL3 trellis decode on the device: 16-bit window extraction with compile-time offsets and the three
// codebooks (3inst, mcg, mul1), producing fp16 pairs.  Bit-exact with the CPU codec
// (rexl3_b200/format/exl3.py; format semantics as in reference crates/exl3/src/lib.rs:94-154).
//
// Work split: a 16x16 tile (256 values) is decoded by 4 threads; thread h takes stream positions
// [64h, 64h+64) whose new bits are exactly TWICE 32-bit words (TWICE = 2 * bits per weight), so the
// split is word aligned for every width including 1.5 / 2.5 / 3.5 bpw.  Those 64 values are the 16 k-rows
// of the 4 tile columns n = 2h, 2h+1, 2h+8, 2h+9, which is what lets a thread emit whole 16-byte K-major
// chunks of the tensor-core operand.
#pragma once
#include "common.cuh"

namespace rx {

enum : int { CB_3INST = 0, CB_MCG = 1, CB_MUL1 = 2 };

template <int TWICE>
__host__ __device__ constexpr int rel_end(int q) {  // end bit (exclusive) of value q in [0, 64) relative to the chunk start
  return (TWICE % 2 == 0) ? (q + 1) * (TWICE / 2) : ((q + 1) * TWICE - ((q + 1) & 1)) / 2;
}

// w[0] = the word before the span (ring wrap handled by the caller), w[1..NW] = the span's words.
template <int TWICE, int Q, int NW>
__device__ __forceinline__ uint32_t state_of(const uint32_t (&w)[NW + 1]) {
  constexpr int s = rel_end<TWICE>(Q) + 16;  // start bit of the 16-bit window inside w[]
  constexpr int wi = s / 32, off = s % 32;
  if constexpr (off == 0) {
    return w[wi] >> 16;
  } else if constexpr (off == 16) {
    return w[wi] & 0xFFFFu;
  } else if constexpr (off < 16) {
    return (w[wi] >> (16 - off)) & 0xFFFFu;
  } else {
    return __funnelshift_l(w[wi + 1], w[wi], off) >> 16;
  }
}

// Pipe balance of the decode (measured on B200 with register-only loops, lane-operations per clock per SM): the integer ALU pipe
// (LOP3, SHF, PRMT) issues 64, the multiply pipe (IMAD, HADD2 / HFMA2, DP2A / DP4A: they share ONE pipe) issues 64, and the two run
// side by side.  The decode is bound by whichever pipe gets more operations per weight, so the work is split evenly between them:
//  * (x & mask) ^ flip is ONE three-input LOP3.  Written with two literals the compiler emits an AND and an XOR (a LOP3 takes a single
//    immediate); with the constants read from constant memory, which it cannot fold, it keeps the one instruction.
//  * half of the "low 16 bits" extractions are DP2A(x, 1) on the multiply pipe instead of an AND on the ALU pipe.
static __constant__ uint32_t rx_dec_consts[4] = {0x8FFF8FFFu, 0x3B603B60u, 1u, 0u};

__device__ __forceinline__ uint32_t mask_flip(uint32_t x) {
  uint32_t y;
  asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(y) : "r"(x), "r"(rx_dec_consts[0]), "r"(rx_dec_consts[1]));   // (x & mask) ^ flip
  return y;
}
// x & 0xFFFF computed on the multiply pipe: x.h0 * 1 + x.h1 * 0 + 0
__device__ __forceinline__ uint32_t low16_mul(uint32_t x) {
  uint32_t s;
  asm("dp2a.lo.u32.u32 %0, %1, %2, %3;" : "=r"(s) : "r"(x), "r"(rx_dec_consts[2]), "r"(rx_dec_consts[3]));
  return s;
}

template <int CB>
__device__ __forceinline__ uint32_t pair_to_half2(uint32_t sa, uint32_t sb) {
  if constexpr (CB == CB_MUL1) {
    const uint32_t xa = sa * 0x83DCD12Du, xb = sb * 0x83DCD12Du;
    // 1024 + byte sum as an fp16 bit pattern: integers in [1024, 2048) are 0x6400 + (h - 1024)
    const uint32_t ha = __dp4a(xa, 0x01010101u, 0x6400u), hb = __dp4a(xb, 0x01010101u, 0x6400u);
    const uint32_t packed = __byte_perm(ha, hb, 0x5410);
    const __half2 sc = __halves2half2(__ushort_as_half(0x1EEE), __ushort_as_half(0x1EEE));
    const __half2 bi = __halves2half2(__ushort_as_half(0xC931), __ushort_as_half(0xC931));
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&packed), sc, bi);
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    uint32_t xa, xb;
    if constexpr (CB == CB_MCG) {
      xa = sa * 0xCBAC1FEDu; xb = sb * 0xCBAC1FEDu;
    } else {
      xa = sa * 89226354u + 64248484u; xb = sb * 89226354u + 64248484u;
    }
    xa = mask_flip(xa);
    xb = mask_flip(xb);
    // lo + hi of each word as a half2 add with swizzled operands (multiply pipe), then ONE byte permute packs the pair
    const __half2 a = *reinterpret_cast<const __half2*>(&xa), b = *reinterpret_cast<const __half2*>(&xb);
    const __half2 ra = __hadd2(__low2half2(a), __high2half2(a)), rb = __hadd2(__low2half2(b), __high2half2(b));
    return __byte_perm(*reinterpret_cast<const uint32_t*>(&ra), *reinterpret_cast<const uint32_t*>(&rb), 0x7610);
  }
}

// 4 sixteen-bit fields of X at MSB-first bit offsets 4, 8, 12, 16: a shift and two byte permutes on the ALU pipe; the two
// "low 16 bits" go to the multiply pipe when the codebook leaves it room (MUL_LOW), else they are two ANDs
template <bool MUL_LOW = false>
__device__ __forceinline__ void extract4(uint32_t X, uint32_t& s0, uint32_t& s1, uint32_t& s2, uint32_t& s3) {
  const uint32_t X4 = X >> 4;
  s0 = __byte_perm(X4, 0, 0x4421);
  s1 = __byte_perm(X, 0, 0x4421);
  if constexpr (MUL_LOW) {
    s2 = low16_mul(X4);
    s3 = low16_mul(X);
  } else {
    s2 = X4 & 0xFFFFu;
    s3 = X & 0xFFFFu;
  }
}

// 4.0 bpw fast path: 32 consecutive values from their 4 words (w[1..4]) and the word before them (w[0]).
// Value q's window starts at bit 20 + 4q of w[]: per word pair the windows sit at offsets 4, 8, 12, 16 of
// A = bits 16..47 of the pair and at the same offsets of the second word.
template <int CB>
__device__ __forceinline__ void decode32_b4(const uint32_t (&w)[5], uint32_t (&h2)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t A = __funnelshift_l(w[i + 1], w[i], 16), B = w[i + 1];
    uint32_t s0, s1, s2, s3, s4, s5, s6, s7;
    extract4<CB != CB_MUL1>(A, s0, s1, s2, s3);
    extract4<CB != CB_MUL1>(B, s4, s5, s6, s7);
    h2[4 * i + 0] = pair_to_half2<CB>(s0, s1);
    h2[4 * i + 1] = pair_to_half2<CB>(s2, s3);
    h2[4 * i + 2] = pair_to_half2<CB>(s4, s5);
    h2[4 * i + 3] = pair_to_half2<CB>(s6, s7);
  }
}

template <int TWICE, int CB, int NV, int I>
__device__ __forceinline__ void decode_rec(const uint32_t (&w)[NV * TWICE / 64 + 1], uint32_t (&h2)[NV / 2]) {
  if constexpr (I < NV / 2) {
    h2[I] = pair_to_half2<CB>(state_of<TWICE, 2 * I, NV * TWICE / 64>(w), state_of<TWICE, 2 * I + 1, NV * TWICE / 64>(w));
    decode_rec<TWICE, CB, NV, I + 1>(w, h2);
  }
}

// NV (32 or 64) consecutive stream values starting at 32-bit word `first_word` of the tile's ring -> NV/2 half2;
// h2[i] = (value 2i, value 2i+1) = two consecutive k of one column.  `tile` points at the tile's 4*TWICE words
// (shared or global memory).  NV = 32 needs an even TWICE (word-aligned eighths).
template <int TWICE, int CB, int NV>
__device__ __forceinline__ void decode_span(const uint32_t* tile, int first_word, uint32_t (&h2)[NV / 2]) {
  constexpr int NW = NV * TWICE / 64;
  static_assert(NV == 64 || (NV == 32 && TWICE % 2 == 0), "eighth-tile spans need an integer width");
  uint32_t w[NW + 1];
  w[0] = tile[(first_word + 4 * TWICE - 1) % (4 * TWICE)];
#pragma unroll
  for (int i = 0; i < NW; ++i) w[i + 1] = tile[first_word + i];
  decode_rec<TWICE, CB, NV, 0>(w, h2);
}

// Quarter h (64 values) covers tile columns n = 2h + a + 8*b2 (a, b2 in {0,1}); its 16-byte chunk (a, b2, kc) holds
// k = 8kc .. 8kc+7 of that column and is built from h2[16a + 4m + 2*b2 + kc], m = 0..3.
__device__ __forceinline__ uint4 quarter_chunk(const uint32_t (&h2)[32], int a, int b2, int kc) {
  const int base = 16 * a + 2 * b2 + kc;
  return make_uint4(h2[base], h2[base + 4], h2[base + 8], h2[base + 12]);
}
// Eighth g (32 values) covers tile columns n = g + 8*b2; chunk (b2, kc) is built from h2[4m + 2*b2 + kc].
__device__ __forceinline__ uint4 eighth_chunk(const uint32_t (&h2)[16], int b2, int kc) {
  const int base = 2 * b2 + kc;
  return make_uint4(h2[base], h2[base + 4], h2[base + 8], h2[base + 12]);
}

#define RX_DISPATCH_TWICE(TW, ...)                                   \
  switch (TW) {                                                      \
    case 2: { constexpr int T_ = 2; __VA_ARGS__; } break;            \
    case 3: { constexpr int T_ = 3; __VA_ARGS__; } break;            \
    case 4: { constexpr int T_ = 4; __VA_ARGS__; } break;            \
    case 5: { constexpr int T_ = 5; __VA_ARGS__; } break;            \
    case 6: { constexpr int T_ = 6; __VA_ARGS__; } break;            \
    case 7: { constexpr int T_ = 7; __VA_ARGS__; } break;            \
    case 8: { constexpr int T_ = 8; __VA_ARGS__; } break;            \
    case 10: { constexpr int T_ = 10; __VA_ARGS__; } break;          \
    case 12: { constexpr int T_ = 12; __VA_ARGS__; } break;          \
    case 14: { constexpr int T_ = 14; __VA_ARGS__; } break;          \
    case 16: { constexpr int T_ = 16; __VA_ARGS__; } break;          \
    default: return (int)cudaErrorInvalidValue;                      \
  }

}  // namespace rx
