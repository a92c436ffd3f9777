// Paged GQA attention for sm_100a: split-KV decode (+ merge fused with o_proj's input rotation) and causal flash
// prefill, bf16 KV in 64-token pages.
//
// Cache layout (chosen so that one page of one KV head is ONE contiguous 64 x head_dim tile, i.e. one TMA box):
//     k_cache, v_cache : bf16 [num_pages][n_kv_heads][64][head_dim]
//     block_table      : int32 [num_seqs][max_blocks]   (page index of each 64-token block of a sequence)
// K/V tiles are brought in by TMA (2-D tiled, SWIZZLE_128B, no multicast) through a small ring of stages; the
// matrix math is bf16 mma.sync with fp32 online softmax, which is enough for a kernel whose roofline is HBM.
//
// Decode: one CTA per (row, kv head, 256-key chunk); chunks are ABSOLUTE key ranges and partials are merged in chunk
// order, so a row's bits never depend on the batch (same idea as the reference's 512-key chunks,
// crates/cuda/csrc/attention.cu:16-21; geometry, page size, KV layout and schedule are new).  The 4 warps of a CTA
// each take 16 keys of every page and are merged in warp order.
// Prefill (this file: FP8 caches and 64-wide heads): one CTA per (64 query rows, q head, sequence); warps own 16 query rows each and
// walk the pages causally.  bf16 caches with 128-wide heads run the tcgen05 / tensor-memory kernel of attention_tc.cu instead.
#include <cuda.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include "common.cuh"

namespace rx {

constexpr int PAGE = 64;
constexpr int DEC_CHUNK = 256;              // keys per decode CTA (4 pages)
constexpr int ATT_THREADS = 128;
constexpr int KV_STAGES = 3;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// a bf16 pair (as loaded from the query buffer) as an fp16 pair
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t u) {
  return pack_f16(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// A K or V page tile in shared memory: HD/64 boxes of [64 keys x 64 d] (128-byte rows, 128B swizzle), box b at b*8192.
// Byte address of the 16-byte chunk `dchunk` (8 bf16) of key `key`.
template <int HD>
__device__ __forceinline__ uint32_t kv_chunk_addr(uint32_t base, int key, int dchunk) {
  return base + (dchunk >> 3) * 8192 + key * 128 + (((dchunk & 7) ^ (key & 7)) << 4);
}

template <int HD>
__device__ __forceinline__ void load_kv_page(uint8_t* kdst, uint8_t* vdst, const CUtensorMap* tk, const CUtensorMap* tv, int page, int kvh,
                                             int n_kv, uint64_t* bar) {
  constexpr int BYTES = PAGE * HD * 2;
  mbar_arrive_expect_tx(bar, 2 * BYTES);
  const int y = (page * n_kv + kvh) * PAGE;
#pragma unroll
  for (int b = 0; b < HD / 64; ++b) {
    tma_load_2d(kdst + b * 8192, tk, b * 64, y, bar);
    tma_load_2d(vdst + b * 8192, tv, b * 64, y, bar);
  }
}

// FP8 (E4M3) cache: a page of one KV head is 64 x HD bytes, loaded unswizzled, then expanded by the whole CTA to an fp16 tile in the
// swizzled layout the fragment loads expect.  E4M3 -> fp16 is exact; the per-head scale is applied to the scores / the output.
template <int HD>
__device__ __forceinline__ void load_kv_page8(uint8_t* kdst, uint8_t* vdst, const CUtensorMap* tk, const CUtensorMap* tv, int page, int kvh,
                                              int n_kv, uint64_t* bar) {
  constexpr int BYTES = PAGE * HD;
  mbar_arrive_expect_tx(bar, 2 * BYTES);
  const int y = (page * n_kv + kvh) * PAGE;
  tma_load_2d(kdst, tk, 0, y, bar);
  tma_load_2d(vdst, tv, 0, y, bar);
}

// KV cache element formats of the attention kernels
constexpr int KVQ_BF16 = 0, KVQ_FP8 = 1, KVQ_I8 = 2;
// (template parameter I8 of the byte-page kernels: 0 = E4M3 with per-head scales, 1 = int8 with a scale per token and head, 2 = q4)

// int8 cache with one power-of-two scale per (token, KV head) (the reference's format, crates/cuda/csrc/nemotron_kv8.cuh:1-14): a page of one KV
// head is 64 x HD bytes plus 64 f32 scales for K and 64 for V ([pages][n_kv][64] each); the scales ride on the page's barrier as two 256-byte
// bulk copies.  The expansion multiplies them in: int8 x 2^e is exact in fp16, so the tile holds the dequantised values and the attention
// step is the fp16 one with no further scale.
template <int HD>
__device__ __forceinline__ void load_kv_page_i8(uint8_t* kdst, uint8_t* vdst, float* sc, const CUtensorMap* tk, const CUtensorMap* tv,
                                                const float* __restrict__ k_ts, const float* __restrict__ v_ts, int page, int kvh, int n_kv,
                                                uint64_t* bar) {
  constexpr int BYTES = PAGE * HD;
  mbar_arrive_expect_tx(bar, 2 * BYTES + 2 * PAGE * 4);
  const int y = (page * n_kv + kvh) * PAGE;
  tma_load_2d(kdst, tk, 0, y, bar);
  tma_load_2d(vdst, tv, 0, y, bar);
  bulk_g2s(sc, k_ts + (size_t)y, PAGE * 4, bar);
  bulk_g2s(sc + PAGE, v_ts + (size_t)y, PAGE * 4, bar);
}

// sc != nullptr: the bytes are int8 and sc[key] is the key's scale (else: E4M3 bytes)
template <int HD>
__device__ __forceinline__ void expand_page8(const uint8_t* src, uint8_t* dst, const float* sc = nullptr) {
  constexpr int CHUNKS = PAGE * HD / 16;          // 16 values each
  const uint32_t dbase = smem_u32(dst);
  for (int c = threadIdx.x; c < CHUNKS; c += blockDim.x) {
    const int key = c / (HD / 16), j = c % (HD / 16);
    const uint4 r = *reinterpret_cast<const uint4*>(src + (size_t)c * 16);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    uint32_t h[8];
    if (sc != nullptr) {
      // (b ^ 0x80) under the exponent byte 0x64 is the fp16 number 1024 + 128 + b; one fused multiply-add takes it to b * scale, exactly
      const __half2 s2 = __float2half2_rn(sc[key]);
      const __half2 off = __hmul2(__float2half2_rn(-1152.f), s2);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t u = w[i] ^ 0x80808080u;
        const uint32_t lo = __byte_perm(u, 0x64646464u, 0x4140), hi = __byte_perm(u, 0x64646464u, 0x4342);
        const __half2 a = __hfma2(*reinterpret_cast<const __half2*>(&lo), s2, off), b = __hfma2(*reinterpret_cast<const __half2*>(&hi), s2, off);
        h[2 * i] = *reinterpret_cast<const uint32_t*>(&a);
        h[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&b);
      }
    } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] & 0xFFFFu), __NV_E4M3);
      const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] >> 16), __NV_E4M3);
      h[2 * i] = *reinterpret_cast<const uint32_t*>(&lo);
      h[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&hi);
    }
    }
    const uint32_t a0 = kv_chunk_addr<HD>(dbase, key, 2 * j), a1 = kv_chunk_addr<HD>(dbase, key, 2 * j + 1);
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a0), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a1), "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]) : "memory");
  }
}

// q4 cache (E2M1 nibbles with one E8M0 scale per 32 values: the MXFP4 element format on K / V rows; reference crates/cuda/csrc/dsv4_kvq4.cu:1-16
// for the row format): a page of one KV head is 64 x HD/2 bytes plus 64 x HD/32 scale bytes for K and for V ([pages][n_kv][64][HD/32] uint8).
// The scale bytes ride on the page's barrier as two bulk copies; the expansion multiplies them in (E2M1 x 2^e is exact in fp16 inside the
// clamped exponent range), so the attention step is the fp16 one.
template <int HD>
__device__ __forceinline__ void load_kv_page_q4(uint8_t* kdst, uint8_t* vdst, uint8_t* sc, const CUtensorMap* tk, const CUtensorMap* tv,
                                                const uint8_t* __restrict__ k_s4, const uint8_t* __restrict__ v_s4, int page, int kvh, int n_kv,
                                                uint64_t* bar) {
  constexpr int BYTES = PAGE * HD / 2, SB = PAGE * HD / 32;
  mbar_arrive_expect_tx(bar, 2 * BYTES + 2 * SB);
  const int y = (page * n_kv + kvh) * PAGE;
  tma_load_2d(kdst, tk, 0, y, bar);
  tma_load_2d(vdst, tv, 0, y, bar);
  bulk_g2s(sc, k_s4 + (size_t)y * (HD / 32), SB, bar);
  bulk_g2s(sc + PAGE * 4, v_s4 + (size_t)y * (HD / 32), SB, bar);
}

__device__ __forceinline__ uint32_t e8m0_half2(uint32_t b) {      // 2^(b - 127) as two fp16 (the writer keeps b - 127 in -14 .. 12)
  const int e = (int)b - 127;
  const uint32_t h = e < -14 ? 0u : (e > 15 ? 0x7C00u : (uint32_t)(e + 15) << 10);
  return h | (h << 16);
}

template <int HD>
__device__ __forceinline__ void expand_page4(const uint8_t* src, uint8_t* dst, const uint8_t* sc) {
  constexpr int G = HD / 32;                      // scale groups per key
  constexpr int CHUNKS = PAGE * G;                // one 16-byte source chunk = one group of 32 values
  const uint32_t dbase = smem_u32(dst);
  for (int c = threadIdx.x; c < CHUNKS; c += blockDim.x) {
    const int key = c / G, g = c % G;
    const uint4 r = *reinterpret_cast<const uint4*>(src + (size_t)c * 16);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    const uint32_t s2u = e8m0_half2(sc[key * G + g]);
    const __half2 s2 = *reinterpret_cast<const __half2*>(&s2u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {               // word i: 8 values = one 16-byte chunk of the fp16 row
      uint32_t h[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((w[i] >> (8 * q)) & 0xFFu), __NV_E2M1);
        const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&hr), s2);
        h[q] = *reinterpret_cast<const uint32_t*>(&v);
      }
      const uint32_t a = kv_chunk_addr<HD>(dbase, key, 4 * g + i);
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
    }
  }
}

// One 16-row x NK-key step of flash attention for a warp.  qa: Q fragments [HD/16][4]; keys [key0, key0 + NK) of the
// page tile at (ksm, vsm).  valid = number of unmasked keys counted from key0 for rows (r_lo) and (r_hi) (causal/ctx).
template <int HD, int NK, bool F16 = false>
__device__ __forceinline__ void attn_step(const uint32_t (&qa)[HD / 16][4], uint32_t ksm, uint32_t vsm, int key0, int valid_lo, int valid_hi,
                                          float scale_log2, float (&m)[2], float (&l)[2], float (&o)[HD / 8][4]) {
  const int lane = threadIdx.x & 31;
  constexpr int NT = NK / 8;
  float s[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      uint32_t b0, b1, b2, b3;
      const int mi = lane >> 3;
      const int key = key0 + jp * 16 + (mi >> 1) * 8 + (lane & 7);
      ldsm_x4(kv_chunk_addr<HD>(ksm, key, ks * 2 + (mi & 1)), b0, b1, b2, b3);
      if constexpr (F16) { mma_f16(s[2 * jp], qa[ks], b0, b1); mma_f16(s[2 * jp + 1], qa[ks], b2, b3); }
      else { mma_bf16(s[2 * jp], qa[ks], b0, b1); mma_bf16(s[2 * jp + 1], qa[ks], b2, b3); }
    }
  }
  // mask + row max
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = j * 8 + 2 * (lane & 3) + (e & 1);
      const int lim = (e < 2) ? valid_lo : valid_hi;
      const float v = (kk < lim) ? s[j][e] * scale_log2 : -INFINITY;
      s[j][e] = v;
      mx[e >> 1] = fmaxf(mx[e >> 1], v);
    }
  }
  float corr[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float mn = fmaxf(m[r], mx[r]);
    corr[r] = (mn == -INFINITY) ? 1.f : exp2f(m[r] - mn);
    m[r] = mn;
  }
  float rs[2] = {0.f, 0.f};
  uint32_t pa[NT / 2][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    float p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float mm = m[e >> 1];
      p[e] = (mm == -INFINITY) ? 0.f : exp2f(s[j][e] - mm);
      rs[e >> 1] += p[e];
    }
    pa[j >> 1][(j & 1) * 2 + 0] = F16 ? pack_f16(p[0], p[1]) : pack_bf16(p[0], p[1]);
    pa[j >> 1][(j & 1) * 2 + 1] = F16 ? pack_f16(p[2], p[3]) : pack_bf16(p[2], p[3]);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) l[r] = l[r] * corr[r] + rs[r];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) {
    o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1];
  }
#pragma unroll
  for (int kp = 0; kp < NT / 2; ++kp) {
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
      uint32_t b0, b1, b2, b3;
      const int mi = lane >> 3;
      const int key = key0 + kp * 16 + (mi & 1) * 8 + (lane & 7);
      ldsm_x4_t(kv_chunk_addr<HD>(vsm, key, dp * 2 + (mi >> 1)), b0, b1, b2, b3);
      if constexpr (F16) { mma_f16(o[2 * dp], pa[kp], b0, b1); mma_f16(o[2 * dp + 1], pa[kp], b2, b3); }
      else { mma_bf16(o[2 * dp], pa[kp], b0, b1); mma_bf16(o[2 * dp + 1], pa[kp], b2, b3); }
    }
  }
}


// The decode kernel's step: like attn_step for MT tiles at once over the same 16 keys.  Each K / V fragment is fetched from shared memory once
// and feeds every tile's MMA; a row's running maximum is only moved when the new scores exceed it by more than 2^8 (the accumulators are then
// rescaled; otherwise the stale maximum stays and P holds values up to 256, well inside bf16 / fp16 range), so the 64 multiplies of the
// rescale are skipped for most pages.  `ntiles` (uniform) = tiles that hold a live row.
template <int HD, int MT, bool F16>
__device__ __forceinline__ void attn_step_mt(const uint32_t (&qa)[MT][HD / 16][4], uint32_t ksm, uint32_t vsm, int key0, const int (&valid)[MT][2],
                                             int ntiles, float scale_log2, float (&m)[MT][2], float (&l)[MT][2], float (&o)[MT][HD / 8][4]) {
  const int lane = threadIdx.x & 31;
  float s[MT][2][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j) { s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.f; }
  {
    const int mi = lane >> 3;
    const int key = key0 + (mi >> 1) * 8 + (lane & 7);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(kv_chunk_addr<HD>(ksm, key, ks * 2 + (mi & 1)), b0, b1, b2, b3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if (mt < ntiles) {
          if constexpr (F16) { mma_f16(s[mt][0], qa[mt][ks], b0, b1); mma_f16(s[mt][1], qa[mt][ks], b2, b3); }
          else { mma_bf16(s[mt][0], qa[mt][ks], b0, b1); mma_bf16(s[mt][1], qa[mt][ks], b2, b3); }
        }
      }
    }
  }
  uint32_t pa[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    if (mt < ntiles) {
      // mask + row max
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int kk = j * 8 + 2 * (lane & 3) + (e & 1);
          const float v = (kk < valid[mt][e >> 1]) ? s[mt][j][e] * scale_log2 : -INFINITY;
          s[mt][j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2];
      bool moved = false;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        corr[r] = 1.f;
        if (mx[r] > m[mt][r] + 8.f) {              // also the first valid keys of a row (m = -inf)
          corr[r] = (m[mt][r] == -INFINITY) ? 1.f : exp2f(m[mt][r] - mx[r]);
          m[mt][r] = mx[r];
          moved = moved || corr[r] != 1.f;
        }
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float mm = m[mt][e >> 1];
          p[e] = (mm == -INFINITY) ? 0.f : exp2f(s[mt][j][e] - mm);
          rs[e >> 1] += p[e];
        }
        pa[mt][j * 2 + 0] = F16 ? pack_f16(p[0], p[1]) : pack_bf16(p[0], p[1]);
        pa[mt][j * 2 + 1] = F16 ? pack_f16(p[2], p[3]) : pack_bf16(p[2], p[3]);
      }
      if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int r = 0; r < 2; ++r) l[mt][r] *= corr[r];
#pragma unroll
        for (int d = 0; d < HD / 8; ++d) {
          o[mt][d][0] *= corr[0]; o[mt][d][1] *= corr[0]; o[mt][d][2] *= corr[1]; o[mt][d][3] *= corr[1];
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) l[mt][r] += rs[r];
    }
  }
  {
    const int mi = lane >> 3;
    const int key = key0 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(kv_chunk_addr<HD>(vsm, key, dp * 2 + (mi >> 1)), b0, b1, b2, b3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if (mt < ntiles) {
          if constexpr (F16) { mma_f16(o[mt][2 * dp], pa[mt], b0, b1); mma_f16(o[mt][2 * dp + 1], pa[mt], b2, b3); }
          else { mma_bf16(o[mt][2 * dp], pa[mt], b0, b1); mma_bf16(o[mt][2 * dp + 1], pa[mt], b2, b3); }
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ decode (split-KV)
// Bytes of the decode kernel's main shared region: the K / V stages (and the FP8 expansion tiles) while pages stream, the per-warp partial
// outputs [4 MT][16][HD] f32 once they are done.  The barriers and the per-warp (max, sum) pairs sit behind it.
__host__ __device__ constexpr int dec_region_bytes(int hd, bool fp8, int mt) {
  const int stages = fp8 ? 2 * KV_STAGES * PAGE * hd + 2 * PAGE * hd * 2 : 2 * KV_STAGES * PAGE * hd * 2;
  const int merge = mt * 4 * 16 * (hd + 8) * 4;   // rows padded by 8 floats
  return stages > merge ? stages : merge;
}
__host__ __device__ constexpr int dec_smem_bytes(int hd, bool fp8, int mt) { return dec_region_bytes(hd, fp8, mt) + 64 + mt * 4 * 16 * 2 * 4 + 128 + KV_STAGES * 2 * PAGE * 4 + 1024; }
// ---- the window plan: which rows share a CTA's MMA tiles, and the flat list of work items
// Row blocking: the 16 * MT rows of a CTA's MMA tiles hold RB = 16 MT / G consecutive window rows of ONE sequence (a verify window feeds
// [last, d1 .. dk] of a sequence as adjacent rows) times the G query heads of one KV head, so the sequence's K / V chunk is read once per RB
// rows instead of once per row (the reference packs RBLK * GRP = 48 (row, head) pairs the same way, crates/cuda/csrc/attention.cu:42-50).
// The plan is a function of row_seq and ctx_len only, so one plan serves every layer of a forward.  Layout (int32):
//   [0] work items in total   [1] blocks   [2] RB   [3] n_kv   then, from PLAN_HEAD on, six arrays of PLAN_MAX_ROWS (+1) entries:
//   first row of block b | rows in block b | chunks of block b (from the largest context among its rows) | items before block b (prefix) |
//   sequence of block b (its block-table row; -1 - r = row r of the private table) | first chunk of block b
// A work item is (block, chunk, kv head): item = prefix[b] + (chunk - first chunk) * n_kv + kvh.
//
// Tree windows (tree_base != nullptr).  A sequence's rows are the nodes of a draft tree: row r stands at position ctx_len[r] - 1 =
// tree_base[r] + depth and must see the committed keys 0 .. tree_base[r] plus ITS OWN ancestors at positions tree_base + 1 .. .  The chunks that
// end at or before tree_base are the same for every node: they are planned as shared blocks over the sequence's block-table row, as in a
// chain window.  The chunks from (tree_base + 1) / DEC_CHUNK on are planned once per row over that row's PRIVATE table (vbt: VBT_W page ids,
// the first one standing for page index first chunk * 4), in which the caller put the pages that hold the row's own path at its true
// positions.  So every (row, chunk) partial is computed over exactly the keys, at exactly the positions, of the serial run that feeds the
// path's tokens one by one, and the bits are the serial run's.  (The reference keeps ancestors' K / V in node buffers for the same end,
// crates/cuda/csrc/attention.cu:443.)
constexpr int PLAN_MAX_ROWS = 1024, PLAN_HEAD = 8;
constexpr int PLAN_INTS = PLAN_HEAD + 6 * PLAN_MAX_ROWS + 8;
constexpr int VBT_W = 2 * (DEC_CHUNK / PAGE);     // a tree's nodes span at most 64 positions: two chunks

__global__ void __launch_bounds__(256) attn_plan_kernel(const int* __restrict__ row_seq, const int* __restrict__ ctx_len, int rows, int RB, int n_kv,
                                                       int* __restrict__ plan, const int* __restrict__ tree_base) {
  pdl_launch();
  pdl_wait();
  __shared__ int s_seq[PLAN_MAX_ROWS], s_ctx[PLAN_MAX_ROWS];
  __shared__ unsigned char s_lead[PLAN_MAX_ROWS];
  for (int r = threadIdx.x; r < rows; r += blockDim.x) { s_seq[r] = row_seq[r]; s_ctx[r] = ctx_len[r]; }
  __syncthreads();
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    int pos = 0;                                   // position of the row inside its run of equal sequence ids
    while (pos < r && s_seq[r - pos - 1] == s_seq[r]) ++pos;
    s_lead[r] = (pos % RB) == 0;
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  int* blk_row = plan + PLAN_HEAD;
  int* blk_n = blk_row + PLAN_MAX_ROWS;
  int* blk_nch = blk_n + PLAN_MAX_ROWS;
  int* prefix = blk_nch + PLAN_MAX_ROWS;
  int* blk_seq = prefix + PLAN_MAX_ROWS + 1;
  int* blk_c0 = blk_seq + PLAN_MAX_ROWS;
  int nb = 0, items = 0;
  for (int r = 0; r < rows; ++r) {
    if (!s_lead[r]) continue;
    int n = 1, cmax = s_ctx[r];
    while (n < RB && r + n < rows && s_seq[r + n] == s_seq[r]) { cmax = max(cmax, s_ctx[r + n]); ++n; }
    // tree window: the shared block covers the chunks below the tree (every row of a sequence has the same tree_base)
    const int nch = tree_base != nullptr ? (tree_base[r] + 1) / DEC_CHUNK : (cmax + DEC_CHUNK - 1) / DEC_CHUNK;
    if (nch == 0) continue;
    blk_row[nb] = r; blk_n[nb] = n; blk_nch[nb] = nch; prefix[nb] = items; blk_seq[nb] = s_seq[r]; blk_c0[nb] = 0;
    items += nch * n_kv;
    ++nb;
  }
  if (tree_base != nullptr) {
    for (int r = 0; r < rows; ++r) {
      const int c0 = (tree_base[r] + 1) / DEC_CHUNK, nch = (s_ctx[r] + DEC_CHUNK - 1) / DEC_CHUNK - c0;
      if (nch <= 0) continue;
      blk_row[nb] = r; blk_n[nb] = 1; blk_nch[nb] = nch; prefix[nb] = items; blk_seq[nb] = -1 - r; blk_c0[nb] = c0;
      items += nch * n_kv;
      ++nb;
    }
  }
  prefix[nb] = items;
  plan[0] = items; plan[1] = nb; plan[2] = RB; plan[3] = n_kv;
}

// part_o  : f32 [rows][n_q][max_chunks][HD]   unnormalised partial outputs
// part_ml : f32 [rows][n_q][max_chunks][2]    (running max in log2 units, sum)
// Persistent kernel: two CTAs per SM walk the plan's work items (item = blockIdx.x, + gridDim.x, ...), so no CTA is launched for a row that a
// block mate computes, barriers are set up once, and the page counter runs on across items (stage = page % KV_STAGES).
// MT = m16 tiles per CTA.  Each of the four warps owns a 16-key slice of every page and carries MT tiles of accumulators over it; a tile is
// computed exactly as the one-tile kernel computes it, and a tile row only ever meets its own accumulators and its own key mask, so a row's
// bits depend neither on MT nor on its block mates; more tiles only let more (row, head) pairs of one sequence share one pass over the
// K / V chunk.  (Giving each tile its own four warps halved the CTAs per SM and was slower than two one-tile CTAs; launching one CTA per
// row and letting the non-leaders exit cost more than the K / V reads it saved.)
template <int HD, bool FP8, int MT, int I8 = 0>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attn_decode_kernel(const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv, const uint16_t* __restrict__ q,
                   const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_seq, const int* __restrict__ ctx_len,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int n_q, int n_kv, int max_chunks, float scale_log2_in, int* status,
                   const float* __restrict__ kv_scale, const int* __restrict__ plan, const float* __restrict__ k_ts, const float* __restrict__ v_ts,
                   const int* __restrict__ vbt) {
  static_assert(!I8 || FP8, "the int8 cache uses the byte-page path");
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int T16 = PAGE * HD * 2;
  constexpr int TILE = FP8 ? PAGE * HD : T16;       // bytes of one stage of K (or V)
  uint8_t* conv = smem + 2 * KV_STAGES * TILE;       // FP8: the expanded fp16 K and V tiles of the page being processed
  uint64_t* bars = (uint64_t*)(smem + dec_region_bytes(HD, FP8, MT));
  volatile int* abort_flag = (volatile int*)(bars + KV_STAGES);
  float* tsc = (float*)(bars + 8) + MT * 4 * 16 * 2 + 32;    // int8 cache: per stage 64 K scales then 64 V scales (behind the merge bookkeeping)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kw = warp;                               // this warp's 16-key slice of every page
  const int G = n_q / n_kv;
  const int total = plan[0], nb = plan[1];
  const int* blk_row = plan + PLAN_HEAD;
  const int* blk_n = blk_row + PLAN_MAX_ROWS;
  const int* prefix = blk_n + 2 * PLAN_MAX_ROWS;
  const int* blk_seq = prefix + PLAN_MAX_ROWS + 1;
  const int* blk_c0 = blk_seq + PLAN_MAX_ROWS;
  if ((int)blockIdx.x >= total) return;
  if (threadIdx.x == 0) {
    for (int i = 0; i < KV_STAGES; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  int gp = 0;                                        // pages this CTA has consumed so far: stage and barrier phase follow it
  for (int item = blockIdx.x; item < total; item += gridDim.x) {
    int lo = 0, hi = nb - 1;                         // the block whose item range holds `item`
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (prefix[mid] <= item) lo = mid; else hi = mid - 1;
    }
    const int local = item - prefix[lo];
    const int row = blk_row[lo], nblk = blk_n[lo], kvh = local % n_kv, chunk = blk_c0[lo] + local / n_kv;
    const int seq = blk_seq[lo];
    const float scale_log2 = (FP8 && !I8) ? scale_log2_in * kv_scale[kvh] : scale_log2_in;     // K was stored as k / k_scale
    const float v_scale = (FP8 && !I8) ? kv_scale[n_kv + kvh] : 1.f;
    int ctx_max = 0;
    for (int i = 0; i < nblk; ++i) ctx_max = max(ctx_max, ctx_len[row + i]);
    const int k_begin = chunk * DEC_CHUNK;
    const int k_end_max = min(ctx_max, k_begin + DEC_CHUNK);
    const int npages = (k_end_max - k_begin + PAGE - 1) / PAGE;
    const int ntiles = (nblk * G + 15) >> 4;            // tiles that hold a live row
    // a tree row's private table starts at the page index of its block's first chunk
    const int* bt = seq >= 0 ? block_table + (size_t)seq * max_blocks : vbt + (size_t)(-1 - seq) * VBT_W - blk_c0[lo] * (DEC_CHUNK / PAGE);
    if (threadIdx.x == 0) {
      fence_proxy_async();                           // the previous item's merge wrote this memory with plain stores
      for (int p = 0; p < npages && p < KV_STAGES - 1; ++p) {
        const int sg = (gp + p) % KV_STAGES;
        if constexpr (I8 == 2) load_kv_page_q4<HD>(smem + sg * TILE, smem + (KV_STAGES + sg) * TILE, (uint8_t*)(tsc + sg * 2 * PAGE), &tk, &tv, (const uint8_t*)k_ts, (const uint8_t*)v_ts, bt[k_begin / PAGE + p], kvh, n_kv, &bars[sg]);
        else if constexpr (I8 == 1) load_kv_page_i8<HD>(smem + sg * TILE, smem + (KV_STAGES + sg) * TILE, tsc + sg * 2 * PAGE, &tk, &tv, k_ts, v_ts, bt[k_begin / PAGE + p], kvh, n_kv, &bars[sg]);
        else if constexpr (FP8) load_kv_page8<HD>(smem + sg * TILE, smem + (KV_STAGES + sg) * TILE, &tk, &tv, bt[k_begin / PAGE + p], kvh, n_kv, &bars[sg]);
        else load_kv_page<HD>(smem + sg * TILE, smem + (KV_STAGES + sg) * TILE, &tk, &tv, bt[k_begin / PAGE + p], kvh, n_kv, &bars[sg]);
      }
    }
    // the two rows of this lane in every tile: (block row, head) and the last key + 1 that row may see inside this chunk
    int kend[MT][2];
    // Q fragments straight from global: tile row t = (block row t / G, query head t % G of this KV head)
    uint32_t qa[MT][HD / 16][4];
    float m[MT][2], l[MT][2];
    float o[MT][HD / 8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      bool live[2];
      const uint16_t* qrow[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int t = mt * 16 + (lane >> 2) + 8 * r, rb = t / G, hh = t % G;
        live[r] = rb < nblk;
        kend[mt][r] = live[r] ? min(ctx_len[row + rb], k_begin + DEC_CHUNK) : 0;
        qrow[r] = q + ((size_t)(row + (live[r] ? rb : 0)) * n_q + (size_t)kvh * G + hh) * HD;
      }
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const int c = ks * 16 + 2 * (lane & 3);
        qa[mt][ks][0] = live[0] ? *reinterpret_cast<const uint32_t*>(qrow[0] + c) : 0u;
        qa[mt][ks][1] = live[1] ? *reinterpret_cast<const uint32_t*>(qrow[1] + c) : 0u;
        qa[mt][ks][2] = live[0] ? *reinterpret_cast<const uint32_t*>(qrow[0] + c + 8) : 0u;
        qa[mt][ks][3] = live[1] ? *reinterpret_cast<const uint32_t*>(qrow[1] + c + 8) : 0u;
        if constexpr (FP8) {
#pragma unroll
          for (int i = 0; i < 4; ++i) qa[mt][ks][i] = bf16x2_to_f16x2(qa[mt][ks][i]);
        }
      }
      m[mt][0] = m[mt][1] = -INFINITY;
      l[mt][0] = l[mt][1] = 0.f;
#pragma unroll
      for (int d = 0; d < HD / 8; ++d) { o[mt][d][0] = o[mt][d][1] = o[mt][d][2] = o[mt][d][3] = 0.f; }
    }

    bool ok = true;
    for (int p = 0; p < npages; ++p) {
      const int s = (gp + p) % KV_STAGES;
      if (threadIdx.x == 0 && p + KV_STAGES - 1 < npages) {
        const int pn = p + KV_STAGES - 1, sn = (gp + pn) % KV_STAGES;  // stage sn was consumed in iteration p-1 (barrier below)
        if constexpr (I8 == 2) load_kv_page_q4<HD>(smem + sn * TILE, smem + (KV_STAGES + sn) * TILE, (uint8_t*)(tsc + sn * 2 * PAGE), &tk, &tv, (const uint8_t*)k_ts, (const uint8_t*)v_ts, bt[k_begin / PAGE + pn], kvh, n_kv, &bars[sn]);
        else if constexpr (I8 == 1) load_kv_page_i8<HD>(smem + sn * TILE, smem + (KV_STAGES + sn) * TILE, tsc + sn * 2 * PAGE, &tk, &tv, k_ts, v_ts, bt[k_begin / PAGE + pn], kvh, n_kv, &bars[sn]);
        else if constexpr (FP8) load_kv_page8<HD>(smem + sn * TILE, smem + (KV_STAGES + sn) * TILE, &tk, &tv, bt[k_begin / PAGE + pn], kvh, n_kv, &bars[sn]);
        else load_kv_page<HD>(smem + sn * TILE, smem + (KV_STAGES + sn) * TILE, &tk, &tv, bt[k_begin / PAGE + pn], kvh, n_kv, &bars[sn]);
      }
      ok = mbar_wait(&bars[s], ((gp + p) / KV_STAGES) & 1, abort_flag, status, 50);
      if (!ok) break;
      const int key0 = kw * 16;
      const int kpos = k_begin + p * PAGE + key0;
      const bool any = k_end_max - kpos > 0;                        // uniform for the warp
      if constexpr (FP8) {
        if constexpr (I8 == 2) {
          expand_page4<HD>(smem + s * TILE, conv, (const uint8_t*)(tsc + s * 2 * PAGE));
          expand_page4<HD>(smem + (KV_STAGES + s) * TILE, conv + T16, (const uint8_t*)(tsc + s * 2 * PAGE + PAGE));
        } else {
          expand_page8<HD>(smem + s * TILE, conv, I8 ? tsc + s * 2 * PAGE : nullptr);
          expand_page8<HD>(smem + (KV_STAGES + s) * TILE, conv + T16, I8 ? tsc + s * 2 * PAGE + PAGE : nullptr);
        }
        __syncthreads();
      }
      if (any) {
        int valid[MT][2];                                           // per tile row: keys of this 16-key slice the row may see
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) { valid[mt][0] = kend[mt][0] - kpos; valid[mt][1] = kend[mt][1] - kpos; }
        if constexpr (FP8) attn_step_mt<HD, MT, true>(qa, smem_u32(conv), smem_u32(conv + T16), key0, valid, ntiles, scale_log2, m, l, o);
        else attn_step_mt<HD, MT, false>(qa, smem_u32(smem + s * TILE), smem_u32(smem + (KV_STAGES + s) * TILE), key0, valid, ntiles, scale_log2, m, l, o);
      }
      fence_proxy_async();      // this page was read with ordinary loads; the refill of its stage (next iteration) writes through the async proxy
      __syncthreads();
    }
    if (!ok || *abort_flag != 0) return;
    gp += npages;
    // merge the 4 warps (key slices) through shared memory; the stages are free now: the last iteration ended with a barrier
    constexpr int HDP = HD + 8;                       // padded row: the float2 stores of a warp then spread over all banks
    float* sm_o = (float*)smem;                       // [tile][key slice][16][HDP]
    float* sm_ml = (float*)(bars + 8);                // [tile][key slice][16][2], behind the barriers
    int* s_ctx = (int*)(sm_ml + MT * 4 * 16 * 2);     // context length of each row of the block
    const int r0 = lane >> 2, c0 = 2 * (lane & 3);
    if ((int)threadIdx.x < nblk) s_ctx[threadIdx.x] = ctx_len[row + threadIdx.x];
    // 1. every warp publishes its rows' running maxima and keeps the quad-reduced sums
    float ls[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int wslot = mt * 4 + warp;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        ls[mt][r] = l[mt][r];
        ls[mt][r] += __shfl_xor_sync(0xffffffffu, ls[mt][r], 1);
        ls[mt][r] += __shfl_xor_sync(0xffffffffu, ls[mt][r], 2);
      }
      if ((lane & 3) == 0) {
        sm_ml[(wslot * 16 + r0) * 2] = m[mt][0];
        sm_ml[(wslot * 16 + r0 + 8) * 2] = m[mt][1];
      }
    }
    __syncthreads();
    // 2. rescale the own partial to the row's maximum over the four slices, then publish it
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int wslot = mt * 4 + warp;
      float f[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int tr = r0 + 8 * r;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_ml[((mt * 4 + w) * 16 + tr) * 2]);
        f[r] = (m[mt][r] == -INFINITY) ? 0.f : exp2f(m[mt][r] - mm);
      }
      float* base = sm_o + ((size_t)wslot * 16) * HDP + c0;
#pragma unroll
      for (int d = 0; d < HD / 8; ++d) {
        *reinterpret_cast<float2*>(base + (size_t)r0 * HDP + d * 8) = make_float2(o[mt][d][0] * f[0], o[mt][d][1] * f[0]);
        *reinterpret_cast<float2*>(base + (size_t)(r0 + 8) * HDP + d * 8) = make_float2(o[mt][d][2] * f[1], o[mt][d][3] * f[1]);
      }
      if ((lane & 3) == 0) {
        sm_ml[(wslot * 16 + r0) * 2 + 1] = ls[mt][0] * f[0];
        sm_ml[(wslot * 16 + r0 + 8) * 2 + 1] = ls[mt][1] * f[1];
      }
    }
    __syncthreads();
    // 3. sum the four slices in slice order, four outputs per thread
    for (int idx = threadIdx.x; idx < nblk * G * (HD / 4); idx += blockDim.x) {
      const int t = idx / (HD / 4), d4 = (idx % (HD / 4)) * 4;          // tile row = (block row, head)
      const int rb = t / G, hq = t % G;
      if (s_ctx[rb] <= k_begin) continue;            // this chunk lies beyond that row's context: nothing of it is ever read
      const int wb = (t >> 4) * 4, tr = t & 15;      // the four key-slice warps of the row's tile
      float4 acc = *reinterpret_cast<const float4*>(sm_o + ((size_t)wb * 16 + tr) * HDP + d4);
#pragma unroll
      for (int w = 1; w < 4; ++w) {
        const float4 v = *reinterpret_cast<const float4*>(sm_o + ((size_t)(wb + w) * 16 + tr) * HDP + d4);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      const size_t pidx = ((size_t)(row + rb) * n_q + (size_t)kvh * G + hq) * max_chunks + chunk;
      *reinterpret_cast<float4*>(part_o + pidx * HD + d4) = make_float4(acc.x * v_scale, acc.y * v_scale, acc.z * v_scale, acc.w * v_scale);
      if (d4 == 0) {
        float mm = -INFINITY, lsum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          mm = fmaxf(mm, sm_ml[((wb + w) * 16 + tr) * 2]);
          lsum += sm_ml[((wb + w) * 16 + tr) * 2 + 1];
        }
        part_ml[pidx * 2] = mm;
        part_ml[pidx * 2 + 1] = lsum;
      }
    }
    __syncthreads();                                  // the next item's loads overwrite the merge scratch
  }
}

// Merge chunk partials in chunk order -> attention output; then (suh != nullptr) xr = fp16(H(out * suh)) per 128-block
// (the o_proj input rotation), else plain bf16 output.  One warp per 128 output elements.
template <int HD>
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ ctx_len, int n_q,
                                  int max_chunks, const __half* __restrict__ suh, __half* __restrict__ xr, uint16_t* __restrict__ out_bf16) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int nch = (ctx_len[row] + DEC_CHUNK - 1) / DEC_CHUNK;
  const int width = n_q * HD;
  for (int b = blockIdx.y * nw + warp; b < width / 128; b += gridDim.y * nw) {
    const int e0 = b * 128 + lane * 4;
    const int hq = e0 / HD, d0 = e0 % HD;
    const size_t base = ((size_t)row * n_q + hq) * max_chunks;
    // GL chunks at a time (GL = lanes that share this head): lane c of the group fetches chunk c's (max, sum), the group reduces
    // the max, then every lane walks the chunks in order with the factors broadcast by shuffle and the partial-output loads
    // issued four at a time
    constexpr int GL = HD / 4 < 32 ? HD / 4 : 32;
    const int gl = lane % GL, gbase = lane - gl;
    float mm = -INFINITY;
    for (int c0 = 0; c0 < nch; c0 += GL) {
      float m_l = (c0 + gl < nch) ? part_ml[(base + c0 + gl) * 2] : -INFINITY;
#pragma unroll
      for (int o = GL / 2; o > 0; o >>= 1) m_l = fmaxf(m_l, __shfl_xor_sync(0xffffffffu, m_l, o));
      mm = fmaxf(mm, m_l);
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, lsum = 0.f;
    for (int c0 = 0; c0 < nch; c0 += GL) {
      const bool in = c0 + gl < nch;
      const float m_l = in ? part_ml[(base + c0 + gl) * 2] : -INFINITY;
      const float l_l = in ? part_ml[(base + c0 + gl) * 2 + 1] : 0.f;
      const float f_l = (m_l == -INFINITY) ? 0.f : exp2f(m_l - mm);
      const int cnt = min(GL, nch - c0);
      for (int j0 = 0; j0 < cnt; j0 += 4) {
        float4 p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j0 + j < cnt) p[j] = *reinterpret_cast<const float4*>(part_o + (base + c0 + j0 + j) * HD + d0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int src = gbase + ((j0 + j) % GL);
          const float f = __shfl_sync(0xffffffffu, f_l, src), ll = __shfl_sync(0xffffffffu, l_l, src);
          if (j0 + j < cnt) {
            acc[0] += f * p[j].x; acc[1] += f * p[j].y; acc[2] += f * p[j].z; acc[3] += f * p[j].w;
            lsum += f * ll;
          }
        }
      }
    }
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat16 t = __float2bfloat16_rn(acc[i] * inv);
      v[i] = __bfloat162float(t);
    }
    if (out_bf16 != nullptr) {
      uint2 u;
      u.x = pack_bf16(v[0], v[1]); u.y = pack_bf16(v[2], v[3]);
      *reinterpret_cast<uint2*>(out_bf16 + (size_t)row * width + e0) = u;
    }
    if (suh != nullptr) {
      const uint2 su = *reinterpret_cast<const uint2*>(suh + e0);
      const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
      v[0] *= s01.x; v[1] *= s01.y; v[2] *= s23.x; v[3] *= s23.y;
      fwht128_warp(v);
      const __half2 a = __floats2half2_rn(v[0], v[1]), c2 = __floats2half2_rn(v[2], v[3]);
      uint2 u;
      u.x = *reinterpret_cast<const uint32_t*>(&a); u.y = *reinterpret_cast<const uint32_t*>(&c2);
      *reinterpret_cast<uint2*>(xr + (size_t)row * width + e0) = u;
    }
  }
}

// ------------------------------------------------------------------------------------------------ prefill (causal flash)
// Queries: rows [q_start[s], q_start[s] + q_len[s]) of `q` belong to sequence s at positions pos0[s].. ; keys are the
// sequence's cached tokens [0, pos0 + local row] (the chunk's own K/V are already in the cache).  out: bf16 [rows][n_q*HD].
template <int HD, bool FP8, int I8 = 0>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv, const uint16_t* __restrict__ q,
                    const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_ids, const int* __restrict__ q_start,
                    const int* __restrict__ q_len, const int* __restrict__ pos0, uint16_t* __restrict__ out, int n_q, int n_kv, float scale_log2_in,
                    int* status, const float* __restrict__ kv_scale, const float* __restrict__ k_ts, const float* __restrict__ v_ts) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int T16 = PAGE * HD * 2;
  constexpr int TILE = FP8 ? PAGE * HD : T16;
  uint8_t* conv = smem + 2 * KV_STAGES * TILE;
  uint64_t* bars = (uint64_t*)(conv + (FP8 ? 2 * T16 : 0));
  volatile int* abort_flag = (volatile int*)(bars + KV_STAGES);
  float* tsc = (float*)(bars + 8);                   // int8 cache: per stage 64 K scales then 64 V scales
  const int s_idx = blockIdx.z, hq = blockIdx.y;
  const int qlen = q_len[s_idx];
  // heaviest (latest) query tiles first
  const int ntiles = (qlen + 63) / 64;
  const int qt = ntiles - 1 - (int)blockIdx.x;
  if (qt < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = n_q / n_kv, kvh = hq / G;
  const float scale_log2 = (FP8 && !I8) ? scale_log2_in * kv_scale[kvh] : scale_log2_in;
  const float v_scale = (FP8 && !I8) ? kv_scale[n_kv + kvh] : 1.f;
  const int p0 = pos0[s_idx], r_base = q_start[s_idx];
  const int* bt = block_table + (size_t)seq_ids[s_idx] * max_blocks;
  const int q_lo = qt * 64;
  const int last_q = min(qlen, q_lo + 64) - 1;
  const int npages = (p0 + last_q) / PAGE + 1;  // keys 0 .. p0 + last_q

  if (threadIdx.x == 0) {
    for (int i = 0; i < KV_STAGES; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int p = 0; p < npages && p < KV_STAGES - 1; ++p) {
      if constexpr (I8 == 2) load_kv_page_q4<HD>(smem + p * TILE, smem + (KV_STAGES + p) * TILE, (uint8_t*)(tsc + p * 2 * PAGE), &tk, &tv, (const uint8_t*)k_ts, (const uint8_t*)v_ts, bt[p], kvh, n_kv, &bars[p]);
        else if constexpr (I8 == 1) load_kv_page_i8<HD>(smem + p * TILE, smem + (KV_STAGES + p) * TILE, tsc + p * 2 * PAGE, &tk, &tv, k_ts, v_ts, bt[p], kvh, n_kv, &bars[p]);
      else if constexpr (FP8) load_kv_page8<HD>(smem + p * TILE, smem + (KV_STAGES + p) * TILE, &tk, &tv, bt[p], kvh, n_kv, &bars[p]);
      else load_kv_page<HD>(smem + p * TILE, smem + (KV_STAGES + p) * TILE, &tk, &tv, bt[p], kvh, n_kv, &bars[p]);
    }
  }
  uint32_t qa[HD / 16][4];
  const int lr0 = q_lo + warp * 16 + (lane >> 2), lr1 = lr0 + 8;  // local query rows of this lane
  {
    const uint16_t* q0 = q + ((size_t)(r_base + lr0) * n_q + hq) * HD;
    const uint16_t* q1 = q + ((size_t)(r_base + lr1) * n_q + hq) * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const int c = ks * 16 + 2 * (lane & 3);
      qa[ks][0] = lr0 < qlen ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
      qa[ks][1] = lr1 < qlen ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
      qa[ks][2] = lr0 < qlen ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
      qa[ks][3] = lr1 < qlen ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
      if constexpr (FP8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) qa[ks][i] = bf16x2_to_f16x2(qa[ks][i]);
      }
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
  const int warp_last_key = p0 + min(qlen - 1, q_lo + warp * 16 + 15);  // last key any row of this warp may see

  bool ok = true;
  for (int p = 0; p < npages; ++p) {
    const int s = p % KV_STAGES;
    if (threadIdx.x == 0 && p + KV_STAGES - 1 < npages) {
      const int pn = p + KV_STAGES - 1, sn = pn % KV_STAGES;
      if constexpr (I8 == 2) load_kv_page_q4<HD>(smem + sn * TILE, smem + (KV_STAGES + sn) * TILE, (uint8_t*)(tsc + sn * 2 * PAGE), &tk, &tv, (const uint8_t*)k_ts, (const uint8_t*)v_ts, bt[pn], kvh, n_kv, &bars[sn]);
        else if constexpr (I8 == 1) load_kv_page_i8<HD>(smem + sn * TILE, smem + (KV_STAGES + sn) * TILE, tsc + sn * 2 * PAGE, &tk, &tv, k_ts, v_ts, bt[pn], kvh, n_kv, &bars[sn]);
      else if constexpr (FP8) load_kv_page8<HD>(smem + sn * TILE, smem + (KV_STAGES + sn) * TILE, &tk, &tv, bt[pn], kvh, n_kv, &bars[sn]);
      else load_kv_page<HD>(smem + sn * TILE, smem + (KV_STAGES + sn) * TILE, &tk, &tv, bt[pn], kvh, n_kv, &bars[sn]);
    }
    ok = mbar_wait(&bars[s], (p / KV_STAGES) & 1, abort_flag, status, 60);
    if (!ok) break;
    const int kbase = p * PAGE;
    const bool mine = kbase <= warp_last_key && q_lo + warp * 16 < qlen;
    const int v0 = lr0 < qlen ? (p0 + lr0 + 1 - kbase) : 0, v1 = lr1 < qlen ? (p0 + lr1 + 1 - kbase) : 0;
    if constexpr (FP8) {
      if constexpr (I8 == 2) {
        expand_page4<HD>(smem + s * TILE, conv, (const uint8_t*)(tsc + s * 2 * PAGE));
        expand_page4<HD>(smem + (KV_STAGES + s) * TILE, conv + T16, (const uint8_t*)(tsc + s * 2 * PAGE + PAGE));
      } else {
        expand_page8<HD>(smem + s * TILE, conv, I8 ? tsc + s * 2 * PAGE : nullptr);
        expand_page8<HD>(smem + (KV_STAGES + s) * TILE, conv + T16, I8 ? tsc + s * 2 * PAGE + PAGE : nullptr);
      }
      __syncthreads();
      if (mine) attn_step<HD, 64, true>(qa, smem_u32(conv), smem_u32(conv + T16), 0, v0, v1, scale_log2, m, l, o);
    } else {
      if (mine) attn_step<HD, 64>(qa, smem_u32(smem + s * TILE), smem_u32(smem + (KV_STAGES + s) * TILE), 0, v0, v1, scale_log2, m, l, o);
    }
    fence_proxy_async();        // ordinary loads of this page before the async-proxy refill of its stage
    __syncthreads();
  }
  if (!ok || *abort_flag != 0) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  const float i0 = l[0] > 0.f ? v_scale / l[0] : 0.f, i1 = l[1] > 0.f ? v_scale / l[1] : 0.f;
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) {
    const int c = d * 8 + 2 * (lane & 3);
    if (lr0 < qlen) *reinterpret_cast<uint32_t*>(out + ((size_t)(r_base + lr0) * n_q + hq) * HD + c) = pack_bf16(o[d][0] * i0, o[d][1] * i0);
    if (lr1 < qlen) *reinterpret_cast<uint32_t*>(out + ((size_t)(r_base + lr1) * n_q + hq) * HD + c) = pack_bf16(o[d][2] * i1, o[d][3] * i1);
  }
}


// ------------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn att_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

static int att_smem_bytes(int hd, bool fp8 = false) {
  return (fp8 ? 2 * KV_STAGES * PAGE * hd + 2 * PAGE * hd * 2 : 2 * KV_STAGES * PAGE * hd * 2) + 64 + KV_STAGES * 2 * PAGE * 4 + 1024;
}

}  // namespace rx

using namespace rx;

// Writes a 128-byte tensor map for a bf16 cache [num_pages][n_kv][64][hd] viewed as 2-D [num_pages*n_kv*64, hd].
RX_API int rx_make_kv_tmap(void* out128, const void* base, long long total_rows, int hd) {
  EncodeTiledFn enc = att_encode_tiled();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  if (hd % 64 != 0 || (((uintptr_t)base) & 127) != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)total_rows};
  cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
  cuuint32_t box[2] = {64, PAGE};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc((CUtensorMap*)out128, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Tensor map of an FP8 (E4M3) cache [num_pages][n_kv][64][hd] viewed as bytes [num_pages*n_kv*64, hd]; one page of one head is one box.
RX_API int rx_make_kv_tmap8(void* out128, const void* base, long long total_rows, int hd) {
  EncodeTiledFn enc = att_encode_tiled();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  if (hd % 64 != 0 || hd > 256 || (((uintptr_t)base) & 127) != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)total_rows};
  cuuint64_t strides[1] = {(cuuint64_t)hd};
  cuuint32_t box[2] = {(cuuint32_t)hd, PAGE};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc((CUtensorMap*)out128, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

RX_API int rx_attn_decode_chunk() { return DEC_CHUNK; }

// tiles per CTA for the longest run of rows one sequence has in a window (all of its (row, head) pairs in one pass over K / V where two
// tiles hold them), and the rows of one sequence a CTA then takes
static int dec_tiles(int max_seq_rows, int G) { return (max_seq_rows > 1 ? max_seq_rows * G + 15 : 16) / 16 > 1 ? 2 : 1; }
static int dec_rows_per_block(int tiles, int G) { return 16 * tiles / G > 0 ? 16 * tiles / G : 1; }
static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// scratch sizes (floats) for `rows` rows and contexts up to max_ctx
RX_API long long rx_attn_decode_scratch_floats(int rows, int n_q, int hd, int max_ctx) {
  const long long mc = (max_ctx + DEC_CHUNK - 1) / DEC_CHUNK;
  return PLAN_INTS + (long long)rows * n_q * mc * (hd + 2);
}
RX_API int rx_attn_plan_ints() { return PLAN_INTS; }

// The window plan of a decode / verify step (see attn_plan_kernel): computed once per forward from row_seq and ctx_len and handed to every
// layer's rx_attn_decode call of that forward (same rows, n_q, n_kv and max_seq_rows).
// tree_base: nullptr for a chain window; int32 [rows] for a tree window (see attn_plan_kernel), whose plan holds up to two blocks per row.
RX_API int rx_attn_plan(const void* row_seq, const void* ctx_len, int rows, int n_q, int n_kv, int max_seq_rows, void* plan, void* stream,
                        const void* tree_base) {
  if (rows <= 0 || rows > PLAN_MAX_ROWS || n_kv <= 0 || n_q % n_kv != 0 || n_q / n_kv > 16) return (int)cudaErrorInvalidValue;
  if (tree_base != nullptr && 2 * rows > PLAN_MAX_ROWS) return (int)cudaErrorInvalidValue;
  const int G = n_q / n_kv;
  rx::launch(attn_plan_kernel, dim3(1), dim3(256), 0, (cudaStream_t)stream, (const int*)row_seq, (const int*)ctx_len, rows,
             dec_rows_per_block(dec_tiles(max_seq_rows, G), G), n_kv, (int*)plan, (const int*)tree_base);
  return (int)cudaGetLastError();
}
RX_API int rx_attn_vbt_width() { return VBT_W; }

template <int HD, bool FP8, int MT, int I8>
static int launch_decode_kernel(const CUtensorMap* tk, const CUtensorMap* tv, const void* q, const int* bt, int max_blocks, const int* row_seq,
                                const int* ctx_len, float* part_o, float* part_ml, int rows, int n_q, int n_kv, int mc, float scale, int* status,
                                cudaStream_t st, const float* kv_scale, const int* plan, const float* k_ts, const float* v_ts, const int* vbt) {
  constexpr int smem = dec_smem_bytes(HD, FP8, MT);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, FP8, MT, I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // persistent: two CTAs per SM at most, never more than the items the window can have
  const long long bound = (long long)rows * n_kv * mc;
  const int grid = (int)(bound < 2 * sm_count() ? bound : 2 * sm_count());
  rx::launch(attn_decode_kernel<HD, FP8, MT, I8>, dim3(grid), dim3(ATT_THREADS), smem, st, *tk, *tv, (const uint16_t*)q, bt, max_blocks, row_seq,
             ctx_len, part_o, part_ml, n_q, n_kv, mc, scale * 1.4426950408889634f, status, kv_scale, plan, k_ts, v_ts, vbt);
  return (int)cudaGetLastError();
}

template <int HD, bool FP8, int I8 = 0>
static int launch_decode(const CUtensorMap* tk, const CUtensorMap* tv, const void* q, const int* bt, int max_blocks, const int* row_seq,
                         const int* ctx_len, float* scratch, int rows, int n_q, int n_kv, int max_ctx, float scale, const void* suh, void* xr,
                         void* out_bf16, int* status, cudaStream_t st, const float* kv_scale, int max_seq_rows, const int* plan,
                         const float* k_ts = nullptr, const float* v_ts = nullptr, const int* vbt = nullptr) {
  const int mc = (max_ctx + DEC_CHUNK - 1) / DEC_CHUNK;
  int* own_plan = (int*)scratch;                    // the head of the scratch holds a plan for callers that bring none
  float* part_o = scratch + PLAN_INTS;
  float* part_ml = part_o + (size_t)rows * n_q * mc * HD;
  // tiles per CTA: enough for the longest run of rows one sequence has in this window (all of its (row, head) pairs in one pass over K / V)
  const int G = n_q / n_kv;
  const int tiles = dec_tiles(max_seq_rows, G);
  if (plan == nullptr) {
    rx::launch(attn_plan_kernel, dim3(1), dim3(256), 0, st, row_seq, ctx_len, rows, dec_rows_per_block(tiles, G), n_kv, own_plan, (const int*)nullptr);
    plan = own_plan;
  }
  int e;
#define RX_DEC_T(MT) launch_decode_kernel<HD, FP8, MT, I8>(tk, tv, q, bt, max_blocks, row_seq, ctx_len, part_o, part_ml, rows, n_q, n_kv, mc, scale, status, st, kv_scale, plan, k_ts, v_ts, vbt)
  if (tiles <= 1) e = RX_DEC_T(1);
  else e = RX_DEC_T(2);
#undef RX_DEC_T
  if (e != 0) return e;
  const int blocks128 = n_q * HD / 128;
  int gy = (296 + rows - 1) / rows;
  if (gy > (blocks128 + 3) / 4) gy = (blocks128 + 3) / 4;
  if (gy < 1) gy = 1;
  rx::launch(attn_merge_kernel<HD>, dim3(dim3(rows, gy)), dim3(128), 0, st, part_o, part_ml, ctx_len, n_q, mc, (const __half*)suh, (__half*)xr, (uint16_t*)out_bf16);
  return (int)cudaGetLastError();
}

// q: bf16 [rows][n_q*hd] (already rotated by RoPE).  Either/both outputs: xr = fp16(H(out*suh)) [rows][n_q*hd], out_bf16.
// max_seq_rows: the most adjacent rows any one sequence has in this launch (1 = plain decode; a verify window's 1 + drafts); it only
// picks how many MMA tiles a CTA carries, results do not depend on it.  plan: rx_attn_plan's output for this window (same max_seq_rows), or
// nullptr to have it computed here into the head of the scratch.
RX_API int rx_attn_decode(const void* tmap_k, const void* tmap_v, const void* q, const void* block_table, int max_blocks, const void* row_seq,
                          const void* ctx_len, void* scratch, int rows, int n_q, int n_kv, int hd, int max_ctx, float scale, const void* suh,
                          void* xr, void* out_bf16, int* status, void* stream, const void* kv_scale, int max_seq_rows, const void* plan,
                          const void* k_tscale, const void* v_tscale, const void* vbt) {
  // vbt: int32 [rows][rx_attn_vbt_width()], the private page tables of a tree window whose `plan` was made with tree_base; nullptr otherwise
  if (vbt != nullptr && plan == nullptr) return (int)cudaErrorInvalidValue;
  if (n_q % n_kv != 0 || n_q / n_kv > 16 || (n_q * hd) % 128 != 0 || rows <= 0 || rows > PLAN_MAX_ROWS || max_ctx <= 0) return (int)cudaErrorInvalidValue;
  if ((k_tscale == nullptr) != (v_tscale == nullptr) || (k_tscale != nullptr && kv_scale != nullptr)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  if (k_tscale != nullptr) {
    // int8 cache: the maps describe byte pages, k_tscale / v_tscale are f32 [pages][n_kv][64] (one power-of-two scale per token and KV head)
#define RX_DEC8(HDV) launch_decode<HDV, true, 1>((const CUtensorMap*)tmap_k, (const CUtensorMap*)tmap_v, q, (const int*)block_table, max_blocks, \
    (const int*)row_seq, (const int*)ctx_len, (float*)scratch, rows, n_q, n_kv, max_ctx, scale, suh, xr, out_bf16, status, st, nullptr, max_seq_rows, \
    (const int*)plan, (const float*)k_tscale, (const float*)v_tscale, (const int*)vbt)
    if (hd == 128) return RX_DEC8(128);
    if (hd == 64) return RX_DEC8(64);
#undef RX_DEC8
    return (int)cudaErrorInvalidValue;
  }
  // kv_scale != nullptr: the maps describe an FP8 cache and kv_scale is f32 [2][n_kv] (K scales, then V scales) of this layer
#define RX_DEC(HDV, F8) launch_decode<HDV, F8>((const CUtensorMap*)tmap_k, (const CUtensorMap*)tmap_v, q, (const int*)block_table, max_blocks, \
    (const int*)row_seq, (const int*)ctx_len, (float*)scratch, rows, n_q, n_kv, max_ctx, scale, suh, xr, out_bf16, status, st, (const float*)kv_scale, \
    max_seq_rows, (const int*)plan, nullptr, nullptr, (const int*)vbt)
  if (hd == 128) return kv_scale ? RX_DEC(128, true) : RX_DEC(128, false);
  if (hd == 64) return kv_scale ? RX_DEC(64, true) : RX_DEC(64, false);
#undef RX_DEC
  return (int)cudaErrorInvalidValue;
}

// Copies runs of KV rows inside the paged caches: moves int32 [n_moves][3] = (source slot, destination slot, rows), slot = page * 64 + offset, a
// run stays inside one page on both sides; tensors = the base addresses of n_tensors caches laid out [pages][n_kv][64][row_bytes].  No
// destination row of one move may be a source or destination row of another (the moves run in parallel).  Used by tree windows: before a
// layer's attention the committed rows and the ancestors of each node are copied into the node's private pages, and after the window the
// accepted path's rows are copied to their positions.
__global__ void __launch_bounds__(128) kv_move_rows_kernel(const unsigned long long* __restrict__ tensors, int row_bytes, int n_kv, const int* __restrict__ moves) {
  pdl_launch();
  pdl_wait();
  uint8_t* base = (uint8_t*)tensors[blockIdx.z];
  const int h = blockIdx.y;
  const int src = moves[3 * blockIdx.x], dst = moves[3 * blockIdx.x + 1], n = moves[3 * blockIdx.x + 2];
  const uint8_t* sp = base + (((size_t)(src / PAGE) * n_kv + h) * PAGE + src % PAGE) * row_bytes;
  uint8_t* dp = base + (((size_t)(dst / PAGE) * n_kv + h) * PAGE + dst % PAGE) * row_bytes;
  if (row_bytes % 16 == 0) {
    for (int c = threadIdx.x * 16; c < n * row_bytes; c += blockDim.x * 16)
      *reinterpret_cast<uint4*>(dp + c) = *reinterpret_cast<const uint4*>(sp + c);
  } else {            // the per-token scale planes of the int8 cache: 4 bytes per row
    for (int c = threadIdx.x * 4; c < n * row_bytes; c += blockDim.x * 4)
      *reinterpret_cast<uint32_t*>(dp + c) = *reinterpret_cast<const uint32_t*>(sp + c);
  }
}

RX_API int rx_kv_move_rows(const void* tensors, int n_tensors, int row_bytes, int n_kv, const void* moves, int n_moves, void* stream) {
  if (n_tensors <= 0 || n_tensors > 65535 || n_kv <= 0 || n_kv > 65535 || row_bytes <= 0 || row_bytes % 4 != 0 || n_moves < 0) return (int)cudaErrorInvalidValue;
  if (n_moves == 0) return 0;
  rx::launch(kv_move_rows_kernel, dim3(n_moves, n_kv, n_tensors), dim3(128), 0, (cudaStream_t)stream, (const unsigned long long*)tensors, row_bytes, n_kv,
             (const int*)moves);
  return (int)cudaGetLastError();
}

template <int HD, bool FP8, int I8 = 0>
static int launch_prefill(const CUtensorMap* tk, const CUtensorMap* tv, const void* q, const int* bt, int max_blocks, const int* seq_ids,
                          const int* q_start, const int* q_len, const int* pos0, void* out, int nseq, int max_qlen, int n_q, int n_kv, float scale,
                          int* status, cudaStream_t st, const float* kv_scale, const float* k_ts = nullptr, const float* v_ts = nullptr) {
  const int smem = att_smem_bytes(HD, FP8);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD, FP8, I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((max_qlen + 63) / 64, n_q, nseq);
  rx::launch(attn_prefill_kernel<HD, FP8, I8>, dim3(grid), dim3(ATT_THREADS), smem, st, *tk, *tv, (const uint16_t*)q, bt, max_blocks, seq_ids, q_start, q_len, pos0,
                                                          (uint16_t*)out, n_q, n_kv, scale * 1.4426950408889634f, status, kv_scale, k_ts, v_ts);
  return (int)cudaGetLastError();
}

// q4 cache (head dim 128): the maps describe [pages * n_kv * 64][64] byte pages (rx_make_kv_tmap8 with width 64), k_s4 / v_s4 are the E8M0
// scale bytes uint8 [pages][n_kv][64][4].
RX_API int rx_attn_decode_q4(const void* tmap_k, const void* tmap_v, const void* q, const void* block_table, int max_blocks, const void* row_seq,
                             const void* ctx_len, void* scratch, int rows, int n_q, int n_kv, int hd, int max_ctx, float scale, const void* suh, void* xr,
                             void* out_bf16, int* status, void* stream, int max_seq_rows, const void* plan, const void* k_s4, const void* v_s4) {
  if (hd != 128 || n_q % n_kv != 0 || n_q / n_kv > 16 || rows <= 0 || rows > PLAN_MAX_ROWS || max_ctx <= 0 || k_s4 == nullptr || v_s4 == nullptr)
    return (int)cudaErrorInvalidValue;
  return launch_decode<128, true, 2>((const CUtensorMap*)tmap_k, (const CUtensorMap*)tmap_v, q, (const int*)block_table, max_blocks, (const int*)row_seq,
                                     (const int*)ctx_len, (float*)scratch, rows, n_q, n_kv, max_ctx, scale, suh, xr, out_bf16, status, (cudaStream_t)stream,
                                     nullptr, max_seq_rows, (const int*)plan, (const float*)k_s4, (const float*)v_s4);
}

RX_API int rx_attn_prefill_q4(const void* tmap_k, const void* tmap_v, const void* q, const void* block_table, int max_blocks, const void* seq_ids,
                              const void* q_start, const void* q_len, const void* pos0, void* out, int nseq, int max_qlen, int n_q, int n_kv, int hd,
                              float scale, int* status, void* stream, const void* k_s4, const void* v_s4) {
  if (hd != 128 || n_q % n_kv != 0 || nseq <= 0 || max_qlen <= 0 || k_s4 == nullptr || v_s4 == nullptr) return (int)cudaErrorInvalidValue;
  return launch_prefill<128, true, 2>((const CUtensorMap*)tmap_k, (const CUtensorMap*)tmap_v, q, (const int*)block_table, max_blocks, (const int*)seq_ids,
                                      (const int*)q_start, (const int*)q_len, (const int*)pos0, out, nseq, max_qlen, n_q, n_kv, scale, status,
                                      (cudaStream_t)stream, nullptr, (const float*)k_s4, (const float*)v_s4);
}

extern "C" int rx_attn_prefill_tc(const void* tmap_k, const void* tmap_v, const void* q, const void* block_table, int max_blocks, const void* seq_ids,
                                  const void* q_start, const void* q_len, const void* pos0, void* out, int nseq, int max_qlen, int n_q, int n_kv, int hd,
                                  float scale, int* status, void* stream, int reserved);

RX_API int rx_attn_prefill(const void* tmap_k, const void* tmap_v, const void* q, const void* block_table, int max_blocks, const void* seq_ids,
                           const void* q_start, const void* q_len, const void* pos0, void* out, int nseq, int max_qlen, int n_q, int n_kv, int hd,
                           float scale, int* status, void* stream, const void* kv_scale, const void* k_tscale, const void* v_tscale) {
  if (n_q % n_kv != 0 || nseq <= 0 || max_qlen <= 0) return (int)cudaErrorInvalidValue;
  if ((k_tscale == nullptr) != (v_tscale == nullptr) || (k_tscale != nullptr && kv_scale != nullptr)) return (int)cudaErrorInvalidValue;
  if (k_tscale != nullptr) {
    // int8 cache with per-token scales: the mma.sync kernel over byte pages
    cudaStream_t st8 = (cudaStream_t)stream;
#define RX_PF8(HDV) launch_prefill<HDV, true, 1>((const CUtensorMap*)tmap_k, (const CUtensorMap*)tmap_v, q, (const int*)block_table, max_blocks, \
    (const int*)seq_ids, (const int*)q_start, (const int*)q_len, (const int*)pos0, out, nseq, max_qlen, n_q, n_kv, scale, status, st8, nullptr, \
    (const float*)k_tscale, (const float*)v_tscale)
    if (hd == 128) return RX_PF8(128);
    if (hd == 64) return RX_PF8(64);
#undef RX_PF8
    return (int)cudaErrorInvalidValue;
  }
  // bf16 caches with 128-wide heads: the tcgen05 / tensor-memory kernel (attention_tc.cu); FP8 caches and 64-wide heads: mma.sync below
  if (hd == 128 && kv_scale == nullptr)
    return rx_attn_prefill_tc(tmap_k, tmap_v, q, block_table, max_blocks, seq_ids, q_start, q_len, pos0, out, nseq, max_qlen, n_q, n_kv, hd, scale,
                              status, stream, 0);
  cudaStream_t st = (cudaStream_t)stream;
#define RX_PF(HDV, F8) launch_prefill<HDV, F8>((const CUtensorMap*)tmap_k, (const CUtensorMap*)tmap_v, q, (const int*)block_table, max_blocks, \
    (const int*)seq_ids, (const int*)q_start, (const int*)q_len, (const int*)pos0, out, nseq, max_qlen, n_q, n_kv, scale, status, st, (const float*)kv_scale)
  if (hd == 128) return kv_scale ? RX_PF(128, true) : RX_PF(128, false);
  if (hd == 64) return kv_scale ? RX_PF(64, true) : RX_PF(64, false);
#undef RX_PF
  return (int)cudaErrorInvalidValue;
}
