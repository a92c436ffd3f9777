// Multi-head latent attention (absorbed form) for sm_100a: paged latent cache, split-KV flash kernel, merge, the per-head
// absorb / expand GEMMs and the row kernels around them.
//
// Cache (one tensor per layer): bf16 [pages][9][64 tokens][64] - boxes 0..7 hold the 512 normalised latent dims, box 8 the 64
// RoPE'd key dims; a (page, box) is one contiguous 8 KB TMA tile with 128-byte swizzle.  Every head shares the row, so the
// score is q_lat . c + q_rope . k_rope and the value is c itself:
//     q_lat[h] = q_nope[h] @ W_uk[h]   (absorb, 128 -> 512),   out[h] = (softmax . c) @ W_uv[h]   (expand, 512 -> 128).
// mla_attn_kernel: one CTA per (row, 16 heads, 1024-key split); per 64-key page the four warps split the keys for Q.K^T
// (bf16 mma.sync, fp32 online softmax), share the probabilities through shared memory, and split the 512 value columns for
// P.V.  Splits are ABSOLUTE key ranges merged in split order, so a row's bits do not depend on the batch; the same kernel
// serves decode windows and prefill rows (each row attends to its own ctx_len keys).  With 8-way head parallelism a rank
// owns exactly one 16-head group.  Semantics: reference crates/cuda/csrc/mla_gated.cu / ling_mla_attn.cu (nope + rope, cache
// row 576) and glm_p2_mla.cu (absorb / expand on tensor cores); layout, split geometry and schedule are new.
#include <cuda.h>
#include "common.cuh"

namespace rx {

constexpr int ML_PAGE = 64;
constexpr int ML_LAT = 512, ML_ROPE = 64, ML_QK = 576;
constexpr int ML_BOXES = 9;
constexpr int ML_TILE = ML_BOXES * 8192;
constexpr int ML_HG = 16;                 // heads per CTA (one m16 MMA tile)
constexpr int ML_SPLIT_PAGES = 16;        // 1024 keys per split
constexpr int ML_QSTRIDE = ML_QK * 2 + 16;
constexpr int ML_PSTRIDE = ML_PAGE * 2 + 16;

__device__ __forceinline__ void ml_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ml_ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ml_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ml_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ml_bf(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t ml_tobf(float f) {
  __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<uint16_t*>(&b);
}
// 16-byte chunk `dchunk` (8 bf16) of key `key` inside a page tile
__device__ __forceinline__ uint32_t ml_chunk_addr(uint32_t base, int key, int dchunk) {
  return base + (dchunk >> 3) * 8192 + key * 128 + (((dchunk & 7) ^ (key & 7)) << 4);
}

// q: bf16 [rows][H][576] (q_lat | q_rope).  part_o: f32 [rows][H][max_splits][512], part_ml: f32 [rows][H][max_splits][2].
__global__ void __launch_bounds__(128, 1)
mla_attn_kernel(const __grid_constant__ CUtensorMap tc, const uint16_t* __restrict__ q, const int* __restrict__ block_table, int max_blocks,
                const int* __restrict__ row_seq, const int* __restrict__ ctx_len, float* __restrict__ part_o, float* __restrict__ part_ml, int H,
                int max_splits, float scale_log2, int* status, const int* __restrict__ row_sel, int want) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* qs = smem + 2 * ML_TILE;
  uint8_t* ps = qs + ML_HG * ML_QSTRIDE;
  float* wmax = (float*)(ps + ML_HG * ML_PSTRIDE);      // [4][16]
  float* wsum = wmax + 64;                              // [4][16]
  uint64_t* bars = (uint64_t*)(wsum + 64);
  volatile int* abort_flag = (volatile int*)(bars + 2);
  const int row = blockIdx.x, hg = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (row_sel != nullptr && row_sel[row] != want) return;      // rows of the other regime belong to the other call
  const int ctx = ctx_len[row];
  const int k_begin = split * ML_SPLIT_PAGES * ML_PAGE;
  if (k_begin >= ctx) return;
  const int k_end = min(ctx, k_begin + ML_SPLIT_PAGES * ML_PAGE);
  const int npages = (k_end - k_begin + ML_PAGE - 1) / ML_PAGE;
  const int* bt = block_table + (size_t)row_seq[row] * max_blocks + k_begin / ML_PAGE;

  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  // stage Q of this head group: 16 rows x 576 bf16 (16-byte copies)
  {
    const uint16_t* qg = q + ((size_t)row * H + (size_t)hg * ML_HG) * ML_QK;
    for (int i = threadIdx.x; i < ML_HG * (ML_QK / 8); i += 128) {
      const int r = i / (ML_QK / 8), c = i % (ML_QK / 8);
      *reinterpret_cast<uint4*>(qs + r * ML_QSTRIDE + c * 16) = *reinterpret_cast<const uint4*>(qg + (size_t)r * ML_QK + c * 8);
    }
  }
  __syncthreads();
  auto load_page = [&](int p) {
    uint8_t* dst = smem + (p & 1) * ML_TILE;
    mbar_arrive_expect_tx(&bars[p & 1], ML_TILE);
    const int y = bt[p] * ML_BOXES * ML_PAGE;
#pragma unroll
    for (int b = 0; b < ML_BOXES; ++b) tma_load_2d(dst + b * 8192, &tc, 0, y + b * ML_PAGE, &bars[p & 1]);
  };
  if (threadIdx.x == 0) {
    load_page(0);
    if (npages > 1) load_page(1);
  }
  const uint32_t qs_u = smem_u32(qs), ps_u = smem_u32(ps);
  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  const int mi = lane >> 3;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[16][4];
#pragma unroll
  for (int d = 0; d < 16; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

  for (int p = 0; p < npages; ++p) {
    if (!mbar_wait(&bars[p & 1], (p >> 1) & 1, abort_flag, status, 70)) break;
    const uint32_t tile = smem_u32(smem + (p & 1) * ML_TILE);
    // ---- scores of this warp's 16 keys against the 16 heads
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
    for (int ks = 0; ks < ML_QK / 16; ++ks) {
      uint32_t a[4], b0, b1, b2, b3;
      ml_ldsm_x4(qs_u + ((lane & 7) + ((lane >> 3) & 1) * 8) * ML_QSTRIDE + (ks * 16 + (lane >> 4) * 8) * 2, a[0], a[1], a[2], a[3]);
      ml_ldsm_x4(ml_chunk_addr(tile, warp * 16 + (mi >> 1) * 8 + (lane & 7), ks * 2 + (mi & 1)), b0, b1, b2, b3);
      ml_mma(s[0], a, b0, b1);
      ml_mma(s[1], a, b2, b3);
    }
    const int key_base = k_begin + p * ML_PAGE + warp * 16;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key_base + j * 8 + 2 * (lane & 3) + (e & 1);
        const float v = key < ctx ? s[j][e] * scale_log2 : -INFINITY;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    if ((lane & 3) == 0) { wmax[warp * 16 + r_lo] = mx[0]; wmax[warp * 16 + r_hi] = mx[1]; }
    __syncthreads();
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int rr = r == 0 ? r_lo : r_hi;
      const float pm = fmaxf(fmaxf(wmax[rr], wmax[16 + rr]), fmaxf(wmax[32 + rr], wmax[48 + rr]));
      const float mn = fmaxf(m[r], pm);
      corr[r] = (mn == -INFINITY) ? 1.f : exp2f(m[r] - mn);
      m[r] = mn;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mm = m[e >> 1];
        pv[e] = (mm == -INFINITY) ? 0.f : exp2f(s[j][e] - mm);
        rs[e >> 1] += pv[e];
      }
      const int col = warp * 16 + j * 8 + 2 * (lane & 3);
      *reinterpret_cast<uint32_t*>(ps + r_lo * ML_PSTRIDE + col * 2) = ml_pack(pv[0], pv[1]);
      *reinterpret_cast<uint32_t*>(ps + r_hi * ML_PSTRIDE + col * 2) = ml_pack(pv[2], pv[3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
    }
    if ((lane & 3) == 0) { wsum[warp * 16 + r_lo] = rs[0]; wsum[warp * 16 + r_hi] = rs[1]; }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int rr = r == 0 ? r_lo : r_hi;
      l[r] = l[r] * corr[r] + (((wsum[rr] + wsum[16 + rr]) + wsum[32 + rr]) + wsum[48 + rr]);
    }
    // ---- values: this warp owns latent columns [128 warp, 128 warp + 128)
#pragma unroll
    for (int d = 0; d < 16; ++d) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
#pragma unroll
    for (int kp = 0; kp < ML_PAGE / 16; ++kp) {
      uint32_t a[4];
      ml_ldsm_x4(ps_u + ((lane & 7) + ((lane >> 3) & 1) * 8) * ML_PSTRIDE + (kp * 16 + (lane >> 4) * 8) * 2, a[0], a[1], a[2], a[3]);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t b0, b1, b2, b3;
        ml_ldsm_x4_t(ml_chunk_addr(tile, kp * 16 + (mi & 1) * 8 + (lane & 7), warp * 16 + dp * 2 + (mi >> 1)), b0, b1, b2, b3);
        ml_mma(o[2 * dp], a, b0, b1);
        ml_mma(o[2 * dp + 1], a, b2, b3);
      }
    }
    fence_proxy_async(); // the tile was read with ordinary loads; its refill writes through the async proxy
    __syncthreads();     // the tile and the probability buffer are free again
    if (threadIdx.x == 0 && p + 2 < npages) load_page(p + 2);
  }
  if (*abort_flag != 0) return;
  // ---- unnormalised partials of this split
  const int h0 = hg * ML_HG;
  float* po_lo = part_o + (((size_t)row * H + h0 + r_lo) * max_splits + split) * ML_LAT + warp * 128;
  float* po_hi = part_o + (((size_t)row * H + h0 + r_hi) * max_splits + split) * ML_LAT + warp * 128;
#pragma unroll
  for (int d = 0; d < 16; ++d) {
    const int c = d * 8 + 2 * (lane & 3);
    *reinterpret_cast<float2*>(po_lo + c) = make_float2(o[d][0], o[d][1]);
    *reinterpret_cast<float2*>(po_hi + c) = make_float2(o[d][2], o[d][3]);
  }
  if (warp == 0 && (lane & 3) == 0) {
    float* ml_lo = part_ml + (((size_t)row * H + h0 + r_lo) * max_splits + split) * 2;
    float* ml_hi = part_ml + (((size_t)row * H + h0 + r_hi) * max_splits + split) * 2;
    ml_lo[0] = m[0]; ml_lo[1] = l[0];
    ml_hi[0] = m[1]; ml_hi[1] = l[1];
  }
}

// grid (rows, H), 128 threads: out_lat bf16 [rows][H][512] = merged splits (split order).
__global__ void mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ ctx_len, int H,
                                 int max_splits, uint16_t* __restrict__ out, const int* __restrict__ row_sel, int want) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, h = blockIdx.y;
  if (row_sel != nullptr && row_sel[row] != want) return;
  const int ctx = ctx_len[row];
  const int ns = (ctx + ML_SPLIT_PAGES * ML_PAGE - 1) / (ML_SPLIT_PAGES * ML_PAGE);
  const float* ml = part_ml + ((size_t)row * H + h) * max_splits * 2;
  const float* po = part_o + ((size_t)row * H + h) * max_splits * ML_LAT;
  float M = -INFINITY;
  for (int s = 0; s < ns; ++s) M = fmaxf(M, ml[2 * s]);
  float den = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < ns; ++s) {
    const float w = (M == -INFINITY) ? 0.f : exp2f(ml[2 * s] - M);
    den += ml[2 * s + 1] * w;
    const float4 v = *reinterpret_cast<const float4*>(po + (size_t)s * ML_LAT + threadIdx.x * 4);
    acc.x = fmaf(v.x, w, acc.x); acc.y = fmaf(v.y, w, acc.y); acc.z = fmaf(v.z, w, acc.z); acc.w = fmaf(v.w, w, acc.w);
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  uint2 u;
  u.x = (uint32_t)ml_tobf(acc.x * inv) | ((uint32_t)ml_tobf(acc.y * inv) << 16);
  u.y = (uint32_t)ml_tobf(acc.z * inv) | ((uint32_t)ml_tobf(acc.w * inv) << 16);
  *reinterpret_cast<uint2*>(out + ((size_t)row * H + h) * ML_LAT + threadIdx.x * 4) = u;
}

// Per-head GEMM: out[m][h][n] = sum_k in[m][h][k] * W[h][k][n].  in: bf16, row stride in_ld, head stride in_hs; out likewise.
// grid (H, ceil(M / 64), N / 128), 128 threads; K % 16 == 0, N % 128 == 0.
__global__ void __launch_bounds__(128) head_gemm_kernel(const uint16_t* __restrict__ in, int in_ld, int in_hs, const uint16_t* __restrict__ W, int K, int N,
                                                        uint16_t* __restrict__ out, int out_ld, int out_hs, int M) {
  pdl_launch();
  pdl_wait();
  constexpr int WSTRIDE = 128 * 2 + 16;
  constexpr int KS = 64;                         // k rows staged per step (one barrier pair per 64 k instead of per 16)
  __shared__ __align__(16) uint8_t ws[KS * WSTRIDE];
  const int h = blockIdx.x, m0 = blockIdx.y * 64, n0 = blockIdx.z * 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, mi = lane >> 3;
  const int r_lo = m0 + warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const uint16_t* Wh = W + (size_t)h * K * N + n0;
  const uint16_t* a_lo = in + (size_t)r_lo * in_ld + (size_t)h * in_hs;
  const uint16_t* a_hi = in + (size_t)r_hi * in_ld + (size_t)h * in_hs;
  const uint32_t ws_u = smem_u32(ws);
  float acc[16][4];
#pragma unroll
  for (int d = 0; d < 16; ++d) { acc[d][0] = acc[d][1] = acc[d][2] = acc[d][3] = 0.f; }
  for (int k0 = 0; k0 < K; k0 += KS) {
    const int kn = min(KS, K - k0);              // K is a multiple of 16
    __syncthreads();
    for (int i = threadIdx.x; i < kn * 16; i += 128) {      // kn k rows x 16 chunks of 8 columns
      const int kr = i >> 4, c = i & 15;
      *reinterpret_cast<uint4*>(ws + kr * WSTRIDE + c * 16) = __ldg(reinterpret_cast<const uint4*>(Wh + (size_t)(k0 + kr) * N + c * 8));
    }
    __syncthreads();
    for (int kk = 0; kk < kn; kk += 16) {
      uint32_t a[4];
      const int kc = k0 + kk + 2 * (lane & 3);
      a[0] = r_lo < M ? *reinterpret_cast<const uint32_t*>(a_lo + kc) : 0u;
      a[1] = r_hi < M ? *reinterpret_cast<const uint32_t*>(a_hi + kc) : 0u;
      a[2] = r_lo < M ? *reinterpret_cast<const uint32_t*>(a_lo + kc + 8) : 0u;
      a[3] = r_hi < M ? *reinterpret_cast<const uint32_t*>(a_hi + kc + 8) : 0u;
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t b0, b1, b2, b3;
        ml_ldsm_x4_t(ws_u + (kk + (mi & 1) * 8 + (lane & 7)) * WSTRIDE + (dp * 16 + (mi >> 1) * 8) * 2, b0, b1, b2, b3);
        ml_mma(acc[2 * dp], a, b0, b1);
        ml_mma(acc[2 * dp + 1], a, b2, b3);
      }
    }
  }
  uint16_t* o_lo = out + (size_t)r_lo * out_ld + (size_t)h * out_hs + n0;
  uint16_t* o_hi = out + (size_t)r_hi * out_ld + (size_t)h * out_hs + n0;
#pragma unroll
  for (int d = 0; d < 16; ++d) {
    const int c = d * 8 + 2 * (lane & 3);
    if (r_lo < M) *reinterpret_cast<uint32_t*>(o_lo + c) = ml_pack(acc[d][0], acc[d][1]);
    if (r_hi < M) *reinterpret_cast<uint32_t*>(o_hi + c) = ml_pack(acc[d][2], acc[d][3]);
  }
}

// Row kernel after the fused q_a | kv_a projection.  a: bf16 [M][1536 + 640] (q_a 1536 | latent 512 | rope 64 | pad 64).
//   xr_q  = fp16(H(rmsnorm(q_a) * q_norm * suh_qb))                       [M][1536]   (rotated input of q_b)
//   cache row at `slot`: boxes 0..7 = rmsnorm(latent) * kv_norm, box 8 = RoPE(rope dims)   (rotate-half pairs (i, i + 32))
// 17 warps: warp b owns 128-block b of the row.
__global__ void __launch_bounds__(544) mla_row_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ q_norm, const uint16_t* __restrict__ kv_norm,
                                                      float eps, const __half* __restrict__ suh_qb, const int* __restrict__ positions,
                                                      const float* __restrict__ inv_freq, const int* __restrict__ slot, __half* __restrict__ xr_q,
                                                      uint16_t* __restrict__ cache, int a_ld) {
  pdl_launch();
  pdl_wait();
  __shared__ float ss[17];
  const int row = blockIdx.x, lane = threadIdx.x & 31, b = threadIdx.x >> 5;
  const int n0 = b * 128 + lane * 4;
  const uint2 u = *reinterpret_cast<const uint2*>(a + (size_t)row * a_ld + n0);
  float v[4] = {__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xFFFF0000u)};
  float s2 = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
  s2 = warp_sum(s2);
  if (lane == 0) ss[b] = s2;
  __syncthreads();
  if (b < 12) {
    float tot = 0.f;
    for (int i = 0; i < 12; ++i) tot += ss[i];
    const float rinv = rsqrtf(tot / 1536.f + eps);
    const uint2 wu = *reinterpret_cast<const uint2*>(q_norm + n0);
    const float w[4] = {__uint_as_float(wu.x << 16), __uint_as_float(wu.x & 0xFFFF0000u), __uint_as_float(wu.y << 16), __uint_as_float(wu.y & 0xFFFF0000u)};
    const uint2 su = *reinterpret_cast<const uint2*>(suh_qb + n0);
    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
    const float sc[4] = {s01.x, s01.y, s23.x, s23.y};
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = ml_bf(ml_tobf(v[i] * rinv)) * w[i] * sc[i];
    fwht128_warp(v);
    const __half2 p0 = __floats2half2_rn(v[0], v[1]), p1 = __floats2half2_rn(v[2], v[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&p0); o.y = *reinterpret_cast<const uint32_t*>(&p1);
    *reinterpret_cast<uint2*>(xr_q + (size_t)row * 1536 + n0) = o;
    return;
  }
  const int sl = slot[row];
  const int page = sl / ML_PAGE, tok = sl % ML_PAGE;
  uint16_t* base = cache + (size_t)page * ML_BOXES * ML_PAGE * 64;
  if (b < 16) {
    float tot = 0.f;
    for (int i = 12; i < 16; ++i) tot += ss[i];
    const float rinv = rsqrtf(tot / 512.f + eps);
    const int c = (b - 12) * 128 + lane * 4;              // latent column
    const uint2 wu = *reinterpret_cast<const uint2*>(kv_norm + c);
    const float w[4] = {__uint_as_float(wu.x << 16), __uint_as_float(wu.x & 0xFFFF0000u), __uint_as_float(wu.y << 16), __uint_as_float(wu.y & 0xFFFF0000u)};
    uint2 o;
    o.x = (uint32_t)ml_tobf(ml_bf(ml_tobf(v[0] * rinv)) * w[0]) | ((uint32_t)ml_tobf(ml_bf(ml_tobf(v[1] * rinv)) * w[1]) << 16);
    o.y = (uint32_t)ml_tobf(ml_bf(ml_tobf(v[2] * rinv)) * w[2]) | ((uint32_t)ml_tobf(ml_bf(ml_tobf(v[3] * rinv)) * w[3]) << 16);
    *reinterpret_cast<uint2*>(base + ((size_t)(c >> 6) * ML_PAGE + tok) * 64 + (c & 63)) = o;
    return;
  }
  // rope block: lanes 0..15 hold the 64 rope dims (lane L: dims 4L..4L+3); the partner of dim i < 32 is i + 32 (lane L + 8)
  float other[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) other[i] = __shfl_xor_sync(0xffffffffu, v[i], 8);
  if (lane < 16) {
    const float pos = (float)positions[row];
    uint16_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int dim = lane * 4 + i, f = dim & 31;
      float sn, cs;
      sincosf(pos * inv_freq[f], &sn, &cs);
      const float y = dim < 32 ? v[i] * cs - other[i] * sn : v[i] * cs + other[i] * sn;
      r[i] = ml_tobf(y);
    }
    uint2 o;
    o.x = (uint32_t)r[0] | ((uint32_t)r[1] << 16);
    o.y = (uint32_t)r[2] | ((uint32_t)r[3] << 16);
    *reinterpret_cast<uint2*>(base + ((size_t)8 * ML_PAGE + tok) * 64 + lane * 4) = o;
  }
}

// q_full: bf16 [M][H][192] (nope 128 | rope 64) -> q[row][h][512..575] = RoPE(rope part).  grid (M), H * 16 threads.
__global__ void mla_q_rope_kernel(const uint16_t* __restrict__ q_full, const int* __restrict__ positions, const float* __restrict__ inv_freq, int H,
                                  uint16_t* __restrict__ q, int q_ld) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x;
  const float pos = (float)positions[row];
  for (int i = threadIdx.x; i < H * 32; i += blockDim.x) {
    const int h = i >> 5, f = i & 31;
    const uint16_t* src = q_full + (size_t)row * q_ld + (size_t)h * 192 + 128;
    const float x1 = ml_bf(src[f]), x2 = ml_bf(src[f + 32]);
    float sn, cs;
    sincosf(pos * inv_freq[f], &sn, &cs);
    uint16_t* dst = q + ((size_t)row * H + h) * ML_QK + ML_LAT;
    dst[f] = ml_tobf(x1 * cs - x2 * sn);
    dst[f + 32] = ml_tobf(x2 * cs + x1 * sn);
  }
}

}  // namespace rx

using namespace rx;

RX_API long long rx_mla_scratch_floats(int rows, int H, int max_ctx) {
  const int splits = (max_ctx + ML_SPLIT_PAGES * ML_PAGE - 1) / (ML_SPLIT_PAGES * ML_PAGE);
  return (long long)rows * H * splits * (ML_LAT + 2);
}

// tmap: a tensor map made by rx_make_kv_tmap over the cache viewed as [pages * 9 * 64 rows][64].
// row_sel / want: only rows with row_sel[row] == want are computed and written (nullptr: every row).  The sparse-attention path calls this twice
// per layer: rows of the dense regime over the layer's cache, rows of the sparse regime over the gathered scratch pages.
RX_API int rx_mla_attn_sel(const void* tmap, const void* q, const void* block_table, int max_blocks, const void* row_seq, const void* ctx_len, void* scratch,
                           int rows, int H, int max_ctx, float scale, void* out_lat, int* status, const void* row_sel, int want, void* stream) {
  if (rows < 1 || H % ML_HG != 0 || max_ctx < 1) return (int)cudaErrorInvalidValue;
  const int splits = (max_ctx + ML_SPLIT_PAGES * ML_PAGE - 1) / (ML_SPLIT_PAGES * ML_PAGE);
  float* part_o = (float*)scratch;
  float* part_ml = part_o + (size_t)rows * H * splits * ML_LAT;
  const int smem = 2 * ML_TILE + ML_HG * ML_QSTRIDE + ML_HG * ML_PSTRIDE + 512 + 64 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mla_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap tm;
  memcpy(&tm, tmap, sizeof(tm));
  cudaStream_t st = (cudaStream_t)stream;
  int e = (int)rx::launch(mla_attn_kernel, dim3(rows, H / ML_HG, splits), dim3(128), (size_t)smem, st, tm, (const uint16_t*)q, (const int*)block_table,
                          max_blocks, (const int*)row_seq, (const int*)ctx_len, part_o, part_ml, H, splits, scale * 1.4426950408889634f, status,
                          (const int*)row_sel, want);
  if (e != 0) return e;
  return (int)rx::launch(mla_merge_kernel, dim3(rows, H), dim3(128), 0, st, (const float*)part_o, (const float*)part_ml, (const int*)ctx_len, H, splits,
                         (uint16_t*)out_lat, (const int*)row_sel, want);
}
RX_API int rx_mla_attn(const void* tmap, const void* q, const void* block_table, int max_blocks, const void* row_seq, const void* ctx_len, void* scratch,
                       int rows, int H, int max_ctx, float scale, void* out_lat, int* status, void* stream) {
  return rx_mla_attn_sel(tmap, q, block_table, max_blocks, row_seq, ctx_len, scratch, rows, H, max_ctx, scale, out_lat, status, nullptr, 0, stream);
}

RX_API int rx_head_gemm(const void* in, int in_ld, int in_hs, const void* W, int H, int K, int N, void* out, int out_ld, int out_hs, int M, void* stream) {
  if (M < 1 || K % 16 != 0 || N % 128 != 0 || (in_ld | in_hs | out_ld | out_hs) % 2 != 0) return (int)cudaErrorInvalidValue;
  return (int)rx::launch(head_gemm_kernel, dim3(H, (M + 63) / 64, N / 128), dim3(128), 0, (cudaStream_t)stream, (const uint16_t*)in, in_ld, in_hs,
                         (const uint16_t*)W, K, N, (uint16_t*)out, out_ld, out_hs, M);
}

// a_ld: elements between rows of `a` (2176, or wider when the projection carries the sparse indexer's columns after the pad)
RX_API int rx_mla_row_ld(const void* a, int a_ld, const void* q_norm, const void* kv_norm, float eps, const void* suh_qb, const void* positions,
                         const void* inv_freq, const void* slot, void* xr_q, void* cache, int M, void* stream) {
  if (M < 1 || a_ld < 2176 || a_ld % 4 != 0) return (int)cudaErrorInvalidValue;
  return (int)rx::launch(mla_row_kernel, dim3(M), dim3(544), 0, (cudaStream_t)stream, (const uint16_t*)a, (const uint16_t*)q_norm, (const uint16_t*)kv_norm,
                         eps, (const __half*)suh_qb, (const int*)positions, (const float*)inv_freq, (const int*)slot, (__half*)xr_q, (uint16_t*)cache, a_ld);
}
RX_API int rx_mla_row(const void* a, const void* q_norm, const void* kv_norm, float eps, const void* suh_qb, const void* positions, const void* inv_freq,
                      const void* slot, void* xr_q, void* cache, int M, void* stream) {
  return rx_mla_row_ld(a, 2176, q_norm, kv_norm, eps, suh_qb, positions, inv_freq, slot, xr_q, cache, M, stream);
}

RX_API int rx_mla_q_rope_ld(const void* q_full, int q_ld, const void* positions, const void* inv_freq, int H, void* q, int M, void* stream) {
  if (M < 1 || H < 1 || q_ld < H * 192) return (int)cudaErrorInvalidValue;
  int threads = H * 32;
  if (threads > 1024) threads = 1024;
  return (int)rx::launch(mla_q_rope_kernel, dim3(M), dim3(threads), 0, (cudaStream_t)stream, (const uint16_t*)q_full, (const int*)positions,
                         (const float*)inv_freq, H, (uint16_t*)q, q_ld);
}
RX_API int rx_mla_q_rope(const void* q_full, const void* positions, const void* inv_freq, int H, void* q, int M, void* stream) {
  return rx_mla_q_rope_ld(q_full, H * 192, positions, inv_freq, H, q, M, stream);
}
