// Sparse-attention indexer (DeepSeek sparse attention with pooled index keys) for sm_100a: which tokens a long row attends to.
//
//   index key   k_t = LayerNorm(idx_k(x_t))                      128 values (biased LayerNorm), bf16
//   gate        g_t = idx_gate(x_t)                              128 values, bf16
//   pooled key  K_p = sum_{j<4} softmax_j(g_{4p+j} + ape_j) * k_{4p+j}     per dimension, fp32 math, one rounding to bf16
//   score       S[r, p] = fp16(scale * sum_{h<32} relu(q[r, h] . K_p) * w[r, h])     for pools p < (pos_r + 1) / 4
//   selection   the `sel_pools` highest scores, ties to the LOWEST pool index, emitted ascending; a pool expands to its 4 tokens;
//               then the 0..3 raw tokens of the row's incomplete last pool
//   regime      a row with pos + 1 > dense_below is sparse, every other row attends to its whole context
// (semantics: reference crates/cuda/csrc/dsa.cuh:1-16, dsa_index.cu:1-24, dsa_score.cu:1-20, dsa_select.cu:1-22).
//
// Layout here.  The raw (key | gate) rows of the CURRENT call sit in a staging buffer [rows][256]; a ring [seqs][ring_len][256] keeps each
// sequence's last tokens so that a pool straddling two calls can be completed (ring_len >= the widest decode window + 4; a row of a long prefill
// slice writes the ring only if no later row of the call lands on its ring slot: rows of a sequence are consecutive, so that is row + ring_len).  Pooled keys live in a plane bf16 [pages][16][128] addressed by
// the latent cache's block table (64-token pages = 16 pools).  A pool is (re)computed whenever its last member (pos % 4 == 3) is a row of the
// call - always, so rejected draft rows are repaired when the accepted tokens arrive again.
// Scoring: one CTA per (row, 128 pools): pools and the row's 32 index queries staged in shared memory (16-byte chunks, XOR swizzle), bf16
// mma.sync m16n8k16 with pools as the M side, head sum in a fixed order (8 heads per thread, then the quad butterfly).  The op reads the pool
// plane once per row from L2 and is bandwidth-trivial next to the attention it replaces (16.8 MB of pooled keys for a 262,144-token context).
// Selection: one CTA per row, 16-bit order keys, a two-pass 8-bit radix count (integer atomics: exact in any order) finds the threshold key
// and how many of its ties to take, then one pass in index order emits every key above it and the first ties at closed-form positions from a
// block scan - which makes the tie rule an index rule and the output ascending.
// Gather: the selected tokens' latent rows are copied into scratch pages of the cache's own layout ([9][64][64] per page), so the unchanged
// split-KV attention kernel runs over them through a virtual block table (2051 rows instead of the whole context).
// Every output element is a function of one row's inputs and the planes: nothing depends on which rows share a call.
#include "common.cuh"

namespace rx {

constexpr int DS_D = 128;             // index head dim
constexpr int DS_H = 32;              // index heads
constexpr int DS_P = 4;               // tokens per pool
constexpr int DS_PAGE = 64;           // tokens per cache page
constexpr int DS_PPP = DS_PAGE / DS_P;
constexpr int DS_CHUNK = 128;         // pools per scoring CTA
constexpr int DS_ROW = 2 * DS_D;      // staging / ring row: key | gate
constexpr int DS_PAGE_ROWS = 9 * 64;  // 64-column rows of one latent-cache page

__device__ __forceinline__ float ds_bf(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t ds_tobf(float f) {
  __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<uint16_t*>(&b);
}
__device__ __forceinline__ void ds_unpack4(uint2 v, float (&x)[4]) {
  x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xFFFF0000u);
  x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xFFFF0000u);
}
__device__ __forceinline__ uint2 ds_pack4(const float (&x)[4]) {
  uint2 o;
  o.x = (uint32_t)ds_tobf(x[0]) | ((uint32_t)ds_tobf(x[1]) << 16);
  o.y = (uint32_t)ds_tobf(x[2]) | ((uint32_t)ds_tobf(x[3]) << 16);
  return o;
}

// grid = rows, one warp per row; lane l owns dims 4l .. 4l + 3.  a: bf16 [rows][a_ld], raw key at col_k, gate at col_g.  Writes the staging row.
__global__ void __launch_bounds__(32) dsa_stage_kernel(const uint16_t* __restrict__ a, int a_ld, int col_k, int col_g, const float* __restrict__ ln_w,
                                                       const float* __restrict__ ln_b, float eps, uint16_t* __restrict__ stage) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x;
  const uint16_t* src = a + (size_t)row * a_ld;
  float x[4];
  ds_unpack4(*reinterpret_cast<const uint2*>(src + col_k + lane * 4), x);
  const float mean = warp_sum((x[0] + x[1]) + (x[2] + x[3])) * (1.f / DS_D);
  float dv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) dv[i] = x[i] - mean;
  const float var = warp_sum((dv[0] * dv[0] + dv[1] * dv[1]) + (dv[2] * dv[2] + dv[3] * dv[3])) * (1.f / DS_D);
  const float rs = rsqrtf(var + eps);
  const float4 w = *reinterpret_cast<const float4*>(ln_w + lane * 4), b = *reinterpret_cast<const float4*>(ln_b + lane * 4);
  const float y[4] = {dv[0] * rs * w.x + b.x, dv[1] * rs * w.y + b.y, dv[2] * rs * w.z + b.z, dv[3] * rs * w.w + b.w};
  uint16_t* st = stage + (size_t)row * DS_ROW;
  *reinterpret_cast<uint2*>(st + lane * 4) = ds_pack4(y);
  *reinterpret_cast<uint2*>(st + DS_D + lane * 4) = *reinterpret_cast<const uint2*>(src + col_g + lane * 4);
}

// grid = rows, one warp per row: the staging row goes to the sequence's ring, AFTER the pool kernel has read the earlier calls' tokens from it
// (a row of a long slice can land on the slot of a token the same call's first pool still needs).
__global__ void __launch_bounds__(32) dsa_ring_kernel(const uint16_t* __restrict__ stage, const int* __restrict__ row_seq, const int* __restrict__ positions,
                                                      int rows, uint16_t* __restrict__ ring, int ring_len) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x;
  const int pos = positions[row], seq = row_seq[row];
  // the rows of a sequence are consecutive positions in order, so the only row that can land on this ring slot again is ring_len rows later
  const int r2 = row + ring_len;
  if (r2 < rows && row_seq[r2] == seq && positions[r2] == pos + ring_len) return;
  const uint4* src = reinterpret_cast<const uint4*>(stage + (size_t)row * DS_ROW);
  uint4* dst = reinterpret_cast<uint4*>(ring + ((size_t)seq * ring_len + pos % ring_len) * DS_ROW);
  dst[lane] = src[lane];          // 32 lanes x 16 bytes = the 512-byte row
}

// grid = rows, one warp per row; only rows that complete a pool (pos % 4 == 3) work.  ape: f32 [4][128].
__global__ void __launch_bounds__(32) dsa_pool_kernel(const uint16_t* __restrict__ stage, const uint16_t* __restrict__ ring, int ring_len,
                                                      const float* __restrict__ ape, const int* __restrict__ row_seq, const int* __restrict__ positions,
                                                      const int* __restrict__ block_table, int max_blocks, uint16_t* __restrict__ pool) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x;
  const int pos = positions[row];
  if ((pos & (DS_P - 1)) != DS_P - 1) return;
  const int seq = row_seq[row];
  float k[DS_P][4], g[DS_P][4];
#pragma unroll
  for (int j = 0; j < DS_P; ++j) {
    const int m = pos - (DS_P - 1) + j, r = row - (DS_P - 1) + j;
    const uint16_t* src;
    if (r >= 0 && row_seq[r] == seq && positions[r] == m) src = stage + (size_t)r * DS_ROW;      // a row of this call
    else src = ring + ((size_t)seq * ring_len + m % ring_len) * DS_ROW;                            // an earlier call's token
    ds_unpack4(*reinterpret_cast<const uint2*>(src + lane * 4), k[j]);
    ds_unpack4(*reinterpret_cast<const uint2*>(src + DS_D + lane * 4), g[j]);
  }
  float out[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float l[DS_P], mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < DS_P; ++j) {
      l[j] = g[j][c] + ape[j * DS_D + lane * 4 + c];
      mx = fmaxf(mx, l[j]);
    }
    float den = 0.f;
#pragma unroll
    for (int j = 0; j < DS_P; ++j) {
      l[j] = __expf(l[j] - mx);
      den += l[j];
    }
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < DS_P; ++j) acc = fmaf(l[j] / den, k[j][c], acc);
    out[c] = acc;
  }
  const int p = pos / DS_P;
  const size_t at = ((size_t)block_table[(size_t)seq * max_blocks + p / DS_PPP] * DS_PPP + p % DS_PPP) * DS_D;
  *reinterpret_cast<uint2*>(pool + at + lane * 4) = ds_pack4(out);
}

__device__ __forceinline__ void ds_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ds_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// grid = (pool chunks, rows), 256 threads.  q: bf16, row r at q + r * q_ld, [32][128]; head weights bf16 at wsrc + r * w_ld + col_w.
// scores: fp16 [rows][s_stride].
__global__ void __launch_bounds__(256) dsa_score_kernel(const uint16_t* __restrict__ q, int q_ld, const uint16_t* __restrict__ wsrc, int w_ld, int col_w,
                                                        const uint16_t* __restrict__ pool, const int* __restrict__ block_table, int max_blocks,
                                                        const int* __restrict__ row_seq, const int* __restrict__ positions, int dense_below, float scale,
                                                        __half* __restrict__ scores, int s_stride) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) uint8_t tile[DS_CHUNK * 256];
  __shared__ __align__(16) uint8_t qs[DS_H * 256];
  __shared__ float ws[DS_H];
  const int row = blockIdx.y, pos = positions[row];
  if (pos + 1 <= dense_below) return;
  const int npools = (pos + 1) / DS_P, p0 = blockIdx.x * DS_CHUNK;
  if (p0 >= npools) return;
  const int* bt = block_table + (size_t)row_seq[row] * max_blocks;
  for (int i = threadIdx.x; i < DS_CHUNK * 16; i += 256) {
    const int p = i >> 4, c = i & 15, gp = p0 + p;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (gp < npools) v = __ldg(reinterpret_cast<const uint4*>(pool + ((size_t)bt[gp / DS_PPP] * DS_PPP + gp % DS_PPP) * DS_D + c * 8));
    *reinterpret_cast<uint4*>(tile + p * 256 + ((c ^ (p & 7)) << 4)) = v;
  }
  for (int i = threadIdx.x; i < DS_H * 16; i += 256) {
    const int h = i >> 4, c = i & 15;
    *reinterpret_cast<uint4*>(qs + h * 256 + ((c ^ (h & 7)) << 4)) = *reinterpret_cast<const uint4*>(q + (size_t)row * q_ld + h * DS_D + c * 8);
  }
  if (threadIdx.x < DS_H) ws[threadIdx.x] = ds_bf(wsrc[(size_t)row * w_ld + col_w + threadIdx.x]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const uint32_t tile_u = smem_u32(tile), qs_u = smem_u32(qs);
  float acc[4][4];
#pragma unroll
  for (int t = 0; t < 4; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
#pragma unroll
  for (int ks = 0; ks < DS_D / 16; ++ks) {
    uint32_t a0, a1, a2, a3;
    const int pr = warp * 16 + (lane & 15), ch = 2 * ks + (lane >> 4);
    ds_ldsm_x4(tile_u + pr * 256 + ((ch ^ (pr & 7)) << 4), a0, a1, a2, a3);
#pragma unroll
    for (int tp = 0; tp < 2; ++tp) {
      uint32_t b0, b1, b2, b3;
      const int hh = 16 * tp + (lane & 7) + ((lane >> 4) << 3), ch2 = 2 * ks + ((lane >> 3) & 1);
      ds_ldsm_x4(qs_u + hh * 256 + ((ch2 ^ (hh & 7)) << 4), b0, b1, b2, b3);
      ds_mma(acc[2 * tp], a0, a1, a2, a3, b0, b1);
      ds_mma(acc[2 * tp + 1], a0, a1, a2, a3, b2, b3);
    }
  }
  float s_lo = 0.f, s_hi = 0.f;          // pools g and g + 8 of this warp's 16; the thread's 8 heads in (tile, column) order
#pragma unroll
  for (int t = 0; t < 4; ++t)
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const float w = ws[8 * t + 2 * tg + c];
      s_lo += fmaxf(acc[t][c], 0.f) * w;
      s_hi += fmaxf(acc[t][2 + c], 0.f) * w;
    }
  s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1); s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1);
  s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2); s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
  if (tg == 0) {
    const __half ninf = __ushort_as_half((unsigned short)0xfc00u);
    __half* srow = scores + (size_t)row * s_stride;
    const int gp = p0 + warp * 16 + g;
    if (gp < s_stride) srow[gp] = gp < npools ? __float2half_rn(s_lo * scale) : ninf;
    if (gp + 8 < s_stride) srow[gp + 8] = gp + 8 < npools ? __float2half_rn(s_hi * scale) : ninf;
  }
}

// fp16 bits -> 16-bit key in IEEE order; -0 == +0; NaN and -inf are invalid (0); every valid key is > 0
__device__ __forceinline__ uint32_t ds_key(uint32_t u) {
  u &= 0xffffu;
  if ((u & 0x7fffu) > 0x7c00u || u == 0xfc00u) return 0u;
  if (u == 0x8000u) u = 0u;
  return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
}

// grid = rows, 1024 threads.  out: int32 [rows][k_stride] (selected tokens ascending, tail, then -1); sp_flag / sp_ctx: int32 [rows].
__global__ void __launch_bounds__(1024) dsa_select_kernel(const uint16_t* __restrict__ scores, int s_stride, const int* __restrict__ positions,
                                                          int dense_below, int sel_pools, int k_stride, int* __restrict__ out, int* __restrict__ sp_flag,
                                                          int* __restrict__ sp_ctx) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int pos = positions[row];
  if (pos + 1 <= dense_below) {
    if (t == 0) { sp_flag[row] = 0; sp_ctx[row] = 0; }
    return;
  }
  const int T = (pos + 1) / DS_P, tail = (pos + 1) % DS_P;
  const uint16_t* srow = scores + (size_t)row * s_stride;
  int* orow = out + (size_t)row * k_stride;
  __shared__ int hist[256];
  __shared__ int s_bucket, s_above;
  __shared__ int wsum[32], wpre[32], tile_total;

  // ---- threshold key: 8 high bits, then 8 low bits
  if (t < 256) hist[t] = 0;
  __syncthreads();
  for (int i = t; i < T; i += 1024) {
    const uint32_t k = ds_key(srow[i]);
    if (k) atomicAdd(&hist[k >> 8], 1);
  }
  __syncthreads();
  if (t == 0) {
    int run = 0, b = 255;
    for (; b >= 0; --b) {
      if (run + hist[b] >= sel_pools) break;
      run += hist[b];
    }
    s_bucket = b;          // -1: fewer than sel_pools + 1 valid keys ... (run == all valid keys < sel_pools) or exactly reached at b
    s_above = run;
  }
  __syncthreads();
  uint32_t thresh = 0u;      // keys above it are taken; with thresh 0 every valid key is
  int take_eq = 0;
  const int hi = s_bucket, above_hi = s_above;
  __syncthreads();
  if (hi >= 0) {
    if (t < 256) hist[t] = 0;
    __syncthreads();
    for (int i = t; i < T; i += 1024) {
      const uint32_t k = ds_key(srow[i]);
      if (k && (int)(k >> 8) == hi) atomicAdd(&hist[k & 255u], 1);
    }
    __syncthreads();
    if (t == 0) {
      int run = above_hi, b = 255;
      for (; b > 0; --b) {
        if (run + hist[b] >= sel_pools) break;
        run += hist[b];
      }
      s_bucket = b;
      s_above = run;
    }
    __syncthreads();
    thresh = ((uint32_t)hi << 8) | (uint32_t)s_bucket;
    take_eq = sel_pools - s_above;
  }

  // ---- emission in index order
  int gt_base = 0, eq_base = 0;
  for (int i0 = 0; i0 < T; i0 += 8192) {
    const int base = i0 + t * 8;
    uint32_t kk[8];
    if (base + 8 <= T) {
      const uint4 v = *reinterpret_cast<const uint4*>(srow + base);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) kk[e] = ds_key(w[e >> 1] >> (16 * (e & 1)));
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) kk[e] = base + e < T ? ds_key(srow[base + e]) : 0u;
    }
    unsigned gtm = 0, eqm = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (kk[e] > thresh) gtm |= 1u << e;
      else if (kk[e] == thresh && kk[e] != 0u) eqm |= 1u << e;
    }
    const int packed = __popc(gtm) | (__popc(eqm) << 16);     // at most 8192 of each per tile: the halves cannot carry into each other
    int incl = packed;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int x = wsum[lane];
      int wi = x;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += n;
      }
      wpre[lane] = wi - x;
      if (lane == 31) tile_total = wi;
    }
    __syncthreads();
    const int excl = wpre[warp] + incl - packed;
    int gt_before = gt_base + (excl & 0xffff), eq_before = eq_base + (excl >> 16);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      int at = -1;
      if ((gtm >> e) & 1u) {
        at = gt_before + min(eq_before, take_eq);
        ++gt_before;
      } else if ((eqm >> e) & 1u) {
        if (eq_before < take_eq) at = gt_before + eq_before;
        ++eq_before;
      }
      if (at >= 0 && at < sel_pools) {
        const int id = (base + e) * DS_P;
        *reinterpret_cast<int4*>(orow + at * DS_P) = make_int4(id, id + 1, id + 2, id + 3);
      }
    }
    gt_base += tile_total & 0xffff;
    eq_base += tile_total >> 16;
    __syncthreads();       // tile_total / wpre are rewritten by the next tile
  }
  const int found = min(gt_base + min(eq_base, take_eq), sel_pools);
  const int first = found * DS_P, tail0 = pos + 1 - tail;
  for (int i = t; i < k_stride - first; i += 1024) orow[first + i] = i < tail ? tail0 + i : -1;
  if (t == 0) { sp_flag[row] = 1; sp_ctx[row] = first + tail; }
}

// grid = (pages per row, rows), 256 threads.  cache / scratch: bf16 [pages][9][64][64].
__global__ void __launch_bounds__(256) dsa_gather_kernel(const uint16_t* __restrict__ cache, const int* __restrict__ block_table, int max_blocks,
                                                         const int* __restrict__ row_seq, const int* __restrict__ sel, int k_stride,
                                                         const int* __restrict__ sp_flag, const int* __restrict__ sp_ctx, uint16_t* __restrict__ scratch,
                                                         int pages_per_row) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.y, pg = blockIdx.x;
  if (!sp_flag[row]) return;
  const int cnt = sp_ctx[row], j0 = pg * DS_PAGE;
  if (j0 >= cnt) return;
  __shared__ long long src_row[DS_PAGE];
  const int* bt = block_table + (size_t)row_seq[row] * max_blocks;
  if (threadIdx.x < DS_PAGE) {
    const int j = j0 + threadIdx.x;
    const int tok = j < cnt ? sel[(size_t)row * k_stride + j] : -1;
    src_row[threadIdx.x] = tok < 0 ? -1ll : (long long)bt[tok / DS_PAGE] * DS_PAGE_ROWS + tok % DS_PAGE;
  }
  __syncthreads();
  const size_t dst_base = ((size_t)row * pages_per_row + pg) * DS_PAGE_ROWS;
  for (int i = threadIdx.x; i < DS_PAGE * 9 * 8; i += 256) {
    const int c = i & 7, b = (i >> 3) % 9, tk = i / 72;
    const long long s = src_row[tk];
    if (s < 0) continue;
    *reinterpret_cast<uint4*>(scratch + (dst_base + (size_t)b * 64 + tk) * 64 + c * 8) =
        __ldg(reinterpret_cast<const uint4*>(cache + ((size_t)s + (size_t)b * 64) * 64 + c * 8));
  }
}

}  // namespace rx

using namespace rx;

// The (key | gate) rows of this call: LayerNorm into the staging rows, every pool whose last member is a row of the call, then the ring.
RX_API int rx_dsa_append(const void* a, int a_ld, int col_k, int col_g, const void* ln_w, const void* ln_b, float eps, const void* ape, const void* row_seq,
                         const void* positions, const void* block_table, int max_blocks, void* stage, void* ring, int ring_len, void* pool, int rows,
                         void* stream) {
  if (rows < 1 || (a_ld | col_k | col_g) % 4 != 0 || ring_len < DS_P || ring_len % DS_P != 0) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  int e = (int)rx::launch(dsa_stage_kernel, dim3(rows), dim3(32), 0, st, (const uint16_t*)a, a_ld, col_k, col_g, (const float*)ln_w, (const float*)ln_b, eps,
                          (uint16_t*)stage);
  if (e != 0) return e;
  e = (int)rx::launch(dsa_pool_kernel, dim3(rows), dim3(32), 0, st, (const uint16_t*)stage, (const uint16_t*)ring, ring_len, (const float*)ape,
                      (const int*)row_seq, (const int*)positions, (const int*)block_table, max_blocks, (uint16_t*)pool);
  if (e != 0) return e;
  return (int)rx::launch(dsa_ring_kernel, dim3(rows), dim3(32), 0, st, (const uint16_t*)stage, (const int*)row_seq, (const int*)positions, rows,
                         (uint16_t*)ring, ring_len);
}

// Scores and selection of `rows` rows (rows of the dense regime are skipped and get sp_flag 0).  max_pools bounds (pos + 1) / 4 over the rows.
RX_API int rx_dsa_select(const void* q, int q_ld, const void* wsrc, int w_ld, int col_w, const void* pool, const void* block_table, int max_blocks,
                         const void* row_seq, const void* positions, int dense_below, float scale, int sel_pools, int max_pools, void* scores, int s_stride,
                         void* out, int k_stride, void* sp_flag, void* sp_ctx, int rows, void* stream) {
  if (rows < 1 || q_ld % 8 != 0 || sel_pools < 1 || sel_pools > 8192 || k_stride % 4 != 0 || k_stride < sel_pools * DS_P + DS_P - 1 || s_stride % 8 != 0 ||
      max_pools > s_stride || max_pools < 1)
    return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  int e = (int)rx::launch(dsa_score_kernel, dim3((max_pools + DS_CHUNK - 1) / DS_CHUNK, rows), dim3(256), 0, st, (const uint16_t*)q, q_ld, (const uint16_t*)wsrc,
                          w_ld, col_w, (const uint16_t*)pool, (const int*)block_table, max_blocks, (const int*)row_seq, (const int*)positions, dense_below,
                          scale, (__half*)scores, s_stride);
  if (e != 0) return e;
  return (int)rx::launch(dsa_select_kernel, dim3(rows), dim3(1024), 0, st, (const uint16_t*)scores, s_stride, (const int*)positions, dense_below, sel_pools,
                         k_stride, (int*)out, (int*)sp_flag, (int*)sp_ctx);
}

RX_API int rx_dsa_gather(const void* cache, const void* block_table, int max_blocks, const void* row_seq, const void* sel, int k_stride, const void* sp_flag,
                         const void* sp_ctx, void* scratch, int pages_per_row, int rows, void* stream) {
  if (rows < 1 || pages_per_row < 1 || pages_per_row * DS_PAGE < k_stride - 1) return (int)cudaErrorInvalidValue;
  return (int)rx::launch(dsa_gather_kernel, dim3(pages_per_row, rows), dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)cache, (const int*)block_table,
                         max_blocks, (const int*)row_seq, (const int*)sel, k_stride, (const int*)sp_flag, (const int*)sp_ctx, (uint16_t*)scratch, pages_per_row);
}
