// Causal flash prefill attention on the 5th-generation tensor cores (sm_100a): S = Q K^T and O += P V are tcgen05 MMAs whose
// accumulators live in tensor memory, K / V pages arrive by TMA, and the online softmax runs in registers one query row per thread.
//
// One CTA = two tiles of 128 query rows of one query head of one sequence.  A step covers one 64-token page in ABSOLUTE key order, so a
// row's arithmetic does not depend on how the prompt was cut into chunks (chunked == whole, as the reference's prefill requires,
// crates/cuda/csrc/attention.cu:768, nemotron_attn_prefill.cu:1-8; tiles, schedule and data path are new).
//
// Tensor memory (512 columns, 256 per tile): Q as the MMA's A operand (64 columns: 128 rows x 128 bf16), the scores S (64 fp32
// columns; the bf16 probabilities P overwrite its first 32 columns and are the A operand of the PV MMA) and the output accumulator O
// (128 fp32 columns).  Both MMAs therefore read only their B operand (a K or V page) from shared memory, and every page brought by
// TMA serves both tiles.
//
// Warps: 0 = TMA producer, 1 = MMA issuer and TMEM owner, 2..5 / 6..9 = softmax of tile 0 / 1 (thread = query row = TMEM lane).  The
// issuer alternates between the tiles (PV_t(j), QK_t(j+1) for t = 0, 1), so one tile's softmax runs while the tensor core works for the
// other, and two softmax warps per scheduler hide each other's latencies.  The running maximum of a row moves only when it grows by more than 2^8 (the probabilities then stay below 2^8, harmless in fp32
// sums and bf16 products); O is rescaled only in those steps.  Every such decision is per row, so a row's bits never depend on its
// neighbours in the tile.  All waits are bounded (status words), no cluster multicast.
#include <cuda.h>
#include "common.cuh"

namespace rx {

constexpr int TC_PAGE = 64;                        // keys per step = one cache page
constexpr int TC_HD = 128;
constexpr int TC_ROWS = 128;                       // query rows per tile (TMEM lanes)
constexpr int TC_TILES = 2;                        // tiles per CTA: two softmax warpgroups take turns on the tensor core
constexpr int TC_STAGES = 4;
constexpr int TC_TILE = TC_PAGE * TC_HD * 2;       // bytes of one K (or V) page of one head: 16 KB
constexpr int TC_THREADS = 64 + TC_TILES * 128;
// tensor-memory columns of tile t: base 256 t; Q (A operand, 64) | S (64 fp32, P bf16 overwrites its first 32) | O (128 fp32)
constexpr int TC_Q = 0, TC_S = 64, TC_O = 128, TC_TCOLS = 256, TC_COLS = 512;

__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
      "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Shared-memory descriptor of an MN-major operand (the contiguous dimension is N; here a V page: keys x head_dim with the head
// dimension contiguous), SWIZZLE_128B: 64 elements of N per 128-byte row, rows = consecutive K (keys) 128 bytes apart, 8 rows per
// 1024-byte swizzle group.  Leading-dimension offset = distance between the 64-element column blocks of N, stride offset = distance
// between the 8-key groups (checked against a plain reference on the device: the swapped assignment gives wrong results).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

struct TcAttnArgs {
  const uint16_t* q;
  const int* block_table;
  const int* seq_ids;
  const int* q_start;
  const int* q_len;
  const int* pos0;
  uint16_t* out;
  int* status;
  int max_blocks, n_q, n_kv;
  float scale_log2;
};

__global__ void __launch_bounds__(TC_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv, const __grid_constant__ TcAttnArgs a) {
  pdl_launch();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* k_sm = smem;                                  // [stage][box (64 d)][64 keys][128 B]
  uint8_t* v_sm = smem + TC_STAGES * TC_TILE;
  uint64_t* bars = (uint64_t*)(smem + 2 * TC_STAGES * TC_TILE);
  uint64_t* k_full = bars;                         // [STAGES] TMA
  uint64_t* v_full = k_full + TC_STAGES;           // [STAGES] TMA
  uint64_t* k_empty = v_full + TC_STAGES;          // [STAGES] commit after the page's last QK
  uint64_t* v_empty = k_empty + TC_STAGES;         // [STAGES] commit after the page's last PV
  uint64_t* s_full = v_empty + TC_STAGES;          // [TILES] commit after QK
  uint64_t* p_ready = s_full + TC_TILES;           // [TILES] the tile's 4 softmax warps
  uint64_t* pv_done = p_ready + TC_TILES;          // [TILES] commit after PV
  uint64_t* q_ready = pv_done + TC_TILES;          // [1] all 8 softmax warps
  uint64_t* drained = q_ready + 1;                 // [1] commit after the last MMA
  uint32_t* tmem_slot = (uint32_t*)(drained + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int s_idx = blockIdx.z, hq = blockIdx.y;
  const int qlen = a.q_len[s_idx];
  const int ntiles = (qlen + TC_TILES * TC_ROWS - 1) / (TC_TILES * TC_ROWS);
  const int qt = ntiles - 1 - (int)blockIdx.x;           // heaviest (latest) query tiles first
  if (qt < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.n_q / a.n_kv, kvh = hq / G;
  const int p0 = a.pos0[s_idx], r_base = a.q_start[s_idx];
  const int* bt = a.block_table + (size_t)a.seq_ids[s_idx] * a.max_blocks;
  const int q_lo = qt * TC_TILES * TC_ROWS;
  // pages tile t needs: keys 0 .. p0 + (its last live row); a tile without live rows needs none (only the second tile can be empty)
  int nst[TC_TILES];
#pragma unroll
  for (int t = 0; t < TC_TILES; ++t) {
    const int first = q_lo + t * TC_ROWS;
    nst[t] = first < qlen ? (p0 + min(qlen, first + TC_ROWS) - 1) / TC_PAGE + 1 : 0;
  }
  const int npages = max(nst[0], nst[1]);

  if (threadIdx.x == 0) {
    for (int i = 0; i < TC_STAGES; ++i) { mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1); }
    for (int i = 0; i < TC_TILES; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 4); mbar_init(&pv_done[i], 1); }
    mbar_init(q_ready, 4 * TC_TILES);
    mbar_init(drained, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tk);
    prefetch_tmap(&tv);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TC_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();                                            // q and the caches were written by the previous kernels
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer: one page of K and of V per step
    if (lane == 0) {
      for (int j = 0; j < npages; ++j) {
        const int st = j % TC_STAGES;
        const int y = (bt[j] * a.n_kv + kvh) * TC_PAGE;
        if (j >= TC_STAGES && !mbar_wait(&k_empty[st], ((j / TC_STAGES) - 1) & 1, abort_flag, a.status, 70, 100)) break;
        mbar_arrive_expect_tx(&k_full[st], TC_TILE);
        tma_load_2d(k_sm + st * TC_TILE, &tk, 0, y, &k_full[st]);
        tma_load_2d(k_sm + st * TC_TILE + 8192, &tk, 64, y, &k_full[st]);
        if (j >= TC_STAGES && !mbar_wait(&v_empty[st], ((j / TC_STAGES) - 1) & 1, abort_flag, a.status, 71, 100)) break;
        mbar_arrive_expect_tx(&v_full[st], TC_TILE);
        tma_load_2d(v_sm + st * TC_TILE, &tv, 0, y, &v_full[st]);
        tma_load_2d(v_sm + st * TC_TILE + 8192, &tv, 64, y, &v_full[st]);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc_f16(TC_ROWS, TC_PAGE, 1, 1);                 // bf16 x bf16, both K-major
      const uint32_t idesc_pv = umma_idesc_f16(TC_ROWS, TC_HD, 1, 1) | (1u << 16);      // B (V) is MN-major
      bool ok = mbar_wait(q_ready, 0, abort_flag, a.status, 72);
      tc_fence_after();
      // S_t = Q_t K(j)^T; the page's last user (the second tile while it still has steps, else the first) frees the K stage
      auto issue_qk = [&](int t, int j) -> bool {
        const int st = j % TC_STAGES;
        if (!mbar_wait(&k_full[st], (j / TC_STAGES) & 1, abort_flag, a.status, 73)) return false;
        tc_fence_after();
        const uint64_t kd = umma_desc_k_sw128(smem_u32(k_sm + st * TC_TILE));
        const uint32_t tb = tmem_base + t * TC_TCOLS;
#pragma unroll
        for (int kk = 0; kk < TC_HD / 16; ++kk)
          tc_mma_f16_ts(tb + TC_S, tb + TC_Q + kk * 8, kd + (uint64_t)((kk >> 2) * (8192 >> 4) + (kk & 3) * 2), idesc_qk, kk != 0);
        if (t == 1 || j >= nst[1]) tc_commit(&k_empty[st]);
        tc_commit(&s_full[t]);
        return true;
      };
      for (int t = 0; t < TC_TILES && ok; ++t)
        if (nst[t] > 0) ok = issue_qk(t, 0);
      for (int j = 0; j < npages && ok; ++j) {
        const int st = j % TC_STAGES;
        for (int t = 0; t < TC_TILES && ok; ++t) {
          if (j >= nst[t]) continue;
          if (!mbar_wait(&p_ready[t], j & 1, abort_flag, a.status, 74)) { ok = false; break; }
          if (!mbar_wait(&v_full[st], (j / TC_STAGES) & 1, abort_flag, a.status, 75)) { ok = false; break; }
          tc_fence_after();
          const uint32_t vbase = smem_u32(v_sm + st * TC_TILE);
          const uint32_t tb = tmem_base + t * TC_TCOLS;
#pragma unroll
          for (int kk = 0; kk < TC_PAGE / 16; ++kk)
            tc_mma_f16_ts(tb + TC_O, tb + TC_S + kk * 8, umma_desc_mn_sw128(vbase + kk * 2048, 8192u, 1024u), idesc_pv, (j | kk) != 0);
          if (t == 1 || j >= nst[1]) tc_commit(&v_empty[st]);
          tc_commit(&pv_done[t]);
          if (j + 1 < nst[t]) ok = issue_qk(t, j + 1);      // overwrites S_t / P_t after PV_t(j) has read it (MMAs run in issue order)
        }
      }
      // every MMA issued so far has completed when this commit arrives: the columns may then be returned
      tc_commit(drained);
      for (int i = 0; i < (1 << 22) && !mbar_try_wait(drained, 0); ++i) {}   // bounded, and not cut short by the abort word
    }
  } else {
    // ---------------------------------------------------------------- softmax warps: thread = query row = TMEM lane of its tile
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                  // row inside the tile
    const int lrow = q_lo + t * TC_ROWS + row;            // row inside the chunk
    const bool live = lrow < qlen;
    const int kmax = p0 + lrow;                           // last key this row may see
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + t * TC_TCOLS;
    const int nsteps = nst[t];
    // Q row -> tensor memory (A operand layout: column c = elements 2c, 2c + 1)
    {
      const uint4* src = reinterpret_cast<const uint4*>(a.q + ((size_t)(r_base + (live ? lrow : 0)) * a.n_q + hq) * TC_HD);
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint4 v = live ? __ldg(src + part * 8 + i) : make_uint4(0u, 0u, 0u, 0u);
          r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
        tc_st_32x32b_x32(lane_addr + TC_Q + part * 32, r);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_ready);
    }
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nsteps && ok; ++j) {
      const uint32_t s_addr = lane_addr + TC_S;
      ok = mbar_wait(&s_full[t], j & 1, abort_flag, a.status, 76);
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * TC_PAGE;
      const bool masked = key0 + TC_PAGE - 1 > kmax;      // some key of this step is beyond this row's last key
      // the row's 64 scores stay in registers for both passes
      uint32_t s0[32], s1[32];
      tc_ld_32x32b_x32(s_addr, s0);
      tc_ld_32x32b_x32(s_addr + 32, s1);
      tc_wait_ld();
      if (masked) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (key0 + i > kmax) s0[i] = 0xFF800000u;        // -inf
          if (key0 + 32 + i > kmax) s1[i] = 0xFF800000u;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])));
      const float ms = mx * a.scale_log2;
      float alpha = 1.f;
      if (ms > m + 8.f || m == -INFINITY) {               // per-row rule: the maximum moves only by big steps
        const float m_new = fmaxf(m, ms);
        alpha = (m == -INFINITY) ? 1.f : ex2(m - m_new);
        m = m_new;
      }
      const float m_use = (m == -INFINITY) ? 0.f : m;
      // probabilities -> bf16 P (the first 32 columns of S), row sum.  exp2(-inf) = 0 covers the masked keys.
      float lsum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float pa = ex2(fmaf(__uint_as_float(s0[2 * i]), a.scale_log2, -m_use));
        const float pb = ex2(fmaf(__uint_as_float(s0[2 * i + 1]), a.scale_log2, -m_use));
        const float pc = ex2(fmaf(__uint_as_float(s1[2 * i]), a.scale_log2, -m_use));
        const float pd = ex2(fmaf(__uint_as_float(s1[2 * i + 1]), a.scale_log2, -m_use));
        lsum += (pa + pb) + (pc + pd);
        pk[i] = pack_bf16x2(pa, pb);
        pk[16 + i] = pack_bf16x2(pc, pd);
      }
      tc_st_32x32b_x32(s_addr, pk);
      l = l * alpha + lsum;
      // O was last written by PV(j-1): rescale it where a row's maximum moved
      if (j > 0) {
        ok = mbar_wait(&pv_done[t], (j - 1) & 1, abort_flag, a.status, 77);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t r[32];
            tc_ld_32x32b_x32(lane_addr + TC_O + ch * 32, r);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tc_st_32x32b_x32(lane_addr + TC_O + ch * 32, r);
          }
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
    // epilogue: O / l -> bf16 -> out
    if (ok && nsteps > 0) ok = mbar_wait(&pv_done[t], (nsteps - 1) & 1, abort_flag, a.status, 78);
    if (ok && nsteps > 0 && *abort_flag == 0) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(a.out + ((size_t)(r_base + (live ? lrow : 0)) * a.n_q + hq) * TC_HD);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t r[32];
        tc_ld_32x32b_x32(lane_addr + TC_O + ch * 32, r);
        tc_wait_ld();
        if (live) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
            dst[ch * 4 + i] = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TC_COLS);
}

}  // namespace rx

using namespace rx;

// Same arguments as rx_attn_prefill (bf16 caches, head_dim 128 only) plus the V-descriptor variant used while the layout is pinned down.
RX_API int rx_attn_prefill_tc(const void* tmap_k, const void* tmap_v, const void* q, const void* block_table, int max_blocks, const void* seq_ids,
                              const void* q_start, const void* q_len, const void* pos0, void* out, int nseq, int max_qlen, int n_q, int n_kv, int hd,
                              float scale, int* status, void* stream, int v_desc_variant) {
  if (hd != TC_HD || n_q % n_kv != 0 || nseq <= 0 || max_qlen <= 0) return (int)cudaErrorInvalidValue;
  const int smem = 2 * TC_STAGES * TC_TILE + 256 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  TcAttnArgs a;
  a.q = (const uint16_t*)q; a.block_table = (const int*)block_table; a.seq_ids = (const int*)seq_ids; a.q_start = (const int*)q_start;
  a.q_len = (const int*)q_len; a.pos0 = (const int*)pos0; a.out = (uint16_t*)out; a.status = status; a.max_blocks = max_blocks;
  a.n_q = n_q; a.n_kv = n_kv; a.scale_log2 = scale * 1.4426950408889634f;
  (void)v_desc_variant;
  dim3 grid((max_qlen + TC_TILES * TC_ROWS - 1) / (TC_TILES * TC_ROWS), n_q, nseq);
  rx::launch(attn_prefill_tc_kernel, dim3(grid), dim3(TC_THREADS), smem, (cudaStream_t)stream, *(const CUtensorMap*)tmap_k, *(const CUtensorMap*)tmap_v, a);
  return (int)cudaGetLastError();
}
