// EXL3 4.0 bpw trellis-dequant GEMM with the decoded weights held in TENSOR MEMORY (sm_100a).
//
// Same contract as exl3_gemm.cu (part[split][row][n] = partial sums of xr @ W_q; finish kernels apply the output
// rotation), different data path: the decode warps never write the fp16 weight tile to shared memory.  Each decode
// thread owns ONE output column n of the 128-column strip (TMEM lane n) and produces that column's 64 k-values of the
// K chunk as 32 packed registers, which one tcgen05.st puts into TMEM; the MMA then takes A from TMEM and only B (the
// activations, brought by TMA) from shared memory.  That removes 32 KB of shared-memory traffic per K chunk (the
// operand write and its read by the tensor core), the swizzled-store address arithmetic, the bank conflicts and the
// generic->async proxy fence, which together bounded the shared-memory variant well below the tensor-core rate.
//
// Why a thread can own a column: stream positions 32g..32g+31 of a 16x16 tile are the 16 k-rows of tile columns g and
// g+8, interleaved four values at a time, so "column g (or g+8) of tile (kt, nt)" is every other group of four values
// of eighth g: all 4 words are read, half the values are decoded, nothing is decoded twice.
//
// Warp roles: warp 0 producer (bulk copies of compressed trellis rows, 2-D tiled TMA of xr), warp 1 TMEM owner + MMA
// issuer, then NG decode groups of 4 warps (a group covers the 4 TMEM lane quarters and takes every NG-th K chunk);
// the first group also runs the epilogue.  Bounded waits everywhere; no cluster multicast.
#include <cuda.h>
#include "exl3_decode.cuh"
#include "tp.cuh"

namespace rx {

constexpr int TM_KCH = 128;                       // k per pipeline chunk: 8 k-tiles, two 128-byte swizzle rows of fp16
constexpr int TM_STRIP = 128;
constexpr int TM_RAW_STAGES_MAX = 6;
__host__ __device__ constexpr int tm_raw_stages(int ng) { return ng == 4 ? 4 : 6; }   // ring of compressed chunks (8 KB each); the 256-row variant needs the room for B
constexpr int TM_OP_STAGES = 3;                   // activation (B) ring depth
// A-stage ring depth.  A decode group waits for "the MMA that last read this stage"; that wait is only sound while the group
// cannot run two phases ahead of the barrier, which needs at least as many A stages as decode groups.
__host__ __device__ constexpr int tm_a_stages(int ng) { return ng > 3 ? ng : 3; }
constexpr int TM_RAW_STAGE_BYTES = 8 * 8 * 128;   // 8 k-tile rows x 8 tiles x 128 B (4.0 bpw)
constexpr int TM_A_COLS = TM_KCH / 2;             // TMEM columns of one A stage (two fp16 per column)

__host__ __device__ inline int tm_smem_bytes(int brows, int ng) { return TM_OP_STAGES * brows * 256 + tm_raw_stages(ng) * TM_RAW_STAGE_BYTES + 256; }

// Warps: 0 = weight producer, 1 = MMA issuer (+TMEM owner), 2 = activation producer, then NG decode groups of 4 consecutive warps.
// A warp may touch the TMEM lane quarter (warp index mod 4); any 4 consecutive warps cover the four quarters, so the groups need
// no alignment and no spare warp (fewer threads per CTA leave more registers per decode thread at two CTAs per SM).
constexpr int TM_ROLE_WARPS = 3;
template <int CB, int NG>
__global__ void __launch_bounds__(TM_ROLE_WARPS * 32 + NG * 128, (NG <= 3 ? 2 : 1))
exl3_gemm_tm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, float* __restrict__ part, int rows,
                    int K, int N, int splits, int brows, int* status, const __grid_constant__ GemmTp tp) {
  constexpr int TM_RAW_STAGES = tm_raw_stages(NG);
  pdl_launch();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int b_half = brows * 128;                    // one [brows x 64] swizzled sub-tile
  const int b_stage = 2 * b_half;
  uint8_t* b_base = smem;
  uint8_t* raw_base = smem + TM_OP_STAGES * b_stage;
  uint64_t* bars = (uint64_t*)(raw_base + TM_RAW_STAGES * TM_RAW_STAGE_BYTES);
  constexpr int SA = tm_a_stages(NG);
  uint64_t* a_full = bars;                           // [SA] 4 decode warps
  uint64_t* a_empty = a_full + SA;                   // [SA] tcgen05.commit
  uint64_t* b_full = a_empty + SA;                   // [OP] activation producer expect_tx
  uint64_t* b_empty = b_full + TM_OP_STAGES;         // [OP] tcgen05.commit
  uint64_t* raw_full = b_empty + TM_OP_STAGES;       // [RAW] weight producer expect_tx
  uint64_t* raw_empty = raw_full + TM_RAW_STAGES;    // [RAW] 4 decode warps
  uint64_t* acc_full = raw_empty + TM_RAW_STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int strip = blockIdx.x, split = blockIdx.y, row_tile = blockIdx.z;
  const int nchunks_total = K / TM_KCH;
  const int c_begin = (int)((long long)nchunks_total * split / splits);
  const int c_end = (int)((long long)nchunks_total * (split + 1) / splits);
  const int nchunks = c_end - c_begin;
  const int acc_cols = (brows + 31) & ~31;
  uint32_t ncols = 32;
  while ((int)ncols < acc_cols + tm_a_stages(NG) * TM_A_COLS) ncols <<= 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < SA; ++i) { mbar_init(&a_full[i], 4); mbar_init(&a_empty[i], 1); }
    for (int i = 0; i < TM_OP_STAGES; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
    for (int i = 0; i < TM_RAW_STAGES; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 4); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_w);
    // the weight stream does not wait for the rest of the prologue (TMEM allocation, CTA barrier)
    for (int c = 0; c < nchunks && c < TM_RAW_STAGES; ++c) {
      mbar_arrive_expect_tx(&raw_full[c], TM_RAW_STAGE_BYTES);
      tma_load_2d(raw_base + c * TM_RAW_STAGE_BYTES, &tmap_w, strip * 256, (c_begin + c) * 8, &raw_full[c]);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, ncols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();   // the weights were not written by the previous kernel, everything else may have been
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t a_tmem0 = tmem_base + acc_cols;

  if (warp == 0) {
    // ---- weight producer: ONE 2-D tiled copy per chunk (8 k-tile rows x 1 KB of this strip)
    if (lane == 0) {
      int y = (c_begin + TM_RAW_STAGES) * 8;
      const int x = strip * 256;
      for (int c = TM_RAW_STAGES; c < nchunks; ++c, y += 8) {   // the first ring's worth was issued in the prologue
        const int s = c % TM_RAW_STAGES;
        if (!mbar_wait(&raw_empty[s], ((c / TM_RAW_STAGES) - 1) & 1, abort_flag, status, 110, 1000)) break;
        mbar_arrive_expect_tx(&raw_full[s], TM_RAW_STAGE_BYTES);
        tma_load_2d(raw_base + s * TM_RAW_STAGE_BYTES, &tmap_w, x, y, &raw_full[s]);
      }
    }
  } else if (warp == 2) {
    // ---- activation producer: two [brows x 64] swizzled boxes per chunk
    if (lane == 0) {
      int x = c_begin * TM_KCH;
      const int y = row_tile * brows;
      int waited_src = -1;
      const unsigned ticket = (tp.in_flag != nullptr) ? tp_ticket(tp.epoch, tp.use_index) : 0u;
      for (int c = 0; c < nchunks; ++c, x += TM_KCH) {
        const int s = c % TM_OP_STAGES;
        if (tp.in_flag != nullptr) {
          // all-gather -> GEMM: this K chunk was pushed into the local buffer by rank `src`; consume it as soon as it has landed
          const int src = x / tp.in_cols_per_src;
          if (src != waited_src) {
            if (!tp_wait_flag(tp.in_flag + src, ticket, status, 150)) { *abort_flag = 1; break; }
            waited_src = src;
          }
        }
        if (c >= TM_OP_STAGES && !mbar_wait(&b_empty[s], ((c / TM_OP_STAGES) - 1) & 1, abort_flag, status, 111, NG <= 3 ? 500 : 0)) break;
        mbar_arrive_expect_tx(&b_full[s], (uint32_t)b_stage);
        tma_load_2d(b_base + s * b_stage, &tmap_x, x, y, &b_full[s]);
        tma_load_2d(b_base + s * b_stage + b_half, &tmap_x, x + 64, y, &b_full[s]);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: A from tensor memory, B from shared memory
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(TM_STRIP, brows, 0, 0);
      const uint64_t desc0 = umma_desc_k_sw128(smem_u32(b_base));
      const uint32_t half_units = (uint32_t)b_half >> 4, stage_units = (uint32_t)b_stage >> 4;
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % TM_OP_STAGES, sa = c % SA;
        if (!mbar_wait(&b_full[s], (c / TM_OP_STAGES) & 1, abort_flag, status, 120)) break;
        if (!mbar_wait(&a_full[sa], (c / SA) & 1, abort_flag, status, 121, NG <= 3 ? 250 : 0)) break;   // decode class: the decode warps set the pace
        tc_fence_after();
        const uint64_t bd = desc0 + (uint64_t)(s * stage_units);
        const uint32_t at = a_tmem0 + sa * TM_A_COLS;
#pragma unroll
        for (int k = 0; k < TM_KCH / 16; ++k)
          tc_mma_f16_ts(tmem_base, at + k * 8, bd + (uint64_t)((k >> 2) * half_units + (k & 3) * 2), idesc, (c | k) != 0);
        tc_commit(&a_empty[sa]);
        tc_commit(&b_empty[s]);
      }
      tc_commit(acc_full);
    }
  } else if (warp >= TM_ROLE_WARPS) {
    const int dw = warp - TM_ROLE_WARPS;
    const int grp = dw >> 2;
    const int q = warp & 3;                       // TMEM lane quarter this warp may touch
    const int n = q * 32 + lane;                  // output column of the strip owned by this thread
    const int nt = n >> 4, b2 = (n >> 3) & 1, g = n & 7;
    const uint32_t sh = b2 ? 32u : 16u;           // b2 = 0: the 4 values that straddle the word boundary; b2 = 1: the word's own 4
    const int prev_lane = (lane & ~7) | ((lane + 7) & 7);
    const uint32_t st_addr = a_tmem0 + ((uint32_t)(q * 32) << 16);
    const int tile_off = nt * 8 + g;              // uint4 index of this thread's eighth inside a k-tile row
    bool ok = true;
    for (int c = grp; c < nchunks && ok; c += NG) {
      const int rs = c % TM_RAW_STAGES, os = c % SA;
      ok = mbar_wait(&raw_full[rs], (c / TM_RAW_STAGES) & 1, abort_flag, status, 130, 200);
      if (!ok) break;
      const uint32_t raw4 = smem_u32(raw_base + rs * TM_RAW_STAGE_BYTES) + (uint32_t)tile_off * 16u;
      bool waited = false;
#pragma unroll
      for (int qt = 0; qt < 4; ++qt) {
        // two k-tiles at a time: the thread's eighth of each (4 words) and, from the lane before it, the word those follow.
        // Small steps keep the live registers low (more resident decode warps) and the unrolled body short.
        uint4 cur[2];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) cur[kk] = lds128(raw4 + (uint32_t)((qt * 2 + kk) * 1024));
        uint32_t prev[2];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) prev[kk] = __shfl_sync(0xffffffffu, cur[kk].w, prev_lane);
        if (qt == 3) {
          release_read_stage(&raw_empty[rs], lane);   // the stage's last read has landed in registers; proxy fence before the refill
        }
        uint32_t regs[16];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const uint32_t w[5] = {prev[kk], cur[kk].x, cur[kk].y, cur[kk].z, cur[kk].w};
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            const uint32_t X = __funnelshift_lc(w[m + 1], w[m], sh);
            uint32_t s0, s1, s2, s3;
            extract4<CB != CB_MUL1>(X, s0, s1, s2, s3);
            regs[8 * kk + m] = pair_to_half2<CB>(s0, s1);       // k = 16 kt + 2m, 2m+1
            regs[8 * kk + 4 + m] = pair_to_half2<CB>(s2, s3);   // k = 16 kt + 8 + 2m, +1
          }
        }
        if (!waited) {
          if (c >= SA) ok = mbar_wait(&a_empty[os], ((c / SA) - 1) & 1, abort_flag, status, 131, NG == 4 ? 64 : 0);   // prefill class: the tensor core sets the pace
          waited = true;
          if (!ok) break;
          tc_fence_after();
        }
        tc_st_32x32b_x16(st_addr + os * TM_A_COLS + qt * 16, regs);
      }
      if (!ok) break;
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[os]);
    }
    if (dw < 4) {
      const bool done = mbar_wait(acc_full, 0, abort_flag, status, 140, 100);
      tc_fence_after();
      if (done && *abort_flag == 0) {
        float* out;
        size_t ld;
        if (tp.strips_per_rank > 0) {
          // GEMM -> reduce-scatter: the tile goes straight into the owning rank's buffer over NVLink (plane [src = this rank][split])
          const int dest = strip / tp.strips_per_rank;
          ld = (size_t)tp.out_ld;
          out = tp.out[dest] + ((size_t)(tp.rank * splits + split) * tp.rows_cap) * ld + (strip % tp.strips_per_rank) * TM_STRIP + n;
        } else {
          ld = (size_t)N;
          out = part + ((size_t)split * rows) * N + strip * TM_STRIP + n;
        }
        const int row0 = row_tile * brows;
        for (int cb = 0; cb < brows; cb += 16) {
          if (row0 + cb >= rows) break;
          uint32_t r[16];
          tc_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + cb, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int row = row0 + cb + i;
            if (row < rows) out[(size_t)row * ld] = __uint_as_float(r[i]);
          }
        }
      }
      if (tp.strips_per_rank > 0) {
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
        if (dw == 0 && lane == 0 && *abort_flag == 0)
          tp_publish_last(tp.local_count, gridDim.x * gridDim.y * gridDim.z, tp.out_flag, tp.ranks, tp.rank, tp_ticket(tp.epoch, tp.use_index));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag != 0 && lane == 0) mbar_wait(acc_full, 0, abort_flag, nullptr, 141);
    __syncwarp();
    tmem_dealloc(tmem_base, ncols);
  }
}

int make_tmap_f16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

int make_tmap_trellis(CUtensorMap* out, const void* base, uint64_t kt_rows, uint64_t row_words, uint32_t box_words, uint32_t box_rows);

template <int CB, int NG>
static int launch_tm(const CUtensorMap& tm, const CUtensorMap& tw, float* part, int rows, int K, int N, int splits, int brows, int row_tiles,
                     int* status, cudaStream_t st, const GemmTp& tp) {
  int smem = tm_smem_bytes(brows, NG) + 1024;
  if (NG <= 3 && smem < 80 * 1024) smem = 80 * 1024;   // at most two CTAs per SM: each allocates 256 TMEM columns
  if (smem > 232448) return (int)cudaErrorInvalidValue;
  auto kern = exl3_gemm_tm_kernel<CB, NG>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(N / TM_STRIP, splits, row_tiles);
  rx::launch(kern, dim3(grid), dim3(TM_ROLE_WARPS * 32 + NG * 128), smem, st, tm, tw, part, rows, K, N, splits, brows, status, tp);
  return (int)cudaGetLastError();
}

}  // namespace rx

using namespace rx;

extern "C" int rx_exl3_tile_rows(int rows);

static int gemm_b4(const void* xr, int rows, int K, const void* trellis, int N, int codebook, void* part, int splits, int* status, void* stream,
                   const GemmTp& tp) {
  if (rows <= 0 || K % 128 != 0 || N % 128 != 0 || splits < 1 || splits > K / TM_KCH) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)xr) & 15) != 0 || (((uintptr_t)trellis) & 15) != 0) return (int)cudaErrorMisalignedAddress;
  const int brows = rx_exl3_tile_rows(rows);
  const int row_tiles = (rows + brows - 1) / brows;
  CUtensorMap tm;
  int e = make_tmap_f16_2d(&tm, xr, (uint64_t)rows, (uint64_t)K, (uint32_t)brows);
  if (e != 0) return e;
  CUtensorMap tw;
  e = make_tmap_trellis(&tw, trellis, (uint64_t)(K / 16), (uint64_t)(N / 16) * 32, 256, 8);
  if (e != 0) return e;
  cudaStream_t st = (cudaStream_t)stream;
  float* p = (float*)part;
  const bool big = brows > 64;   // one CTA per SM with 16 decode warps, else two CTAs per SM with 12 each
#define RX_TM(CBV) (big ? launch_tm<CBV, 4>(tm, tw, p, rows, K, N, splits, brows, row_tiles, status, st, tp) \
                        : launch_tm<CBV, 3>(tm, tw, p, rows, K, N, splits, brows, row_tiles, status, st, tp))
  switch (codebook) {
    case CB_3INST: return RX_TM(CB_3INST);
    case CB_MCG: return RX_TM(CB_MCG);
    case CB_MUL1: return RX_TM(CB_MUL1);
    default: return (int)cudaErrorInvalidValue;
  }
#undef RX_TM
}

// 4.0 bpw only (twice == 8), codebooks 3inst / mcg / mul1.  Same arguments as rx_exl3_gemm.
RX_API int rx_exl3_gemm_b4(const void* xr, int rows, int K, const void* trellis, int N, int codebook, void* part, int splits, int* status,
                           void* stream) {
  GemmTp tp = {};
  tp.ranks = 1;
  return gemm_b4(xr, rows, K, trellis, N, codebook, part, splits, status, stream, tp);
}

// Tensor-parallel form.  `tp_desc` points at a HOST copy of GemmTp (filled by the comm layer: peer buffers, flags, ticket source).
// strips_per_rank > 0 makes the epilogue a reduce-scatter (tiles pushed to their owner); in_flag != nullptr makes the activation
// loads wait for the all-gathered input to land, source rank by source rank.
RX_API int rx_exl3_gemm_b4_tp(const void* xr, int rows, int K, const void* trellis, int N, int codebook, void* part, int splits, int* status,
                              void* stream, const void* tp_desc) {
  if (tp_desc == nullptr) return (int)cudaErrorInvalidValue;
  const GemmTp tp = *(const GemmTp*)tp_desc;
  if (tp.ranks < 1 || tp.ranks > TP_MAX) return (int)cudaErrorInvalidValue;
  if (tp.strips_per_rank > 0 && (N / TM_STRIP) != tp.strips_per_rank * tp.ranks) return (int)cudaErrorInvalidValue;
  if (tp.in_flag != nullptr && (tp.in_cols_per_src % TM_KCH != 0 || tp.in_cols_per_src * tp.ranks != K)) return (int)cudaErrorInvalidValue;
  return gemm_b4(xr, rows, K, trellis, N, codebook, part, splits, status, stream, tp);
}
