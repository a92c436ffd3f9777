// EXL3 trellis-dequant GEMM on tcgen05 (sm_100a).
//
//   part[split][row][n] = sum over this split's k of  xr[row][k] * W_q[k][n]
//
// xr is the already rotated input (x * suh -> 128-point Hadamard -> fp16), W_q the trellis-coded weight.
// The output Hadamard, svh scale, bias, split reduction and whatever follows (residual add, RMSNorm, SwiGLU,
// next layer's input rotation) are applied by the finish kernels in exl3_aux.cu, in split order, so the
// K reduction order is a function of (K, N) alone and a row's bits never depend on the other rows.
// Semantics to match: reference crates/cuda/csrc/exl3_linear.cu:136-412 (rot_in -> linear -> rot_out) and the
// float64 layer crates/exl3/src/lib.rs:215-260; the schedule is new.
//
// CTA = one 128-column strip x one K range x one row tile.  "Swap-AB": the decoded weight strip is the MMA's
// A operand (M = 128 output columns, K-major, SWIZZLE_128B in shared memory), the activations are the B operand
// (N = rows of the tile, 16..256), so one weight decode serves every row and a batch-1 step still runs a
// full-width tensor-core instruction.  Accumulator D^T[n][row] lives in TMEM (lane = output column).
//
// Warp roles (320 threads): warp 0 = TMA producer (1-D bulk copies of the compressed trellis into a deep ring,
// 2-D tiled loads of xr), warp 1 = TMEM owner + single-thread tcgen05.mma issuer, warps 2..9 = two decode groups
// that turn compressed tiles into fp16 operand tiles (alternating K chunks), warps 2..5 double as the epilogue.
// No cluster multicast anywhere; every wait is bounded and unwinds through the abort flag.
#include <cuda.h>
#include "exl3_decode.cuh"

namespace rx {

constexpr int KCH = 64;            // k per pipeline chunk (= one 128-byte swizzle row of fp16)
constexpr int STRIP = 128;         // output columns per CTA (= one output Hadamard block = MMA M)
constexpr int NDEC_GROUPS = 2;
constexpr int NDEC_WARPS = 8;
constexpr int GEMM_THREADS = 64 + NDEC_WARPS * 32;
constexpr int RAW_STAGES = 8;      // compressed-trellis ring depth
constexpr int OP_STAGES = 3;       // operand (A + B) ring depth; must be >= NDEC_GROUPS (a group may not run two barrier phases ahead)
static_assert(OP_STAGES >= NDEC_GROUPS, "operand ring shallower than the number of decode groups");

struct GemmSmemLayout {
  int a_off, b_off, raw_off, bar_off, total;
};

__host__ __device__ inline GemmSmemLayout gemm_layout(int twice, int brows) {
  GemmSmemLayout L;
  const int a_stage = STRIP * KCH * 2;        // 16 KB
  const int b_stage = brows * KCH * 2;
  const int raw_stage = 4 * 8 * 16 * twice;   // 4 k-tiles x 8 n-tiles x (32*bits) bytes
  L.a_off = 0;
  L.b_off = L.a_off + OP_STAGES * a_stage;
  L.raw_off = L.b_off + OP_STAGES * b_stage;
  L.bar_off = L.raw_off + RAW_STAGES * raw_stage;
  L.total = L.bar_off + 256;
  return L;
}

template <int TWICE, int CB>
__global__ void __launch_bounds__(GEMM_THREADS, 2)
exl3_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const uint32_t* __restrict__ trellis, float* __restrict__ part,
                 int rows, int K, int N, int splits, int brows, int row_tiles, int* status, const int* __restrict__ tile_tab,
                 size_t expert_words) {
  pdl_launch();
  // Row window of this CTA.  Plain GEMM: tile z of the row dimension.  Grouped (mixture-of-experts) form: tile_tab[z] =
  // {expert, first row, row count} written by the planning kernel; rows are pairs sorted by expert, every expert has its own
  // trellis (expert_words apart); a tile with no rows exits before it allocates anything.
  int g_row0 = blockIdx.z * brows;
  int g_nrows = rows - g_row0 < brows ? rows - g_row0 : brows;
  if (tile_tab != nullptr) {
    pdl_wait();
    const int e = tile_tab[3 * blockIdx.z];
    g_row0 = tile_tab[3 * blockIdx.z + 1];
    g_nrows = tile_tab[3 * blockIdx.z + 2];
    if (g_nrows <= 0) return;
    trellis += (size_t)e * expert_words;
  }
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled operand tiles
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const GemmSmemLayout L = gemm_layout(TWICE, brows);
  constexpr int A_STAGE = STRIP * KCH * 2;
  const int b_stage = brows * KCH * 2;
  constexpr int RAW_STAGE = 4 * 8 * 16 * TWICE;
  constexpr int TILE_WORDS = 4 * TWICE;           // 32-bit words per 16x16 tile
  constexpr int ROW_BYTES = 8 * TILE_WORDS * 4;   // one k-tile row of the strip (8 tiles)

  uint64_t* bars = (uint64_t*)(smem + L.bar_off);
  uint64_t* op_full = bars;                       // [OP_STAGES] decode warps (4) + producer expect_tx (1)
  uint64_t* op_empty = bars + OP_STAGES;          // [OP_STAGES] tcgen05.commit
  uint64_t* raw_full = bars + 2 * OP_STAGES;      // [RAW_STAGES] producer expect_tx
  uint64_t* raw_empty = raw_full + RAW_STAGES;    // [RAW_STAGES] decode warps of the owning group (4)
  uint64_t* acc_full = raw_empty + RAW_STAGES;    // [1]
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int strip = blockIdx.x;
  const int split = blockIdx.y;
  const int nchunks_total = K / KCH;
  const int c_begin = (int)((long long)nchunks_total * split / splits);
  const int c_end = (int)((long long)nchunks_total * (split + 1) / splits);
  const int nchunks = c_end - c_begin;
  const int nt_total = N / 16;
  uint32_t ncols = 32;
  while ((int)ncols < brows) ncols <<= 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < OP_STAGES; ++i) { mbar_init(&op_full[i], NDEC_WARPS / NDEC_GROUPS + 1); mbar_init(&op_empty[i], 1); }
    for (int i = 0; i < RAW_STAGES; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], NDEC_WARPS / NDEC_GROUPS); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_x);
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

  if (warp == 0) {
    // ------------------------------------------------ producer
    if (lane == 0) {
      // Step i issues the compressed weights of chunk i and the activation tile of chunk i - AHEAD: the weight
      // stream (HBM) runs ahead of the activation tiles (L2 hits).  Neither wait can block the other ring for good:
      // decode warps release a raw stage before they wait for an operand stage.
      constexpr int AHEAD = 4;
      bool ok = true;
      for (int i = 0; i < nchunks + AHEAD && ok; ++i) {
        if (i < nchunks) {
          const int c = i, s = c % RAW_STAGES;
          if (c >= RAW_STAGES) ok = mbar_wait(&raw_empty[s], ((c / RAW_STAGES) - 1) & 1, abort_flag, status, 10);
          if (!ok) break;
          mbar_arrive_expect_tx(&raw_full[s], RAW_STAGE);
          const int kt0 = (c_begin + c) * 4;
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const uint32_t* src = trellis + ((size_t)(kt0 + r) * nt_total + (size_t)strip * 8) * TILE_WORDS;
            bulk_g2s(smem + L.raw_off + s * RAW_STAGE + r * ROW_BYTES, src, ROW_BYTES, &raw_full[s]);
          }
        }
        if (i >= AHEAD) {
          const int c = i - AHEAD, s = c % OP_STAGES;
          if (c >= OP_STAGES) ok = mbar_wait(&op_empty[s], ((c / OP_STAGES) - 1) & 1, abort_flag, status, 11);
          if (!ok) break;
          mbar_arrive_expect_tx(&op_full[s], (uint32_t)b_stage);
          tma_load_2d(smem + L.b_off + s * b_stage, &tmap_x, (c_begin + c) * KCH, g_row0, &op_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(STRIP, brows, 0, 0);
      bool ok = true;
      for (int c = 0; c < nchunks && ok; ++c) {
        const int s = c % OP_STAGES;
        ok = mbar_wait(&op_full[s], (c / OP_STAGES) & 1, abort_flag, status, 20);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + L.a_off + s * A_STAGE);
        const uint32_t b_addr = smem_u32(smem + L.b_off + s * b_stage);
#pragma unroll
        for (int k = 0; k < KCH / 16; ++k) {
          tc_mma_f16(tmem_base, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc, (c | k) != 0);
        }
        tc_commit(&op_empty[s]);
      }
      tc_commit(acc_full);  // arrives when every MMA issued so far has completed (also on the abort path)
    }
  } else {
    // ------------------------------------------------ decode warps
    const int dw = warp - 2;
    const int grp = dw / (NDEC_WARPS / NDEC_GROUPS);
    const int t = (dw % (NDEC_WARPS / NDEC_GROUPS)) * 32 + lane;  // 0..127 inside the group
    const int h = t & 3, ktl = (t >> 2) & 3, nt = t >> 4;
    bool ok = true;
    if constexpr (TWICE == 8) {
      // ---- 4.0 bpw fast path.  A thread owns the two eighths 2h and 2h+1 of its tile (two 16-byte loads, conflict free
      // because odd k-tiles take them in the other order), gets the one word before each from its own other eighth or from
      // the neighbouring lane, and releases the raw stage as soon as everything is in registers.
      const int x = ktl & 1;
      const int g1 = 2 * h + x, g2 = 2 * h + 1 - x;
      const int n1 = 16 * nt + g1, n2 = 16 * nt + g2;
      const int o1 = (n1 >> 3) * 1024 + (n1 & 7) * 128 + (((2 * ktl) ^ (g1 & 7)) << 4);
      const int o2 = (n2 >> 3) * 1024 + (n2 & 7) * 128 + (((2 * ktl) ^ (g2 & 7)) << 4);
      const int src = (lane & ~3) | ((h + 3) & 3);
      for (int c = grp; c < nchunks && ok; c += NDEC_GROUPS) {
        const int rs = c % RAW_STAGES, os = c % OP_STAGES;
        ok = mbar_wait(&raw_full[rs], (c / RAW_STAGES) & 1, abort_flag, status, 30);
        if (!ok) break;
        const uint4* tile4 = reinterpret_cast<const uint4*>(smem + L.raw_off + rs * RAW_STAGE) + (ktl * 8 + nt) * 8;
        const uint4 first = tile4[g1], second = tile4[g2];
        const uint32_t sh_second = __shfl_sync(0xffffffffu, second.w, src), sh_first = __shfl_sync(0xffffffffu, first.w, src);
        const uint32_t w1[5] = {x ? second.w : sh_second, first.x, first.y, first.z, first.w};
        const uint32_t w2[5] = {x ? sh_first : first.w, second.x, second.y, second.z, second.w};
        release_read_stage(&raw_empty[rs], lane);      // generic-proxy reads, async-proxy refill: proxy fence before the release
        if (c >= OP_STAGES) ok = mbar_wait(&op_empty[os], ((c / OP_STAGES) - 1) & 1, abort_flag, status, 31);
        if (!ok) break;
        uint8_t* a_tile = smem + L.a_off + os * A_STAGE;
        {
          uint32_t h2[16];
          decode32_b4<CB>(w1, h2);
          uint8_t* p = a_tile + o1;
          *reinterpret_cast<uint4*>(p) = eighth_chunk(h2, 0, 0);
          *reinterpret_cast<uint4*>((uint8_t*)((uintptr_t)p ^ 16)) = eighth_chunk(h2, 0, 1);
          *reinterpret_cast<uint4*>(p + 1024) = eighth_chunk(h2, 1, 0);
          *reinterpret_cast<uint4*>((uint8_t*)((uintptr_t)(p + 1024) ^ 16)) = eighth_chunk(h2, 1, 1);
        }
        {
          uint32_t h2[16];
          decode32_b4<CB>(w2, h2);
          uint8_t* p = a_tile + o2;
          *reinterpret_cast<uint4*>(p) = eighth_chunk(h2, 0, 0);
          *reinterpret_cast<uint4*>((uint8_t*)((uintptr_t)p ^ 16)) = eighth_chunk(h2, 0, 1);
          *reinterpret_cast<uint4*>(p + 1024) = eighth_chunk(h2, 1, 0);
          *reinterpret_cast<uint4*>((uint8_t*)((uintptr_t)(p + 1024) ^ 16)) = eighth_chunk(h2, 1, 1);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&op_full[os]);
      }
    } else
    for (int c = grp; c < nchunks && ok; c += NDEC_GROUPS) {
      const int rs = c % RAW_STAGES, os = c % OP_STAGES;
      ok = mbar_wait(&raw_full[rs], (c / RAW_STAGES) & 1, abort_flag, status, 30);
      if (!ok) break;
      const uint32_t* tile = (const uint32_t*)(smem + L.raw_off + rs * RAW_STAGE) + (ktl * 8 + nt) * TILE_WORDS;
      if (c >= OP_STAGES) ok = mbar_wait(&op_empty[os], ((c / OP_STAGES) - 1) & 1, abort_flag, status, 31);
      if (!ok) break;
      uint8_t* a_tile = smem + L.a_off + os * A_STAGE;
      if constexpr (TWICE % 2 == 0) {
        // two word-aligned eighths per thread; odd k-tiles take them in the other order, which makes the 8 threads
        // of a store phase hit 8 distinct 16-byte columns of the swizzled tile (no bank conflicts)
        const int x = ktl & 1;
#pragma unroll
        for (int slot = 0; slot < 2; ++slot) {
          const int g = 2 * h + (slot ^ x);
          uint32_t h2[16];
          decode_span<TWICE, CB, 32>(tile, g * (TWICE / 2), h2);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int b2 = i >> 1, kc = i & 1;
            const int n_local = 16 * nt + g + 8 * b2;
            const int chunk = (2 * ktl + kc) ^ (g & 7);
            *reinterpret_cast<uint4*>(a_tile + (n_local >> 3) * 1024 + (n_local & 7) * 128 + chunk * 16) = eighth_chunk(h2, b2, kc);
          }
        }
      } else {
        uint32_t h2[32];
        decode_span<TWICE, CB, 64>(tile, h * TWICE, h2);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int a = i >> 2, b2 = (i >> 1) & 1, kc = i & 1;
          const int n_local = 16 * nt + 2 * h + a + 8 * b2;
          const int chunk = (2 * ktl + kc) ^ (n_local & 7);
          *reinterpret_cast<uint4*>(a_tile + (n_local >> 3) * 1024 + (n_local & 7) * 128 + chunk * 16) = quarter_chunk(h2, a, b2, kc);
        }
      }
      release_read_stage(&raw_empty[rs], lane);        // (the fence also covers the operand tile written above)
      __syncwarp();
      if (lane == 0) mbar_arrive(&op_full[os]);
    }
    // ------------------------------------------------ epilogue (warps 2..5 cover TMEM lane quarters 2,3,0,1)
    if (dw < 4) {
      const bool done = mbar_wait(acc_full, 0, abort_flag, status, 40);
      tc_fence_after();
      if (done && *abort_flag == 0) {
        const int q = warp & 3;
        const int n = strip * STRIP + q * 32 + lane;
        float* out = part + ((size_t)split * rows) * N + n;
        const int row0 = g_row0;
        for (int cb = 0; cb < brows; cb += 16) {
          if (cb >= g_nrows) break;  // warp-uniform
          uint32_t r[16];
          tc_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + cb, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (cb + i < g_nrows) out[(size_t)(row0 + cb + i) * N] = __uint_as_float(r[i]);
          }
        }
      }
    }
  }
  // ------------------------------------------------ teardown: every role falls through to here
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag != 0 && lane == 0) {
      // make sure no MMA is still writing TMEM before it is freed (bounded)
      mbar_wait(acc_full, 0, abort_flag, nullptr, 41);
    }
    __syncwarp();
    tmem_dealloc(tmem_base, ncols);
  }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 2-D fp16 row-major [rows, cols] tensor map with a (64 x box_rows) box and 128-byte swizzle.
int make_tmap_f16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Trellis viewed as uint32 [K/16 rows, row_words]: a box is `box_rows` k-tile rows x `box_words` words, unswizzled.
int make_tmap_trellis(CUtensorMap* out, const void* base, uint64_t kt_rows, uint64_t row_words, uint32_t box_words, uint32_t box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {row_words, kt_rows};
  cuuint64_t strides[1] = {row_words * 4};
  cuuint32_t box[2] = {box_words, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int TWICE, int CB>
static int launch_gemm(const CUtensorMap& tm, const uint32_t* trellis, float* part, int rows, int K, int N, int splits, int brows,
                       int row_tiles, int* status, cudaStream_t st, const int* tile_tab = nullptr, size_t expert_words = 0) {
  const GemmSmemLayout L = gemm_layout(TWICE, brows);
  const int smem = L.total + 1024;
  auto kern = exl3_gemm_kernel<TWICE, CB>;
  static int configured = 0;
  if (configured < smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return (int)e;
    configured = 232448;
  }
  if (smem > 232448) return (int)cudaErrorInvalidValue;
  dim3 grid(N / STRIP, splits, row_tiles);
  rx::launch(kern, dim3(grid), dim3(GEMM_THREADS), smem, st, tm, trellis, part, rows, K, N, splits, brows, row_tiles, status, tile_tab, expert_words);
  return (int)cudaGetLastError();
}

}  // namespace rx

using namespace rx;

// Split plan: a function of (K, N) and the row class only, never of the row count inside a class.
// Decode class: as many K splits as keep strips * splits within ONE wave of the machine (148 SMs x 2 resident CTAs), so no
// second, mostly empty wave is paid; every split keeps at least two 128-wide K chunks.
RX_API int rx_exl3_plan_splits(int K, int N, int decode_class) {
  if (!decode_class) return 1;
  const int strips = N / STRIP, chunks = K / 128;
  const int slots = 2 * 148;
  int s = slots / strips;
  if (s > chunks / 2) s = chunks / 2;
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  return s;
}

// MMA N (rows per tile) used for `rows` rows: 16, 32, 64, 128 or 256.
RX_API int rx_exl3_tile_rows(int rows) {
  int b = 16;
  while (b < rows && b < 256) b <<= 1;
  return b;
}

// xr: fp16 [rows, K] (rotated input).  trellis: int16 [K/16, N/16, 16*bits].  part: fp32 [splits, rows, N].
RX_API int rx_exl3_gemm(const void* xr, int rows, int K, const void* trellis, int N, int twice, int codebook, void* part, int splits,
                        int* status, void* stream) {
  if (rows <= 0 || K % 128 != 0 || N % 128 != 0 || splits < 1 || splits > K / KCH) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)xr) & 15) != 0 || (((uintptr_t)trellis) & 15) != 0) return (int)cudaErrorMisalignedAddress;
  const int brows = rx_exl3_tile_rows(rows);
  const int row_tiles = (rows + brows - 1) / brows;
  CUtensorMap tm;
  int e = make_tmap_f16_2d(&tm, xr, (uint64_t)rows, (uint64_t)K, (uint32_t)brows);
  if (e != 0) return e;
  cudaStream_t st = (cudaStream_t)stream;
  const uint32_t* tr = (const uint32_t*)trellis;
  float* p = (float*)part;
#define RX_GO(CBV) RX_DISPATCH_TWICE(twice, return launch_gemm<T_, CBV>(tm, tr, p, rows, K, N, splits, brows, row_tiles, status, st))
  switch (codebook) {
    case CB_3INST: RX_GO(CB_3INST); break;
    case CB_MCG: RX_GO(CB_MCG); break;
    case CB_MUL1: RX_GO(CB_MUL1); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef RX_GO
  return (int)cudaErrorInvalidValue;
}

// Grouped (mixture-of-experts) form.  xs: fp16 [pairs_cap, K], rows sorted by expert (each row already rotated with its expert's
// suh).  trellis: int16 [E][K/16, N/16, 16*bits].  tile_tab: device int32 [max_tiles][3] = {expert, first row, rows} (rows == 0: idle
// tile).  part: fp32 [splits, pairs_cap, N].  `tile_rows` is the MMA N of every tile (16..256, fixed for the launch).
RX_API int rx_exl3_gemm_grouped(const void* xs, int pairs_cap, int K, const void* trellis, long long expert_elems, int N, int twice, int codebook,
                                void* part, int splits, const void* tile_tab, int max_tiles, int tile_rows, int* status, void* stream) {
  if (pairs_cap <= 0 || K % 128 != 0 || N % 128 != 0 || splits < 1 || splits > K / KCH || max_tiles < 1 || max_tiles > 65535) return (int)cudaErrorInvalidValue;
  if (tile_rows != rx_exl3_tile_rows(tile_rows) || (expert_elems % 2) != 0) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)xs) & 15) != 0 || (((uintptr_t)trellis) & 15) != 0) return (int)cudaErrorMisalignedAddress;
  CUtensorMap tm;
  int e = make_tmap_f16_2d(&tm, xs, (uint64_t)pairs_cap, (uint64_t)K, (uint32_t)tile_rows);
  if (e != 0) return e;
  cudaStream_t st = (cudaStream_t)stream;
  const uint32_t* tr = (const uint32_t*)trellis;
  float* p = (float*)part;
  const size_t ew = (size_t)expert_elems / 2;
#define RX_GO(CBV) RX_DISPATCH_TWICE(twice, return launch_gemm<T_, CBV>(tm, tr, p, pairs_cap, K, N, splits, tile_rows, max_tiles, status, st, (const int*)tile_tab, ew))
  switch (codebook) {
    case CB_3INST: RX_GO(CB_3INST); break;
    case CB_MCG: RX_GO(CB_MCG); break;
    case CB_MUL1: RX_GO(CB_MUL1); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef RX_GO
  return (int)cudaErrorInvalidValue;
}
