// Grouped MXFP4 (E2M1 values, one E8M0 scale per 32 elements) expert GEMM on tcgen05 (sm_100a).
//
//   part[split][pos][n] = sum over this split's k of  xs[pos][k] * W_e[n][k]        (pos = a (row, slot) pair sorted by expert)
//
// Same skeleton as the EXL3 GEMM (exl3_gemm.cu): swap-AB, the weight strip of 128 output features is the MMA's A operand
// (K-major, SWIZZLE_128B), the rows of the tile are B, the accumulator lives in TMEM.  Warp 0 streams the packed nibbles with
// 2-D TMA tiles (128 rows x 32 bytes per 64-wide K chunk) and the fp16 activation tiles; two groups of four warps expand the
// nibbles through a 256-entry byte -> half2 table in shared memory, apply the block scale, and write swizzled fp16 operand tiles;
// warp 1 issues tcgen05.mma; warps 2..5 read the accumulator back.  Tile table, early exit of idle tiles and the per-expert
// weight offset are as in the grouped EXL3 launch.  Format: reference crates/cuda/csrc/fp4_linear.cu:5-18,36-44 (its kernel is a
// scalar LUT FMA loop; the tensor-core schedule here is new).  Scales outside the fp16 range saturate (to 0 below 2^-24, to inf
// above 2^15); 0xFF is NaN.
#include <cuda.h>
#include <cuda_fp4.h>
#include "common.cuh"

namespace rx {

constexpr int MX_KCH = 64;
constexpr int MX_STRIP = 128;
constexpr int MX_GROUPS = 2;
constexpr int MX_DEC_WARPS = 8;
constexpr int MX_THREADS = 64 + MX_DEC_WARPS * 32;
constexpr int MX_RAW_STAGES = 4;
constexpr int MX_SC_ROW = 256;                          // scale bytes per weight row a CTA may need: K range <= 8192
constexpr int MX_OP_STAGES = 3;
static_assert(MX_OP_STAGES >= MX_GROUPS, "operand ring shallower than the number of decode groups");
constexpr int MX_A_STAGE = MX_STRIP * MX_KCH * 2;       // 16 KB of fp16
constexpr int MX_RAW_STAGE = MX_STRIP * (MX_KCH / 2);   // 4 KB of nibbles

struct MxLayout {
  int a_off, b_off, raw_off, sc_off, lut_off, bar_off, total;
};
__host__ __device__ inline MxLayout mx_layout(int brows) {
  MxLayout L;
  L.a_off = 0;
  L.b_off = L.a_off + MX_OP_STAGES * MX_A_STAGE;
  L.raw_off = L.b_off + MX_OP_STAGES * brows * MX_KCH * 2;
  L.sc_off = L.raw_off + MX_RAW_STAGES * MX_RAW_STAGE;
  L.lut_off = L.sc_off + MX_STRIP * MX_SC_ROW;
  L.bar_off = L.lut_off + 1024;
  L.total = L.bar_off + 256;
  return L;
}

__device__ __forceinline__ uint32_t e8m0_to_half2(uint32_t b) {
  const int e = (int)b - 127;
  uint32_t h;
  if (b == 0xFFu) h = 0x7E00u;
  else if (e > 15) h = 0x7C00u;
  else if (e >= -14) h = (uint32_t)(e + 15) << 10;
  else if (e >= -24) h = 1u << (e + 24);
  else h = 0u;
  return h | (h << 16);
}

__global__ void __launch_bounds__(MX_THREADS, 2)
mxfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const uint8_t* __restrict__ scales,
                  float* __restrict__ part, int rows, int K, int N, int splits, int brows, int* status, const int* __restrict__ tile_tab) {
  pdl_launch();
  pdl_wait();                       // the tile table comes from the planning kernel just before
  const int e = tile_tab[3 * blockIdx.z];
  const int g_row0 = tile_tab[3 * blockIdx.z + 1];
  const int g_nrows = tile_tab[3 * blockIdx.z + 2];
  if (g_nrows <= 0) return;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const MxLayout L = mx_layout(brows);
  const int b_stage = brows * MX_KCH * 2;
  uint32_t* lut = (uint32_t*)(smem + L.lut_off);
  uint64_t* bars = (uint64_t*)(smem + L.bar_off);
  uint64_t* op_full = bars;
  uint64_t* op_empty = bars + MX_OP_STAGES;
  uint64_t* raw_full = bars + 2 * MX_OP_STAGES;
  uint64_t* raw_empty = raw_full + MX_RAW_STAGES;
  uint64_t* acc_full = raw_empty + MX_RAW_STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int strip = blockIdx.x, split = blockIdx.y;
  const int nchunks_total = K / MX_KCH;
  const int c_begin = (int)((long long)nchunks_total * split / splits);
  const int c_end = (int)((long long)nchunks_total * (split + 1) / splits);
  const int nchunks = c_end - c_begin;
  uint32_t ncols = 32;
  while ((int)ncols < brows) ncols <<= 1;

  if (threadIdx.x < 256) {
    // byte -> half2(low nibble value, high nibble value); magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}, bit 3 of a nibble is the sign
    const uint32_t mag[8] = {0x0000u, 0x3800u, 0x3C00u, 0x3E00u, 0x4000u, 0x4200u, 0x4400u, 0x4600u};
    const uint32_t b = threadIdx.x, lo = b & 15u, hi = b >> 4;
    lut[b] = (mag[lo & 7] | ((lo & 8u) << 12)) | ((mag[hi & 7] | ((hi & 8u) << 12)) << 16);
  }
  const int w_row0 = e * N + strip * MX_STRIP;      // row of the stacked weight matrix [E * N, K / 2]
  if (warp >= 2) {
    // the block scales of this CTA's K range, two bytes per 64-wide chunk: all loads are independent, so their latencies overlap
    const int dt = threadIdx.x - 64;
    const int srow_i = dt & 127, half = dt >> 7;
    const uint8_t* srow = scales + (size_t)(w_row0 + srow_i) * (K / 32) + (size_t)c_begin * 2;
    uint16_t* dsts = (uint16_t*)(smem + L.sc_off + srow_i * MX_SC_ROW);
    for (int c = half; c < nchunks; c += 2) dsts[c] = *reinterpret_cast<const uint16_t*>(srow + 2 * c);
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < MX_OP_STAGES; ++i) { mbar_init(&op_full[i], MX_DEC_WARPS / MX_GROUPS + 1); mbar_init(&op_empty[i], 1); }
    for (int i = 0; i < MX_RAW_STAGES; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], MX_DEC_WARPS / MX_GROUPS); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, ncols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      constexpr int AHEAD = 4;
      bool ok = true;
      for (int i = 0; i < nchunks + AHEAD && ok; ++i) {
        if (i < nchunks) {
          const int c = i, s = c % MX_RAW_STAGES;
          if (c >= MX_RAW_STAGES) ok = mbar_wait(&raw_empty[s], ((c / MX_RAW_STAGES) - 1) & 1, abort_flag, status, 60);
          if (!ok) break;
          mbar_arrive_expect_tx(&raw_full[s], MX_RAW_STAGE);
          tma_load_2d(smem + L.raw_off + s * MX_RAW_STAGE, &tmap_w, (c_begin + c) * (MX_KCH / 2), w_row0, &raw_full[s]);
        }
        if (i >= AHEAD) {
          const int c = i - AHEAD, s = c % MX_OP_STAGES;
          if (c >= MX_OP_STAGES) ok = mbar_wait(&op_empty[s], ((c / MX_OP_STAGES) - 1) & 1, abort_flag, status, 61);
          if (!ok) break;
          mbar_arrive_expect_tx(&op_full[s], (uint32_t)b_stage);
          tma_load_2d(smem + L.b_off + s * b_stage, &tmap_x, (c_begin + c) * MX_KCH, g_row0, &op_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(MX_STRIP, brows, 0, 0);
      bool ok = true;
      for (int c = 0; c < nchunks && ok; ++c) {
        const int s = c % MX_OP_STAGES;
        ok = mbar_wait(&op_full[s], (c / MX_OP_STAGES) & 1, abort_flag, status, 62);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + L.a_off + s * MX_A_STAGE);
        const uint32_t b_addr = smem_u32(smem + L.b_off + s * b_stage);
#pragma unroll
        for (int k = 0; k < MX_KCH / 16; ++k)
          tc_mma_f16(tmem_base, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc, (c | k) != 0);
        tc_commit(&op_empty[s]);
      }
      tc_commit(acc_full);
    }
  } else {
    const int dw = warp - 2;
    const int grp = dw / (MX_DEC_WARPS / MX_GROUPS);
    const int t = (dw % (MX_DEC_WARPS / MX_GROUPS)) * 32 + lane;     // row of the strip this thread expands
    const uint16_t* srow = (const uint16_t*)(smem + L.sc_off + t * MX_SC_ROW);
    bool ok = true;
    for (int c = grp; c < nchunks && ok; c += MX_GROUPS) {
      const int rs = c % MX_RAW_STAGES, os = c % MX_OP_STAGES;
      const uint32_t sc = srow[c];
      ok = mbar_wait(&raw_full[rs], (c / MX_RAW_STAGES) & 1, abort_flag, status, 63);
      if (!ok) break;
      const uint4* raw = reinterpret_cast<const uint4*>(smem + L.raw_off + rs * MX_RAW_STAGE + t * 32);
      const uint4 r0 = raw[0], r1 = raw[1];
      release_read_stage(&raw_empty[rs], lane);      // generic-proxy reads, async-proxy refill: proxy fence before the release
      if (c >= MX_OP_STAGES) ok = mbar_wait(&op_empty[os], ((c / MX_OP_STAGES) - 1) & 1, abort_flag, status, 64);
      if (!ok) break;
      uint8_t* a_row = smem + L.a_off + os * MX_A_STAGE + (t >> 3) * 1024 + (t & 7) * 128;
      const uint32_t words[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
      const uint32_t s_lo = e8m0_to_half2(sc & 0xFFu), s_hi = e8m0_to_half2(sc >> 8);   // k 0..31 and 32..63 of the chunk
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // word j holds k = 8j .. 8j+7: one 16-byte column of the operand row
        const uint32_t w = words[j];
        const __half2 s2 = *reinterpret_cast<const __half2*>(j < 4 ? &s_lo : &s_hi);
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // one hardware conversion per byte (two E2M1 values -> half2); the table in shared memory costs bank conflicts instead
          const __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((w >> (8 * q)) & 0xFFu), __NV_E2M1);
          const __half2 p = __hmul2(*reinterpret_cast<const __half2*>(&hr), s2);
          o[q] = *reinterpret_cast<const uint32_t*>(&p);
        }
        *reinterpret_cast<uint4*>(a_row + ((j ^ (t & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&op_full[os]);
    }
    if (dw < 4) {
      const bool done = mbar_wait(acc_full, 0, abort_flag, status, 65);
      tc_fence_after();
      if (done && *abort_flag == 0) {
        const int q = warp & 3;
        const int n = strip * MX_STRIP + q * 32 + lane;
        float* out = part + ((size_t)split * rows) * N + n;
        for (int cb = 0; cb < brows; cb += 16) {
          if (cb >= g_nrows) break;
          uint32_t r[16];
          tc_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + cb, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (cb + i < g_nrows) out[(size_t)(g_row0 + cb + i) * N] = __uint_as_float(r[i]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag != 0 && lane == 0) mbar_wait(acc_full, 0, abort_flag, nullptr, 66);
    __syncwarp();
    tmem_dealloc(tmem_base, ncols);
  }
}

int make_tmap_f16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);   // exl3_gemm.cu

typedef CUresult (*MxEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tmap_u8_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_bytes, uint32_t box_rows) {
  static MxEncodeFn enc = nullptr;
  if (enc == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return (int)cudaErrorNotSupported;
    enc = (MxEncodeFn)p;
  }
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace rx

using namespace rx;

// xs: fp16 [pairs_cap, K] sorted by expert.  w: uint8 [E, N, K/2] (low nibble = even k), scales: uint8 [E, N, K/32], both starting at
// expert 0 of the id space the tile table uses (`experts` = size of that space).  part: fp32 [splits, pairs_cap, N].
RX_API int rx_mxfp4_gemm_grouped(const void* xs, int pairs_cap, int K, const void* w, const void* scales, int experts, int N, void* part,
                                 int splits, const void* tile_tab, int max_tiles, int tile_rows, int* status, void* stream) {
  if (pairs_cap <= 0 || K % 128 != 0 || N % 128 != 0 || splits < 1 || splits > K / MX_KCH || max_tiles < 1 || max_tiles > 65535 || experts < 1)
    return (int)cudaErrorInvalidValue;
  if (((K / MX_KCH + splits - 1) / splits + 1) * 2 > MX_SC_ROW) return (int)cudaErrorInvalidValue;   // a split's scale bytes must fit its shared-memory row
  int b = 16;
  while (b < tile_rows && b < 256) b <<= 1;
  if (b != tile_rows) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)xs) & 15) != 0 || (((uintptr_t)w) & 15) != 0 || (((uintptr_t)scales) & 1) != 0) return (int)cudaErrorMisalignedAddress;
  CUtensorMap tx, tw;
  int e = make_tmap_f16_2d(&tx, xs, (uint64_t)pairs_cap, (uint64_t)K, (uint32_t)tile_rows);
  if (e != 0) return e;
  e = make_tmap_u8_2d(&tw, w, (uint64_t)experts * N, (uint64_t)K / 2, MX_KCH / 2, MX_STRIP);
  if (e != 0) return e;
  const MxLayout L = mx_layout(tile_rows);
  const int smem = L.total + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(mxfp4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  if (smem > 232448) return (int)cudaErrorInvalidValue;
  return (int)rx::launch(mxfp4_gemm_kernel, dim3(N / MX_STRIP, splits, max_tiles), dim3(MX_THREADS), (size_t)smem, (cudaStream_t)stream, tx, tw,
                         (const uint8_t*)scales, (float*)part, pairs_cap, K, N, splits, tile_rows, status, (const int*)tile_tab);
}
