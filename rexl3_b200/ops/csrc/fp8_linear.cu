// FP8 (E4M3) block-scaled linear on tcgen05 (sm_100a):  y[m, n] = sum_k x[m, k] * W[n, k] * 2^(scale[n / 32][k / 32] - 127), fp32 accumulate.
// W: E4M3 bytes [N, K]; scale: E8M0 bytes [N / 32, K / 32] (one power of two per 32 x 32 tile); x: bf16 [M, K]; y: bf16, fp16 or fp32 [M, N].
// Format and semantics: reference crates/cuda/csrc/fp8_linear.cu:1 (its kernel is a warp-per-row FMA loop; the tensor-core schedule is new).
//
// An E4M3 value times a power of two is EXACT in bf16 (4 significant bits, 8-bit exponent), so the weight strip is expanded to bf16 operand
// tiles in shared memory with its block scales applied and the products are those of the definition; only the fp32 summation order differs
// from a scalar loop, and that order is a function of (K, splits, rows per tile): a row's bits do not depend on its batch mates or its place.  Same skeleton as the MXFP4
// expert GEMM (swap-AB: the 128-feature weight strip is the MMA's A operand, the rows are B, accumulator in TMEM): warp 0 streams the raw
// bytes (TMA, 128 rows x 64 bytes per 64-wide K chunk) and the bf16 activation tiles, two groups of four warps expand, warp 1 issues
// tcgen05.mma kind::f16 with bf16 operands, warps 2..5 read the accumulator back.  K splits write fp32 planes that a finish kernel sums in
// split order (+ bias) into the output type.  Scales below 2^-126 flush to zero, 0xFF is NaN.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include "common.cuh"

namespace rx {

constexpr int F8_KCH = 64;
constexpr int F8_STRIP = 128;
constexpr int F8_GROUPS = 2;
constexpr int F8_DEC_WARPS = 8;
constexpr int F8_THREADS = 64 + F8_DEC_WARPS * 32;
// Ring depths: 3 operand stages and 4 raw stages keep two CTAs on an SM at window sizes.  Deeper rings were measured and change nothing
// (4 / 4, 3 / 6: the same 43.8 us at one row; 6 / 8 drops to one CTA per SM and 68 us), so the chain is not what bounds the kernel - see the
// profile summary for what does (shared-memory traffic of the expansion at many rows, 64-byte row pieces per bulk copy at few rows).
constexpr int F8_RAW_STAGES_MAX = 4;
constexpr int F8_OP_STAGES_MAX = 3;
static_assert(3 >= F8_GROUPS, "operand ring shallower than the number of expand groups");
constexpr int F8_A_STAGE = F8_STRIP * F8_KCH * 2;       // 16 KB of bf16
constexpr int F8_RAW_STAGE = F8_STRIP * F8_KCH;         // 8 KB of E4M3 bytes

struct F8Layout {
  int a_off, b_off, raw_off, bar_off, total;
};
__host__ __device__ inline F8Layout f8_layout(int brows, int ops, int raws) {
  F8Layout L;
  L.a_off = 0;
  L.b_off = L.a_off + ops * F8_A_STAGE;
  L.raw_off = L.b_off + ops * brows * F8_KCH * 2;
  L.bar_off = L.raw_off + raws * F8_RAW_STAGE;
  L.total = L.bar_off + 512;
  return L;
}

__device__ __forceinline__ float f8_e8m0(uint32_t b) {
  return __uint_as_float(b == 0u ? 0u : (b == 0xFFu ? 0x7fc00000u : (b << 23)));
}

template <int OPS, int RAWS>
__global__ void __launch_bounds__(F8_THREADS, 2)
fp8_linear_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const uint8_t* __restrict__ scales,
                  float* __restrict__ part, int rows, int K, int N, int splits, int brows, int* status, int AHEAD_B) {
  pdl_launch();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const F8Layout L = f8_layout(brows, OPS, RAWS);
  const int b_stage = brows * F8_KCH * 2;
  uint64_t* bars = (uint64_t*)(smem + L.bar_off);
  uint64_t* op_full = bars;
  uint64_t* op_empty = bars + F8_OP_STAGES_MAX;
  uint64_t* raw_full = bars + 2 * F8_OP_STAGES_MAX;
  uint64_t* raw_empty = raw_full + F8_RAW_STAGES_MAX;
  uint64_t* acc_full = raw_empty + F8_RAW_STAGES_MAX;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int strip = blockIdx.x, split = blockIdx.y;
  const int g_row0 = blockIdx.z * brows;
  const int g_nrows = min(brows, rows - g_row0);
  const int nchunks_total = K / F8_KCH;
  const int c_begin = (int)((long long)nchunks_total * split / splits);
  const int c_end = (int)((long long)nchunks_total * (split + 1) / splits);
  const int nchunks = c_end - c_begin;
  uint32_t ncols = 32;
  while ((int)ncols < brows) ncols <<= 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < OPS; ++i) { mbar_init(&op_full[i], F8_DEC_WARPS / F8_GROUPS + 1); mbar_init(&op_empty[i], 1); }
    for (int i = 0; i < RAWS; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], F8_DEC_WARPS / F8_GROUPS); }
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
  const int w_row0 = strip * F8_STRIP;

  if (warp == 0) {
    if (lane == 0) {
      const int AHEAD = AHEAD_B;
      bool ok = true;
      bool waited = false;
      for (int i = 0; i < nchunks + AHEAD && ok; ++i) {
        if (i < nchunks) {            // weights do not depend on the previous kernel: they stream before griddepcontrol.wait
          const int c = i, s = c % RAWS;
          if (c >= RAWS) ok = mbar_wait(&raw_empty[s], ((c / RAWS) - 1) & 1, abort_flag, status, 180);
          if (!ok) break;
          mbar_arrive_expect_tx(&raw_full[s], F8_RAW_STAGE);
          tma_load_2d(smem + L.raw_off + s * F8_RAW_STAGE, &tmap_w, (c_begin + c) * F8_KCH, w_row0, &raw_full[s]);
        }
        if (i >= AHEAD) {
          if (!waited) { pdl_wait(); waited = true; }
          const int c = i - AHEAD, s = c % OPS;
          if (c >= OPS) ok = mbar_wait(&op_empty[s], ((c / OPS) - 1) & 1, abort_flag, status, 181);
          if (!ok) break;
          mbar_arrive_expect_tx(&op_full[s], (uint32_t)b_stage);
          tma_load_2d(smem + L.b_off + s * b_stage, &tmap_x, (c_begin + c) * F8_KCH, g_row0, &op_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(F8_STRIP, brows, 1, 1);
      bool ok = true;
      for (int c = 0; c < nchunks && ok; ++c) {
        const int s = c % OPS;
        ok = mbar_wait(&op_full[s], (c / OPS) & 1, abort_flag, status, 182);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + L.a_off + s * F8_A_STAGE);
        const uint32_t b_addr = smem_u32(smem + L.b_off + s * b_stage);
#pragma unroll
        for (int k = 0; k < F8_KCH / 16; ++k)
          tc_mma_f16(tmem_base, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc, (c | k) != 0);
        tc_commit(&op_empty[s]);
      }
      tc_commit(acc_full);
    }
  } else {
    const int dw = warp - 2;
    const int grp = dw / (F8_DEC_WARPS / F8_GROUPS);
    // A warp expands 32 rows of the strip (one scale tile) in four 8-row slabs: lane = (row of the slab, 16-byte quarter of the 64-byte raw
    // row), so one load instruction reads 512 contiguous bytes - free of bank conflicts (a thread per row would read at a 64-byte stride,
    // 16 ways conflicted: measured 2x slower end to end) - and a lane turns its 16 weights into two 16-byte pieces of the bf16 operand row.
    const int wq = dw % (F8_DEC_WARPS / F8_GROUPS), sub_r = lane >> 2, sub_c = lane & 3;
    const uint8_t* srow = scales + (size_t)((w_row0 + 32 * wq) >> 5) * (K / 32) + (size_t)c_begin * 2;
    bool ok = true;
    for (int c = grp; c < nchunks && ok; c += F8_GROUPS) {
      const int rs = c % RAWS, os = c % OPS;
      const uint32_t sc = *reinterpret_cast<const uint16_t*>(srow + 2 * c);
      ok = mbar_wait(&raw_full[rs], (c / RAWS) & 1, abort_flag, status, 183);
      if (!ok) break;
      const uint32_t raw = smem_u32(smem + L.raw_off + rs * F8_RAW_STAGE + (32 * wq + sub_r) * 64 + sub_c * 16);
      uint4 rw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) rw[i] = lds128(raw + i * 8 * 64);
      // Handing the stage back to the bulk-copy engine: the reads above went through the generic proxy, the next chunk's copy writes through
      // the async proxy, and nothing orders the two but a proxy fence BEFORE the release (measured without it: the copy for chunk c + 4
      // overtook these reads in half of the launches at 32 chunks per CTA, whole 32-row blocks of an operand tile then mixed two chunks;
      // with the fence 0 of 120 launches).
      release_read_stage(&raw_empty[rs], lane);
      if (c >= OPS) ok = mbar_wait(&op_empty[os], ((c / OPS) - 1) & 1, abort_flag, status, 184);
      if (!ok) break;
      uint8_t* a_stage = smem + L.a_off + os * F8_A_STAGE;
      // E4M3 -> bf16 without a conversion instruction: the byte s eeee mmm, moved to the top of a halfword and shifted right by 4 under a mask, IS
      // the bf16 number (-1)^s 2^(e - 127) (1 + m / 8) (exponent field = e, mantissa = m << 4; e = 0 gives the matching bf16 subnormal), i.e. the
      // value times 2^-120.  One packed bf16 multiply by 2^(120 + scale exponent) - a power of two, exact, subnormals included - finishes it:
      // PRMT, SHF, LOP3, HMUL2 per two weights.  (Scales of 2^8 and more would overflow that constant: those chunks take the float path.)
      const uint32_t scb = sub_c < 2 ? (sc & 0xFFu) : (sc >> 8);           // this lane's 16 weights lie in k 0..31 or 32..63 of the chunk
      const int se = (int)scb - 127;
      const bool fast = se <= 7 && se >= -126 && scb != 0xFFu;
      const uint32_t kbits = (uint32_t)(se + 120 + 127) << 7;              // bf16 bits of 2^(120 + se)
      const uint32_t mulw = kbits | (kbits << 16);
      const __nv_bfloat162 mul = *reinterpret_cast<const __nv_bfloat162*>(&mulw);
      const float sf = f8_e8m0(scb);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = 32 * wq + 8 * i + sub_r;
        uint8_t* a_row = a_stage + (r >> 3) * 1024 + (r & 7) * 128;
        const uint32_t words[4] = {rw[i].x, rw[i].y, rw[i].z, rw[i].w};
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {              // words 2 hf, 2 hf + 1 = k 8 (2 sub_c + hf) .. + 7 = one 16-byte piece of the bf16 row
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t w = words[2 * hf + (q >> 1)];
            if (fast) {
              const uint32_t pair = __byte_perm(w, 0u, (q & 1) ? 0x3424u : 0x1404u);      // (b1 << 24) | (b0 << 8) of this pair of bytes
              const uint32_t bits = (pair & 0x80008000u) | ((pair >> 4) & 0x07F007F0u);
              const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&bits), mul);
              o[q] = *reinterpret_cast<const uint32_t*>(&v);
            } else {
              const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w >> (16 * (q & 1))) & 0xFFFFu), __NV_E4M3);
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
              const __nv_bfloat162 pv = __floats2bfloat162_rn(f.x * sf, f.y * sf);
              o[q] = *reinterpret_cast<const uint32_t*>(&pv);
            }
          }
          const int j = 2 * sub_c + hf;
          *reinterpret_cast<uint4*>(a_row + ((j ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&op_full[os]);
    }
    if (dw < 4) {
      const bool done = mbar_wait(acc_full, 0, abort_flag, status, 185);
      tc_fence_after();
      if (done && *abort_flag == 0) {
        const int q = warp & 3;
        const int n = strip * F8_STRIP + q * 32 + lane;
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
    if (*abort_flag != 0 && lane == 0) mbar_wait(acc_full, 0, abort_flag, nullptr, 186);
    __syncwarp();
    tmem_dealloc(tmem_base, ncols);
  }
}

// grid = (N / 128, rows), 32 threads: y[row][n0 .. n0 + 127] = sum over splits (split order) + bias.  out_type: 0 bf16, 1 fp16, 2 fp32.
__global__ void __launch_bounds__(32) fp8_finish_kernel(const float* __restrict__ part, int splits, int rows, int N, const float* __restrict__ bias,
                                                        void* __restrict__ out, int out_type) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.y, n0 = blockIdx.x * 128 + threadIdx.x * 4;
  float4 acc = *reinterpret_cast<const float4*>(part + (size_t)row * N + n0);
  for (int s = 1; s < splits; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(part + ((size_t)s * rows + row) * N + n0);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  if (bias != nullptr) {
    const float4 b = *reinterpret_cast<const float4*>(bias + n0);
    acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
  }
  const size_t at = (size_t)row * N + n0;
  if (out_type == 2) {
    *reinterpret_cast<float4*>((float*)out + at) = acc;
  } else if (out_type == 1) {
    const __half2 a = __floats2half2_rn(acc.x, acc.y), b = __floats2half2_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>((__half*)out + at) = o;
  } else {
    const __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y), b = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>((__nv_bfloat16*)out + at) = o;
  }
}

int make_tmap_f16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);                          // exl3_gemm.cu
int make_tmap_u8_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_bytes, uint32_t box_rows);    // mxfp4_gemm.cu

}  // namespace rx

using namespace rx;

RX_API long long rx_fp8_linear_scratch_floats(int rows, int N, int splits) { return (long long)splits * rows * N; }

// x: bf16 [rows, K]; w: E4M3 [N, K]; scales: E8M0 [N / 32, K / 32]; part: fp32 [splits, rows, N] scratch; bias: f32 [N] or nullptr;
// out: [rows, N] of out_type (0 bf16, 1 fp16, 2 fp32).  tile_rows: rows per CTA, a power of two in 16..256.
RX_API int rx_fp8_linear(const void* x, int rows, int K, const void* w, const void* scales, int N, void* part, int splits, int tile_rows, const void* bias,
                         void* out, int out_type, int* status, void* stream) {
  if (rows < 1 || K % 64 != 0 || N % 128 != 0 || splits < 1 || splits > K / F8_KCH || out_type < 0 || out_type > 2) return (int)cudaErrorInvalidValue;
  int b = 16;
  while (b < tile_rows && b < 256) b <<= 1;
  if (b != tile_rows) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)x) & 15) != 0 || (((uintptr_t)w) & 15) != 0 || (((uintptr_t)scales) & 1) != 0) return (int)cudaErrorMisalignedAddress;
  CUtensorMap tx, tw;
  int e = make_tmap_f16_2d(&tx, x, (uint64_t)rows, (uint64_t)K, (uint32_t)tile_rows);
  if (e != 0) return e;
  e = make_tmap_u8_2d(&tw, w, (uint64_t)N, (uint64_t)K, F8_KCH, F8_STRIP);
  if (e != 0) return e;
  const F8Layout L = f8_layout(tile_rows, 3, 4);
  const int smem = L.total + 1024;
  if (smem > 232448) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(fp8_linear_kernel<3, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  e = (int)rx::launch(fp8_linear_kernel<3, 4>, dim3(N / F8_STRIP, splits, (rows + tile_rows - 1) / tile_rows), dim3(F8_THREADS), (size_t)smem, st, tx, tw,
                      (const uint8_t*)scales, (float*)part, rows, K, N, splits, tile_rows, status, 4);
  if (e != 0) return e;
  return (int)rx::launch(fp8_finish_kernel, dim3(N / 128, rows), dim3(32), 0, st, (const float*)part, splits, rows, N, (const float*)bias, out, out_type);
}
