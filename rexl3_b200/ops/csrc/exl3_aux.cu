// Everything around the EXL3 GEMM: input rotation (x * suh -> Hadamard -> fp16) fused with RMSNorm, and the finish
// kernels that sum the GEMM's K-split partials in split order, apply the output Hadamard, svh and bias, and fuse what
// follows (residual add + RMSNorm + the next layer's input rotation, or SwiGLU + the down projection's rotation).
// Also: trellis -> dense W_q unpack (test oracle / weight reconstruction) and embedding gather.
//
// What these match in the reference: crates/cuda/csrc/exl3_linear.cu:136-208 (rot_in / rot_out), glue.cu:99 (add_rmsnorm),
// :139 (swiglu), ling_kda_proj_fused.cu:1432,1595,2088 (the fused forms).  One warp owns one 128-wide Hadamard block;
// lane L holds elements 4L..4L+3.  All reductions have a fixed order, so results never depend on the row count.
#include "exl3_decode.cuh"

namespace rx {

__device__ __forceinline__ float bf16_to_f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t f_to_bf16(float f) {
  __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<uint16_t*>(&b);
}

__device__ __forceinline__ void load4_bf16(const uint16_t* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xFFFF0000u);
  v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xFFFF0000u);
}
__device__ __forceinline__ void store4_bf16(uint16_t* p, const float (&v)[4]) {
  uint2 u;
  u.x = (uint32_t)f_to_bf16(v[0]) | ((uint32_t)f_to_bf16(v[1]) << 16);
  u.y = (uint32_t)f_to_bf16(v[2]) | ((uint32_t)f_to_bf16(v[3]) << 16);
  *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ void load4_f16(const __half* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4_f16(__half* p, const float (&v)[4]) {
  const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&a); u.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// Block-wide sum with a fixed order: warp shuffles, then warp 0 adds the per-warp values in warp order.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// ------------------------------------------------------------------------------------------------ unpack
template <int TWICE, int CB>
__global__ void unpack_kernel(const uint32_t* __restrict__ trellis, __half* __restrict__ w, int kt, int nt) {
  pdl_launch();
  pdl_wait();
  const int tile = blockIdx.x * (blockDim.x / 4) + threadIdx.x / 4;
  if (tile >= kt * nt) return;
  const int h = threadIdx.x & 3;
  uint32_t h2[32];
  decode_span<TWICE, CB, 64>(trellis + (size_t)tile * 4 * TWICE, h * TWICE, h2);
  const int tk = tile / nt, tn = tile % nt, N = nt * 16;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int q = 2 * i, lanep = (64 * h + q) / 8, j = q % 8;
    const int r = 2 * (lanep % 4) + (j & 1) + 8 * ((j >> 1) & 1), c = lanep / 4 + 8 * (j >> 2);
    const __half2 v = *reinterpret_cast<const __half2*>(&h2[i]);
    w[(size_t)(tk * 16 + r) * N + tn * 16 + c] = __low2half(v);
    w[(size_t)(tk * 16 + r + 1) * N + tn * 16 + c] = __high2half(v);
  }
}

// ------------------------------------------------------------------------------------------------ embed
__global__ void embed_kernel(const int* __restrict__ ids, const uint16_t* __restrict__ table, uint16_t* __restrict__ h, int d, int vocab) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * d);
  uint4* dst = reinterpret_cast<uint4*>(h + (size_t)row * d);
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------------------------------------ norm + rot_in
// xr[row] = fp16( H( rmsnorm(x[row]) * w * suh ) ), one block per row.  norm_w == nullptr: no norm (plain rotation).
__global__ void __launch_bounds__(1024) norm_rot_in_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ norm_w, float eps,
                                   const __half* __restrict__ suh, __half* __restrict__ xr, int K) {
  pdl_launch();
  pdl_wait();
  __shared__ float blk_ss[512];   // one partial per 128-block (K <= 65536), added in block order: independent of the block size
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const uint16_t* xrow = x + (size_t)row * K;
  float rinv = 1.f;
  if (norm_w != nullptr) {
    for (int b = warp; b < K / 128; b += nw) {
      float v[4];
      load4_bf16(xrow + b * 128 + lane * 4, v);
      const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
      if (lane == 0) blk_ss[b] = ss;
    }
    __syncthreads();
    float tot = 0.f;
    for (int b = 0; b < K / 128; ++b) tot += blk_ss[b];
    rinv = rsqrtf(tot / (float)K + eps);
  }
  for (int b = warp; b < K / 128; b += nw) {
    const int i = b * 128 + lane * 4;
    float v[4], s[4];
    load4_bf16(xrow + i, v);
    load4_f16(suh + i, s);
    if (norm_w != nullptr) {
      float w[4];
      load4_bf16(norm_w + i, w);
#pragma unroll
      for (int r = 0; r < 4; ++r) v[r] = bf16_to_f(f_to_bf16(v[r] * rinv)) * w[r];
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) v[r] *= s[r];
    fwht128_warp(v);
    store4_f16(xr + (size_t)row * K + i, v);
  }
}

// ------------------------------------------------------------------------------------------------ finish kernels
// y[row][n] = H_N( sum_s part[s][row][:] )[n] * svh[n] + bias[n] for one 128-block, lane holds 4 consecutive n.
__device__ __forceinline__ void finish_block(const float* __restrict__ part, int S, size_t split_stride, size_t off, const __half* svh,
                                             const float* bias, int n0, float (&y)[4]) {
  // loads are issued eight at a time (independent, so their latencies overlap) and added in split order
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (S == 1) acc = __ldg(reinterpret_cast<const float4*>(part + off));
  else
  for (int s0 = 0; s0 < S; s0 += 8) {
    float4 p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (s0 + j < S) p[j] = __ldg(reinterpret_cast<const float4*>(part + (size_t)(s0 + j) * split_stride + off));
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (s0 + j < S) {
        if (s0 + j == 0) acc = p[j];
        else { acc.x += p[j].x; acc.y += p[j].y; acc.z += p[j].z; acc.w += p[j].w; }
      }
  }
  y[0] = acc.x; y[1] = acc.y; y[2] = acc.z; y[3] = acc.w;
  fwht128_warp(y);
  float sv[4];
  load4_f16(svh + n0, sv);
#pragma unroll
  for (int r = 0; r < 4; ++r) y[r] *= sv[r];
  if (bias != nullptr) {
    const float4 b = *reinterpret_cast<const float4*>(bias + n0);
    y[0] += b.x; y[1] += b.y; y[2] += b.z; y[3] += b.w;
  }
}

// mode 0: out bf16 [M, N];  mode 1: out f32 [M, N]
__global__ void finish_store_kernel(const float* __restrict__ part, int S, int M, int N, const __half* __restrict__ svh,
                                    const float* __restrict__ bias, void* __restrict__ out, int f32_out) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int b = blockIdx.y * nw + warp; b < N / 128; b += gridDim.y * nw) {
    const int n0 = b * 128 + lane * 4;
    float y[4];
    finish_block(part, S, (size_t)M * N, (size_t)row * N + n0, svh, bias, n0, y);
    if (f32_out) *reinterpret_cast<float4*>((float*)out + (size_t)row * N + n0) = make_float4(y[0], y[1], y[2], y[3]);
    else store4_bf16((uint16_t*)out + (size_t)row * N + n0, y);
  }
}

// h[row] += y (bf16 residual stream, updated in place); then xr = fp16(H(rmsnorm(h) * w * suh_next)).
// norm_w == nullptr skips the norm, suh_next == nullptr skips the rotation output entirely (residual update only).
__global__ void __launch_bounds__(1024) finish_add_norm_rot_kernel(const float* __restrict__ part, int S, int M, int N, const __half* __restrict__ svh,
                                           const float* __restrict__ bias, uint16_t* __restrict__ h, const uint16_t* __restrict__ norm_w,
                                           float eps, const __half* __restrict__ suh_next, __half* __restrict__ xr,
                                           uint16_t* __restrict__ xn_out) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float rowbuf[];  // N floats: the updated residual row (as stored, bf16-rounded)
  __shared__ float blk_ss[512];      // per-128-block sums of squares, added in block order (independent of the block size)
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int b = warp; b < N / 128; b += nw) {
    float ss = 0.f;
    const int n0 = b * 128 + lane * 4;
    float y[4], r[4];
    finish_block(part, S, (size_t)M * N, (size_t)row * N + n0, svh, bias, n0, y);
    load4_bf16(h + (size_t)row * N + n0, r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      r[i] = bf16_to_f(f_to_bf16(r[i] + y[i]));
      ss += r[i] * r[i];
      rowbuf[n0 + i] = r[i];
    }
    store4_bf16(h + (size_t)row * N + n0, r);
    ss = warp_sum(ss);
    if (lane == 0) blk_ss[b] = ss;
  }
  if (suh_next == nullptr && xn_out == nullptr) return;
  float rinv = 1.f;
  __syncthreads();  // orders the rowbuf / blk_ss writes before the reads below
  if (norm_w != nullptr) {
    float tot = 0.f;
    for (int b = 0; b < N / 128; ++b) tot += blk_ss[b];
    rinv = rsqrtf(tot / (float)N + eps);
  }
  for (int b = warp; b < N / 128; b += nw) {
    const int n0 = b * 128 + lane * 4;
    float v[4], s[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = rowbuf[n0 + i];
    if (suh_next != nullptr) load4_f16(suh_next + n0, s);
    if (norm_w != nullptr) {
      float w[4];
      load4_bf16(norm_w + n0, w);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = bf16_to_f(f_to_bf16(v[i] * rinv)) * w[i];
    }
    if (xn_out != nullptr) store4_bf16(xn_out + (size_t)row * N + n0, v);   // the normalised row itself (router input, per-expert rotations)
    if (suh_next == nullptr) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= s[i];
    fwht128_warp(v);
    store4_f16(xr + (size_t)row * N + n0, v);
  }
}

// part [S, M, 2F] = gate | up.  act = silu(gate) * up (bf16-rounded like an unfused pipeline would store it), then
// xr[row][F] = fp16(H(act * suh_down)).
__global__ void finish_swiglu_rot_kernel(const float* __restrict__ part, int S, int M, int F, const __half* __restrict__ svh,
                                         const float* __restrict__ bias, const __half* __restrict__ suh_down, __half* __restrict__ xr) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int N = 2 * F;
  for (int b = blockIdx.y * nw + warp; b < F / 128; b += gridDim.y * nw) {
    const int n0 = b * 128 + lane * 4;
    float g[4], u[4], s[4];
    finish_block(part, S, (size_t)M * N, (size_t)row * N + n0, svh, bias, n0, g);
    finish_block(part, S, (size_t)M * N, (size_t)row * N + F + n0, svh, bias, F + n0, u);
    load4_f16(suh_down + n0, s);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = g[i] / (1.f + __expf(-g[i])) * u[i];
      g[i] = bf16_to_f(f_to_bf16(a)) * s[i];
    }
    fwht128_warp(g);
    store4_f16(xr + (size_t)row * F + n0, g);
  }
}

}  // namespace rx

using namespace rx;

RX_API int rx_exl3_unpack(const void* trellis, int K, int N, int twice, int codebook, void* w_f16, void* stream) {
  if (K % 16 || N % 16) return (int)cudaErrorInvalidValue;
  const int kt = K / 16, nt = N / 16, tiles = kt * nt;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid((tiles + 31) / 32), block(128);
#define RX_GO(CBV) RX_DISPATCH_TWICE(twice, rx::launch(unpack_kernel<T_, CBV>, dim3(grid), dim3(block), 0, st, (const uint32_t*)trellis, (__half*)w_f16, kt, nt))
  switch (codebook) {
    case CB_3INST: RX_GO(CB_3INST); break;
    case CB_MCG: RX_GO(CB_MCG); break;
    case CB_MUL1: RX_GO(CB_MUL1); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef RX_GO
  return (int)cudaGetLastError();
}

RX_API int rx_embed(const void* ids, const void* table, void* h, int rows, int d, int vocab, void* stream) {
  if (d % 8) return (int)cudaErrorInvalidValue;
  rx::launch(embed_kernel, dim3(rows), dim3(128), 0, (cudaStream_t)stream, (const int*)ids, (const uint16_t*)table, (uint16_t*)h, d, vocab);
  return (int)cudaGetLastError();
}

RX_API int rx_norm_rot_in(const void* x_bf16, const void* norm_w_bf16, float eps, const void* suh, void* xr, int rows, int K, void* stream) {
  if (K % 128 || K / 128 > 512) return (int)cudaErrorInvalidValue;
  rx::launch(norm_rot_in_kernel, dim3(rows), dim3(rows >= 512 ? 256 : 1024), 0, (cudaStream_t)stream, (const uint16_t*)x_bf16, (const uint16_t*)norm_w_bf16, eps, (const __half*)suh,
                                                            (__half*)xr, K);
  return (int)cudaGetLastError();
}

static int blocks_y(int rows, int nblocks128) {
  // one warp per 128-block (8 warps per CTA): the kernels without a row-wide reduction get their memory-level parallelism
  // from many resident warps with one or two loads each.  For a few rows that means one CTA per 8 blocks; for a prefill
  // chunk of thousands of rows the CTAs take several blocks each instead (a grid of 10^5 very short CTAs is bound by the
  // rate at which CTAs can be launched, not by memory).
  int per_row = (nblocks128 + 7) / 8;
  if (per_row < 1) per_row = 1;
  int cap = 16384 / (rows < 1 ? 1 : rows);
  if (cap < 1) cap = 1;
  return per_row < cap ? per_row : cap;
}

RX_API int rx_finish_store(const void* part, int S, int M, int N, const void* svh, const void* bias, void* out, int f32_out, void* stream) {
  if (N % 128) return (int)cudaErrorInvalidValue;
  dim3 grid(M, blocks_y(M, N / 128));
  rx::launch(finish_store_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const float*)part, S, M, N, (const __half*)svh, (const float*)bias, out, f32_out);
  return (int)cudaGetLastError();
}

RX_API int rx_finish_add_norm_rot(const void* part, int S, int M, int N, const void* svh, const void* bias, void* h_bf16, const void* norm_w,
                                  float eps, const void* suh_next, void* xr, void* stream, void* xn_out) {
  if (N % 128 || N * 4 > 200 * 1024 || N / 128 > 512) return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(finish_add_norm_rot_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // a window of a few rows wants every row finished fast (1024 threads per row); a prefill chunk wants many rows in flight per SM
  const int threads = M >= 512 ? 256 : 1024;
  rx::launch(finish_add_norm_rot_kernel, dim3(M), dim3(threads), (size_t)N * 4, (cudaStream_t)stream, (const float*)part, S, M, N, (const __half*)svh, (const float*)bias,
                                                                     (uint16_t*)h_bf16, (const uint16_t*)norm_w, eps, (const __half*)suh_next,
                                                                     (__half*)xr, (uint16_t*)xn_out);
  return (int)cudaGetLastError();
}

RX_API int rx_finish_swiglu_rot(const void* part, int S, int M, int F, const void* svh, const void* bias, const void* suh_down, void* xr,
                                void* stream) {
  if (F % 128) return (int)cudaErrorInvalidValue;
  dim3 grid(M, blocks_y(M, F / 128));
  rx::launch(finish_swiglu_rot_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const float*)part, S, M, F, (const __half*)svh, (const float*)bias,
                                                                  (const __half*)suh_down, (__half*)xr);
  return (int)cudaGetLastError();
}

// Turn programmatic dependent launch on (1, default) or off (0) for every later launch of this library.
RX_API int rx_set_pdl(int on) {
  rx::pdl_enabled() = on ? 1 : 0;
  return 0;
}
