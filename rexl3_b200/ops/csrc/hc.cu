// Manifold-constrained hyper-connections (mHC): NS = 4 residual streams per row, x f32 [rows][4][D].  Semantics matched: reference
// crates/cuda/csrc/mhc.cu:6-12,355-384 (one site = attention or FFN):
//   mix:   S[q] = x . fn[q] over the 4 D stream values (q = 0..23), ss = sum x^2;  r = 1 / sqrt(ss / (4 D) + rms_eps)
//          pre[h]  = sigmoid(S[h] r scale0 + base[h]) + hc_eps
//          post[h] = 2 sigmoid(S[4 + h] r scale1 + base[4 + h])
//          comb    = sinkhorn(softmax_rows(S[8 + 4 i + j] r scale2 + base[8 + 4 i + j]) + hc_eps): columns normalised, then (iters - 1) x (rows, columns)
//          collapsed[d] = sum_h pre[h] x[h][d], then the layer's RMSNorm -> bf16 (the sublayer's input)
//   apply: x[h][d] <- post[h] y[d] + sum_g comb[g][h] x[g][d], in place (y = the sublayer's output, f32)
// This engine's schedule: the mix is ONE kernel with one CTA per row (the reference splits it into atom partials + finalize): 256 threads walk the
// row's float4 columns in a fixed order, every reduction is a fixed tree (lane butterfly, then the eight warp sums in order), so a row's bits do
// not depend on the other rows of the launch.  The 25 running sums and the row's collapsed values stay in registers between the two passes.
#include "common.cuh"

namespace rx {

constexpr int HC_NS = 4, HC_NM = 24, HC_THREADS = 256, HC_MAXV = 8;      // D <= 4 * 256 * 8 = 8192

__device__ __forceinline__ float hc_sigmoid(float v) { return 1.f / (1.f + expf(-v)); }

__global__ void __launch_bounds__(HC_THREADS) hc_mix_kernel(const float* __restrict__ x, const float* __restrict__ fn, const float* __restrict__ base,
                                                           float s0, float s1, float s2, const uint16_t* __restrict__ norm_w, float rms_eps,
                                                           float hc_eps, float norm_eps, int iters, int D, float* __restrict__ coef,
                                                           uint16_t* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[8][HC_NM + 2];
  __shared__ float S[HC_NM + 2];
  __shared__ float cf[HC_NM];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = D / 4;                               // float4 columns per stream
  const float* xr = x + (size_t)row * HC_NS * D;
  float acc[HC_NM + 1];
#pragma unroll
  for (int q = 0; q <= HC_NM; ++q) acc[q] = 0.f;
  float4 xv[HC_MAXV][HC_NS];
#pragma unroll
  for (int k = 0; k < HC_MAXV; ++k) {
    const int c = tid + k * HC_THREADS;
    if (c < V) {
#pragma unroll
      for (int h = 0; h < HC_NS; ++h) {
        const float4 v = *reinterpret_cast<const float4*>(xr + (size_t)h * D + 4 * c);
        xv[k][h] = v;
        acc[HC_NM] = fmaf(v.x, v.x, acc[HC_NM]); acc[HC_NM] = fmaf(v.y, v.y, acc[HC_NM]);
        acc[HC_NM] = fmaf(v.z, v.z, acc[HC_NM]); acc[HC_NM] = fmaf(v.w, v.w, acc[HC_NM]);
#pragma unroll
        for (int q = 0; q < HC_NM; ++q) {
          const float4 f = __ldg(reinterpret_cast<const float4*>(fn + ((size_t)q * HC_NS + h) * D + 4 * c));
          acc[q] = fmaf(v.x, f.x, acc[q]); acc[q] = fmaf(v.y, f.y, acc[q]); acc[q] = fmaf(v.z, f.z, acc[q]); acc[q] = fmaf(v.w, f.w, acc[q]);
        }
      }
    }
  }
#pragma unroll
  for (int q = 0; q <= HC_NM; ++q) {
    float v = acc[q];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp][q] = v;
  }
  __syncthreads();
  if (tid <= HC_NM) {
    float v = red[0][tid];
#pragma unroll
    for (int w = 1; w < 8; ++w) v += red[w][tid];
    S[tid] = v;
  }
  __syncthreads();
  if (warp == 0) {
    const float rmr = 1.f / sqrtf(S[HC_NM] / (float)(HC_NS * D) + rms_eps);
    if (lane < HC_NS) {
      cf[lane] = hc_sigmoid(fmaf(S[lane] * rmr, s0, base[lane])) + hc_eps;
      cf[HC_NS + lane] = 2.f * hc_sigmoid(fmaf(S[HC_NS + lane] * rmr, s1, base[HC_NS + lane]));
    }
    if (lane < HC_NS * HC_NS) {                      // lane = 4 i + j: row sums over xor 1, 2; column sums over xor 4, 8
      const unsigned mask = 0xFFFFu;
      float v = fmaf(S[2 * HC_NS + lane] * rmr, s2, base[2 * HC_NS + lane]);
      float mx = fmaxf(v, __shfl_xor_sync(mask, v, 1));
      mx = fmaxf(mx, __shfl_xor_sync(mask, mx, 2));
      v = expf(v - mx);
      float s = v;
      s += __shfl_xor_sync(mask, s, 1);
      s += __shfl_xor_sync(mask, s, 2);
      v = v / s + hc_eps;
      float cs = v;
      cs += __shfl_xor_sync(mask, cs, 4);
      cs += __shfl_xor_sync(mask, cs, 8);
      v = v / (cs + hc_eps);
      for (int it = 0; it < iters - 1; ++it) {
        float rs = v;
        rs += __shfl_xor_sync(mask, rs, 1);
        rs += __shfl_xor_sync(mask, rs, 2);
        v = v / (rs + hc_eps);
        cs = v;
        cs += __shfl_xor_sync(mask, cs, 4);
        cs += __shfl_xor_sync(mask, cs, 8);
        v = v / (cs + hc_eps);
      }
      cf[2 * HC_NS + lane] = v;
    }
  }
  __syncthreads();
  if (tid < HC_NM) coef[(size_t)row * HC_NM + tid] = cf[tid];
  // collapse with pre, then RMSNorm
  const float p0 = cf[0], p1 = cf[1], p2 = cf[2], p3 = cf[3];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < HC_MAXV; ++k) {
    if (tid + k * HC_THREADS < V) {
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int h = 0; h < HC_NS; ++h) {
        const float p = h == 0 ? p0 : (h == 1 ? p1 : (h == 2 ? p2 : p3));
        o.x = fmaf(p, xv[k][h].x, o.x); o.y = fmaf(p, xv[k][h].y, o.y); o.z = fmaf(p, xv[k][h].z, o.z); o.w = fmaf(p, xv[k][h].w, o.w);
      }
      xv[k][0] = o;
      ss = fmaf(o.x, o.x, ss); ss = fmaf(o.y, o.y, ss); ss = fmaf(o.z, o.z, ss); ss = fmaf(o.w, o.w, ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) red[warp][HC_NM + 1] = ss;
  __syncthreads();
  float tot = red[0][HC_NM + 1];
#pragma unroll
  for (int w = 1; w < 8; ++w) tot += red[w][HC_NM + 1];
  const float rinv = 1.f / sqrtf(tot / (float)D + norm_eps);
#pragma unroll
  for (int k = 0; k < HC_MAXV; ++k) {
    const int c = tid + k * HC_THREADS;
    if (c < V) {
      const uint2 w2 = *reinterpret_cast<const uint2*>(norm_w + 4 * c);
      const float w0 = __uint_as_float(w2.x << 16), w1 = __uint_as_float(w2.x & 0xFFFF0000u), w2f = __uint_as_float(w2.y << 16), w3 = __uint_as_float(w2.y & 0xFFFF0000u);
      const float4 o = xv[k][0];
      __nv_bfloat162 a = __floats2bfloat162_rn(o.x * rinv * w0, o.y * rinv * w1), b = __floats2bfloat162_rn(o.z * rinv * w2f, o.w * rinv * w3);
      uint2 u;
      u.x = *reinterpret_cast<uint32_t*>(&a);
      u.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(out + (size_t)row * D + 4 * c) = u;
    }
  }
}

// grid (rows, ceil(D / 4 / 256)): one float4 column of all four streams per thread
__global__ void __launch_bounds__(HC_THREADS) hc_apply_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ coef, int D) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, c = blockIdx.y * HC_THREADS + threadIdx.x;
  if (4 * c >= D) return;
  const float* cf = coef + (size_t)row * HC_NM;
  float* xr = x + (size_t)row * HC_NS * D + 4 * c;
  float4 xs[HC_NS];
#pragma unroll
  for (int g = 0; g < HC_NS; ++g) xs[g] = *reinterpret_cast<const float4*>(xr + (size_t)g * D);
  const float4 yv = *reinterpret_cast<const float4*>(y + (size_t)row * D + 4 * c);
#pragma unroll
  for (int h = 0; h < HC_NS; ++h) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int g = 0; g < HC_NS; ++g) {
      const float w = cf[2 * HC_NS + g * HC_NS + h];
      s.x = fmaf(w, xs[g].x, s.x); s.y = fmaf(w, xs[g].y, s.y); s.z = fmaf(w, xs[g].z, s.z); s.w = fmaf(w, xs[g].w, s.w);
    }
    const float p = cf[HC_NS + h];
    *reinterpret_cast<float4*>(xr + (size_t)h * D) = make_float4(fmaf(p, yv.x, s.x), fmaf(p, yv.y, s.y), fmaf(p, yv.z, s.z), fmaf(p, yv.w, s.w));
  }
}

}  // namespace rx

using namespace rx;

// x f32 [rows][4][D]; fn f32 [24][4 * D]; base f32 [24]; scale f32 x 3; norm_w bf16 [D]; coef f32 [rows][24] out; out bf16 [rows][D]
RX_API int rx_hc_mix(const void* x, const void* fn, const void* base, float s0, float s1, float s2, const void* norm_w, float rms_eps, float hc_eps,
                     float norm_eps, int iters, int rows, int D, void* coef, void* out, void* stream) {
  if (rows <= 0 || D <= 0 || D % 4 || D > 4 * HC_THREADS * HC_MAXV || iters < 1 || iters > 256) return (int)cudaErrorInvalidValue;
  rx::launch(hc_mix_kernel, dim3(rows), dim3(HC_THREADS), 0, (cudaStream_t)stream, (const float*)x, (const float*)fn, (const float*)base, s0, s1, s2,
             (const uint16_t*)norm_w, rms_eps, hc_eps, norm_eps, iters, D, (float*)coef, (uint16_t*)out);
  return (int)cudaGetLastError();
}

// x f32 [rows][4][D] in place; y f32 [rows][D]; coef from rx_hc_mix
RX_API int rx_hc_apply(void* x, const void* y, const void* coef, int rows, int D, void* stream) {
  if (rows <= 0 || D <= 0 || D % 4) return (int)cudaErrorInvalidValue;
  rx::launch(hc_apply_kernel, dim3(rows, (D / 4 + HC_THREADS - 1) / HC_THREADS), dim3(HC_THREADS), 0, (cudaStream_t)stream, (float*)x, (const float*)y,
             (const float*)coef, D);
  return (int)cudaGetLastError();
}
