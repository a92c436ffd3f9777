// EXL3 trellis encoder on the GPU: tail-biting Viterbi over the 65,536 sixteen-bit states of each 16x16 tile, one CTA per tile.
//
// Same search as the host encoder (native/csrc/trellis_encode.cpp), operation for operation, so both emit the same bits: a step is
// "best predecessor per shared prefix" (65,536 >> nb prefixes, 2^nb predecessors each, strict < in predecessor order) followed by one
// add per state; pass 1 runs over the ring rotated by half a tile with free ends and yields the seam, pass 2 is constrained to it.
// Path costs live in global memory (two 256 KB arrays per CTA, L2-resident), the per-prefix minima in shared memory (128 KB), the
// back pointers in global memory (256 x 32,768 bytes per CTA).  Contract: reference crates/quant/src/exl3_trellis.rs:6-24 and its
// CUDA encoder crates/quant/csrc/exl3_trellis.cu:1-25 (a bit ring whose decoded values minimise the squared error to the tile).
#include "common.cuh"

namespace rx {

constexpr int TE_THREADS = 1024;
constexpr size_t TE_BACK = (size_t)256 * 32768;
constexpr size_t TE_SCRATCH_PER_CTA = 2 * 65536 * sizeof(float) + TE_BACK;

__device__ __forceinline__ int te_end(int twice, int p1) { return (twice % 2 == 0) ? p1 * (twice / 2) : (p1 * twice - (p1 & 1)) / 2; }
__device__ __forceinline__ int te_nb(int twice, int p) { return te_end(twice, p + 1) - (p == 0 ? 0 : te_end(twice, p)); }

// One pass.  Returns (in *out_cost, by thread 0) the total cost; writes the states of all 256 values to `states` (shared memory).
__device__ void te_viterbi(int twice, const float* __restrict__ w, const float* __restrict__ table, int rot, int seam, float* cost, float* next,
                           uint8_t* back, float* best, uint16_t* states, float* red_c, int* red_s, float* out_cost) {
  const float INF = __int_as_float(0x7f800000);
  const int tid = threadIdx.x;
  {
    const int p = rot % 256, nb = te_nb(twice, p);
    const float x = w[p];
    for (int s = tid; s < 65536; s += TE_THREADS) {
      const float d = __fsub_rn(x, table[s]);
      cost[s] = (seam >= 0 && (s >> nb) != seam) ? INF : __fmul_rn(d, d);
    }
  }
  __syncthreads();
  for (int i = 1; i < 256; ++i) {
    const int p = (rot + i) % 256, nb = te_nb(twice, p);
    const int npre = 65536 >> nb, fan = 1 << nb;
    uint8_t* bk = back + (size_t)i * 32768;
    for (int u = tid; u < npre; u += TE_THREADS) {
      float b = cost[u];
      int arg = 0;
      for (int t = 1; t < fan; ++t) {
        const float c = cost[(t << (16 - nb)) | u];
        if (c < b) { b = c; arg = t; }
      }
      best[u] = b;
      bk[u] = (uint8_t)arg;
    }
    __syncthreads();
    const float x = w[p];
    for (int s = tid; s < 65536; s += TE_THREADS) {
      const float d = __fsub_rn(x, table[s]);
      next[s] = __fadd_rn(best[s >> nb], __fmul_rn(d, d));       // no fused multiply-add: the host encoder rounds the square first
    }
    __syncthreads();
    float* t = cost; cost = next; next = t;
  }
  // final state: lowest cost, lowest state among equals (the host scans states in order with a strict <)
  const int mask = (1 << (16 - te_nb(twice, rot % 256))) - 1;
  float bc = INF;
  int bs = 0x7fffffff;
  for (int s = tid; s < 65536; s += TE_THREADS) {
    if (seam >= 0 && (s & mask) != seam) continue;
    const float c = cost[s];
    if (c < bc || (c == bc && s < bs)) { bc = c; bs = s; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float oc = __shfl_xor_sync(0xffffffffu, bc, o);
    const int os = __shfl_xor_sync(0xffffffffu, bs, o);
    if (oc < bc || (oc == bc && os < bs)) { bc = oc; bs = os; }
  }
  if ((tid & 31) == 0) { red_c[tid >> 5] = bc; red_s[tid >> 5] = bs; }
  __syncthreads();
  if (tid == 0) {
    for (int k = 1; k < TE_THREADS / 32; ++k)
      if (red_c[k] < bc || (red_c[k] == bc && red_s[k] < bs)) { bc = red_c[k]; bs = red_s[k]; }
    int s = bs;
    for (int i = 255; i >= 0; --i) {
      states[(rot + i) % 256] = (uint16_t)s;
      if (i == 0) break;
      const int p = (rot + i) % 256, nb = te_nb(twice, p);
      const int u = s >> nb;
      const int t = back[(size_t)i * 32768 + u];
      s = (t << (16 - nb)) | u;
    }
    *out_cost = bc;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(TE_THREADS, 1) trellis_encode_kernel(const float* __restrict__ tiles, int T, int twice, const float* __restrict__ table,
                                                                       int16_t* __restrict__ out, float* __restrict__ err, uint8_t* __restrict__ scratch) {
  extern __shared__ float best[];           // 32,768 per-prefix minima
  __shared__ uint16_t states[256];
  __shared__ float w[256];
  __shared__ float red_c[TE_THREADS / 32];
  __shared__ int red_s[TE_THREADS / 32];
  __shared__ float total;
  uint8_t* mine = scratch + (size_t)blockIdx.x * TE_SCRATCH_PER_CTA;
  float* cost = (float*)mine;
  float* next = cost + 65536;
  uint8_t* back = mine + 2 * 65536 * sizeof(float);
  const int words = 8 * twice;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    if (threadIdx.x < 256) w[threadIdx.x] = tiles[(size_t)t * 256 + threadIdx.x];
    __syncthreads();
    te_viterbi(twice, w, table, 128, -1, cost, next, back, best, states, red_c, red_s, &total);
    const int seam = states[0] >> te_nb(twice, 0);
    __syncthreads();
    te_viterbi(twice, w, table, 0, seam, cost, next, back, best, states, red_c, red_s, &total);
    // pack: value p contributes its nb fresh bits, MSB first; words are 32 bits of the ring, stored as (low half, high half)
    if (threadIdx.x < words / 2) {
      const int wi = threadIdx.x;
      uint32_t v = 0;
      int start = 0;
      for (int p = 0; p < 256; ++p) {
        const int nb = te_nb(twice, p);
        if (start + nb > wi * 32 && start < wi * 32 + 32) {
          for (int b = 0; b < nb; ++b) {
            const int pos = start + b;
            if (pos >= wi * 32 && pos < wi * 32 + 32) v |= (uint32_t)((states[p] >> (nb - 1 - b)) & 1) << (31 - (pos - wi * 32));
          }
        }
        start += nb;
      }
      out[(size_t)t * words + 2 * wi] = (int16_t)(v & 0xFFFF);
      out[(size_t)t * words + 2 * wi + 1] = (int16_t)(v >> 16);
    }
    if (threadIdx.x == 0 && err != nullptr) err[t] = total;
    __syncthreads();
  }
}

}  // namespace rx

using namespace rx;

RX_API long long rx_trellis_encode_scratch_bytes(int ctas) { return (long long)ctas * (long long)TE_SCRATCH_PER_CTA; }

// tiles: f32 [T][256] in stream order (divided by the layer scale), table: f32 [65536] codebook values, out: int16 [T][16 * bits],
// err: f32 [T] or null, scratch: rx_trellis_encode_scratch_bytes(ctas) bytes.  All device pointers.
RX_API int rx_trellis_encode_cuda(const void* tiles, int T, int twice, const void* table, void* out, void* err, void* scratch, int ctas, void* stream) {
  static const int ok_twice[] = {2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16};
  bool ok = false;
  for (int v : ok_twice) ok |= (v == twice);
  if (!ok || T < 1 || ctas < 1) return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(trellis_encode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * (int)sizeof(float));
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int grid = T < ctas ? T : ctas;
  trellis_encode_kernel<<<grid, TE_THREADS, 32768 * sizeof(float), (cudaStream_t)stream>>>((const float*)tiles, T, twice, (const float*)table, (int16_t*)out,
                                                                                         (float*)err, (uint8_t*)scratch);
  return (int)cudaGetLastError();
}
