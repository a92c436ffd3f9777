// Glue kernels: the qkv finish fused with q/k RMSNorm, RoPE and the paged KV write; exact top-k candidates.
//
// Semantics matched: reference crates/cuda/csrc/glue.cu:182 (attn_prep: q/k norm + RoPE), attention.cu:234 (kv_write),
// glue.cu:667-709 (two-stage exact top-k with 64-bit keys, value desc / id asc).  KV layout is this engine's own:
// bf16 [num_pages][n_kv][64][head_dim].
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include "exl3_decode.cuh"

namespace rx {

__device__ __forceinline__ float g_bf16_to_f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t g_f_to_bf16(float f) {
  __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<uint16_t*>(&b);
}

// part: f32 [S][M][Nqkv], Nqkv = (n_q + 2 n_kv) * hd, column order q heads | k heads | v heads.
// For each 128-block: sum splits, Hadamard, * svh (+bias); q/k heads: optional RMSNorm over the head, RoPE (rotate-half);
// q -> q_out bf16 [M][n_q*hd]; k, v -> paged cache at slot[row] = page*64 + offset (slot < 0: row not cached).
template <int HD>
__global__ void finish_qkv_rope_kernel(const float* __restrict__ part, int S, int M, int n_q, int n_kv, const __half* __restrict__ svh,
                                       const float* __restrict__ bias, const uint16_t* __restrict__ q_norm, const uint16_t* __restrict__ k_norm,
                                       float eps, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                       const int* __restrict__ slot, uint16_t* __restrict__ q_out, uint16_t* __restrict__ k_cache,
                                       uint16_t* __restrict__ v_cache, const float* __restrict__ kv_scale, float* __restrict__ kv_amax,
                                       const int* __restrict__ pos3, int lim_h, int lim_w, float* __restrict__ k_ts, float* __restrict__ v_ts, int q4) {
  // q4 != 0 (with k_ts / v_ts): the caches are q4 rows - E2M1 nibbles, one E8M0 scale per 32 values in k_ts / v_ts read as uint8
  // [pages][n_kv][64][HD / 32]; scale = 2^ceil(log2(max(amax, 1e-4) / 6)) kept in 2^-14 .. 2^12, values rounded to nearest by the hardware conversion.
  // k_ts != nullptr: the caches are int8 with one power-of-two scale per (token, KV head), written to k_ts / v_ts (f32 [pages][n_kv][64]):
  // scale = 2^ceil(log2(amax / 127)), value = round(x / scale) (the reference's format, crates/cuda/csrc/nemotron_kv8.cuh:1-14).
  // pos3 != nullptr: interleaved M-RoPE (reference crates/cuda/csrc/glue.cu:178-180): int32 [rows][3] = the T, H and W position of each row;
  // frequency pair i rotates by the position of axis i % 3, the H axis only below pair lim_h = 3 * section_h and the W axis only below
  // lim_w = 3 * section_w (T elsewhere).  With T = H = W this is plain RoPE, bit for bit.
  // kv_scale != nullptr: the caches are FP8 (E4M3) bytes and K / V are stored as value / scale[head] (f32 [2][n_kv]: K scales, V scales),
  // saturating.  kv_amax != nullptr: the largest |K| and |V| per head are tracked there (f32 [2][n_kv]; used to calibrate the scales).
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int N = (n_q + 2 * n_kv) * HD;
  const size_t sstride = (size_t)M * N;
  const float pos = (float)positions[row];
  const int sl = slot[row];
  constexpr int GL = HD / 4;  // lanes per head
  for (int b = blockIdx.y * nw + warp; b < N / 128; b += gridDim.y * nw) {
    const int n0 = b * 128 + lane * 4;
    const size_t off = (size_t)row * N + n0;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (S == 1) acc = __ldg(reinterpret_cast<const float4*>(part + off));
    else
    for (int s0 = 0; s0 < S; s0 += 8) {   // eight independent loads in flight, added in split order
      float4 p[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < S) p[j] = __ldg(reinterpret_cast<const float4*>(part + (size_t)(s0 + j) * sstride + off));
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < S) {
          if (s0 + j == 0) acc = p[j];
          else { acc.x += p[j].x; acc.y += p[j].y; acc.z += p[j].z; acc.w += p[j].w; }
        }
    }
    float y[4] = {acc.x, acc.y, acc.z, acc.w};
    fwht128_warp(y);
    {
      const uint2 su = *reinterpret_cast<const uint2*>(svh + n0);
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), c = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
      y[0] *= a.x; y[1] *= a.y; y[2] *= c.x; y[3] *= c.y;
      if (bias != nullptr) {
        const float4 bb = *reinterpret_cast<const float4*>(bias + n0);
        y[0] += bb.x; y[1] += bb.y; y[2] += bb.z; y[3] += bb.w;
      }
    }
    const int head = n0 / HD, d0 = n0 % HD;
    const bool is_q = head < n_q, is_k = !is_q && head < n_q + n_kv;
    if (is_q || is_k) {
      const uint16_t* nw_ptr = is_q ? q_norm : k_norm;
      if (nw_ptr != nullptr) {
        float ss = y[0] * y[0] + y[1] * y[1] + y[2] * y[2] + y[3] * y[3];
#pragma unroll
        for (int o = 1; o < GL; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rinv = rsqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) y[i] = y[i] * rinv * g_bf16_to_f(nw_ptr[d0 + i]);
      }
      // rotate-half RoPE: element i pairs with i + HD/2, which lives GL/2 lanes away
      const bool first = (lane & (GL / 2)) == 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, y[i], GL / 2);
        const int fi = (d0 + i) % (HD / 2);
        float p = pos;
        if (pos3 != nullptr) {
          const int axis = (fi % 3 == 1 && fi < lim_h) ? 1 : ((fi % 3 == 2 && fi < lim_w) ? 2 : 0);
          p = (float)pos3[row * 3 + axis];
        }
        float sn, cs;
        sincosf(p * inv_freq[fi], &sn, &cs);
        y[i] = first ? (y[i] * cs - other * sn) : (y[i] * cs + other * sn);
      }
    }
    uint2 u;
    u.x = (uint32_t)g_f_to_bf16(y[0]) | ((uint32_t)g_f_to_bf16(y[1]) << 16);
    u.y = (uint32_t)g_f_to_bf16(y[2]) | ((uint32_t)g_f_to_bf16(y[3]) << 16);
    if (is_q) {
      *reinterpret_cast<uint2*>(q_out + (size_t)row * n_q * HD + n0) = u;
    } else if (sl >= 0) {
      const int kvh = is_k ? head - n_q : head - n_q - n_kv;
      const size_t addr = (((size_t)(sl / 64) * n_kv + kvh) * 64 + (sl % 64)) * HD + d0;
      if (kv_amax != nullptr) {
        float am = fmaxf(fmaxf(fabsf(y[0]), fabsf(y[1])), fmaxf(fabsf(y[2]), fabsf(y[3])));
#pragma unroll
        for (int o = 1; o < GL; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        if ((lane % GL) == 0) atomicMax(reinterpret_cast<unsigned*>(kv_amax) + (is_k ? 0 : n_kv) + kvh, __float_as_uint(am));   // non-negative floats order like their bits
      }
      if (k_ts != nullptr && q4) {
        float am = fmaxf(fmaxf(fabsf(y[0]), fabsf(y[1])), fmaxf(fabsf(y[2]), fabsf(y[3])));
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));       // 8 lanes x 4 values = one group of 32
        int e = (int)ceilf(log2f(fmaxf(am, 1e-4f) * (1.f / 6.f)));
        e = max(-14, min(12, e));
        const float inv = exp2f((float)-e);
        const __nv_fp4x2_storage_t a = __nv_cvt_float2_to_fp4x2(make_float2(y[0] * inv, y[1] * inv), __NV_E2M1, cudaRoundNearest);
        const __nv_fp4x2_storage_t b2 = __nv_cvt_float2_to_fp4x2(make_float2(y[2] * inv, y[3] * inv), __NV_E2M1, cudaRoundNearest);
        *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(is_k ? k_cache : v_cache) + addr / 2) = (uint16_t)((uint32_t)a | ((uint32_t)b2 << 8));
        if ((lane & 7) == 0)
          reinterpret_cast<uint8_t*>(is_k ? k_ts : v_ts)[(((size_t)(sl / 64) * n_kv + kvh) * 64 + (sl % 64)) * (HD / 32) + d0 / 32] = (uint8_t)(e + 127);
      } else if (k_ts != nullptr) {
        float am = fmaxf(fmaxf(fabsf(y[0]), fabsf(y[1])), fmaxf(fabsf(y[2]), fabsf(y[3])));
#pragma unroll
        for (int o = 1; o < GL; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        // smallest power of two with amax / scale <= 127, kept inside what fp16 can carry when the attention kernels multiply it back in
        int e = am > 0.f ? (int)ceilf(log2f(am * (1.f / 127.f))) : -14;
        e = max(-14, min(8, e));
        const float sc = exp2f((float)e), inv = exp2f((float)-e);
        int qv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) qv[i] = max(-127, min(127, __float2int_rn(y[i] * inv)));
        const uint32_t packed = (uint32_t)(qv[0] & 0xFF) | ((uint32_t)(qv[1] & 0xFF) << 8) | ((uint32_t)(qv[2] & 0xFF) << 16) | ((uint32_t)(qv[3] & 0xFF) << 24);
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(is_k ? k_cache : v_cache) + addr) = packed;
        if ((lane % GL) == 0) (is_k ? k_ts : v_ts)[((size_t)(sl / 64) * n_kv + kvh) * 64 + (sl % 64)] = sc;
      } else if (kv_scale != nullptr) {
        const float inv = 1.f / kv_scale[(is_k ? 0 : n_kv) + kvh];
        const __nv_fp8x2_storage_t a = __nv_cvt_float2_to_fp8x2(make_float2(y[0] * inv, y[1] * inv), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t b2 = __nv_cvt_float2_to_fp8x2(make_float2(y[2] * inv, y[3] * inv), __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(is_k ? k_cache : v_cache) + addr) = (uint32_t)a | ((uint32_t)b2 << 16);
      } else {
        *reinterpret_cast<uint2*>((is_k ? k_cache : v_cache) + addr) = u;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ exact top-k
// key = (order-preserving bits of the float) << 32 | ~id : bigger key = bigger value, then lower id.
__device__ __forceinline__ uint64_t topk_key(float v, uint32_t id) {
  uint32_t b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((uint64_t)b << 32) | (uint32_t)(~id);
}
__device__ __forceinline__ float topk_val(uint64_t k) {
  uint32_t b = (uint32_t)(k >> 32);
  b = (b & 0x80000000u) ? (b & 0x7FFFFFFFu) : ~b;
  return __uint_as_float(b);
}
__device__ __forceinline__ uint64_t u64_max(uint64_t a, uint64_t b) { return a > b ? a : b; }

constexpr int TOPK_THREADS = 256;
constexpr int TOPK_PER_THREAD = 16;
constexpr int TOPK_CHUNK = TOPK_THREADS * TOPK_PER_THREAD;

// `count` rounds of block-wide max over keys held in registers; winners are removed (set to 0) by their owner.
__device__ __forceinline__ void block_select(uint64_t (&k)[TOPK_PER_THREAD], int count, uint64_t* out, uint64_t* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = 0; r < count; ++r) {
    uint64_t best = 0;
#pragma unroll
    for (int i = 0; i < TOPK_PER_THREAD; ++i) best = u64_max(best, k[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = u64_max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (lane == 0) red[warp] = best;
    __syncthreads();
    uint64_t all = 0;
#pragma unroll
    for (int w = 0; w < TOPK_THREADS / 32; ++w) all = u64_max(all, red[w]);
    if (threadIdx.x == 0) out[r] = all;
#pragma unroll
    for (int i = 0; i < TOPK_PER_THREAD; ++i)
      if (k[i] == all) k[i] = 0;  // keys are unique (ids differ), so exactly one slot matches
    __syncthreads();
  }
}

__global__ void topk_stage1_kernel(const float* __restrict__ logits, int vocab, int count, uint64_t* __restrict__ cand, int nchunks) {
  pdl_launch();
  pdl_wait();
  __shared__ uint64_t red[TOPK_THREADS / 32];
  const int row = blockIdx.y, chunk = blockIdx.x;
  const float* lr = logits + (size_t)row * vocab;
  uint64_t k[TOPK_PER_THREAD];
#pragma unroll
  for (int i = 0; i < TOPK_PER_THREAD; ++i) {
    const int id = chunk * TOPK_CHUNK + i * TOPK_THREADS + threadIdx.x;
    k[i] = id < vocab ? topk_key(lr[id], (uint32_t)id) : 0;
  }
  block_select(k, count, cand + ((size_t)row * nchunks + chunk) * count, red);
}

__global__ void topk_stage2_kernel(const uint64_t* __restrict__ cand, int total, int count, int* __restrict__ ids, float* __restrict__ vals) {
  pdl_launch();
  pdl_wait();
  __shared__ uint64_t red[TOPK_THREADS / 32];
  __shared__ uint64_t outk[64];
  const int row = blockIdx.x;
  const uint64_t* c = cand + (size_t)row * total;
  uint64_t k[TOPK_PER_THREAD];
#pragma unroll
  for (int i = 0; i < TOPK_PER_THREAD; ++i) k[i] = 0;
  // fold candidates beyond the register capacity by keeping the per-slot maximum of a strided sweep's survivors:
  // total <= TOPK_CHUNK is guaranteed by the launcher (it runs stage 2 repeatedly otherwise)
#pragma unroll
  for (int i = 0; i < TOPK_PER_THREAD; ++i) {
    const int j = i * TOPK_THREADS + threadIdx.x;
    if (j < total) k[i] = c[j];
  }
  block_select(k, count, outk, red);
  if (threadIdx.x < count) {
    const uint64_t kk = outk[threadIdx.x];
    ids[(size_t)row * count + threadIdx.x] = (int)(~(uint32_t)kk);
    vals[(size_t)row * count + threadIdx.x] = topk_val(kk);
  }
}

}  // namespace rx

using namespace rx;

RX_API int rx_finish_qkv_rope(const void* part, int S, int M, int n_q, int n_kv, int hd, const void* svh, const void* bias, const void* q_norm,
                              const void* k_norm, float eps, const void* positions, const void* inv_freq, const void* slot, void* q_out,
                              void* k_cache, void* v_cache, void* stream, const void* kv_scale, void* kv_amax, const void* pos3, int section_h,
                              int section_w, void* k_tscale, void* v_tscale, int q4) {
  const int N = (n_q + 2 * n_kv) * hd;
  if (N % 128) return (int)cudaErrorInvalidValue;
  const int per_row = (N / 128 + 7) / 8;   // one warp per 128-block
  dim3 grid(M, per_row < 1 ? 1 : per_row);
  cudaStream_t st = (cudaStream_t)stream;
#define RX_ARGS (const float*)part, S, M, n_q, n_kv, (const __half*)svh, (const float*)bias, (const uint16_t*)q_norm, (const uint16_t*)k_norm, eps, \
                (const int*)positions, (const float*)inv_freq, (const int*)slot, (uint16_t*)q_out, (uint16_t*)k_cache, (uint16_t*)v_cache, \
                (const float*)kv_scale, (float*)kv_amax, (const int*)pos3, 3 * section_h, 3 * section_w, (float*)k_tscale, (float*)v_tscale, q4
  if (hd == 128) rx::launch(finish_qkv_rope_kernel<128>, dim3(grid), dim3(256), 0, st, RX_ARGS);
  else if (hd == 64) rx::launch(finish_qkv_rope_kernel<64>, dim3(grid), dim3(256), 0, st, RX_ARGS);
  else return (int)cudaErrorInvalidValue;
#undef RX_ARGS
  return (int)cudaGetLastError();
}

// scratch: uint64 [rows * nchunks * count] with nchunks = ceil(vocab / 4096); ids int32 [rows, count], vals f32 [rows, count]
RX_API long long rx_topk_scratch_bytes(int rows, int vocab, int count) {
  return (long long)rows * ((vocab + TOPK_CHUNK - 1) / TOPK_CHUNK) * count * 8;
}

RX_API int rx_topk(const void* logits, int rows, int vocab, int count, void* scratch, void* ids, void* vals, void* stream) {
  if (count < 1 || count > 64) return (int)cudaErrorInvalidValue;
  const int nchunks = (vocab + TOPK_CHUNK - 1) / TOPK_CHUNK;
  if (nchunks * count > TOPK_CHUNK) return (int)cudaErrorInvalidValue;  // vocab up to 65536 * 2048 / count: never hit in practice
  cudaStream_t st = (cudaStream_t)stream;
  rx::launch(topk_stage1_kernel, dim3(dim3(nchunks, rows)), dim3(TOPK_THREADS), 0, st, (const float*)logits, vocab, count, (uint64_t*)scratch, nchunks);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  rx::launch(topk_stage2_kernel, dim3(rows), dim3(TOPK_THREADS), 0, st, (const uint64_t*)scratch, nchunks * count, count, (int*)ids, (float*)vals);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ content digest of device memory
// digest = sum over 8-byte words w_i of mix(w_i xor (i + 1) * 0x9E3779B97F4A7C15) modulo 2^64, mix = the splitmix64 finaliser: keyed by the
// word's position, and a sum, so any grid computes the same value.  A tail of fewer than 8 bytes is zero-extended.  Role: checking that a
// snapshot of recurrent state or of KV pages restored from a cache holds what was stored (reference crates/cuda/csrc/state_digest.cu).
namespace rx {
__device__ __forceinline__ unsigned long long digest_mix(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__global__ void __launch_bounds__(256) state_digest_kernel(const uint8_t* __restrict__ p, long long bytes, unsigned long long* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  const long long words = bytes >> 3;
  unsigned long long acc = 0;
  const unsigned long long* w = reinterpret_cast<const unsigned long long*>(p);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (long long)gridDim.x * blockDim.x)
    acc += digest_mix(w[i] ^ ((unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull));
  if (blockIdx.x == 0 && threadIdx.x == 0 && (bytes & 7)) {
    unsigned long long t = 0;
    for (int k = 0; k < (int)(bytes & 7); ++k) t |= (unsigned long long)p[(words << 3) + k] << (8 * k);
    acc += digest_mix(t ^ ((unsigned long long)(words + 1) * 0x9E3779B97F4A7C15ull));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0 && acc != 0) atomicAdd(out, acc);
}
}  // namespace rx

// *out (a device uint64 the caller zeroed) += digest of `bytes` bytes at `p` (8-byte aligned).  Several calls into the same word digest a
// scattered object; the order of the calls does not matter only if each part is keyed by the caller (here: it is not - digest parts in a fixed order
// into separate words when the order must count).
RX_API int rx_state_digest(const void* p, long long bytes, void* out, void* stream) {
  if (p == nullptr || out == nullptr || bytes < 0 || ((uintptr_t)p & 7)) return (int)cudaErrorInvalidValue;
  if (bytes == 0) return 0;
  long long blocks = (bytes / 8 + 256 * 8 - 1) / (256 * 8);
  if (blocks < 1) blocks = 1;
  if (blocks > 1024) blocks = 1024;
  rx::launch(state_digest_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const uint8_t*)p, bytes, (unsigned long long*)out);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ allocation-free top-k
// Scratch for rx_topk_static: the stage-1 candidate keys of up to TOPK_STATIC_ROWS rows.  It lives in the library image, so
// every GPU that loads the library holds these 2 MiB until the process exits.
namespace rx {
constexpr int TOPK_STATIC_ROWS = 64;
constexpr int TOPK_STATIC_CHUNKS = 64;      // vocabularies up to 64 * 4096 = 262,144 entries
constexpr int TOPK_STATIC_COUNT = 64;
static __device__ __align__(256) unsigned long long g_topk_static_scratch[(size_t)TOPK_STATIC_ROWS * TOPK_STATIC_CHUNKS * TOPK_STATIC_COUNT];
constexpr int TOPK_STATIC_MAX_DEVICES = 64;
static void* g_topk_static_ptr[TOPK_STATIC_MAX_DEVICES];   // per device: the array's DEVICE address (the symbol itself is a host stand-in)
}  // namespace rx

// Exact top-`count` candidates of every row, like rx_topk, for callers that cannot allocate device memory: a serving
// loop whose memory plan is sealed after start-up, a plugin called from someone else's stream callback, code running
// while a pool allocator is locked.  The caller passes only inputs and outputs; the intermediate candidate list goes to
// a fixed array inside this library.
//   limits : rows <= 64, vocab <= 262,144, 1 <= count <= 64 (anything larger is refused with cudaErrorInvalidValue)
//   set-up : the first call on each device looks up the array's device address (cudaGetSymbolAddress with that device
//            current).  Make that first call outside any stream capture.
//   sharing: all calls use the same array, which keeps whatever the last call left in it; this routine overwrites every
//            slot it later reads, so no clearing is needed, but two calls that overlap on the GPU (different streams)
//            race on it.  Serialise them.
// No cudaMalloc / cudaFree / allocating library call is made, here or in the kernels.
RX_API int rx_topk_static(const void* logits, int rows, int vocab, int count, void* ids, void* vals, void* stream) {
  if (logits == nullptr || ids == nullptr || vals == nullptr) return (int)cudaErrorInvalidValue;
  if (rows < 1 || rows > TOPK_STATIC_ROWS || count < 1 || count > TOPK_STATIC_COUNT || vocab < 1) return (int)cudaErrorInvalidValue;
  const int nchunks = (vocab + TOPK_CHUNK - 1) / TOPK_CHUNK;
  if (nchunks > TOPK_STATIC_CHUNKS || nchunks * count > TOPK_CHUNK) return (int)cudaErrorInvalidValue;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= TOPK_STATIC_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
  if (g_topk_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_topk_static_scratch);
    if (e != cudaSuccess) return (int)e;
    g_topk_static_ptr[dev] = p;
  }
  uint64_t* scratch = (uint64_t*)g_topk_static_ptr[dev];
  cudaStream_t st = (cudaStream_t)stream;
  e = rx::launch(topk_stage1_kernel, dim3(nchunks, rows), dim3(TOPK_THREADS), 0, st, (const float*)logits, vocab, count, scratch, nchunks);
  if (e != cudaSuccess) return (int)e;
  e = rx::launch(topk_stage2_kernel, dim3(rows), dim3(TOPK_THREADS), 0, st, (const uint64_t*)scratch, nchunks * count, count, (int*)ids,
                 (float*)vals);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}
