// Device twin of the keyed sampler and the speculative accept rule (sm_100a).
//
// One thread per window row: from the row's top candidates (value desc, id asc - as the top-k kernel leaves them) it computes the
// keyed sample at the row's absolute position: T == 0 is the first candidate; else top-k cut, temperature, top-p (float64 softmax with
// numpy's pairwise sum order), min-p, then argmax of scaled logit + Gumbel(splitmix64(seed, position, id)).  Then one thread per
// sequence walks its rows: draft j is accepted iff it equals the sample of row j - 1, and the walk stops at the first miss.
// Arithmetic is float64 in the order of the host sampler, so the device and host paths pick the same token except where the
// device's exp/log differ from the host's in the last bit on an exact tie of scores.
// Semantics: reference crates/sampling/src/lib.rs:126-150 (uniform), :152-182 (pairwise sum), :210-268 (choose);
// crates/spec/src/lib.rs:33-35 (accept); crates/cuda/csrc/keyed.cuh (its device twin).
#include "common.cuh"

namespace rx {

struct SeqSampling {
  unsigned long long seed;
  double temperature, top_p, min_p;
  int top_k;
  int first_row;      // first row of the sequence in the window
  int n_rows;         // rows of the sequence: the base row + its drafts
  int position;       // absolute position of the token sampled from the first row
};

__device__ __forceinline__ unsigned long long vk_mix(unsigned long long x) {
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ double vk_uniform(unsigned long long seed, unsigned long long position, unsigned long long tid) {
  unsigned long long x = vk_mix(seed + 0x9E3779B97F4A7C15ull);
  x = vk_mix(x ^ (position * 0xD1B54A32D192ED03ull));
  x = vk_mix(x ^ tid);
  const double two_m53 = 1.0 / 9007199254740992.0;
  const double u = (double)(x >> 11) * two_m53 + two_m53 / 2.0;
  return fmin(u, 1.0 - two_m53);
}
// numpy's pairwise summation for n <= 128
__device__ __forceinline__ double vk_pairwise(const double* a, int n) {
  if (n < 8) {
    double r = 0.0;
    for (int i = 0; i < n; ++i) r += a[i];
    return r;
  }
  double r[8];
  for (int j = 0; j < 8; ++j) r[j] = a[j];
  int i = 8;
  for (; i < n - (n % 8); i += 8)
    for (int j = 0; j < 8; ++j) r[j] += a[i + j];
  double res = ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]));
  for (; i < n; ++i) res += a[i];
  return res;
}

// ids / vals: [rows, count].  drafts: int32 [rows] (the token fed at the row; row 0 of a sequence is its last sampled token).
// samples: int32 [rows] out.  accepted: int32 [n_seqs] out.  error: int32 [1], set to 1 when a row holds a NaN logit.
__global__ void __launch_bounds__(256) verify_accept_kernel(const int* __restrict__ ids, const float* __restrict__ vals, int rows, int count,
                                                            const SeqSampling* __restrict__ seqs, int n_seqs, const int* __restrict__ row_seq,
                                                            const int* __restrict__ drafts, int* __restrict__ samples, int* __restrict__ accepted,
                                                            int* __restrict__ error) {
  pdl_launch();
  pdl_wait();
  const int row = threadIdx.x;
  if (row < rows) {
    const SeqSampling s = seqs[row_seq[row]];
    const int* rid = ids + (size_t)row * count;
    const float* rv = vals + (size_t)row * count;
    const int position = s.position + (row - s.first_row);
    int pick = rid[0];
    bool nan = false;
    for (int i = 0; i < count; ++i) nan |= (rv[i] != rv[i]);
    if (nan) atomicExch(error, 1);
    if (s.temperature != 0.0 && !nan) {
      int k = s.top_k > 0 ? min(s.top_k, count) : count;
      if (k < 1) k = 1;
      const double t = fmax(s.temperature, 1e-6);
      double scaled[64];
      for (int i = 0; i < k; ++i) scaled[i] = (double)rv[i] / t;
      if (s.top_p > 0.0 && s.top_p < 1.0) {
        double probs[64];
        const double mx = scaled[0];
        for (int i = 0; i < k; ++i) probs[i] = exp(scaled[i] - mx);
        const double total = vk_pairwise(probs, k);
        double c = 0.0;
        int below = 0;
        for (int i = 0; i < k; ++i) {
          c += probs[i] / total;
          if (c < s.top_p) ++below;
        }
        k = min(below + 1, k);
      }
      if (s.min_p > 0.0) {
        const double floor_ = scaled[0] + log(s.min_p);
        int keep = 0;
        for (int i = 0; i < k; ++i) keep += scaled[i] >= floor_ ? 1 : 0;
        k = max(keep, 1);
      }
      int best = 0;
      double best_score = -INFINITY;
      for (int i = 0; i < k; ++i) {
        const double u = vk_uniform(s.seed, (unsigned long long)position, (unsigned long long)(unsigned)rid[i]);
        const double score = scaled[i] + (-log(-log(u)));
        if (score > best_score) { best_score = score; best = i; }
      }
      pick = rid[best];
    }
    samples[row] = pick;
  }
  __syncthreads();
  if (threadIdx.x < n_seqs) {
    const SeqSampling s = seqs[threadIdx.x];
    int a = 0;
    while (a + 1 < s.n_rows && drafts[s.first_row + a + 1] == samples[s.first_row + a]) ++a;
    accepted[threadIdx.x] = a;
  }
}

}  // namespace rx

using namespace rx;

RX_API int rx_verify_desc_size() { return (int)sizeof(SeqSampling); }

RX_API int rx_verify_accept(const void* ids, const void* vals, int rows, int count, const void* seqs, int n_seqs, const void* row_seq,
                            const void* drafts, void* samples, void* accepted, void* error, void* stream) {
  if (rows < 1 || rows > 256 || count < 1 || count > 64 || n_seqs < 1 || n_seqs > 256) return (int)cudaErrorInvalidValue;
  return (int)rx::launch(verify_accept_kernel, dim3(1), dim3(256), 0, (cudaStream_t)stream, (const int*)ids, (const float*)vals, rows, count,
                         (const SeqSampling*)seqs, n_seqs, (const int*)row_seq, (const int*)drafts, (int*)samples, (int*)accepted, (int*)error);
}
