// Mamba2 (SSD) token mixer for hybrid decoders: causal depthwise conv over x | B | C, discretization, fp32 state recurrence,
// grouped gated RMSNorm.  Semantics matched: reference crates/cuda/csrc/nemotron_ssm.cu:1-45 (conv k=4 with a 3-row history,
// dt = softplus(dt + bias), decay exp(dt * A), y = C . S + D * x, gated norm over d_inner / groups channels) and
// crates/model/src/families/nemotron_h_omni/ssm_ref.rs.
//
// This engine's own layout and schedule:
//   proj      f32 [M][ldp]: the in_proj output row, columns z (d_inner) | x (d_inner) | B (G*N) | C (G*N) | dt (H) | padding
//   conv pool f32 [slots][3][C]      C = d_inner + 2 G N; the last three pre-conv x|B|C rows of the sequence, oldest first
//   ssm pool  f32 [slots][H][P][N]   P = 64 (head dim), N = 128 (state); n contiguous
// Rows of one sequence are consecutive and in position order (a "segment"); a sequence appears in at most one segment of a
// launch.  A row at position 0 starts from a zero state whatever the pools hold, so a slot needs no reset when it is reused.
// Record / commit split (reference crates/cuda/csrc/gdn.cu:253-322: a verify window reads the pools, a later commit replays the accepted
// prefix): the recurrence kernels take a mode.  SCAN_OUT alone = a window whose rows may still be rejected: the pools are read, outputs are
// written, nothing is stored back; the caller keeps that launch's `proj` and `xbc` rows (per layer) as the record.  SCAN_STATE alone = the
// commit: the same kernel walks the first `keep` recorded rows of each sequence again (the same arithmetic on the same inputs, so the state
// equals what a serial decode of those rows leaves, bit for bit) and stores the state and the conv history; outputs are not written.
// SCAN_OUT | SCAN_STATE = rows that are final when fed (prefill, windows without drafts).
//
// The conv is parallel over rows (each row reads its three predecessors from the launch's own rows or from the pool); the
// recurrence is sequential over the rows of a segment with the state of one head in the registers of a 256-thread CTA
// (thread = one p, 32 of the 128 n), so a decode step moves each state once: 2 x 32 KB per (sequence, head).
#include "common.cuh"

namespace rx {

constexpr int SSM_P = 64, SSM_N = 128, SSM_HIST = 3;
constexpr int SCAN_OUT = 1, SCAN_STATE = 2;
constexpr int SCAN_PF = 4;                        // tokens whose inputs the split scans keep in flight

__device__ __forceinline__ float ssm_silu(float v) { return v / (1.f + __expf(-v)); }
__device__ __forceinline__ float ssm_bf(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// the pre-conv value of channel c at `back` positions before row r (back 1..3), or of row r itself (back 0)
__device__ __forceinline__ float ssm_conv_in(const float* __restrict__ proj, int ldp, int xoff, const float* pool, int C,
                                             const int* __restrict__ row_seq, const int* __restrict__ positions, int r, int back, int c) {
  const int pos = positions[r];
  if (pos - back < 0) return 0.f;
  const int seq = row_seq[r];
  if (r - back >= 0 && row_seq[r - back] == seq) return proj[(size_t)(r - back) * ldp + xoff + c];
  // not in this launch: the pool holds positions (first - 3, first - 2, first - 1) of the segment's first row
  int o = 0;                                   // rows of the segment before r (only 0..2 can get here)
  while (o < back && r - o - 1 >= 0 && row_seq[r - o - 1] == seq) ++o;
  return pool[((size_t)seq * SSM_HIST + (SSM_HIST - back + o)) * C + c];
}

// the segment's last three pre-conv rows become the sequence's conv history.  Every CTA of the segment (one per head) commits its own
// share of the channels after its recurrence: left to one CTA, this loop of dependent loads was most of a decode step's kernel time.
__device__ __forceinline__ void ssm_conv_commit(const float* __restrict__ proj, int ldp, int xoff, float* conv_pool, int C,
                                                const int* __restrict__ row_seq, const int* __restrict__ positions, int last, int seq, int part,
                                                int nparts) {
  const int chunk = (C + nparts - 1) / nparts, c0 = part * chunk, c1 = min(C, c0 + chunk);
  for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
    float v[SSM_HIST];
#pragma unroll
    for (int k = 0; k < SSM_HIST; ++k) v[k] = ssm_conv_in(proj, ldp, xoff, conv_pool, C, row_seq, positions, last, SSM_HIST - 1 - k, c);
#pragma unroll
    for (int k = 0; k < SSM_HIST; ++k) conv_pool[((size_t)seq * SSM_HIST + k) * C + c] = v[k];
  }
}

// xbc[r][c] = silu(b[c] + sum_j w[c][j] * in(pos - 3 + j)), grid (M, ceil(C / 256))
__global__ void __launch_bounds__(256) ssm_conv_kernel(const float* __restrict__ proj, int ldp, int xoff, int C, const int* __restrict__ row_seq,
                                                      const int* __restrict__ positions, const uint16_t* __restrict__ conv_w,
                                                      const uint16_t* __restrict__ conv_b, const float* __restrict__ pool, float* __restrict__ xbc) {
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
  if (c >= C) return;
  float acc = ssm_bf(conv_b[c]);
#pragma unroll
  for (int j = 0; j < 4; ++j) acc += ssm_bf(conv_w[c * 4 + j]) * ssm_conv_in(proj, ldp, xoff, pool, C, row_seq, positions, r, 3 - j, c);
  xbc[(size_t)r * C + c] = ssm_silu(acc);
}

// Recurrence.  grid (segments or rows, H).  With a segment table (seg_start != nullptr) block x is segment x; without one block x is
// row x and returns unless that row opens a segment.  Each block also writes its share of the segment's last three pre-conv rows to the conv pool.
__global__ void __launch_bounds__(256) ssm_scan_kernel(const float* __restrict__ xbc, int C, const float* __restrict__ proj, int ldp, int xoff,
                                                      int dtoff, int M, int H, int G, const int* __restrict__ row_seq,
                                                      const int* __restrict__ positions, const int* __restrict__ seg_start,
                                                      const int* __restrict__ seg_len, const float* __restrict__ dt_bias,
                                                      const float* __restrict__ a_neg, const float* __restrict__ d_skip,
                                                      float* __restrict__ ssm_pool, float* conv_pool, float* __restrict__ y, int mode) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float sB[SSM_N], sC[SSM_N], sx[SSM_P];
  int r0, len;
  if (seg_start != nullptr) {
    r0 = seg_start[blockIdx.x];
    len = seg_len[blockIdx.x];
  } else {
    r0 = blockIdx.x;
    if (r0 > 0 && row_seq[r0 - 1] == row_seq[r0]) return;
    len = 1;
    while (r0 + len < M && row_seq[r0 + len] == row_seq[r0]) ++len;
  }
  if (len <= 0) return;
  const int h = blockIdx.y, tid = threadIdx.x, p = tid >> 2, nq = tid & 3;
  const int seq = row_seq[r0], g = h / (H / G), DI = H * SSM_P;
  float st[32];
  float* sp = ssm_pool + (((size_t)seq * H + h) * SSM_P + p) * SSM_N + nq * 32;
  if (positions[r0] == 0) {
#pragma unroll
    for (int i = 0; i < 32; ++i) st[i] = 0.f;
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(sp + i);
      st[i] = v.x, st[i + 1] = v.y, st[i + 2] = v.z, st[i + 3] = v.w;
    }
  }
  const float A = a_neg[h], Dh = d_skip[h], dtb = dt_bias[h];
  // this thread's share of a token's inputs (one B or C value, one x value for the first 64 threads, the head's dt); the next token's are
  // fetched while the current one is computed, so a long segment is not a chain of dependent global loads
  const int bc_off = tid < SSM_N ? DI + g * SSM_N + tid : DI + G * SSM_N + g * SSM_N + (tid - SSM_N);
  float n_bc = xbc[(size_t)r0 * C + bc_off], n_x = tid < SSM_P ? xbc[(size_t)r0 * C + h * SSM_P + tid] : 0.f, n_dt = proj[(size_t)r0 * ldp + dtoff + h];
  for (int t = 0; t < len; ++t) {
    const int r = r0 + t;
    const float c_bc = n_bc, c_x = n_x, c_dt = n_dt;
    if (t + 1 < len) {
      const float* xn = xbc + (size_t)(r + 1) * C;
      n_bc = xn[bc_off];
      if (tid < SSM_P) n_x = xn[h * SSM_P + tid];
      n_dt = proj[(size_t)(r + 1) * ldp + dtoff + h];
    }
    __syncthreads();
    if (tid < SSM_N) sB[tid] = c_bc;
    else sC[tid - SSM_N] = c_bc;
    if (tid < SSM_P) sx[tid] = c_x;
    __syncthreads();
    float dt = c_dt + dtb;
    dt = dt > 20.f ? dt : log1pf(__expf(dt));            // softplus
    const float dA = __expf(dt * A), xdt = sx[p] * dt;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;     // four partial sums: dependent chains of 8 instead of 32
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 bb = *reinterpret_cast<const float4*>(sB + nq * 32 + i), cc = *reinterpret_cast<const float4*>(sC + nq * 32 + i);
      st[i] = st[i] * dA + xdt * bb.x; st[i + 1] = st[i + 1] * dA + xdt * bb.y; st[i + 2] = st[i + 2] * dA + xdt * bb.z; st[i + 3] = st[i + 3] * dA + xdt * bb.w;
      a0 += st[i] * cc.x; a1 += st[i + 1] * cc.y; a2 += st[i + 2] * cc.z; a3 += st[i + 3] * cc.w;
    }
    float acc = (a0 + a1) + (a2 + a3);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (nq == 0 && (mode & SCAN_OUT)) y[(size_t)r * DI + h * SSM_P + p] = acc + Dh * sx[p];
  }
  if (!(mode & SCAN_STATE)) return;
#pragma unroll
  for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(sp + i) = make_float4(st[i], st[i + 1], st[i + 2], st[i + 3]);
  ssm_conv_commit(proj, ldp, xoff, conv_pool, C, row_seq, positions, r0 + len - 1, seq, h, (int)gridDim.y);
}

// Prefill / commit form of the recurrence: a head's 64 state rows p are split over SSM_PS one-warp CTAs (row p only meets x_p, B, C and dt), with
// the SAME (p, quarter of n) -> lane mapping and arithmetic as ssm_scan_kernel, so states and outputs are bit-identical; one warp per CTA means no
// block barrier on the per-token path and 8 x more CTAs for a one-sequence prefill.  grid (segments, H, SSM_PS), 32 threads.
constexpr int SSM_PS = 8;
__global__ void __launch_bounds__(32) ssm_scan_split_kernel(const float* __restrict__ xbc, int C, const float* __restrict__ proj, int ldp, int xoff,
                                                           int dtoff, int M, int H, int G, const int* __restrict__ row_seq,
                                                           const int* __restrict__ positions, const int* __restrict__ seg_start,
                                                           const int* __restrict__ seg_len, const float* __restrict__ dt_bias,
                                                           const float* __restrict__ a_neg, const float* __restrict__ d_skip,
                                                           float* __restrict__ ssm_pool, float* conv_pool, float* __restrict__ y, int mode) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float sB[SSM_N], sC[SSM_N];
  const int r0 = seg_start[blockIdx.x], len = seg_len[blockIdx.x];
  if (len <= 0) return;
  const int h = blockIdx.y, pz = blockIdx.z, lane = threadIdx.x, p = pz * 8 + (lane >> 2), nq = lane & 3;
  const int seq = row_seq[r0], g = h / (H / G), DI = H * SSM_P;
  float st[32];
  float* sp = ssm_pool + (((size_t)seq * H + h) * SSM_P + p) * SSM_N + nq * 32;
  if (positions[r0] == 0) {
#pragma unroll
    for (int i = 0; i < 32; ++i) st[i] = 0.f;
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(sp + i);
      st[i] = v.x, st[i + 1] = v.y, st[i + 2] = v.z, st[i + 3] = v.w;
    }
  }
  const float A = a_neg[h], Dh = d_skip[h], dtb = dt_bias[h];
  // a lane's share of a token's inputs: B and C values 32 c + lane (c = 0..3), its row's x, the head's dt; the next token's are in flight while
  // the current one is computed
  struct In { float b[4], c[4], x, dt; };
  auto fetch = [&](int r) {
    In in;
    const float* xr = xbc + (size_t)r * C;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      in.b[c] = xr[DI + g * SSM_N + 32 * c + lane];
      in.c[c] = xr[DI + G * SSM_N + g * SSM_N + 32 * c + lane];
    }
    in.x = xr[h * SSM_P + p];
    in.dt = proj[(size_t)r * ldp + dtoff + h];
    return in;
  };
  // a ring of SCAN_PF tokens' inputs in registers: one iteration is far shorter than a trip to memory, so the loads run SCAN_PF tokens ahead
  In ring[SCAN_PF];
#pragma unroll
  for (int k = 0; k < SCAN_PF; ++k)
    if (k < len) ring[k] = fetch(r0 + k);
  for (int t0 = 0; t0 < len; t0 += SCAN_PF) {
#pragma unroll
  for (int k = 0; k < SCAN_PF; ++k) {
    const int t = t0 + k;
    if (t >= len) break;
    const int r = r0 + t;
    const In cur = ring[k];
    if (t + SCAN_PF < len) ring[k] = fetch(r + SCAN_PF);
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 4; ++c) { sB[32 * c + lane] = cur.b[c]; sC[32 * c + lane] = cur.c[c]; }
    __syncwarp();
    float dt = cur.dt + dtb;
    dt = dt > 20.f ? dt : log1pf(__expf(dt));            // softplus
    const float dA = __expf(dt * A), xdt = cur.x * dt;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 bb = *reinterpret_cast<const float4*>(sB + nq * 32 + i), cc = *reinterpret_cast<const float4*>(sC + nq * 32 + i);
      st[i] = st[i] * dA + xdt * bb.x; st[i + 1] = st[i + 1] * dA + xdt * bb.y; st[i + 2] = st[i + 2] * dA + xdt * bb.z; st[i + 3] = st[i + 3] * dA + xdt * bb.w;
      a0 += st[i] * cc.x; a1 += st[i + 1] * cc.y; a2 += st[i + 2] * cc.z; a3 += st[i + 3] * cc.w;
    }
    float acc = (a0 + a1) + (a2 + a3);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (nq == 0 && (mode & SCAN_OUT)) y[(size_t)r * DI + h * SSM_P + p] = acc + Dh * cur.x;
  }
  }
  if (!(mode & SCAN_STATE)) return;
#pragma unroll
  for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(sp + i) = make_float4(st[i], st[i + 1], st[i + 2], st[i + 3]);
  ssm_conv_commit(proj, ldp, xoff, conv_pool, C, row_seq, positions, r0 + len - 1, seq, h * SSM_PS + pz, (int)(gridDim.y * SSM_PS));
}

// out[r][c] = bf16( rmsnorm_group( y * silu(z) )[c] * w[c] ), grid (M, G); the group is d_inner / G channels wide
__global__ void __launch_bounds__(256) ssm_gate_norm_kernel(const float* __restrict__ y, const float* __restrict__ proj, int ldp, int DI, int G,
                                                           const uint16_t* __restrict__ norm_w, float eps, uint16_t* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[8];
  const int r = blockIdx.x, g = blockIdx.y, W = DI / G, c0 = g * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += 256) {
    const float v = y[(size_t)r * DI + c0 + c] * ssm_silu(proj[(size_t)r * ldp + c0 + c]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rinv = rsqrtf(tot / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += 256) {
    const float v = y[(size_t)r * DI + c0 + c] * ssm_silu(proj[(size_t)r * ldp + c0 + c]);
    __nv_bfloat16 b = __float2bfloat16_rn(v * rinv * ssm_bf(norm_w[c0 + c]));
    out[(size_t)r * DI + c0 + c] = *reinterpret_cast<uint16_t*>(&b);
  }
}

// ------------------------------------------------------------------------------------------------ gated delta net
// Gated DeltaNet linear attention (reference crates/cuda/csrc/gdn.cu:1-25: 16 key heads x 128, 32/48/64 value heads x 128, conv
// width 4 over q | k | v, l2-normalised q and k, q scaled by 1/sqrt(128), decay exp(g) with g = A * softplus(a + dt_bias), A < 0,
// beta = sigmoid(b); delta rule S = S e^g; S += k (x) (beta (v - S^T k)); o = S^T q; per-head RMSNorm(o) * w * silu(z)).
//   proj     f32 [M][ldp]: z (Hv*128) | q (Hk*128) | k (Hk*128) | v (Hv*128) | b (Hv) | a (Hv) | padding
//   S pool   f32 [slots][Hv][64 KB], one head's state S[value j][key i] stored in the order the kernel reads it: thread (j, half) owns
//            i = 64 half + 4 s + e (s = 0..15 load steps, e = 0..3), and the float4 of step s sits at ((warp * 16 + s) * 32 + lane) * 4 with
//            warp = j / 16, lane = 2 (j % 16) + half: every load and store instruction of a warp covers one contiguous 512-byte run
//            (the obvious [j][i] layout made each instruction touch 32 different 128-byte lines; measured in the profile note).
//            conv pool as above with C = (2 Hk + Hv) * 128
// One CTA per (segment, value head), 256 threads: thread = value column j and one half of the 128 keys (64 state values in registers);
// the two halves meet in one shuffle.  The gated norm runs in the same kernel (the CTA holds the head's whole output row).
//
// KDA = true: Kimi delta attention (reference crates/cuda/csrc/kda.cu: per-key-channel decay).  The decay is a vector over the key
// channels, exp(A * softplus(a_i + dt_bias_i)) with a_i taken from 128 columns per head (proj: ... | b (Hv) | a (Hv*128)), and the
// output gate is a sigmoid instead of SiLU.  Everything else is the same code.
constexpr int GDN_D = 128;

// One token of the delta rule for the 64 state values of a thread (value column j, one half of the keys): decay, S.k (both halves meet in one
// shuffle), the rank-one write, S.q.  Four partial sums per dot product keep the dependent chains at 16 instead of 64; both scan kernels call
// this, which is what keeps their states and outputs bit-identical.  sk / sq / sd: this half's 64 keys, queries and (KDA) decays in shared memory,
// 16-byte aligned.  o is returned before the 1 / |q| factor.
template <bool KDA>
__device__ __forceinline__ void gdn_token_update(float (&st)[64], const float* sk, const float* sq, const float* sd, float decay, float v, float beta,
                                                 float kinv, float& kv_out, float& o_out) {
  float k0 = 0.f, k1 = 0.f, k2 = 0.f, k3 = 0.f;
#pragma unroll
  for (int i = 0; i < 64; i += 4) {
    const float4 kk = *reinterpret_cast<const float4*>(sk + i);
    if (KDA) {
      const float4 dd = *reinterpret_cast<const float4*>(sd + i);
      st[i] *= dd.x; st[i + 1] *= dd.y; st[i + 2] *= dd.z; st[i + 3] *= dd.w;
    } else {
      st[i] *= decay; st[i + 1] *= decay; st[i + 2] *= decay; st[i + 3] *= decay;
    }
    k0 += st[i] * kk.x; k1 += st[i + 1] * kk.y; k2 += st[i + 2] * kk.z; k3 += st[i + 3] * kk.w;
  }
  float kv = (k0 + k1) + (k2 + k3);
  kv = (kv + __shfl_xor_sync(0xffffffffu, kv, 1)) * kinv;
  const float delta = (v - kv) * beta * kinv;          // k enters the update normalised as well
  float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
  for (int i = 0; i < 64; i += 4) {
    const float4 kk = *reinterpret_cast<const float4*>(sk + i);
    const float4 qq = *reinterpret_cast<const float4*>(sq + i);
    st[i] += kk.x * delta; st[i + 1] += kk.y * delta; st[i + 2] += kk.z * delta; st[i + 3] += kk.w * delta;
    o0 += st[i] * qq.x; o1 += st[i + 1] * qq.y; o2 += st[i + 2] * qq.z; o3 += st[i + 3] * qq.w;
  }
  float o = (o0 + o1) + (o2 + o3);
  o = o + __shfl_xor_sync(0xffffffffu, o, 1);
  kv_out = kv;
  o_out = o;
}

// Two CTAs per SM (128 registers, a few dozen bytes of spill): a decode step is a chain of dependent loads per CTA, and a second resident
// CTA hides it; measured 54 us -> see the profile note for 16 streams x 48 heads.
template <bool KDA>
__global__ void __launch_bounds__(256, 2) gdn_scan_kernel(const float* __restrict__ xbc, int C, const float* __restrict__ proj, int ldp, int xoff,
                                                      int goff, int M, int Hk, int Hv, const int* __restrict__ row_seq,
                                                      const int* __restrict__ positions, const int* __restrict__ seg_start,
                                                      const int* __restrict__ seg_len, const float* __restrict__ dt_bias,
                                                      const float* __restrict__ a_neg, const uint16_t* __restrict__ norm_w, float eps,
                                                      float* __restrict__ s_pool, float* conv_pool, uint16_t* __restrict__ out, int mode) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float sqk[2 * GDN_D], sdec[KDA ? GDN_D : 4];
  __shared__ float red[8], red2[8];
  int r0, len;
  if (seg_start != nullptr) {
    r0 = seg_start[blockIdx.x];
    len = seg_len[blockIdx.x];
  } else {
    r0 = blockIdx.x;
    if (r0 > 0 && row_seq[r0 - 1] == row_seq[r0]) return;
    len = 1;
    while (r0 + len < M && row_seq[r0 + len] == row_seq[r0]) ++len;
  }
  if (len <= 0) return;
  const int h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, j = tid >> 1, half = tid & 1;
  const int seq = row_seq[r0], hk = h / (Hv / Hk), DI = Hv * GDN_D;
  float st[64];
  float* sp = s_pool + ((size_t)seq * Hv + h) * (GDN_D * GDN_D) + (size_t)warp * (16 * 128) + lane * 4;   // step s adds 128 floats
  if (positions[r0] == 0) {
#pragma unroll
    for (int i = 0; i < 64; ++i) st[i] = 0.f;
  } else {
#pragma unroll
    for (int i = 0; i < 64; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(sp + (i >> 2) * 128);
      st[i] = v.x, st[i + 1] = v.y, st[i + 2] = v.z, st[i + 3] = v.w;
    }
  }
  const float A = a_neg[h], dtb = KDA ? 0.f : dt_bias[h], wj = ssm_bf(norm_w[j]);
  const float* sq = sqk + half * 64;
  const float* sk = sqk + GDN_D + half * 64;
  for (int t = 0; t < len; ++t) {
    const int r = r0 + t;
    const float* xr = xbc + (size_t)r * C;
    __syncthreads();
    const float val = tid < GDN_D ? xr[hk * GDN_D + tid] : xr[(Hk + hk) * GDN_D + (tid - GDN_D)];
    sqk[tid] = val;
    const float ss = warp_sum(val * val);
    if (lane == 0) red[warp] = ss;
    if (KDA && tid < GDN_D) {
      float ai = proj[(size_t)r * ldp + goff + Hv + h * GDN_D + tid] + dt_bias[h * GDN_D + tid];
      ai = ai > 20.f ? ai : log1pf(__expf(ai));
      sdec[tid] = __expf(A * ai);
    }
    __syncthreads();
    const float qinv = rsqrtf(red[0] + red[1] + red[2] + red[3] + 1e-6f) * 0.08838834764831845f;
    const float kinv = rsqrtf(red[4] + red[5] + red[6] + red[7] + 1e-6f);
    const float v = xr[2 * Hk * GDN_D + h * GDN_D + j];
    float decay = 1.f;
    if (!KDA) {
      float a = proj[(size_t)r * ldp + goff + Hv + h] + dtb;
      a = a > 20.f ? a : log1pf(__expf(a));
      decay = __expf(A * a);
    }
    const float beta = 1.f / (1.f + __expf(-proj[(size_t)r * ldp + goff + h]));
    float kv, o;
    gdn_token_update<KDA>(st, sk, sq, sdec + (KDA ? half * 64 : 0), decay, v, beta, kinv, kv, o);
    o *= qinv;
    const float ss2 = warp_sum(half == 0 ? o * o : 0.f);
    if (lane == 0) red2[warp] = ss2;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red2[i];
    if (half == 0 && (mode & SCAN_OUT)) {
      const float z = proj[(size_t)r * ldp + h * GDN_D + j];
      const float gate = KDA ? 1.f / (1.f + __expf(-z)) : ssm_silu(z);
      __nv_bfloat16 b = __float2bfloat16_rn(o * rsqrtf(tot / (float)GDN_D + eps) * wj * gate);
      out[(size_t)r * DI + h * GDN_D + j] = *reinterpret_cast<uint16_t*>(&b);
    }
  }
  if (!(mode & SCAN_STATE)) return;
#pragma unroll
  for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(sp + (i >> 2) * 128) = make_float4(st[i], st[i + 1], st[i + 2], st[i + 3]);
  ssm_conv_commit(proj, ldp, xoff, conv_pool, C, row_seq, positions, r0 + len - 1, seq, h, (int)gridDim.y);
}

// ---- prefill form of the delta-rule scan: a head's 128 value columns are split over GDN_JS CTAs (the columns evolve independently: S_j only
// meets q and k), each ONE warp (no block barrier on the per-token path) with the SAME (column, key half) -> thread mapping and arithmetic as gdn_scan_kernel, so every state value
// and every output is bit-identical to the unsplit kernel's; the per-head gated norm, which needs all 128 outputs, runs afterwards in
// gdn_norm_kernel with the unsplit kernel's reduction order.  The inputs of token t + 1 are fetched while token t is computed: a one-sequence
// prefill was a chain of dependent global loads per token on 48 CTAs; it now runs 192 CTAs with the loads off the critical path.
constexpr int GDN_JS = 8;
template <bool KDA>
__global__ void __launch_bounds__(32) gdn_scan_split_kernel(const float* __restrict__ xbc, int C, const float* __restrict__ proj, int ldp, int xoff,
                                                           int goff, int M, int Hk, int Hv, const int* __restrict__ row_seq,
                                                           const int* __restrict__ positions, const int* __restrict__ seg_start,
                                                           const int* __restrict__ seg_len, const float* __restrict__ dt_bias,
                                                           const float* __restrict__ a_neg, float* __restrict__ s_pool, float* conv_pool,
                                                           float* __restrict__ y32, int mode) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float sqk[2 * GDN_D], sdec[KDA ? GDN_D : 4];
  const int r0 = seg_start[blockIdx.x], len = seg_len[blockIdx.x];
  if (len <= 0) return;
  const int h = blockIdx.y, gw = blockIdx.z, lane = threadIdx.x;      // one warp = one of the head's eight state warps
  const int j = gw * 16 + (lane >> 1), half = lane & 1;
  const int seq = row_seq[r0], hk = h / (Hv / Hk), DI = Hv * GDN_D;
  float st[64];
  float* sp = s_pool + ((size_t)seq * Hv + h) * (GDN_D * GDN_D) + (size_t)gw * (16 * 128) + lane * 4;
  if (positions[r0] == 0) {
#pragma unroll
    for (int i = 0; i < 64; ++i) st[i] = 0.f;
  } else {
#pragma unroll
    for (int i = 0; i < 64; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(sp + (i >> 2) * 128);
      st[i] = v.x, st[i + 1] = v.y, st[i + 2] = v.z, st[i + 3] = v.w;
    }
  }
  const float A = a_neg[h], dtb = KDA ? 0.f : dt_bias[h];
  float kb[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) kb[c] = KDA ? dt_bias[h * GDN_D + 32 * c + lane] : 0.f;
  const float* sq = sqk + half * 64;
  const float* sk = sqk + GDN_D + half * 64;
  // inputs of one token as this lane needs them: q and k values 32 c + lane (c = 0..3), its column's v, the head's gates
  struct In { float q[4], k[4], ka[4], v, a, b; };
  auto fetch = [&](int r) {
    In in;
    const float* xr = xbc + (size_t)r * C;
    const float* pr = proj + (size_t)r * ldp + goff;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      in.q[c] = xr[hk * GDN_D + 32 * c + lane];
      in.k[c] = xr[(Hk + hk) * GDN_D + 32 * c + lane];
      in.ka[c] = KDA ? pr[Hv + h * GDN_D + 32 * c + lane] : 0.f;
    }
    in.v = xr[2 * Hk * GDN_D + h * GDN_D + j];
    in.b = pr[h];
    in.a = KDA ? 0.f : pr[Hv + h];
    return in;
  };
  In ring[SCAN_PF];                                  // inputs of the next SCAN_PF tokens, in flight while the current one is computed
#pragma unroll
  for (int k = 0; k < SCAN_PF; ++k)
    if (k < len) ring[k] = fetch(r0 + k);
  for (int t0 = 0; t0 < len; t0 += SCAN_PF) {
#pragma unroll
  for (int k = 0; k < SCAN_PF; ++k) {
    const int t = t0 + k;
    if (t >= len) break;
    const int r = r0 + t;
    const In cur = ring[k];
    if (t + SCAN_PF < len) ring[k] = fetch(r + SCAN_PF);
    __syncwarp();
    float rq[4], rk[4];                              // the unsplit kernel's eight warp sums: q[32 c .. 32 c + 31], k likewise
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      sqk[32 * c + lane] = cur.q[c];
      sqk[GDN_D + 32 * c + lane] = cur.k[c];
      rq[c] = warp_sum(cur.q[c] * cur.q[c]);
      rk[c] = warp_sum(cur.k[c] * cur.k[c]);
      if (KDA) {
        float a = cur.ka[c] + kb[c];
        a = a > 20.f ? a : log1pf(__expf(a));
        sdec[32 * c + lane] = __expf(A * a);
      }
    }
    __syncwarp();
    const float qinv = rsqrtf(rq[0] + rq[1] + rq[2] + rq[3] + 1e-6f) * 0.08838834764831845f;
    const float kinv = rsqrtf(rk[0] + rk[1] + rk[2] + rk[3] + 1e-6f);
    float decay = 1.f;
    if (!KDA) {
      float a = cur.a + dtb;
      a = a > 20.f ? a : log1pf(__expf(a));
      decay = __expf(A * a);
    }
    const float beta = 1.f / (1.f + __expf(-cur.b));
    float kv, o;
    gdn_token_update<KDA>(st, sk, sq, sdec + (KDA ? half * 64 : 0), decay, cur.v, beta, kinv, kv, o);
    o *= qinv;
    if (half == 0 && (mode & SCAN_OUT)) y32[(size_t)r * DI + h * GDN_D + j] = o;
  }
  }
  if (!(mode & SCAN_STATE)) return;
#pragma unroll
  for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(sp + (i >> 2) * 128) = make_float4(st[i], st[i + 1], st[i + 2], st[i + 3]);
  ssm_conv_commit(proj, ldp, xoff, conv_pool, C, row_seq, positions, r0 + len - 1, seq, h * GDN_JS + gw, (int)(gridDim.y * GDN_JS));
}

// out[r][h][j] = bf16( o * rsqrt(mean_j o^2 + eps) * w[j] * gate(z) ) with the sum of squares taken exactly as gdn_scan_kernel takes it
// (thread = (j, half), per-warp butterfly over the half == 0 lanes, the eight warp sums added in order).  grid (M, Hv), 256 threads.
template <bool KDA>
__global__ void __launch_bounds__(256) gdn_norm_kernel(const float* __restrict__ y32, const float* __restrict__ proj, int ldp, int Hv,
                                                      const uint16_t* __restrict__ norm_w, float eps, uint16_t* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  __shared__ float red2[8];
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, j = tid >> 1, half = tid & 1;
  const int DI = Hv * GDN_D;
  const float o = y32[(size_t)r * DI + h * GDN_D + j];
  const float ss2 = warp_sum(half == 0 ? o * o : 0.f);
  if (lane == 0) red2[warp] = ss2;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red2[i];
  if (half == 0) {
    const float z = proj[(size_t)r * ldp + h * GDN_D + j];
    const float gate = KDA ? 1.f / (1.f + __expf(-z)) : ssm_silu(z);
    __nv_bfloat16 b = __float2bfloat16_rn(o * rsqrtf(tot / (float)GDN_D + eps) * ssm_bf(norm_w[j]) * gate);
    out[(size_t)r * DI + h * GDN_D + j] = *reinterpret_cast<uint16_t*>(&b);
  }
}

}  // namespace rx

// One Mamba2 mixer between its two projections: conv, recurrence (pools updated), gated norm.  seg_start / seg_len (device, nseg
// entries) describe the segments when the host knows them (prefill, commit); pass nullptr and nseg = 0 to have the kernel find them.
// mode: 3 = rows are final (outputs and pools written), 1 = window record (outputs only; keep proj and xbc for the commit),
// 2 = commit (the recurrence over the recorded proj / xbc rows of the given segments, pools written; conv and norm are not launched).
RX_API int rx_ssm_mixer(const void* proj, int ldp, int M, int H, int P, int G, int N, const void* row_seq, const void* positions,
                        const void* seg_start, const void* seg_len, int nseg, const void* conv_w, const void* conv_b, const void* dt_bias,
                        const void* a_neg, const void* d_skip, const void* norm_w, float eps, void* conv_pool, void* ssm_pool, void* xbc,
                        void* y, void* out_bf16, void* stream, int mode) {
  using namespace rx;
  if (mode < 1 || mode > 3) return (int)cudaErrorInvalidValue;
  if (P != SSM_P || N != SSM_N || G <= 0 || H % G || M <= 0) return (int)cudaErrorInvalidValue;
  const int DI = H * P, C = DI + 2 * G * N, xoff = DI, dtoff = DI + C;
  if (ldp < dtoff + H) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  if (mode & SCAN_OUT)
    launch(ssm_conv_kernel, dim3(M, (C + 255) / 256), dim3(256), 0, st, (const float*)proj, ldp, xoff, C, (const int*)row_seq, (const int*)positions,
           (const uint16_t*)conv_w, (const uint16_t*)conv_b, (const float*)conv_pool, (float*)xbc);
  if (seg_start != nullptr)
    launch(ssm_scan_split_kernel, dim3(nseg, H, SSM_PS), dim3(32), 0, st, (const float*)xbc, C, (const float*)proj, ldp, xoff, dtoff, M, H, G,
           (const int*)row_seq, (const int*)positions, (const int*)seg_start, (const int*)seg_len, (const float*)dt_bias, (const float*)a_neg,
           (const float*)d_skip, (float*)ssm_pool, (float*)conv_pool, (float*)y, mode);
  else
  launch(ssm_scan_kernel, dim3(seg_start ? nseg : M, H), dim3(256), 0, st, (const float*)xbc, C, (const float*)proj, ldp, xoff, dtoff, M, H, G,
         (const int*)row_seq, (const int*)positions, (const int*)seg_start, (const int*)seg_len, (const float*)dt_bias, (const float*)a_neg,
         (const float*)d_skip, (float*)ssm_pool, (float*)conv_pool, (float*)y, mode);
  if (mode & SCAN_OUT)
    launch(ssm_gate_norm_kernel, dim3(M, G), dim3(256), 0, st, (const float*)y, (const float*)proj, ldp, DI, G, (const uint16_t*)norm_w, eps,
         (uint16_t*)out_bf16);
  return (int)cudaGetLastError();
}

// One gated-delta-net (kda = 0) or Kimi-delta-attention (kda = 1; dt_bias then has Hv*128 entries) mixer between its two projections:
// conv, then recurrence + gated norm (pools updated).  Two launches; with a host segment table and y32 (f32 [M][Hv*128] scratch) the
// recurrence runs column-split with the norm as a third launch (prefill and commit).
RX_API int rx_gdn_mixer(const void* proj, int ldp, int M, int Hk, int Hv, int D, const void* row_seq, const void* positions, const void* seg_start,
                        const void* seg_len, int nseg, const void* conv_w, const void* conv_b, const void* dt_bias, const void* a_neg,
                        const void* norm_w, float eps, void* conv_pool, void* s_pool, void* xbc, void* out_bf16, void* stream, int kda, int mode,
                        void* y32) {
  using namespace rx;
  if (mode < 1 || mode > 3) return (int)cudaErrorInvalidValue;
  if (D != GDN_D || Hk <= 0 || Hv % Hk || M <= 0) return (int)cudaErrorInvalidValue;
  const int DI = Hv * D, C = (2 * Hk + Hv) * D, xoff = DI, goff = DI + C;
  if (ldp < goff + Hv + (kda ? Hv * D : Hv)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  if (mode & SCAN_OUT)
    launch(ssm_conv_kernel, dim3(M, (C + 255) / 256), dim3(256), 0, st, (const float*)proj, ldp, xoff, C, (const int*)row_seq, (const int*)positions,
           (const uint16_t*)conv_w, (const uint16_t*)conv_b, (const float*)conv_pool, (float*)xbc);
  if (seg_start != nullptr && y32 != nullptr) {
    // segments known on the host (prefill, commit): the column-split scan with prefetched inputs, then the norm (same bits as the fused kernel)
    launch(kda ? gdn_scan_split_kernel<true> : gdn_scan_split_kernel<false>, dim3(nseg, Hv, GDN_JS), dim3(32), 0, st, (const float*)xbc, C,
           (const float*)proj, ldp, xoff, goff, M, Hk, Hv, (const int*)row_seq, (const int*)positions, (const int*)seg_start, (const int*)seg_len,
           (const float*)dt_bias, (const float*)a_neg, (float*)s_pool, (float*)conv_pool, (float*)y32, mode);
    if (mode & SCAN_OUT)
      launch(kda ? gdn_norm_kernel<true> : gdn_norm_kernel<false>, dim3(M, Hv), dim3(256), 0, st, (const float*)y32, (const float*)proj, ldp, Hv,
             (const uint16_t*)norm_w, eps, (uint16_t*)out_bf16);
    return (int)cudaGetLastError();
  }
  launch(kda ? gdn_scan_kernel<true> : gdn_scan_kernel<false>, dim3(seg_start ? nseg : M, Hv), dim3(256), 0, st, (const float*)xbc, C, (const float*)proj, ldp, xoff, goff, M, Hk, Hv,
         (const int*)row_seq, (const int*)positions, (const int*)seg_start, (const int*)seg_len, (const float*)dt_bias, (const float*)a_neg,
         (const uint16_t*)norm_w, eps, (float*)s_pool, (float*)conv_pool, (uint16_t*)out_bf16, mode);
  return (int)cudaGetLastError();
}
