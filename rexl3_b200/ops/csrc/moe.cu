// Mixture-of-experts glue around the grouped EXL3 GEMM (sm_100a):
//
//   moe_router_kernel       gate logits (f16/bf16 gate matrix, fp32 accumulate) + scoring + exact top-k per row
//                           mode 0: softmax over all experts, top-k, renormalised over the picks   (Qwen-MoE style)
//                           mode 1: sigmoid scores, picks ranked by score + bias, weights = score / sum(picked) * scale (DeepSeek-V3 style)
//   moe_plan_kernel         counting sort of the (row, slot) pairs by expert in (expert, row, slot) order -> positions, per-expert
//                           offsets, the tile table of the grouped GEMM.  Only experts in [e_lo, e_hi) are planned (expert parallelism:
//                           a rank plans its own experts; activations are replicated, so "dispatch" moves no bytes).
//   moe_gather_rot_kernel   xs[pos] = fp16(H(x[row] * suh[expert]))   - the expert's own input rotation
//   moe_swiglu_rot_kernel   finish of the gate|up GEMM per pair: split sum, Hadamard, svh, SwiGLU, the down projection's rotation
//   moe_combine_kernel      finish of the down GEMM per pair and the top-k weighted sum in slot order (+ an optional shared-expert
//                           row) -> f32 row, written to every rank's all-reduce slot (one rank: a local buffer)
//
// Semantics matched: reference crates/cuda/csrc/moe_router.cu:3-13 (sigmoid+bias router), coopmk.cu:66 / fmoe.cu:11-13 (softmax
// top-k), moe_experts.cu:379 and moe_prefill.cu:444 (combine order: slot order, fp32), moe_prefill.cu:6-12 (on-device planning),
// moe_owned.cu:1-25 (owned experts only; the others contribute nothing).  All reductions have a fixed order.
#include "tp.cuh"

namespace rx {

__device__ __forceinline__ float m_bf16_to_f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t m_f_to_bf16(float f) {
  __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<uint16_t*>(&b);
}

// Gate logits as a small tiled product: CTA = (2 experts, 16 rows); warp w takes rows 2w and 2w + 1 against both experts, so the
// work of a 64-row window spreads over hundreds of CTAs instead of one CTA per row.  logits: f32 [M, E].
__global__ void __launch_bounds__(256) moe_router_logits_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate, int M, int d, int E,
                                                                float* __restrict__ logits) {
  pdl_launch();
  pdl_wait();
  const int e0 = blockIdx.x * 2, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = blockIdx.y * 16 + warp * 2;
  if (r0 >= M) return;
  const bool two = r0 + 1 < M;
  const uint16_t* xa = x + (size_t)r0 * d;
  const uint16_t* xb = x + (size_t)(two ? r0 + 1 : r0) * d;
  const uint16_t* ga = gate + (size_t)e0 * d;
  const uint16_t* gb = gate + (size_t)(e0 + 1 < E ? e0 + 1 : e0) * d;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};     // (row a, expert a), (a, b), (b, a), (b, b); each lane walks k in a fixed order
  for (int k = lane * 8; k < d; k += 256) {
    const uint4 va = *reinterpret_cast<const uint4*>(xa + k), vb = *reinterpret_cast<const uint4*>(xb + k);
    const uint4 wa = __ldg(reinterpret_cast<const uint4*>(ga + k)), wb = __ldg(reinterpret_cast<const uint4*>(gb + k));
    const uint32_t xs0[4] = {va.x, va.y, va.z, va.w}, xs1[4] = {vb.x, vb.y, vb.z, vb.w};
    const uint32_t gs0[4] = {wa.x, wa.y, wa.z, wa.w}, gs1[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a0 = __uint_as_float(xs0[i] << 16), a1 = __uint_as_float(xs0[i] & 0xFFFF0000u);
      const float b0 = __uint_as_float(xs1[i] << 16), b1 = __uint_as_float(xs1[i] & 0xFFFF0000u);
      const float g0 = __uint_as_float(gs0[i] << 16), g1 = __uint_as_float(gs0[i] & 0xFFFF0000u);
      const float h0 = __uint_as_float(gs1[i] << 16), h1 = __uint_as_float(gs1[i] & 0xFFFF0000u);
      acc[0] = fmaf(a0, g0, acc[0]); acc[0] = fmaf(a1, g1, acc[0]);
      acc[1] = fmaf(a0, h0, acc[1]); acc[1] = fmaf(a1, h1, acc[1]);
      acc[2] = fmaf(b0, g0, acc[2]); acc[2] = fmaf(b1, g1, acc[2]);
      acc[3] = fmaf(b0, h0, acc[3]); acc[3] = fmaf(b1, h1, acc[3]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = warp_sum(acc[i]);
  if (lane == 0) {
    logits[(size_t)r0 * E + e0] = acc[0];
    if (e0 + 1 < E) logits[(size_t)r0 * E + e0 + 1] = acc[1];
    if (two) {
      logits[(size_t)(r0 + 1) * E + e0] = acc[2];
      if (e0 + 1 < E) logits[(size_t)(r0 + 1) * E + e0 + 1] = acc[3];
    }
  }
}

// x: bf16 [M, d] (normalised hidden rows).  gate: bf16 [E, d].  bias: f32 [E] or nullptr (mode 1).
// `logits_in` (f32 [M, E]) given: the dot products were done by moe_router_logits_kernel and this kernel only scores and picks.
// out_ids: int32 [M, topk], out_w: f32 [M, topk].  One CTA per row; warp w scores experts w, w + nw, ...
__global__ void __launch_bounds__(256) moe_router_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate, const float* __restrict__ bias,
                                                         int M, int d, int E, int topk, int mode, float scale, int* __restrict__ out_ids,
                                                         float* __restrict__ out_w, const float* __restrict__ logits_in, int n_group, int topk_group) {
  pdl_launch();
  pdl_wait();
  __shared__ float score[512];     // selection key
  __shared__ float prob[512];      // weight source
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const uint16_t* xr = x + (size_t)row * d;
  if (logits_in != nullptr) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) prob[e] = logits_in[(size_t)row * E + e];
  } else
  for (int e = warp; e < E; e += nw) {
    const uint16_t* g = gate + (size_t)e * d;
    float acc = 0.f;
    for (int k = lane * 8; k < d; k += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(xr + k), b = __ldg(reinterpret_cast<const uint4*>(g + k));
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), acc);
        acc = fmaf(__uint_as_float(aw[i] & 0xFFFF0000u), __uint_as_float(bw[i] & 0xFFFF0000u), acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) prob[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  // scoring (warp 0; every lane walks experts lane, lane + 32, ... so each reduction has a fixed order)
  if (mode == 0) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, prob[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float p = __expf(prob[e] - mx);
      prob[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) {
      prob[e] /= sum;
      score[e] = prob[e];
    }
  } else {
    for (int e = lane; e < E; e += 32) {
      const float s = 1.f / (1.f + __expf(-prob[e]));
      prob[e] = s;
      score[e] = s + (bias != nullptr ? bias[e] : 0.f);
    }
  }
  __syncwarp();
  if (n_group > 1 && topk_group < n_group) {
    // group-limited routing (DeepSeek-V3 / Bailing: reference crates/cuda/csrc/ling_fmoe.cu:694): a group's score is the sum of its two best
    // selection keys; only the experts of the `topk_group` best groups (ties to the lowest group) stay eligible.  Lane g owns group g.
    const int per = E / n_group;
    float gs = -INFINITY;
    if (lane < n_group) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int e = lane * per; e < (lane + 1) * per; ++e) {
        const float v = score[e];
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) b2 = v;
      }
      gs = per > 1 ? b1 + b2 : b1;
    }
    unsigned keep = 0u;
    for (int j = 0; j < topk_group; ++j) {
      float best = gs;
      int bi = lane < n_group ? lane : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (bi < 0 || bi >= n_group) bi = j;
      keep |= 1u << bi;
      if (lane == bi) gs = -INFINITY;
    }
    for (int e = lane; e < E; e += 32)
      if (!((keep >> (e / per)) & 1u)) score[e] = -INFINITY;
    __syncwarp();
  }
  // exact top-k: k rounds of arg-max, ties to the lowest expert id
  float picked_sum = 0.f;
  for (int j = 0; j < topk; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float s = score[e];
      if (s > best || (s == best && e < bi)) { best = s; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi < 0 || bi >= E) bi = j;   // a row of NaN scores selects nothing: keep the indices in range
    const float p = prob[bi];
    picked_sum += p;
    if (lane == 0) {
      out_ids[(size_t)row * topk + j] = bi;
      out_w[(size_t)row * topk + j] = p;
      score[bi] = -INFINITY;
    }
    __syncwarp();
  }
  // renormalise over the picks (slot order sum, identical on every lane)
  if (lane < topk) out_w[(size_t)row * topk + lane] = out_w[(size_t)row * topk + lane] / picked_sum * scale;
}

// Single CTA.  ids: int32 [pairs].  Outputs: offs int32 [E + 1] (positions of expert e are offs[e] .. offs[e+1]; experts outside
// [e_lo, e_hi) get empty ranges), pos_of_pair int32 [pairs] (-1: not owned), pair_of_pos / expert_of_pos int32 [pairs],
// tile_tab int32 [max_tiles][3], total int32 [1].
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* ids, int pairs, int E, int e_lo, int e_hi, int tile_rows, int max_tiles,
                                                        int* __restrict__ offs, int* __restrict__ pos_of_pair, int* __restrict__ pair_of_pos,
                                                        int* __restrict__ expert_of_pos, int* __restrict__ tile_tab, int* __restrict__ total) {
  pdl_launch();
  pdl_wait();
  __shared__ int cnt[513];
  __shared__ int start[513];
  __shared__ int ids_sh[4096];       // windows: the pair list fits and every scan below reads it as a broadcast
  const int t = threadIdx.x;
  for (int e = t; e <= E; e += blockDim.x) cnt[e] = 0;
  const bool staged = pairs <= 4096;
  if (staged)
    for (int p = t; p < pairs; p += blockDim.x) ids_sh[p] = ids[p];
  __syncthreads();
  if (staged) ids = ids_sh;
  // One warp per expert (warps take experts round robin): the pair list is walked 32 pairs at a time and a ballot says which of them chose
  // the expert, so a pass costs pairs / 32 steps per expert instead of `pairs`.  Ranks inside a ballot follow the lane order = pair order.
  const int lane = t & 31, warp = t >> 5, nw = blockDim.x >> 5;
  for (int e = e_lo + warp; e < e_hi; e += nw) {
    int c = 0;
    for (int p0 = 0; p0 < pairs; p0 += 32) {
      const int p = p0 + lane;
      c += __popc(__ballot_sync(0xffffffffu, p < pairs && ids[p] == e));
    }
    if (lane == 0) cnt[e] = c;
  }
  __syncthreads();
  if (t == 0) {
    int run = 0, tile = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = run;
      offs[e] = run;
      for (int r0 = 0; r0 < cnt[e] && tile < max_tiles; r0 += tile_rows, ++tile) {
        tile_tab[3 * tile] = e;
        tile_tab[3 * tile + 1] = run + r0;
        tile_tab[3 * tile + 2] = min(tile_rows, cnt[e] - r0);
      }
      run += cnt[e];
    }
    offs[E] = run;
    *total = run;
    for (; tile < max_tiles; ++tile) { tile_tab[3 * tile] = 0; tile_tab[3 * tile + 1] = 0; tile_tab[3 * tile + 2] = 0; }
  }
  __syncthreads();
  for (int e = e_lo + warp; e < e_hi; e += nw) {
    int at = start[e];
    for (int p0 = 0; p0 < pairs; p0 += 32) {
      const int p = p0 + lane;
      const bool hit = p < pairs && ids[p] == e;
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int pos = at + __popc(mask & ((1u << lane) - 1u));
        pos_of_pair[p] = pos;
        pair_of_pos[pos] = p;
        expert_of_pos[pos] = e;
      }
      at += __popc(mask);
    }
  }
  for (int p = t; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e < e_lo || e >= e_hi) pos_of_pair[p] = -1;
  }
}

// grid = pairs.  x: bf16 [M, d]; suh: f16 [E, d]; xs: f16 [pairs_cap, d].
__global__ void moe_gather_rot_kernel(const uint16_t* __restrict__ x, const int* __restrict__ ids, const int* __restrict__ pos_of_pair, int topk, int d,
                                      const __half* __restrict__ suh, __half* __restrict__ xs) {
  pdl_launch();
  pdl_wait();
  const int pair = blockIdx.x;
  const int pos = pos_of_pair[pair];
  if (pos < 0) return;
  const int row = pair / topk, e = ids[pair];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int b = warp; b < d / 128; b += nw) {
    const int n0 = b * 128 + lane * 4;
    const uint2 u = *reinterpret_cast<const uint2*>(x + (size_t)row * d + n0);
    float v[4] = {__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xFFFF0000u)};
    if (suh != nullptr) {          // EXL3 experts: the expert's own input rotation; plain formats (MXFP4) take the row as it is
      const uint2 su = *reinterpret_cast<const uint2*>(suh + (size_t)e * d + n0);
      const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
      v[0] *= s01.x; v[1] *= s01.y; v[2] *= s23.x; v[3] *= s23.y;
      fwht128_warp(v);
    }
    const __half2 a = __floats2half2_rn(v[0], v[1]), bb = __floats2half2_rn(v[2], v[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&bb);
    *reinterpret_cast<uint2*>(xs + (size_t)pos * d + n0) = o;
  }
}

// Sum of S split planes of one 128-block, output Hadamard, svh.  part: f32 [S][pairs_cap][N].
__device__ __forceinline__ void moe_finish_block(const float* __restrict__ part, int S, size_t plane, size_t off, const __half* svh_n0, float (&y)[4]) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < S; s0 += 8) {
    float4 p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (s0 + j < S) p[j] = __ldg(reinterpret_cast<const float4*>(part + (size_t)(s0 + j) * plane + off));
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (s0 + j < S) {
        if (s0 + j == 0) acc = p[j];
        else { acc.x += p[j].x; acc.y += p[j].y; acc.z += p[j].z; acc.w += p[j].w; }
      }
  }
  y[0] = acc.x; y[1] = acc.y; y[2] = acc.z; y[3] = acc.w;
  if (svh_n0 == nullptr) return;   // plain formats: no output rotation, no column scale
  fwht128_warp(y);
  const uint2 su = *reinterpret_cast<const uint2*>(svh_n0);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), c = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
  y[0] *= a.x; y[1] *= a.y; y[2] *= c.x; y[3] *= c.y;
}

// grid = (pairs_cap, gy).  part: f32 [S][pairs_cap][2F] (gate | up).  xs2: f16 [pairs_cap, F] = H(silu(gate) * up * suh_down[e]).
__global__ void moe_swiglu_rot_kernel(const float* __restrict__ part, int S, int pairs_cap, int F, const int* __restrict__ expert_of_pos,
                                      const int* __restrict__ total, const __half* __restrict__ svh_gu, const __half* __restrict__ suh_down,
                                      __half* __restrict__ xs2) {
  pdl_launch();
  pdl_wait();
  const int pos = blockIdx.x;
  if (pos >= *total) return;
  const int e = expert_of_pos[pos];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int N = 2 * F;
  const size_t plane = (size_t)pairs_cap * N;
  for (int b = blockIdx.y * nw + warp; b < F / 128; b += gridDim.y * nw) {
    const int n0 = b * 128 + lane * 4;
    float g[4], u[4];
    moe_finish_block(part, S, plane, (size_t)pos * N + n0, svh_gu == nullptr ? nullptr : svh_gu + (size_t)e * N + n0, g);
    moe_finish_block(part, S, plane, (size_t)pos * N + F + n0, svh_gu == nullptr ? nullptr : svh_gu + (size_t)e * N + F + n0, u);
    float s[4] = {1.f, 1.f, 1.f, 1.f};
    if (suh_down != nullptr) {
      const uint2 su = *reinterpret_cast<const uint2*>(suh_down + (size_t)e * F + n0);
      const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
      s[0] = s01.x; s[1] = s01.y; s[2] = s23.x; s[3] = s23.y;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = g[i] / (1.f + __expf(-g[i])) * u[i];
      g[i] = m_bf16_to_f(m_f_to_bf16(a)) * s[i];
    }
    if (suh_down != nullptr) fwht128_warp(g);
    const __half2 a = __floats2half2_rn(g[0], g[1]), bb = __floats2half2_rn(g[2], g[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&bb);
    *reinterpret_cast<uint2*>(xs2 + (size_t)pos * F + n0) = o;
  }
}

// The same finish for experts WITHOUT a gate (the latent-MoE feed-forward of the Mamba2 hybrids: down(relu(up(x))^2), reference
// crates/cuda/csrc/nemotron_moe.cu): part is f32 [S][pairs_cap][F] (the up projection alone), xs2 = H(relu(up)^2 * suh_down[e]).
__global__ void moe_relu2_rot_kernel(const float* __restrict__ part, int S, int pairs_cap, int F, const int* __restrict__ expert_of_pos,
                                     const int* __restrict__ total, const __half* __restrict__ svh_up, const __half* __restrict__ suh_down,
                                     __half* __restrict__ xs2) {
  pdl_launch();
  pdl_wait();
  const int pos = blockIdx.x;
  if (pos >= *total) return;
  const int e = expert_of_pos[pos];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const size_t plane = (size_t)pairs_cap * F;
  for (int b = blockIdx.y * nw + warp; b < F / 128; b += gridDim.y * nw) {
    const int n0 = b * 128 + lane * 4;
    float u[4];
    moe_finish_block(part, S, plane, (size_t)pos * F + n0, svh_up == nullptr ? nullptr : svh_up + (size_t)e * F + n0, u);
    float s[4] = {1.f, 1.f, 1.f, 1.f};
    if (suh_down != nullptr) {
      const uint2 su = *reinterpret_cast<const uint2*>(suh_down + (size_t)e * F + n0);
      const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
      s[0] = s01.x; s[1] = s01.y; s[2] = s23.x; s[3] = s23.y;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float r = fmaxf(u[i], 0.f);
      u[i] = m_bf16_to_f(m_f_to_bf16(r * r)) * s[i];
    }
    if (suh_down != nullptr) fwht128_warp(u);
    const __half2 a = __floats2half2_rn(u[0], u[1]), bb = __floats2half2_rn(u[2], u[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&bb);
    *reinterpret_cast<uint2*>(xs2 + (size_t)pos * F + n0) = o;
  }
}

struct CombineDst {
  int ranks, rank;
  float* dst[TP_MAX];            // f32 [ranks][rows_cap][d] on every rank (one rank: a local buffer)
  unsigned* dst_flag[TP_MAX];    // nullptr on one rank
  unsigned* local_count;
  const unsigned* epoch;
  unsigned use_index;
  int rows_cap;
};

// grid = (M, gy).  part: f32 [S][pairs_cap][d] (down GEMM).  y[row] = sum_slot w[row][slot] * finish(part[pos(row, slot)]) in slot order,
// skipping pairs this rank does not own; + shared[row] (f32 [M, d] or nullptr; only one rank passes it).  The row goes to slot `rank`
// of every rank's all-reduce buffer, then the last CTA publishes the flags.
__global__ void moe_combine_kernel(const float* __restrict__ part, int S, int pairs_cap, int M, int d, int topk, const int* __restrict__ ids,
                                   const float* __restrict__ w, const int* __restrict__ pos_of_pair, const __half* __restrict__ svh_down,
                                   const float* __restrict__ shared, const __grid_constant__ CombineDst tp) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const size_t plane = (size_t)pairs_cap * d;
  for (int b = blockIdx.y * nw + warp; b < d / 128; b += gridDim.y * nw) {
    const int n0 = b * 128 + lane * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < topk; ++j) {
      const int pair = row * topk + j;
      const int pos = pos_of_pair[pair];
      if (pos < 0) continue;     // warp-uniform
      const int e = ids[pair];
      float y[4];
      moe_finish_block(part, S, plane, (size_t)pos * d + n0, svh_down == nullptr ? nullptr : svh_down + (size_t)e * d + n0, y);
      const float wj = w[pair];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(wj, y[i], acc[i]);
    }
    if (shared != nullptr) {
      const float4 sh = *reinterpret_cast<const float4*>(shared + (size_t)row * d + n0);
      acc[0] += sh.x; acc[1] += sh.y; acc[2] += sh.z; acc[3] += sh.w;
    }
    if (tp.dst_flag[0] == nullptr) {       // one rank: a plain f32 slot read by the next kernel of this stream
      *reinterpret_cast<float4*>(tp.dst[0] + ((size_t)tp.rank * tp.rows_cap + row) * d + n0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else if (M <= LL_MAX_ROWS) {         // several ranks, small window: self-validating packets into every rank's slot (see tp.cuh)
      const unsigned ticket = tp_ticket(tp.epoch, tp.use_index);
      const size_t at = (((size_t)tp.rank * tp.rows_cap + row) * d + n0) / 2;
      for (int r = 0; r < tp.ranks; ++r) {
        uint4* dd = reinterpret_cast<uint4*>(tp.dst[r]) + at;
        ll_store(dd, acc[0], acc[1], ticket);
        ll_store(dd + 1, acc[2], acc[3], ticket);
      }
    } else {                               // several ranks, larger window: f32 rows, then one flag per source rank
      const float4 o = make_float4(acc[0], acc[1], acc[2], acc[3]);
      const size_t at = ((size_t)tp.rank * tp.rows_cap + row) * d + n0;
      for (int r = 0; r < tp.ranks; ++r) *reinterpret_cast<float4*>(tp.dst[r] + at) = o;
    }
  }
  if (tp.dst_flag[0] == nullptr || M <= LL_MAX_ROWS) return;
  __syncthreads();
  if (threadIdx.x == 0)
    tp_publish_last(tp.local_count, gridDim.x * gridDim.y, tp.dst_flag, tp.ranks, tp.rank, tp_ticket(tp.epoch, tp.use_index));
}

// ------------------------------------------------------------------------------------------------ token all-to-all (data-parallel rows)
// Expert parallelism when every rank holds DIFFERENT rows (attention ran data-parallel): a (row, slot) pair travels to the rank that owns its
// expert and its result travels back (the reference's dispatch / combine all-to-all over NCCL, BASELINE named path 3).  Over NVLink peer memory:
//   dispatch   every local pair's normalised row (bf16 [d]) is stored into the OWNER's receive region of this source rank at a position taken from
//              a local counter, with (expert, source pair) beside it; the grid's last CTA publishes the per-destination counts and a ticket.
//   recv_ids   the owner waits (bounded) for every source's ticket and lists the expert of every received row (-1 past a source's count); the
//              existing plan / gather-rotate / grouped GEMM / SwiGLU kernels then run over that list as pairs with one slot per "row".
//   return     finish of the down GEMM per received row (split sum, Hadamard, svh) stored as f32 into the HOME rank's return buffer at the
//              source pair's index; last CTA publishes a ticket to every home rank.
//   home       waits (bounded) for every owner's ticket, y[row] = sum_slot w * ret[row * topk + slot] as an fma chain in slot order - the
//              arithmetic of moe_combine_kernel, so the result equals the one-GPU executor's bit for bit - into the f32 slot the residual /
//              norm / rotation kernel reads.
// Positions inside a receive region depend on the order the source's CTAs ran; nothing downstream depends on them (the grouped GEMM is
// row-invariant and the sum is ordered by slot).  Every transfer is a plain peer store, every wait reads a LOCAL flag.
struct A2aDesc {
  int ranks, rank;
  int cap;                        // rows one source may send to one destination
  int d;
  int e_lo[TP_MAX + 1];           // rank r owns experts [e_lo[r], e_lo[r + 1])
  uint16_t* rx_rows[TP_MAX];      // per destination: bf16 [ranks][cap][d]
  int* rx_meta[TP_MAX];           // per destination: int32 [ranks][cap][2] = (expert, source pair)
  int* rx_count[TP_MAX];          // per destination: int32 [ranks]
  unsigned* rx_flag[TP_MAX];      // per destination: [ranks]
  float* ret[TP_MAX];             // per home rank: f32 [pairs_cap][d]
  unsigned* ret_flag[TP_MAX];     // per home rank: [ranks]
  int* send_count;                // local: int32 [ranks], zero between uses
  unsigned* local_count;          // local CTA counters: [0] dispatch, [1] return
  const unsigned* epoch;
  unsigned use_index;
};

// grid = pairs (one CTA per local pair), 128 threads
__global__ void __launch_bounds__(128) moe_a2a_dispatch_kernel(const uint16_t* __restrict__ xn, const int* __restrict__ ids, int pairs, int topk,
                                                              int* status, const __grid_constant__ A2aDesc a) {
  pdl_launch();
  pdl_wait();
  __shared__ int s_pos, s_owner;
  const int pair = blockIdx.x;
  const int e = ids[pair];
  if (threadIdx.x == 0) {
    int o = 0;
    while (o + 1 < a.ranks && e >= a.e_lo[o + 1]) ++o;
    const int pos = atomicAdd(a.send_count + o, 1);
    if (pos >= a.cap) set_status(status, ST_BAD_ARG, 170, pair);     // cannot happen: cap = the most pairs a source has
    s_owner = o;
    s_pos = pos < a.cap ? pos : -1;
  }
  __syncthreads();
  const int o = s_owner, pos = s_pos;
  if (pos >= 0) {
    const uint4* src = reinterpret_cast<const uint4*>(xn + (size_t)(pair / topk) * a.d);
    uint4* dst = reinterpret_cast<uint4*>(a.rx_rows[o] + ((size_t)a.rank * a.cap + pos) * a.d);
    for (int c = threadIdx.x; c < a.d / 8; c += blockDim.x) dst[c] = src[c];
    if (threadIdx.x == 0) {
      int* meta = a.rx_meta[o] + ((size_t)a.rank * a.cap + pos) * 2;
      meta[0] = e;
      meta[1] = pair;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned old = atomicAdd(a.local_count, 1u);
    if (old == gridDim.x - 1) {
      atomicExch(a.local_count, 0u);
      __threadfence_system();
      const unsigned ticket = tp_ticket(a.epoch, a.use_index);
      for (int r = 0; r < a.ranks; ++r) {
        const int n = atomicExch(a.send_count + r, 0);
        a.rx_count[r][a.rank] = n < a.cap ? n : a.cap;
      }
      __threadfence_system();
      for (int r = 0; r < a.ranks; ++r) st_release_sys(a.rx_flag[r] + a.rank, ticket);
    }
  }
}

// grid = ranks, 256 threads: recv_ids[s * cap + i] = expert of the i-th row received from source s, -1 past its count
__global__ void __launch_bounds__(256) moe_a2a_recv_ids_kernel(int* __restrict__ recv_ids, int* status, const __grid_constant__ A2aDesc a) {
  pdl_launch();
  pdl_wait();
  __shared__ int s_n;
  const int s = blockIdx.x;
  if (threadIdx.x == 0) {
    const bool ok = tp_wait_flag(a.rx_flag[a.rank] + s, tp_ticket(a.epoch, a.use_index), status, 171);
    s_n = ok ? (int)ld_acquire_sys(reinterpret_cast<const unsigned*>(a.rx_count[a.rank] + s)) : 0;
  }
  __syncthreads();
  const int n = s_n;
  const int* meta = a.rx_meta[a.rank] + (size_t)s * a.cap * 2;
  for (int i = threadIdx.x; i < a.cap; i += blockDim.x) recv_ids[(size_t)s * a.cap + i] = i < n ? meta[2 * i] : -1;
}

// grid = (positions capacity, gy).  part: f32 [S][pairs_cap][d] (down GEMM over the received rows); pair_of_pos maps a position to the flat receive
// index q = source * cap + i.
__global__ void moe_a2a_return_kernel(const float* __restrict__ part, int S, int pairs_cap, const int* __restrict__ pair_of_pos,
                                      const int* __restrict__ expert_of_pos, const int* __restrict__ total, const __half* __restrict__ svh_down,
                                      const __grid_constant__ A2aDesc a) {
  pdl_launch();
  pdl_wait();
  const int pos = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (pos < *total) {
    const int q = pair_of_pos[pos], e = expert_of_pos[pos];
    const int src = q / a.cap;
    const int src_pair = a.rx_meta[a.rank][(size_t)q * 2 + 1];
    const size_t plane = (size_t)pairs_cap * a.d;
    for (int b = blockIdx.y * nw + warp; b < a.d / 128; b += gridDim.y * nw) {
      const int n0 = b * 128 + lane * 4;
      float y[4];
      moe_finish_block(part, S, plane, (size_t)pos * a.d + n0, svh_down == nullptr ? nullptr : svh_down + (size_t)e * a.d + n0, y);
      *reinterpret_cast<float4*>(a.ret[src] + (size_t)src_pair * a.d + n0) = make_float4(y[0], y[1], y[2], y[3]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) tp_publish_last(a.local_count + 1, gridDim.x * gridDim.y, a.ret_flag, a.ranks, a.rank, tp_ticket(a.epoch, a.use_index));
}

// grid = (M, gy): out f32 [M][d] = sum over slots (in slot order) of w * returned row (+ shared[row])
__global__ void moe_a2a_home_kernel(const float* __restrict__ w, int M, int topk, const float* __restrict__ shared, float* __restrict__ out, int* status,
                                    const __grid_constant__ A2aDesc a) {
  pdl_launch();
  pdl_wait();
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    bool ok = true;
    const unsigned ticket = tp_ticket(a.epoch, a.use_index);
    for (int r = 0; r < a.ranks && ok; ++r) ok = tp_wait_flag(a.ret_flag[a.rank] + r, ticket, status, 172);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* ret = a.ret[a.rank];
  for (int b = blockIdx.y * nw + warp; b < a.d / 128; b += gridDim.y * nw) {
    const int n0 = b * 128 + lane * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < topk; ++j) {
      const int pair = row * topk + j;
      // written by a peer: read around the non-coherent cache
      float4 y;
      asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(y.x), "=f"(y.y), "=f"(y.z), "=f"(y.w) : "l"(ret + (size_t)pair * a.d + n0));
      const float wj = w[pair];
      acc[0] = fmaf(wj, y.x, acc[0]); acc[1] = fmaf(wj, y.y, acc[1]); acc[2] = fmaf(wj, y.z, acc[2]); acc[3] = fmaf(wj, y.w, acc[3]);
    }
    if (shared != nullptr) {
      const float4 sh = *reinterpret_cast<const float4*>(shared + (size_t)row * a.d + n0);
      acc[0] += sh.x; acc[1] += sh.y; acc[2] += sh.z; acc[3] += sh.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)row * a.d + n0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  }
}

}  // namespace rx

using namespace rx;

RX_API int rx_moe_router(const void* x, const void* gate, const void* bias, int M, int d, int E, int topk, int mode, float scale, void* out_ids,
                         void* out_w, void* stream) {
  if (M < 1 || d % 256 != 0 || E < 1 || E > 512 || topk < 1 || topk > 32 || topk > E || (mode != 0 && mode != 1)) return (int)cudaErrorInvalidValue;
  return (int)rx::launch(moe_router_kernel, dim3(M), dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)x, (const uint16_t*)gate, (const float*)bias, M,
                         d, E, topk, mode, scale, (int*)out_ids, (float*)out_w, (const float*)nullptr, 0, 0);
}

// Two-kernel form for windows of many rows: tiled logits, then scoring + top-k per row.  logits: f32 scratch [M, E].
RX_API int rx_moe_router2(const void* x, const void* gate, const void* bias, int M, int d, int E, int topk, int mode, float scale, void* logits,
                          void* out_ids, void* out_w, void* stream) {
  if (M < 1 || d % 256 != 0 || E < 1 || E > 512 || topk < 1 || topk > 32 || topk > E || (mode != 0 && mode != 1) || logits == nullptr)
    return (int)cudaErrorInvalidValue;
  int e = (int)rx::launch(moe_router_logits_kernel, dim3((E + 1) / 2, (M + 15) / 16), dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)x,
                          (const uint16_t*)gate, M, d, E, (float*)logits);
  if (e != 0) return e;
  return (int)rx::launch(moe_router_kernel, dim3(M), dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)x, (const uint16_t*)gate, (const float*)bias, M,
                         d, E, topk, mode, scale, (int*)out_ids, (float*)out_w, (const float*)logits, 0, 0);
}

// Group-limited form: the experts are `n_group` equal groups; a row picks its `topk_group` best groups (a group's score = its two best selection
// keys added) and then its top-k among their experts only.  n_group <= 32, E % n_group == 0.  logits: f32 scratch [M, E].
RX_API int rx_moe_router_grouped(const void* x, const void* gate, const void* bias, int M, int d, int E, int topk, int mode, float scale, int n_group,
                                 int topk_group, void* logits, void* out_ids, void* out_w, void* stream) {
  if (M < 1 || d % 256 != 0 || E < 1 || E > 512 || topk < 1 || topk > 32 || (mode != 0 && mode != 1) || logits == nullptr || n_group < 1 || n_group > 32 ||
      E % n_group != 0 || topk_group < 1 || topk_group > n_group || topk > topk_group * (E / n_group))
    return (int)cudaErrorInvalidValue;
  int e = (int)rx::launch(moe_router_logits_kernel, dim3((E + 1) / 2, (M + 15) / 16), dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)x,
                          (const uint16_t*)gate, M, d, E, (float*)logits);
  if (e != 0) return e;
  return (int)rx::launch(moe_router_kernel, dim3(M), dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)x, (const uint16_t*)gate, (const float*)bias, M,
                         d, E, topk, mode, scale, (int*)out_ids, (float*)out_w, (const float*)logits, n_group, topk_group);
}

RX_API int rx_moe_plan(const void* ids, int pairs, int E, int e_lo, int e_hi, int tile_rows, int max_tiles, void* offs, void* pos_of_pair,
                       void* pair_of_pos, void* expert_of_pos, void* tile_tab, void* total, void* stream) {
  if (pairs < 1 || E < 1 || E > 512 || e_lo < 0 || e_hi > E || e_lo >= e_hi || tile_rows < 16 || max_tiles < 1) return (int)cudaErrorInvalidValue;
  const int threads = 1024;        // 32 warps share the owned experts
  return (int)rx::launch(moe_plan_kernel, dim3(1), dim3(threads), 0, (cudaStream_t)stream, (const int*)ids, pairs, E, e_lo, e_hi, tile_rows, max_tiles,
                         (int*)offs, (int*)pos_of_pair, (int*)pair_of_pos, (int*)expert_of_pos, (int*)tile_tab, (int*)total);
}

RX_API int rx_moe_gather_rot(const void* x, const void* ids, const void* pos_of_pair, int pairs, int topk, int d, const void* suh, void* xs, void* stream) {
  if (pairs < 1 || d % 128 != 0) return (int)cudaErrorInvalidValue;
  int warps = d / 128;
  if (warps > 8) warps = 8;
  return (int)rx::launch(moe_gather_rot_kernel, dim3(pairs), dim3(32 * warps), 0, (cudaStream_t)stream, (const uint16_t*)x, (const int*)ids,
                         (const int*)pos_of_pair, topk, d, (const __half*)suh, (__half*)xs);
}

RX_API int rx_moe_swiglu_rot(const void* part, int S, int pairs_cap, int F, const void* expert_of_pos, const void* total, const void* svh_gu,
                             const void* suh_down, void* xs2, void* stream) {
  if (pairs_cap < 1 || F % 128 != 0 || S < 1) return (int)cudaErrorInvalidValue;
  int warps = F / 128;
  if (warps > 8) warps = 8;
  return (int)rx::launch(moe_swiglu_rot_kernel, dim3(pairs_cap, 1), dim3(32 * warps), 0, (cudaStream_t)stream, (const float*)part, S, pairs_cap, F,
                         (const int*)expert_of_pos, (const int*)total, (const __half*)svh_gu, (const __half*)suh_down, (__half*)xs2);
}

RX_API int rx_moe_relu2_rot(const void* part, int S, int pairs_cap, int F, const void* expert_of_pos, const void* total, const void* svh_up,
                            const void* suh_down, void* xs2, void* stream) {
  if (pairs_cap < 1 || F % 128 != 0 || S < 1) return (int)cudaErrorInvalidValue;
  int warps = F / 128;
  if (warps > 8) warps = 8;
  return (int)rx::launch(moe_relu2_rot_kernel, dim3(pairs_cap, 1), dim3(32 * warps), 0, (cudaStream_t)stream, (const float*)part, S, pairs_cap, F,
                         (const int*)expert_of_pos, (const int*)total, (const __half*)svh_up, (const __half*)suh_down, (__half*)xs2);
}

RX_API int rx_moe_combine_desc_size() { return (int)sizeof(CombineDst); }

RX_API int rx_moe_combine(const void* part, int S, int pairs_cap, int M, int d, int topk, const void* ids, const void* w, const void* pos_of_pair,
                          const void* svh_down, const void* shared, const void* desc, void* stream) {
  if (desc == nullptr || M < 1 || d % 128 != 0 || S < 1) return (int)cudaErrorInvalidValue;
  const CombineDst tp = *(const CombineDst*)desc;
  if (tp.ranks < 1 || tp.ranks > TP_MAX || M > tp.rows_cap) return (int)cudaErrorInvalidValue;
  const int blocks = d / 128;
  int gy;
  if (M <= LL_MAX_ROWS) {              // packet mode: many small CTAs (a chain of dependent loads and R remote stores per block)
    gy = (592 + M - 1) / M;
    if (gy > blocks) gy = blocks;
  } else {                             // one system-scope fence per CTA: few, fat CTAs
    gy = 1;
    if (M < 64) { gy = (blocks + 3) / 4; if (gy > 16) gy = 16; }
  }
  if (gy < 1) gy = 1;
  int warps = (blocks + gy - 1) / gy;
  if (warps > 8) warps = 8;
  return (int)rx::launch(moe_combine_kernel, dim3(M, gy), dim3(32 * warps), 0, (cudaStream_t)stream, (const float*)part, S, pairs_cap, M, d, topk,
                         (const int*)ids, (const float*)w, (const int*)pos_of_pair, (const __half*)svh_down, (const float*)shared, tp);
}

// ---- token all-to-all launchers (desc: host copy of A2aDesc)
RX_API int rx_moe_a2a_desc_size() { return (int)sizeof(A2aDesc); }

RX_API int rx_moe_a2a_dispatch(const void* xn, const void* ids, int pairs, int topk, int* status, const void* desc, void* stream) {
  if (desc == nullptr || pairs < 1 || topk < 1) return (int)cudaErrorInvalidValue;
  const A2aDesc a = *(const A2aDesc*)desc;
  if (a.ranks < 1 || a.ranks > TP_MAX || a.d % 128 != 0 || pairs > a.cap) return (int)cudaErrorInvalidValue;
  return (int)rx::launch(moe_a2a_dispatch_kernel, dim3(pairs), dim3(128), 0, (cudaStream_t)stream, (const uint16_t*)xn, (const int*)ids, pairs, topk, status, a);
}

RX_API int rx_moe_a2a_recv_ids(void* recv_ids, int* status, const void* desc, void* stream) {
  if (desc == nullptr) return (int)cudaErrorInvalidValue;
  const A2aDesc a = *(const A2aDesc*)desc;
  return (int)rx::launch(moe_a2a_recv_ids_kernel, dim3(a.ranks), dim3(256), 0, (cudaStream_t)stream, (int*)recv_ids, status, a);
}

RX_API int rx_moe_a2a_return(const void* part, int S, int pairs_cap, const void* pair_of_pos, const void* expert_of_pos, const void* total,
                             const void* svh_down, const void* desc, void* stream) {
  if (desc == nullptr || S < 1 || pairs_cap < 1) return (int)cudaErrorInvalidValue;
  const A2aDesc a = *(const A2aDesc*)desc;
  const int blocks = a.d / 128;
  int warps = blocks < 8 ? blocks : 8;
  return (int)rx::launch(moe_a2a_return_kernel, dim3(pairs_cap, 1), dim3(32 * warps), 0, (cudaStream_t)stream, (const float*)part, S, pairs_cap,
                         (const int*)pair_of_pos, (const int*)expert_of_pos, (const int*)total, (const __half*)svh_down, a);
}

RX_API int rx_moe_a2a_home(const void* w, int M, int topk, const void* shared, void* out, int* status, const void* desc, void* stream) {
  if (desc == nullptr || M < 1) return (int)cudaErrorInvalidValue;
  const A2aDesc a = *(const A2aDesc*)desc;
  const int blocks = a.d / 128;
  int warps = blocks < 8 ? blocks : 8;
  return (int)rx::launch(moe_a2a_home_kernel, dim3(M, 1), dim3(32 * warps), 0, (cudaStream_t)stream, (const float*)w, M, topk, (const float*)shared, (float*)out,
                         status, a);
}
