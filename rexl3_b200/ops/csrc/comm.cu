// Tensor-parallel collectives fused with the EXL3 finish stages (sm_100a, NVLink peer memory).
//
//   GEMM (row-parallel o_proj / down_proj)  --tiles pushed to the owner by the GEMM epilogue (exl3_gemm_tm.cu)-->
//   finish_rs_kernel    : owner sums the R x S partial planes in (rank, split) order, output Hadamard, svh, bias, residual add on
//                         its d/R columns, and pushes the row's partial sum of squares to every rank            (reduce-scatter end)
//   norm_rot_push_kernel: every rank normalises its columns with the all-rank sum of squares, applies the next layer's
//                         input rotation and pushes the fp16 slice into every rank's gathered activation buffer (all-gather start)
//   GEMM (column-parallel qkv / gate_up / lm_head) waits per source rank for the slices to land and consumes them chunk by chunk.
//
// Each kernel's CTAs wait only for kernels launched EARLIER on the other ranks' streams, so nothing here needs co-scheduling.
// Every wait is bounded (2 s) and reports through the status words.  Semantics matched: the reference's TP arms sum disjoint
// or partial buffers in a fixed rank order (crates/cuda/csrc/tp_oneshot.cu:1-83; nemotron_h_omni/tp_arm.rs:556-584); the
// schedule (push + flags instead of ncclAllReduce) is new.
#include "tp.cuh"

namespace rx {

__device__ __forceinline__ float c_bf16_to_f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t c_f_to_bf16(float f) {
  __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<uint16_t*>(&b);
}

struct FinishTp {
  int ranks, rank;
  const unsigned* in_flag;        // local flags [ranks]: partial tiles of source rank r have landed
  float* ss[TP_MAX];              // per destination rank: sum-of-squares buffer f32 [ranks][rows_cap]
  unsigned* ss_flag[TP_MAX];      // per destination rank: flags [ranks]
  unsigned* local_count;
  const unsigned* epoch;
  unsigned use_index;
  int rows_cap;
};

struct PushTp {
  int ranks, rank;
  const float* ss;                // local sum-of-squares buffer f32 [ranks][rows_cap]
  const unsigned* ss_flag;        // local flags [ranks]
  __half* xr[TP_MAX];             // per destination rank: gathered activation buffer fp16 [rows][d]
  unsigned* xr_flag[TP_MAX];      // per destination rank: flags [ranks]
  unsigned* local_count;
  const unsigned* epoch;
  unsigned use_index;
  int rows_cap;
};

__global__ void tp_bump_epoch_kernel(unsigned* epoch) {
  pdl_launch();
  pdl_wait();
  *epoch += 1;
}

// part: f32 [ranks][S][M][n_own].  h: bf16 [M][d], this rank owns columns [col0, col0 + n_own).
__global__ void __launch_bounds__(1024) finish_rs_kernel(const float* __restrict__ part, int S, int M, int n_own, int d, int col0,
                                                         const __half* __restrict__ svh_own, const float* __restrict__ bias_own,
                                                         uint16_t* __restrict__ h, int* status, const __grid_constant__ FinishTp tp) {
  pdl_launch();
  pdl_wait();
  __shared__ float blk_ss[64];
  __shared__ int ok_sh;
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const unsigned ticket = tp_ticket(tp.epoch, tp.use_index);
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < tp.ranks && ok; ++r) ok = tp_wait_flag(tp.in_flag + r, ticket, status, 160) ? 1 : 0;
    ok_sh = ok;
  }
  __syncthreads();
  if (!ok_sh) return;
  const size_t plane = (size_t)M * n_own;   // the GEMM epilogue laid the planes out for exactly M rows
  for (int b = warp; b < n_own / 128; b += nw) {
    const int n0 = b * 128 + lane * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const int total = tp.ranks * S;      // planes in (rank, split) order: the reduction order is fixed by the layout
    for (int s0 = 0; s0 < total; s0 += 8) {
      float4 p[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < total) p[j] = *reinterpret_cast<const float4*>(part + (size_t)(s0 + j) * plane + (size_t)row * n_own + n0);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < total) {
          if (s0 + j == 0) acc = p[j];
          else { acc.x += p[j].x; acc.y += p[j].y; acc.z += p[j].z; acc.w += p[j].w; }
        }
    }
    float y[4] = {acc.x, acc.y, acc.z, acc.w};
    fwht128_warp(y);
    const uint2 su = *reinterpret_cast<const uint2*>(svh_own + n0);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), c = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
    y[0] *= a.x; y[1] *= a.y; y[2] *= c.x; y[3] *= c.y;
    if (bias_own != nullptr) {
      const float4 bb = *reinterpret_cast<const float4*>(bias_own + n0);
      y[0] += bb.x; y[1] += bb.y; y[2] += bb.z; y[3] += bb.w;
    }
    uint16_t* hp = h + (size_t)row * d + col0 + n0;
    const uint2 hu = *reinterpret_cast<const uint2*>(hp);
    float r[4] = {__uint_as_float(hu.x << 16), __uint_as_float(hu.x & 0xFFFF0000u), __uint_as_float(hu.y << 16), __uint_as_float(hu.y & 0xFFFF0000u)};
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      r[i] = c_bf16_to_f(c_f_to_bf16(r[i] + y[i]));
      ss += r[i] * r[i];
    }
    uint2 o;
    o.x = (uint32_t)c_f_to_bf16(r[0]) | ((uint32_t)c_f_to_bf16(r[1]) << 16);
    o.y = (uint32_t)c_f_to_bf16(r[2]) | ((uint32_t)c_f_to_bf16(r[3]) << 16);
    *reinterpret_cast<uint2*>(hp) = o;
    ss = warp_sum(ss);
    if (lane == 0) blk_ss[b] = ss;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int b = 0; b < n_own / 128; ++b) tot += blk_ss[b];
    for (int r = 0; r < tp.ranks; ++r) tp.ss[r][(size_t)tp.rank * tp.rows_cap + row] = tot;     // push to every rank (self included)
    tp_publish_last(tp.local_count, gridDim.x, tp.ss_flag, tp.ranks, tp.rank, ticket);
  }
}

// h: bf16 [M][d]; this rank normalises and rotates its columns [col0, col0 + n_own) and pushes them into every rank's xr [M][d].
// norm_w, suh_next: full-width vectors (the next layer's input rotation spans the whole hidden size).
__global__ void __launch_bounds__(1024) norm_rot_push_kernel(const uint16_t* __restrict__ h, int M, int n_own, int d, int col0,
                                                             const uint16_t* __restrict__ norm_w, float eps, const __half* __restrict__ suh_next,
                                                             int* status, const __grid_constant__ PushTp tp) {
  pdl_launch();
  pdl_wait();
  __shared__ float rinv_sh;
  __shared__ int ok_sh;
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const unsigned ticket = tp_ticket(tp.epoch, tp.use_index);
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < tp.ranks && ok; ++r) ok = tp_wait_flag(tp.ss_flag + r, ticket, status, 170) ? 1 : 0;
    float tot = 0.f;
    if (ok)
      for (int r = 0; r < tp.ranks; ++r) tot += __ldcg(tp.ss + (size_t)r * tp.rows_cap + row);   // rank order
    rinv_sh = rsqrtf(tot / (float)d + eps);
    ok_sh = ok;
  }
  __syncthreads();
  if (!ok_sh) return;
  const float rinv = norm_w != nullptr ? rinv_sh : 1.f;
  for (int b = warp; b < n_own / 128; b += nw) {
    const int c = col0 + b * 128 + lane * 4;
    const uint2 hu = *reinterpret_cast<const uint2*>(h + (size_t)row * d + c);
    float v[4] = {__uint_as_float(hu.x << 16), __uint_as_float(hu.x & 0xFFFF0000u), __uint_as_float(hu.y << 16), __uint_as_float(hu.y & 0xFFFF0000u)};
    if (norm_w != nullptr) {
      const uint2 wu = *reinterpret_cast<const uint2*>(norm_w + c);
      const float w[4] = {__uint_as_float(wu.x << 16), __uint_as_float(wu.x & 0xFFFF0000u), __uint_as_float(wu.y << 16), __uint_as_float(wu.y & 0xFFFF0000u)};
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = c_bf16_to_f(c_f_to_bf16(v[i] * rinv)) * w[i];
    }
    const uint2 su = *reinterpret_cast<const uint2*>(suh_next + c);
    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
    v[0] *= s01.x; v[1] *= s01.y; v[2] *= s23.x; v[3] *= s23.y;
    fwht128_warp(v);
    const __half2 a = __floats2half2_rn(v[0], v[1]), bb = __floats2half2_rn(v[2], v[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&bb);
    for (int r = 0; r < tp.ranks; ++r) *reinterpret_cast<uint2*>(tp.xr[r] + (size_t)row * d + c) = o;   // all-gather by push
  }
  __syncthreads();
  if (threadIdx.x == 0) tp_publish_last(tp.local_count, gridDim.x, tp.xr_flag, tp.ranks, tp.rank, ticket);
}

// Blocks the stream until every flag in flags[0..ranks) has reached the ticket (for host-launched library ops, e.g. a row
// gather, that read a buffer peers push into).
__global__ void tp_wait_flags_kernel(const unsigned* flags, int ranks, const unsigned* epoch, unsigned use_index, int* status) {
  pdl_launch();
  pdl_wait();
  const unsigned ticket = tp_ticket(epoch, use_index);
  for (int r = 0; r < ranks; ++r)
    if (!tp_wait_flag(flags + r, ticket, status, 180)) return;
}


// ---- one-shot all-reduce for decode windows (rows <= 256): latency matters more than bytes, so every rank finishes its OWN
// partial product (split sum, output Hadamard, svh - all linear, so they commute with the sum over ranks) and pushes the
// f32 row to every rank; one kernel later each rank adds the R rows in rank order, the residual, and goes on to the norm
// and the next rotation for the whole hidden size.  One NVLink hop per projection instead of three; the residual stream is
// replicated.  Bias (if any) rides on rank 0's contribution.
struct BcastTp {
  int ranks, rank;
  float* dst[TP_MAX];            // per destination rank: f32 [ranks][rows_cap][N] of this parity
  unsigned* dst_flag[TP_MAX];    // per destination rank: flags [ranks]
  unsigned* local_count;
  const unsigned* epoch;
  unsigned use_index;
  int rows_cap;
};

// 16 bytes of the element-wise f32 sum, over all GPUs of the multicast object, of the values at this offset (reduced in the switch)
__device__ __forceinline__ float4 multimem_sum_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

// `mm_local` (NVLS form, windows above the packet size): when set, the f32 rows go ONLY to this rank's own copy of a buffer that is bound
// to an NVLink multicast object ([rows_cap][N], no source dimension); the consumers read the sum over ranks with multimem.ld_reduce, so
// the R - 1 peer copies of every row never cross NVLink.  The flags still travel as plain peer stores.
__global__ void finish_bcast_kernel(const float* __restrict__ part, int S, int M, int N, const __half* __restrict__ svh,
                                    const float* __restrict__ bias, const __grid_constant__ BcastTp tp, float* __restrict__ mm_local) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const size_t plane = (size_t)M * N;
  const unsigned ticket = tp_ticket(tp.epoch, tp.use_index);
  const bool ll = M <= LL_MAX_ROWS;
  for (int b = blockIdx.y * nw + warp; b < N / 128; b += gridDim.y * nw) {
    const int n0 = b * 128 + lane * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < S; s0 += 8) {
      float4 p[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < S) p[j] = __ldg(reinterpret_cast<const float4*>(part + (size_t)(s0 + j) * plane + (size_t)row * N + n0));
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < S) {
          if (s0 + j == 0) acc = p[j];
          else { acc.x += p[j].x; acc.y += p[j].y; acc.z += p[j].z; acc.w += p[j].w; }
        }
    }
    float y[4] = {acc.x, acc.y, acc.z, acc.w};
    fwht128_warp(y);
    const uint2 su = *reinterpret_cast<const uint2*>(svh + n0);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), c = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
    y[0] *= a.x; y[1] *= a.y; y[2] *= c.x; y[3] *= c.y;
    if (bias != nullptr) {
      const float4 bb = *reinterpret_cast<const float4*>(bias + n0);
      y[0] += bb.x; y[1] += bb.y; y[2] += bb.z; y[3] += bb.w;
    }
    if (ll) {
      // two self-validating packets per lane (8 bytes per value in the slot): no fence, no flag, the consumer polls its own data
      const size_t at = (((size_t)tp.rank * tp.rows_cap + row) * N + n0) / 2;
      for (int r = 0; r < tp.ranks; ++r) {
        uint4* d = reinterpret_cast<uint4*>(tp.dst[r]) + at;
        ll_store(d, y[0], y[1], ticket);
        ll_store(d + 1, y[2], y[3], ticket);
      }
    } else if (mm_local != nullptr) {
      *reinterpret_cast<float4*>(mm_local + (size_t)row * N + n0) = make_float4(y[0], y[1], y[2], y[3]);
    } else {
      const float4 o = make_float4(y[0], y[1], y[2], y[3]);
      const size_t at = ((size_t)tp.rank * tp.rows_cap + row) * N + n0;
      for (int r = 0; r < tp.ranks; ++r) *reinterpret_cast<float4*>(tp.dst[r] + at) = o;
    }
  }
  if (ll) return;
  __syncthreads();
  if (threadIdx.x == 0) tp_publish_last(tp.local_count, gridDim.x * gridDim.y, tp.dst_flag, tp.ranks, tp.rank, ticket);
}

// ar: local f32 [ranks][rows_cap][N] filled by every rank's finish_bcast_kernel.  h[row] += sum_r ar[r][row] (rank order), then
// xr = fp16(H(rmsnorm(h) * w * suh_next)) for the full row - the multi-rank form of the single-GPU residual/norm/rotate kernel.
__global__ void __launch_bounds__(1024) allsum_add_norm_rot_kernel(const float* __restrict__ ar, const unsigned* __restrict__ flags, int ranks,
                                                                   int rows_cap, const unsigned* epoch, unsigned use_index, int M, int N,
                                                                   uint16_t* __restrict__ h, const uint16_t* __restrict__ norm_w, float eps,
                                                                   const __half* __restrict__ suh_next, __half* __restrict__ xr, int* status,
                                                                   uint16_t* __restrict__ xn_out, const float* __restrict__ mc) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float rowbuf[];
  __shared__ float blk_ss[512];
  __shared__ int ok_sh;
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  // flags == nullptr: plain f32 slots filled by an earlier kernel of this stream (one rank).  Otherwise every rank pushed its rows: small
  // windows as self-validating packets that each thread polls itself, larger ones as f32 rows behind one flag per source rank.
  const bool ll = flags != nullptr && M <= LL_MAX_ROWS;
  const unsigned ticket = flags != nullptr ? tp_ticket(epoch, use_index) : 0u;
  if (flags != nullptr && !ll) {
    if (threadIdx.x == 0) {
      int ok = 1;
      for (int r = 0; r < ranks && ok; ++r) ok = tp_wait_flag(flags + r, ticket, status, 202) ? 1 : 0;
      ok_sh = ok;
    }
    __syncthreads();
    if (!ok_sh) return;
  }
  const size_t plane = (size_t)rows_cap * N;
  const bool nvls = mc != nullptr && flags != nullptr && !ll;      // every rank wrote its rows to its own copy; the switch adds them
  for (int b = warp; b < N / 128; b += nw) {
    const int n0 = b * 128 + lane * 4;
    float4 p[TP_MAX];
    if (nvls) p[0] = multimem_sum_f32x4(mc + (size_t)row * N + n0);
#pragma unroll
    for (int r = 0; r < TP_MAX; ++r)
      if (r < ranks && !nvls) {
        if (ll) {
          // both packets of a rank are requested together; ranks one after another (holding all ranks' packets at once costs more
          // registers than a 1024-thread CTA has, and the spills cost more than the overlap gains - measured)
          const uint4* src = reinterpret_cast<const uint4*>(ar) + ((size_t)r * plane + (size_t)row * N + n0) / 2;
          uint4 a = ll_load(src), c = ll_load(src + 1);
          if (a.y != ticket || a.w != ticket) a = ll_wait(src, ticket, status, 200);
          if (c.y != ticket || c.w != ticket) c = ll_wait(src + 1, ticket, status, 201);
          p[r] = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(c.x), __uint_as_float(c.z));
        } else {
          p[r] = __ldcg(reinterpret_cast<const float4*>(ar + (size_t)r * plane + (size_t)row * N + n0));
        }
      }
    float4 acc = p[0];
#pragma unroll
    for (int r = 1; r < TP_MAX; ++r)
      if (r < ranks && !nvls) { acc.x += p[r].x; acc.y += p[r].y; acc.z += p[r].z; acc.w += p[r].w; }
    const float y[4] = {acc.x, acc.y, acc.z, acc.w};
    uint16_t* hp = h + (size_t)row * N + n0;
    const uint2 hu = *reinterpret_cast<const uint2*>(hp);
    float rr[4] = {__uint_as_float(hu.x << 16), __uint_as_float(hu.x & 0xFFFF0000u), __uint_as_float(hu.y << 16), __uint_as_float(hu.y & 0xFFFF0000u)};
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      rr[i] = c_bf16_to_f(c_f_to_bf16(rr[i] + y[i]));
      ss += rr[i] * rr[i];
      rowbuf[n0 + i] = rr[i];
    }
    uint2 o;
    o.x = (uint32_t)c_f_to_bf16(rr[0]) | ((uint32_t)c_f_to_bf16(rr[1]) << 16);
    o.y = (uint32_t)c_f_to_bf16(rr[2]) | ((uint32_t)c_f_to_bf16(rr[3]) << 16);
    *reinterpret_cast<uint2*>(hp) = o;
    ss = warp_sum(ss);
    if (lane == 0) blk_ss[b] = ss;
  }
  if (suh_next == nullptr && xn_out == nullptr) return;
  __syncthreads();
  float rinv = 1.f;
  if (norm_w != nullptr) {
    float tot = 0.f;
    for (int b = 0; b < N / 128; ++b) tot += blk_ss[b];
    rinv = rsqrtf(tot / (float)N + eps);
  }
  for (int b = warp; b < N / 128; b += nw) {
    const int n0 = b * 128 + lane * 4;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = rowbuf[n0 + i];
    if (norm_w != nullptr) {
      const uint2 wu = *reinterpret_cast<const uint2*>(norm_w + n0);
      const float w[4] = {__uint_as_float(wu.x << 16), __uint_as_float(wu.x & 0xFFFF0000u), __uint_as_float(wu.y << 16), __uint_as_float(wu.y & 0xFFFF0000u)};
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = c_bf16_to_f(c_f_to_bf16(v[i] * rinv)) * w[i];
    }
    if (xn_out != nullptr) {       // the normalised row itself (router input, per-expert rotations)
      uint2 o;
      o.x = (uint32_t)c_f_to_bf16(v[0]) | ((uint32_t)c_f_to_bf16(v[1]) << 16);
      o.y = (uint32_t)c_f_to_bf16(v[2]) | ((uint32_t)c_f_to_bf16(v[3]) << 16);
      *reinterpret_cast<uint2*>(xn_out + (size_t)row * N + n0) = o;
    }
    if (suh_next == nullptr) continue;
    const uint2 su = *reinterpret_cast<const uint2*>(suh_next + n0);
    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&su.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
    v[0] *= s01.x; v[1] *= s01.y; v[2] *= s23.x; v[3] *= s23.y;
    fwht128_warp(v);
    const __half2 a = __floats2half2_rn(v[0], v[1]), bb = __floats2half2_rn(v[2], v[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&bb);
    *reinterpret_cast<uint2*>(xr + (size_t)row * N + n0) = o;
  }
}

// ---- candidate gather: every rank pushes its local top-`count` (ids offset to global vocabulary ids) to the leader, which merges the
// R sorted lists into the global top-`count` in (value desc, id asc) order.  Full logits never cross NVLink.
struct CandTp {
  int ranks, rank;
  unsigned* dst_ids;             // leader's buffer u32 [ranks][rows_cap * 64], as mapped into this rank
  float* dst_vals;               // leader's buffer f32 [ranks][rows_cap * 64]
  unsigned* dst_flag;            // leader's flags [ranks]
  const unsigned* epoch;
  unsigned use_index;
  int rows_cap;
  int id_offset;                 // first vocabulary id of this rank's lm_head shard
};

__global__ void __launch_bounds__(1024) cand_push_kernel(const int* __restrict__ ids, const float* __restrict__ vals, int n,
                                                         const __grid_constant__ CandTp tp) {
  pdl_launch();
  pdl_wait();
  const size_t base = (size_t)tp.rank * tp.rows_cap * 64;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    tp.dst_ids[base + i] = (unsigned)(ids[i] + tp.id_offset);
    tp.dst_vals[base + i] = vals[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) st_release_sys(tp.dst_flag + tp.rank, tp_ticket(tp.epoch, tp.use_index));
}

// One CTA per row, one thread per candidate (ranks * count <= 512).  The output slot of a candidate is the number of candidates
// that precede it; ids are distinct, so the order is total.
__global__ void __launch_bounds__(512) cand_merge_kernel(const unsigned* __restrict__ in_ids, const float* __restrict__ in_vals,
                                                         const unsigned* __restrict__ flags, int ranks, int count, int rows_cap,
                                                         const unsigned* epoch, unsigned use_index, int* __restrict__ out_ids,
                                                         float* __restrict__ out_vals, int* status) {
  pdl_launch();
  pdl_wait();
  __shared__ float sv[512];
  __shared__ unsigned si[512];
  __shared__ int ok_sh;
  if (threadIdx.x == 0) {
    const unsigned ticket = tp_ticket(epoch, use_index);
    int ok = 1;
    for (int r = 0; r < ranks && ok; ++r) ok = tp_wait_flag(flags + r, ticket, status, 190) ? 1 : 0;
    ok_sh = ok;
  }
  __syncthreads();
  if (!ok_sh) return;
  const int row = blockIdx.x, n = ranks * count, t = threadIdx.x;
  float v = 0.f;
  unsigned id = 0;
  if (t < n) {
    const size_t at = (size_t)(t / count) * rows_cap * 64 + (size_t)row * count + (t % count);
    v = in_vals[at];
    id = in_ids[at];
    sv[t] = v;
    si[t] = id;
  }
  __syncthreads();
  if (t >= n) return;
  int before = 0;
  for (int j = 0; j < n; ++j) {
    const float w = sv[j];
    before += (w > v || (w == v && si[j] < id)) ? 1 : 0;
  }
  if (before < count) {
    out_ids[(size_t)row * count + before] = (int)id;
    out_vals[(size_t)row * count + before] = v;
  }
}

}  // namespace rx

using namespace rx;

RX_API int rx_tp_wait_flags(const void* flags, int ranks, const void* epoch, unsigned use_index, int* status, void* stream) {
  return (int)rx::launch(tp_wait_flags_kernel, dim3(1), dim3(1), 0, (cudaStream_t)stream, (const unsigned*)flags, ranks, (const unsigned*)epoch,
                         use_index, status);
}

RX_API int rx_tp_desc_sizes(int* gemm, int* finish, int* push) {
  *gemm = (int)sizeof(GemmTp); *finish = (int)sizeof(FinishTp); *push = (int)sizeof(PushTp);
  return 0;
}

RX_API int rx_tp_bump_epoch(void* epoch, void* stream) {
  return (int)rx::launch(tp_bump_epoch_kernel, dim3(1), dim3(1), 0, (cudaStream_t)stream, (unsigned*)epoch);
}

RX_API int rx_tp_finish_rs(const void* part, int S, int M, int n_own, int d, int col0, const void* svh_own, const void* bias_own, void* h,
                           int* status, const void* desc, void* stream) {
  if (desc == nullptr || n_own % 128 || n_own / 128 > 64 || M < 1) return (int)cudaErrorInvalidValue;
  const FinishTp tp = *(const FinishTp*)desc;
  if (tp.ranks < 1 || tp.ranks > TP_MAX || M > tp.rows_cap) return (int)cudaErrorInvalidValue;
  int threads = 32 * (n_own / 128);
  if (threads > 1024) threads = 1024;
  return (int)rx::launch(finish_rs_kernel, dim3(M), dim3(threads), 0, (cudaStream_t)stream, (const float*)part, S, M, n_own, d, col0,
                         (const __half*)svh_own, (const float*)bias_own, (uint16_t*)h, status, tp);
}

RX_API int rx_tp_norm_rot_push(const void* h, int M, int n_own, int d, int col0, const void* norm_w, float eps, const void* suh_next, int* status,
                               const void* desc, void* stream) {
  if (desc == nullptr || n_own % 128 || M < 1) return (int)cudaErrorInvalidValue;
  const PushTp tp = *(const PushTp*)desc;
  if (tp.ranks < 1 || tp.ranks > TP_MAX || M > tp.rows_cap) return (int)cudaErrorInvalidValue;
  int threads = 32 * (n_own / 128);
  if (threads > 1024) threads = 1024;
  return (int)rx::launch(norm_rot_push_kernel, dim3(M), dim3(threads), 0, (cudaStream_t)stream, (const uint16_t*)h, M, n_own, d, col0,
                         (const uint16_t*)norm_w, eps, (const __half*)suh_next, status, tp);
}

RX_API int rx_tp_bcast_desc_size() { return (int)sizeof(BcastTp); }

static int finish_bcast_launch(const void* part, int S, int M, int N, const void* svh, const void* bias, const void* desc, void* stream, void* mm_local);

RX_API int rx_tp_finish_bcast(const void* part, int S, int M, int N, const void* svh, const void* bias, const void* desc, void* stream) {
  return finish_bcast_launch(part, S, M, N, svh, bias, desc, stream, nullptr);
}

// The same with the NVLS destination (this rank's own address of the multicast-bound buffer of this parity; nullptr = peer stores).
RX_API int rx_tp_finish_bcast_mm(const void* part, int S, int M, int N, const void* svh, const void* bias, const void* desc, void* stream,
                                 void* mm_local) {
  return finish_bcast_launch(part, S, M, N, svh, bias, desc, stream, mm_local);
}

static int finish_bcast_launch(const void* part, int S, int M, int N, const void* svh, const void* bias, const void* desc, void* stream, void* mm_local) {
  if (desc == nullptr || N % 128 || M < 1 || S < 1) return (int)cudaErrorInvalidValue;
  const BcastTp tp = *(const BcastTp*)desc;
  if (tp.ranks < 1 || tp.ranks > TP_MAX || M > tp.rows_cap) return (int)cudaErrorInvalidValue;
  // one warp per 128-block.  Small windows (packet mode): a chain of dependent loads and R remote stores per block wants many small CTAs
  // in flight.  Larger windows end with one system-scope fence per CTA, so they keep few, fat CTAs.
  const int blocks = N / 128;
  int gy;
  if (M <= LL_MAX_ROWS) {
    gy = (592 + M - 1) / M;
    if (gy > blocks) gy = blocks;
  } else {
    gy = 1;
    if (M < 64) { gy = (blocks + 3) / 4; if (gy > 32) gy = 32; }
  }
  if (gy < 1) gy = 1;
  int warps = (blocks + gy - 1) / gy;
  if (warps > 8) warps = 8;
  return (int)rx::launch(finish_bcast_kernel, dim3(M, gy), dim3(32 * warps), 0, (cudaStream_t)stream, (const float*)part, S, M, N, (const __half*)svh,
                         (const float*)bias, tp, (float*)mm_local);
}

static int allsum_launch(const void* ar, const void* flags, int ranks, int rows_cap, const void* epoch, unsigned use_index, int M, int N,
                         void* h, const void* norm_w, float eps, const void* suh_next, void* xr, int* status, void* stream, void* xn_out, const void* mc) {
  if (N % 128 || N / 128 > 512 || M < 1 || M > rows_cap || ranks < 1 || ranks > TP_MAX) return (int)cudaErrorInvalidValue;
  int threads = 32 * (N / 128);
  if (threads > 1024) threads = 1024;
  const size_t smem = (size_t)N * sizeof(float);
  static bool attr_set = false;
  if (smem > 48 * 1024 && !attr_set) {
    cudaError_t e = cudaFuncSetAttribute(allsum_add_norm_rot_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  return (int)rx::launch(allsum_add_norm_rot_kernel, dim3(M), dim3(threads), smem, (cudaStream_t)stream, (const float*)ar, (const unsigned*)flags, ranks,
                         rows_cap, (const unsigned*)epoch, use_index, M, N, (uint16_t*)h, (const uint16_t*)norm_w, eps, (const __half*)suh_next,
                         (__half*)xr, status, (uint16_t*)xn_out, (const float*)mc);
}

RX_API int rx_tp_allsum_add_norm_rot(const void* ar, const void* flags, int ranks, int rows_cap, const void* epoch, unsigned use_index, int M, int N,
                                     void* h, const void* norm_w, float eps, const void* suh_next, void* xr, int* status, void* stream, void* xn_out) {
  return allsum_launch(ar, flags, ranks, rows_cap, epoch, use_index, M, N, h, norm_w, eps, suh_next, xr, status, stream, xn_out, nullptr);
}

// The same with `mc`: the NVLink-multicast address of the buffer every rank's finish kernel wrote its rows to (BcastTp::mm_local is that
// rank's own address of it).  Windows above the packet size then take the sum from multimem.ld_reduce instead of R local slots.
RX_API int rx_tp_allsum_add_norm_rot_mm(const void* ar, const void* flags, int ranks, int rows_cap, const void* epoch, unsigned use_index, int M, int N,
                                        void* h, const void* norm_w, float eps, const void* suh_next, void* xr, int* status, void* stream, void* xn_out,
                                        const void* mc) {
  return allsum_launch(ar, flags, ranks, rows_cap, epoch, use_index, M, N, h, norm_w, eps, suh_next, xr, status, stream, xn_out, mc);
}

RX_API int rx_tp_cand_desc_size() { return (int)sizeof(CandTp); }

RX_API int rx_tp_cand_push(const void* ids, const void* vals, int rows, int count, const void* desc, void* stream) {
  if (desc == nullptr || rows < 1 || count < 1 || count > 64) return (int)cudaErrorInvalidValue;
  const CandTp tp = *(const CandTp*)desc;
  if (tp.ranks < 1 || tp.ranks > TP_MAX || rows > tp.rows_cap) return (int)cudaErrorInvalidValue;
  return (int)rx::launch(cand_push_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, (const int*)ids, (const float*)vals, rows * count, tp);
}

RX_API int rx_tp_cand_merge(const void* in_ids, const void* in_vals, const void* flags, int ranks, int rows, int count, int rows_cap,
                            const void* epoch, unsigned use_index, void* out_ids, void* out_vals, int* status, void* stream) {
  if (ranks < 1 || ranks > TP_MAX || rows < 1 || rows > rows_cap || count < 1 || count > 64) return (int)cudaErrorInvalidValue;
  return (int)rx::launch(cand_merge_kernel, dim3(rows), dim3(512), 0, (cudaStream_t)stream, (const unsigned*)in_ids, (const float*)in_vals,
                         (const unsigned*)flags, ranks, count, rows_cap, (const unsigned*)epoch, use_index, (int*)out_ids, (float*)out_vals, status);
}

// ---- device memory owned by the library: an arena that is its own allocation, so that its IPC handle maps exactly it
RX_API int rx_dev_alloc(long long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, (size_t)bytes);
}
RX_API int rx_dev_free(void* p) { return (int)cudaFree(p); }

// ---- CUDA IPC helpers for the symmetric arena (one process per GPU)
RX_API int rx_ipc_get_handle(void* dev_ptr, void* out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, dev_ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(out64, &h, sizeof(h));
  return 0;
}
RX_API int rx_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
RX_API int rx_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

// ------------------------------------------------------------------------------------------------ generic collectives (TpComm)
// The family-neutral collective interface (parallel/tpcomm.py) over the symmetric arena: a rank PUSHES its buffer into slot `rank` of every
// rank's arena with plain peer stores (the last CTA publishes a ticket to every destination), then every rank combines the R slots it holds
// LOCALLY: a sum in rank order (all-reduce: the same bits on every rank), or a plain copy-out (all-gather).  One hop, every wait bounded and on
// a local flag.  Semantics: reference crates/model/src/families/nemotron_h_omni/tp.rs:37-130 (allreduce_sum_f32 in place, the one-shot form)
// and crates/cuda/csrc/tp_oneshot.cu:1-83 (R operands summed in fixed rank order).
namespace rx {

struct CollTp {
  int ranks, rank;
  long long cap;                  // floats per slot
  float* slots[TP_MAX];           // per destination rank: f32 [ranks][cap] of this parity set
  unsigned* flags[TP_MAX];        // per destination rank: [ranks]
  unsigned* local_count;
  const unsigned* epoch;
  unsigned use_index;
};

// grid-stride copy of `count` floats (count % 4 == 0) into slot `rank` of every rank
__global__ void __launch_bounds__(256) tp_coll_push_kernel(const float* __restrict__ src, long long count, const __grid_constant__ CollTp tp) {
  pdl_launch();
  pdl_wait();
  const long long n4 = count / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    for (int r = 0; r < tp.ranks; ++r) reinterpret_cast<float4*>(tp.slots[r] + (size_t)tp.rank * tp.cap)[i] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) tp_publish_last(tp.local_count, gridDim.x, tp.flags, tp.ranks, tp.rank, tp_ticket(tp.epoch, tp.use_index));
}

// mode 0: dst[i] = sum over ranks (rank order) of slot[r][i];  mode 1: dst[r * count + i] = slot[r][i]
__global__ void __launch_bounds__(256) tp_coll_combine_kernel(float* __restrict__ dst, long long count, int mode, int* status, const __grid_constant__ CollTp tp) {
  pdl_launch();
  pdl_wait();
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    bool ok = true;
    const unsigned ticket = tp_ticket(tp.epoch, tp.use_index);
    for (int r = 0; r < tp.ranks && ok; ++r) ok = tp_wait_flag(tp.flags[tp.rank] + r, ticket, status, 190);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const float* mine = tp.slots[tp.rank];
  const long long n4 = count / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    if (mode == 0) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < tp.ranks; ++r) {
        float4 v;      // written by a peer: read around the non-coherent cache
        asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mine + (size_t)r * tp.cap + 4 * i));
        if (r == 0) acc = v;
        else { acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w; }
      }
      reinterpret_cast<float4*>(dst)[i] = acc;
    } else {
      for (int r = 0; r < tp.ranks; ++r) {
        float4 v;
        asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mine + (size_t)r * tp.cap + 4 * i));
        reinterpret_cast<float4*>(dst + (size_t)r * count)[i] = v;
      }
    }
  }
}

}  // namespace rx

RX_API int rx_tp_coll_desc_size() { return (int)sizeof(rx::CollTp); }

RX_API int rx_tp_coll_push(const void* src, long long count, const void* desc, void* stream) {
  if (desc == nullptr || count < 4 || count % 4 != 0) return (int)cudaErrorInvalidValue;
  const rx::CollTp tp = *(const rx::CollTp*)desc;
  if (tp.ranks < 1 || tp.ranks > rx::TP_MAX || count > tp.cap || (((uintptr_t)src) & 15) != 0) return (int)cudaErrorInvalidValue;
  long long blocks = (count / 4 + 255) / 256;
  if (blocks > 592) blocks = 592;
  return (int)rx::launch(rx::tp_coll_push_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const float*)src, count, tp);
}

RX_API int rx_tp_coll_combine(void* dst, long long count, int mode, int* status, const void* desc, void* stream) {
  if (desc == nullptr || count < 4 || count % 4 != 0 || (mode != 0 && mode != 1)) return (int)cudaErrorInvalidValue;
  const rx::CollTp tp = *(const rx::CollTp*)desc;
  if (tp.ranks < 1 || tp.ranks > rx::TP_MAX || count > tp.cap || (((uintptr_t)dst) & 15) != 0) return (int)cudaErrorInvalidValue;
  long long blocks = (count / 4 + 255) / 256;
  if (blocks > 592) blocks = 592;
  return (int)rx::launch(rx::tp_coll_combine_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (float*)dst, count, mode, status, tp);
}
