// Shared device helpers for the sm_100a kernels: mbarrier with bounded waits, TMA bulk copies,
// tcgen05 (alloc / mma / commit / ld), UMMA descriptors, error status words.
//
// Every launcher in this library is extern "C", takes raw device pointers and a stream, returns
// 0 or a cudaError_t, never allocates and never synchronises (same ABI idea as the reference's
// crates/cuda/csrc/common.cuh:1-12).
//
// Waits are bounded: a wait that runs out records {code, site} in the status words the caller
// passed and returns false; the kernel then unwinds (frees TMEM, returns) instead of spinning.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define RX_API extern "C" __attribute__((visibility("default")))

namespace rx {

// ---------------------------------------------------------------- status words
// status[0] = first error code (0 = ok), status[1] = site, status[2] = blockIdx.x, status[3] = aux;
// status[4] = wait limit in microseconds set by the host (0 = the 2 s default), status[5] = abort word: the host (or a watchdog) sets it
// non-zero and every bounded wait that polls it gives up with ST_ABORTED (the role of the reference's abort word,
// crates/cuda/csrc/roce_dev.cuh:173-205).  The buffer has 8 words.
enum : int { ST_OK = 0, ST_TIMEOUT = 1, ST_BAD_ARG = 2, ST_PEER_TIMEOUT = 3, ST_ABORTED = 4 };

__device__ __forceinline__ void set_status(int* status, int code, int site, int aux = 0) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = site;
    status[2] = (int)blockIdx.x;
    status[3] = aux;
  }
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

#ifndef RX_WAIT_LIMIT_NS
#define RX_WAIT_LIMIT_NS 2000000000ull  // 2 s: far above any legitimate wait inside one kernel
#endif
// the limit of a wait that reports to `status`: the host's override in status[4] (microseconds), else the default
__device__ __forceinline__ uint64_t wait_limit_ns(const int* status) {
  if (status != nullptr) {
    const int us = *reinterpret_cast<const volatile int*>(status + 4);
    if (us > 0) return (uint64_t)us * 1000ull;
  }
  return RX_WAIT_LIMIT_NS;
}
__device__ __forceinline__ bool host_abort(const int* status) {
  return status != nullptr && *reinterpret_cast<const volatile int*>(status + 5) != 0;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` is a CTA-shared word every role polls, so one role's timeout unwinds all.
// `sleep_ns` > 0: the waiter sleeps that long between polls.  A role that waits most of the time (a producer for its consumers, the
// MMA issuer for the decode warps) then costs a few hundred instructions per kernel instead of a poll loop that competes with the
// working warps for issue slots (measured: polling was one instruction in five of the decode GEMM).  0: poll back to back, for waits
// on the critical path.  The abort word and the clock are read every 16th failed poll.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int site, uint32_t sleep_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  const uint64_t limit = wait_limit_ns(status);
  uint32_t polls = 0;
  while (true) {
    if (sleep_ns != 0) __nanosleep(sleep_ns);
    if (mbar_try_wait(bar, parity)) return true;
    if ((++polls & 15u) == 0) {
      if (*abort_flag != 0) return false;
      if (host_abort(status)) {
        *abort_flag = 1;
        set_status(status, ST_ABORTED, site, (int)parity);
        return false;
      }
      if (globaltimer_ns() - t0 > limit) {
        *abort_flag = 1;
        set_status(status, ST_TIMEOUT, site, (int)parity);
        return false;
      }
    }
  }
}

// Release of a shared-memory stage that this warp READ with ordinary loads (generic proxy) back to a writer of the async proxy (a bulk / tensor
// copy): the proxy fence orders the reads before whatever the arrive lets the copy engine write.  Without it the copy may overtake the reads
// (seen on B200: operand rows that mixed two K chunks).  Every reading lane runs the fence; one lane arrives.
__device__ __forceinline__ void release_read_stage(uint64_t* empty_bar, int lane) {
  fence_proxy_async();
  __syncwarp();
  if (lane == 0) mbar_arrive(empty_bar);
}

// ---------------------------------------------------------------- TMA
// 1-D bulk copy global -> this CTA's shared memory, completion on an mbarrier (no multicast anywhere).
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// 2-D tiled tensor copy global -> shared (tensor map created on the host).
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const void* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst_smem)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// 16-byte shared-memory load by shared-window address (a plain pointer dereference compiles to a generic load here)
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; kind::f16 (fp16/bf16 operands, fp32 accumulate)
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc]: the A operand (M = 128 lanes, K packed two 16-bit values per 32-bit column) is read from TMEM
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 bit, 32 consecutive columns: thread t of the warp writes TMEM lane (base lane + t)
__device__ __forceinline__ void tc_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
      "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// 32 lanes x 32 bit, 16 consecutive columns: thread t of the warp writes TMEM lane (base lane + t)
__device__ __forceinline__ void tc_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// 32 lanes x 32 bit, 16 consecutive columns: thread t of the warp reads TMEM lane (base lane + t)
__device__ __forceinline__ void tc_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Shared-memory matrix descriptor, K-major operand, SWIZZLE_128B (rows of 128 bytes, 8-row groups 1024 B apart).
// Field layout: [0,14) start>>4 | [16,30) LBO>>4 | [32,46) SBO>>4 | [46,48) version=1 | [61,64) layout (2 = 128B swizzle).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;                  // LBO (ignored for swizzled K-major), canonical value 1
  d |= (uint64_t)(1024 >> 4) << 32;        // SBO: 8 rows * 128 B
  d |= (uint64_t)1 << 46;                  // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: fp32 accumulator, A/B formats (0 = f16, 1 = bf16), both K-major.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n, int a_fmt, int b_fmt) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------- programmatic dependent launch
// Every kernel of this library is launched with programmatic stream serialization allowed: a kernel calls pdl_launch() at its
// start (the next kernel in the stream may begin its prologue, e.g. stream its weights) and pdl_wait() before it touches
// anything the previous kernel wrote.  pdl_wait() returns once the previous kernel has fully completed and flushed.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline int& pdl_enabled() { static int on = 1; return on; }

template <typename... P, typename... A>
inline cudaError_t launch(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}

// ---------------------------------------------------------------- small math helpers
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// In-place 128-point Walsh-Hadamard transform of one 128-block held by a warp: lane L owns x[4L..4L+3].
// Result scaled by 1/sqrt(128).  Element index i = 4*lane + r.
__device__ __forceinline__ void fwht128_warp(float (&v)[4]) {
  // strides 1, 2 inside the lane
  float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
  v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float sgn = (lane & o) ? -1.f : 1.f;   // upper half of the butterfly: other - v, lower half: other + v
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float other = __shfl_xor_sync(0xffffffffu, v[r], o);
      v[r] = fmaf(sgn, v[r], other);
    }
  }
  const float s = 0.08838834764831845f;  // 1/sqrt(128)
#pragma unroll
  for (int r = 0; r < 4; ++r) v[r] *= s;
}

}  // namespace rx
