// Tensor-parallel plumbing shared by the fused compute+collective kernels: peer tables, tickets, bounded peer waits and
// the "last CTA publishes" signal.
//
// Every rank owns one symmetric arena (same layout on every GPU, mapped into every peer through CUDA IPC).  Data moves by
// plain vectorised stores into the CONSUMER's arena (push model), so every TMA / tensor-core read is from local memory.
// A producer kernel finishes with: each CTA fences to system scope and bumps a local counter; the CTA that sees the last
// count writes ticket = epoch * 4096 + use_index into flag[src] on every destination.  A consumer spins (bounded, 2 s)
// on its LOCAL flag word until it reaches the ticket.  The epoch lives in device memory and is bumped by a one-thread
// kernel at the start of every forward, so captured CUDA graphs replay with fresh tickets.
// Counterpart in the reference: the flag/sequence protocol of its RDMA transport (crates/cuda/csrc/roce_dev.cuh:118-260);
// NVLink peer stores replace the proxy thread and the RDMA writes.
#pragma once
#include "common.cuh"

namespace rx {

constexpr int TP_MAX = 8;

struct GemmTp {
  int ranks;                    // all-zero struct = single GPU: strips_per_rank == 0 and in_flag == nullptr switch both hooks off
  int rank;
  int strips_per_rank;          // > 0: reduce-scatter epilogue, strip s goes to rank s / strips_per_rank
  int out_ld;                   // leading dimension of the destination buffers (owned columns)
  int rows_cap;                 // rows each [src][split] plane of a destination buffer can hold
  float* out[TP_MAX];           // destination buffers, one per rank: f32 [ranks][splits][rows_cap][out_ld]
  unsigned* out_flag[TP_MAX];   // per destination: flags [ranks] of this site; flag[src] = ticket when src's tiles have landed
  unsigned* local_count;        // this rank's CTA counter for the site
  const unsigned* in_flag;      // local flags [ranks] of the all-gathered input (nullptr: input is local)
  int in_cols_per_src;          // K columns each source rank contributes to the gathered input
  const unsigned* epoch;
  unsigned use_index;
};

__device__ __forceinline__ unsigned tp_ticket(const unsigned* epoch, unsigned use_index) { return *epoch * 4096u + use_index; }

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for a local flag word to reach `ticket` (tickets only grow).  Returns false and records the site on timeout.
__device__ __forceinline__ bool tp_wait_flag(const unsigned* flag, unsigned ticket, int* status, int site) {
  if ((int)(ld_acquire_sys(flag) - ticket) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  const uint64_t limit = wait_limit_ns(status);
  while (true) {
    if ((int)(ld_acquire_sys(flag) - ticket) >= 0) return true;
    if (host_abort(status)) {
      set_status(status, ST_ABORTED, site, (int)ticket);
      return false;
    }
    if (globaltimer_ns() - t0 > limit) {
      set_status(status, ST_PEER_TIMEOUT, site, (int)ticket);
      return false;
    }
    __nanosleep(64);
  }
}

// ---- self-validating 16-byte packets for latency-bound exchanges (two (value, ticket) pairs each; the 8-byte halves are written
// atomically, so a reader that sees the ticket in both halves has the data: no fence, no separate flag, no kernel-level wait).
// The same idea as NCCL's LL protocol; tickets are unique per collective (epoch and use index), so stale slots never match.
// Windows of at most LL_MAX_ROWS rows use the packets (latency-bound: one NVLink hop, no fence); larger windows use plain f32 rows plus one
// flag per source rank (half the bytes; the system-scope fence is then amortised over more data).  Measured on 8 GPUs: packets take a
// batch-1 step from 7.6 to 5.9 ms, but a 64-row step from 15.0 to 19.4 ms, hence the split.  Producer and consumer derive the mode from the
// row count of the window, which both know.
constexpr int LL_MAX_ROWS = 16;

__device__ __forceinline__ void ll_store(uint4* dst, float a, float b, unsigned ticket) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(__float_as_uint(a)), "r"(ticket), "r"(__float_as_uint(b)), "r"(ticket)
               : "memory");
}
__device__ __forceinline__ uint4 ll_load(const uint4* src) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
  return v;
}
// Bounded wait for one packet.  On a timeout the status words are set and whatever is there is returned (the caller's result is then
// garbage, and the host turns the status into a fatal error); nothing hangs.
__device__ __forceinline__ uint4 ll_wait(const uint4* src, unsigned ticket, int* status, int site) {
  uint4 v = ll_load(src);
  if (v.y == ticket && v.w == ticket) return v;
  const uint64_t t0 = globaltimer_ns();
  const uint64_t limit = wait_limit_ns(status);
  for (unsigned it = 0;; ++it) {
    v = ll_load(src);
    if (v.y == ticket && v.w == ticket) return v;
    if ((it & 63u) == 63u) {
      if (host_abort(status)) {
        set_status(status, ST_ABORTED, site, (int)ticket);
        return v;
      }
      if (globaltimer_ns() - t0 > limit) {
        set_status(status, ST_PEER_TIMEOUT, site, (int)ticket);
        return v;
      }
    }
  }
}

// Called by ONE thread of every CTA after the CTA's peer stores are complete and fenced: the last CTA of the grid resets the
// counter and publishes the ticket to flag[src = rank] on every destination rank.
__device__ __forceinline__ void tp_publish_last(unsigned* local_count, unsigned total_ctas, unsigned* const* flags, int ranks, int rank,
                                                unsigned ticket) {
  __threadfence_system();
  const unsigned old = atomicAdd(local_count, 1u);
  if (old == total_ctas - 1) {
    atomicExch(local_count, 0u);
    __threadfence_system();
    for (int r = 0; r < ranks; ++r) st_release_sys(flags[r] + rank, ticket);
  }
}

}  // namespace rx
