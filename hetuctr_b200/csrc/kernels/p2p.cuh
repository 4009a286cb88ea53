// Device-side pieces of the peer-to-peer exchange that several kernels share: system-scope release/acquire
// accesses, the bounded wait for the peers' sequence numbers, and "the last thread block of a launch publishes".
#pragma once
#include "common.cuh"

namespace hctr {

constexpr int kHdrWords = 16;  // one 64-byte line per (mailbox, source)
constexpr int kMaxRanks = 256;  // owner ids are one byte

__device__ __forceinline__ u32 ld_acquire_sys(const u32 *p) {
  u32 v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(u32 *p, u32 v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ u64 now_ns() {
  u64 t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Polls word `flag` of this rank's own mailbox until it holds `seq`, for at most timeout_ns.  Returns false when
// the time ran out.  *waited_ns = how long the poll took.
__device__ __forceinline__ bool poll_seq(const u32 *flag, u32 seq, u64 timeout_ns, u64 *waited_ns) {
  const u64 t0 = now_ns();
  bool ok = false;
  for (;;) {
    if (ld_acquire_sys(flag) == seq) {
      ok = true;
      break;
    }
    if (now_ns() - t0 > timeout_ns) break;
    __nanosleep(200);
  }
  *waited_ns = now_ns() - t0;
  return ok;
}

// True in exactly one thread block of the launch: the one that arrives last.  Every thread of every block must
// call it after its last store of the launch.  The block barrier orders the block's stores before thread 0's
// system-scope fence and arrival, and the last arriver has therefore observed every other block's arrival (and,
// through their fences, their stores): what it releases afterwards is ordered after all stores of the launch.
// The counter is left at zero for the next launch.
__device__ __forceinline__ bool last_block_of_launch(u32 *ticket) {
  __shared__ bool s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const u32 t = atomicAdd(ticket, 1u);
    s_last = t == gridDim.x - 1;
    if (s_last) {
      *ticket = 0;
      __threadfence_system();
    }
  }
  __syncthreads();
  return s_last;
}

// Phase 0 of a step, receiving side, for a whole thread block (blockDim.x >= nrank): thread s waits (bounded) for
// source s's sequence number and reads the counts it announced; the block then holds, in shared memory, the
// exclusive prefixes of the query counts (qstart, nrank + 1 entries) and of the push counts (gstart).  With
// `publish` the block also stores counts and prefixes to c.cnt_in for later kernels and for the host.
// A silent or over-long source counts as zero rows and sets the error word.
__device__ __forceinline__ void wait_queries(const hctr_p2p_ctx &c, u32 seq, u32 *qstart, u32 *gstart, bool publish) {
  __shared__ u32 s_q[kMaxRanks], s_g[kMaxRanks];
  __shared__ u32 s_wait;
  const int s = threadIdx.x;
  const int n = c.nrank;
  if (s == 0) s_wait = 0;
  __syncthreads();
  if (s < n) {
    const u32 *hdr = c.box[c.rank].hdr + (size_t)s * kHdrWords;
    u64 waited;
    const bool ok = poll_seq(hdr + 0, seq, c.timeout_ns, &waited);
    if (!ok) atomicOr(c.err, HCTR_ERR_TIMEOUT);
    u32 q = ok ? hdr[1] : 0u, g = ok ? hdr[2] : 0u;
    if (q > c.cap || g > c.cap) {
      atomicOr(c.err, HCTR_ERR_CAPACITY);
      q = 0;
      g = 0;
    }
    s_q[s] = q;
    s_g[s] = g;
    atomicMax(&s_wait, (u32)min(waited / 1000, (u64)0xffffffffu));
  }
  __syncthreads();
  if (s == 0) {
    u32 acc = 0, accg = 0;
    for (int i = 0; i < n; i++) {
      qstart[i] = acc;
      gstart[i] = accg;
      acc += s_q[i];
      accg += s_g[i];
    }
    qstart[n] = acc;
    gstart[n] = accg;
  }
  __syncthreads();
  if (publish) {
    if (s < n) {
      c.cnt_in[s] = s_q[s];
      c.cnt_in[n + s] = s_g[s];
    }
    for (int i = s; i <= n; i += blockDim.x) {
      c.cnt_in[3 * n + i] = qstart[i];      // flat index space [0, Q) over all received queries
      c.cnt_in[4 * n + 1 + i] = gstart[i];  // flat index space over all pushed rows
    }
    if (s == 0) {
      c.cnt_in[HCTR_P2P_WAIT0(n)] = s_wait;
      // counters the pull kernels of this step add to
      c.cnt_in[HCTR_P2P_SERVED(n)] = 0;
      c.cnt_in[2 * n] = 0;
    }
  }
}

// Phase 1, receiving side: thread s waits for owner s's return sequence number; ret_base (nrank + 1 entries, shared
// memory) receives the exclusive prefix of the row counts the owners announced.  `publish` stores the counts to
// c.cnt_in, `publish_wait` the longest wait.
__device__ __forceinline__ void wait_returns(const hctr_p2p_ctx &c, u32 seq, u32 *ret_base, bool publish,
                                             bool publish_wait) {
  __shared__ u32 s_r[kMaxRanks];
  __shared__ u32 s_wait;
  const int s = threadIdx.x;
  const int n = c.nrank;
  if (s == 0) s_wait = 0;
  __syncthreads();
  if (s < n) {
    const u32 *hdr = c.box[c.rank].hdr + (size_t)s * kHdrWords;
    u64 waited;
    const bool ok = poll_seq(hdr + 8, seq, c.timeout_ns, &waited);
    if (!ok) atomicOr(c.err, HCTR_ERR_TIMEOUT);
    u32 r = ok ? hdr[9] : 0u;
    if (r > c.cap) {
      atomicOr(c.err, HCTR_ERR_CAPACITY);
      r = 0;
    }
    s_r[s] = r;
    atomicMax(&s_wait, (u32)min(waited / 1000, (u64)0xffffffffu));
  }
  __syncthreads();
  if (s == 0) {
    u32 acc = 0;
    for (int i = 0; i < n; i++) {
      ret_base[i] = acc;
      acc += s_r[i];
    }
    ret_base[n] = acc;
  }
  __syncthreads();
  if (publish && s < n) c.cnt_in[2 * n + s] = s_r[s];
  if (publish_wait && s == 0) c.cnt_in[HCTR_P2P_WAIT1(n)] = s_wait;
}

// Flat index f in [0, start[n]) -> the segment it falls into (start: n + 1 ascending entries).
__device__ __forceinline__ unsigned segment_of(const u32 *start, int n, u32 f) {
  int lo = 0, hi = n;  // start[lo] <= f < start[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (start[mid] <= f) lo = mid;
    else hi = mid;
  }
  return (unsigned)lo;
}

}  // namespace hctr
