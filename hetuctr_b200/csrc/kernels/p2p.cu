// Peer-to-peer exchange kernels: queries, pushed rows and returned rows are written straight into the
// destination rank's mailbox (plain stores to peer memory over NVLink); a release-store of a sequence
// number publishes them, a bounded acquire-poll on the receiver's own memory consumes them.
// No multicast, no TMA on peer memory: ordinary ld/st only.
#include "rowops.cuh"

namespace hctr {

constexpr int kThreads = 256;
constexpr long long kInvalidVersion = INT64_MIN;
constexpr int kHdrWords = 16;  // one 64-byte line per (mailbox, source)

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

__global__ void __launch_bounds__(kThreads) p2p_query_send(hctr_p2p_ctx c, const u32 *__restrict__ meta,
                                                           const long long *__restrict__ uniq,
                                                           const uint8_t *__restrict__ uniq_owner,
                                                           const int32_t *__restrict__ uniq_row,
                                                           const long long *__restrict__ version) {
  const size_t U = meta[HCTR_META_UNIQUE];
  const u32 *seg = meta + HCTR_META_SEG;
  for (size_t u = (size_t)blockIdx.x * kThreads + threadIdx.x; u < U; u += (size_t)gridDim.x * kThreads) {
    const unsigned p = uniq_owner[u];
    const u32 j = (u32)u - seg[p];
    if (j >= c.cap) {
      atomicOr(c.err, HCTR_ERR_CAPACITY);
      continue;
    }
    const hctr_p2p_box b = c.box[p];
    const size_t slot = (size_t)c.rank * c.cap + j;
    const int32_t row = uniq_row[u];
    b.qkey[slot] = uniq[u];
    b.qver[slot] = row >= 0 ? version[row] : kInvalidVersion;
  }
}

// One thread per peer.  Runs after the kernels that filled the peers' mailboxes (stream order); the
// system-scope fence + release store make those rows visible before the sequence number.
__global__ void p2p_signal(hctr_p2p_ctx c, int phase, u32 seq, const u32 *__restrict__ meta,
                           const u32 *__restrict__ counts) {
  const int p = threadIdx.x;
  if (p >= c.nrank) return;
  __threadfence_system();
  u32 *hdr = c.box[p].hdr + (size_t)c.rank * kHdrWords;
  if (phase == 0) {
    const u32 *seg = meta + HCTR_META_SEG;
    hdr[1] = seg[p + 1] - seg[p];
    hdr[2] = counts ? counts[p] : 0u;
    st_release_sys(hdr + 0, seq);
  } else {
    hdr[9] = counts[p];
    st_release_sys(hdr + 8, seq);
  }
}

// One thread per source.  Polls this rank's own memory; gives up after timeout_ns.
__global__ void p2p_wait(hctr_p2p_ctx c, int phase, u32 seq) {
  const int s = threadIdx.x;
  if (s >= c.nrank) return;
  const u32 *hdr = c.box[c.rank].hdr + (size_t)s * kHdrWords;
  const u32 *flag = hdr + (phase == 0 ? 0 : 8);
  const u64 t0 = now_ns();
  bool ok = false;
  for (;;) {
    if (ld_acquire_sys(flag) == seq) {
      ok = true;
      break;
    }
    if (now_ns() - t0 > c.timeout_ns) break;
    __nanosleep(200);
  }
  if (!ok) atomicOr(c.err, HCTR_ERR_TIMEOUT);
  if (phase == 0) {
    u32 q = ok ? hdr[1] : 0u, g = ok ? hdr[2] : 0u;
    if (q > c.cap || g > c.cap) {
      atomicOr(c.err, HCTR_ERR_CAPACITY);
      q = 0;
      g = 0;
    }
    c.cnt_in[s] = q;
    c.cnt_in[c.nrank + s] = g;
  } else {
    u32 r = ok ? hdr[9] : 0u;
    if (r > c.cap) {
      atomicOr(c.err, HCTR_ERR_CAPACITY);
      r = 0;
    }
    c.cnt_in[2 * c.nrank + s] = r;
  }
}

__global__ void __launch_bounds__(kThreads) p2p_stale_check(hctr_p2p_ctx c, const int32_t *__restrict__ row_of,
                                                            size_t length, size_t n_cached,
                                                            const long long *__restrict__ version,
                                                            long long pull_bound, u32 *__restrict__ flags32) {
  const size_t total = (size_t)c.nrank * c.cap;
  const hctr_p2p_box me = c.box[c.rank];
  for (size_t q = (size_t)blockIdx.x * kThreads + threadIdx.x; q < total; q += (size_t)gridDim.x * kThreads) {
    const unsigned s = (unsigned)(q / c.cap);
    const u32 j = (u32)(q % c.cap);
    u32 f = 0;
    if (j < c.cnt_in[s]) {
      const long long k = me.qkey[q];
      int32_t row = -1;
      if (k >= 0 && (size_t)k < length) row = row_of[k];
      if (row < 0 || (size_t)row < n_cached) {
        atomicOr(c.err, HCTR_ERR_NOT_OWNER);
      } else {
        const long long lv = me.qver[q], gv = version[row];
        const bool stale = lv == kInvalidVersion || (long long)((u64)lv + (u64)pull_bound) < gv;
        f = (stale && s != (unsigned)c.rank) ? 1u : 0u;
      }
      c.box[s].flag[(size_t)c.rank * c.cap + j] = (uint8_t)f;
    }
    flags32[q] = f;
  }
}

__global__ void p2p_return_counts(hctr_p2p_ctx c, const u32 *__restrict__ ret_slot, u32 *__restrict__ ret_count) {
  const int s = threadIdx.x;
  if (s < c.nrank) ret_count[s] = ret_slot[(size_t)(s + 1) * c.cap] - ret_slot[(size_t)s * c.cap];
}

// A warp scans 32 consecutive slots, then copies the flagged rows one after the other with all lanes.
template <bool VEC>
__global__ void __launch_bounds__(kThreads) p2p_gather(hctr_p2p_ctx c, const u32 *__restrict__ flags32,
                                                       const u32 *__restrict__ ret_slot,
                                                       const int32_t *__restrict__ row_of,
                                                       const float *__restrict__ embedding,
                                                       const long long *__restrict__ version) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  const unsigned lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const size_t n_warps = ((size_t)gridDim.x * kThreads) >> 5;
  const size_t total = (size_t)c.nrank * c.cap;
  const size_t E = R::elems(c.width);
  const hctr_p2p_box me = c.box[c.rank];
  for (size_t q0 = warp * 32; q0 < total; q0 += n_warps * 32) {
    const size_t q = q0 + lane;
    const bool f = q < total && flags32[q] != 0;
    unsigned live = __ballot_sync(0xffffffffu, f);
    while (live) {
      const int src = __ffs(live) - 1;
      live &= live - 1;
      const size_t qq = q0 + src;
      const unsigned s = (unsigned)(qq / c.cap);
      const u32 slot = ret_slot[qq] - ret_slot[(size_t)s * c.cap];
      const int32_t row = row_of[me.qkey[qq]];
      const hctr_p2p_box b = c.box[s];
      const size_t dst = (size_t)c.rank * c.cap + slot;
      if (lane == 0) b.rver[dst] = version[row];
      const T *from = reinterpret_cast<const T *>(embedding) + (size_t)row * E;
      T *to = reinterpret_cast<T *>(b.rval) + dst * E;
      for (size_t e = lane; e < E; e += 32) to[e] = from[e];
    }
  }
}

__global__ void __launch_bounds__(kThreads) p2p_recv_flags(hctr_p2p_ctx c, const u32 *__restrict__ meta, size_t u_max,
                                                           const uint8_t *__restrict__ uniq_owner,
                                                           uint8_t *__restrict__ flags, u32 *__restrict__ flags32) {
  const size_t U = meta[HCTR_META_UNIQUE];
  const u32 *seg = meta + HCTR_META_SEG;
  const hctr_p2p_box me = c.box[c.rank];
  for (size_t u = (size_t)blockIdx.x * kThreads + threadIdx.x; u < u_max; u += (size_t)gridDim.x * kThreads) {
    uint8_t f = 0;
    if (u < U) {
      const unsigned p = uniq_owner[u];
      const u32 j = (u32)u - seg[p];
      if (j < c.cap) f = me.flag[(size_t)p * c.cap + j] ? 1 : 0;
    }
    flags[u] = f;
    flags32[u] = f;
  }
}

__global__ void __launch_bounds__(kThreads) p2p_recv_index(hctr_p2p_ctx c, const u32 *__restrict__ meta, size_t u_max,
                                                           const uint8_t *__restrict__ uniq_owner,
                                                           const u32 *__restrict__ recv_slot,
                                                           u32 *__restrict__ recv_index) {
  const size_t U = meta[HCTR_META_UNIQUE];
  const u32 *seg = meta + HCTR_META_SEG;
  for (size_t u = (size_t)blockIdx.x * kThreads + threadIdx.x; u < u_max; u += (size_t)gridDim.x * kThreads) {
    u32 idx = 0;
    if (u < U) {
      const unsigned p = uniq_owner[u];
      idx = p * c.cap + (recv_slot[u] - recv_slot[seg[p]]);
    }
    recv_index[u] = idx;
  }
}

static unsigned persistent_grid(size_t items) {
  size_t g = (items + kThreads - 1) / kThreads;
  const size_t cap = (size_t)kSMs * 8;
  if (g > cap) g = cap;
  return (unsigned)(g == 0 ? 1 : g);
}

}  // namespace hctr

using namespace hctr;

extern "C" int hctr_p2p_query_send(const hctr_p2p_ctx *c, const uint32_t *meta, size_t u_max, const int64_t *uniq,
                                   const uint8_t *uniq_owner, const int32_t *uniq_row, const int64_t *version,
                                   void *stream) {
  p2p_query_send<<<persistent_grid(u_max), kThreads, 0, (cudaStream_t)stream>>>(
      *c, meta, (const long long *)uniq, uniq_owner, uniq_row, (const long long *)version);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_signal(const hctr_p2p_ctx *c, int phase, uint32_t seq, const uint32_t *meta,
                               const uint32_t *counts, void *stream) {
  if (c->nrank > 1024) return (int)cudaErrorInvalidValue;
  p2p_signal<<<1, 1024, 0, (cudaStream_t)stream>>>(*c, phase, seq, meta, counts);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_wait(const hctr_p2p_ctx *c, int phase, uint32_t seq, void *stream) {
  if (c->nrank > 1024) return (int)cudaErrorInvalidValue;
  p2p_wait<<<1, 1024, 0, (cudaStream_t)stream>>>(*c, phase, seq);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_stale_check(const hctr_p2p_ctx *c, const int32_t *row_of, size_t length, size_t n_cached,
                                    const int64_t *version, int64_t pull_bound, uint32_t *flags32, void *stream) {
  p2p_stale_check<<<persistent_grid((size_t)c->nrank * c->cap), kThreads, 0, (cudaStream_t)stream>>>(
      *c, row_of, length, n_cached, (const long long *)version, pull_bound, flags32);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_return_counts(const hctr_p2p_ctx *c, const uint32_t *ret_slot, uint32_t *ret_count,
                                      void *stream) {
  if (c->nrank > 1024) return (int)cudaErrorInvalidValue;
  p2p_return_counts<<<1, 1024, 0, (cudaStream_t)stream>>>(*c, ret_slot, ret_count);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_gather(const hctr_p2p_ctx *c, const uint32_t *flags32, const uint32_t *ret_slot,
                               const int32_t *row_of, const float *embedding, const int64_t *version, void *stream) {
  const unsigned g = persistent_grid((size_t)c->nrank * c->cap);
  const bool vec = c->width % 4 == 0 && host_aligned16(embedding);
  if (vec)
    p2p_gather<true><<<g, kThreads, 0, (cudaStream_t)stream>>>(*c, flags32, ret_slot, row_of, embedding,
                                                               (const long long *)version);
  else
    p2p_gather<false><<<g, kThreads, 0, (cudaStream_t)stream>>>(*c, flags32, ret_slot, row_of, embedding,
                                                                (const long long *)version);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_recv_flags(const hctr_p2p_ctx *c, const uint32_t *meta, size_t u_max,
                                   const uint8_t *uniq_owner, uint8_t *flags, uint32_t *flags32, void *stream) {
  p2p_recv_flags<<<persistent_grid(u_max), kThreads, 0, (cudaStream_t)stream>>>(*c, meta, u_max, uniq_owner, flags,
                                                                                flags32);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_recv_index(const hctr_p2p_ctx *c, const uint32_t *meta, size_t u_max,
                                   const uint8_t *uniq_owner, const uint32_t *recv_slot, uint32_t *recv_index,
                                   void *stream) {
  p2p_recv_index<<<persistent_grid(u_max), kThreads, 0, (cudaStream_t)stream>>>(*c, meta, u_max, uniq_owner,
                                                                                recv_slot, recv_index);
  count_launches(1);
  return launch_status();
}
