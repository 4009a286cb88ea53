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

// Signal and wait in one launch: thread p publishes this rank's counts to peer p, then waits for peer p's.
// Phase 1 derives the per-requester return counts from the scan itself (ret_slot at the segment bounds).
__global__ void p2p_signal_wait(hctr_p2p_ctx c, int phase, u32 seq, const u32 *__restrict__ meta,
                                const u32 *__restrict__ counts, const u32 *__restrict__ ret_slot);

// One thread per source.  Polls this rank's own memory; gives up after timeout_ns.
__device__ __forceinline__ void p2p_wait_body(const hctr_p2p_ctx &c, int phase, u32 seq, int s);

__global__ void p2p_wait(hctr_p2p_ctx c, int phase, u32 seq) {
  p2p_wait_body(c, phase, seq, threadIdx.x);  // launched with exactly nrank threads
}

__device__ __forceinline__ void p2p_wait_body(const hctr_p2p_ctx &c, int phase, u32 seq, int s) {
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
    // exclusive prefix of the query counts: flat index space [0, Q) over all received queries
    __shared__ u32 s_q[1024], s_g[1024];
    s_q[s] = q;
    s_g[s] = g;
    __syncthreads();
    if (s == 0) {
      u32 acc = 0, accg = 0;
      for (int i = 0; i < c.nrank; i++) {
        c.cnt_in[3 * c.nrank + i] = acc;
        c.cnt_in[4 * c.nrank + 1 + i] = accg;
        acc += s_q[i];
        accg += s_g[i];
      }
      c.cnt_in[4 * c.nrank] = acc;
      c.cnt_in[5 * c.nrank + 1] = accg;  // flat index space over all pushed rows
    }
  } else {
    u32 r = ok ? hdr[9] : 0u;
    if (r > c.cap) {
      atomicOr(c.err, HCTR_ERR_CAPACITY);
      r = 0;
    }
    c.cnt_in[2 * c.nrank + s] = r;
  }
}

// Flat index q in [0, Q) over all received queries -> (source s, index j inside s's sub-region).
__device__ __forceinline__ unsigned source_of(const u32 *qstart, int nrank, u32 q) {
  int lo = 0, hi = nrank;  // qstart[lo] <= q < qstart[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (qstart[mid] <= q) lo = mid;
    else hi = mid;
  }
  return (unsigned)lo;
}

__global__ void p2p_signal_wait(hctr_p2p_ctx c, int phase, u32 seq, const u32 *__restrict__ meta,
                                const u32 *__restrict__ counts, const u32 *__restrict__ ret_slot) {
  const int p = threadIdx.x;  // launched with exactly nrank threads
  __threadfence_system();
  u32 *hdr = c.box[p].hdr + (size_t)c.rank * kHdrWords;
  if (phase == 0) {
    const u32 *seg = meta + HCTR_META_SEG;
    hdr[1] = seg[p + 1] - seg[p];
    hdr[2] = counts ? counts[p] : 0u;
    st_release_sys(hdr + 0, seq);
  } else {
    const u32 *qstart = c.cnt_in + 3 * c.nrank;
    hdr[9] = ret_slot[qstart[p + 1]] - ret_slot[qstart[p]];
    st_release_sys(hdr + 8, seq);
  }
  p2p_wait_body(c, phase, seq, p);
}

__global__ void __launch_bounds__(kThreads) p2p_stale_check(hctr_p2p_ctx c, const int32_t *__restrict__ row_of,
                                                            size_t length, size_t n_cached,
                                                            const long long *__restrict__ version,
                                                            long long pull_bound, u32 *__restrict__ flags32) {
  __shared__ u32 qstart[1025];
  for (int i = threadIdx.x; i <= c.nrank; i += kThreads) qstart[i] = c.cnt_in[3 * c.nrank + i];
  __syncthreads();
  const u32 Q = qstart[c.nrank];
  const hctr_p2p_box me = c.box[c.rank];
  for (size_t q = (size_t)blockIdx.x * kThreads + threadIdx.x; q < Q; q += (size_t)gridDim.x * kThreads) {
    const unsigned s = source_of(qstart, c.nrank, (u32)q);
    const u32 j = (u32)q - qstart[s];
    const size_t slot = (size_t)s * c.cap + j;
    const long long k = me.qkey[slot];
    int32_t row = -1;
    if (k >= 0 && (size_t)k < length) row = row_of[k];
    u32 f = 0;
    if (row < 0 || (size_t)row < n_cached) {
      atomicOr(c.err, HCTR_ERR_NOT_OWNER);
    } else {
      const long long lv = me.qver[slot], gv = version[row];
      const bool stale = lv == kInvalidVersion || (long long)((u64)lv + (u64)pull_bound) < gv;
      f = (stale && s != (unsigned)c.rank) ? 1u : 0u;
    }
    c.box[s].flag[(size_t)c.rank * c.cap + j] = (uint8_t)f;
    flags32[q] = f;
  }
}

__global__ void p2p_return_counts(hctr_p2p_ctx c, const u32 *__restrict__ ret_slot, u32 *__restrict__ ret_count) {
  const int s = threadIdx.x;
  if (s < c.nrank) {
    const u32 *qstart = c.cnt_in + 3 * c.nrank;
    ret_count[s] = ret_slot[qstart[s + 1]] - ret_slot[qstart[s]];
  }
}

// ret_q[r] = flat query index of the r-th returned row (inverse of the scan), so that the gather can
// give every returned row its own group of lanes.
__global__ void __launch_bounds__(kThreads) p2p_return_list(hctr_p2p_ctx c, const u32 *__restrict__ flags32,
                                                            const u32 *__restrict__ ret_slot, u32 *__restrict__ ret_q) {
  const u32 Q = c.cnt_in[4 * c.nrank];
  for (size_t q = (size_t)blockIdx.x * kThreads + threadIdx.x; q < Q; q += (size_t)gridDim.x * kThreads)
    if (flags32[q]) ret_q[ret_slot[q]] = (u32)q;
}

// One group of LANES lanes per returned row, rows written straight into the requester's mailbox.  A group takes
// kGatherRows rows per iteration and issues the loads of all of them stage by stage (list entry, key, row number,
// then the rows), so that the chains of dependent accesses of several rows overlap.
constexpr int kGatherRows = 4;

template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) p2p_gather(hctr_p2p_ctx c, const u32 *__restrict__ ret_q,
                                                       const u32 *__restrict__ ret_slot,
                                                       const int32_t *__restrict__ row_of,
                                                       const float *__restrict__ embedding,
                                                       const long long *__restrict__ version) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  __shared__ u32 qstart[1025];
  for (int i = threadIdx.x; i <= c.nrank; i += kThreads) qstart[i] = c.cnt_in[3 * c.nrank + i];
  __syncthreads();
  const u32 Q = qstart[c.nrank];
  const u32 n_ret = ret_slot[Q];
  const unsigned gl = threadIdx.x % LANES;
  const size_t groups = ((size_t)gridDim.x * kThreads) / LANES;
  const size_t E = R::elems(c.width);
  const hctr_p2p_box me = c.box[c.rank];
  for (size_t r0 = (((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES) * kGatherRows; r0 < n_ret;
       r0 += groups * kGatherRows) {
    u32 qq[kGatherRows];
    unsigned src[kGatherRows];
    long long key[kGatherRows];
    int32_t row[kGatherRows];
    size_t dst[kGatherRows];
#pragma unroll
    for (int k = 0; k < kGatherRows; k++) qq[k] = r0 + k < n_ret ? ret_q[r0 + k] : 0u;
#pragma unroll
    for (int k = 0; k < kGatherRows; k++) {
      src[k] = source_of(qstart, c.nrank, qq[k]);
      key[k] = r0 + k < n_ret ? me.qkey[(size_t)src[k] * c.cap + (qq[k] - qstart[src[k]])] : 0;
    }
#pragma unroll
    for (int k = 0; k < kGatherRows; k++) {
      row[k] = r0 + k < n_ret ? row_of[key[k]] : -1;
      dst[k] = (size_t)c.rank * c.cap + ((u32)(r0 + k) - ret_slot[qstart[src[k]]]);
    }
    if (gl == 0) {
#pragma unroll
      for (int k = 0; k < kGatherRows; k++)
        if (row[k] >= 0) c.box[src[k]].rver[dst[k]] = version[row[k]];
    }
    for (size_t e = gl; e < E; e += LANES) {
      T v[kGatherRows];
#pragma unroll
      for (int k = 0; k < kGatherRows; k++)
        if (row[k] >= 0) v[k] = reinterpret_cast<const T *>(embedding)[(size_t)row[k] * E + e];
#pragma unroll
      for (int k = 0; k < kGatherRows; k++)
        if (row[k] >= 0) reinterpret_cast<T *>(c.box[src[k]].rval)[dst[k] * E + e] = v[k];
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

// ---- fused flag + scan kernels ---------------------------------------------------------------------
// A tile of kTileThreads * kTileItems entries per thread block: every thread computes the flags of its
// kTileItems consecutive entries, the block scans them and the tile totals are chained across blocks
// (chained_cta_prefix), so flags, slots and the lists derived from them come out of one launch.
constexpr int kTileThreads = 1024;
constexpr int kTileItems = 4;
constexpr size_t kTile = (size_t)kTileThreads * kTileItems;

// exclusive prefix of `s` over the thread block (kTileThreads threads); *total = sum over the block
__device__ __forceinline__ u32 tile_exclusive_scan(u32 s, u32 *total) {
  __shared__ u32 warp_sums[32];
  __shared__ u32 s_total;
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  u32 incl = s;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const u32 t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= (unsigned)d) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const u32 w = warp_sums[lane];
    u32 wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const u32 t = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= (unsigned)d) wi += t;
    }
    warp_sums[lane] = wi - w;
    if (lane == 31) s_total = wi;
  }
  __syncthreads();
  *total = s_total;
  return incl - s + warp_sums[warp];
}

// Owner: staleness flag of every received query (stored into the requester's mailbox), slot of every
// returned row (ret_slot, Q + 1 entries, entry Q = number of returned rows) and the list of returned
// queries (ret_q[slot] = flat query index) in one launch.  Same decisions as p2p_stale_check.
__global__ void __launch_bounds__(kTileThreads) p2p_stale_scan(hctr_p2p_ctx c, const int32_t *__restrict__ row_of,
                                                               size_t length, size_t n_cached,
                                                               const long long *__restrict__ version,
                                                               long long pull_bound, u32 *__restrict__ ret_slot,
                                                               u32 *__restrict__ ret_q, u64 *agg, u32 epoch) {
  __shared__ u32 qstart[1025];
  for (int i = threadIdx.x; i <= c.nrank; i += kTileThreads) qstart[i] = c.cnt_in[3 * c.nrank + i];
  __syncthreads();
  const u32 Q = qstart[c.nrank];
  const size_t tile_base = (size_t)blockIdx.x * kTile;
  if (tile_base > Q) return;  // the tile that holds entry Q still runs: it writes the total
  const hctr_p2p_box me = c.box[c.rank];
  const size_t base = tile_base + (size_t)threadIdx.x * kTileItems;
  u32 v[kTileItems];
  u32 sum = 0;
#pragma unroll
  for (int k = 0; k < kTileItems; k++) {
    const size_t q = base + k;
    u32 f = 0;
    if (q < Q) {
      const unsigned s = source_of(qstart, c.nrank, (u32)q);
      const u32 j = (u32)q - qstart[s];
      const size_t slot = (size_t)s * c.cap + j;
      const long long key = me.qkey[slot];
      int32_t row = -1;
      if (key >= 0 && (size_t)key < length) row = row_of[key];
      if (row < 0 || (size_t)row < n_cached) {
        atomicOr(c.err, HCTR_ERR_NOT_OWNER);
      } else {
        const long long lv = me.qver[slot], gv = version[row];
        const bool stale = lv == kInvalidVersion || (long long)((u64)lv + (u64)pull_bound) < gv;
        f = (stale && s != (unsigned)c.rank) ? 1u : 0u;
      }
      c.box[s].flag[(size_t)c.rank * c.cap + j] = (uint8_t)f;
    }
    v[k] = f;
    sum += f;
  }
  u32 total;
  u32 ex = tile_exclusive_scan(sum, &total);
  ex += chained_cta_prefix(agg, epoch, blockIdx.x, total, c.err);
#pragma unroll
  for (int k = 0; k < kTileItems; k++) {
    const size_t q = base + k;
    if (q <= Q) ret_slot[q] = ex;
    if (q < Q && v[k]) ret_q[ex] = (u32)q;
    ex += v[k];
  }
}

// Requester: flag of every unique key collected from its mailbox (flags[u], zero for u >= U) and the
// index of the row returned for it (recv_index[u], in rows relative to box[rank].rval / rver) in one launch.
// Rows returned by owner p sit in sub-region p in the order of the flagged keys, so the index is
// p * cap + (flagged keys before u) - (flagged keys of earlier owners); the latter are the per-owner
// returned-row counts the second exchange delivered (cnt_in[2n + p]).
__global__ void __launch_bounds__(kTileThreads) p2p_recv_scan(hctr_p2p_ctx c, const u32 *__restrict__ meta, size_t u_max,
                                                              const uint8_t *__restrict__ uniq_owner,
                                                              uint8_t *__restrict__ flags,
                                                              u32 *__restrict__ recv_index, u64 *agg, u32 epoch) {
  __shared__ u32 owner_base[1025];
  const size_t U = meta[HCTR_META_UNIQUE];
  const u32 *seg = meta + HCTR_META_SEG;
  const size_t tile_base = (size_t)blockIdx.x * kTile;
  const size_t base = tile_base + (size_t)threadIdx.x * kTileItems;
  if (tile_base >= U) {  // nothing to rank here (and nobody waits for this block): clear and leave
#pragma unroll
    for (int k = 0; k < kTileItems; k++)
      if (base + k < u_max) flags[base + k] = 0, recv_index[base + k] = 0;
    return;
  }
  if (threadIdx.x == 0) {
    u32 acc = 0;
    for (int p = 0; p < c.nrank; p++) {
      owner_base[p] = acc;
      acc += c.cnt_in[2 * c.nrank + p];
    }
  }
  __syncthreads();
  const hctr_p2p_box me = c.box[c.rank];
  u32 v[kTileItems];
  unsigned owner[kTileItems];
  u32 sum = 0;
#pragma unroll
  for (int k = 0; k < kTileItems; k++) {
    const size_t u = base + k;
    u32 f = 0;
    owner[k] = 0;
    if (u < U) {
      owner[k] = uniq_owner[u];
      const u32 j = (u32)u - seg[owner[k]];
      if (j < c.cap) f = me.flag[(size_t)owner[k] * c.cap + j] ? 1u : 0u;
    }
    if (u < u_max) flags[u] = (uint8_t)f;
    v[k] = f;
    sum += f;
  }
  u32 total;
  u32 ex = tile_exclusive_scan(sum, &total);
  ex += chained_cta_prefix(agg, epoch, blockIdx.x, total, c.err);
#pragma unroll
  for (int k = 0; k < kTileItems; k++) {
    const size_t u = base + k;
    if (u < u_max) recv_index[u] = u < U ? owner[k] * (u32)c.cap + (ex - owner_base[owner[k]]) : 0u;
    ex += v[k];
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

extern "C" int hctr_p2p_signal_wait(const hctr_p2p_ctx *c, int phase, uint32_t seq, const uint32_t *meta,
                                    const uint32_t *counts, const uint32_t *ret_slot, void *stream) {
  if (c->nrank > 1024) return (int)cudaErrorInvalidValue;
  p2p_signal_wait<<<1, c->nrank, 0, (cudaStream_t)stream>>>(*c, phase, seq, meta, counts, ret_slot);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_wait(const hctr_p2p_ctx *c, int phase, uint32_t seq, void *stream) {
  if (c->nrank > 1024) return (int)cudaErrorInvalidValue;
  p2p_wait<<<1, c->nrank, 0, (cudaStream_t)stream>>>(*c, phase, seq);
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
                               uint32_t *ret_q, const int32_t *row_of, const float *embedding, const int64_t *version,
                               void *stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const size_t slots = (size_t)c->nrank * c->cap;
  p2p_return_list<<<persistent_grid(slots), kThreads, 0, st>>>(*c, flags32, ret_slot, ret_q);
  const bool al = host_aligned16(embedding);
  const size_t width = c->width;
#define CALL(L, V)                                                                                         \
  p2p_gather<L, V><<<(unsigned)((size_t)kSMs * 8), kThreads, 0, st>>>(*c, ret_q, ret_slot, row_of, embedding, \
                                                                      (const long long *)version)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(2);
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

extern "C" size_t hctr_p2p_scan_scratch_words(size_t entries) { return 2 * ((entries + 1 + kTile - 1) / kTile + 1); }

extern "C" int hctr_p2p_stale_scan(const hctr_p2p_ctx *c, const int32_t *row_of, size_t length, size_t n_cached,
                                   const int64_t *version, int64_t pull_bound, uint32_t *ret_slot, uint32_t *ret_q,
                                   uint32_t *scratch, uint32_t epoch, void *stream) {
  if (c->nrank > 1024 || epoch == 0) return (int)cudaErrorInvalidValue;
  const size_t slots = (size_t)c->nrank * c->cap;
  const unsigned grid = (unsigned)((slots + 1 + kTile - 1) / kTile);
  p2p_stale_scan<<<grid, kTileThreads, 0, (cudaStream_t)stream>>>(*c, row_of, length, n_cached,
                                                                  (const long long *)version, pull_bound, ret_slot,
                                                                  ret_q, reinterpret_cast<u64 *>(scratch), epoch);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_gather_listed(const hctr_p2p_ctx *c, const uint32_t *ret_q, const uint32_t *ret_slot,
                                      const int32_t *row_of, const float *embedding, const int64_t *version,
                                      void *stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const bool al = host_aligned16(embedding);
  const size_t width = c->width;
#define CALL(L, V)                                                                                         \
  p2p_gather<L, V><<<(unsigned)((size_t)kSMs * 8), kThreads, 0, st>>>(*c, ret_q, ret_slot, row_of, embedding, \
                                                                      (const long long *)version)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_recv_scan(const hctr_p2p_ctx *c, const uint32_t *meta, size_t u_max, const uint8_t *uniq_owner,
                                  uint8_t *flags, uint32_t *recv_index, uint32_t *scratch, uint32_t epoch,
                                  void *stream) {
  if (c->nrank > 1024 || epoch == 0) return (int)cudaErrorInvalidValue;
  if (u_max == 0) return 0;
  const unsigned grid = (unsigned)((u_max + kTile - 1) / kTile);
  p2p_recv_scan<<<grid, kTileThreads, 0, (cudaStream_t)stream>>>(*c, meta, u_max, uniq_owner, flags, recv_index,
                                                                 reinterpret_cast<u64 *>(scratch), epoch);
  count_launches(1);
  return launch_status();
}
