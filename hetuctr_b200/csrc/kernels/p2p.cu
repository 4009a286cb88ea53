// Peer-to-peer exchange kernels: queries, pushed rows and returned rows are written straight into the
// destination rank's mailbox (plain stores to peer memory over NVLink); a release-store of a sequence
// number publishes them, a bounded acquire-poll on the receiver's own memory consumes them.
// No multicast, no TMA on peer memory: ordinary ld/st only.
#include "p2p.cuh"
#include "rowops.cuh"

namespace hctr {

constexpr int kThreads = 256;
constexpr long long kInvalidVersion = INT64_MIN;

// Requester: (key, local version) of every unique key goes into its owner's mailbox; the thread block that
// finishes last then publishes this rank's counts (queries per owner from the batch's segment starts, pushed rows
// per owner from `push_counts`, null = none) and releases sequence number `seq` to every peer.  The pushed rows
// themselves were written by the gradient reduction, an earlier kernel.
// (Publishing kernels run at most one thread block per SM: every block ends with a system-scope fence, and an SM
// works through the fences of its resident blocks one after the other - with 832 small blocks this kernel took 25 us
// for 77 k keys, most of it fences.)
constexpr int kPubThreads = 1024;

__global__ void __launch_bounds__(kPubThreads) p2p_query_send(hctr_p2p_ctx c, const u32 *__restrict__ meta,
                                                           const long long *__restrict__ uniq,
                                                           const uint8_t *__restrict__ uniq_owner,
                                                           const int32_t *__restrict__ uniq_row,
                                                           const long long *__restrict__ version, u32 seq,
                                                           const u32 *__restrict__ push_counts) {
  const size_t U = meta[HCTR_META_UNIQUE];
  const u32 *seg = meta + HCTR_META_SEG;
  for (size_t u = (size_t)blockIdx.x * kPubThreads + threadIdx.x; u < U; u += (size_t)gridDim.x * kPubThreads) {
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
  if (!last_block_of_launch(c.cnt_in + HCTR_P2P_TICKET0(c.nrank))) return;
  for (int p = threadIdx.x; p < c.nrank; p += kPubThreads) {
    __threadfence_system();
    u32 *hdr = c.box[p].hdr + (size_t)c.rank * kHdrWords;
    hdr[1] = seg[p + 1] - seg[p];
    hdr[2] = push_counts ? push_counts[p] : 0u;
    st_release_sys(hdr + 0, seq);
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

// One thread block; thread s waits for source s (bounded) and the counts land in c.cnt_in.
__global__ void __launch_bounds__(kMaxRanks) p2p_wait(hctr_p2p_ctx c, int phase, u32 seq) {
  __shared__ u32 a[kMaxRanks + 1], b[kMaxRanks + 1];
  if (phase == 0) wait_queries(c, seq, a, b, true);
  else wait_returns(c, seq, a, true);
}

// Returned rows go straight into the requesters' mailboxes.  A warp takes 32 consecutive returned rows: lane i
// fetches the list entries of row i (ret_q[r] = flat query index of returned row r, ret_row[r] = its local row,
// both written by p2p_stale_scan; coalesced, one load per 32 rows) and works out where the row goes; then all
// lanes move the elements of the 32 rows as one flat range, several independent loads in flight per lane.  The
// thread block that finishes last publishes the per-requester row counts and releases `seq` (phase 1) to every
// peer.
constexpr int kGatherUnroll = 4;

template <bool VEC>
__global__ void __launch_bounds__(kPubThreads) p2p_gather(hctr_p2p_ctx c, u32 seq, const u32 *__restrict__ ret_q,
                                                       const int32_t *__restrict__ ret_row,
                                                       const u32 *__restrict__ ret_slot,
                                                       const float *__restrict__ embedding,
                                                       const long long *__restrict__ version) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  __shared__ u32 qstart[kMaxRanks + 1];
  for (int i = threadIdx.x; i <= c.nrank; i += kPubThreads) qstart[i] = c.cnt_in[3 * c.nrank + i];
  __syncthreads();
  const u32 Q = qstart[c.nrank];
  const u32 n_ret = ret_slot[Q];
  const unsigned lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * kPubThreads + threadIdx.x) >> 5;
  const size_t n_warps = ((size_t)gridDim.x * kPubThreads) >> 5;
  const u32 E = (u32)R::elems(c.width);
  for (size_t r0 = warp * 32; r0 < n_ret; r0 += n_warps * 32) {
    const u32 cnt = (u32)min((size_t)32, (size_t)n_ret - r0);
    const T *src_row = nullptr;
    T *dst_row = nullptr;
    if (lane < cnt) {
      const u32 qq = ret_q[r0 + lane];
      const int32_t row = ret_row[r0 + lane];
      const unsigned s = segment_of(qstart, c.nrank, qq);
      const size_t dst = (size_t)c.rank * c.cap + ((u32)(r0 + lane) - ret_slot[qstart[s]]);
      const hctr_p2p_box b = c.box[s];
      b.rver[dst] = version[row];
      src_row = reinterpret_cast<const T *>(embedding) + (size_t)row * E;
      dst_row = reinterpret_cast<T *>(b.rval) + dst * E;
    }
    const u32 total = cnt * E;  // elements of the block's rows, as one flat range
    for (u32 t0 = 0; t0 < total; t0 += 32 * kGatherUnroll) {
      T v[kGatherUnroll];
      T *d[kGatherUnroll];
      u32 ee[kGatherUnroll];
#pragma unroll
      for (int k = 0; k < kGatherUnroll; k++) {
        const u32 t = t0 + 32u * k + lane;
        const u32 j = t / E, e = t - j * E;
        ee[k] = e;
        const bool act = t < total;
        // (shuffles are executed by all lanes; rows beyond the block read lane 0's pointers and are not used)
        const T *sp = reinterpret_cast<const T *>(__shfl_sync(0xffffffffu, (unsigned long long)src_row, act ? j : 0));
        d[k] = reinterpret_cast<T *>(__shfl_sync(0xffffffffu, (unsigned long long)dst_row, act ? j : 0));
        if (act) v[k] = sp[e];
        else d[k] = nullptr;
      }
#pragma unroll
      for (int k = 0; k < kGatherUnroll; k++)
        if (d[k]) d[k][ee[k]] = v[k];
    }
  }
  if (!last_block_of_launch(c.cnt_in + HCTR_P2P_TICKET1(c.nrank))) return;
  for (int p = threadIdx.x; p < c.nrank; p += kPubThreads) {
    __threadfence_system();
    u32 *hdr = c.box[p].hdr + (size_t)c.rank * kHdrWords;
    hdr[9] = ret_slot[qstart[p + 1]] - ret_slot[qstart[p]];
    st_release_sys(hdr + 8, seq);
  }
  if (threadIdx.x == 0) c.cnt_in[HCTR_P2P_SERVED(c.nrank)] = n_ret;
}

// ---- fused flag + scan kernels ---------------------------------------------------------------------
// A tile of kTileThreads * kTileItems entries per thread block: every thread computes the flags of its
// kTileItems consecutive entries, the block scans them and the tile totals are chained across blocks
// (chained_cta_prefix), so flags, slots and the lists derived from them come out of one launch.  Tiles are small
// (1024 entries) so that a step's ~10^5 queries spread over many SMs; a block adds up at most a few hundred
// predecessor totals.
constexpr int kTileThreads = 256;
constexpr int kTileItems = 4;
constexpr size_t kTile = (size_t)kTileThreads * kTileItems;

// exclusive prefix of `s` over the thread block (kTileThreads threads); *total = sum over the block
__device__ __forceinline__ u32 tile_exclusive_scan(u32 s, u32 *total) {
  __shared__ u32 warp_sums[32];
  __shared__ u32 s_total;
  constexpr unsigned kWarps = kTileThreads / 32;
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
    const u32 w = lane < kWarps ? warp_sums[lane] : 0u;
    u32 wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const u32 t = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= (unsigned)d) wi += t;
    }
    if (lane < kWarps) warp_sums[lane] = wi - w;
    if (lane == 31) s_total = wi;
  }
  __syncthreads();
  *total = s_total;
  return incl - s + warp_sums[warp];
}

// Owner: staleness flag of every received query (stored into the requester's mailbox), slot of every
// returned row (ret_slot, Q + 1 entries, entry Q = number of returned rows), the list of returned
// queries (ret_q[slot] = flat query index) and their local rows (ret_row[slot]) in one launch.
// stale = (requester's version is INT64_MIN or version + pull_bound < owner's version) and the requester is not
// this rank (csrc/core/handle_query.cu:7-22).
__global__ void __launch_bounds__(kTileThreads) p2p_stale_scan(hctr_p2p_ctx c, const int32_t *__restrict__ row_of,
                                                               size_t length, size_t n_cached,
                                                               const long long *__restrict__ version,
                                                               long long pull_bound, u32 *__restrict__ ret_slot,
                                                               u32 *__restrict__ ret_q, int32_t *__restrict__ ret_row,
                                                               u64 *agg, u32 epoch) {
  __shared__ u32 qstart[kMaxRanks + 1];
  for (int i = threadIdx.x; i <= c.nrank; i += kTileThreads) qstart[i] = c.cnt_in[3 * c.nrank + i];
  __syncthreads();
  const u32 Q = qstart[c.nrank];
  const size_t tile_base = (size_t)blockIdx.x * kTile;
  if (tile_base > Q) return;  // the tile that holds entry Q still runs: it writes the total
  const hctr_p2p_box me = c.box[c.rank];
  const size_t base = tile_base + (size_t)threadIdx.x * kTileItems;
  u32 v[kTileItems];
  int32_t rows[kTileItems];
  u32 sum = 0;
#pragma unroll
  for (int k = 0; k < kTileItems; k++) {
    const size_t q = base + k;
    u32 f = 0;
    rows[k] = -1;
    if (q < Q) {
      const unsigned s = segment_of(qstart, c.nrank, (u32)q);
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
        rows[k] = row;
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
    if (q < Q && v[k]) {
      ret_q[ex] = (u32)q;
      ret_row[ex] = rows[k];
    }
    ex += v[k];
  }
}

// Requester: waits (bounded) for every owner's returned rows, then collects the flag of every unique key from
// its mailbox (flags[u], zero for u >= U) and computes the index of the row returned for it (recv_index[u], in
// rows relative to box[rank].rval / rver), all in one launch.  Rows returned by owner p sit in sub-region p in
// the order of the flagged keys, so the index is p * cap + (flagged keys before u) - (flagged keys of earlier
// owners); the latter are the prefix of the per-owner returned-row counts the owners announced.
__global__ void __launch_bounds__(kTileThreads) p2p_recv_scan(hctr_p2p_ctx c, u32 seq, const u32 *__restrict__ meta,
                                                              size_t u_max, const uint8_t *__restrict__ uniq_owner,
                                                              uint8_t *__restrict__ flags,
                                                              u32 *__restrict__ recv_index,
                                                              u32 *__restrict__ recv_list, u64 *agg, u32 epoch) {
  __shared__ u32 owner_base[kMaxRanks + 1];
  const size_t U = meta[HCTR_META_UNIQUE];
  const u32 *seg = meta + HCTR_META_SEG;
  const size_t tile_base = (size_t)blockIdx.x * kTile;
  const size_t base = tile_base + (size_t)threadIdx.x * kTileItems;
  if (blockIdx.x != 0 && tile_base >= U) {  // nothing to rank here (and nobody waits for this block): clear and leave
#pragma unroll
    for (int k = 0; k < kTileItems; k++)
      if (base + k < u_max) flags[base + k] = 0, recv_index[base + k] = 0;
    return;
  }
  wait_returns(c, seq, owner_base, blockIdx.x == 0);  // block 0 always runs: it records the counts for the host
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
    if (v[k]) recv_list[ex] = (u32)u;  // the ex-th key (in unique order) a row came back for
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
                                   uint32_t seq, const uint32_t *push_counts, void *stream) {
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  size_t g = (u_max + kPubThreads - 1) / kPubThreads;
  if (g > (size_t)kSMs) g = kSMs;
  p2p_query_send<<<(unsigned)(g ? g : 1), kPubThreads, 0, (cudaStream_t)stream>>>(
      *c, meta, (const long long *)uniq, uniq_owner, uniq_row, (const long long *)version, seq, push_counts);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_signal(const hctr_p2p_ctx *c, int phase, uint32_t seq, const uint32_t *meta,
                               const uint32_t *counts, void *stream) {
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  p2p_signal<<<1, kMaxRanks, 0, (cudaStream_t)stream>>>(*c, phase, seq, meta, counts);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_wait(const hctr_p2p_ctx *c, int phase, uint32_t seq, void *stream) {
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  p2p_wait<<<1, kMaxRanks, 0, (cudaStream_t)stream>>>(*c, phase, seq);
  count_launches(1);
  return launch_status();
}

extern "C" size_t hctr_p2p_scan_scratch_words(size_t entries) { return 2 * ((entries + 1 + kTile - 1) / kTile + 1); }

extern "C" int hctr_p2p_stale_scan(const hctr_p2p_ctx *c, const int32_t *row_of, size_t length, size_t n_cached,
                                   const int64_t *version, int64_t pull_bound, uint32_t *ret_slot, uint32_t *ret_q,
                                   int32_t *ret_row, uint32_t *scratch, uint32_t epoch, void *stream) {
  if (c->nrank > kMaxRanks || epoch == 0) return (int)cudaErrorInvalidValue;
  const size_t slots = (size_t)c->nrank * c->cap;
  const unsigned grid = (unsigned)((slots + 1 + kTile - 1) / kTile);
  p2p_stale_scan<<<grid, kTileThreads, 0, (cudaStream_t)stream>>>(*c, row_of, length, n_cached,
                                                                  (const long long *)version, pull_bound, ret_slot,
                                                                  ret_q, ret_row, reinterpret_cast<u64 *>(scratch),
                                                                  epoch);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_gather(const hctr_p2p_ctx *c, uint32_t seq, const uint32_t *ret_q, const int32_t *ret_row,
                               const uint32_t *ret_slot, const float *embedding, const int64_t *version,
                               void *stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  // one warp per 32 returned rows; at most nrank * cap rows exist, a few resident rounds of blocks cover them
  size_t g = ((size_t)c->nrank * c->cap / 32 + 1 + kPubThreads / 32 - 1) / (kPubThreads / 32);
  if (g > (size_t)kSMs) g = kSMs;  // a publishing kernel: one block per SM at most
  if (g == 0) g = 1;
  const bool vec = host_aligned16(embedding) && c->width % 4 == 0;
  if (vec) p2p_gather<true><<<(unsigned)g, kPubThreads, 0, st>>>(*c, seq, ret_q, ret_row, ret_slot, embedding, (const long long *)version);
  else p2p_gather<false><<<(unsigned)g, kPubThreads, 0, st>>>(*c, seq, ret_q, ret_row, ret_slot, embedding, (const long long *)version);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_recv_scan(const hctr_p2p_ctx *c, uint32_t seq, const uint32_t *meta, size_t u_max,
                                  const uint8_t *uniq_owner, uint8_t *flags, uint32_t *recv_index,
                                  uint32_t *recv_list, uint32_t *scratch, uint32_t epoch, void *stream) {
  if (c->nrank > kMaxRanks || epoch == 0) return (int)cudaErrorInvalidValue;
  const unsigned grid = (unsigned)((u_max + kTile - 1) / kTile);
  p2p_recv_scan<<<grid ? grid : 1, kTileThreads, 0, (cudaStream_t)stream>>>(*c, seq, meta, u_max, uniq_owner, flags,
                                                                            recv_index, recv_list,
                                                                            reinterpret_cast<u64 *>(scratch), epoch);
  count_launches(1);
  return launch_status();
}
