// Pull side of the peer-to-peer exchange: the owner answers the queries in its mailbox, the requester takes the
// answers in.  Nothing is compacted: the row returned for the j-th query of requester s goes to row
// (owner * cap + j) of s's mailbox, the place s can compute for each of its unique keys without knowing what the
// owner decided.  So neither side needs a prefix sum over flags (the reference compacts on the owner,
// csrc/core/handle_query.cu:24-73, and scans again on the requester, csrc/core/writeback.cu:43-50), and the
// owner's staleness test and row gather are one launch, the requester's flag collection and cache refresh another.
#include "p2p.cuh"
#include "rowops.cuh"

namespace hctr {

constexpr int kPullThreads = 1024;  // fat blocks, at most a few per SM: every block polls or fences at system scope
constexpr long long kInvalidVersion = INT64_MIN;
constexpr int kCopyUnroll = 4;

// The elements of `cnt` rows (cnt <= 32; lane i holds the pointers of row i) moved as ONE flat range by the
// warp, kCopyUnroll independent loads in flight per lane.  COMBINE: dst = src + add (the cache refresh), else a
// plain copy.  All 32 lanes must call it.
template <class R, bool COMBINE>
__device__ __forceinline__ void warp_move_rows(u32 cnt, u32 E, const typename R::T *src_row,
                                               const typename R::T *add_row, typename R::T *dst_row) {
  typedef typename R::T T;
  const unsigned lane = threadIdx.x & 31;
  const u32 total = cnt * E;
  for (u32 t0 = 0; t0 < total; t0 += 32 * kCopyUnroll) {
    T v[kCopyUnroll], w[kCopyUnroll];
    T *d[kCopyUnroll];
    u32 ee[kCopyUnroll];
#pragma unroll
    for (int k = 0; k < kCopyUnroll; k++) {
      const u32 t = t0 + 32u * k + lane;
      const u32 j = t / E, e = t - j * E;
      ee[k] = e;
      const bool act = t < total;
      // (shuffles are executed by all lanes; slots beyond the range read lane 0's pointers and are not used)
      const T *sp = reinterpret_cast<const T *>(__shfl_sync(0xffffffffu, (unsigned long long)src_row, act ? j : 0));
      const T *ap = reinterpret_cast<const T *>(__shfl_sync(0xffffffffu, (unsigned long long)add_row, act ? j : 0));
      d[k] = reinterpret_cast<T *>(__shfl_sync(0xffffffffu, (unsigned long long)dst_row, act ? j : 0));
      if (act) {
        v[k] = sp[e];
        if (COMBINE) w[k] = ap[e];
      } else {
        d[k] = nullptr;
      }
    }
#pragma unroll
    for (int k = 0; k < kCopyUnroll; k++)
      if (d[k]) d[k][ee[k]] = COMBINE ? R::add(v[k], w[k]) : v[k];
  }
}

// Lane i of the warp receives the value that the i-th lane with its bit set in `mask` holds.
template <class V>
__device__ __forceinline__ V warp_compact(unsigned mask, V value) {
  const unsigned lane = threadIdx.x & 31;
  const unsigned from = __fns(mask, 0, (int)lane + 1);  // 0xffffffff when there is no such lane
  return __shfl_sync(0xffffffffu, value, from < 32 ? (int)from : 0);
}

// Owner.  For every received query (flat index q over the sources' sub-regions; counts and starts were recorded
// in c.cnt_in by the kernel that waited for them): stale = (requester's version is INT64_MIN or version +
// pull_bound < owner's version) and the requester is not this rank (csrc/core/handle_query.cu:7-22).  The flag
// byte goes to the requester's mailbox; a stale key's row and version follow, to row rank * cap + j of that
// mailbox (write_return_value_kernel, csrc/core/handle_query.cu:24-40).  A warp takes 32 queries, one per lane for
// the decision, then moves the rows of the stale ones together.  The block that finishes last releases `seq`
// (phase 1) to every peer, all2allReturnOutdated / all2allReturnValue in one, csrc/core/all2all.cu:89-130.
template <bool VEC>
__global__ void __launch_bounds__(kPullThreads) p2p_stale_gather(hctr_p2p_ctx c, u32 seq,
                                                                 const int32_t *__restrict__ row_of, size_t length,
                                                                 size_t n_cached, const float *__restrict__ embedding,
                                                                 const long long *__restrict__ version,
                                                                 long long pull_bound) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  __shared__ u32 qstart[kMaxRanks + 1];
  __shared__ u32 s_served;
  for (int i = threadIdx.x; i <= c.nrank; i += kPullThreads) qstart[i] = c.cnt_in[3 * c.nrank + i];
  if (threadIdx.x == 0) s_served = 0;
  __syncthreads();
  const u32 Q = qstart[c.nrank];
  const unsigned lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * kPullThreads + threadIdx.x) >> 5;
  const size_t n_warps = ((size_t)gridDim.x * kPullThreads) >> 5;
  const u32 E = (u32)R::elems(c.width);
  const hctr_p2p_box me = c.box[c.rank];
  u32 served = 0;
  for (size_t q0 = warp * 32; q0 < Q; q0 += n_warps * 32) {
    const size_t q = q0 + lane;
    bool stale = false;
    const T *src_row = nullptr;
    T *dst_row = nullptr;
    if (q < Q) {
      const unsigned s = segment_of(qstart, c.nrank, (u32)q);
      const u32 j = (u32)q - qstart[s];
      const size_t slot = (size_t)s * c.cap + j;
      const long long key = me.qkey[slot];
      int32_t row = -1;
      if (key >= 0 && (size_t)key < length) row = row_of[key];
      const size_t out = (size_t)c.rank * c.cap + j;
      const hctr_p2p_box b = c.box[s];
      if (row < 0 || (size_t)row < n_cached) {
        atomicOr(c.err, HCTR_ERR_NOT_OWNER);
      } else {
        const long long lv = me.qver[slot], gv = version[row];
        stale = (lv == kInvalidVersion || (long long)((u64)lv + (u64)pull_bound) < gv) && s != (unsigned)c.rank;
        if (stale) {
          b.rver[out] = gv;
          src_row = reinterpret_cast<const T *>(embedding) + (size_t)row * E;
          dst_row = reinterpret_cast<T *>(b.rval) + out * E;
        }
      }
      b.flag[out] = stale ? 1 : 0;
    }
    const unsigned m = __ballot_sync(0xffffffffu, stale);
    if (m == 0) continue;
    const u32 cnt = __popc(m);
    served += cnt;
    const T *sp = reinterpret_cast<const T *>(warp_compact(m, (unsigned long long)src_row));
    T *dp = reinterpret_cast<T *>(warp_compact(m, (unsigned long long)dst_row));
    warp_move_rows<R, false>(cnt, E, sp, nullptr, dp);
  }
  if (lane == 0 && served) atomicAdd(&s_served, served);
  __syncthreads();
  if (threadIdx.x == 0 && s_served) atomicAdd(c.cnt_in + HCTR_P2P_SERVED(c.nrank), s_served);
  if (!last_block_of_launch(c.cnt_in + HCTR_P2P_TICKET1(c.nrank))) return;
  for (int p = threadIdx.x; p < c.nrank; p += kPullThreads) {
    __threadfence_system();
    u32 *hdr = c.box[p].hdr + (size_t)c.rank * kHdrWords;
    hdr[9] = 0;
    st_release_sys(hdr + 8, seq);
  }
}

// Requester.  Waits (bounded) for every owner's phase-1 release of `seq`, then for each unique key u of the batch:
// recv_index[u] = owner * cap + j, the row of this rank's mailbox the owner of u would have written (j = u's place
// among the keys sent to that owner); flags[u] = what the owner decided; and, for a flagged key that is cached
// here, the cache refresh embedding[row] = returned row + pending[row], version[row] = returned version
// (csrc/core/writeback.cu:8-27).  A warp takes 32 unique keys and moves the rows of those to refresh together.
// The number of flagged keys of the step is added to c.cnt_in[2 * nrank] (statistics).
template <bool VEC>
__global__ void __launch_bounds__(kPullThreads) p2p_refresh_index(hctr_p2p_ctx c, u32 seq,
                                                                  const u32 *__restrict__ meta,
                                                                  const uint8_t *__restrict__ uniq_owner,
                                                                  const int32_t *__restrict__ uniq_row,
                                                                  size_t n_cached, const float *__restrict__ pending,
                                                                  float *__restrict__ embedding,
                                                                  long long *__restrict__ version,
                                                                  uint8_t *__restrict__ flags,
                                                                  u32 *__restrict__ recv_index) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  __shared__ u32 ret_base[kMaxRanks + 1];
  __shared__ u32 s_flagged;
  if (threadIdx.x == 0) s_flagged = 0;
  wait_returns(c, seq, ret_base, false, blockIdx.x == 0);  // (ends with a block barrier)
  const size_t U = meta[HCTR_META_UNIQUE];
  const u32 *seg = meta + HCTR_META_SEG;
  const unsigned lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * kPullThreads + threadIdx.x) >> 5;
  const size_t n_warps = ((size_t)gridDim.x * kPullThreads) >> 5;
  const u32 E = (u32)R::elems(c.width);
  const hctr_p2p_box me = c.box[c.rank];
  u32 flagged = 0;
  for (size_t u0 = warp * 32; u0 < U; u0 += n_warps * 32) {
    const size_t u = u0 + lane;
    bool refresh = false, f = false;
    const T *src_row = nullptr, *add_row = nullptr;
    T *dst_row = nullptr;
    if (u < U) {
      const unsigned p = uniq_owner[u];
      const u32 j = (u32)u - seg[p];
      u32 idx = 0;
      if (j < c.cap) {  // (a larger j was reported when the query was sent)
        idx = p * c.cap + j;
        f = me.flag[idx] != 0;
      }
      flags[u] = f ? 1 : 0;
      recv_index[u] = idx;
      const int32_t row = uniq_row[u];
      refresh = f && row >= 0 && (size_t)row < n_cached;
      if (refresh) {
        version[row] = reinterpret_cast<const long long *>(me.rver)[idx];
        src_row = reinterpret_cast<const T *>(me.rval) + (size_t)idx * E;
        add_row = reinterpret_cast<const T *>(pending) + (size_t)row * E;
        dst_row = reinterpret_cast<T *>(embedding) + (size_t)row * E;
      }
    }
    flagged += __popc(__ballot_sync(0xffffffffu, f));
    const unsigned m = __ballot_sync(0xffffffffu, refresh);
    if (m == 0) continue;
    const T *sp = reinterpret_cast<const T *>(warp_compact(m, (unsigned long long)src_row));
    const T *ap = reinterpret_cast<const T *>(warp_compact(m, (unsigned long long)add_row));
    T *dp = reinterpret_cast<T *>(warp_compact(m, (unsigned long long)dst_row));
    warp_move_rows<R, true>(__popc(m), E, sp, ap, dp);
  }
  if (lane == 0 && flagged) atomicAdd(&s_flagged, flagged);
  __syncthreads();
  if (threadIdx.x == 0 && s_flagged) atomicAdd(c.cnt_in + 2 * c.nrank, s_flagged);
}

// Requester, everything after the owners' answers in ONE launch: the cache refresh of p2p_refresh_index and the row
// expansion (writeBack, csrc/core/writeback.cu:8-71) without the per-key flag / row-index arrays between them.
// Every block waits (bounded) for the owners' phase-1 release, then takes a share of the unique keys (refresh of the
// flagged cached rows, as above) and a share of the batch positions.  A position's row comes from
//   the table            when the key is owned here, or cached and not flagged,
//   the mailbox          when the key is not stored here (row owner * cap + j, j = its place among the keys sent there),
//   mailbox + pending    when the key is cached and flagged - the same sum the refresh stores into the cache row,
//                        computed again here so that no block has to wait for the block that refreshes that row.
// The refresh writes only flagged cached rows, which the expansion never reads: the two parts are independent.
constexpr int kFusedRows = 4;  // rows per lane group and iteration, as in the plain expansion
constexpr int kFusedThreads = 256;  // >= kMaxRanks: thread s of every block polls owner s

template <int LANES, bool VEC>
__global__ void __launch_bounds__(kFusedThreads) p2p_refresh_expand(hctr_p2p_ctx c, u32 seq, const u32 *__restrict__ meta,
                                                               const uint8_t *__restrict__ uniq_owner,
                                                               const int32_t *__restrict__ uniq_row, size_t n_cached,
                                                               const float *__restrict__ pending,
                                                               float *__restrict__ embedding,
                                                               long long *__restrict__ version, size_t batch,
                                                               const int32_t *__restrict__ pos_row,
                                                               const int32_t *__restrict__ idx_map,
                                                               float *__restrict__ dst) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  __shared__ u32 ret_base[kMaxRanks + 1];
  __shared__ u32 seg[kMaxRanks + 1];
  __shared__ u32 s_flagged, s_n;
  __shared__ u32 s_idx[kFusedThreads], s_row[kFusedThreads];
  if (threadIdx.x == 0) s_flagged = s_n = 0;
  for (int i = threadIdx.x; i <= c.nrank; i += kFusedThreads) seg[i] = meta[HCTR_META_SEG + i];
  wait_returns(c, seq, ret_base, false, blockIdx.x == 0);  // (ends with a block barrier)
  const size_t U = meta[HCTR_META_UNIQUE];
  const unsigned lane = threadIdx.x & 31;
  const u32 E = (u32)R::elems(c.width);
  const hctr_p2p_box me = c.box[c.rank];
  const T *rval = reinterpret_cast<const T *>(me.rval);

  // refresh of the flagged cached rows: the block looks at kFusedThreads unique keys at a time, one per thread, lists
  // the rows to refresh in shared memory and then shares them out evenly among its lane groups (a few rows per
  // block: spread over the whole block they cost one round of loads, left to the warp that found them, several)
  {
    const unsigned n_groups = kFusedThreads / LANES, group = threadIdx.x / LANES, gl = threadIdx.x % LANES;
    u32 flagged = 0;
    for (size_t base = (size_t)blockIdx.x * kFusedThreads; base < U; base += (size_t)gridDim.x * kFusedThreads) {
      const size_t u = base + threadIdx.x;
      bool f = false;
      if (u < U) {
        const unsigned p = uniq_owner[u];
        const u32 j = (u32)u - seg[p];
        if (j < c.cap) {  // (a larger j was reported when the query was sent)
          const u32 idx = p * c.cap + j;
          f = me.flag[idx] != 0;
          const int32_t row = uniq_row[u];
          if (f && row >= 0 && (size_t)row < n_cached) {
            version[row] = reinterpret_cast<const long long *>(me.rver)[idx];
            const u32 e = atomicAdd(&s_n, 1u);
            s_idx[e] = idx;
            s_row[e] = (u32)row;
          }
        }
      }
      flagged += f ? 1u : 0u;
      __syncthreads();
      const u32 n = s_n;
      for (u32 e0 = group * kFusedRows; e0 < n; e0 += n_groups * kFusedRows) {
        for (u32 col = gl; col < E; col += LANES) {
          T v[kFusedRows], w[kFusedRows];
#pragma unroll
          for (int k = 0; k < kFusedRows; k++)
            if (e0 + k < n) {
              v[k] = rval[(size_t)s_idx[e0 + k] * E + col];
              w[k] = reinterpret_cast<const T *>(pending)[(size_t)s_row[e0 + k] * E + col];
            }
#pragma unroll
          for (int k = 0; k < kFusedRows; k++)
            if (e0 + k < n) reinterpret_cast<T *>(embedding)[(size_t)s_row[e0 + k] * E + col] = R::add(v[k], w[k]);
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) s_n = 0;
      // (the next round's first barrier orders this store before the next list is read; its appends come after the
      // barrier below)
      __syncthreads();
    }
    flagged = __reduce_add_sync(0xffffffffu, flagged);
    if (lane == 0 && flagged) atomicAdd(&s_flagged, flagged);
  }

  // expansion: a group of LANES lanes takes kFusedRows positions per iteration
  const size_t groups = ((size_t)gridDim.x * kFusedThreads) / LANES;
  const unsigned gl = threadIdx.x % LANES;
  for (size_t i0 = (((size_t)blockIdx.x * kFusedThreads + threadIdx.x) / LANES) * kFusedRows; i0 < batch;
       i0 += groups * kFusedRows) {
    const T *src[kFusedRows], *add[kFusedRows];
#pragma unroll
    for (int k = 0; k < kFusedRows; k++) {
      src[k] = nullptr;
      add[k] = nullptr;
      const size_t i = i0 + k;
      if (i < batch) {
        const int32_t row = pos_row[i];
        if (row >= 0 && (size_t)row >= n_cached) {
          src[k] = reinterpret_cast<const T *>(embedding) + (size_t)row * E;
        } else {
          const int32_t u = idx_map[i];  // < 0: key was out of range (the host reports it); write zeros
          if (u >= 0) {
            const unsigned p = uniq_owner[u];
            const u32 j = (u32)u - seg[p];
            const u32 idx = j < c.cap ? p * c.cap + j : 0u;
            if (row < 0) {
              src[k] = rval + (size_t)idx * E;
            } else if (j < c.cap && me.flag[idx] != 0) {
              src[k] = rval + (size_t)idx * E;
              add[k] = reinterpret_cast<const T *>(pending) + (size_t)row * E;
            } else {
              src[k] = reinterpret_cast<const T *>(embedding) + (size_t)row * E;
            }
          }
        }
      }
    }
    for (size_t col = gl; col < E; col += LANES) {
      T v[kFusedRows];
#pragma unroll
      for (int k = 0; k < kFusedRows; k++) {
        v[k] = src[k] ? src[k][col] : R::zero();
        if (add[k]) v[k] = R::add(v[k], add[k][col]);
      }
#pragma unroll
      for (int k = 0; k < kFusedRows; k++)
        if (i0 + k < batch) R::st_once(reinterpret_cast<T *>(dst) + (i0 + k) * E + col, v[k]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_flagged) atomicAdd(c.cnt_in + 2 * c.nrank, s_flagged);
}

}  // namespace hctr

using namespace hctr;

extern "C" int hctr_p2p_stale_gather(const hctr_p2p_ctx *c, uint32_t seq, const int32_t *row_of, size_t length,
                                     size_t n_cached, const float *embedding, const int64_t *version,
                                     int64_t pull_bound, void *stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  // one warp per 32 queries; a publishing kernel runs one block per SM at most
  size_t g = ((size_t)c->nrank * c->cap / 32 + 1 + kPullThreads / 32 - 1) / (kPullThreads / 32);
  if (g > (size_t)kSMs) g = kSMs;
  if (g == 0) g = 1;
  const bool vec = host_aligned16(embedding) && c->width % 4 == 0;
  if (vec)
    p2p_stale_gather<true><<<(unsigned)g, kPullThreads, 0, st>>>(*c, seq, row_of, length, n_cached, embedding,
                                                                 (const long long *)version, pull_bound);
  else
    p2p_stale_gather<false><<<(unsigned)g, kPullThreads, 0, st>>>(*c, seq, row_of, length, n_cached, embedding,
                                                                  (const long long *)version, pull_bound);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_refresh_index(const hctr_p2p_ctx *c, uint32_t seq, const uint32_t *meta, size_t u_max,
                                      const uint8_t *uniq_owner, const int32_t *uniq_row, size_t n_cached,
                                      const float *pending, float *embedding, int64_t *version, uint8_t *flags,
                                      uint32_t *recv_index, void *stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  size_t g = (u_max / 32 + 1 + kPullThreads / 32 - 1) / (kPullThreads / 32);
  if (g > (size_t)kSMs) g = kSMs;  // every block starts by polling the mailbox headers
  if (g == 0) g = 1;               // (an empty batch still waits for the peers: the step's protocol)
  const bool vec = host_aligned16(embedding) && host_aligned16(pending) && c->width % 4 == 0;
  if (vec)
    p2p_refresh_index<true><<<(unsigned)g, kPullThreads, 0, st>>>(*c, seq, meta, uniq_owner, uniq_row, n_cached,
                                                                  pending, embedding, (long long *)version, flags,
                                                                  recv_index);
  else
    p2p_refresh_index<false><<<(unsigned)g, kPullThreads, 0, st>>>(*c, seq, meta, uniq_owner, uniq_row, n_cached,
                                                                   pending, embedding, (long long *)version, flags,
                                                                   recv_index);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_refresh_expand(const hctr_p2p_ctx *c, uint32_t seq, const uint32_t *meta,
                                       const uint8_t *uniq_owner, const int32_t *uniq_row, size_t n_cached,
                                       const float *pending, float *embedding, int64_t *version, size_t batch,
                                       const int32_t *pos_row, const int32_t *idx_map, float *dst, void *stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  const size_t width = c->width;
  // (the mailbox arrays are device allocations of their own: aligned; c->box is a device array)
  const bool al = host_aligned16(embedding) && host_aligned16(pending) && host_aligned16(dst);
#define CALL(L, V)                                                                                         \
  do {                                                                                                     \
    size_t g_ = (((size_t)batch + kFusedRows - 1) / kFusedRows * L + kFusedThreads - 1) / kFusedThreads;              \
    const size_t cap_ = (size_t)kSMs * 4; /* one resident round (64 registers); every block polls the headers */ \
    if (g_ > cap_) g_ = cap_;                                                                              \
    if (g_ == 0) g_ = 1; /* an empty batch still waits for the peers: the step's protocol */               \
    p2p_refresh_expand<L, V><<<(unsigned)g_, kFusedThreads, 0, st>>>(*c, seq, meta, uniq_owner, uniq_row, n_cached, \
                                                                pending, embedding, (long long *)version, batch, \
                                                                pos_row, idx_map, dst);                    \
  } while (0)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}
