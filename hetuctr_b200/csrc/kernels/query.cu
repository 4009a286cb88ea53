// Pull side of a step: query versions, owner-side staleness check + row gather, requester-side cache
// refresh and the final expansion of unique rows to batch order.
#include "rowops.cuh"

namespace hctr {

constexpr int kThreads = 256;
constexpr long long kInvalidVersion = INT64_MIN;

__global__ void __launch_bounds__(kThreads) query_versions(size_t n_unique, const int32_t *__restrict__ uniq_row,
                                                           const long long *__restrict__ version,
                                                           long long *__restrict__ query_version) {
  const size_t u = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (u >= n_unique) return;
  const int32_t row = uniq_row[u];
  query_version[u] = row >= 0 ? version[row] : kInvalidVersion;
}

__global__ void __launch_bounds__(kThreads) stale_check(size_t n_query, int nrank, int rank,
                                                        const u32 *__restrict__ seg_start,
                                                        const long long *__restrict__ key,
                                                        const long long *__restrict__ req_version,
                                                        const int32_t *__restrict__ row_of, size_t length,
                                                        size_t n_cached, const long long *__restrict__ version,
                                                        long long pull_bound, uint8_t *__restrict__ flags,
                                                        u32 *__restrict__ flags32, u32 *err) {
  const size_t q = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (q >= n_query) return;
  const long long k = key[q];
  int32_t row = -1;
  if (k >= 0 && (size_t)k < length) row = row_of[k];
  if (row < 0 || (size_t)row < n_cached) {
    atomicOr(err, HCTR_ERR_NOT_OWNER);
    flags[q] = 0;
    flags32[q] = 0;
    return;
  }
  const bool from_self = q >= seg_start[rank] && q < seg_start[rank + 1];
  const long long lv = req_version[q], gv = version[row];
  const bool stale = lv == kInvalidVersion || (long long)((u64)lv + (u64)pull_bound) < gv;
  const u32 f = (stale && !from_self) ? 1u : 0u;
  flags[q] = (uint8_t)f;
  flags32[q] = f;
}

__global__ void pack_counts(const u32 *__restrict__ meta, const u32 *__restrict__ push_count, int nrank,
                            u32 *__restrict__ out) {
  const int p = threadIdx.x;
  if (p < nrank) {
    const u32 *seg = meta + HCTR_META_SEG;
    out[2 * p] = seg[p + 1] - seg[p];
    out[2 * p + 1] = push_count ? push_count[p] : 0u;
  }
}

__global__ void segment_counts(int nrank, const u32 *__restrict__ seg_start, const u32 *__restrict__ slot,
                               u32 *__restrict__ count) {
  const int p = threadIdx.x;
  if (p < nrank) count[p] = slot[seg_start[p + 1]] - slot[seg_start[p]];
}

template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) gather_rows(size_t n_query, size_t width, const long long *__restrict__ key,
                                                        const uint8_t *__restrict__ flags,
                                                        const u32 *__restrict__ ret_slot,
                                                        const int32_t *__restrict__ row_of,
                                                        const float *__restrict__ embedding,
                                                        const long long *__restrict__ version,
                                                        float *__restrict__ ret_val,
                                                        long long *__restrict__ ret_version) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  const size_t q = ((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES;
  const unsigned gl = threadIdx.x % LANES;
  if (q >= n_query || !flags[q]) return;
  const int32_t row = row_of[key[q]];
  const size_t slot = ret_slot[q];
  if (gl == 0) ret_version[slot] = version[row];
  const size_t E = R::elems(width);
  const T *src = reinterpret_cast<const T *>(embedding) + (size_t)row * E;
  T *dst = reinterpret_cast<T *>(ret_val) + slot * E;
  for (size_t c = gl; c < E; c += LANES) dst[c] = src[c];
}

__global__ void __launch_bounds__(kThreads) widen_flags(size_t n, const uint8_t *__restrict__ flags,
                                                        u32 *__restrict__ flags32) {
  const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (i < n) flags32[i] = flags[i] ? 1u : 0u;
}

template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) cache_refresh(size_t n_unique, size_t width, const uint8_t *__restrict__ flags,
                                                          const u32 *__restrict__ recv_slot,
                                                          const int32_t *__restrict__ uniq_row,
                                                          const float *__restrict__ recv_val,
                                                          const long long *__restrict__ recv_version,
                                                          const float *__restrict__ pending,
                                                          float *__restrict__ embedding,
                                                          long long *__restrict__ version) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  const size_t u = ((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES;
  const unsigned gl = threadIdx.x % LANES;
  if (u >= n_unique || !flags[u]) return;
  const int32_t row = uniq_row[u];
  if (row < 0) return;
  const size_t slot = recv_slot[u];
  if (gl == 0) version[row] = recv_version[slot];
  const size_t E = R::elems(width);
  const T *src = reinterpret_cast<const T *>(recv_val) + slot * E;
  const T *pend = reinterpret_cast<const T *>(pending) + (size_t)row * E;
  T *emb = reinterpret_cast<T *>(embedding) + (size_t)row * E;
  for (size_t c = gl; c < E; c += LANES) emb[c] = R::add(src[c], pend[c]);
}

// dst[i] = row of batch key i.  Row reads use default caching (duplicates and the rows just updated
// hit L2); dst is written once and never re-read by this path, so it is stored evict-first.
// A group moves kExpandRows rows per iteration so that several independent row reads are in flight
// per lane; the source row comes straight from the per-position row index computed at preprocess.
constexpr int kExpandRows = 4;

template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) expand_rows(size_t batch, size_t width, const int32_t *__restrict__ pos_row,
                                                        const int32_t *__restrict__ idx_map,
                                                        const u32 *__restrict__ recv_slot,
                                                        const float *__restrict__ recv_val,
                                                        const float *__restrict__ embedding,
                                                        float *__restrict__ dst) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  const size_t groups = ((size_t)gridDim.x * kThreads) / LANES;
  const unsigned gl = threadIdx.x % LANES;
  const size_t E = R::elems(width);
  for (size_t i0 = (((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES) * kExpandRows; i0 < batch;
       i0 += groups * kExpandRows) {
    const T *src[kExpandRows];
#pragma unroll
    for (int k = 0; k < kExpandRows; k++) {
      src[k] = nullptr;
      const size_t i = i0 + k;
      if (i < batch) {
        const int32_t row = pos_row[i];
        if (row >= 0) {
          src[k] = reinterpret_cast<const T *>(embedding) + (size_t)row * E;
        } else {
          const int32_t u = idx_map[i];  // < 0: key was out of range (the host reports it); write zeros
          if (u >= 0 && recv_slot) src[k] = reinterpret_cast<const T *>(recv_val) + (size_t)recv_slot[u] * E;
        }
      }
    }
    for (size_t c = gl; c < E; c += LANES) {
      T v[kExpandRows];
#pragma unroll
      for (int k = 0; k < kExpandRows; k++) v[k] = src[k] ? src[k][c] : R::zero();
#pragma unroll
      for (int k = 0; k < kExpandRows; k++)
        if (i0 + k < batch) R::st_once(reinterpret_cast<T *>(dst) + (i0 + k) * E + c, v[k]);
    }
  }
}

}  // namespace hctr

using namespace hctr;

extern "C" int hctr_pack_counts(const uint32_t *meta, const uint32_t *push_count, int nrank, uint32_t *out,
                                void *stream) {
  if (nrank > 1024) return (int)cudaErrorInvalidValue;
  pack_counts<<<1, 1024, 0, (cudaStream_t)stream>>>(meta, push_count, nrank, out);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_query_versions(size_t n_unique, const int32_t *uniq_row, const int64_t *version,
                                   int64_t *query_version, void *stream) {
  if (n_unique == 0) return 0;
  query_versions<<<grid_for(n_unique, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
      n_unique, uniq_row, (const long long *)version, (long long *)query_version);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_stale_check(size_t n_query, int nrank, int rank, const uint32_t *seg_start,
                                const int64_t *key, const int64_t *req_version, const int32_t *row_of,
                                size_t length, size_t n_cached, const int64_t *version, int64_t pull_bound,
                                uint8_t *flags, uint32_t *flags32, uint32_t *ret_slot, uint32_t *scan_scratch,
                                uint32_t *ret_count, uint32_t *err, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (nrank > 1024) return (int)cudaErrorInvalidValue;
  count_launches(n_query ? 2 : 1);
  if (n_query)
    stale_check<<<grid_for(n_query, kThreads), kThreads, 0, s>>>(
        n_query, nrank, rank, seg_start, (const long long *)key, (const long long *)req_version, row_of, length,
        n_cached, (const long long *)version, pull_bound, flags, flags32, err);
  int rc = hctr_scan_exclusive_u32(flags32, ret_slot, n_query, nullptr, scan_scratch, stream);
  if (rc) return rc;
  segment_counts<<<1, 1024, 0, s>>>(nrank, seg_start, ret_slot, ret_count);
  return launch_status();
}

extern "C" int hctr_gather_rows(size_t n_query, size_t width, const int64_t *key, const uint8_t *flags,
                                const uint32_t *ret_slot, const int32_t *row_of, const float *embedding,
                                const int64_t *version, float *ret_val, int64_t *ret_version, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (n_query == 0) return 0;
  const bool al = host_aligned16(embedding) && host_aligned16(ret_val);
#define CALL(L, V)                                                                                     \
  gather_rows<L, V><<<grid_for(n_query * L, kThreads), kThreads, 0, s>>>(                              \
      n_query, width, (const long long *)key, flags, ret_slot, row_of, embedding, (const long long *)version, \
      ret_val, (long long *)ret_version)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_recv_slots(size_t n_unique, const uint8_t *flags, uint32_t *flags32, uint32_t *recv_slot,
                               uint32_t *scan_scratch, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  count_launches(n_unique ? 1 : 0);
  if (n_unique) widen_flags<<<grid_for(n_unique, kThreads), kThreads, 0, s>>>(n_unique, flags, flags32);
  return hctr_scan_exclusive_u32(flags32, recv_slot, n_unique, nullptr, scan_scratch, stream);
}

extern "C" int hctr_cache_refresh(size_t n_unique, size_t width, const uint8_t *flags, const uint32_t *recv_slot,
                                  const int32_t *uniq_row, const float *recv_val, const int64_t *recv_version,
                                  const float *pending, float *embedding, int64_t *version, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (n_unique == 0) return 0;
  const bool al = host_aligned16(recv_val) && host_aligned16(pending) && host_aligned16(embedding);
#define CALL(L, V)                                                                               \
  cache_refresh<L, V><<<grid_for(n_unique * L, kThreads), kThreads, 0, s>>>(                     \
      n_unique, width, flags, recv_slot, uniq_row, recv_val, (const long long *)recv_version, pending, \
      embedding, (long long *)version)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_expand_rows(size_t batch, size_t width, const int32_t *pos_row, const int32_t *idx_map,
                                const uint32_t *recv_slot, const float *recv_val, const float *embedding,
                                float *dst, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (batch == 0) return 0;
  const bool al = host_aligned16(recv_val) && host_aligned16(embedding) && host_aligned16(dst);
#define CALL(L, V)                                                                       \
  do {                                                                                   \
    size_t g_ = (((size_t)batch + kExpandRows - 1) / kExpandRows * L + kThreads - 1) / kThreads; \
    /* persistent, exactly one resident wave: the kernel needs ~80 registers, i.e. 3 CTAs per SM */ \
    const size_t cap_ = (size_t)kSMs * 3;                                                \
    if (g_ > cap_) g_ = cap_;                                                            \
    expand_rows<L, V><<<(unsigned)g_, kThreads, 0, s>>>(batch, width, pos_row, idx_map,  \
                                                        recv_slot, recv_val, embedding, dst); \
  } while (0)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}
