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

// One half of the row expansion of a single-rank table: only the positions whose key is (in_prev != 0) or is not
// (in_prev == 0) among the unique keys of the previous batch.  The gradients of the previous batch change exactly the
// rows of those keys, so the "is not" half can run before they are applied - while they are still on their way from
// host memory - and the "is" half after.  prev_uniq is ascending (single owner); every lane of a group searches it
// for the same key, which the hardware serves as one broadcast access per step.
template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) expand_rows_subset(size_t batch, size_t width, const int32_t *__restrict__ pos_row,
                                                               const long long *__restrict__ keys,
                                                               const long long *__restrict__ prev_uniq,
                                                               const u32 *__restrict__ prev_meta, int in_prev,
                                                               const float *__restrict__ embedding,
                                                               float *__restrict__ dst) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  const size_t groups = ((size_t)gridDim.x * kThreads) / LANES;
  const unsigned gl = threadIdx.x % LANES;
  const size_t E = R::elems(width);
  const size_t U = prev_meta[HCTR_META_UNIQUE];
  for (size_t i0 = (((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES) * kExpandRows; i0 < batch;
       i0 += groups * kExpandRows) {
    const T *src[kExpandRows];
    bool mine[kExpandRows];
#pragma unroll
    for (int k = 0; k < kExpandRows; k++) {
      src[k] = nullptr;
      mine[k] = false;
      const size_t i = i0 + k;
      if (i < batch) {
        const long long key = keys[i];
        size_t lo = 0, hi = U;  // first entry >= key
        while (lo < hi) {
          const size_t mid = (lo + hi) >> 1;
          if (prev_uniq[mid] < key) lo = mid + 1;
          else hi = mid;
        }
        const bool found = lo < U && prev_uniq[lo] == key;
        mine[k] = found == (in_prev != 0);
        const int32_t row = pos_row[i];  // < 0: key was out of range (the host reports it); write zeros
        if (mine[k] && row >= 0) src[k] = reinterpret_cast<const T *>(embedding) + (size_t)row * E;
      }
    }
    for (size_t c = gl; c < E; c += LANES) {
      T v[kExpandRows];
#pragma unroll
      for (int k = 0; k < kExpandRows; k++) v[k] = src[k] ? src[k][c] : R::zero();
#pragma unroll
      for (int k = 0; k < kExpandRows; k++)
        if (mine[k]) R::st_once(reinterpret_cast<T *>(dst) + (i0 + k) * E + c, v[k]);
    }
  }
}


// ---- expand through the bulk-copy engine ---------------------------------------------------------------
// Each lane moves whole rows with two asynchronous bulk copies (cp.async.bulk): table (or receive-buffer) row ->
// shared memory, completion counted on the warp's mbarrier, then shared memory -> dst.  A warp owns two buffers
// of `rows_per_round` row slots and loads round r+1 while round r is being stored, so tens of row transfers per
// warp are in flight without occupying registers or issue slots.  Waits on the mbarrier are bounded; when one
// runs out the kernel records HCTR_ERR_TIMEOUT, drains its own copies and returns.
constexpr int kBulkWarps = 4;
constexpr unsigned kBulkBufBytes = 8192;  // per warp and buffer

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
  for (int tries = 0; tries < (1 << 22); tries++) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

__global__ void __launch_bounds__(kBulkWarps * 32) expand_rows_bulk(size_t batch, unsigned row_bytes,
                                                                    unsigned rows_per_round,
                                                                    const int32_t *__restrict__ pos_row,
                                                                    const int32_t *__restrict__ idx_map,
                                                                    const u32 *__restrict__ recv_slot,
                                                                    const float *__restrict__ recv_val,
                                                                    const float *__restrict__ embedding,
                                                                    float *__restrict__ dst, u32 *__restrict__ err) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  __shared__ __align__(8) unsigned long long bars[kBulkWarps][2];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned char *my_buf = bulk_smem + (size_t)warp * 2 * kBulkBufBytes;
  const unsigned bar0 = smem_u32(&bars[warp][0]), bar1 = smem_u32(&bars[warp][1]);
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 32;" ::"r"(bar0) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 32;" ::"r"(bar1) : "memory");
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncwarp();

  const size_t n_warps = (size_t)gridDim.x * kBulkWarps;
  const size_t gwarp = (size_t)blockIdx.x * kBulkWarps + warp;
  const size_t stride = n_warps * rows_per_round;
  const bool active = lane < rows_per_round;
  const size_t row_elems = row_bytes / sizeof(float);

  // issue the loads of the round that starts at position i0 into buffer b (all lanes arrive on its barrier)
  auto load_round = [&](size_t i0, unsigned b) {
    const size_t i = i0 + lane;
    const float *src = nullptr;
    bool zero_fill = false;
    if (active && i < batch) {
      const int32_t row = pos_row[i];
      if (row >= 0) {
        src = embedding + (size_t)row * row_elems;
      } else {
        const int32_t u = idx_map[i];  // < 0: key was out of range (the host reports it); write zeros
        if (u >= 0 && recv_slot) src = recv_val + (size_t)recv_slot[u] * row_elems;
        else zero_fill = true;
      }
    }
    unsigned char *slot = my_buf + (size_t)b * kBulkBufBytes + (size_t)lane * row_bytes;
    const unsigned bar = b ? bar1 : bar0;
    if (src) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(row_bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       smem_u32(slot)),
                   "l"(src), "r"(row_bytes), "r"(bar)
                   : "memory");
    } else {
      if (zero_fill) {
        for (unsigned o = 0; o < row_bytes; o += 16) *reinterpret_cast<float4 *>(slot + o) = make_float4(0.f, 0.f, 0.f, 0.f);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the bulk store
      }
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
    }
  };

  size_t i0 = gwarp * rows_per_round;
  unsigned parity0 = 0, parity1 = 0, b = 0;
  bool failed = false;
  if (i0 < batch) load_round(i0, 0);
  for (; i0 < batch; i0 += stride, b ^= 1) {
    const size_t next = i0 + stride;
    if (next < batch) {
      // the other buffer was the source of the stores of the previous round: they must have read it
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      __syncwarp();
      load_round(next, b ^ 1);
    }
    const bool ok = mbar_wait(b ? bar1 : bar0, b ? parity1 : parity0);
    if (b) parity1 ^= 1;
    else parity0 ^= 1;
    if (!__all_sync(0xffffffffu, ok)) {
      failed = true;
      break;
    }
    const size_t i = i0 + lane;
    if (active && i < batch) {
      const unsigned char *slot = my_buf + (size_t)b * kBulkBufBytes + (size_t)lane * row_bytes;
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + i * row_elems),
                   "r"(smem_u32(slot)), "r"(row_bytes)
                   : "memory");
    }
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (failed) {
    if (lane == 0) atomicOr(err, HCTR_ERR_TIMEOUT);
    // loads of the round issued last may still be in flight into this block's shared memory: give them a bounded
    // chance to land before the block (and its shared memory) goes away
    mbar_wait(b ? bar0 : bar1, b ? parity0 : parity1);
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

extern "C" int hctr_expand_rows_bulk(size_t batch, size_t width, const int32_t *pos_row, const int32_t *idx_map,
                                     const uint32_t *recv_slot, const float *recv_val, const float *embedding,
                                     float *dst, uint32_t *err, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (batch == 0) return 0;
  const size_t row_bytes = width * sizeof(float);
  const bool al = host_aligned16(recv_val) && host_aligned16(embedding) && host_aligned16(dst);
  if (!al || width % 4 != 0 || row_bytes < 128 || row_bytes > kBulkBufBytes / 2 || err == nullptr)
    return hctr_expand_rows(batch, width, pos_row, idx_map, recv_slot, recv_val, embedding, dst, stream);
  unsigned rows_per_round = (unsigned)(kBulkBufBytes / row_bytes);
  if (rows_per_round > 32) rows_per_round = 32;
  const size_t smem = (size_t)kBulkWarps * 2 * kBulkBufBytes;  // 64 KB
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(expand_rows_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const size_t rounds = (batch + rows_per_round - 1) / rows_per_round;
  size_t ctas = (rounds + kBulkWarps - 1) / kBulkWarps;
  const size_t cap = (size_t)kSMs * 3;  // 3 blocks of 64 KB per SM
  if (ctas > cap) ctas = cap;
  expand_rows_bulk<<<(unsigned)ctas, kBulkWarps * 32, smem, s>>>(batch, (unsigned)row_bytes, rows_per_round, pos_row,
                                                                idx_map, recv_slot, recv_val, embedding, dst, err);
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

extern "C" int hctr_expand_rows_subset(size_t batch, size_t width, const int32_t *pos_row, const int64_t *keys,
                                       const int64_t *prev_uniq, const uint32_t *prev_meta, int in_prev,
                                       const float *embedding, float *dst, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (batch == 0) return 0;
  const bool al = host_aligned16(embedding) && host_aligned16(dst);
#define CALL(L, V)                                                                       \
  do {                                                                                   \
    size_t g_ = (((size_t)batch + kExpandRows - 1) / kExpandRows * L + kThreads - 1) / kThreads; \
    const size_t cap_ = (size_t)kSMs * 3;                                                \
    if (g_ > cap_) g_ = cap_;                                                            \
    expand_rows_subset<L, V><<<(unsigned)g_, kThreads, 0, s>>>(                          \
        batch, width, pos_row, (const long long *)keys, (const long long *)prev_uniq, prev_meta, in_prev, embedding, dst); \
  } while (0)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}
