// Gradient side of a step: push decision, duplicate-gradient reduction fused with the local SGD
// apply and the packing of pushed rows, and the owner-side apply of received rows.
#include "rowops.cuh"

namespace hctr {

constexpr int kThreads = 256;

// ---- push decision ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) push_decide(const u32 *__restrict__ meta, int rank,
                                                        const uint8_t *__restrict__ uniq_owner,
                                                        const int32_t *__restrict__ uniq_row,
                                                        const u32 *__restrict__ cnt,
                                                        const long long *__restrict__ pending_cnt,
                                                        long long push_bound, u32 *__restrict__ need_push) {
  const size_t u = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (u >= meta[HCTR_META_UNIQUE]) return;
  u32 need;
  const int32_t row = uniq_row[u];
  if (uniq_owner[u] == rank) need = 0;
  else if (row < 0) need = 1;
  else need = (pending_cnt[row] + (long long)cnt[u] <= push_bound) ? 0u : 1u;
  need_push[u] = need;
}

__global__ void push_counts(const u32 *__restrict__ meta, int nrank, const u32 *__restrict__ push_slot,
                            u32 *__restrict__ push_count) {
  const int p = threadIdx.x;
  if (p < nrank) {
    const u32 *seg = meta + HCTR_META_SEG;
    push_count[p] = push_slot[seg[p + 1]] - push_slot[seg[p]];
  }
}

// ---- reduce + apply + pack -------------------------------------------------------------------
// One group of LANES lanes per unique key of the previous batch.  The duplicate sum runs over the
// key's positions in ascending batch order, then one multiply by -lr: the reference's order of
// operations (csrc/core/generate_query.cu:34-40), so single-rank results are bit-identical.
template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) grad_reduce_apply_pack(hctr_reduce_args a) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  const size_t gid = ((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES;
  const unsigned gl = threadIdx.x % LANES;
  if (gid >= a.n_unique) return;
  const size_t u = gid;
  const int32_t row = a.uniq_row[u];
  const bool need = a.need_push ? a.need_push[u] != 0 : false;
  int type;
  if (row < 0) type = 0;                           // not stored: push the batch sum
  else if ((size_t)row >= a.n_cached) type = 1;    // owned: apply
  else type = need ? 2 : 3;                        // cached: apply + accumulate (+ push and clear)
  const u32 l = a.run_start[u], r = a.run_start[u + 1];
  const size_t slot = need ? a.push_slot[u] : 0;

  if (gl == 0) {
    long long c = (long long)(r - l);
    if (type == 1) a.version[row] = (long long)((u64)a.version[row] + (u64)c);
    else if (type >= 2) {
      long long pc = a.pending_cnt[row] + c;
      if (type == 2) {
        c = pc;
        pc = 0;
        a.version[row] = (long long)((u64)a.version[row] + (u64)c);
      }
      a.pending_cnt[row] = pc;
    }
    if (need) {
      a.push_key[slot] = a.uniq[u];
      a.push_updates[slot] = c;
    }
  }

  const size_t E = R::elems(a.width);
  const T *grad = reinterpret_cast<const T *>(a.grad);
  T *emb = reinterpret_cast<T *>(a.embedding) + (row >= 0 ? (size_t)row * E : 0);
  T *pend = reinterpret_cast<T *>(a.pending) + (type >= 2 ? (size_t)row * E : 0);
  T *out = reinterpret_cast<T *>(a.push_val) + slot * E;
  for (size_t c = gl; c < E; c += LANES) {
    T sum = R::zero();
    u32 j = l;
    // 4 independent loads in flight per lane; adds stay in position order
    for (; j + 4 <= r; j += 4) {
      const T g0 = R::ld_once(grad + (size_t)a.sorted_pos[j] * E + c);
      const T g1 = R::ld_once(grad + (size_t)a.sorted_pos[j + 1] * E + c);
      const T g2 = R::ld_once(grad + (size_t)a.sorted_pos[j + 2] * E + c);
      const T g3 = R::ld_once(grad + (size_t)a.sorted_pos[j + 3] * E + c);
      sum = R::add(R::add(R::add(R::add(sum, g0), g1), g2), g3);
    }
    for (; j < r; j++) sum = R::add(sum, R::ld_once(grad + (size_t)a.sorted_pos[j] * E + c));
    sum = R::scale(sum, a.neg_lr);
    if (type == 0) {
      out[c] = sum;
    } else {
      emb[c] = R::add(emb[c], sum);
      if (type >= 2) {
        const T p = R::add(pend[c], sum);
        if (type == 2) {
          out[c] = p;
          pend[c] = R::zero();
        } else {
          pend[c] = p;
        }
      }
    }
  }
}

// ---- owner-side apply of one source's rows -----------------------------------------------------
template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) owner_update(size_t n_rows, size_t width, const long long *__restrict__ key,
                                                         const long long *__restrict__ updates,
                                                         const float *__restrict__ val,
                                                         const int32_t *__restrict__ row_of, size_t length,
                                                         size_t n_cached, float *__restrict__ embedding,
                                                         long long *__restrict__ version, u32 *err) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  const size_t m = ((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES;
  const unsigned gl = threadIdx.x % LANES;
  if (m >= n_rows) return;
  const long long k = key[m];
  int32_t row = -1;
  if (k >= 0 && (size_t)k < length) row = row_of[k];
  if (row < 0 || (size_t)row < n_cached) {  // only an owner may receive pushes for a key
    if (gl == 0) atomicOr(err, HCTR_ERR_NOT_OWNER);
    return;
  }
  if (gl == 0) version[row] = (long long)((u64)version[row] + (u64)updates[m]);
  const size_t E = R::elems(width);
  T *emb = reinterpret_cast<T *>(embedding) + (size_t)row * E;
  const T *v = reinterpret_cast<const T *>(val) + m * E;
  for (size_t c = gl; c < E; c += LANES) emb[c] = R::add(emb[c], R::ld_once(v + c));
}

}  // namespace hctr

using namespace hctr;

extern "C" int hctr_push_decide(const uint32_t *meta, int nrank, int rank, size_t u_max,
                                const uint8_t *uniq_owner, const int32_t *uniq_row, const uint32_t *cnt,
                                const int64_t *pending_cnt, int64_t push_bound, uint32_t *need_push,
                                uint32_t *push_slot, uint32_t *scan_scratch, uint32_t *push_count,
                                void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (nrank > 1024) return (int)cudaErrorInvalidValue;
  push_decide<<<grid_for(u_max, kThreads), kThreads, 0, s>>>(meta, rank, uniq_owner, uniq_row, cnt,
                                                              (const long long *)pending_cnt, push_bound,
                                                              need_push);
  int rc = hctr_scan_exclusive_u32(need_push, push_slot, u_max, meta + HCTR_META_UNIQUE, scan_scratch, stream);
  if (rc) return rc;
  push_counts<<<1, 1024, 0, s>>>(meta, nrank, push_slot, push_count);
  count_launches(2);
  return launch_status();
}

extern "C" int hctr_grad_reduce_apply_pack(const hctr_reduce_args *ap, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const hctr_reduce_args a = *ap;
  if (a.n_unique == 0) return 0;
  const bool al = host_aligned16(a.grad) && host_aligned16(a.embedding) && host_aligned16(a.pending) &&
                  host_aligned16(a.push_val);
#define CALL(L, V) \
  grad_reduce_apply_pack<L, V><<<grid_for(a.n_unique * L, kThreads), kThreads, 0, s>>>(a)
  HCTR_DISPATCH_ROWS(a.width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_owner_update(size_t n_rows, size_t width, const int64_t *key, const int64_t *updates,
                                 const float *val, const int32_t *row_of, size_t length, size_t n_cached,
                                 float *embedding, int64_t *version, uint32_t *err, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (n_rows == 0) return 0;
  const bool al = host_aligned16(val) && host_aligned16(embedding);
#define CALL(L, V)                                                                                    \
  owner_update<L, V><<<grid_for(n_rows * L, kThreads), kThreads, 0, s>>>(                             \
      n_rows, width, (const long long *)key, (const long long *)updates, val, row_of, length, n_cached, \
      embedding, (long long *)version, err)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}
