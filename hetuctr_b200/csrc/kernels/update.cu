// Gradient side of a step: push decision, duplicate-gradient reduction fused with the local SGD
// apply and the packing of pushed rows, and the owner-side apply of received rows.
#include <cooperative_groups.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "p2p.cuh"
#include "rowops.cuh"

namespace hctr {

constexpr int kThreads = 256;

// ---- push decision ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) push_decide(const u32 *__restrict__ meta, int rank,
                                                        const uint8_t *__restrict__ uniq_owner,
                                                        const int32_t *__restrict__ uniq_row,
                                                        const u32 *__restrict__ run_start,
                                                        const long long *__restrict__ pending_cnt,
                                                        long long push_bound, u32 *__restrict__ need_push) {
  const size_t u = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (u >= meta[HCTR_META_UNIQUE]) return;
  u32 need;
  const int32_t row = uniq_row[u];
  if (uniq_owner[u] == rank) need = 0;
  else if (row < 0) need = 1;
  else need = (pending_cnt[row] + (long long)(run_start[u + 1] - run_start[u]) <= push_bound) ? 0u : 1u;
  need_push[u] = need;
}

// Decision + slot assignment in one launch: every CTA decides a tile of 4096 unique keys, scans the flags
// locally and chains the tile totals (chained_cta_prefix), so need_push[] and push_slot[] (U+1 entries)
// come out of a single kernel.
constexpr int kDecideThreads = 1024;
constexpr int kDecideItems = 4;

__global__ void __launch_bounds__(kDecideThreads) push_decide_scan(const u32 *__restrict__ meta, int rank,
                                                                   const uint8_t *__restrict__ uniq_owner,
                                                                   const int32_t *__restrict__ uniq_row,
                                                                   const u32 *__restrict__ run_start,
                                                                   const long long *__restrict__ pending_cnt,
                                                                   long long push_bound, u32 *__restrict__ need_push,
                                                                   u32 *__restrict__ push_slot, u64 *agg, u32 epoch,
                                                                   u32 *err) {
  __shared__ u32 warp_sums[32];
  const size_t U = meta[HCTR_META_UNIQUE];
  const size_t base = ((size_t)blockIdx.x * kDecideThreads + threadIdx.x) * kDecideItems;
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  u32 v[kDecideItems];
  u32 s = 0;
#pragma unroll
  for (int k = 0; k < kDecideItems; k++) {
    const size_t u = base + k;
    u32 need = 0;
    if (u < U) {
      const int32_t row = uniq_row[u];
      if (uniq_owner[u] == rank) need = 0;
      else if (row < 0) need = 1;
      else need = (pending_cnt[row] + (long long)(run_start[u + 1] - run_start[u]) <= push_bound) ? 0u : 1u;
      need_push[u] = need;
    }
    v[k] = need;
    s += need;
  }
  // block-wide exclusive scan of s
  u32 incl = s;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    u32 t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= (unsigned)d) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    u32 w = warp_sums[lane], wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      u32 t = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= (unsigned)d) wi += t;
    }
    warp_sums[lane] = wi - w;
  }
  __syncthreads();
  u32 ex = incl - s + warp_sums[warp];
  __shared__ u32 cta_total;
  if (threadIdx.x == kDecideThreads - 1) cta_total = ex + s;
  __syncthreads();
  ex += chained_cta_prefix(agg, epoch, blockIdx.x, cta_total, err);
#pragma unroll
  for (int k = 0; k < kDecideItems; k++) {
    if (base + k <= U) push_slot[base + k] = ex;  // entry U receives the total
    ex += v[k];
  }
}

__global__ void push_counts(const u32 *__restrict__ meta, int nrank, const u32 *__restrict__ push_slot,
                            u32 *__restrict__ push_count, u32 *__restrict__ push_base) {
  const int p = threadIdx.x;
  if (p < nrank) {
    const u32 *seg = meta + HCTR_META_SEG;
    push_count[p] = push_slot[seg[p + 1]] - push_slot[seg[p]];
    if (push_base) push_base[p] = push_slot[seg[p]];
  }
}

// ---- reduce + apply + pack -------------------------------------------------------------------
// For every unique key of the previous batch: s = (sum of its gradient rows, in ascending batch
// position) * (-lr), then the update its storage class asks for.  The sum order and the single
// multiply are the reference's (csrc/core/generate_query.cu:34-40), so results are bit-identical
// to a sequential evaluation.
//   type 0  not stored      -> push s
//   type 1  owned           -> emb += s, version += count
//   type 2  cached, push    -> emb += s, pending += s, push pending, clear it, version += pending count
//   type 3  cached, hold    -> emb += s, pending += s, pending count += count

// number of unique keys / of long runs of the batch: from the batch's meta words when the host passed them
__device__ __forceinline__ size_t unique_count(const hctr_reduce_args &a) {
  return a.meta ? (size_t)a.meta[HCTR_META_UNIQUE] : a.n_unique;
}

struct RowTarget {
  int type;
  size_t slot;
  int32_t row;
};

// Where a pushed row goes: the local send buffers, or (peer-to-peer routing) this rank's sub-region in
// the owner's mailbox.
struct PushDest {
  long long *key, *upd;
  float *val;
};

struct ReduceKernelArgs {
  hctr_reduce_args a;
  hctr_p2p_ctx p2p;  // valid when a.p2p != nullptr
};

__device__ __forceinline__ PushDest push_dest(const hctr_reduce_args &a, const hctr_p2p_ctx &c, size_t u,
                                              size_t slot) {
  PushDest d;
  if (a.p2p) {
    const unsigned p = a.uniq_owner[u];
    size_t j = slot - a.push_base[p];
    if (j >= c.cap) {  // cannot happen when every rank uses the same batch size; never write out of bounds
      atomicOr(c.err, HCTR_ERR_CAPACITY);
      j = 0;
    }
    const hctr_p2p_box b = c.box[p];
    const size_t idx = (size_t)c.rank * c.cap + j;
    d.key = reinterpret_cast<long long *>(b.pkey) + idx;
    d.upd = reinterpret_cast<long long *>(b.pupd) + idx;
    d.val = b.pval + idx * a.width;
  } else {
    d.key = reinterpret_cast<long long *>(a.push_key) + slot;
    d.upd = reinterpret_cast<long long *>(a.push_updates) + slot;
    d.val = a.push_val + slot * a.width;
  }
  return d;
}

// bookkeeping of one unique key (one thread): versions, pending counts, packed id + update count
__device__ __forceinline__ RowTarget reduce_bookkeeping(const hctr_reduce_args &a, const hctr_p2p_ctx &c, size_t u,
                                                        u32 count, bool lead, PushDest *dest) {
  RowTarget t;
  t.row = a.uniq_row[u];
  const bool need = a.need_push ? a.need_push[u] != 0 : false;
  if (t.row < 0) t.type = 0;
  else if ((size_t)t.row >= a.n_cached) t.type = 1;
  else t.type = need ? 2 : 3;
  t.slot = need ? a.push_slot[u] : 0;
  if (need) *dest = push_dest(a, c, u, t.slot);
  else dest->key = nullptr, dest->upd = nullptr, dest->val = nullptr;
  if (lead) {
    long long cnt = (long long)count;
    if (t.type == 1) a.version[t.row] = (long long)((u64)a.version[t.row] + (u64)cnt);
    else if (t.type >= 2) {
      long long pc = a.pending_cnt[t.row] + cnt;
      if (t.type == 2) {
        cnt = pc;
        pc = 0;
        a.version[t.row] = (long long)((u64)a.version[t.row] + (u64)cnt);
      }
      a.pending_cnt[t.row] = pc;
    }
    if (need) {
      *dest->key = a.uniq[u];
      *dest->upd = cnt;
    }
  }
  return t;
}

template <class R>
__device__ __forceinline__ void reduce_apply(const RowTarget &t, typename R::T sum, typename R::T *emb,
                                             typename R::T *pend, typename R::T *out, size_t c) {
  if (t.type == 0) {
    out[c] = sum;
  } else {
    emb[c] = R::add(emb[c], sum);
    if (t.type >= 2) {
      const typename R::T p = R::add(pend[c], sum);
      if (t.type == 2) {
        out[c] = p;
        pend[c] = R::zero();
      } else {
        pend[c] = p;
      }
    }
  }
}

// Short runs (<= HCTR_LIGHT_RUN positions): one group of LANES lanes per unique key.
template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) grad_reduce_short(ReduceKernelArgs ka) {
  const hctr_reduce_args &a = ka.a;
  typedef RowT<VEC> R;
  typedef typename R::T T;
  const size_t u = ((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES;
  const unsigned gl = threadIdx.x % LANES;
  if (u >= unique_count(a)) return;
  const u32 l = a.run_start[u], r = a.run_start[u + 1];
  if (r - l > HCTR_LIGHT_RUN) return;  // handled by grad_reduce_long
  PushDest dest;
  const RowTarget t = reduce_bookkeeping(a, ka.p2p, u, r - l, gl == 0, &dest);
  const size_t E = R::elems(a.width);
  const T *grad = reinterpret_cast<const T *>(a.grad);
  T *emb = reinterpret_cast<T *>(a.embedding) + (t.row >= 0 ? (size_t)t.row * E : 0);
  T *pend = reinterpret_cast<T *>(a.pending) + (t.type >= 2 ? (size_t)t.row * E : 0);
  T *out = reinterpret_cast<T *>(dest.val);
  for (size_t c = gl; c < E; c += LANES) {
    T sum = R::zero();
    u32 j = l;
    // the table row does not depend on the gradient chain: start its load first
    T e_old = R::zero(), p_old = R::zero();
    if (t.type != 0) e_old = emb[c];
    if (t.type >= 2) p_old = pend[c];
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
    if (t.type == 0) {
      out[c] = sum;
    } else {
      emb[c] = R::add(e_old, sum);
      if (t.type >= 2) {
        const T p = R::add(p_old, sum);
        if (t.type == 2) {
          out[c] = p;
          pend[c] = R::zero();
        } else {
          pend[c] = p;
        }
      }
    }
  }
}

// Short runs, rows of at least 32 float4 (width >= 128): a warp takes kWideChunk consecutive unique
// keys.  Run bounds, rows, push slots and first positions are fetched by the first lanes (one key per
// lane) and the per-key bookkeeping runs one key per lane; the warp then walks the keys, and while it
// sums and applies key k the first gradient row and the table row of the next key are already in
// flight.  The chunk is small so that a batch still yields enough warps to fill every SM.
constexpr unsigned kWideChunk = 8;
// (Capping registers to raise occupancy was measured: 48 registers / 5 CTAs per SM made the warm kernel
// slower, 84 us vs 71 us for the reduce phase, so the compiler keeps its 80.)
__global__ void __launch_bounds__(kThreads) grad_reduce_short_wide(ReduceKernelArgs ka) {
  const hctr_reduce_args &a = ka.a;
  typedef RowT<true> R;
  typedef float4 T;
  const unsigned lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const size_t n_warps = ((size_t)gridDim.x * kThreads) >> 5;
  const size_t E = a.width / 4;
  const T *grad = reinterpret_cast<const T *>(a.grad);
  T *emb_base = reinterpret_cast<T *>(a.embedding);
  T *pend_base = reinterpret_cast<T *>(a.pending);
  // (A one-wave grid with chunks drawn from a shared counter was measured and was slower: 105 us vs 92 us.)
  const size_t n_unique = unique_count(a);
  for (size_t u0 = warp * kWideChunk; u0 < n_unique; u0 += n_warps * kWideChunk) {
    const size_t my_u = u0 + lane;
    u32 l = 0, len = 0, p0 = 0;
    unsigned long long outp = 0;  // destination of this lane's key if it is pushed
    int row = 0, type = -1;       // type -1: nothing to do for this lane's key
    if (lane < kWideChunk && my_u < n_unique) {
      l = a.run_start[my_u];
      len = a.run_start[my_u + 1] - l;
      if (len > 0 && len <= HCTR_LIGHT_RUN) {
        p0 = a.sorted_pos[l];
        PushDest dest;
        const RowTarget t = reduce_bookkeeping(a, ka.p2p, my_u, len, true, &dest);
        row = t.row;
        type = t.type;
        outp = (unsigned long long)dest.val;
      }
    }
    unsigned todo = __ballot_sync(0xffffffffu, type >= 0);
    if (!todo) continue;
    // prefetch for the first key
    int k = __ffs(todo) - 1;
    todo &= todo - 1;
    T g_next, e_next;
    {
      const u32 pk = __shfl_sync(0xffffffffu, p0, k);
      const int rk = __shfl_sync(0xffffffffu, row, k), tk = __shfl_sync(0xffffffffu, type, k);
      g_next = R::ld_once(grad + (size_t)pk * E + lane);
      e_next = tk != 0 ? emb_base[(size_t)rk * E + lane] : R::zero();
    }
    while (k >= 0) {
      const u32 lk = __shfl_sync(0xffffffffu, l, k), lenk = __shfl_sync(0xffffffffu, len, k);
      const unsigned long long outk = __shfl_sync(0xffffffffu, outp, k);
      const int rowk = __shfl_sync(0xffffffffu, row, k), typek = __shfl_sync(0xffffffffu, type, k);
      const T g0 = g_next, e0 = e_next;
      const int kn = todo ? __ffs(todo) - 1 : -1;
      todo &= todo - 1;
      if (kn >= 0) {
        const u32 pk = __shfl_sync(0xffffffffu, p0, kn);
        const int rk = __shfl_sync(0xffffffffu, row, kn), tk = __shfl_sync(0xffffffffu, type, kn);
        g_next = R::ld_once(grad + (size_t)pk * E + lane);
        e_next = tk != 0 ? emb_base[(size_t)rk * E + lane] : R::zero();
      }
      T *emb = emb_base + (typek != 0 ? (size_t)rowk * E : 0);
      T *pend = pend_base + (typek >= 2 ? (size_t)rowk * E : 0);
      T *out = reinterpret_cast<T *>(outk);
      for (size_t c = lane; c < E; c += 32) {
        T sum, e_old;
        if (c == lane) {
          sum = R::add(R::zero(), g0);
          e_old = e0;
        } else {
          sum = R::add(R::zero(), R::ld_once(grad + (size_t)a.sorted_pos[lk] * E + c));
          e_old = typek != 0 ? emb[c] : R::zero();
        }
        u32 j = 1;
        for (; j + 4 <= lenk; j += 4) {
          const T g1 = R::ld_once(grad + (size_t)a.sorted_pos[lk + j] * E + c);
          const T g2 = R::ld_once(grad + (size_t)a.sorted_pos[lk + j + 1] * E + c);
          const T g3 = R::ld_once(grad + (size_t)a.sorted_pos[lk + j + 2] * E + c);
          const T g4 = R::ld_once(grad + (size_t)a.sorted_pos[lk + j + 3] * E + c);
          sum = R::add(R::add(R::add(R::add(sum, g1), g2), g3), g4);
        }
        for (; j < lenk; j++) sum = R::add(sum, R::ld_once(grad + (size_t)a.sorted_pos[lk + j] * E + c));
        sum = R::scale(sum, a.neg_lr);
        if (typek == 0) {
          out[c] = sum;
        } else {
          emb[c] = R::add(e_old, sum);
          if (typek >= 2) {
            const T p = R::add(pend[c], sum);
            if (typek == 2) {
              out[c] = p;
              pend[c] = R::zero();
            } else {
              pend[c] = p;
            }
          }
        }
      }
      k = kn;
    }
  }
}

// Work-balanced streaming variant of the kernel above (rows of 128..512 floats).
// Balance: a key costs (its gradient rows + 2) row transfers - the rows it sums plus the read and write of
// its table row - and cost(k) = run_start[k] + 2k, the cost of all keys before k, grows strictly with k.
// Warp w of n_warps takes the keys whose cost(k) falls into [w*T, (w+1)*T), T = ceil(cost(U) / n_warps): every
// warp moves about the same number of rows however the run lengths are distributed over the key space
// (small-vocabulary fields sit at the end of the unique list and have runs tens of times longer than the
// rest).  The two range ends are found with a 32-way search (one probe per lane).

// first k in [0, n_unique] with run_start[k] + 2k >= target; the caller guarantees cost(n_unique) >= target
__device__ __forceinline__ u32 first_key_at_cost(const u32 *__restrict__ run_start, u32 n_unique, u64 target,
                                                 unsigned lane) {
  u32 lo = 0, hi = n_unique;
  while (hi > lo) {
    const u32 span = hi - lo;
    const u32 step = (span + 30) / 31;  // 31 steps cover the span: the last lane always probes hi
    const u64 off = (u64)lane * step;
    const u32 probe = off >= span ? hi : lo + (u32)off;
    const bool ge = (u64)run_start[probe] + 2ull * probe >= target;
    const unsigned m = __ballot_sync(0xffffffffu, ge);  // monotone: true from some lane upwards (lane 31 is true)
    const int f = __ffs(m) - 1;
    const u32 new_hi = __shfl_sync(0xffffffffu, probe, f);
    const u32 below = __shfl_sync(0xffffffffu, probe, f > 0 ? f - 1 : 0);
    lo = f > 0 ? below + 1 : lo;
    hi = f > 0 ? new_hi : lo;
  }
  return lo;
}

// Streaming: the rows travel through shared memory.  Every warp owns a
// ring of D row slots; each lane copies its own 16-byte pieces of a row with cp.async (one commit group per
// row) and later reads back exactly those pieces, so no barrier is needed, and D-1 row transfers stay in
// flight per warp without holding them in registers.  The rows of a warp form one stream: for every key its
// table row (if it is stored here), then its gradient rows in batch order; the consumer adds them in that
// order, so the sums are the ones a sequential loop produces.
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
  const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
// Gradient rows are read exactly once: their copies carry an evict-first L2 policy so that 100+ MB of them per
// step do not push the table rows and the (L2-resident) dedupe structures of the concurrently running
// preprocess out of the cache.
__device__ __forceinline__ u64 l2_evict_first_policy() {
  u64 p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void cp_async16_once(void *smem, const void *gmem, u64 policy) {
  const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(sa), "l"(gmem), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct RowCursor {  // warp-uniform position in the row stream of one 32-key chunk
  unsigned mask;    // keys not yet started
  int k;            // lane that holds the current key, -1 = stream exhausted
  int j;            // -1 = the key's table row, 0..len-1 = its gradient rows
  u32 l, len;
  int type, row;
};

__device__ __forceinline__ void cursor_next_key(RowCursor &c, u32 l, u32 len, int type, int row) {
  c.k = c.mask ? __ffs(c.mask) - 1 : -1;
  c.mask &= c.mask - 1;
  if (c.k >= 0) {
    c.l = __shfl_sync(0xffffffffu, l, c.k);
    c.len = __shfl_sync(0xffffffffu, len, c.k);
    c.type = __shfl_sync(0xffffffffu, type, c.k);
    c.row = __shfl_sync(0xffffffffu, row, c.k);
    c.j = c.type != 0 ? -1 : 0;
  }
}

// EC: row size in float4 when known at compile time (32, 64 or 128 for rows of 128, 256 or 512 floats - the
// bounds checks and multiplications by the row size then fold away), 0: taken from the arguments.
template <int D, int EPL, int EC>
__global__ void __launch_bounds__(kThreads) grad_reduce_short_stream(ReduceKernelArgs ka) {
  extern __shared__ float4 ring_all[];
  const hctr_reduce_args &a = ka.a;
  typedef RowT<true> R;
  typedef float4 T;
  const unsigned lane = threadIdx.x & 31;
  // The warps of one thread block take shares that lie far apart in the key space: the shares that fall on long
  // runs (left to the long-run kernel) are empty, and they are neighbours, so consecutive shares per block
  // would leave whole blocks - and with them whole SMs - without work.
  const u64 warp = (u64)(threadIdx.x >> 5) * gridDim.x + blockIdx.x;
  const u64 n_warps = ((u64)gridDim.x * kThreads) >> 5;
  const size_t E = EC ? (size_t)EC : a.width / 4;
  const u32 U = (u32)unique_count(a);
  const T *grad = reinterpret_cast<const T *>(a.grad);
  T *emb_base = reinterpret_cast<T *>(a.embedding);
  T *pend_base = reinterpret_cast<T *>(a.pending);
  T *ring = ring_all + (size_t)(threadIdx.x >> 5) * D * E;
  __shared__ u32 sort_all[kThreads];  // 32 words per warp
  u32 *sort_buf = sort_all + (threadIdx.x & ~31u);
  const bool unordered = a.short_runs_unordered != 0;
  const u64 once = l2_evict_first_policy();
  const u32 n_pos = a.run_start[U];
  const u64 total = (u64)n_pos + 2ull * U;
  const u64 per_warp = (total + n_warps - 1) / n_warps;
  if (warp * per_warp >= total) return;
  const u32 k_lo = first_key_at_cost(a.run_start, U, warp * per_warp, lane);
  const u32 k_hi = (warp + 1) * per_warp >= total ? U : first_key_at_cost(a.run_start, U, (warp + 1) * per_warp, lane);
  for (u32 u0 = k_lo; u0 < k_hi; u0 += 32) {
    const u32 my_u = u0 + lane;
    u32 l = 0, len = 0;
    unsigned long long outp = 0;  // destination of this lane's key if it is pushed
    int row = 0, type = -1;       // type -1: nothing to do for this lane's key
    if (my_u < k_hi) {
      l = a.run_start[my_u];
      len = a.run_start[my_u + 1] - l;
      if (len > 0 && len <= HCTR_LIGHT_RUN) {
        PushDest dest;
        const RowTarget t = reduce_bookkeeping(a, ka.p2p, my_u, len, true, &dest);
        row = t.row;
        type = t.type;
        outp = (unsigned long long)dest.val;
      }
    }
    const unsigned todo = __ballot_sync(0xffffffffu, type >= 0);
    if (!todo) continue;
    RowCursor P, C;
    P.mask = C.mask = todo;
    cursor_next_key(P, l, len, type, row);
    cursor_next_key(C, l, len, type, row);
    // window of 32 batch positions, one per lane (the positions of consecutive keys are consecutive)
    u32 q_base = 0, sp = 0;
    bool have_window = false;
    int slot_p = 0, slot_c = 0;
    T sum[EPL], e_old[EPL];
#pragma unroll
    for (int i = 0; i < EPL; i++) sum[i] = R::zero(), e_old[i] = R::zero();

    auto issue = [&]() {  // copy the producer's current row into slot_p, then move the producer on
      if (P.k >= 0) {
        const T *src;
        if (P.j < 0) {
          src = emb_base + (size_t)P.row * E;
        } else {
          const u32 q = P.l + (u32)P.j;
          if (unordered && P.j == 0 && P.len >= 2) {
            // First gradient row of a key whose run is still in arrival order: bring the whole run (at most 32
            // positions) into the window, then put it in ascending order - a lane's place is the number of smaller
            // positions in the run (positions are distinct).  Sums stay in batch order without a separate pass.
            if (!have_window || q - q_base + P.len > 32u) {
              q_base = q;
              have_window = true;
              sp = q_base + lane < n_pos ? a.sorted_pos[q_base + lane] : 0u;
            }
            const u32 s0 = q - q_base;
            const bool in_run = lane - s0 < P.len;
            u32 place = 0;
            for (u32 k2 = 0; k2 < P.len; k2++) place += __shfl_sync(0xffffffffu, sp, (int)(s0 + k2)) < sp ? 1u : 0u;
            if (in_run) sort_buf[place] = sp;
            __syncwarp();
            if (in_run) sp = sort_buf[lane - s0];
            __syncwarp();
          }
          if (!have_window || q - q_base >= 32u) {
            q_base = q;
            have_window = true;
            sp = q_base + lane < n_pos ? a.sorted_pos[q_base + lane] : 0u;
          }
          const u32 pos = __shfl_sync(0xffffffffu, sp, (int)(q - q_base));
          src = grad + (size_t)pos * E;
        }
        T *dst = ring + (size_t)slot_p * E;
        const bool is_grad = P.j >= 0;  // a gradient row (read once), not the key's table row
#pragma unroll
        for (int i = 0; i < EPL; i++) {
          const size_t c = lane + 32u * i;
          if (c < E) {
            if (is_grad) cp_async16_once(dst + c, src + c, once);
            else cp_async16(dst + c, src + c);
          }
        }
        if (++P.j == (int)P.len) cursor_next_key(P, l, len, type, row);
      }
      cp_async_commit();
      slot_p = slot_p + 1 == D ? 0 : slot_p + 1;
    };

#pragma unroll
    for (int i = 0; i < D - 1; i++) issue();
    while (C.k >= 0) {
      issue();
      cp_async_wait<D - 1>();
      const T *src = ring + (size_t)slot_c * E;
      slot_c = slot_c + 1 == D ? 0 : slot_c + 1;
      if (C.j < 0) {
#pragma unroll
        for (int i = 0; i < EPL; i++) {
          const size_t c = lane + 32u * i;
          if (c < E) e_old[i] = src[c];
        }
      } else {
#pragma unroll
        for (int i = 0; i < EPL; i++) {
          const size_t c = lane + 32u * i;
          if (c < E) sum[i] = R::add(sum[i], src[c]);
        }
      }
      if (++C.j == (int)C.len) {
        // the key is complete: scale once, then the update its storage class asks for
        // (only a pushed key - not stored, or cached with its push due - has a destination to fetch)
        const unsigned long long outk = (C.type == 0 || C.type == 2) ? __shfl_sync(0xffffffffu, outp, C.k) : 0ull;
        T *emb = emb_base + (C.type != 0 ? (size_t)C.row * E : 0);
        T *pend = pend_base + (C.type >= 2 ? (size_t)C.row * E : 0);
        T *out = reinterpret_cast<T *>(outk);
#pragma unroll
        for (int i = 0; i < EPL; i++) {
          const size_t c = lane + 32u * i;
          if (c < E) {
            const T sc = R::scale(sum[i], a.neg_lr);
            if (C.type == 0) {
              out[c] = sc;
            } else {
              emb[c] = R::add(e_old[i], sc);
              if (C.type >= 2) {
                const T p = R::add(pend[c], sc);
                if (C.type == 2) {
                  out[c] = p;
                  pend[c] = R::zero();
                } else {
                  pend[c] = p;
                }
              }
            }
          }
          sum[i] = R::zero();
        }
        cursor_next_key(C, l, len, type, row);
      }
    }
    cp_async_wait<0>();
  }
}

// Long runs (hot keys, up to the whole batch): one CTA per key.  All threads stream the key's
// gradient rows into a ring of shared-memory stages with cp.async (16-byte copies, several stages in
// flight), and one thread per row element adds the staged rows in order.  The sequential sum of a
// 1000-row run becomes shared-memory-latency bound instead of DRAM-latency bound, without
// reassociating it.  CTAs take keys from a shared counter, so a CTA that drew short runs moves on.
constexpr int kLongThreads = 256;
constexpr int kLongWarps = kLongThreads / 32;
constexpr int kLongStages = 4;
constexpr int kLongStageBytes = 16 * 1024;
constexpr int kLongPosChunk = 2048;  // positions staged in shared memory at a time
constexpr u32 kVeryLongRun = 256;     // runs at least this long are started first

template <bool VEC>
__device__ __forceinline__ void cp_async_elem(void *smem_dst, const void *gsrc, u64 policy) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  if (VEC)
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gsrc), "l"(policy)
                 : "memory");
  else
    asm volatile("cp.async.ca.shared.global.L2::cache_hint [%0], [%1], 4, %2;\n" ::"r"(s), "l"(gsrc), "l"(policy)
                 : "memory");
}

template <bool VEC>
__global__ void __launch_bounds__(kLongThreads) grad_reduce_long(ReduceKernelArgs ka, u32 n_heavy_host, u32 *work_counter) {
  const hctr_reduce_args &a = ka.a;
  const u32 n_heavy = a.meta ? a.meta[HCTR_META_NHEAVY] : n_heavy_host;
  const u64 once = l2_evict_first_policy();
  typedef RowT<VEC> R;
  typedef typename R::T T;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ u32 pos_s[kLongPosChunk];
  __shared__ u32 next_item;
  const size_t E = R::elems(a.width);  // T elements per row
  const size_t W = a.width;            // floats per row
  const u32 rows_per_stage = (u32)max((size_t)1, (size_t)kLongStageBytes / (W * sizeof(float)));
  const size_t stage_elems = (size_t)rows_per_stage * E;
  const size_t stage_floats = (size_t)rows_per_stage * W;
  T *stage = reinterpret_cast<T *>(smem_raw);
  const float *stage_f = reinterpret_cast<const float *>(smem_raw);
  const T *grad = reinterpret_cast<const T *>(a.grad);
  const unsigned tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // lanes per row for the copies: a power of two <= 32 covering the row when it is narrow
  unsigned lpr = 32;
  while (lpr > 1 && (size_t)(lpr / 2) >= E) lpr /= 2;
  const unsigned rows_per_warp_iter = 32 / lpr, sub = lane / lpr, sl = lane % lpr;

  // two passes over the list: the longest runs bound the kernel's duration, so they start first
  for (int pass = 0; pass < 2;) {
    __syncthreads();
    if (tid == 0) next_item = atomicAdd(work_counter + pass, 1u);
    __syncthreads();
    const u32 h = next_item;
    if (h >= n_heavy) {
      pass++;
      continue;
    }
    const size_t u = a.heavy_list[h];
    const u32 l = a.run_start[u], len = a.run_start[u + 1] - l;
    if ((len >= kVeryLongRun) != (pass == 0)) continue;
    PushDest dest;
    const RowTarget t = reduce_bookkeeping(a, ka.p2p, u, len, tid == 0, &dest);
    // columns are processed in slabs of up to 4 per thread (width <= 1024 needs a single pass)
    for (size_t col0 = 0; col0 < W; col0 += 4 * kLongThreads) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (u32 p0 = 0; p0 < len; p0 += kLongPosChunk) {
        const u32 plen = min((u32)kLongPosChunk, len - p0);
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();  // previous chunk fully consumed before its positions and stages are reused
        for (u32 k = tid; k < plen; k += kLongThreads) pos_s[k] = a.sorted_pos[l + p0 + k];
        __syncthreads();
        const u32 n_tiles = (plen + rows_per_stage - 1) / rows_per_stage;
        const u32 E32 = (u32)E, W32 = (u32)W;
        auto issue = [&](u32 tile) {
          if (tile < n_tiles) {
            const u32 r0 = tile * rows_per_stage;
            const u32 nr = min(rows_per_stage, plen - r0);
            T *dst = stage + (size_t)(tile % kLongStages) * stage_elems;
            for (u32 rr = warp * rows_per_warp_iter + sub; rr < nr; rr += kLongWarps * rows_per_warp_iter) {
              const T *src = grad + (size_t)pos_s[r0 + rr] * E;
              T *d = dst + rr * E32;
              for (u32 cc = sl; cc < E32; cc += lpr) cp_async_elem<VEC>(d + cc, src + cc, once);
            }
          }
          asm volatile("cp.async.commit_group;\n" ::: "memory");  // one group per tile slot, even if empty
        };
        for (int p = 0; p < kLongStages - 1; p++) issue(p);
        for (u32 tile = 0; tile < n_tiles; tile++) {
          // groups in flight: tiles tile .. tile+S-2; all but the newest S-2 done => this tile landed
          asm volatile("cp.async.wait_group %0;\n" ::"n"(kLongStages - 2) : "memory");
          // one barrier per tile: every thread's copies of this tile are visible, and every thread has
          // finished adding the previous tile, whose stage the next issue overwrites
          __syncthreads();
          issue(tile + kLongStages - 1);
          const u32 nr = min(rows_per_stage, plen - tile * rows_per_stage);
          const float *src = stage_f + (size_t)(tile % kLongStages) * stage_floats;
#pragma unroll
          for (int k = 0; k < 4; k++) {
            const u32 col = (u32)col0 + tid + (u32)k * kLongThreads;
            if (col < W32) {
              const float *sc = src + col;
              float sacc = acc[k];
              u32 rr = 0;
              for (; rr + 8 <= nr; rr += 8) {
                float v[8];
#pragma unroll
                for (int q = 0; q < 8; q++) v[q] = sc[(rr + q) * W32];
#pragma unroll
                for (int q = 0; q < 8; q++) sacc = __fadd_rn(sacc, v[q]);
              }
              for (; rr < nr; rr++) sacc = __fadd_rn(sacc, sc[rr * W32]);
              acc[k] = sacc;
            }
          }
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      }
      float *emb = a.embedding + (t.row >= 0 ? (size_t)t.row * W : 0);
      float *pend = a.pending + (t.type >= 2 ? (size_t)t.row * W : 0);
      float *out = dest.val;
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const size_t col = col0 + tid + (size_t)k * kLongThreads;
        if (col < W) reduce_apply<RowT<false>>(t, __fmul_rn(acc[k], a.neg_lr), emb, pend, out, col);
      }
    }
  }
}

// ---- owner-side apply of one source's rows -----------------------------------------------------
template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) owner_update(size_t n_rows_max, const u32 *__restrict__ n_rows_dev, size_t width,
                                                         const long long *__restrict__ key,
                                                         const long long *__restrict__ updates,
                                                         const float *__restrict__ val,
                                                         const int32_t *__restrict__ row_of, size_t length,
                                                         size_t n_cached, float *__restrict__ embedding,
                                                         long long *__restrict__ version, u32 *err) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  const unsigned gl = threadIdx.x % LANES;
  const size_t groups = ((size_t)gridDim.x * kThreads) / LANES;
  const size_t n_rows = n_rows_dev ? min((size_t)*n_rows_dev, n_rows_max) : n_rows_max;
  const size_t E = R::elems(width);
  for (size_t m = ((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES; m < n_rows; m += groups) {
    const long long k = key[m];
    int32_t row = -1;
    if (k >= 0 && (size_t)k < length) row = row_of[k];
    if (row < 0 || (size_t)row < n_cached) {  // only an owner may receive pushes for a key
      if (gl == 0) atomicOr(err, HCTR_ERR_NOT_OWNER);
      continue;
    }
    if (gl == 0) version[row] = (long long)((u64)version[row] + (u64)updates[m]);
    T *emb = reinterpret_cast<T *>(embedding) + (size_t)row * E;
    const T *v = reinterpret_cast<const T *>(val) + m * E;
    for (size_t c = gl; c < E; c += LANES) emb[c] = R::add(emb[c], R::ld_once(v + c));
  }
}

// ---- owner-side apply of all sources, order-preserving, two launches ------------------------------
// The reference applies the sources one after the other because two sources may push the same row
// and fp32 adds must happen in a fixed order.  Here pass A (mark) records, per owned row, WHICH sources push it
// (one bit per source) and adds every entry's update count to the row's version - integer adds commute, so the
// versions are final after pass A and the owner's staleness test can start while pass B still moves rows.  Pass B
// (apply) lets the lowest source of each row add every contribution to the row in ascending source order.  Each
// source's list is sorted by key (it is a slice of that source's unique list), so the other sources' entries are
// found by binary search, all of them at once: one lane of the row's lane group per source.  Same arithmetic
// and order as source-by-source launches, hence bit-identical.
// A mask word is [epoch:32 | source bits:32]; bits under an older epoch count as empty, so nothing has to be
// cleared between steps (clearing inside pass B would race with the readers of the same word).
struct PushLists {  // where every source's pushed rows are, as seen by the owner
  const long long *key;
  const long long *upd;
  const float *val;
  const unsigned long long *src_off;  // device [nsrc]: first entry of source s in key/upd/val; null: s * src_stride
  size_t src_stride;
  const u32 *flat_start;              // device [nsrc+1]: exclusive prefix of the per-source row counts
  int nsrc;
  // chain of the entries that push the same row, built by pass A and walked by pass B: head[row] =
  // [epoch:32 | flat entry:32] of the entry marked last, next[f] = the entry marked before f (kNoEntry: none)
  u64 *head;
  u32 *next;
};
constexpr u32 kNoEntry = 0xffffffffu;

__device__ __forceinline__ size_t push_list_base(const PushLists &p, int s) {
  return p.src_off ? (size_t)p.src_off[s] : (size_t)s * p.src_stride;
}

__device__ __forceinline__ int32_t owned_row(const int32_t *row_of, size_t length, size_t n_cached, long long k) {
  int32_t row = -1;
  if (k >= 0 && (size_t)k < length) row = row_of[k];
  return (row < 0 || (size_t)row < n_cached) ? -1 : row;
}

// Pass A.  ent_row[f] = owned row of flat entry f, or -1 (reported through err).  With WAIT the kernel first waits
// (bounded) for the peers' counts of this step (peer-to-peer exchange: the lists are the sub-regions of this rank's
// mailbox) and block 0 records them for the kernels that follow.
template <bool WAIT>
__global__ void __launch_bounds__(kThreads) owner_mark_sources(PushLists p, hctr_p2p_ctx c, u32 seq,
                                                               const int32_t *__restrict__ row_of, size_t length,
                                                               size_t n_cached, u64 *__restrict__ mask, u32 epoch,
                                                               int32_t *__restrict__ ent_row,
                                                               long long *__restrict__ version, u32 *err) {
  __shared__ u32 start[kMaxRanks + 1];
  if (WAIT) {
    __shared__ u32 qstart[kMaxRanks + 1];
    wait_queries(c, seq, qstart, start, blockIdx.x == 0);
  } else {
    for (int i = threadIdx.x; i <= p.nsrc; i += kThreads) start[i] = p.flat_start[i];
    __syncthreads();
  }
  const u32 total = start[p.nsrc];
  for (size_t f = (size_t)blockIdx.x * kThreads + threadIdx.x; f < total; f += (size_t)gridDim.x * kThreads) {
    const int s = (int)segment_of(start, p.nsrc, (u32)f);
    const size_t ent = push_list_base(p, s) + (f - start[s]);
    const long long k = p.key[ent];
    const int32_t row = owned_row(row_of, length, n_cached, k);
    ent_row[f] = row;
    if (row < 0) {
      atomicOr(err, HCTR_ERR_NOT_OWNER);
      continue;
    }
    atomicAdd(reinterpret_cast<u64 *>(version) + row, (u64)p.upd[ent]);
    const u64 before = atomicExch(&p.head[(size_t)row - n_cached], ((u64)epoch << 32) | (u32)f);
    p.next[f] = (u32)(before >> 32) == epoch ? (u32)before : kNoEntry;
    u64 *w = &mask[(size_t)row - n_cached];
    u64 old = *w;
    for (;;) {  // terminates: at most nsrc writers per word, each CAS failure means another one got through
      const u64 want = ((u32)(old >> 32) == epoch ? old : ((u64)epoch << 32)) | (1ull << s);
      const u64 seen = atomicCAS(w, old, want);
      if (seen == old) break;
      old = seen;
    }
  }
}

// entry of key k in source s2's key-sorted list
__device__ __forceinline__ size_t push_entry_of(const PushLists &p, const u32 *start, int s2, long long k) {
  const size_t off2 = push_list_base(p, s2);
  size_t lo = 0, hi = start[s2 + 1] - start[s2];
  while (lo < hi) {
    const size_t mid = (lo + hi) >> 1;
    if (p.key[off2 + mid] < k) lo = mid + 1;
    else hi = mid;
  }
  return off2 + lo;
}

// Pass B.  One group of LANES lanes per pushed entry; the group of a row's lowest source adds all contributions.
template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) owner_apply_sources(PushLists p, size_t width, size_t n_cached,
                                                                const int32_t *__restrict__ ent_row,
                                                                const u64 *__restrict__ mask,
                                                                float *__restrict__ embedding) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  __shared__ u32 start[33];
  if (threadIdx.x <= (unsigned)p.nsrc) start[threadIdx.x] = p.flat_start[threadIdx.x];
  __syncthreads();
  const u32 total = start[p.nsrc];
  const unsigned gl = threadIdx.x % LANES;
  // lanes of this group inside its warp, for the shuffles
  const unsigned gmask = LANES == 32 ? 0xffffffffu : ((1u << LANES) - 1u) << ((threadIdx.x & 31u) / LANES * LANES);
  const size_t groups = ((size_t)gridDim.x * kThreads) / LANES;
  const size_t E = R::elems(width);
  const T *val = reinterpret_cast<const T *>(p.val);
  for (size_t f = ((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES; f < total; f += groups) {
    const int32_t row = ent_row[f];
    if (row < 0) continue;  // not owned here: reported by pass A
    const int s = (int)segment_of(start, p.nsrc, (u32)f);
    const u32 mk = (u32)mask[(size_t)row - n_cached];  // this step's epoch, set by pass A
    if (mk & ((1u << s) - 1u)) continue;                // a lower source pushes this row too: it applies everything
    u32 rest = mk & ~((2u << s) - 1u);                  // higher sources that also push it
    const size_t ent = push_list_base(p, s) + (f - start[s]);
    T *emb = reinterpret_cast<T *>(embedding) + (size_t)row * E;
    if (rest == 0) {
      for (size_t e = gl; e < E; e += LANES) emb[e] = R::add(emb[e], R::ld_once(val + ent * E + e));
      continue;
    }
    const int others = __popc(rest);
    if (others < LANES) {
      // Walk the row's chain (all of its entries, this one included, in the order pass A happened to mark them):
      // lane i keeps the i-th entry, then the lanes rank their entries by flat index - which ascends with the
      // source - and the group adds the rows in that order.  One dependent load per pusher, nothing to search.
      const int total_e = others + 1;
      u32 cur = (u32)p.head[(size_t)row - n_cached], mine_f = kNoEntry;
      for (int i = 0; i < total_e && cur != kNoEntry; i++) {
        if (i == (int)gl) mine_f = cur;
        cur = p.next[cur];
      }
      int place = 0;
      for (int i = 0; i < total_e; i++) place += __shfl_sync(gmask, mine_f, i, LANES) < mine_f ? 1 : 0;
      size_t mine_ent = 0;
      if ((int)gl < total_e && mine_f != kNoEntry) {
        const int s2 = (int)segment_of(start, p.nsrc, mine_f);
        mine_ent = push_list_base(p, s2) + (mine_f - start[s2]);
      }
      // lane q of the group ends up with the entry of place q
      size_t ordered = 0;
      for (int i = 0; i < total_e; i++) {
        const int pl = __shfl_sync(gmask, place, i, LANES);
        const size_t en = __shfl_sync(gmask, mine_ent, i, LANES);
        if (pl == (int)gl) ordered = en;
      }
      for (size_t e0 = 0; e0 < E; e0 += LANES) {  // same trip count in every lane: the loop body shuffles
        const size_t e = e0 + gl;
        const bool act = e < E;
        T acc = R::zero();
        if (act) acc = emb[e];
        for (int j0 = 0; j0 < total_e; j0 += 4) {  // ascending source order, as source-by-source launches would
          T v[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const size_t ej = __shfl_sync(gmask, ordered, (j0 + j) % LANES, LANES);
            if (act && j0 + j < total_e) v[j] = R::ld_once(val + ej * E + e);
          }
#pragma unroll
          for (int j = 0; j < 4; j++)
            if (act && j0 + j < total_e) acc = R::add(acc, v[j]);
        }
        if (act) emb[e] = acc;
      }
      continue;
    }
    // more pushers than the group has lanes (narrow rows, many ranks): find the other sources' entries by binary
    // search in their key-sorted lists, LANES of them per round
    const long long key = p.key[ent];
    bool first = true;
    while (rest) {
      // up to LANES further sources per round: lane j finds the entry of the j-th of them
      const int cnt = min(__popc(rest), LANES);
      size_t mine = 0;
      if ((int)gl < cnt) mine = push_entry_of(p, start, (int)__fns(rest, 0, (int)gl + 1), key);
      for (int j = 0; j < cnt; j++) rest &= rest - 1;
      for (size_t e0 = 0; e0 < E; e0 += LANES) {  // same trip count in every lane: the loop body shuffles
        const size_t e = e0 + gl;
        const bool act = e < E;
        T acc = R::zero();
        if (act) {
          acc = emb[e];
          if (first) acc = R::add(acc, R::ld_once(val + ent * E + e));
        }
        for (int j0 = 0; j0 < cnt; j0 += 4) {  // ascending source order, as source-by-source launches would
          T v[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const size_t ej = __shfl_sync(gmask, mine, (j0 + j) % LANES, LANES);
            if (act && j0 + j < cnt) v[j] = R::ld_once(val + ej * E + e);
          }
#pragma unroll
          for (int j = 0; j < 4; j++)
            if (act && j0 + j < cnt) acc = R::add(acc, v[j]);
        }
        if (act) emb[e] = acc;
      }
      first = false;
    }
  }
}

// All sources in ONE launch (peer-to-peer exchange): the pushed rows of source s sit in sub-region s of this
// rank's mailbox.  Sources are applied one after the other with a grid-wide barrier in between, which keeps
// the reference's deterministic per-row apply order (two sources may push the same row) without one launch
// per source.  Launched cooperatively, so all CTAs are co-resident and the barrier cannot deadlock.
template <int LANES, bool VEC>
__global__ void __launch_bounds__(kThreads) owner_update_all(hctr_p2p_ctx c, const int32_t *__restrict__ row_of,
                                                             size_t length, size_t n_cached,
                                                             float *__restrict__ embedding,
                                                             long long *__restrict__ version) {
  typedef RowT<VEC> R;
  typedef typename R::T T;
  cooperative_groups::grid_group grid = cooperative_groups::this_grid();
  const hctr_p2p_box me = c.box[c.rank];
  const unsigned gl = threadIdx.x % LANES;
  const size_t groups = ((size_t)gridDim.x * kThreads) / LANES;
  const size_t E = R::elems(c.width);
  for (int s = 0; s < c.nrank; s++) {
    if (s == c.rank) continue;  // a rank never pushes to itself
    const size_t n_rows = min((size_t)c.cnt_in[c.nrank + s], (size_t)c.cap);
    if (n_rows == 0) continue;  // uniform across the grid
    const long long *key = reinterpret_cast<const long long *>(me.pkey) + (size_t)s * c.cap;
    const long long *updates = reinterpret_cast<const long long *>(me.pupd) + (size_t)s * c.cap;
    const T *val = reinterpret_cast<const T *>(me.pval + (size_t)s * c.cap * c.width);
    for (size_t m = ((size_t)blockIdx.x * kThreads + threadIdx.x) / LANES; m < n_rows; m += groups) {
      const long long k = key[m];
      int32_t row = -1;
      if (k >= 0 && (size_t)k < length) row = row_of[k];
      if (row < 0 || (size_t)row < n_cached) {
        if (gl == 0) atomicOr(c.err, HCTR_ERR_NOT_OWNER);
        continue;
      }
      if (gl == 0) version[row] = (long long)((u64)version[row] + (u64)updates[m]);
      T *emb = reinterpret_cast<T *>(embedding) + (size_t)row * E;
      const T *v = val + m * E;
      for (size_t e = gl; e < E; e += LANES) emb[e] = R::add(emb[e], R::ld_once(v + e));
    }
    grid.sync();
  }
}

}  // namespace hctr

using namespace hctr;

static int launch_owner_apply(const PushLists &p, size_t rows_hint, size_t width, size_t n_cached,
                              const int32_t *ent_row, const unsigned long long *row_mask, float *embedding,
                              cudaStream_t st) {
  const bool al = host_aligned16(p.val) && host_aligned16(embedding);
#define CALL(L, V)                                                                                                \
  do {                                                                                                            \
    size_t g_ = (rows_hint * L + kThreads - 1) / kThreads;                                                        \
    if (g_ > (size_t)kSMs * 8) g_ = (size_t)kSMs * 8;                                                             \
    owner_apply_sources<L, V><<<(unsigned)g_, kThreads, 0, st>>>(p, width, n_cached, ent_row, row_mask, embedding); \
  } while (0)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}

static unsigned mark_grid(size_t rows_hint) {
  // at most two blocks per SM: in the peer-to-peer exchange every block starts by polling the mailbox headers
  size_t g = (rows_hint + kThreads - 1) / kThreads;
  if (g > (size_t)kSMs * 2) g = (size_t)kSMs * 2;
  return (unsigned)(g ? g : 1);
}

extern "C" int hctr_owner_update_merged(int nsrc, size_t rows_hint, size_t width, const int64_t *key,
                                        const int64_t *updates, const float *val, const unsigned long long *src_off,
                                        const uint32_t *flat_start, const int32_t *row_of, size_t length,
                                        size_t n_cached, unsigned long long *row_mask,
                                        unsigned long long *row_head, uint32_t epoch, int32_t *ent_row,
                                        uint32_t *ent_next, float *embedding, int64_t *version, uint32_t *err,
                                        void *stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (nsrc > 32 || epoch == 0) return (int)cudaErrorInvalidValue;
  if (rows_hint == 0) return 0;
  PushLists p;
  p.key = (const long long *)key;
  p.upd = (const long long *)updates;
  p.val = val;
  p.src_off = src_off;
  p.src_stride = 0;
  p.flat_start = flat_start;
  p.nsrc = nsrc;
  p.head = row_head;
  p.next = ent_next;
  hctr_p2p_ctx none;
  memset(&none, 0, sizeof(none));
  owner_mark_sources<false><<<mark_grid(rows_hint), kThreads, 0, st>>>(p, none, 0u, row_of, length, n_cached, row_mask,
                                                                      epoch, ent_row, (long long *)version, err);
  count_launches(1);
  return launch_owner_apply(p, rows_hint, width, n_cached, ent_row, row_mask, embedding, st);
}

static PushLists mailbox_lists(const hctr_p2p_ctx *c, const hctr_p2p_box *mine, unsigned long long *row_head,
                               uint32_t *ent_next) {
  PushLists p;
  p.key = (const long long *)mine->pkey;
  p.upd = (const long long *)mine->pupd;
  p.val = mine->pval;
  p.src_off = nullptr;
  p.src_stride = c->cap;
  p.flat_start = c->cnt_in + 4 * c->nrank + 1;
  p.nsrc = c->nrank;
  p.head = row_head;
  p.next = ent_next;
  return p;
}

extern "C" int hctr_p2p_owner_mark(const hctr_p2p_ctx *c, const hctr_p2p_box *mine, uint32_t seq,
                                   const int32_t *row_of, size_t length, size_t n_cached,
                                   unsigned long long *row_mask, unsigned long long *row_head, uint32_t epoch,
                                   int32_t *ent_row, uint32_t *ent_next, int64_t *version, void *stream) {
  if (c->nrank > 32 || epoch == 0) return (int)cudaErrorInvalidValue;
  const PushLists p = mailbox_lists(c, mine, row_head, ent_next);
  owner_mark_sources<true><<<mark_grid(c->cap), kThreads, 0, (cudaStream_t)stream>>>(
      p, *c, seq, row_of, length, n_cached, row_mask, epoch, ent_row, (long long *)version, c->err);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_owner_apply(const hctr_p2p_ctx *c, const hctr_p2p_box *mine, size_t n_cached,
                                    const int32_t *ent_row, const unsigned long long *row_mask,
                                    unsigned long long *row_head, uint32_t *ent_next, float *embedding,
                                    void *stream) {
  if (c->nrank > 32) return (int)cudaErrorInvalidValue;
  return launch_owner_apply(mailbox_lists(c, mine, row_head, ent_next), c->cap, c->width, n_cached, ent_row, row_mask,
                            embedding, (cudaStream_t)stream);
}

extern "C" int hctr_p2p_owner_update(const hctr_p2p_ctx *cp, const int32_t *row_of, size_t length, size_t n_cached,
                                     float *embedding, int64_t *version, void *stream) {
  hctr_p2p_ctx c = *cp;
  long long *ver = (long long *)version;
  void *args[] = {&c, &row_of, &length, &n_cached, &embedding, &ver};
  const bool al = host_aligned16(embedding);
  cudaError_t e = cudaSuccess;
#define CALL(L, V)                                                                                              \
  e = cudaLaunchCooperativeKernel((const void *)owner_update_all<L, V>, dim3(kSMs * 2), dim3(kThreads), args, 0, \
                                  (cudaStream_t)stream)
  HCTR_DISPATCH_ROWS(c.width, al, CALL);
#undef CALL
  count_launches(1);
  return (int)e;
}

extern "C" int hctr_push_decide(const uint32_t *meta, int nrank, int rank, size_t u_max,
                                const uint8_t *uniq_owner, const int32_t *uniq_row, const uint32_t *run_start,
                                const int64_t *pending_cnt, int64_t push_bound, uint32_t *need_push,
                                uint32_t *push_slot, uint32_t *scan_scratch, uint32_t *push_count,
                                uint32_t *push_base, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (nrank > 1024) return (int)cudaErrorInvalidValue;
  push_decide<<<grid_for(u_max, kThreads), kThreads, 0, s>>>(meta, rank, uniq_owner, uniq_row, run_start,
                                                              (const long long *)pending_cnt, push_bound,
                                                              need_push);
  int rc = hctr_scan_exclusive_u32(need_push, push_slot, u_max, meta + HCTR_META_UNIQUE, scan_scratch, stream);
  if (rc) return rc;
  push_counts<<<1, 1024, 0, s>>>(meta, nrank, push_slot, push_count, push_base);
  count_launches(2);
  return launch_status();
}

extern "C" int hctr_push_decide_fused(const uint32_t *meta, int nrank, int rank, size_t u_max,
                                      const uint8_t *uniq_owner, const int32_t *uniq_row, const uint32_t *run_start,
                                      const int64_t *pending_cnt, int64_t push_bound, uint32_t *need_push,
                                      uint32_t *push_slot, uint32_t *chain_scratch, uint32_t epoch,
                                      uint32_t *push_count, uint32_t *push_base, uint32_t *err, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (nrank > 1024 || epoch == 0) return (int)cudaErrorInvalidValue;
  const size_t per = (size_t)kDecideThreads * kDecideItems;
  const size_t tiles = (u_max + 1 + per - 1) / per;
  push_decide_scan<<<(unsigned)tiles, kDecideThreads, 0, s>>>(meta, rank, uniq_owner, uniq_row, run_start,
                                                             (const long long *)pending_cnt, push_bound, need_push,
                                                             push_slot, reinterpret_cast<u64 *>(chain_scratch), epoch,
                                                             err);
  push_counts<<<1, 1024, 0, s>>>(meta, nrank, push_slot, push_count, push_base);
  count_launches(2);
  return launch_status();
}

// the streaming short-run kernel is the variant that can order its runs itself
static bool streaming_shape(size_t width, bool aligned) { return aligned && width % 4 == 0 && width >= 128 && width <= 512; }

extern "C" int hctr_reduce_orders_short_runs(size_t width, const float *grad) {
  return streaming_shape(width, host_aligned16(grad)) ? 1 : 0;
}

extern "C" int hctr_grad_reduce_apply_pack(const hctr_reduce_args *ap, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const hctr_reduce_args a = *ap;
  if (a.n_unique == 0) return 0;
  ReduceKernelArgs ka;
  ka.a = a;
  if (a.p2p) ka.p2p = *a.p2p;
  else memset(&ka.p2p, 0, sizeof(ka.p2p));
  const bool al = host_aligned16(a.grad) && host_aligned16(a.embedding) && host_aligned16(a.pending) &&
                  host_aligned16(a.push_val);  // mailbox regions are 256-byte aligned by construction
  if (a.n_heavy > 0 && a.side_stream && a.fork_event && a.join_event) {
    cudaError_t e = cudaEventRecord((cudaEvent_t)a.fork_event, s);
    if (e != cudaSuccess) return (int)e;
  }
  if (a.short_runs_unordered && !streaming_shape(a.width, al)) return (int)cudaErrorInvalidValue;

  // Two kernels: the long runs (one thread block per hot key) and everything else.  They touch different keys, so
  // with a second stream they run side by side.  The long-run kernel is launched FIRST and with at most
  // `long_per_sm` blocks per SM, the short-run kernel then fills what is left of every SM: launched the other way
  // round, the short-run kernel's single resident round of blocks occupies all SMs and the long runs only start
  // when it ends.
  // (Measured on config 2, one GPU: 1 long-run block + 3 short-run blocks per SM gave 0.146 ms per step; 2 + 4,
  // 3 + 3 and the old order - short-run kernel first - 0.147, 0.147 and 0.160.)
  // A multi-rank table runs the dedupe of the next batch beside this reduction, and both are on the step's critical
  // path: two short-run blocks per SM leave its small kernels room (config 2, two GPUs: 0.314 ms per step against
  // 0.323 with three blocks and 0.369 with one; the dedupe 108 against 122 us, the reduction 113 against 120 us).
  const int long_per_sm = 1, short_cap = a.need_push ? 2 : 3;
  const bool forked = a.n_heavy > 0 && a.side_stream && a.fork_event && a.join_event;
  cudaStream_t ls = forked ? (cudaStream_t)a.side_stream : s;
  if (a.n_heavy > 0) {
    static bool attr_set = false;
    size_t need = (size_t)kLongStages * max((size_t)kLongStageBytes, a.width * sizeof(float));
    if (need > 200 * 1024) return (int)cudaErrorInvalidValue;  // rows wider than 12800 floats
    if (!attr_set) {
      cudaError_t e1 = cudaFuncSetAttribute(grad_reduce_long<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      cudaError_t e2 = cudaFuncSetAttribute(grad_reduce_long<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e1 != cudaSuccess) return (int)e1;
      if (e2 != cudaSuccess) return (int)e2;
      attr_set = true;
    }
    if (forked) {
      cudaError_t e = cudaStreamWaitEvent(ls, (cudaEvent_t)a.fork_event, 0);
      if (e != cudaSuccess) return (int)e;
    }
    if (a.long_wait_event) {  // ordering of the long runs, done on another stream
      cudaError_t e = cudaStreamWaitEvent(ls, (cudaEvent_t)a.long_wait_event, 0);
      if (e != cudaSuccess) return (int)e;
    }
    cudaError_t em = cudaMemsetAsync(a.work_counter, 0, 2 * sizeof(u32), ls);
    if (em != cudaSuccess) return (int)em;
    const size_t per = need > 100 * 1024 ? 1 : (forked ? (size_t)long_per_sm : 3);
    const unsigned grid = (unsigned)min((size_t)a.n_heavy, (size_t)kSMs * per);
    if (al && a.width % 4 == 0) grad_reduce_long<true><<<grid, kLongThreads, need, ls>>>(ka, (u32)a.n_heavy, a.work_counter);
    else grad_reduce_long<false><<<grid, kLongThreads, need, ls>>>(ka, (u32)a.n_heavy, a.work_counter);
    count_launches(1);
    if (forked) {
      cudaError_t e = cudaEventRecord((cudaEvent_t)a.join_event, ls);
      if (e != cudaSuccess) return (int)e;
    }
  }

  if (streaming_shape(a.width, al) && a.n_unique < 0x7fffffffu) {
    const size_t E = a.width / 4;
    const int variant = E <= 32 ? 0 : E <= 64 ? 1 : 2;
    void (*kernel)(ReduceKernelArgs) = E == 32    ? grad_reduce_short_stream<8, 1, 32>
                                       : E == 64    ? grad_reduce_short_stream<4, 2, 64>
                                       : E == 128   ? grad_reduce_short_stream<2, 4, 128>
                                       : variant == 0 ? grad_reduce_short_stream<8, 1, 0>
                                       : variant == 1 ? grad_reduce_short_stream<4, 2, 0>
                                                      : grad_reduce_short_stream<2, 4, 0>;
    const int depth = variant == 0 ? 8 : variant == 1 ? 4 : 2;
    const size_t smem = (size_t)(kThreads / 32) * depth * E * sizeof(float4);  // at most 32 KB
    static int per_sm_of[3][3] = {};  // resident thread blocks per SM, by kernel variant and ring size class
    int &per_sm = per_sm_of[variant][smem <= 16384 ? 0 : smem <= 24576 ? 1 : 2];
    if (per_sm == 0) {
      cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem);
      if (e != cudaSuccess) return (int)e;
      if (per_sm < 1) per_sm = 1;
    }
    // Equal-cost thread blocks, at most one resident round of them (one, two and three rounds measured the
    // same; a few blocks left over for another round would double the kernel's duration).  A warp should get
    // at least ~48 row transfers; every key costs at least 3, so 3U bounds the total from below.  Next to the
    // long-run kernel the round is one block per SM smaller.
    const size_t slots = (size_t)kSMs * (forked ? std::min(per_sm, short_cap) : per_sm);
    const size_t wanted = (3 * a.n_unique / 48 * 32 + kThreads - 1) / kThreads + 1;
    const size_t ctas = std::min(wanted, slots);
    kernel<<<(unsigned)ctas, kThreads, smem, s>>>(ka);
  } else if (al && a.width % 4 == 0 && a.width >= 128) {
    size_t ctas = ((a.n_unique + kWideChunk - 1) / kWideChunk * 32 + kThreads - 1) / kThreads;
    const size_t cap = (size_t)kSMs * 8;
    if (ctas > cap) ctas = cap;
    grad_reduce_short_wide<<<(unsigned)ctas, kThreads, 0, s>>>(ka);
  } else {
#define CALL(L, V) \
  grad_reduce_short<L, V><<<grid_for(a.n_unique * L, kThreads), kThreads, 0, s>>>(ka)
    HCTR_DISPATCH_ROWS(a.width, al, CALL);
#undef CALL
  }
  count_launches(1);
  if (forked) {
    cudaError_t e = cudaStreamWaitEvent(s, (cudaEvent_t)a.join_event, 0);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_status();
}

extern "C" int hctr_owner_update_dev(size_t n_rows_max, const uint32_t *n_rows_dev, size_t width, const int64_t *key,
                                     const int64_t *updates, const float *val, const int32_t *row_of, size_t length,
                                     size_t n_cached, float *embedding, int64_t *version, uint32_t *err,
                                     void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (n_rows_max == 0) return 0;
  const bool al = host_aligned16(val) && host_aligned16(embedding);
#define CALL(L, V)                                                                                          \
  do {                                                                                                      \
    size_t g_ = (n_rows_max * L + kThreads - 1) / kThreads;                                                 \
    if (g_ > (size_t)kSMs * 8) g_ = (size_t)kSMs * 8;                                                       \
    owner_update<L, V><<<(unsigned)g_, kThreads, 0, s>>>(n_rows_max, n_rows_dev, width, (const long long *)key, \
                                                         (const long long *)updates, val, row_of, length,   \
                                                         n_cached, embedding, (long long *)version, err);   \
  } while (0)
  HCTR_DISPATCH_ROWS(width, al, CALL);
#undef CALL
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_owner_update(size_t n_rows, size_t width, const int64_t *key, const int64_t *updates,
                                 const float *val, const int32_t *row_of, size_t length, size_t n_cached,
                                 float *embedding, int64_t *version, uint32_t *err, void *stream) {
  return hctr_owner_update_dev(n_rows, nullptr, width, key, updates, val, row_of, length, n_cached, embedding, version,
                               err, stream);
}
