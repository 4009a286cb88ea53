// Preprocess: batch keys -> unique keys in (owner, key) order, occurrences, batch->unique map and
// per-unique position lists.
//
// The key space is dense ([0, length) with a 1-byte owner per key), so instead of sorting
// (owner,key,position) triples the batch is RANKED through a bitmap over the sort-key space
//     sk = key + length_pad * owner          (length_pad = length rounded up to 4096)
//   mark     one bit per distinct sk (atomicOr); the first setter flags its 4096-key block as touched
//   ranks    ONE launch: touched blocks are popcounted (distinct keys per block - counting by popcount
//            instead of an atomic per key keeps dense blocks, i.e. small vocabularies, from serialising
//            on one counter), block counts are scanned inside each CTA and chained across CTAs, and the
//            popcount prefix inside each block gives every 64-key word the rank of its first set bit =
//            index in the sorted unique list
//   rank     per batch position: unique index = word base + popcount(bits below); an atomic counter
//            per unique key hands out a slot inside the key's run, and the position that draws slot 0
//            writes the unique key, its owner and its local row
//   scan     occurrences -> run starts (single launch, chained)
//   scatter  positions into their runs; the slot-0 position also clears the bitmap word and counter
//   order    each run is put in ascending position order so that gradient sums are taken in batch
//            order (runs up to 32 by one warp, longer runs through a shared-memory position bitmap)
// Work is O(batch) plus one pass over the block counts; nothing probes, nothing can overflow, and
// cost does not depend on how skewed the keys are.
#include "common.cuh"

namespace hctr {

constexpr int kThreads = 256;
constexpr u32 kLightRun = HCTR_LIGHT_RUN;  // runs up to this length are ordered by one warp
constexpr int kHeavyWindowBits = 1 << 20;  // positions covered by one shared-memory window (128 KB)

// Thread -> batch position.  CTR batches are sample-major: position = sample * F + field, and the keys of one
// field come from one contiguous (often small) key range, while neighbouring positions belong to different
// fields.  With the identity mapping the 32 lanes of a warp touch 32 unrelated places of the bitmap and of the
// per-key arrays, and the few cache lines of a small vocabulary receive thousands of separate requests per
// batch.  With stride F a warp takes the SAME field of 32 consecutive samples: its lanes hit the same lines
// (one request instead of up to 32) and duplicates inside the warp are merged before they reach an atomic.
// Positions beyond the last whole group of 32 samples keep the identity mapping.  Any mapping gives the same
// results: which thread handles a position is invisible in the outputs.
__device__ __forceinline__ size_t mapped_pos(size_t t, size_t batch, u32 stride) {
  if (stride <= 1) return t;
  const size_t group = (size_t)32 * stride;
  if (t >= batch / group * group) return t;
  const size_t r = t % group;
  return t - r + (r % 32) * stride + r / 32;
}

// The kernel is a chain of dependent memory operations per position (key -> owner -> bitmap word ->
// atomic), so it is latency-bound; a single-rank table skips the owner lookup (every key is rank 0's).
__global__ void __launch_bounds__(kThreads) dedupe_mark(hctr_dedupe_args a) {
  const size_t t = (size_t)blockIdx.x * kThreads + threadIdx.x;
  const unsigned lane = threadIdx.x & 31;
  u64 sk = ~0ull;
  bool ok = false;
  if (t < a.batch) {
    const size_t i = mapped_pos(t, a.batch, a.stride);
    const long long key = a.keys[i];
    unsigned o = 0;
    ok = key >= 0 && (size_t)key < a.length;
    if (ok && a.nrank > 1) {
      o = a.owner_of[key];
      ok = o < (unsigned)a.nrank;
    }
    if (ok) sk = (u64)key + (u64)a.length_pad * o;
    else atomicOr(&a.meta[HCTR_META_ERR], HCTR_ERR_KEY_RANGE);
    a.sk[i] = sk;
  }
  // one lane per distinct key of the warp goes on (whole warps get here: no thread has returned)
  const unsigned peers = __match_any_sync(0xffffffffu, ok ? sk : ~(u64)lane);
  if (!ok || lane != (unsigned)(__ffs(peers) - 1)) return;
  // the bitmap is addressed as 32-bit words here (little-endian halves of the 64-bit words)
  const u32 bit = 1u << (sk & 31);
  u32 *word = reinterpret_cast<u32 *>(a.bits) + (sk >> 5);
  // Skip the atomic when an earlier duplicate is already visible, and let only the first setter of a bit touch
  // the block flag (unconditional flag stores from every position made one L2 slice 12x hotter than the
  // average in profiles).
  if (*word & bit) return;
  const u32 old = atomicOr(word, bit);
  if (!(old & bit)) a.blk_flag[sk >> 12] = 1;
}

__device__ __forceinline__ u32 warp_excl_scan_total(u32 v, u32 *total) {
  const unsigned lane = threadIdx.x & 31;
  u32 incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    u32 t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= (unsigned)d) incl += t;
  }
  *total = __shfl_sync(0xffffffffu, incl, 31);
  return incl - v;
}

// count + scan + extract in one launch.  Every warp owns `group` (1..32) consecutive bitmap blocks, one
// per lane.  (1) touched blocks are popcounted by the whole warp; (2) counts are scanned inside the CTA
// and chained across CTAs (chained_cta_prefix), which gives every block the rank of its first key;
// (3) the warp ranks the 64 words of each touched block.  Small tables use group = 1 (maximum
// parallelism); huge, sparsely hit tables use 32 so that untouched blocks cost one coalesced flag load
// per 32 and the number of CTAs in the chain stays small.
__global__ void __launch_bounds__(kThreads) dedupe_block_ranks(hctr_dedupe_args a, size_t n_blocks,
                                                               size_t blocks_per_owner, unsigned group, u64 *agg,
                                                               u32 epoch) {
  __shared__ u32 warp_tot[kThreads / 32];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t g = ((size_t)blockIdx.x * (kThreads / 32) + warp) * group;  // first block of this warp
  const size_t b = g + lane;
  bool touched = false;
  if (lane < group && b < n_blocks) {
    touched = a.blk_flag[b] != 0;
    if (touched) a.blk_flag[b] = 0;  // consumed: all-zero again for the next batch
  }
  const unsigned live = __ballot_sync(0xffffffffu, touched);
  u32 cnt = 0;
  for (unsigned todo = live; todo;) {
    const int src = __ffs(todo) - 1;
    todo &= todo - 1;
    const size_t w0 = (g + src) * HCTR_BLOCK_WORDS + lane;
    u32 c = __popcll(a.bits[w0]) + __popcll(a.bits[w0 + 32]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) c += __shfl_xor_sync(0xffffffffu, c, d);
    if ((int)lane == src) cnt = c;
  }
  u32 wtotal;
  u32 base = warp_excl_scan_total(cnt, &wtotal);
  if (lane == 0) warp_tot[warp] = wtotal;
  __syncthreads();
  u32 cta_total = 0, before = 0;
#pragma unroll
  for (unsigned w = 0; w < kThreads / 32; w++) {
    if (w < warp) before += warp_tot[w];
    cta_total += warp_tot[w];
  }
  const u32 prefix = chained_cta_prefix(agg, epoch, blockIdx.x, cta_total, &a.meta[HCTR_META_ERR]);
  base += before + prefix;
  if (lane < group && b < n_blocks && b % blocks_per_owner == 0) a.meta[HCTR_META_SEG + b / blocks_per_owner] = base;
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
    const u32 U = prefix + cta_total;
    a.meta[HCTR_META_UNIQUE] = U;
    a.meta[HCTR_META_SEG + a.nrank] = U;
  }
  for (unsigned todo = live; todo;) {
    const int src = __ffs(todo) - 1;
    todo &= todo - 1;
    const u32 blk_base = __shfl_sync(0xffffffffu, base, src);
    const size_t w0 = (g + src) * HCTR_BLOCK_WORDS + lane, w1 = w0 + 32;
    const u64 x0 = a.bits[w0], x1 = a.bits[w1];
    u32 t0, t1;
    const u32 e0 = warp_excl_scan_total(__popcll(x0), &t0);
    const u32 e1 = warp_excl_scan_total(__popcll(x1), &t1);
    a.word_base[w0] = blk_base + e0;
    a.word_base[w1] = blk_base + t0 + e1;
  }
}

__global__ void __launch_bounds__(kThreads) dedupe_rank(hctr_dedupe_args a) {
  const size_t t = (size_t)blockIdx.x * kThreads + threadIdx.x;
  const unsigned lane = threadIdx.x & 31;
  size_t i = 0;
  u64 sk = ~0ull;
  if (t < a.batch) {
    i = mapped_pos(t, a.batch, a.stride);
    sk = a.sk[i];
  }
  const bool ok = sk != ~0ull;
  u32 u = 0;
  if (ok) {
    const u64 w = sk >> 6;
    const u64 below = a.bits[w] & ((1ull << (sk & 63)) - 1);
    u = a.word_base[w] + __popcll(below);
    a.idx_map[i] = (int32_t)u;
  } else if (t < a.batch) {
    a.idx_map[i] = -1;
  }
  // duplicates inside the warp take their ranks from one atomic: the lowest lane adds the group's size
  const unsigned peers = __match_any_sync(0xffffffffu, ok ? (u64)u : ~(u64)lane);
  const unsigned leader = (unsigned)(__ffs(peers) - 1);
  u32 base = 0;
  if (ok && lane == leader) base = atomicAdd(&a.cnt[u], (u32)__popc(peers));
  base = __shfl_sync(0xffffffffu, base, leader);
  if (!ok) return;
  const u32 rk = base + __popc(peers & ((1u << lane) - 1));
  a.rank_in_run[i] = rk;
  if (rk == 0) {  // exactly one position per unique key
    const long long key = a.keys[i];
    a.uniq[u] = key;
    a.uniq_owner[u] = a.owner_of[key];
    a.uniq_row[u] = a.row_of[key];
  }
}

__global__ void __launch_bounds__(kThreads) dedupe_scatter(hctr_dedupe_args a) {
  const size_t t = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (t >= a.batch) return;
  const size_t i = mapped_pos(t, a.batch, a.stride);
  const u64 sk = a.sk[i];
  if (sk == ~0ull) {
    if (a.pos_row) a.pos_row[i] = HCTR_INVALID_ROW;
    return;
  }
  const u32 u = (u32)a.idx_map[i];
  const u32 rk = a.rank_in_run[i];
  a.sorted_pos[a.run_start[u] + rk] = (u32)i;
  if (a.pos_row) a.pos_row[i] = a.uniq_row[u];
  if (rk == 0) {
    // leave the persistent scratch all-zero for the next batch (once per unique key)
    a.bits[sk >> 6] = 0;
    a.cnt[u] = 0;
  }
  // exactly one position per run longer than kLightRun sees this slot: it queues the run as "long"
  // (at most batch/33 such runs exist; the list holds batch/32 + 2 entries)
  if (rk == kLightRun) a.heavy_list[atomicAdd(&a.meta[HCTR_META_NHEAVY], 1u)] = u;
}

// Runs of 2..kLightRun positions.  A warp takes 32 consecutive unique keys (run bounds fetched
// coalesced, one key per lane), then orders the runs that need it one after the other: one position
// per lane, a lane's final slot = number of smaller positions in the run (positions are distinct).
__global__ void __launch_bounds__(kThreads) dedupe_order_light(hctr_dedupe_args a) {
  const unsigned lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const size_t n_warps = ((size_t)gridDim.x * kThreads) >> 5;
  const size_t U = a.meta[HCTR_META_UNIQUE];
  for (size_t u0 = warp * 32; u0 < U; u0 += n_warps * 32) {
    const size_t u = u0 + lane;
    u32 l = 0, len = 0;
    if (u < U) {
      l = a.run_start[u];
      len = a.run_start[u + 1] - l;
    }
    unsigned todo = __ballot_sync(0xffffffffu, len >= 2 && len <= kLightRun);  // longer: dedupe_order_heavy
    while (todo) {
      const int src = __ffs(todo) - 1;
      todo &= todo - 1;
      const u32 rl = __shfl_sync(0xffffffffu, l, src), rlen = __shfl_sync(0xffffffffu, len, src);
      u32 *p = a.sorted_pos + rl;
      const u32 v = lane < rlen ? p[lane] : 0xffffffffu;
      u32 slot = 0;
      for (u32 k = 0; k < rlen; k++) slot += __shfl_sync(0xffffffffu, v, k) < v ? 1u : 0u;
      if (lane < rlen) p[slot] = v;
    }
  }
}

// Long runs: a CTA sets one bit per position in a shared-memory bitmap (window by window when the
// batch exceeds the window), then emits the set bits in order.  Cost per run is O(batch/32) word
// operations, independent of the run length, so even "all keys equal" stays cheap.
__global__ void __launch_bounds__(1024) dedupe_order_heavy(hctr_dedupe_args a, u32 window_bits) {
  extern __shared__ u32 win[];  // window_bits / 32 words
  __shared__ u32 warp_tot[32];
  __shared__ u32 carry;
  const u32 n_heavy = a.meta[HCTR_META_NHEAVY];
  const unsigned tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t batch = a.batch;
  for (u32 h = blockIdx.x; h < n_heavy; h += gridDim.x) {
    const u32 u = a.heavy_list[h];
    const u32 l = a.run_start[u], len = a.run_start[u + 1] - l;
    u32 *p = a.sorted_pos + l;
    // The run is rewritten in place, so stage it first: positions are re-read per window from a
    // copy kept in rank_in_run (free after the scatter step; runs are disjoint slices of it).
    u32 *stage = a.rank_in_run + l;
    for (u32 k = tid; k < len; k += 1024) stage[k] = p[k];
    if (tid == 0) carry = 0;
    __syncthreads();
    for (size_t w0 = 0; w0 < batch; w0 += window_bits) {
      const u32 wbits = (u32)min((size_t)window_bits, batch - w0);
      const u32 wwords = (wbits + 31) / 32;
      for (u32 k = tid; k < wwords; k += 1024) win[k] = 0;
      __syncthreads();
      for (u32 k = tid; k < len; k += 1024) {
        const size_t pos = stage[k];
        if (pos >= w0 && pos < w0 + wbits) atomicOr(&win[(pos - w0) >> 5], 1u << ((pos - w0) & 31));
      }
      __syncthreads();
      // each thread owns a contiguous chunk of words; block scan of the chunk popcounts
      const u32 per = (wwords + 1023) / 1024;
      const u32 beg = min(tid * per, wwords), end = min(beg + per, wwords);
      u32 c = 0;
      for (u32 k = beg; k < end; k++) c += __popc(win[k]);
      u32 incl = c;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        u32 t = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= (unsigned)d) incl += t;
      }
      if (lane == 31) warp_tot[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        u32 t = warp_tot[lane], ti = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          u32 s = __shfl_up_sync(0xffffffffu, ti, d);
          if (lane >= (unsigned)d) ti += s;
        }
        warp_tot[lane] = ti - t;
      }
      __syncthreads();
      u32 o = carry + warp_tot[warp] + incl - c;
      for (u32 k = beg; k < end; k++) {
        u32 x = win[k];
        while (x) {
          const int bp = __ffs(x) - 1;
          x &= x - 1;
          p[o++] = (u32)(w0 + ((size_t)k << 5) + bp);
        }
      }
      __syncthreads();
      if (tid == 1023) carry = o;  // last thread's end = total so far
      __syncthreads();
    }
  }
}

// scores[d] = number of i < limit - d with keys[i] == keys[i + d]; one thread block per distance d = 1..64
__global__ void __launch_bounds__(kThreads) key_stride_scores(const long long *__restrict__ keys, size_t n,
                                                              u32 *__restrict__ scores) {
  __shared__ u32 total;
  const size_t d = blockIdx.x + 1;
  const size_t limit = n < 32768 ? n : 32768;
  if (threadIdx.x == 0) total = 0;
  __syncthreads();
  u32 mine = 0;
  for (size_t i = threadIdx.x; i + d < limit; i += kThreads) mine += keys[i] == keys[i + d] ? 1u : 0u;
  atomicAdd(&total, mine);
  __syncthreads();
  if (threadIdx.x == 0) scores[d] = total;
}

// Private copy of a device-resident key batch + cleared meta words in one launch (one device operation
// in front of the pipeline instead of a copy and a memset).
__global__ void __launch_bounds__(kThreads) ingest_keys(const long long *__restrict__ src, long long *__restrict__ dst,
                                                        size_t n, u32 *__restrict__ meta, unsigned meta_words) {
  const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (i < meta_words) meta[i] = 0;
  if (i < n) dst[i] = src[i];
}

// The same, plus the local row of every batch position (pos_row[i] = row_of[key] or HCTR_INVALID_ROW): all the
// row expansion needs to know about a batch whose keys are stored here, so that it does not have to wait for the
// dedupe pipeline.  src may equal dst (keys already in place).  A key outside [0, length) sets bit
// HCTR_ERR_KEY_RANGE in *err.
__global__ void __launch_bounds__(kThreads) ingest_keys_rows(const long long *__restrict__ src,
                                                             long long *__restrict__ dst, size_t n,
                                                             u32 *__restrict__ meta, unsigned meta_words,
                                                             const int32_t *__restrict__ row_of, size_t length,
                                                             int32_t *__restrict__ pos_row, u32 *__restrict__ err) {
  const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (i < meta_words) meta[i] = 0;
  if (i < n) {
    const long long k = src[i];
    if (src != dst) dst[i] = k;
    int32_t row = HCTR_INVALID_ROW;
    if (k >= 0 && (size_t)k < length) row = row_of[k];
    else atomicOr(err, HCTR_ERR_KEY_RANGE);
    pos_row[i] = row;
  }
}

}  // namespace hctr

using namespace hctr;

extern "C" int hctr_ingest_keys_rows(const int64_t *src, int64_t *dst, size_t n, uint32_t *meta, unsigned meta_words,
                                     const int32_t *row_of, size_t length, int32_t *pos_row, uint32_t *err,
                                     void *stream) {
  const size_t items = n > meta_words ? n : meta_words;
  ingest_keys_rows<<<grid_for(items ? items : 1, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
      (const long long *)src, (long long *)dst, n, meta, meta_words, row_of, length, pos_row, err);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_detect_key_stride(const int64_t *keys, size_t n, uint32_t *scores, void *stream) {
  key_stride_scores<<<64, kThreads, 0, (cudaStream_t)stream>>>((const long long *)keys, n, scores);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_ingest_keys(const int64_t *src, int64_t *dst, size_t n, uint32_t *meta, unsigned meta_words,
                                void *stream) {
  const size_t items = n > meta_words ? n : meta_words;
  ingest_keys<<<grid_for(items ? items : 1, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
      (const long long *)src, (long long *)dst, n, meta, meta_words);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_dedupe_map(const hctr_dedupe_args *ap, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const hctr_dedupe_args a = *ap;
  const size_t n_blocks = (size_t)a.nrank * a.length_pad / HCTR_BLOCK_KEYS;
  const size_t blocks_per_owner = a.length_pad / HCTR_BLOCK_KEYS;
  const unsigned gb = grid_for(a.batch, kThreads);
  dedupe_mark<<<gb, kThreads, 0, s>>>(a);
  // One warp per `group` bitmap blocks; keep the chain of CTAs short (each CTA adds up its predecessors).
  unsigned group = 1;
  while (group < 32 && (n_blocks + group - 1) / group > (size_t)kThreads / 32 * 2048) group *= 2;
  const size_t warps = (n_blocks + group - 1) / group;
  const size_t blk_ctas = (warps + kThreads / 32 - 1) / (kThreads / 32);
  dedupe_block_ranks<<<(unsigned)(blk_ctas ? blk_ctas : 1), kThreads, 0, s>>>(
      a, n_blocks, blocks_per_owner, group, reinterpret_cast<u64 *>(a.chain_scratch), a.epoch);
  dedupe_rank<<<gb, kThreads, 0, s>>>(a);
  int rc = hctr_scan_exclusive_u32_chained(a.cnt, a.run_start, a.batch, a.meta + HCTR_META_UNIQUE, a.scan_scratch,
                                           a.epoch, a.meta + HCTR_META_ERR, stream);
  if (rc) return rc;
  dedupe_scatter<<<gb, kThreads, 0, s>>>(a);
  // Run ordering is only needed by the gradient reduction of the NEXT step, not by anything else in this
  // one.  With a second stream the two ordering kernels leave the caller's stream: they start after the
  // scatter (fork_event) and join_event marks their completion; whoever consumes sorted_pos waits on it.
  // Without a join_event the caller enqueues them itself, later, with hctr_dedupe_order.
  if (a.side_stream && a.fork_event) {
    cudaError_t e = cudaEventRecord((cudaEvent_t)a.fork_event, s);
    if (e != cudaSuccess) return (int)e;
    count_launches(4);
    if (!a.join_event) return launch_status();
    cudaStream_t os = (cudaStream_t)a.side_stream;
    e = cudaStreamWaitEvent(os, (cudaEvent_t)a.fork_event, 0);
    if (e != cudaSuccess) return (int)e;
    const int rc2 = hctr_dedupe_order(ap, a.side_stream);
    if (rc2) return rc2;
    e = cudaEventRecord((cudaEvent_t)a.join_event, os);
    return e != cudaSuccess ? (int)e : launch_status();
  }
  count_launches(4);
  return hctr_dedupe_order(ap, stream);
}

extern "C" int hctr_dedupe_order_light(const hctr_dedupe_args *ap, void *stream) {
  const hctr_dedupe_args a = *ap;
  size_t ctas = ((a.batch + 31) / 32 * 32 + kThreads - 1) / kThreads;  // one warp per 32 unique keys
  if (ctas > (size_t)kSMs * 8) ctas = (size_t)kSMs * 8;
  if (ctas == 0) ctas = 1;
  dedupe_order_light<<<(unsigned)ctas, kThreads, 0, (cudaStream_t)stream>>>(a);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_dedupe_order_heavy(const hctr_dedupe_args *ap, void *stream) {
  const hctr_dedupe_args a = *ap;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(dedupe_order_heavy, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kHeavyWindowBits / 8);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  // window = the batch when it fits (small windows let several CTAs share an SM)
  size_t wbits = (a.batch + 1023) / 1024 * 1024;
  if (wbits > (size_t)kHeavyWindowBits) wbits = kHeavyWindowBits;
  if (wbits < 1024) wbits = 1024;
  const size_t smem = wbits / 8;
  size_t per_sm = (200 * 1024) / (smem + 1024);
  if (per_sm > 2) per_sm = 2;  // 1024-thread CTAs: at most 2 per SM
  if (per_sm < 1) per_sm = 1;
  dedupe_order_heavy<<<(unsigned)(kSMs * per_sm), 1024, smem, (cudaStream_t)stream>>>(a, (u32)wbits);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_dedupe_order(const hctr_dedupe_args *ap, void *stream) {
  const int rc = hctr_dedupe_order_light(ap, stream);
  return rc ? rc : hctr_dedupe_order_heavy(ap, stream);
}
