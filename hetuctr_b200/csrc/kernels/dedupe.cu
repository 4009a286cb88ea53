// Preprocess: batch keys -> unique keys in (owner, key) order, occurrences, batch->unique map and
// per-unique position lists.
//
// The key space is dense ([0, length) with a 1-byte owner per key), so instead of sorting
// (owner,key,position) triples the batch is RANKED through a bitmap over the sort-key space
//     sk = key + length_pad * owner          (length_pad = length rounded up to 4096)
//   mark     one bit per distinct sk (atomicOr); the first setter bumps its 4096-key block's count
//   scan     block counts -> block bases                         (hctr_scan_exclusive_u32)
//   extract  one warp per non-empty block: popcount prefix inside the block gives every set bit its
//            rank = index in the sorted unique list; the warp writes unique key, owner, local row and
//            the per-word base used by the next step
//   rank     per batch position: unique index = word_base + popcount(bits below); an atomic counter
//            per unique key hands out a slot inside the key's run
//   scan     occurrences -> run starts
//   scatter  positions into their runs; clears the bitmap words and block counts it touched
//   order    each run is put in ascending position order so that gradient sums are taken in batch
//            order (short runs in registers, long runs through a shared-memory position bitmap)
// Work is O(batch) plus one pass over the block counts; nothing probes, nothing can overflow.
#include "common.cuh"

namespace hctr {

constexpr int kThreads = 256;
constexpr u32 kLightRun = 32;              // runs up to this length are sorted by one thread
constexpr int kHeavyWindowBits = 1 << 20;  // positions covered by one shared-memory window (128 KB)

__global__ void __launch_bounds__(kThreads) dedupe_mark(hctr_dedupe_args a) {
  const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (i == 0) a.meta[HCTR_META_NHEAVY] = 0;
  if (i >= a.batch) return;
  const long long key = a.keys[i];
  if (key < 0 || (size_t)key >= a.length) {
    atomicOr(&a.meta[HCTR_META_ERR], HCTR_ERR_KEY_RANGE);
    a.sk[i] = ~0ull;
    return;
  }
  const unsigned o = a.owner_of[key];
  if (o >= (unsigned)a.nrank) {
    atomicOr(&a.meta[HCTR_META_ERR], HCTR_ERR_KEY_RANGE);
    a.sk[i] = ~0ull;
    return;
  }
  const u64 sk = (u64)key + (u64)a.length_pad * o;
  a.sk[i] = sk;
  const u64 bit = 1ull << (sk & 63);
  u64 *word = a.bits + (sk >> 6);
  // duplicates of a hot key mostly see the bit already set and skip the atomic
  if (*(volatile u64 *)word & bit) return;
  const u64 old = atomicOr(word, bit);
  if (!(old & bit)) atomicAdd(&a.blk_cnt[sk >> 12], 1u);
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

// Each warp walks groups of 32 consecutive bitmap blocks; lanes fetch the 32 counts/bases at once and
// the warp then expands the non-empty blocks one by one.
__global__ void __launch_bounds__(kThreads) dedupe_extract(hctr_dedupe_args a, size_t n_blocks,
                                                           size_t blocks_per_owner) {
  const unsigned lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const size_t n_warps = ((size_t)gridDim.x * kThreads) >> 5;
  if (warp == 0 && lane == 0) {
    const u32 U = a.blk_base[n_blocks];
    a.meta[HCTR_META_UNIQUE] = U;
    a.meta[HCTR_META_SEG + a.nrank] = U;
    a.cnt[U] = 0;
  }
  for (size_t g = warp * 32; g < n_blocks; g += n_warps * 32) {
    const size_t b = g + lane;
    u32 c = 0, base = 0;
    if (b < n_blocks) {
      c = a.blk_cnt[b];
      base = a.blk_base[b];
      if (b % blocks_per_owner == 0) a.meta[HCTR_META_SEG + b / blocks_per_owner] = base;
    }
    unsigned live = __ballot_sync(0xffffffffu, c != 0);
    while (live) {
      const int src = __ffs(live) - 1;
      live &= live - 1;
      const size_t blk = g + src;
      const u32 blk_base = __shfl_sync(0xffffffffu, base, src);
      const size_t w0 = blk * HCTR_BLOCK_WORDS + lane, w1 = w0 + 32;
      const u64 x0 = a.bits[w0], x1 = a.bits[w1];
      u32 t0, t1;
      const u32 e0 = warp_excl_scan_total(__popcll(x0), &t0);
      const u32 e1 = warp_excl_scan_total(__popcll(x1), &t1);
      const u32 b0 = blk_base + e0, b1 = blk_base + t0 + e1;
      a.word_base[w0] = b0;
      a.word_base[w1] = b1;
      const unsigned owner = (unsigned)(blk / blocks_per_owner);
      const u64 owner_off = (u64)owner * a.length_pad;
#pragma unroll
      for (int h = 0; h < 2; h++) {
        u64 x = h ? x1 : x0;
        u32 u = h ? b1 : b0;
        const u64 sk0 = (u64)(h ? w1 : w0) << 6;
        while (x) {
          const int bitpos = __ffsll((long long)x) - 1;
          x &= x - 1;
          const long long key = (long long)(sk0 + bitpos - owner_off);
          a.uniq[u] = key;
          a.uniq_owner[u] = (uint8_t)owner;
          a.uniq_row[u] = a.row_of[key];
          a.cnt[u] = 0;
          u++;
        }
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads) dedupe_rank(hctr_dedupe_args a) {
  const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= a.batch) return;
  const u64 sk = a.sk[i];
  if (sk == ~0ull) {
    a.idx_map[i] = -1;
    return;
  }
  const u64 w = sk >> 6;
  const u64 below = a.bits[w] & ((1ull << (sk & 63)) - 1);
  const u32 u = a.word_base[w] + __popcll(below);
  a.idx_map[i] = (int32_t)u;
  a.rank_in_run[i] = atomicAdd(&a.cnt[u], 1u);
}

__global__ void __launch_bounds__(kThreads) dedupe_scatter(hctr_dedupe_args a) {
  const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= a.batch) return;
  const u64 sk = a.sk[i];
  if (sk == ~0ull) return;
  const u32 u = (u32)a.idx_map[i];
  a.sorted_pos[a.run_start[u] + a.rank_in_run[i]] = (u32)i;
  // leave the persistent scratch all-zero for the next batch
  a.bits[sk >> 6] = 0;
  a.blk_cnt[sk >> 12] = 0;
}

// Runs of 2..kLightRun positions: one thread sorts its run in registers/local memory.
// Longer runs are queued for dedupe_order_heavy.
__global__ void __launch_bounds__(kThreads) dedupe_order_light(hctr_dedupe_args a) {
  const size_t u = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (u >= a.meta[HCTR_META_UNIQUE]) return;
  const u32 l = a.run_start[u], len = a.run_start[u + 1] - l;
  if (len < 2) return;
  u32 *p = a.sorted_pos + l;
  if (len == 2) {
    const u32 x = p[0], y = p[1];
    if (x > y) {
      p[0] = y;
      p[1] = x;
    }
    return;
  }
  if (len > kLightRun) {
    const u32 slot = atomicAdd(&a.meta[HCTR_META_NHEAVY], 1u);
    a.heavy_list[slot] = (u32)u;  // at most batch/33 such runs exist; the list holds batch/32+1
    return;
  }
  u32 v[kLightRun];
  for (u32 k = 0; k < len; k++) v[k] = p[k];
  for (u32 k = 1; k < len; k++) {  // insertion sort
    const u32 x = v[k];
    u32 j = k;
    while (j > 0 && v[j - 1] > x) {
      v[j] = v[j - 1];
      j--;
    }
    v[j] = x;
  }
  for (u32 k = 0; k < len; k++) p[k] = v[k];
}

// Long runs: a CTA sets one bit per position in a shared-memory bitmap (window by window when the
// batch exceeds the window), then emits the set bits in order.  Cost per run is O(batch/32) word
// operations, independent of the run length, so even "all keys equal" stays cheap.
__global__ void __launch_bounds__(1024) dedupe_order_heavy(hctr_dedupe_args a) {
  extern __shared__ u32 win[];  // kHeavyWindowBits / 32 words
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
    for (size_t w0 = 0; w0 < batch; w0 += kHeavyWindowBits) {
      const u32 wbits = (u32)min((size_t)kHeavyWindowBits, batch - w0);
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

}  // namespace hctr

using namespace hctr;

extern "C" int hctr_dedupe_map(const hctr_dedupe_args *ap, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const hctr_dedupe_args a = *ap;
  const size_t n_blocks = (size_t)a.nrank * a.length_pad / HCTR_BLOCK_KEYS;
  const size_t blocks_per_owner = a.length_pad / HCTR_BLOCK_KEYS;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(dedupe_order_heavy, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kHeavyWindowBits / 8);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const unsigned gb = grid_for(a.batch, kThreads);
  dedupe_mark<<<gb, kThreads, 0, s>>>(a);
  int rc = hctr_scan_exclusive_u32(a.blk_cnt, a.blk_base, n_blocks, nullptr, a.scan_scratch, stream);
  if (rc) return rc;
  {
    size_t warps = (n_blocks + 31) / 32;
    size_t ctas = (warps * 32 + kThreads - 1) / kThreads;
    const size_t cap = (size_t)kSMs * 8;
    if (ctas > cap) ctas = cap;
    if (ctas == 0) ctas = 1;
    dedupe_extract<<<(unsigned)ctas, kThreads, 0, s>>>(a, n_blocks, blocks_per_owner);
  }
  dedupe_rank<<<gb, kThreads, 0, s>>>(a);
  rc = hctr_scan_exclusive_u32(a.cnt, a.run_start, a.batch, a.meta + HCTR_META_UNIQUE, a.scan_scratch, stream);
  if (rc) return rc;
  dedupe_scatter<<<gb, kThreads, 0, s>>>(a);
  dedupe_order_light<<<gb, kThreads, 0, s>>>(a);
  dedupe_order_heavy<<<kSMs, 1024, kHeavyWindowBits / 8, s>>>(a);
  count_launches(6);
  return launch_status();
}
