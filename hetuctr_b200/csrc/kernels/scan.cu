// Exclusive prefix sum over 32-bit counts in two small launches (tile sums; tile-local scan + the sum
// of the preceding tile sums, which every CTA adds up for itself).  No spin-waits and no assumption on CTA dispatch
// order; the inputs on this path are at most a few million entries and L2-resident.
#include <cstdio>

#include "common.cuh"

namespace hctr {

constexpr int kScanThreads = 1024;
constexpr int kScanItems = HCTR_SCAN_TILE / kScanThreads;  // 4

__device__ __forceinline__ u32 warp_incl_scan(u32 v) {
  const unsigned lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    u32 t = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= (unsigned)d) v += t;
  }
  return v;
}

// Block-wide exclusive scan of one value per thread (1024 threads); returns the exclusive prefix and
// the block total through `total`.
__device__ __forceinline__ u32 block_excl_scan(u32 v, u32 *total) {
  __shared__ u32 warp_sums[32];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  u32 incl = warp_incl_scan(v);
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    u32 w = warp_sums[lane];
    u32 wi = warp_incl_scan(w);
    warp_sums[lane] = wi - w;  // exclusive over warps
    if (lane == 31) *total = wi;
  }
  __syncthreads();
  u32 r = incl - v + warp_sums[warp];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(kScanThreads) scan_tile_sums(const u32 *__restrict__ in, size_t n_max,
                                                               const u32 *__restrict__ n_dev,
                                                               u32 *__restrict__ tile_sum) {
  const size_t n = n_dev ? min((size_t)*n_dev, n_max) : n_max;
  const size_t base = (size_t)blockIdx.x * HCTR_SCAN_TILE + (size_t)threadIdx.x * kScanItems;
  u32 s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; k++)
    if (base + k < n) s += in[base + k];
  __shared__ u32 total;
  block_excl_scan(s, &total);
  if (threadIdx.x == 0) tile_sum[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanThreads) scan_apply(const u32 *__restrict__ in, u32 *__restrict__ out,
                                                           size_t n_max, const u32 *__restrict__ n_dev,
                                                           const u32 *__restrict__ tile_sum) {
  const size_t n = n_dev ? min((size_t)*n_dev, n_max) : n_max;
  const size_t base = (size_t)blockIdx.x * HCTR_SCAN_TILE + (size_t)threadIdx.x * kScanItems;
  u32 v[kScanItems];
  u32 s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    v[k] = (base + k < n) ? in[base + k] : 0;
    s += v[k];
  }
  __shared__ u32 total;
  // base of this tile = sum of the tile sums before it (at most a few hundred values, L2-resident)
  u32 before = 0;
  for (unsigned t = threadIdx.x; t < blockIdx.x; t += kScanThreads) before += tile_sum[t];
  __shared__ u32 base_total;
  block_excl_scan(before, &base_total);
  u32 ex = block_excl_scan(s, &total) + base_total;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    if (base + k <= n) out[base + k] = ex;  // entry n receives the grand total
    ex += v[k];
  }
}

// Small inputs (a few tiles): one CTA walks the tiles with a running carry, one launch in total.
__global__ void __launch_bounds__(kScanThreads) scan_single_cta(const u32 *__restrict__ in, u32 *__restrict__ out,
                                                                size_t n_max, const u32 *__restrict__ n_dev) {
  const size_t n = n_dev ? min((size_t)*n_dev, n_max) : n_max;
  __shared__ u32 total;
  u32 carry = 0;
  for (size_t t0 = 0; t0 <= n; t0 += HCTR_SCAN_TILE) {
    const size_t base = t0 + (size_t)threadIdx.x * kScanItems;
    u32 v[kScanItems];
    u32 s = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; k++) {
      v[k] = (base + k < n) ? in[base + k] : 0;
      s += v[k];
    }
    u32 ex = block_excl_scan(s, &total) + carry;
#pragma unroll
    for (int k = 0; k < kScanItems; k++) {
      if (base + k <= n) out[base + k] = ex;
      ex += v[k];
    }
    carry += total;
    __syncthreads();
  }
}

// Single-launch scan for any size: tile-local scan + chained prefix over the preceding tiles.
__global__ void __launch_bounds__(kScanThreads) scan_chained(const u32 *__restrict__ in, u32 *__restrict__ out,
                                                             size_t n_max, const u32 *__restrict__ n_dev,
                                                             u64 *agg, u32 epoch, u32 *err) {
  const size_t n = n_dev ? min((size_t)*n_dev, n_max) : n_max;
  const size_t base = (size_t)blockIdx.x * HCTR_SCAN_TILE + (size_t)threadIdx.x * kScanItems;
  u32 v[kScanItems];
  u32 s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    v[k] = (base + k < n) ? in[base + k] : 0;
    s += v[k];
  }
  __shared__ u32 total;
  u32 ex = block_excl_scan(s, &total);
  ex += chained_cta_prefix(agg, epoch, blockIdx.x, total, err);
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    if (base + k <= n) out[base + k] = ex;  // entry n receives the grand total
    ex += v[k];
  }
}

}  // namespace hctr

using namespace hctr;

unsigned long long hctr::g_launches = 0;

extern "C" unsigned long long hctr_launch_count(void) { return __atomic_load_n(&hctr::g_launches, __ATOMIC_RELAXED); }

extern "C" size_t hctr_scan_scratch_words(size_t n_max) { return (n_max + 1) / HCTR_SCAN_TILE + 2; }

extern "C" int hctr_scan_exclusive_u32(const uint32_t *in, uint32_t *out, size_t n_max, const uint32_t *n_dev,
                                       uint32_t *scratch, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  // n+1 outputs: tiles cover [0, n_max]
  const size_t tiles = (n_max + 1 + HCTR_SCAN_TILE - 1) / HCTR_SCAN_TILE;
  if (tiles <= 4) {
    scan_single_cta<<<1, kScanThreads, 0, s>>>(in, out, n_max, n_dev);
    count_launches(1);
    return launch_status();
  }
  scan_tile_sums<<<(unsigned)tiles, kScanThreads, 0, s>>>(in, n_max, n_dev, scratch);
  scan_apply<<<(unsigned)tiles, kScanThreads, 0, s>>>(in, out, n_max, n_dev, scratch);
  count_launches(2);
  return launch_status();
}

// ------------------------------------------------------------------------------------------------
// Prefix sum for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a scan: code running
// inside a framework's memory-pool callback, a real-time loop whose latency budget excludes the
// driver's allocator lock, or a plugin that is only handed input/output buffers and has no allocator
// of its own.  For them the tile-sum scratch of the scan lives in a file-scope device array that
// every GPU loading this library holds until the process exits (64 KB).
//
// Host code cannot pass `g_noalloc_scan_scratch` to a kernel: in host code that name is only a handle
// of the symbol, not a device address.  The address is obtained once per device with
// cudaGetSymbolAddress, with that device current, and cached.
// ------------------------------------------------------------------------------------------------
namespace hctr {
constexpr size_t kNoAllocScratchWords = HCTR_NOALLOC_SCAN_MAX / HCTR_SCAN_TILE + 2;
static __device__ __align__(256) u32 g_noalloc_scan_scratch[kNoAllocScratchWords];
constexpr int kMaxDevices = 64;
static u32 *g_noalloc_scratch_addr[kMaxDevices] = {};
static thread_local char g_noalloc_error[256] = "";
}  // namespace hctr

extern "C" const char *hctr_noalloc_last_error(void) { return g_noalloc_error; }

extern "C" int hctr_scan_exclusive_u32_noalloc(const uint32_t *in, uint32_t *out, size_t n, void *stream) {
  g_noalloc_error[0] = 0;
  if (n > (size_t)HCTR_NOALLOC_SCAN_MAX) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error),
             "hctr_scan_exclusive_u32_noalloc: n = %zu exceeds the built-in scratch (at most %zu elements); "
             "use hctr_scan_exclusive_u32 with caller-provided scratch",
             n, (size_t)HCTR_NOALLOC_SCAN_MAX);
    return (int)cudaErrorInvalidValue;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "hctr_scan_exclusive_u32_noalloc: no usable current device");
    return (int)(e != cudaSuccess ? e : cudaErrorInvalidDevice);
  }
  // First call on this device: look the scratch array's device address up (no allocation happens).
  u32 *scratch = __atomic_load_n(&g_noalloc_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (!scratch) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scan_scratch);
    if (e != cudaSuccess || !p) {
      snprintf(g_noalloc_error, sizeof(g_noalloc_error), "hctr_scan_exclusive_u32_noalloc: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(e));
      return (int)(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
    }
    scratch = static_cast<u32 *>(p);
    __atomic_store_n(&g_noalloc_scratch_addr[dev], scratch, __ATOMIC_RELEASE);
  }
  cudaStream_t s = (cudaStream_t)stream;
  const size_t tiles = (n + 1 + HCTR_SCAN_TILE - 1) / HCTR_SCAN_TILE;
  // Every tile sum the second kernel reads is written by the first one in the same call, so nothing in the
  // shared scratch has to start at zero and what an earlier call left there is never read.
  scan_tile_sums<<<(unsigned)tiles, kScanThreads, 0, s>>>(in, n, nullptr, scratch);
  scan_apply<<<(unsigned)tiles, kScanThreads, 0, s>>>(in, out, n, nullptr, scratch);
  count_launches(2);
  return launch_status();
}

extern "C" size_t hctr_scan_chained_scratch_words(size_t n_max) { return 2 * ((n_max + 1) / HCTR_SCAN_TILE + 2); }

extern "C" int hctr_scan_exclusive_u32_chained(const uint32_t *in, uint32_t *out, size_t n_max, const uint32_t *n_dev,
                                               uint32_t *scratch, uint32_t epoch, uint32_t *err, void *stream) {
  if (epoch == 0) return (int)cudaErrorInvalidValue;
  const size_t tiles = (n_max + 1 + HCTR_SCAN_TILE - 1) / HCTR_SCAN_TILE;
  scan_chained<<<(unsigned)tiles, kScanThreads, 0, (cudaStream_t)stream>>>(
      in, out, n_max, n_dev, reinterpret_cast<u64 *>(scratch), epoch, err);
  count_launches(1);
  return launch_status();
}
