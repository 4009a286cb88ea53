// Shared device helpers for the HetuTable kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "hctr_kernels.h"

namespace hctr {

constexpr int kSMs = 148;  // B200: 2 dies x 74 SMs; persistent grids are sized in multiples of this

typedef unsigned long long u64;
typedef uint32_t u32;

static inline int launch_status() { return (int)cudaGetLastError(); }

// Kernels enqueued by this library since load (every launcher adds what it launched).
extern unsigned long long g_launches;
static inline void count_launches(int n) { __atomic_fetch_add(&g_launches, (unsigned long long)n, __ATOMIC_RELAXED); }

static inline unsigned grid_for(size_t n, unsigned block) {
  size_t g = (n + block - 1) / block;
  return (unsigned)(g == 0 ? 1 : g);
}

// 16-byte accesses with cache hints.  Gradient input and dst output are touched exactly once per
// step (streamed: evict-first); table rows are re-read by duplicates and by the next kernels, so they
// use default caching and stay in the 126 MB L2.
__device__ __forceinline__ float4 ld_stream(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4 *p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ float4 f4_add(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
__device__ __forceinline__ float4 f4_scale(float4 a, float s) {
  return make_float4(a.x * s, a.y * s, a.z * s, a.w * s);
}

__device__ __forceinline__ bool aligned16(const void *p) { return (((uintptr_t)p) & 15) == 0; }

// Chained prefix across the CTAs of one launch.  CTA `cta` publishes its total, tagged with the launch's
// epoch, then adds up the totals of all CTAs before it.  CTAs are dispatched in index order and a CTA
// only ever waits for lower-indexed ones, so the wait cannot deadlock; it is bounded all the same and
// reports through `err` (HCTR_ERR_TIMEOUT) instead of spinning forever.  `agg` holds one 64-bit word
// per CTA and needs no initialisation as long as epochs differ between launches (0 is never used).
// All threads of the CTA must call it; the result is returned to every thread.
__device__ __forceinline__ u32 chained_cta_prefix(u64 *agg, u32 epoch, u32 cta, u32 total, u32 *err) {
  __shared__ u32 s_part[32];
  __shared__ u32 s_prefix;
  const unsigned tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = (blockDim.x + 31) >> 5;
  if (tid == 0) {
    const u64 v = ((u64)epoch << 32) | total;
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(agg + cta), "l"(v) : "memory");
  }
  u32 sum = 0;
  for (u32 j = tid; j < cta; j += blockDim.x) {
    u64 v = 0;
    u32 spins = 0;
    for (;;) {
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(agg + j) : "memory");
      if ((u32)(v >> 32) == epoch) break;
      if (++spins > 4000000u) {  // ~ a second: a predecessor never published
        atomicOr(err, HCTR_ERR_TIMEOUT);
        v = 0;
        break;
      }
      __nanosleep(100);
    }
    sum += (u32)v;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  if (lane == 0) s_part[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    u32 v = lane < nwarp ? s_part[lane] : 0;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    if (lane == 0) s_prefix = v;
  }
  __syncthreads();
  return s_prefix;
}

// Number of lanes that cooperate on one row: W/4 float4 per row, capped at a warp, at least 1.
// Power of two so groups tile a warp.
static inline int lanes_per_row(size_t width) {
  size_t v = width / 4;
  int g = 1;
  while (g < 32 && (size_t)(g * 2) <= v) g *= 2;
  return g;
}

}  // namespace hctr
