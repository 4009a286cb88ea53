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

// Number of lanes that cooperate on one row: W/4 float4 per row, capped at a warp, at least 1.
// Power of two so groups tile a warp.
static inline int lanes_per_row(size_t width) {
  size_t v = width / 4;
  int g = 1;
  while (g < 32 && (size_t)(g * 2) <= v) g *= 2;
  return g;
}

}  // namespace hctr
