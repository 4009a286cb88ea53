// Set-up side of the path: storage layout, key -> row table, version init, value init.
#include <thrust/random.h>

#include "common.cuh"

namespace hctr {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads) storage_flags(const long long *__restrict__ storage, size_t n,
                                                          size_t length, const uint8_t *__restrict__ owner_of,
                                                          int rank, u32 *__restrict__ is_cached, u32 *err) {
  const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n) return;
  const long long k = storage[i];
  if (k < 0 || (size_t)k >= length) {
    atomicOr(err, HCTR_ERR_KEY_RANGE);
    is_cached[i] = 0;
    return;
  }
  is_cached[i] = owner_of[k] != rank ? 1u : 0u;
}

// Stable two-way split: cached keys keep their relative order at the front, owned keys follow.
__global__ void __launch_bounds__(kThreads) storage_layout(const long long *__restrict__ storage, size_t n,
                                                           const u32 *__restrict__ is_cached,
                                                           const u32 *__restrict__ cached_before,
                                                           long long *__restrict__ stored_keys) {
  const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n) return;
  const size_t n_cached = cached_before[n];
  const size_t before = cached_before[i];
  const size_t dst = is_cached[i] ? before : n_cached + (i - before);
  stored_keys[dst] = storage[i];
}

__global__ void __launch_bounds__(kThreads) table_build(const long long *__restrict__ stored_keys, size_t n,
                                                        size_t n_cached, size_t length, int32_t *row_of,
                                                        long long *__restrict__ version, u32 *err) {
  const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n) return;
  version[i] = i < n_cached ? INT64_MIN : 0;
  const long long k = stored_keys[i];
  if (k < 0 || (size_t)k >= length) {
    atomicOr(err, HCTR_ERR_KEY_RANGE);
    return;
  }
  if (atomicCAS(&row_of[k], HCTR_INVALID_ROW, (int32_t)i) != HCTR_INVALID_ROW) atomicOr(err, HCTR_ERR_CAPACITY);
}

__global__ void __launch_bounds__(kThreads) count_owned(const uint8_t *__restrict__ owner_of, size_t length,
                                                        int rank, u64 *n_owned) {
  u64 c = 0;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < length; i += (size_t)gridDim.x * kThreads)
    c += owner_of[i] == rank;
  for (int d = 16; d > 0; d >>= 1) c += __shfl_down_sync(0xffffffffu, c, d);
  if ((threadIdx.x & 31) == 0 && c) atomicAdd(n_owned, c);
}

// Value init.  Element i restarts a minstd engine from `seed`, skips i draws, then samples: the value
// is a function of (seed, local element index) only, identical on every rank.
__global__ void __launch_bounds__(kThreads) init_values(float *__restrict__ data, size_t len, int kind, float a,
                                                        float b, unsigned int seed) {
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < len; i += (size_t)gridDim.x * kThreads) {
    thrust::minstd_rand rng(seed);
    rng.discard(i);
    float v;
    if (kind == 2) {
      thrust::uniform_real_distribution<float> d(a, b);
      v = d(rng);
    } else {
      thrust::normal_distribution<float> d(a, b);
      v = d(rng);
      if (kind == 3) {
        // rejection with a re-seed from the engine's own next output until inside mean +- 2 sigma
        while (v > a + 2 * b || v < a - 2 * b) {
          rng.seed(rng());
          v = d(rng);
        }
      }
    }
    data[i] = v;
  }
}

}  // namespace hctr

using namespace hctr;

extern "C" int hctr_storage_flags(const int64_t *storage, size_t n, size_t length, const uint8_t *owner_of,
                                  int rank, uint32_t *is_cached, uint32_t *err, void *stream) {
  if (n == 0) return 0;
  storage_flags<<<grid_for(n, kThreads), kThreads, 0, (cudaStream_t)stream>>>((const long long *)storage, n, length,
                                                                             owner_of, rank, is_cached, err);
  return launch_status();
}

extern "C" int hctr_storage_layout(const int64_t *storage, size_t n, const uint32_t *is_cached,
                                   const uint32_t *cached_before, int64_t *stored_keys, void *stream) {
  if (n == 0) return 0;
  storage_layout<<<grid_for(n, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
      (const long long *)storage, n, is_cached, cached_before, (long long *)stored_keys);
  return launch_status();
}

extern "C" int hctr_table_build(const int64_t *stored_keys, size_t n, size_t n_cached, size_t length,
                                int32_t *row_of, int64_t *version, uint32_t *err, void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(row_of, 0xFF, length * sizeof(int32_t), s);
  if (e != cudaSuccess) return (int)e;
  if (n == 0) return 0;
  table_build<<<grid_for(n, kThreads), kThreads, 0, s>>>((const long long *)stored_keys, n, n_cached, length, row_of,
                                                         (long long *)version, err);
  return launch_status();
}

extern "C" int hctr_count_owned(const uint8_t *owner_of, size_t length, int rank, unsigned long long *n_owned,
                                void *stream) {
  count_owned<<<kSMs * 8, kThreads, 0, (cudaStream_t)stream>>>(owner_of, length, rank, n_owned);
  return launch_status();
}

extern "C" int hctr_initialize(float *data, size_t len, int kind, float a, float b, unsigned int seed,
                               void *stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (len == 0) return 0;
  if (kind == 0) return (int)cudaMemsetAsync(data, 0, len * sizeof(float), s);
  if (kind < 0 || kind > 3) return (int)cudaErrorInvalidValue;
  init_values<<<kSMs * 16, kThreads, 0, s>>>(data, len, kind, a, b, seed);
  return launch_status();
}
