// Row-granular helpers: a group of LANES consecutive lanes of a warp cooperates on one table row.
// VEC rows are moved as 16-byte float4 (width % 4 == 0 and 16-byte aligned bases); otherwise the same
// code runs element-wise on floats.
#pragma once
#include "common.cuh"

namespace hctr {

template <bool VEC>
struct RowT;
template <>
struct RowT<true> {
  typedef float4 T;
  static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ T add(T a, T b) {
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
  }
  static __device__ __forceinline__ T scale(T a, float s) {
    return make_float4(__fmul_rn(a.x, s), __fmul_rn(a.y, s), __fmul_rn(a.z, s), __fmul_rn(a.w, s));
  }
  static __device__ __forceinline__ T ld_once(const T *p) { return __ldcs(p); }
  static __device__ __forceinline__ void st_once(T *p, T v) { __stcs(p, v); }
  static __host__ __device__ __forceinline__ size_t elems(size_t width) { return width / 4; }
};
template <>
struct RowT<false> {
  typedef float T;
  static __device__ __forceinline__ T zero() { return 0.f; }
  static __device__ __forceinline__ T add(T a, T b) { return __fadd_rn(a, b); }
  static __device__ __forceinline__ T scale(T a, float s) { return __fmul_rn(a, s); }
  static __device__ __forceinline__ T ld_once(const T *p) { return __ldcs(p); }
  static __device__ __forceinline__ void st_once(T *p, T v) { __stcs(p, v); }
  static __host__ __device__ __forceinline__ size_t elems(size_t width) { return width; }
};

// Dispatch a kernel template <int LANES, bool VEC> on the row width and pointer alignment.
// `ptrs_aligned` must be true only if every row base pointer involved is 16-byte aligned.
#define HCTR_DISPATCH_ROWS(width, ptrs_aligned, CALL)           \
  do {                                                          \
    if (((width) % 4 == 0) && (ptrs_aligned)) {                 \
      const size_t v_ = (width) / 4;                            \
      if (v_ >= 32) { CALL(32, true); }                         \
      else if (v_ >= 16) { CALL(16, true); }                    \
      else if (v_ >= 8) { CALL(8, true); }                      \
      else if (v_ >= 4) { CALL(4, true); }                      \
      else if (v_ >= 2) { CALL(2, true); }                      \
      else { CALL(1, true); }                                   \
    } else {                                                    \
      if ((width) >= 32) { CALL(32, false); }                   \
      else if ((width) >= 8) { CALL(8, false); }                \
      else { CALL(1, false); }                                  \
    }                                                           \
  } while (0)

static inline bool host_aligned16(const void *p) { return (((uintptr_t)p) & 15) == 0; }

}  // namespace hctr
