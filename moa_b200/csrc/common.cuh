// Shared helpers for the moa_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moa_b200.h"

namespace moa {

// Last CUDA error text of the calling host thread (returned by moa_last_error_detail()).
void set_error_detail(const char* what, cudaError_t err);
void set_error_text(const char* what);

#define MOA_CUDA_CHECK(expr)                      \
  do {                                            \
    cudaError_t _e = (expr);                      \
    if (_e != cudaSuccess) {                      \
      moa::set_error_detail(#expr, _e);           \
      return MOA_ERR_CUDA;                        \
    }                                             \
  } while (0)

#define MOA_REQUIRE(cond, what)                   \
  do {                                            \
    if (!(cond)) {                                \
      moa::set_error_text(what);                  \
      return MOA_ERR_INVALID_ARG;                 \
    }                                             \
  } while (0)

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Python/torch integer modulo: the result takes the sign of the (positive) divisor.
__device__ __forceinline__ int64_t pymod(int64_t x, int64_t m) {
  int64_t r = x % m;
  return r < 0 ? r + m : r;
}

// Next write index of a ring after one append (MoA/attention/cache_utils.py:1041-1054).
__device__ __forceinline__ int64_t ring_next_index(int64_t upd, int64_t head_start, int64_t cap,
                                                   int64_t static_h, int64_t kv_len_before) {
  const int64_t cs = head_start + static_h;
  const int64_t circ = cap - static_h;
  if (kv_len_before + 1 > static_h && circ > 0) return pymod(upd + 1 - cs, circ) + cs;
  return upd + 1;
}

// 16-byte streaming load that does not allocate in L1 (cache rows are read once per step).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

template <typename T>
struct Cvt;
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<const __half2*>(&u));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    // bf16 -> fp32 is a 16-bit shift
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = Cvt<T>::unpack(u.x), b = Cvt<T>::unpack(u.y), c = Cvt<T>::unpack(u.z), d = Cvt<T>::unpack(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

}  // namespace moa
