// Shared helpers for the b200q kernels: error reporting, element-type traits and
// the bit-stream accessors of the packed weight layout.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/b200q.h"

namespace b200q {

// ---- host side --------------------------------------------------------------------
// Records a formatted message in the calling thread's error slot and returns `code`.
int fail(int code, const char* fmt, ...);
void count_launch(int n = 1);

#define B200Q_CUDA_OK(expr)                                                          \
  do {                                                                               \
    cudaError_t e__ = (expr);                                                        \
    if (e__ != cudaSuccess)                                                          \
      return ::b200q::fail(B200Q_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

// cudaGetLastError after a launch; kernels are launched with <<<>>> on `stream`.
#define B200Q_LAUNCH_OK(name)                                                        \
  do {                                                                               \
    cudaError_t e__ = cudaGetLastError();                                            \
    if (e__ != cudaSuccess)                                                          \
      return ::b200q::fail(B200Q_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
    ::b200q::count_launch();                                                         \
  } while (0)

inline bool valid_group(int g) { return g == 32 || g == 64 || g == 128; }
inline bool valid_bits(int b) { return b >= 2 && b <= 8 && b != 7; }
inline size_t dtype_size(int dt) { return dt == B200Q_F32 ? 4 : 2; }

// Workspace layout shared by the matmul kernels.  The trailing 16 bytes hold the
// device status word (4 x uint32); counters and partial sums come first.
constexpr size_t kStatusBytes = 16;

// ---- device side ------------------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float to_float(float v) { return v; }
  static __device__ __forceinline__ float from_float(float v) { return v; }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

// Value k of a row stored as an LSB-first bit stream of `bits`-wide fields; `row`
// points at the first 32-bit word of the row.  Reads one or two aligned words.
template <int BITS>
__device__ __forceinline__ uint32_t stream_get(const uint32_t* __restrict__ row, int64_t k) {
  const int64_t bit = k * BITS;
  const int64_t word = bit >> 5;
  const int sh = (int)(bit & 31);
  uint32_t lo = row[word];
  if constexpr (32 % BITS == 0) {
    return (lo >> sh) & ((1u << BITS) - 1u);
  } else {
    uint32_t hi = (sh + BITS > 32) ? row[word + 1] : 0u;
    return __funnelshift_r(lo, hi, sh) & ((1u << BITS) - 1u);
  }
}

__device__ __forceinline__ uint32_t stream_get_rt(const uint32_t* __restrict__ row, int64_t k, int bits) {
  const int64_t bit = k * bits;
  const int64_t word = bit >> 5;
  const int sh = (int)(bit & 31);
  uint32_t lo = row[word];
  uint32_t hi = (sh + bits > 32) ? row[word + 1] : 0u;
  return __funnelshift_r(lo, hi, sh) & ((1u << bits) - 1u);
}

// Dispatch a runtime `bits` value to a compile-time template argument.
#define B200Q_DISPATCH_BITS(bits, BITS, ...)        \
  switch (bits) {                                   \
    case 2: { constexpr int BITS = 2; __VA_ARGS__; } break; \
    case 3: { constexpr int BITS = 3; __VA_ARGS__; } break; \
    case 4: { constexpr int BITS = 4; __VA_ARGS__; } break; \
    case 5: { constexpr int BITS = 5; __VA_ARGS__; } break; \
    case 6: { constexpr int BITS = 6; __VA_ARGS__; } break; \
    case 8: { constexpr int BITS = 8; __VA_ARGS__; } break; \
    default: break;                                 \
  }

}  // namespace b200q
