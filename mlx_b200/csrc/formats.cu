// GGUF quantized blocks -> the affine layout of this library (group size 32), on the device.
// Replaces the host loops extract_q4_0_data / extract_q4_1_data / extract_q8_0_data of the
// reference (mlx/io/gguf_quants.cpp:11-102), which repack on the CPU before upload.  Pure byte
// shuffling: one thread per 32-weight block, whole-block vector stores.
#include "common.cuh"
#include "kernels.h"

namespace b200q {
namespace {

__device__ __forceinline__ uint32_t ld_u16(const unsigned short* p) { return (uint32_t)__ldg(p); }

// TYPE: 2 = Q4_0 (18 B), 3 = Q4_1 (20 B), 8 = Q8_0 (34 B); blocks are 2-byte aligned.
template <int TYPE>
__global__ void __launch_bounds__(256)
gguf_repack_kernel(const unsigned short* __restrict__ blocks, int64_t n_blocks, uint32_t* __restrict__ wq,
                   __half* __restrict__ scales, __half* __restrict__ biases) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_blocks) return;
  constexpr int kHalves = TYPE == 2 ? 9 : (TYPE == 3 ? 10 : 17);
  const unsigned short* b = blocks + i * kHalves;
  const __half d = __ushort_as_half((unsigned short)ld_u16(b));
  scales[i] = d;
  if constexpr (TYPE == 8) {
    biases[i] = __hmul(__float2half(-128.0f), d);
    uint32_t out[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const uint32_t lo = ld_u16(b + 1 + 2 * w), hi = ld_u16(b + 2 + 2 * w);
      out[w] = (lo | (hi << 16)) ^ 0x80808080u;   // int8 -> unsigned field: flip the sign bit
    }
    uint4* o = reinterpret_cast<uint4*>(wq + i * 8);
    o[0] = make_uint4(out[0], out[1], out[2], out[3]);
    o[1] = make_uint4(out[4], out[5], out[6], out[7]);
  } else {
    const unsigned short* q = b + (TYPE == 2 ? 1 : 2);
    if constexpr (TYPE == 2) biases[i] = __hmul(__float2half(-8.0f), d);
    else biases[i] = __ushort_as_half((unsigned short)ld_u16(b + 1));
    // byte j holds weight j (low nibble) and weight j + 16 (high nibble); the affine layout wants
    // weights 0..31 as consecutive nibbles: words 0-1 from the low nibbles, words 2-3 from the high
    uint32_t src[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) src[w] = ld_u16(q + 2 * w) | (ld_u16(q + 2 * w + 1) << 16);
    uint32_t out[4];
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        // eight source bytes (src[2w], src[2w+1]) -> one word of eight nibbles
        uint32_t r = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t byte = (src[2 * w + j / 4] >> (8 * (j % 4))) & 0xFFu;
          r |= ((half ? (byte >> 4) : (byte & 0xFu))) << (4 * j);
        }
        out[2 * half + w] = r;
      }
    *reinterpret_cast<uint4*>(wq + i * 4) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int b200q_gguf_repack(const void* blocks, int gguf_type, int64_t n_blocks, uint32_t* wq, void* scales,
                                 void* biases, void* stream) {
  if (gguf_type != 2 && gguf_type != 3 && gguf_type != 8)
    return fail(B200Q_ERR_UNSUPPORTED, "[gguf_repack] only Q4_0 (2), Q4_1 (3) and Q8_0 (8) blocks are supported (got type %d)", gguf_type);
  if (n_blocks < 0) return fail(B200Q_ERR_INVALID_ARGUMENT, "[gguf_repack] negative block count");
  if (n_blocks == 0) return B200Q_OK;
  if (!blocks || !wq || !scales || !biases) return fail(B200Q_ERR_INVALID_ARGUMENT, "[gguf_repack] null pointer");
  if ((reinterpret_cast<uintptr_t>(blocks) & 1) || (reinterpret_cast<uintptr_t>(wq) & 15))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gguf_repack] blocks must be 2-byte aligned and the packed output 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((n_blocks + 255) / 256);
  const unsigned short* b = static_cast<const unsigned short*>(blocks);
  if (gguf_type == 2) gguf_repack_kernel<2><<<grid, 256, 0, st>>>(b, n_blocks, wq, (__half*)scales, (__half*)biases);
  else if (gguf_type == 3) gguf_repack_kernel<3><<<grid, 256, 0, st>>>(b, n_blocks, wq, (__half*)scales, (__half*)biases);
  else gguf_repack_kernel<8><<<grid, 256, 0, st>>>(b, n_blocks, wq, (__half*)scales, (__half*)biases);
  B200Q_LAUNCH_OK("gguf_repack_kernel");
  return B200Q_OK;
}
