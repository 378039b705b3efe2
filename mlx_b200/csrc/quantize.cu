// Affine group-wise quantize / dequantize kernels (HBM-bound element-wise work).
//
// quantize reproduces, bit for bit, the float arithmetic of the reference CPU
// implementation quantize<T,U> (mlx/backend/cpu/quantized.cpp:1148-1211): three IEEE
// divisions, rint (round half to even), clamp to [0, 2^bits-1], scale/bias rounded to
// T with round-to-nearest-even.  dequantize reproduces the op-composed reference
// (mlx/ops.cpp:5320-5323): multiply then add, each rounded to T.
//
// Data layout: every thread owns 8 consecutive values of the flattened [rows*K]
// tensor (one 128-bit load for 16-bit types).  A group of g values is owned by g/8
// adjacent lanes, which combine min/max with xor-shuffles.  The 8*bits packed bits of
// a thread are merged across each 4-lane quad so that global stores are whole 32-bit
// words for every bit width (3-, 5- and 6-bit fields straddle word boundaries).
#include "common.cuh"

namespace b200q {
namespace {

template <typename T>
__device__ __forceinline__ void load8(const T* __restrict__ p, float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    float4 a = __ldg(reinterpret_cast<const float4*>(p));
    float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = Elem<T>::to_float(e[i]);
  }
}

template <typename T>
__device__ __forceinline__ void store8(T* __restrict__ p, const float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = Elem<T>::from_float(v[i]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
}

template <typename T, int BITS, int GROUP>
__global__ void __launch_bounds__(256)
quantize_kernel(const T* __restrict__ w, uint32_t* __restrict__ wq, T* __restrict__ scales,
                T* __restrict__ biases, int64_t n_chunks) {
  constexpr int LPG = GROUP / 8;  // lanes per group
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = c < n_chunks;
  const int lane = threadIdx.x & 31;

  float v[8];
  float w_min = INFINITY, w_max = -INFINITY;
  if (active) {
    load8(w + c * 8, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      w_max = (w_max < v[i]) ? v[i] : w_max;
      w_min = (v[i] < w_min) ? v[i] : w_min;
    }
  }
#pragma unroll
  for (int off = 1; off < LPG; off <<= 1) {
    float omax = __shfl_xor_sync(0xffffffffu, w_max, off);
    float omin = __shfl_xor_sync(0xffffffffu, w_min, off);
    w_max = (w_max < omax) ? omax : w_max;
    w_min = (omin < w_min) ? omin : w_min;
  }

  constexpr float n_bins = (float)((1 << BITS) - 1);
  const float eps = 1e-7f;
  const bool mask = fabsf(w_min) > fabsf(w_max);
  float scale = __fdiv_rn(__fsub_rn(w_max, w_min), n_bins);
  scale = (scale < eps) ? eps : scale;
  scale = mask ? scale : -scale;
  const float edge = mask ? w_min : w_max;
  const float q0 = rintf(__fdiv_rn(edge, scale));
  float bias = 0.0f;
  if (q0 != 0.0f) {
    scale = __fdiv_rn(edge, q0);
    bias = edge;
  }

  uint64_t packed = 0;
  if (active) {
    // q = rint((w - bias) / scale) with the IEEE division of the reference, but the division is
    // only carried out where it can matter: t = (w - bias) * (1 / scale) is within 1.2e-7 * |t|
    // of the true quotient, so rint(t) equals rint of the rounded quotient unless t lies within
    // that distance of a rounding tie k + 1/2.  Below |t| = 512 that is less than 1e-4; above, both
    // roundings clamp to the same bin.  Threads that see a t closer than 1e-4 to a tie (or a NaN)
    // redo their eight values with the exact division.
    const float inv = __frcp_rn(scale);
    float q[8];
    bool redo = !(fabsf(scale) < 1e30f);   // 1/scale would lose bits as a subnormal
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float t = __fmul_rn(__fsub_rn(v[i], bias), inv);
      q[i] = rintf(t);
      redo |= !(fabsf(fabsf(__fsub_rn(t, q[i])) - 0.5f) >= 1e-4f);   // also true for NaN
    }
    if (redo) {
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = rintf(__fdiv_rn(__fsub_rn(v[i], bias), scale));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float qi = (q[i] < 0.0f) ? 0.0f : q[i];
      qi = (n_bins < qi) ? n_bins : qi;
      packed |= (uint64_t)(uint32_t)qi << (i * BITS);
    }
    if ((c % LPG) == 0) {
      scales[c / LPG] = Elem<T>::from_float(scale);
      biases[c / LPG] = Elem<T>::from_float(bias);
    }
  }

  // 4 and 8 bits: a thread's eight fields are exactly one or two words.
  if constexpr (BITS == 4) {
    if (active) wq[c] = (uint32_t)packed;
    return;
  } else if constexpr (BITS == 8) {
    if (active) reinterpret_cast<uint2*>(wq)[c] = make_uint2((uint32_t)packed, (uint32_t)(packed >> 32));
    return;
  }
  // Merge the four 8*BITS-bit fragments of a quad into BITS whole words.
  constexpr int SEG = 8 * BITS;
  const int qbase = lane & ~3;
  uint64_t seg[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t lo = __shfl_sync(0xffffffffu, (uint32_t)packed, qbase + j);
    uint32_t hi = __shfl_sync(0xffffffffu, (uint32_t)(packed >> 32), qbase + j);
    seg[j] = ((uint64_t)hi << 32) | lo;
  }
  if (active) {
    uint32_t* out = wq + (c >> 2) * BITS;
    const int l = lane & 3;
#pragma unroll
    for (int i = 0; i < BITS; ++i) {
      const int p = 32 * i;
      const int j = p / SEG;
      const int o = p % SEG;
      uint64_t word = seg[j] >> o;
      if (SEG - o < 32 && j + 1 < 4) word |= seg[j + 1] << (SEG - o);
      if ((i & 3) == l) out[i] = (uint32_t)word;
    }
  }
}

template <typename T, int BITS>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint32_t* __restrict__ wq, const T* __restrict__ scales,
                  const T* __restrict__ biases, T* __restrict__ out, int64_t n_chunks,
                  int group_shift /* log2(group/8) */, int64_t n_words) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n_chunks) return;
  // The 8 fields of chunk c start at byte c*BITS; fetch the covering aligned words.
  const int64_t byte = c * BITS;
  const int64_t w0 = byte >> 2;
  const int sh = (int)(byte & 3) * 8;
  uint32_t a = __ldg(wq + w0);
  uint32_t b = (w0 + 1 < n_words) ? __ldg(wq + w0 + 1) : 0u;
  // 8*BITS <= 64 bits starting at a byte offset of 0..3 inside `a`: for every supported
  // width the fields end within the first 64 bits, so two words suffice.
  uint64_t bitsv = ((uint64_t)(b >> sh) << 32) | __funnelshift_r(a, b, sh);
  const int64_t g = c >> group_shift;
  const float s = Elem<T>::to_float(scales[g]);
  const float bs = Elem<T>::to_float(biases[g]);
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float q = (float)(uint32_t)((bitsv >> (i * BITS)) & ((1u << BITS) - 1u));
    // multiply and add are separate operations of type T in the reference.
    float t = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(q, s)));
    v[i] = __fadd_rn(t, bs);
  }
  store8(out + c * 8, v);
}

template <typename T>
int launch_quantize(const T* w, int64_t n_elems, int group, int bits, uint32_t* wq, T* s, T* b,
                    cudaStream_t st) {
  const int64_t n_chunks = n_elems / 8;
  if (n_chunks == 0) return B200Q_OK;
  const unsigned grid = (unsigned)((n_chunks + 255) / 256);
  bool done = false;
  B200Q_DISPATCH_BITS(bits, BITS, {
    if (group == 32) quantize_kernel<T, BITS, 32><<<grid, 256, 0, st>>>(w, wq, s, b, n_chunks);
    else if (group == 64) quantize_kernel<T, BITS, 64><<<grid, 256, 0, st>>>(w, wq, s, b, n_chunks);
    else quantize_kernel<T, BITS, 128><<<grid, 256, 0, st>>>(w, wq, s, b, n_chunks);
    done = true;
  });
  if (!done) return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantize] unsupported bits %d", bits);
  B200Q_LAUNCH_OK("quantize_kernel");
  return B200Q_OK;
}

template <typename T>
int launch_dequantize(const uint32_t* wq, const T* s, const T* b, int64_t n_elems, int group,
                      int bits, T* out, cudaStream_t st) {
  const int64_t n_chunks = n_elems / 8;
  if (n_chunks == 0) return B200Q_OK;
  const unsigned grid = (unsigned)((n_chunks + 255) / 256);
  const int gshift = group == 32 ? 2 : (group == 64 ? 3 : 4);
  const int64_t n_words = n_elems * bits / 32;
  bool done = false;
  B200Q_DISPATCH_BITS(bits, BITS, {
    dequantize_kernel<T, BITS><<<grid, 256, 0, st>>>(wq, s, b, out, n_chunks, gshift, n_words);
    done = true;
  });
  if (!done) return fail(B200Q_ERR_INVALID_ARGUMENT, "[dequantize] unsupported bits %d", bits);
  B200Q_LAUNCH_OK("dequantize_kernel");
  return B200Q_OK;
}

// Rows of the packed matrix chosen by `ids` (an embedding look-up): out[i, :] = dequantize(row ids[i]).
// An id outside [0, rows) gives a row of zeros; nothing is read for it.
template <typename T, int BITS>
__global__ void __launch_bounds__(256)
dequantize_rows_kernel(const uint32_t* __restrict__ wq, const T* __restrict__ scales,
                       const T* __restrict__ biases, const uint32_t* __restrict__ ids, T* __restrict__ out,
                       int64_t rows, int chunks_per_row, int group_shift, int64_t n_words) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= chunks_per_row) return;
  const int64_t i = blockIdx.y;
  const uint32_t id = __ldg(ids + i);
  T* dst = out + (i * chunks_per_row + c) * 8;
  float v[8];
  if ((int64_t)id >= rows) {
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = 0.f;
    store8(dst, v);
    return;
  }
  const int64_t cg = (int64_t)id * chunks_per_row + c;  // chunk index in the whole matrix
  const int64_t byte = cg * BITS;
  const int64_t w0 = byte >> 2;
  const int sh = (int)(byte & 3) * 8;
  uint32_t a = __ldg(wq + w0);
  uint32_t b = (w0 + 1 < n_words) ? __ldg(wq + w0 + 1) : 0u;
  uint64_t bitsv = ((uint64_t)(b >> sh) << 32) | __funnelshift_r(a, b, sh);
  const int64_t g = cg >> group_shift;
  const float s = Elem<T>::to_float(scales[g]);
  const float bs = Elem<T>::to_float(biases[g]);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float q = (float)(uint32_t)((bitsv >> (k * BITS)) & ((1u << BITS) - 1u));
    float t = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(q, s)));
    v[k] = __fadd_rn(t, bs);
  }
  store8(dst, v);
}

template <typename T>
int launch_dequantize_rows(const uint32_t* wq, const T* s, const T* b, const uint32_t* ids, int64_t n_ids,
                           int64_t rows, int64_t K, int group, int bits, T* out, cudaStream_t st) {
  const int cpr = (int)(K / 8);
  const int gshift = group == 32 ? 2 : (group == 64 ? 3 : 4);
  const int64_t n_words = rows * K * bits / 32;
  bool done = false;
  for (int64_t i0 = 0; i0 < n_ids; i0 += 65535) {   // gridDim.y limit
    const unsigned ny = (unsigned)((n_ids - i0) < 65535 ? (n_ids - i0) : 65535);
    dim3 grid((unsigned)((cpr + 255) / 256), ny);
    B200Q_DISPATCH_BITS(bits, BITS, {
      dequantize_rows_kernel<T, BITS><<<grid, 256, 0, st>>>(wq, s, b, ids + i0, out + i0 * K, rows, cpr, gshift, n_words);
      done = true;
    });
    if (!done) return fail(B200Q_ERR_INVALID_ARGUMENT, "[dequantize_rows] unsupported bits %d", bits);
    B200Q_LAUNCH_OK("dequantize_rows_kernel");
  }
  return B200Q_OK;
}

int check_quant_args(const char* tag, int dtype, int64_t rows, int64_t K, int group, int bits) {
  if (dtype != B200Q_F32 && dtype != B200Q_F16 && dtype != B200Q_BF16)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[%s] Only real floating types are supported (dtype code %d).", tag, dtype);
  if (!valid_group(group))
    return fail(B200Q_ERR_INVALID_ARGUMENT,
                "[%s] The requested group size %d is not supported. The supported group sizes are 32, 64, and 128.", tag, group);
  if (!valid_bits(bits))
    return fail(B200Q_ERR_INVALID_ARGUMENT,
                "[%s] The requested number of bits %d is not supported. The supported bits are 2, 3, 4, 5, 6 and 8.", tag, bits);
  if (rows < 0 || K < 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[%s] negative shape (%lld, %lld).", tag, (long long)rows, (long long)K);
  if (K % group != 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT,
                "[%s] The last dimension of the matrix needs to be divisible by the quantization group size %d. "
                "However the provided matrix has shape (%lld, %lld)", tag, group, (long long)rows, (long long)K);
  return B200Q_OK;
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int b200q_quantize(const void* w, int dtype, int64_t rows, int64_t K, int group_size,
                              int bits, uint32_t* wq, void* scales, void* biases, void* stream) {
  if (int rc = check_quant_args("quantize", dtype, rows, K, group_size, bits)) return rc;
  const int64_t n = rows * K;
  if (n == 0) return B200Q_OK;
  if (!w || !wq || !scales || !biases) return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantize] null pointer");
  if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(wq) & 3))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantize] w must be 16-byte aligned and wq 4-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200Q_F32:
      return launch_quantize<float>((const float*)w, n, group_size, bits, wq, (float*)scales, (float*)biases, st);
    case B200Q_F16:
      return launch_quantize<__half>((const __half*)w, n, group_size, bits, wq, (__half*)scales, (__half*)biases, st);
    default:
      return launch_quantize<__nv_bfloat16>((const __nv_bfloat16*)w, n, group_size, bits, wq,
                                            (__nv_bfloat16*)scales, (__nv_bfloat16*)biases, st);
  }
}

extern "C" int b200q_dequantize(const uint32_t* wq, const void* scales, const void* biases, int dtype,
                                int64_t rows, int64_t K, int group_size, int bits, void* out,
                                void* stream) {
  if (int rc = check_quant_args("dequantize", dtype, rows, K, group_size, bits)) return rc;
  const int64_t n = rows * K;
  if (n == 0) return B200Q_OK;
  if (!wq || !scales || !biases || !out) return fail(B200Q_ERR_INVALID_ARGUMENT, "[dequantize] null pointer");
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(wq) & 3))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[dequantize] out must be 16-byte aligned and wq 4-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200Q_F32:
      return launch_dequantize<float>(wq, (const float*)scales, (const float*)biases, n, group_size, bits, (float*)out, st);
    case B200Q_F16:
      return launch_dequantize<__half>(wq, (const __half*)scales, (const __half*)biases, n, group_size, bits, (__half*)out, st);
    default:
      return launch_dequantize<__nv_bfloat16>(wq, (const __nv_bfloat16*)scales, (const __nv_bfloat16*)biases, n,
                                              group_size, bits, (__nv_bfloat16*)out, st);
  }
}

extern "C" int b200q_dequantize_rows(const uint32_t* wq, const void* scales, const void* biases, const uint32_t* ids,
                                     int64_t n_ids, int dtype, int64_t rows, int64_t K, int group_size, int bits,
                                     void* out, void* stream) {
  if (int rc = check_quant_args("dequantize_rows", dtype, rows, K, group_size, bits)) return rc;
  if (n_ids < 0) return fail(B200Q_ERR_INVALID_ARGUMENT, "[dequantize_rows] negative number of ids (%lld).", (long long)n_ids);
  if (K / 8 > INT32_MAX) return fail(B200Q_ERR_UNSUPPORTED, "[dequantize_rows] row too long.");
  if (n_ids == 0 || K == 0) return B200Q_OK;
  if (!out || !ids) return fail(B200Q_ERR_INVALID_ARGUMENT, "[dequantize_rows] null pointer");
  if (rows > 0 && (!wq || !scales || !biases)) return fail(B200Q_ERR_INVALID_ARGUMENT, "[dequantize_rows] null pointer");
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(wq) & 3))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[dequantize_rows] out must be 16-byte aligned and wq 4-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200Q_F32:
      return launch_dequantize_rows<float>(wq, (const float*)scales, (const float*)biases, ids, n_ids, rows, K, group_size,
                                           bits, (float*)out, st);
    case B200Q_F16:
      return launch_dequantize_rows<__half>(wq, (const __half*)scales, (const __half*)biases, ids, n_ids, rows, K,
                                            group_size, bits, (__half*)out, st);
    default:
      return launch_dequantize_rows<__nv_bfloat16>(wq, (const __nv_bfloat16*)scales, (const __nv_bfloat16*)biases, ids,
                                                   n_ids, rows, K, group_size, bits, (__nv_bfloat16*)out, st);
  }
}
