// gather_qmm: out[i] = x[lhs[i]] * dequant(w[rhs[i]])  (GatherQMM::eval_gpu,
// mlx/backend/cuda/quantized/quantized.cpp:154-278; CPU semantics
// mlx/backend/cpu/quantized.cpp:700-747).
#include "common.cuh"
#include "kernels.h"

using namespace b200q;

extern "C" size_t b200q_gather_qmm_workspace_bytes(int dtype, int64_t n_idx, int64_t x_batch, int64_t E,
                                                   int64_t M, int64_t N, int64_t K, int group_size, int bits,
                                                   int transpose) {
  (void)dtype; (void)n_idx; (void)x_batch; (void)E; (void)M; (void)N; (void)K;
  (void)group_size; (void)bits; (void)transpose;
  return 256;  // status word only
}

extern "C" int b200q_gather_qmm(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                                const uint32_t* lhs_idx, const uint32_t* rhs_idx, int64_t n_idx, void* y,
                                int dtype, int64_t x_batch, int64_t E, int64_t M, int64_t N, int64_t K,
                                int group_size, int bits, int transpose, int sorted_flags, void* ws,
                                size_t ws_bytes, void* stream) {
  (void)sorted_flags;
  if (dtype != B200Q_F32 && dtype != B200Q_F16 && dtype != B200Q_BF16)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm] Only real floating types are supported (dtype code %d).", dtype);
  if (!valid_group(group_size))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm] Quantization group size must be 32, 64 or 128 (got %d).", group_size);
  if (!valid_bits(bits))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm] Quantization bits must be 2, 3, 4, 5, 6 or 8 (got %d).", bits);
  if (n_idx < 0 || x_batch < 0 || E < 0 || M < 0 || N < 0 || K < 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm] negative dimension.");
  const int64_t qaxis = transpose ? K : N;
  if (qaxis % group_size != 0 || (qaxis * bits) % 32 != 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT,
                "[gather_qmm] The shapes of the weight and scales are incompatible based on bits and group_size: "
                "quantized axis %lld with group_size=%d and bits=%d", (long long)qaxis, group_size, bits);
  if (x_batch > UINT32_MAX || E > UINT32_MAX || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
    return fail(B200Q_ERR_UNSUPPORTED, "[gather_qmm] No implementation for problem shape: dimension too large.");
  if (n_idx == 0 || M == 0 || N == 0) return B200Q_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0) {
    B200Q_CUDA_OK(cudaMemsetAsync(y, 0, (size_t)n_idx * M * N * dtype_size(dtype), st));
    return B200Q_OK;
  }
  if (!x || !wq || !scales || !biases || !lhs_idx || !rhs_idx || !y)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm] null pointer");
  if (!ws || ws_bytes < kStatusBytes)
    return fail(B200Q_ERR_WORKSPACE, "[gather_qmm] workspace of %zu bytes required, %zu given",
                b200q_gather_qmm_workspace_bytes(dtype, n_idx, x_batch, E, M, N, K, group_size, bits, transpose), ws_bytes);

  QmmArgs a{};
  a.x = x; a.wq = wq; a.scales = scales; a.biases = biases; a.y = y;
  a.dtype = dtype; a.batch = n_idx; a.M = M; a.N = N; a.K = K;
  a.group = group_size; a.bits = bits; a.transpose = transpose != 0; a.w_batched = true;
  a.ws = ws; a.ws_bytes = ws_bytes;
  GatherIdx gi{lhs_idx, rhs_idx, (uint32_t)x_batch, (uint32_t)E,
               reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + ws_bytes - kStatusBytes)};
  return qmm_generic(a, st, &gi);
}
