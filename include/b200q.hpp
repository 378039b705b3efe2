// C++ host shim over the C ABI of b200q.h with the shape of the reference's operator functions
// (mlx/ops.cpp: quantize :5208-5245, dequantize :5465-5517, quantized_matmul :4784-4834,
// gather_qmm :5553-5629): same argument meaning, same validation (mlx/ops.cpp:110-181,
// 4704-4754), std::invalid_argument where the reference throws it and std::runtime_error for
// everything the library reports later.  Arrays are non-owning views of row-contiguous device
// memory; outputs and scratch are allocated by the caller (the reference's eval_gpu does that
// with its own allocator).  Header only; link with libb200q.so.
#pragma once

#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "b200q.h"

namespace b200q {

enum class Dtype : int { float32 = B200Q_F32, float16 = B200Q_F16, bfloat16 = B200Q_BF16, uint32 = 100 };

inline const char* name(Dtype t) {
  switch (t) {
    case Dtype::float32: return "float32";
    case Dtype::float16: return "float16";
    case Dtype::bfloat16: return "bfloat16";
    default: return "uint32";
  }
}
inline bool is_floating(Dtype t) { return t != Dtype::uint32; }

// Row-contiguous device array: shape + dtype + pointer.
struct ArrayView {
  void* data = nullptr;
  Dtype dtype = Dtype::float32;
  std::vector<int64_t> shape;
  int ndim() const { return (int)shape.size(); }
  int64_t dim(int i) const { return shape[i < 0 ? shape.size() + i : i]; }
  int64_t size() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
};

struct Workspace {  // scratch sized with b200q_*_workspace_bytes, zeroed once with b200q_workspace_init
  void* data = nullptr;
  size_t bytes = 0;
};

namespace detail {
inline std::string shape_str(const std::vector<int64_t>& s) {
  std::ostringstream o;
  o << "(";
  for (size_t i = 0; i < s.size(); ++i) o << (i ? "," : "") << s[i];
  o << ")";
  return o.str();
}
inline void check(int rc) {
  if (rc == B200Q_OK) return;
  if (rc == B200Q_ERR_INVALID_ARGUMENT) throw std::invalid_argument(b200q_last_error());
  throw std::runtime_error(b200q_last_error());
}
// mlx/ops.cpp:110-150
inline void validate_quantized_input(const char* tag, const ArrayView& w, const ArrayView& scales, const ArrayView& biases,
                                     int group_size, int bits) {
  if (w.dtype != Dtype::uint32) {
    std::ostringstream m;
    m << "[" << tag << "] The weight matrix should be uint32 but received " << name(w.dtype);
    throw std::invalid_argument(m.str());
  }
  if (scales.shape != biases.shape) {
    std::ostringstream m;
    m << "[" << tag << "] Scales and biases should have the same shape. Received scales with shape "
      << shape_str(scales.shape) << " and biases with " << shape_str(biases.shape);
    throw std::invalid_argument(m.str());
  }
  bool batch_ok = w.ndim() >= 2 && scales.ndim() == w.ndim();
  for (int i = 0; batch_ok && i < w.ndim() - 2; ++i) batch_ok = w.shape[i] == scales.shape[i];
  if (!batch_ok) {
    std::ostringstream m;
    m << "[" << tag << "] Weight and scales should have the same batch shape. Received weight with shape "
      << shape_str(w.shape) << ", scales with " << shape_str(scales.shape) << ".";
    throw std::invalid_argument(m.str());
  }
  if (w.dim(-1) * 32 / bits != scales.dim(-1) * group_size) {
    std::ostringstream m;
    m << "[" << tag << "] The shapes of the weight and scales are incompatible based on bits and group_size. "
      << "w.shape() == " << shape_str(w.shape) << " and scales.shape() == " << shape_str(scales.shape)
      << " with group_size=" << group_size << " and bits=" << bits;
    throw std::invalid_argument(m.str());
  }
}
// mlx/ops.cpp:152-181: returns {w_inner, w_outer}
inline std::pair<int64_t, int64_t> extract_dims(const char* tag, const ArrayView& x, const ArrayView& w, const ArrayView& scales,
                                                const ArrayView& biases, bool transpose, int group_size, int bits) {
  validate_quantized_input(tag, w, scales, biases, group_size, bits);
  if (x.ndim() < 1) throw std::invalid_argument(std::string("[") + tag + "] x must have at least one dimension");
  const int64_t x_inner = x.dim(-1);
  const int64_t w_inner = transpose ? w.dim(-1) * 32 / bits : w.dim(-2);
  const int64_t w_outer = transpose ? w.dim(-2) : w.dim(-1) * 32 / bits;
  if (w_inner != x_inner) {
    std::ostringstream m;
    m << "[" << tag << "] Last dimension of first input with shape (..., " << x_inner
      << ") does not match the expanded quantized matrix (" << w_inner << ", " << w_outer << ") computed from shape "
      << shape_str(w.shape) << " with group_size=" << group_size << ", bits=" << bits << " and transpose=" << transpose;
    throw std::invalid_argument(m.str());
  }
  return {w_inner, w_outer};
}
inline void validate_types(const char* tag, const ArrayView& x, const ArrayView& scales, const ArrayView& biases) {
  // mlx/ops.cpp:4704-4754: only real floating types; this shim does not promote: one dtype for all
  if (!is_floating(scales.dtype) || !is_floating(biases.dtype) || !is_floating(x.dtype)) {
    std::ostringstream m;
    m << "[" << tag << "] Only real floating types are supported but scales.dtype() == " << name(scales.dtype)
      << " and biases.dtype() == " << name(biases.dtype) << ".";
    throw std::invalid_argument(m.str());
  }
  if (x.dtype != scales.dtype || x.dtype != biases.dtype) {
    std::ostringstream m;
    m << "[" << tag << "] x, scales and biases must already have the result type (the reference casts them before the "
      << "primitive, mlx/ops.cpp:4816-4818); got " << name(x.dtype) << ", " << name(scales.dtype) << ", " << name(biases.dtype);
    throw std::invalid_argument(m.str());
  }
}
}  // namespace detail

// w [.., K] -> wq uint32 [.., K*bits/32], scales / biases [.., K/group_size]  (mlx/ops.cpp:5208-5245)
inline void quantize(const ArrayView& w, ArrayView& wq, ArrayView& scales, ArrayView& biases, int group_size = 64,
                     int bits = 4, void* stream = nullptr) {
  if (!is_floating(w.dtype))
    throw std::invalid_argument(std::string("[quantize] Only real floating types can be quantized but w has type ") + name(w.dtype) + ".");
  if (w.ndim() < 2) {
    std::ostringstream m;
    m << "[quantize] The matrix to be quantized must have at least 2 dimension but it has only " << w.ndim() << ".";
    throw std::invalid_argument(m.str());
  }
  const int64_t K = w.dim(-1), rows = K ? w.size() / K : 0;
  detail::check(b200q_quantize(w.data, (int)w.dtype, rows, K, group_size, bits, static_cast<uint32_t*>(wq.data), scales.data,
                               biases.data, stream));
}

// wq, scales, biases -> w [.., K]  (mlx/ops.cpp:5465-5517)
inline void dequantize(const ArrayView& wq, const ArrayView& scales, const ArrayView& biases, ArrayView& out, int group_size = 64,
                       int bits = 4, void* stream = nullptr) {
  detail::validate_quantized_input("dequantize", wq, scales, biases, group_size, bits);
  const int64_t K = wq.dim(-1) * 32 / bits, rows = wq.dim(-1) ? wq.size() / wq.dim(-1) : 0;
  detail::check(b200q_dequantize(static_cast<const uint32_t*>(wq.data), scales.data, biases.data, (int)scales.dtype, rows, K,
                                 group_size, bits, out.data, stream));
}

// out[i, :] = dequantize(row ids[i]) : QuantizedEmbedding.__call__ (python/mlx/nn/layers/quantized.py:149-158)
inline void quantized_embedding(const ArrayView& ids, const ArrayView& wq, const ArrayView& scales, const ArrayView& biases,
                                ArrayView& out, int group_size = 64, int bits = 4, void* stream = nullptr) {
  detail::validate_quantized_input("quantized_embedding", wq, scales, biases, group_size, bits);
  if (ids.dtype != Dtype::uint32) throw std::invalid_argument("[quantized_embedding] ids must be uint32.");
  if (wq.ndim() != 2) throw std::invalid_argument("[quantized_embedding] the table must be a 2-D packed matrix");
  const int64_t K = wq.dim(-1) * 32 / bits;
  detail::check(b200q_dequantize_rows(static_cast<const uint32_t*>(wq.data), scales.data, biases.data,
                                      static_cast<const uint32_t*>(ids.data), ids.size(), (int)scales.dtype, wq.dim(0), K,
                                      group_size, bits, out.data, stream));
}

// x [.., M, K] against one matrix w (2-D) or a stack of matrices with x's batch shape  (mlx/ops.cpp:4784-4834)
inline void quantized_matmul(const ArrayView& x, const ArrayView& w, const ArrayView& scales, const ArrayView& biases, ArrayView& out,
                             const Workspace& ws, bool transpose = true, int group_size = 64, int bits = 4,
                             void* stream = nullptr) {
  detail::validate_types("quantized_matmul", x, scales, biases);
  const auto dims = detail::extract_dims("quantized_matmul", x, w, scales, biases, transpose, group_size, bits);
  const int64_t K = dims.first, N = dims.second;
  const int64_t M = x.ndim() > 1 ? x.dim(-2) : 1;
  const int64_t batch = (M * K) ? x.size() / (M * K) : 0;
  const bool w_batched = w.ndim() > 2;
  detail::check(b200q_qmm(x.data, static_cast<const uint32_t*>(w.data), scales.data, biases.data, out.data, (int)x.dtype, batch, M,
                          N, K, group_size, bits, transpose ? 1 : 0, w_batched ? 1 : 0, ws.data, ws.bytes, stream));
}

// out[i] = x[lhs[i]] * dequant(w[rhs[i]]); indices uint32, already broadcast against each other  (mlx/ops.cpp:5553-5629)
inline void gather_qmm(const ArrayView& x, const ArrayView& w, const ArrayView& scales, const ArrayView& biases,
                       const ArrayView& lhs_indices, const ArrayView& rhs_indices, ArrayView& out, const Workspace& ws,
                       bool transpose = true, int group_size = 64, int bits = 4, bool sorted_indices = false,
                       void* stream = nullptr) {
  detail::validate_types("gather_qmm", x, scales, biases);
  const auto dims = detail::extract_dims("gather_qmm", x, w, scales, biases, transpose, group_size, bits);
  if (lhs_indices.dtype != Dtype::uint32 || rhs_indices.dtype != Dtype::uint32)
    throw std::invalid_argument("[gather_qmm] Got lhs_indices or rhs_indices with invalid dtype. Indices must be integral.");
  if (lhs_indices.shape != rhs_indices.shape)
    throw std::invalid_argument("[gather_qmm] lhs_indices and rhs_indices must be broadcast to one shape by the caller");
  if (x.ndim() < 2 || w.ndim() < 2)
    throw std::invalid_argument("[gather_qmm] x and w must have at least two dimensions");
  const int64_t K = dims.first, N = dims.second, M = x.dim(-2);
  const int64_t x_batch = (M * K) ? x.size() / (M * K) : 0;
  const int64_t E = w.size() / (w.dim(-1) * w.dim(-2));
  detail::check(b200q_gather_qmm(x.data, static_cast<const uint32_t*>(w.data), scales.data, biases.data,
                                 static_cast<const uint32_t*>(lhs_indices.data), static_cast<const uint32_t*>(rhs_indices.data),
                                 lhs_indices.size(), out.data, (int)x.dtype, x_batch, E, M, N, K, group_size, bits, transpose ? 1 : 0,
                                 sorted_indices ? 3 : 0, ws.data, ws.bytes, stream));
}

}  // namespace b200q
