// gather_qmm: out[i] = x[lhs[i]] * dequant(w[rhs[i]])  (GatherQMM::eval_gpu,
// mlx/backend/cuda/quantized/quantized.cpp:154-278; CPU semantics
// mlx/backend/cpu/quantized.cpp:700-747).
//
// Fast path (bf16, transpose, K a multiple of 128, every bit width): the index pairs are sorted by weight matrix (expert)
// with a counting sort on the device, the activation rows are gathered into expert order,
// and ONE grouped launch of the tensor-core kernel (qmm_tcgen05.cu) runs a tile list of
// (expert, up to NT rows, 128 weight rows); its epilogue scatters every row back to the
// position of its index pair.  Each expert's weights are read once per NT rows instead of
// once per index pair (the reference launches one independent M x N x K problem per pair).
// Everything else goes through the shape-agnostic kernel with per-problem index lookups.
//
// Scratch (caller workspace): [header | sorted slots | destination rows | tile table |
// gathered activations | status].  No host synchronisation: tile counts stay on the device.
#include <cmath>

#include "common.cuh"
#include "kernels.h"

namespace b200q {
namespace {

struct MTileRec { int expert, row0, rows, pad; };  // layout of MTile in qmm_tcgen05.cu

struct Header { int n_mtiles; int n_rows_valid; int pad[62]; };

constexpr int kMaxExpertsFast = 1024;

__global__ void __launch_bounds__(1024)
gather_sort_kernel(const uint32_t* __restrict__ lhs, const uint32_t* __restrict__ rhs, int n_idx, uint32_t x_batch,
                   uint32_t E_total, uint32_t e_lo, uint32_t E, int M, int NT, Header* hdr, int* __restrict__ sorted_slot, MTileRec* __restrict__ mtiles,
                   void* y, size_t y_slot_bytes, uint32_t* status) {
  __shared__ int counts[kMaxExpertsFast];
  __shared__ int cursor[kMaxExpertsFast];
  const int tid = threadIdx.x;
  for (int e = tid; e < (int)E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  // Experts [e_lo, e_lo + E) are the ones whose weights this call holds (all of them unless the
  // experts are spread over several GPUs); pairs for other valid experts are somebody else's.
  for (int i = tid; i < n_idx; i += blockDim.x) {
    const uint32_t e = rhs[i], l = lhs[i];
    if (e < E_total && l < x_batch) {
      if (e - e_lo < E) atomicAdd(&counts[e - e_lo], 1);
    } else {
      // out-of-range index: record it; its output rows are zeroed below, nothing is read through it
      atomicMax(&status[0], 1u);
      status[1] = (uint32_t)i;
    }
  }
  __syncthreads();
  if (tid == 0) {
    int slot0 = 0, g = 0;
    for (int e = 0; e < (int)E; ++e) {
      cursor[e] = slot0;
      const int rows = counts[e] * M, row0 = slot0 * M;
      for (int r = 0; r < rows; r += NT) {
        mtiles[g].expert = e;
        mtiles[g].row0 = row0 + r;
        mtiles[g].rows = rows - r < NT ? rows - r : NT;
        mtiles[g].pad = 0;
        ++g;
      }
      slot0 += counts[e];
    }
    hdr->n_mtiles = g;
    hdr->n_rows_valid = slot0 * M;
  }
  __syncthreads();
  for (int i = tid; i < n_idx; i += blockDim.x) {
    const uint32_t e = rhs[i], l = lhs[i];
    if (e < E_total && l < x_batch) {
      if (e - e_lo < E) sorted_slot[atomicAdd(&cursor[e - e_lo], 1)] = i;
    } else {
      unsigned short* dst = reinterpret_cast<unsigned short*>(static_cast<char*>(y) + (size_t)i * y_slot_bytes);
      for (size_t b = 0; b < y_slot_bytes / 2; ++b) dst[b] = 0;
    }
  }
}

// One CTA per activation row of the sorted order: copies x[lhs[slot]] row m and records where
// the result row goes.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ lhs, const Header* hdr,
                   const int* __restrict__ sorted_slot, int M, int K, __nv_bfloat16* __restrict__ x_sorted,
                   int* __restrict__ dst_row) {
  const int r = blockIdx.x;
  if (r >= hdr->n_rows_valid) return;
  const int slot = sorted_slot[r / M], m = r % M;
  const uint4* src = reinterpret_cast<const uint4*>(x + ((size_t)lhs[slot] * M + m) * K);
  uint4* dst = reinterpret_cast<uint4*>(x_sorted + (size_t)r * K);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = __ldg(src + i);
  if (threadIdx.x == 0) dst_row[r] = slot * M + m;
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Rows per tile: the mean rows per expert plus three standard deviations of a uniform
// routing (so that most experts fit one tile without padding it to 256 tokens).
int pick_nt(int64_t n_rows, int64_t E) {
  const double avg = (double)n_rows / (double)(E > 0 ? E : 1);
  int64_t nt = (int64_t)(avg + 3.0 * sqrt(avg) + 8.0);
  nt = (nt + 15) / 16 * 16;
  return (int)(nt < 16 ? 16 : (nt > 256 ? 256 : nt));
}

struct FastLayout {
  size_t hdr, sorted, dst, mtiles, xs, total;
  int64_t n_rows, max_mtiles;
  int nt;
};

FastLayout fast_layout(int64_t n_idx, int64_t E, int64_t M, int64_t K) {
  FastLayout L{};
  L.n_rows = n_idx * M;
  L.nt = pick_nt(L.n_rows, E);
  L.max_mtiles = L.n_rows / L.nt + E + 1;
  size_t off = 0;
  L.hdr = off; off += align256(sizeof(Header));
  L.sorted = off; off += align256((size_t)n_idx * 4);
  L.dst = off; off += align256((size_t)L.n_rows * 4);
  L.mtiles = off; off += align256((size_t)L.max_mtiles * sizeof(MTileRec));
  L.xs = off; off += align256((size_t)L.n_rows * K * 2);
  L.total = off + 256;  // status word lives in the last 16 bytes
  return L;
}

bool fast_supported(int dtype, int64_t n_idx, int64_t x_batch, int64_t E, int64_t M, int64_t N, int64_t K, int group,
                    int bits, int transpose) {
  (void)x_batch; (void)group;
  if (dtype != B200Q_BF16 || !transpose) return false;
  if (E < 1 || E > kMaxExpertsFast || n_idx < 1 || M < 1 || N < 1) return false;
  if (K < 128 || K % 128 != 0 || (K * bits / 8) % 16 != 0) return false;
  if (n_idx * M > (1ll << 30) || E * N > (1ll << 31) - 1) return false;
  return true;
}


// Sort by expert, gather the activation rows, one grouped tensor-core launch.  Experts
// [e_lo, e_lo + E_local) of E_total are the ones whose weights `wq` holds; with `peers` every
// result row is stored into all of the given [n_idx * M, N] buffers.
int run_grouped(const void* x, const uint32_t* wq, const void* scales, const void* biases, const uint32_t* lhs_idx,
                const uint32_t* rhs_idx, int64_t n_idx, void* y, const PeerOut* peers, int64_t x_batch, int64_t E_total,
                int64_t e_lo, int64_t E_local, int64_t M, int64_t N, int64_t K, int group_size, int bits, void* ws,
                size_t ws_bytes, cudaStream_t st) {
  uint32_t* status = reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + ws_bytes - kStatusBytes);
  const FastLayout L = fast_layout(n_idx, E_total, M, K);
  char* base = static_cast<char*>(ws);
  Header* hdr = reinterpret_cast<Header*>(base + L.hdr);
  int* sorted = reinterpret_cast<int*>(base + L.sorted);
  int* dst = reinterpret_cast<int*>(base + L.dst);
  MTileRec* mt = reinterpret_cast<MTileRec*>(base + L.mtiles);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(base + L.xs);
  gather_sort_kernel<<<1, 1024, 0, st>>>(lhs_idx, rhs_idx, (int)n_idx, (uint32_t)x_batch, (uint32_t)E_total, (uint32_t)e_lo,
                                         (uint32_t)E_local, (int)M, L.nt, hdr, sorted, mt, y, (size_t)M * N * 2, status);
  B200Q_LAUNCH_OK("gather_sort_kernel");
  gather_rows_kernel<<<(unsigned)L.n_rows, 256, 0, st>>>((const __nv_bfloat16*)x, lhs_idx, hdr, sorted, (int)M, (int)K,
                                                         xs, dst);
  B200Q_LAUNCH_OK("gather_rows_kernel");
  GroupedArgs g{};
  g.x_sorted = xs; g.wq = wq; g.scales = scales; g.biases = biases; g.y = y;
  g.mtiles = mt; g.n_mtiles = &hdr->n_mtiles; g.dst_row = dst;
  g.n_rows = L.n_rows; g.max_mtiles = L.max_mtiles; g.E = E_local; g.N = N; g.K = K;
  g.group = group_size; g.bits = bits; g.nt = L.nt; g.status = status;
  if (peers) g.peers = *peers;
  return qmm_tc_grouped(g, st);
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" size_t b200q_gather_qmm_workspace_bytes(int dtype, int64_t n_idx, int64_t x_batch, int64_t E,
                                                   int64_t M, int64_t N, int64_t K, int group_size, int bits,
                                                   int transpose) {
  if (fast_supported(dtype, n_idx, x_batch, E, M, N, K, group_size, bits, transpose))
    return fast_layout(n_idx, E, M, K).total;
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
  const size_t need = b200q_gather_qmm_workspace_bytes(dtype, n_idx, x_batch, E, M, N, K, group_size, bits, transpose);
  if (!ws || ws_bytes < need)
    return fail(B200Q_ERR_WORKSPACE, "[gather_qmm] workspace of %zu bytes required, %zu given", need, ws_bytes);
  uint32_t* status = reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + ws_bytes - kStatusBytes);

  const bool aligned = !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wq) |
                          reinterpret_cast<uintptr_t>(ws) | reinterpret_cast<uintptr_t>(y)) & 15);
  if (aligned && fast_supported(dtype, n_idx, x_batch, E, M, N, K, group_size, bits, transpose))
    return run_grouped(x, wq, scales, biases, lhs_idx, rhs_idx, n_idx, y, nullptr, x_batch, E, 0, E, M, N, K, group_size,
                       bits, ws, ws_bytes, st);

  QmmArgs a{};
  a.x = x; a.wq = wq; a.scales = scales; a.biases = biases; a.y = y;
  a.dtype = dtype; a.batch = n_idx; a.M = M; a.N = N; a.K = K;
  a.group = group_size; a.bits = bits; a.transpose = transpose != 0; a.w_batched = true;
  a.ws = ws; a.ws_bytes = ws_bytes;
  GatherIdx gi{lhs_idx, rhs_idx, (uint32_t)x_batch, (uint32_t)E, status};
  return qmm_generic(a, st, &gi);
}

namespace {
int gather_sharded_impl(const void* x, const uint32_t* wq_local, const void* scales_local, const void* biases_local,
                        const uint32_t* lhs_idx, const uint32_t* rhs_idx, int64_t n_idx, void* const* y_peers, int n_peers,
                        int self, int dtype, int64_t x_batch, int64_t E_total, int64_t e_lo, int64_t E_local, int64_t M,
                        int64_t N, int64_t K, int group_size, int bits, uint32_t* const* flag_peers, uint32_t* epoch_local,
                        uint32_t* counter_local, void* ws, size_t ws_bytes, void* stream) {
  if (!y_peers || n_peers < 1 || n_peers > kMaxPeers || self < 0 || self >= n_peers)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_sharded] between 1 and %d output buffers, one of them this rank's (got %d, self %d)",
                kMaxPeers, n_peers, self);
  if (!valid_group(group_size) || !valid_bits(bits))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_sharded] group size must be 32, 64 or 128 and bits 2, 3, 4, 5, 6 or 8");
  if (n_idx < 0 || x_batch < 0 || M < 0 || N < 0 || K < 0 || E_total < 1 || e_lo < 0 || E_local < 0 || e_lo + E_local > E_total)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_sharded] experts [%lld, %lld) are not a range of %lld experts",
                (long long)e_lo, (long long)(e_lo + E_local), (long long)E_total);
  if (K % group_size != 0 || (K * bits) % 32 != 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_sharded] The shapes of the weight and scales are incompatible based on bits and group_size");
  // the signal goes out even when there is nothing to multiply: the other ranks count on it
  if (n_idx == 0 || M == 0 || N == 0)
    return flag_peers ? b200q_peer_signal(flag_peers, n_peers, epoch_local, stream) : B200Q_OK;
  PeerOut peers{};
  for (int q = 0; q < n_peers; ++q) {
    if (!y_peers[q]) return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_sharded] null output buffer %d", q);
    peers.y[q] = y_peers[q];
  }
  peers.n = n_peers; peers.ld = N; peers.col0 = 0;
  if (flag_peers) {
    for (int q = 0; q < n_peers; ++q) {
      if (!flag_peers[q]) return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_sharded] null flag %d", q);
      peers.sig.flags[q] = flag_peers[q];
    }
    peers.sig.epoch = epoch_local;
    peers.sig.counter = counter_local;
    peers.sig.n = n_peers;
  }
  if (!x || !wq_local || !scales_local || !biases_local || !lhs_idx || !rhs_idx)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_sharded] null pointer");
  const size_t need = b200q_gather_qmm_workspace_bytes(dtype, n_idx, x_batch, E_total, M, N, K, group_size, bits, 1);
  if (!ws || ws_bytes < need)
    return fail(B200Q_ERR_WORKSPACE, "[gather_qmm_sharded] workspace of %zu bytes required, %zu given", need, ws_bytes);
  const bool aligned = !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wq_local) |
                          reinterpret_cast<uintptr_t>(ws)) & 15);
  if (!aligned || E_local < 1 || !fast_supported(dtype, n_idx, x_batch, E_total, M, N, K, group_size, bits, 1))
    return fail(B200Q_ERR_UNSUPPORTED, "[gather_qmm_sharded] only bfloat16 with K a multiple of 128 has a peer-store epilogue");
  return run_grouped(x, wq_local, scales_local, biases_local, lhs_idx, rhs_idx, n_idx, y_peers[self], &peers, x_batch, E_total,
                     e_lo, E_local, M, N, K, group_size, bits, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" int b200q_gather_qmm_sharded(const void* x, const uint32_t* wq_local, const void* scales_local,
                                        const void* biases_local, const uint32_t* lhs_idx, const uint32_t* rhs_idx,
                                        int64_t n_idx, void* const* y_peers, int n_peers, int self, int dtype,
                                        int64_t x_batch, int64_t E_total, int64_t e_lo, int64_t E_local, int64_t M,
                                        int64_t N, int64_t K, int group_size, int bits, void* ws, size_t ws_bytes,
                                        void* stream) {
  return gather_sharded_impl(x, wq_local, scales_local, biases_local, lhs_idx, rhs_idx, n_idx, y_peers, n_peers, self, dtype,
                             x_batch, E_total, e_lo, E_local, M, N, K, group_size, bits, nullptr, nullptr, nullptr, ws,
                             ws_bytes, stream);
}

extern "C" int b200q_gather_qmm_sharded_signal(const void* x, const uint32_t* wq_local, const void* scales_local,
                                               const void* biases_local, const uint32_t* lhs_idx, const uint32_t* rhs_idx,
                                               int64_t n_idx, void* const* y_peers, int n_peers, int self, int dtype,
                                               int64_t x_batch, int64_t E_total, int64_t e_lo, int64_t E_local, int64_t M,
                                               int64_t N, int64_t K, int group_size, int bits,
                                               uint32_t* const* flag_peers, uint32_t* epoch_local, uint32_t* counter_local,
                                               void* ws, size_t ws_bytes, void* stream) {
  if (!flag_peers || !epoch_local || !counter_local)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_sharded] null flag list, epoch or counter");
  return gather_sharded_impl(x, wq_local, scales_local, biases_local, lhs_idx, rhs_idx, n_idx, y_peers, n_peers, self, dtype,
                             x_batch, E_total, e_lo, E_local, M, N, K, group_size, bits, flag_peers, epoch_local,
                             counter_local, ws, ws_bytes, stream);
}

// ---------------------------------------------------------------- two chained gather_qmm, one sort
extern "C" size_t b200q_gather_qmm_chain_workspace_bytes(int64_t n_idx, int64_t E, int64_t M, int64_t N1, int64_t K1) {
  if (n_idx < 1 || E < 1 || M < 1 || N1 < 1 || K1 < 1) return 256;
  const FastLayout L = fast_layout(n_idx, E, M, K1);
  return L.total + align256((size_t)L.n_rows * N1 * 2);
}

extern "C" int b200q_gather_qmm_chain(const void* x, const uint32_t* wq1, const void* scales1, const void* biases1,
                                      const uint32_t* wq2, const void* scales2, const void* biases2,
                                      const uint32_t* lhs_idx, const uint32_t* rhs_idx, int64_t n_idx, void* y, int dtype,
                                      int64_t x_batch, int64_t E, int64_t M, int64_t N1, int64_t K1, int64_t N2,
                                      int group_size, int bits, void* ws, size_t ws_bytes, void* stream) {
  if (!valid_group(group_size) || !valid_bits(bits))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_chain] group size must be 32, 64 or 128 and bits 2, 3, 4, 5, 6 or 8");
  if (n_idx < 0 || x_batch < 0 || E < 1 || M < 0 || N1 < 0 || K1 < 0 || N2 < 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_chain] negative dimension.");
  if (K1 % group_size != 0 || (K1 * bits) % 32 != 0 || N1 % group_size != 0 || (N1 * bits) % 32 != 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_chain] The shapes of the weight and scales are incompatible based on bits and group_size");
  if (n_idx == 0 || M == 0 || N2 == 0) return B200Q_OK;
  if (!x || !wq1 || !scales1 || !biases1 || !wq2 || !scales2 || !biases2 || !lhs_idx || !rhs_idx || !y)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_chain] null pointer");
  const bool aligned = !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wq1) | reinterpret_cast<uintptr_t>(wq2) |
                          reinterpret_cast<uintptr_t>(ws) | reinterpret_cast<uintptr_t>(y)) & 15);
  if (!aligned || !fast_supported(dtype, n_idx, x_batch, E, M, N1, K1, group_size, bits, 1) ||
      !fast_supported(dtype, n_idx, n_idx, E, M, N2, N1, group_size, bits, 1))
    return fail(B200Q_ERR_UNSUPPORTED, "[gather_qmm_chain] only bfloat16 with K and the inner width multiples of 128 (two b200q_gather_qmm calls cover the rest)");
  const size_t need = b200q_gather_qmm_chain_workspace_bytes(n_idx, E, M, N1, K1);
  if (!ws || ws_bytes < need)
    return fail(B200Q_ERR_WORKSPACE, "[gather_qmm_chain] workspace of %zu bytes required, %zu given", need, ws_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* status = reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + ws_bytes - kStatusBytes);
  const FastLayout L = fast_layout(n_idx, E, M, K1);
  char* base = static_cast<char*>(ws);
  Header* hdr = reinterpret_cast<Header*>(base + L.hdr);
  int* sorted = reinterpret_cast<int*>(base + L.sorted);
  int* dst = reinterpret_cast<int*>(base + L.dst);
  MTileRec* mt = reinterpret_cast<MTileRec*>(base + L.mtiles);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(base + L.xs);
  __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(base + L.total - 256);   // after the gathered rows
  gather_sort_kernel<<<1, 1024, 0, st>>>(lhs_idx, rhs_idx, (int)n_idx, (uint32_t)x_batch, (uint32_t)E, 0u, (uint32_t)E, (int)M,
                                         L.nt, hdr, sorted, mt, y, (size_t)M * N2 * 2, status);
  B200Q_LAUNCH_OK("gather_sort_kernel");
  gather_rows_kernel<<<(unsigned)L.n_rows, 256, 0, st>>>((const __nv_bfloat16*)x, lhs_idx, hdr, sorted, (int)M, (int)K1, xs, dst);
  B200Q_LAUNCH_OK("gather_rows_kernel");
  GroupedArgs g{};
  g.mtiles = mt; g.n_mtiles = &hdr->n_mtiles;
  g.n_rows = L.n_rows; g.max_mtiles = L.max_mtiles; g.E = E;
  g.group = group_size; g.bits = bits; g.nt = L.nt; g.status = status;
  // first product: rows stay in expert order (no scatter), result = activation of the second
  g.x_sorted = xs; g.wq = wq1; g.scales = scales1; g.biases = biases1; g.y = h; g.dst_row = nullptr; g.N = N1; g.K = K1;
  if (int rc = qmm_tc_grouped(g, st)) return rc;
  // second product: same tile table, rows scattered to the positions of their index pairs
  g.x_sorted = h; g.wq = wq2; g.scales = scales2; g.biases = biases2; g.y = y; g.dst_row = dst; g.N = N2; g.K = N1;
  return qmm_tc_grouped(g, st);
}

// ---------------------------------------------------------------- gated expert MLP: down(silu(gate(x)) * up(x)), one sort
namespace b200q {
namespace {

// g[i] = silu(g[i]) * u[i] on bf16 pairs, fp32 arithmetic, one rounding.
__global__ void __launch_bounds__(256) swiglu_kernel(uint4* __restrict__ g, const uint4* __restrict__ u, int64_t n_vec) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  uint4 a = g[i];
  const uint4 b = __ldg(u + i);
  uint32_t* aw = reinterpret_cast<uint32_t*>(&a);
  const uint32_t* bw = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float g0 = __uint_as_float(aw[k] << 16), g1 = __uint_as_float(aw[k] & 0xffff0000u);
    const float u0 = __uint_as_float(bw[k] << 16), u1 = __uint_as_float(bw[k] & 0xffff0000u);
    const float r0 = __fdividef(g0, 1.f + __expf(-g0)) * u0;
    const float r1 = __fdividef(g1, 1.f + __expf(-g1)) * u1;
    const __nv_bfloat162 r = __floats2bfloat162_rn(r0, r1);
    aw[k] = *reinterpret_cast<const uint32_t*>(&r);
  }
  g[i] = a;
}

}  // namespace
}  // namespace b200q

extern "C" size_t b200q_gather_qmm_swiglu_workspace_bytes(int64_t n_idx, int64_t E, int64_t M, int64_t H, int64_t K1) {
  if (n_idx < 1 || E < 1 || M < 1 || H < 1 || K1 < 1) return 256;
  const FastLayout L = fast_layout(n_idx, E, M, K1);
  return L.total + 2 * align256((size_t)L.n_rows * H * 2);
}

extern "C" int b200q_gather_qmm_swiglu(const void* x, const uint32_t* wq_gate, const void* scales_gate, const void* biases_gate,
                                       const uint32_t* wq_up, const void* scales_up, const void* biases_up,
                                       const uint32_t* wq_down, const void* scales_down, const void* biases_down,
                                       const uint32_t* lhs_idx, const uint32_t* rhs_idx, int64_t n_idx, void* y, int dtype,
                                       int64_t x_batch, int64_t E, int64_t M, int64_t H, int64_t K1, int64_t N2,
                                       int group_size, int bits, void* ws, size_t ws_bytes, void* stream) {
  if (!valid_group(group_size) || !valid_bits(bits))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_swiglu] group size must be 32, 64 or 128 and bits 2, 3, 4, 5, 6 or 8");
  if (n_idx < 0 || x_batch < 0 || E < 1 || M < 0 || H < 0 || K1 < 0 || N2 < 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_swiglu] negative dimension.");
  if (K1 % group_size != 0 || (K1 * bits) % 32 != 0 || H % group_size != 0 || (H * bits) % 32 != 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_swiglu] The shapes of the weight and scales are incompatible based on bits and group_size");
  if (n_idx == 0 || M == 0 || N2 == 0) return B200Q_OK;
  if (!x || !wq_gate || !scales_gate || !biases_gate || !wq_up || !scales_up || !biases_up || !wq_down || !scales_down ||
      !biases_down || !lhs_idx || !rhs_idx || !y)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[gather_qmm_swiglu] null pointer");
  const bool aligned = !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wq_gate) | reinterpret_cast<uintptr_t>(wq_up) |
                          reinterpret_cast<uintptr_t>(wq_down) | reinterpret_cast<uintptr_t>(ws) | reinterpret_cast<uintptr_t>(y)) & 15);
  if (!aligned || !fast_supported(dtype, n_idx, x_batch, E, M, H, K1, group_size, bits, 1) ||
      !fast_supported(dtype, n_idx, n_idx, E, M, N2, H, group_size, bits, 1))
    return fail(B200Q_ERR_UNSUPPORTED, "[gather_qmm_swiglu] only bfloat16 with K and the hidden width multiples of 128");
  const size_t need = b200q_gather_qmm_swiglu_workspace_bytes(n_idx, E, M, H, K1);
  if (!ws || ws_bytes < need)
    return fail(B200Q_ERR_WORKSPACE, "[gather_qmm_swiglu] workspace of %zu bytes required, %zu given", need, ws_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* status = reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + ws_bytes - kStatusBytes);
  const FastLayout L = fast_layout(n_idx, E, M, K1);
  char* base = static_cast<char*>(ws);
  Header* hdr = reinterpret_cast<Header*>(base + L.hdr);
  int* sorted = reinterpret_cast<int*>(base + L.sorted);
  int* dst = reinterpret_cast<int*>(base + L.dst);
  MTileRec* mt = reinterpret_cast<MTileRec*>(base + L.mtiles);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(base + L.xs);
  const size_t h_bytes = align256((size_t)L.n_rows * H * 2);
  __nv_bfloat16* hg = reinterpret_cast<__nv_bfloat16*>(base + L.total - 256);
  __nv_bfloat16* hu = reinterpret_cast<__nv_bfloat16*>(base + L.total - 256 + h_bytes);
  gather_sort_kernel<<<1, 1024, 0, st>>>(lhs_idx, rhs_idx, (int)n_idx, (uint32_t)x_batch, (uint32_t)E, 0u, (uint32_t)E, (int)M,
                                         L.nt, hdr, sorted, mt, y, (size_t)M * N2 * 2, status);
  B200Q_LAUNCH_OK("gather_sort_kernel");
  gather_rows_kernel<<<(unsigned)L.n_rows, 256, 0, st>>>((const __nv_bfloat16*)x, lhs_idx, hdr, sorted, (int)M, (int)K1, xs, dst);
  B200Q_LAUNCH_OK("gather_rows_kernel");
  GroupedArgs g{};
  g.mtiles = mt; g.n_mtiles = &hdr->n_mtiles;
  g.n_rows = L.n_rows; g.max_mtiles = L.max_mtiles; g.E = E;
  g.group = group_size; g.bits = bits; g.nt = L.nt; g.status = status;
  g.x_sorted = xs; g.dst_row = nullptr; g.N = H; g.K = K1;
  g.wq = wq_gate; g.scales = scales_gate; g.biases = biases_gate; g.y = hg;
  if (int rc = qmm_tc_grouped(g, st)) return rc;
  g.wq = wq_up; g.scales = scales_up; g.biases = biases_up; g.y = hu;
  if (int rc = qmm_tc_grouped(g, st)) return rc;
  const int64_t n_vec = (int64_t)L.n_rows * H / 8;   // H is a multiple of 128
  swiglu_kernel<<<(unsigned)((n_vec + 255) / 256), 256, 0, st>>>(reinterpret_cast<uint4*>(hg), reinterpret_cast<const uint4*>(hu), n_vec);
  B200Q_LAUNCH_OK("swiglu_kernel");
  g.x_sorted = hg; g.wq = wq_down; g.scales = scales_down; g.biases = biases_down; g.y = y; g.dst_row = dst; g.N = N2; g.K = H;
  return qmm_tc_grouped(g, st);
}
