// C-ABI entry points of libb200q.so: argument checks, kernel selection, scratch layout.
//
// Kernel selection for b200q_qmm (the role of QuantizedMatmul::eval_gpu's dispatch,
// mlx/backend/cuda/quantized/quantized.cpp:106-136):
//   bf16, transpose, M <= 16, bits 2/4/8, K % (16 * group) == 0 -> qmv_rows    (HBM-bound decode)
//   bf16, transpose, M <= 16, K % 128 == 0 (any width)           -> qmv_mma     (register-path decode)
//   bf16, transpose, M  > 16, K % 128 == 0, N % 8 == 0           -> qmm_tcgen05 (TMA + tcgen05 + TMEM)
//   transpose == 0, M <= 4, bits 2/4/8                           -> qvm
//   everything else                                              -> qmm_generic
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace b200q {

namespace {
thread_local char g_err[512] = "";
thread_local uint64_t g_launches = 0;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(int n) { g_launches += (uint64_t)n; }

namespace {

enum class Path { QmvRows, Qmv, Tc, Qvm, Generic };

int check_qmm_args(const char* tag, const QmmArgs& a) {
  if (a.dtype != B200Q_F32 && a.dtype != B200Q_F16 && a.dtype != B200Q_BF16)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[%s] Only real floating types are supported (dtype code %d).", tag, a.dtype);
  if (!valid_group(a.group))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[%s] Quantization group size must be 32, 64 or 128 (got %d).", tag, a.group);
  if (!valid_bits(a.bits))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[%s] Quantization bits must be 2, 3, 4, 5, 6 or 8 (got %d).", tag, a.bits);
  if (a.batch < 0 || a.M < 0 || a.N < 0 || a.K < 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[%s] negative dimension.", tag);
  // The quantized axis is the last axis of the stored W: K if transposed, N otherwise.
  const int64_t qaxis = a.transpose ? a.K : a.N;
  if (qaxis % a.group != 0 || (qaxis * a.bits) % 32 != 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT,
                "[%s] The shapes of the weight and scales are incompatible based on bits and group_size: "
                "quantized axis %lld with group_size=%d and bits=%d", tag, (long long)qaxis, a.group, a.bits);
  if (a.M > INT32_MAX || a.N > INT32_MAX || a.K > INT32_MAX)
    return fail(B200Q_ERR_UNSUPPORTED, "[%s] No implementation for problem shape: dimension exceeds 2^31-1.", tag);
  return B200Q_OK;
}

// B200Q_QMV_IMPL=mma keeps the row-owning decode kernel out of the selection (testing and tuning).
int qmv_override() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200Q_QMV_IMPL");
    v = (e && strcmp(e, "mma") == 0) ? 2 : 0;
  }
  return v;
}

bool force_tc() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200Q_FORCE_TC");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

Path choose(const QmmArgs& a) {
  const int ov = qmv_override();
  if (force_tc() && qmm_tc_supported(a)) return Path::Tc;  // tuning aid: tensor-memory path for any M
  if (ov == 0 && qmv_rows_supported(a)) return Path::QmvRows;
  if (qmv_mma_supported(a)) return Path::Qmv;
  if (qmm_tc_supported(a)) return Path::Tc;
  if (qvm_supported(a)) return Path::Qvm;
  return Path::Generic;
}

QmmArgs make_args(const void* x, const uint32_t* wq, const void* scales, const void* biases, void* y, int dtype,
                  int64_t batch, int64_t M, int64_t N, int64_t K, int group, int bits, int transpose,
                  int64_t w_batch_stride, void* ws, size_t ws_bytes) {
  QmmArgs a{};
  a.x = x; a.wq = wq; a.scales = scales; a.biases = biases; a.y = y;
  a.dtype = dtype;
  a.group = group; a.bits = bits;
  a.transpose = transpose != 0;
  a.w_batched = w_batch_stride != 0 && batch > 1;
  // A weight matrix shared by all batches: fold the batch into M.
  if (a.w_batched) { a.batch = batch; a.M = M; } else { a.batch = 1; a.M = batch * M; }
  a.N = N; a.K = K;
  a.ws = ws; a.ws_bytes = ws_bytes;
  return a;
}

int run_qmm(const QmmArgs& a, cudaStream_t st) {
  if (a.batch == 0 || a.M == 0 || a.N == 0) return B200Q_OK;
  if (a.K == 0) {
    B200Q_CUDA_OK(cudaMemsetAsync(a.y, 0, (size_t)a.batch * a.M * a.N * dtype_size(a.dtype), st));
    return B200Q_OK;
  }
  if (!a.x || !a.wq || !a.scales || !a.biases || !a.y)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantized_matmul] null pointer");
  switch (choose(a)) {
    case Path::QmvRows: return qmv_rows(a, st);
    case Path::Qmv: return qmv_mma(a, st);
    case Path::Tc: return qmm_tc(a, st);
    case Path::Qvm: return qvm(a, st);
    default: return qmm_generic(a, st);
  }
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int b200q_version(void) { return B200Q_VERSION; }
extern "C" const char* b200q_last_error(void) { return g_err; }
extern "C" uint64_t b200q_launch_count(void) { return g_launches; }

extern "C" void b200q_set_weights_constant(int on) { set_weights_constant(on); }

extern "C" size_t b200q_qmm_workspace_bytes(int dtype, int64_t batch, int64_t M, int64_t N, int64_t K,
                                            int group_size, int bits, int transpose) {
  // Sized for whichever kernel may be selected for this shape, for any pointer alignment.
  QmmArgs a = make_args(nullptr, nullptr, nullptr, nullptr, nullptr, dtype, batch, M, N, K, group_size, bits,
                        transpose, 0, nullptr, 0);
  if (!valid_group(group_size) || !valid_bits(bits) || N <= 0 || K <= 0) return 0;
  size_t need = 0;
  const size_t q = qmv_mma_workspace_bytes(a);
  size_t t = qmm_tc_workspace_bytes(a);
  need = q > t ? q : t;
  if (!transpose) {
    const size_t v = qvm_workspace_bytes(a);
    need = need > v ? need : v;
  }
  return (need + 255) / 256 * 256;
}

extern "C" int b200q_qmm(const void* x, const uint32_t* wq, const void* scales, const void* biases, void* y,
                         int dtype, int64_t batch, int64_t M, int64_t N, int64_t K, int group_size, int bits,
                         int transpose, int64_t w_batch_stride, void* ws, size_t ws_bytes, void* stream) {
  QmmArgs a = make_args(x, wq, scales, biases, y, dtype, batch, M, N, K, group_size, bits, transpose,
                        w_batch_stride, ws, ws_bytes);
  if (int rc = check_qmm_args("quantized_matmul", a)) return rc;
  return run_qmm(a, static_cast<cudaStream_t>(stream));
}

extern "C" const char* b200q_qmm_kernel_name(int dtype, int64_t batch, int64_t M, int64_t N, int64_t K,
                                             int group_size, int bits, int transpose) {
  static const uint32_t aligned_dummy[4] __attribute__((aligned(16))) = {0, 0, 0, 0};
  QmmArgs a = make_args(aligned_dummy, aligned_dummy, aligned_dummy, aligned_dummy, nullptr, dtype, batch, M, N, K,
                        group_size, bits, transpose, 0, nullptr, 0);
  if (check_qmm_args("quantized_matmul", a)) return "invalid";
  switch (choose(a)) {
    case Path::QmvRows: return "qmv_rows";
    case Path::Qmv: return "qmv_mma";
    case Path::Tc: return "qmm_tcgen05";
    case Path::Qvm: return "qvm";
    default: return "qmm_generic";
  }
}

// ---------------------------------------------------------------- N-sharded output with peer stores
namespace b200q {
namespace peer {
__global__ void peer_signal_kernel(uint32_t* f0, uint32_t* f1, uint32_t* f2, uint32_t* f3, uint32_t* f4, uint32_t* f5,
                                   uint32_t* f6, uint32_t* f7, int n, uint32_t* epoch) {
  uint32_t* f[kMaxPeers] = {f0, f1, f2, f3, f4, f5, f6, f7};
  // everything enqueued before this kernel on the stream (the peer stores of the matmul) has
  // completed; the fence orders it before the flag updates for observers on other GPUs
  __threadfence_system();
  *epoch += (uint32_t)n;   // what the local flag must reach before this step's output is complete
  for (int q = 0; q < n; ++q) atomicAdd_system(f[q], 1u);
}
__global__ void peer_wait_kernel(const uint32_t* flag, const uint32_t* epoch, uint32_t* status, long long limit) {
  // Launched with programmatic stream serialization: the block may be resident before the kernel
  // that signals has finished; it reads the epoch only after that kernel has completed, and lets
  // the next kernel of the stream begin its own prologue at once.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t expected = *epoch;
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t)(v - expected) >= 0) break;
    if (clock64() - t0 > limit) {
      atomicMax(&status[0], 6u);
      status[1] = v;
      break;
    }
    __nanosleep(200);
  }
}
// Copies n16 16-byte pieces from (mapped, pinned) host memory to device memory.  The next kernel
// of the stream may start early: it waits for this grid before it reads the destination.
__global__ void __launch_bounds__(256) host_fetch_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t n16) {
  asm volatile("griddepcontrol.launch_dependents;");
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n16) dst[i] = src[i];
}
// y[i] = sum over the n_slots partial results slots[r * stride + i], added in fp32 in slot order,
// rounded once to T.  Eight elements per thread.
template <typename T>
__global__ void __launch_bounds__(256) peer_reduce_kernel(const T* __restrict__ slots, int n_slots, int64_t stride,
                                                          int64_t n, T* __restrict__ y) {
  const int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i0 >= n) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const bool full = i0 + 8 <= n && (((uintptr_t)slots | (uintptr_t)y | (uintptr_t)(stride * sizeof(T))) & 15) == 0;
  for (int r = 0; r < n_slots; ++r) {
    const T* p = slots + r * stride + i0;
    if (full && sizeof(T) == 2) {
      const uint4 v = *reinterpret_cast<const uint4*>(p);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += Elem<T>::to_float(e[j]);
    } else {
      for (int j = 0; j < 8 && i0 + j < n; ++j) acc[j] += Elem<T>::to_float(p[j]);
    }
  }
  for (int j = 0; j < 8 && i0 + j < n; ++j) y[i0 + j] = Elem<T>::from_float(acc[j]);
}
// Copies this rank's block of a finished [M, ld] result (columns [col0, col0 + n_cols)) from its own
// buffer into the buffers of the other ranks with 16-byte loads and stores, then signals.  The
// tensor-core kernel's own peer stores are 64-byte warp stores issued once per destination from
// its epilogue; with more than four ranks they take longer than the product, so the product then
// stores locally only and this kernel moves the block.
struct PushParams {
  char* y[kMaxPeers];
  int n, self;
  int64_t row_bytes, col_bytes, chunks_per_row, total;   // pitch, byte offset of the block, 16-byte chunks
  PeerSignal sig;
};
__global__ void __launch_bounds__(256) peer_push_kernel(const PushParams p) {
  for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < p.total; u += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = u / p.chunks_per_row, c = u - m * p.chunks_per_row;
    const int64_t off = m * p.row_bytes + p.col_bytes + c * 16;
    const uint4 v = *reinterpret_cast<const uint4*>(p.y[p.self] + off);
    for (int q = 0; q < p.n; ++q)
      if (q != p.self) *reinterpret_cast<uint4*>(p.y[q] + off) = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) peer_signal_tail(p.sig);
}
}  // namespace peer
}  // namespace b200q

namespace {
// B200Q_PUSH=0: never the separate push; 1: whenever it is possible (testing); default: above four ranks
// (measured on M=4096, N=14336: 2 ranks 271 us fused / 326 us pushed, 4 ranks 272 / 281, 8 ranks 391 / 254).
int push_mode() {
  static int v = -2;
  if (v == -2) {
    const char* e = getenv("B200Q_PUSH");
    v = e ? atoi(e) : -1;
  }
  return v;
}
// Bound of b200q_peer_wait in SM clock cycles (default about one second).
long long g_peer_wait_limit = 2000000000ll;

int sharded_impl(const void* x, const uint32_t* wq, const void* scales, const void* biases, void* const* y_peers,
                 int n_peers, int64_t ld, int64_t col0, int dtype, int64_t M, int64_t N_local, int64_t K,
                 int group_size, int bits, uint32_t* const* flag_peers, uint32_t* epoch_local, uint32_t* counter_local,
                 const uint32_t* wait_flag, int wait_before_x, int self, void* ws, size_t ws_bytes, void* stream);
}  // namespace

extern "C" void b200q_set_peer_wait_limit_ms(int ms) {
  g_peer_wait_limit = ms <= 0 ? 2000000000ll : (long long)ms * 2000000ll;   // ~2 GHz SM clock
}

extern "C" int b200q_qmm_sharded(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                                 void* const* y_peers, int n_peers, int64_t ld, int64_t col0, int dtype, int64_t M,
                                 int64_t N_local, int64_t K, int group_size, int bits, void* ws, size_t ws_bytes,
                                 void* stream) {
  return sharded_impl(x, wq, scales, biases, y_peers, n_peers, ld, col0, dtype, M, N_local, K, group_size, bits, nullptr,
                      nullptr, nullptr, nullptr, 0, -1, ws, ws_bytes, stream);
}

extern "C" int b200q_qmm_sharded_signal(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                                        void* const* y_peers, int n_peers, int64_t ld, int64_t col0, int dtype, int64_t M,
                                        int64_t N_local, int64_t K, int group_size, int bits, uint32_t* const* flag_peers,
                                        uint32_t* epoch_local, uint32_t* counter_local, const uint32_t* wait_flag_local,
                                        int wait_before_x, int self, void* ws, size_t ws_bytes, void* stream) {
  if (!flag_peers || !epoch_local || !counter_local)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantized_matmul_sharded] null flag list, epoch or counter");
  return sharded_impl(x, wq, scales, biases, y_peers, n_peers, ld, col0, dtype, M, N_local, K, group_size, bits, flag_peers,
                      epoch_local, counter_local, wait_flag_local, wait_before_x, self, ws, ws_bytes, stream);
}

namespace {
int sharded_impl(const void* x, const uint32_t* wq, const void* scales, const void* biases, void* const* y_peers,
                 int n_peers, int64_t ld, int64_t col0, int dtype, int64_t M, int64_t N_local, int64_t K,
                 int group_size, int bits, uint32_t* const* flag_peers, uint32_t* epoch_local, uint32_t* counter_local,
                 const uint32_t* wait_flag, int wait_before_x, int self, void* ws, size_t ws_bytes, void* stream) {
  if (!y_peers || n_peers < 1 || n_peers > kMaxPeers)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantized_matmul_sharded] between 1 and %d output buffers are supported (got %d)", kMaxPeers, n_peers);
  if (ld < N_local || col0 < 0 || col0 + N_local > ld)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantized_matmul_sharded] columns [%lld, %lld) do not fit a row pitch of %lld",
                (long long)col0, (long long)(col0 + N_local), (long long)ld);
  QmmArgs a = make_args(x, wq, scales, biases, y_peers[0], dtype, 1, M, N_local, K, group_size, bits, 1, 0, ws, ws_bytes);
  if (int rc = check_qmm_args("quantized_matmul_sharded", a)) return rc;
  for (int q = 0; q < n_peers; ++q) {
    if (!y_peers[q]) return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantized_matmul_sharded] null output buffer %d", q);
    a.peers.y[q] = y_peers[q];
  }
  a.peers.n = n_peers; a.peers.ld = ld; a.peers.col0 = col0;
  if (flag_peers) {
    for (int q = 0; q < n_peers; ++q) {
      if (!flag_peers[q]) return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantized_matmul_sharded] null flag %d", q);
      a.peers.sig.flags[q] = flag_peers[q];
    }
    a.peers.sig.epoch = epoch_local;
    a.peers.sig.counter = counter_local;
    a.peers.sig.n = n_peers;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the signal goes out even when this rank has nothing to multiply: the other ranks count on it
  auto signal_only = [&]() -> int {
    return flag_peers ? b200q_peer_signal(flag_peers, n_peers, epoch_local, stream) : B200Q_OK;
  };
  // Consumer-side wait for the previous exchange step: inside the row-owning decode kernel (the
  // weight stream starts meanwhile), as a launch of its own in front of the other kernels.
  const bool rows = a.M > 0 && a.N > 0 && a.K > 0 && qmv_override() == 0 && qmv_rows_supported(a);
  if (wait_flag) {
    if (rows) {
      a.peers.sig.wait_flag = wait_flag;
      a.peers.sig.wait_limit = g_peer_wait_limit;
      a.peers.sig.wait_x = wait_before_x ? 1 : 0;
    } else {
      uint32_t* status = (ws && ws_bytes >= kStatusBytes)
                             ? reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + ws_bytes - kStatusBytes) : nullptr;
      if (!status) return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul_sharded] the wait needs the workspace's status word");
      if (int rc = b200q_peer_wait(wait_flag, epoch_local, status, stream)) return rc;
    }
  }
  if (a.M == 0 || a.N == 0) return signal_only();
  if (!x || !wq || !scales || !biases) return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantized_matmul_sharded] null pointer");
  if (rows) return qmv_rows(a, st);   // signals from its last block
  if (a.K > 0 && qmv_mma_supported(a)) {
    a.peers.sig.n = 0;   // the register-path kernel has no fused signal: a launch of its own follows
    if (int rc = qmv_mma(a, st)) return rc;
    return signal_only();
  }
  if (a.K > 0 && qmm_tc_supported(a)) {
    // Large results over more than four ranks: the product stores its block locally, a copy kernel
    // moves it to the other ranks with 16-byte accesses and signals (see peer_push_kernel).
    const int pm = push_mode();
    const int64_t esz = 2;
    bool push = flag_peers && self >= 0 && self < n_peers && n_peers >= 2 && pm != 0 && (pm == 1 || (n_peers > 4 && a.M >= 256));
    push = push && (ld * esz) % 16 == 0 && (col0 * esz) % 16 == 0 && (N_local * esz) % 16 == 0;
    for (int q = 0; push && q < n_peers; ++q) push = (reinterpret_cast<uintptr_t>(y_peers[q]) & 15) == 0;
    if (!push) return qmm_tc(a, st);                                                         // signals from its last block
    const PeerSignal sig = a.peers.sig;
    a.peers.n = 1;
    a.peers.y[0] = y_peers[self];
    a.peers.sig = PeerSignal{};
    if (int rc = qmm_tc(a, st)) return rc;
    peer::PushParams pp{};
    for (int q = 0; q < n_peers; ++q) pp.y[q] = static_cast<char*>(y_peers[q]);
    pp.n = n_peers; pp.self = self;
    pp.row_bytes = ld * esz; pp.col_bytes = col0 * esz;
    pp.chunks_per_row = N_local * esz / 16;
    pp.total = a.M * pp.chunks_per_row;
    pp.sig = sig;
    pp.sig.wait_flag = nullptr;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int64_t blocks = (pp.total + 255) / 256;
    if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
    peer::peer_push_kernel<<<(unsigned)blocks, 256, 0, st>>>(pp);
    B200Q_LAUNCH_OK("peer_push_kernel");
    return B200Q_OK;
  }
  return fail(B200Q_ERR_UNSUPPORTED, "[quantized_matmul_sharded] only bfloat16 with K a multiple of 128 has a peer-store epilogue");
}
}  // namespace

extern "C" int b200q_peer_signal(uint32_t* const* flag_peers, int n_peers, uint32_t* epoch_local, void* stream) {
  if (!flag_peers || !epoch_local || n_peers < 1 || n_peers > kMaxPeers)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[peer_signal] between 1 and %d flags are supported (got %d)", kMaxPeers, n_peers);
  uint32_t* f[kMaxPeers] = {};
  for (int q = 0; q < n_peers; ++q) {
    if (!flag_peers[q]) return fail(B200Q_ERR_INVALID_ARGUMENT, "[peer_signal] null flag %d", q);
    f[q] = flag_peers[q];
  }
  peer::peer_signal_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7], n_peers, epoch_local);
  B200Q_LAUNCH_OK("peer_signal_kernel");
  return B200Q_OK;
}

extern "C" int b200q_peer_wait(const uint32_t* flag_local, const uint32_t* epoch_local, uint32_t* status, void* stream) {
  if (!flag_local || !epoch_local || !status) return fail(B200Q_ERR_INVALID_ARGUMENT, "[peer_wait] null pointer");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, peer::peer_wait_kernel, flag_local, epoch_local, status, g_peer_wait_limit));
  B200Q_LAUNCH_OK("peer_wait_kernel");
  return B200Q_OK;
}

extern "C" int b200q_peer_reduce(const void* slots, int n_slots, int64_t stride, int64_t n, void* y, int dtype, void* stream) {
  if (!slots || !y || n_slots < 1 || n_slots > kMaxPeers || stride < n || n < 0)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[peer_reduce] between 1 and %d slots of at least n elements each are required", kMaxPeers);
  if (n == 0) return B200Q_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((n + 8 * 256 - 1) / (8 * 256));
  if (dtype == B200Q_BF16)
    peer::peer_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)slots, n_slots, stride, n, (__nv_bfloat16*)y);
  else if (dtype == B200Q_F16)
    peer::peer_reduce_kernel<__half><<<grid, 256, 0, st>>>((const __half*)slots, n_slots, stride, n, (__half*)y);
  else if (dtype == B200Q_F32)
    peer::peer_reduce_kernel<float><<<grid, 256, 0, st>>>((const float*)slots, n_slots, stride, n, (float*)y);
  else
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[peer_reduce] Only real floating types are supported (dtype code %d).", dtype);
  B200Q_LAUNCH_OK("peer_reduce_kernel");
  return B200Q_OK;
}

extern "C" int b200q_ipc_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
  if (!ptr || !handle || bytes == 0) return fail(B200Q_ERR_INVALID_ARGUMENT, "[ipc_alloc] bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are 64 bytes");
  B200Q_CUDA_OK(cudaMalloc(ptr, bytes));
  B200Q_CUDA_OK(cudaMemset(*ptr, 0, bytes));
  cudaIpcMemHandle_t h;
  B200Q_CUDA_OK(cudaIpcGetMemHandle(&h, *ptr));
  memcpy(handle, &h, 64);
  return B200Q_OK;
}
extern "C" int b200q_ipc_open(const unsigned char handle[64], void** ptr) {
  if (!ptr || !handle) return fail(B200Q_ERR_INVALID_ARGUMENT, "[ipc_open] bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  B200Q_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return B200Q_OK;
}
extern "C" int b200q_ipc_close(void* ptr) {
  if (ptr) B200Q_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return B200Q_OK;
}
extern "C" int b200q_ipc_free(void* ptr) {
  if (ptr) B200Q_CUDA_OK(cudaFree(ptr));
  return B200Q_OK;
}

extern "C" int b200q_workspace_init(void* ws, size_t ws_bytes, void* stream) {
  if (ws_bytes == 0) return B200Q_OK;
  if (!ws) return fail(B200Q_ERR_INVALID_ARGUMENT, "[workspace_init] null workspace");
  B200Q_CUDA_OK(cudaMemsetAsync(ws, 0, ws_bytes, static_cast<cudaStream_t>(stream)));
  return B200Q_OK;
}

extern "C" int b200q_read_status(void* ws, size_t ws_bytes, void* stream, uint32_t status[4]) {
  if (!ws || ws_bytes < kStatusBytes || !status)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[read_status] workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* p = static_cast<char*>(ws) + ws_bytes - kStatusBytes;
  B200Q_CUDA_OK(cudaMemcpyAsync(status, p, kStatusBytes, cudaMemcpyDeviceToHost, st));
  B200Q_CUDA_OK(cudaMemsetAsync(p, 0, kStatusBytes, st));
  B200Q_CUDA_OK(cudaStreamSynchronize(st));
  return B200Q_OK;
}

namespace {
// B200Q_HOST_DIRECT=0: b200q_qmm_host always uses staged copies
bool host_direct() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200Q_HOST_DIRECT");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}
}  // namespace

extern "C" int b200q_qmm_host(const void* x_host, void* x_dev, const uint32_t* wq, const void* scales,
                              const void* biases, void* y_dev, void* y_host, int dtype, int64_t M, int64_t N,
                              int64_t K, int group_size, int bits, int transpose, void* ws, size_t ws_bytes,
                              void* stream) {
  QmmArgs a = make_args(x_dev, wq, scales, biases, y_dev, dtype, 1, M, N, K, group_size, bits, transpose, 0, ws,
                        ws_bytes);
  if (int rc = check_qmm_args("quantized_matmul", a)) return rc;
  if (!x_host || !y_host || !x_dev || !y_dev)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantized_matmul] null host/staging pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t es = dtype_size(dtype);
  // Small activations in pinned host memory are fetched by a copy kernel instead of a memcpy: the
  // decode kernels start under programmatic dependent launch, so their weight loads overlap the
  // PCIe read instead of queueing behind it.
  bool staged_x = false;
  if (host_direct() && (size_t)M * K * es <= (1u << 20) && ((size_t)M * K * es) % 16 == 0 &&
      !(reinterpret_cast<uintptr_t>(x_dev) & 15)) {
    cudaPointerAttributes xa{};
    if (cudaPointerGetAttributes(&xa, x_host) == cudaSuccess && xa.type == cudaMemoryTypeHost && xa.devicePointer != nullptr &&
        !(reinterpret_cast<uintptr_t>(xa.devicePointer) & 15)) {
      const int64_t n16 = (int64_t)((size_t)M * K * es / 16);
      const unsigned grid = (unsigned)((n16 + 255) / 256);
      peer::host_fetch_kernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(xa.devicePointer), static_cast<uint4*>(x_dev), n16);
      B200Q_LAUNCH_OK("host_fetch_kernel");
      staged_x = true;
    } else {
      cudaGetLastError();
    }
  }
  if (!staged_x) B200Q_CUDA_OK(cudaMemcpyAsync(x_dev, x_host, (size_t)M * K * es, cudaMemcpyHostToDevice, st));
  // A small result in pinned host memory is written by the kernel itself (the stores go out over
  // PCIe as the tiles finish), which saves the separate device-to-host copy and its launch gap.
  // B200Q_HOST_DIRECT=0 keeps the staged copy.
  if (host_direct() && (size_t)M * N * es <= (4u << 20)) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, y_host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer != nullptr) {
      a.y = attr.devicePointer;
      return run_qmm(a, st);
    }
    cudaGetLastError();   // an unregistered host pointer is not an error here
  }
  if (int rc = run_qmm(a, st)) return rc;
  B200Q_CUDA_OK(cudaMemcpyAsync(y_host, y_dev, (size_t)M * N * es, cudaMemcpyDeviceToHost, st));
  return B200Q_OK;
}
