// Internal interface between the C-ABI dispatch layer (api.cu) and the kernel files.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace b200q {

// Output replicated into the buffers of several GPUs (N-sharded linear with the all_gather
// fused into the epilogue): element (m, n) of the local [M, N] result goes to
// y[q][m * ld + col0 + n] for every q < n.  n == 0 means the plain output QmmArgs::y.
constexpr int kMaxPeers = 8;
// Completion signal fused into a kernel whose output goes to peer buffers: when the last thread
// block of the grid has finished (and fenced, at system scope) its peer stores, it adds n to the
// local epoch and 1 to the arrival flag of every rank - what b200q_peer_signal does as a launch of
// its own.  `counter` is a device word of this rank that starts at zero and is left at zero.
struct PeerSignal {
  uint32_t* flags[kMaxPeers];
  uint32_t* epoch;
  uint32_t* counter;
  int n;   // 0: no signal
  // Consumer-side wait: when set, the kernel does not read x or store y before this rank's flag
  // has reached the epoch as the previous kernel of the stream left it, i.e. before every rank
  // has finished the previous exchange step (bounded by wait_limit SM cycles, then status 6).
  const uint32_t* wait_flag;
  long long wait_limit;
  // 1: x is the gathered output of the previous step, so x is not read before the flag either;
  // 0: x comes from elsewhere and only the stores wait (they reuse a buffer the previous step's
  // consumers on other ranks may still be reading).
  int wait_x;
};
struct PeerOut {
  void* y[kMaxPeers];
  int n;
  int64_t ld, col0;
  PeerSignal sig;
};

#ifdef __CUDACC__
// Called by one lane of every warp that is about to touch what the previous exchange step's
// consumers may still be using.  Returns false when the bound ran out (status word set).
__device__ __forceinline__ bool peer_wait_previous(const PeerSignal& ps, uint32_t* status) {
  if (ps.wait_flag == nullptr) return true;
  const uint32_t expected = *reinterpret_cast<const volatile uint32_t*>(ps.epoch);
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ps.wait_flag) : "memory");
    if ((int32_t)(v - expected) >= 0) return true;
    if (clock64() - t0 > ps.wait_limit) {
      if (status) { atomicMax(&status[0], 6u); status[1] = v; }
      return false;
    }
    __nanosleep(100);
  }
}
// Called by ONE thread of every thread block after all peer stores of the block have been issued
// and ordered before this thread (a block- or warp-wide barrier).
__device__ __forceinline__ void peer_signal_tail(const PeerSignal& ps) {
  if (ps.n == 0) return;
  __threadfence_system();
  const unsigned old = atomicAdd(ps.counter, 1u);
  if (old == gridDim.x * gridDim.y * gridDim.z - 1) {
    *ps.counter = 0;
    __threadfence_system();
    *ps.epoch += (uint32_t)ps.n;   // what the local flag must reach before this step's output is complete
    for (int q = 0; q < ps.n; ++q) atomicAdd_system(ps.flags[q], 1u);
  }
}
#endif

struct QmmArgs {
  const void* x;
  const uint32_t* wq;
  const void* scales;
  const void* biases;
  void* y;
  int dtype;
  int64_t batch;  // independent problems (grid z); 1 when W is shared and x is flattened
  int64_t M, N, K;
  int group, bits;
  bool transpose;
  bool w_batched;  // wq/scales/biases hold `batch` matrices
  void* ws;
  size_t ws_bytes;
  PeerOut peers;
};

// Grouped (mixture-of-experts) problem for the tensor-core kernel: activation rows sorted by
// expert; the tile table lives on the device and is produced by the sort kernel of gather.cu.
struct GroupedArgs {
  const void* x_sorted;     // [n_rows, K] bf16, rows in expert order
  const uint32_t* wq;       // [E, N, K*bits/32] packed
  const void* scales;       // [E, N, K/g]
  const void* biases;
  void* y;                  // [n_rows, N]; activation row p is written to row dst_row[p]
  const void* mtiles;       // device: MTile[max_mtiles]
  const int* n_mtiles;      // device scalar
  const int* dst_row;       // device: [n_rows]
  int64_t n_rows, max_mtiles, E, N, K;
  int group, bits, nt;
  uint32_t* status;
  PeerOut peers;            // n > 0: every result row is stored into all of these [n_rows, N] buffers
};

// Per-problem operand selection of the gather form: problem i of `batch` multiplies
// x[lhs[i]] with w[rhs[i]].  Indices are range-checked on the device against
// x_batch / n_mats; a bad index zeroes its output and sets status[0].
struct GatherIdx {
  const uint32_t* lhs;
  const uint32_t* rhs;
  uint32_t x_batch, n_mats;
  uint32_t* status;
};

// qmm_generic.cu
int qmm_generic(const QmmArgs& a, cudaStream_t st, const GatherIdx* gi = nullptr);

// qmv_mma.cu : decode path, M <= 16 rows of x against W^T (transpose only, bf16)
bool qmv_mma_supported(const QmmArgs& a);
size_t qmv_mma_workspace_bytes(const QmmArgs& a);
int qmv_mma(const QmmArgs& a, cudaStream_t st);

// qmv_rows.cu : decode path, bits 2/4/8, every CTA owns whole weight rows (bulk-copy ring, no scratch)
bool qmv_rows_supported(const QmmArgs& a);
int qmv_rows(const QmmArgs& a, cudaStream_t st);
// Promise that weights are not written by the stream operation preceding a matmul (see qmv_rows.cu).
bool weights_constant();
void set_weights_constant(int on);

// qvm.cu : non-transposed decode (M <= 4, bits 2/4/8): y = x * dequant(W[K, N])
bool qvm_supported(const QmmArgs& a);
size_t qvm_workspace_bytes(const QmmArgs& a);
int qvm(const QmmArgs& a, cudaStream_t st);

// qmm_tcgen05.cu : prefill path (TMA + tcgen05 + TMEM), transpose only, bf16
bool qmm_tc_supported(const QmmArgs& a);
size_t qmm_tc_workspace_bytes(const QmmArgs& a);
int qmm_tc(const QmmArgs& a, cudaStream_t st);
int qmm_tc_grouped(const GroupedArgs& a, cudaStream_t st);

}  // namespace b200q
