/*
 * b200q - affine group-wise quantized matmul for NVIDIA B200 (sm_100a).
 *
 * C ABI of libb200q.so.  Every entry point replaces one backend function of the
 * reference project (paths are relative to the reference project root):
 *
 *   b200q_quantize        fast::Quantize::eval_gpu (dequantize_ == false)
 *                         mlx/backend/cuda/quantized/quantized.cpp:280-324, numerics of
 *                         quantize<T,U> mlx/backend/cpu/quantized.cpp:1148-1211
 *   b200q_dequantize      fast::Quantize::eval_gpu (dequantize_ == true), same file;
 *                         numerics of the op-composed form mlx/ops.cpp:5285-5327
 *   b200q_qmm             QuantizedMatmul::eval_gpu
 *                         mlx/backend/cuda/quantized/quantized.cpp:15-152
 *   b200q_gather_qmm      GatherQMM::eval_gpu
 *                         mlx/backend/cuda/quantized/quantized.cpp:154-278
 *   b200q_qmm_host        the same operator called with host buffers (copies inside)
 *
 * Conventions
 *   - plain pointers and sizes only; `stream` is a cudaStream_t passed as void*
 *     (NULL = the legacy default stream);
 *   - all device pointers must be valid on the CURRENT device of the calling thread;
 *   - calls only enqueue work on `stream`; they never synchronise, never allocate and
 *     never free device memory.  Scratch memory is passed in by the caller and sized
 *     with the matching *_workspace_bytes() query.  The first bytes of a workspace
 *     hold self-cleaning counters: zero the workspace once after allocating it
 *     (b200q_workspace_init) and never share one workspace between two calls that
 *     may overlap on the GPU.  b200q_qmm leaves its workspace zeroed again;
 *     b200q_gather_qmm uses everything but the last 16 bytes as plain scratch and
 *     leaves arbitrary data there (it needs only those last 16 bytes to be zero), so
 *     keep a separate workspace for it or re-initialise before reusing the memory
 *     for b200q_qmm;
 *   - return value: 0 on success; negative = rejected on the host before any launch
 *     (see the B200Q_ERR_* codes; the text of the last error of the calling thread is
 *     returned by b200q_last_error()).  B200Q_ERR_INVALID_ARGUMENT corresponds to the
 *     reference's std::invalid_argument (Python ValueError), B200Q_ERR_UNSUPPORTED to
 *     its std::runtime_error "no implementation for problem shape";
 *   - packed weights use the reference layout: each row is a little-endian LSB-first
 *     bit stream, value k in bits [k*bits, (k+1)*bits), viewed as uint32 words
 *     (mlx/backend/cpu/quantized.cpp:1184-1206); scales and biases have one entry
 *     per group of `group_size` consecutive values of a row.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200Q_VERSION 1

/* element types of x / scales / biases / y */
#define B200Q_F32 0
#define B200Q_F16 1
#define B200Q_BF16 2

#define B200Q_OK 0
#define B200Q_ERR_INVALID_ARGUMENT (-1)
#define B200Q_ERR_UNSUPPORTED (-2)
#define B200Q_ERR_CUDA (-3)
#define B200Q_ERR_WORKSPACE (-4)
#define B200Q_ERR_DEVICE (-5) /* device-side status word reported a bounded wait expired */

int b200q_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* b200q_last_error(void);

/*
 * Per-group min/max, scale, bias and pack (bit-exact with the reference CPU quantize).
 *   w       [rows, K]  dtype, row-contiguous          (in)
 *   wq      [rows, K*bits/32] uint32                   (out)
 *   scales  [rows, K/group_size] dtype                 (out)
 *   biases  [rows, K/group_size] dtype                 (out)
 * Requires group_size in {32,64,128}, bits in {2,3,4,5,6,8}, K % group_size == 0.
 */
int b200q_quantize(const void* w, int dtype, int64_t rows, int64_t K, int group_size, int bits,
                   uint32_t* wq, void* scales, void* biases, void* stream);

/*
 * out[r,k] = round_T(round_T(q[r,k] * scales[r,k/g]) + biases[r,k/g]).
 *   out [rows, K] dtype.
 */
int b200q_dequantize(const uint32_t* wq, const void* scales, const void* biases, int dtype,
                     int64_t rows, int64_t K, int group_size, int bits, void* out, void* stream);

/*
 * Quantized embedding look-up: out[i, :] = dequantize(row ids[i] of the packed matrix), the fused form
 * of QuantizedEmbedding.__call__ (python/mlx/nn/layers/quantized.py:149-158), which indexes the
 * three arrays by ids and then dequantizes.
 *   wq [rows, K*bits/32], scales/biases [rows, K/g] dtype, ids uint32 [n_ids], out [n_ids, K] dtype.
 * An id outside [0, rows) gives a row of zeros and reads nothing (the reference leaves it undefined).
 */
int b200q_dequantize_rows(const uint32_t* wq, const void* scales, const void* biases, const uint32_t* ids,
                          int64_t n_ids, int dtype, int64_t rows, int64_t K, int group_size, int bits,
                          void* out, void* stream);

/*
 * y[b] = x[b] * dequant(w[b])^T   (transpose != 0;  wq [N, K*bits/32], scales [N, K/g])
 * y[b] = x[b] * dequant(w[b])     (transpose == 0;  wq [K, N*bits/32], scales [K, N/g])
 *   x [batch, M, K], y [batch, M, N]  dtype, row-contiguous
 *   w_batch_stride: 0 = one weight matrix shared by all batches (x is then treated as
 *   [batch*M, K]); otherwise 1 = wq/scales/biases hold `batch` consecutive matrices.
 *   ws/ws_bytes: scratch of at least b200q_qmm_workspace_bytes(...) bytes (may be NULL
 *   when that query returns 0).
 * Accumulation is in float32; results are rounded once to dtype.
 */
size_t b200q_qmm_workspace_bytes(int dtype, int64_t batch, int64_t M, int64_t N, int64_t K,
                                 int group_size, int bits, int transpose);
int b200q_qmm(const void* x, const uint32_t* wq, const void* scales, const void* biases, void* y,
              int dtype, int64_t batch, int64_t M, int64_t N, int64_t K, int group_size, int bits,
              int transpose, int64_t w_batch_stride, void* ws, size_t ws_bytes, void* stream);

/*
 * out[i] = x[lhs_idx[i]] (M x K) * dequant(w[rhs_idx[i]])   for i in [0, n_idx)
 *   x [x_batch, M, K]; wq [E, ...], scales/biases [E, ...]; lhs_idx/rhs_idx uint32 [n_idx]
 *   (already broadcast against each other, as the reference front-end does,
 *   mlx/ops.cpp:5591-5594); y [n_idx, M, N].
 *   sorted_flags: bit0 = lhs indices sorted, bit1 = rhs indices sorted (hints only).
 * Index values are range-checked on the device; an out-of-range index leaves the
 * corresponding output rows zero and sets the status word (see b200q_read_status).
 */
size_t b200q_gather_qmm_workspace_bytes(int dtype, int64_t n_idx, int64_t x_batch, int64_t E,
                                        int64_t M, int64_t N, int64_t K, int group_size, int bits,
                                        int transpose);
int b200q_gather_qmm(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                     const uint32_t* lhs_idx, const uint32_t* rhs_idx, int64_t n_idx, void* y,
                     int dtype, int64_t x_batch, int64_t E, int64_t M, int64_t N, int64_t K,
                     int group_size, int bits, int transpose, int sorted_flags, void* ws,
                     size_t ws_bytes, void* stream);

/* Zero a freshly allocated workspace (enqueued on `stream`). */
int b200q_workspace_init(void* ws, size_t ws_bytes, void* stream);

/*
 * Device status word: kernels never trap; a bounded wait that expires or a bad gather
 * index records a non-zero code in the last 16 bytes of the workspace.  This helper
 * synchronises `stream`, copies the word to the host, clears it and returns it in
 * *status (0 = clean).
 */
int b200q_read_status(void* ws, size_t ws_bytes, void* stream, uint32_t status[4]);

/*
 * Host-buffer form of b200q_qmm for callers that hold activations in host memory:
 * copies x (host, ideally pinned) to x_dev, runs the operator, copies y_dev back to
 * y_host, all on `stream`, and returns without synchronising.  When y_host is pinned and the
 * result is at most 4 MiB the kernel writes it to host memory itself and y_dev is not used.  Weights, scales and
 * biases are device resident.  x_dev / y_dev are caller-provided device staging
 * buffers of M*K and M*N elements.
 */
int b200q_qmm_host(const void* x_host, void* x_dev, const uint32_t* wq, const void* scales,
                   const void* biases, void* y_dev, void* y_host, int dtype, int64_t M, int64_t N,
                   int64_t K, int group_size, int bits, int transpose, void* ws, size_t ws_bytes,
                   void* stream);

/*
 * Decode (1 <= M <= 16 rows of bfloat16 x, transpose form) for callers that cannot
 * allocate device memory and therefore cannot supply the workspace b200q_qmm needs:
 * e.g. a plugin running under a host framework's allocator or capture rules, or a
 * serving loop that bans allocator calls after start-up.  This entry point has no
 * counterpart in the reference project.  It allocates nothing: its scratch is a fixed
 * array inside the library image (about 2 MiB of device memory on every GPU that loads
 * the library, held until the process exits), large enough for
 * N <= B200Q_STATIC_SCRATCH_MAX_N weight rows; a larger N is rejected with
 * B200Q_ERR_UNSUPPORTED.  The first call on each device looks up the array's device
 * address; make that first call outside any stream capture.  All calls on a device
 * share the array: calls that may overlap on the GPU race on it and must be
 * serialised by the caller.  The used part is cleared on `stream` before every launch.
 * Same results as b200q_qmm on the same inputs.
 */
#define B200Q_STATIC_SCRATCH_MAX_N 32768
int b200q_qmm_decode_static(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                            void* y, int dtype, int64_t M, int64_t N, int64_t K, int group_size,
                            int bits, void* stream);

/*
 * Two chained gather_qmm over the same index pairs (the expert MLP of a mixture-of-experts
 * block as the reference benchmarks it, benchmarks/python/gather_qmm_bench.py:52-63):
 *   h[i] = x[lhs_idx[i]] * dequant(w1[rhs_idx[i]])^T    (M x N1, rounded to bfloat16)
 *   y[i] = h[i]          * dequant(w2[rhs_idx[i]])^T    (M x N2)
 * The index pairs are sorted by expert once, the first product leaves its rows in expert
 * order in the workspace and the second reads them there: one sort, one row gather and one
 * scatter instead of two of each.  w1 [E, N1, K1*bits/32], w2 [E, N2, N1*bits/32]; bfloat16,
 * transpose form, K1 and N1 multiples of 128 (B200Q_ERR_UNSUPPORTED otherwise: call
 * b200q_gather_qmm twice).  Index checks and status word as b200q_gather_qmm.
 */
size_t b200q_gather_qmm_chain_workspace_bytes(int64_t n_idx, int64_t E, int64_t M, int64_t N1, int64_t K1);
int b200q_gather_qmm_chain(const void* x, const uint32_t* wq1, const void* scales1, const void* biases1,
                           const uint32_t* wq2, const void* scales2, const void* biases2,
                           const uint32_t* lhs_idx, const uint32_t* rhs_idx, int64_t n_idx, void* y, int dtype,
                           int64_t x_batch, int64_t E, int64_t M, int64_t N1, int64_t K1, int64_t N2,
                           int group_size, int bits, void* ws, size_t ws_bytes, void* stream);

/*
 * Gated expert MLP of a mixture-of-experts block over one set of index pairs, one sort:
 *   g[i] = x[lhs_idx[i]] * dequant(w_gate[rhs_idx[i]])^T,  u[i] = x[lhs_idx[i]] * dequant(w_up[rhs_idx[i]])^T
 *   h[i] = bfloat16( silu(g[i]) * u[i] )        silu(t) = t / (1 + exp(-t)), fp32 on the bfloat16 g and u
 *   y[i] = h[i] * dequant(w_down[rhs_idx[i]])^T
 * i.e. three gather_qmm (mlx/ops.cpp:5553-5629) and the activation between them, which the
 * reference runs as separate operators with a sort and a scatter around each.
 * w_gate, w_up [E, H, K1*bits/32]; w_down [E, N2, H*bits/32]; bfloat16, transpose form, K1 and H
 * multiples of 128 (B200Q_ERR_UNSUPPORTED otherwise).  Index checks and status word as
 * b200q_gather_qmm.
 */
size_t b200q_gather_qmm_swiglu_workspace_bytes(int64_t n_idx, int64_t E, int64_t M, int64_t H, int64_t K1);
int b200q_gather_qmm_swiglu(const void* x, const uint32_t* wq_gate, const void* scales_gate, const void* biases_gate,
                            const uint32_t* wq_up, const void* scales_up, const void* biases_up,
                            const uint32_t* wq_down, const void* scales_down, const void* biases_down,
                            const uint32_t* lhs_idx, const uint32_t* rhs_idx, int64_t n_idx, void* y, int dtype,
                            int64_t x_batch, int64_t E, int64_t M, int64_t H, int64_t K1, int64_t N2,
                            int group_size, int bits, void* ws, size_t ws_bytes, void* stream);

/*
 * N-sharded linear with the all_gather fused into the matmul epilogue.  Replaces the pair
 * QuantizedAllToShardedLinear.__call__ + all_gather of the reference
 * (python/mlx/nn/layers/distributed.py:357-455, mlx/distributed/ops.cpp:62-84,
 * mlx/distributed/nccl/nccl.cpp:346-358): rank r holds rows [r*N/R, (r+1)*N/R) of
 * wq / scales / biases, x is replicated, and every rank ends up with the full [M, N].
 * Instead of a collective after the kernel, the kernel stores every finished output
 * tile straight into the output buffer of EVERY rank (peer stores over NVLink):
 *   y_peers[q][m * ld + col0 + n] = y_local[m][n]   for q < n_peers, n < N_local
 * y_peers are device pointers valid on the current device (the local buffer and the
 * peer-mapped buffers of the other ranks, see b200q_ipc_*), ld = N (row pitch of the
 * full output), col0 = rank * N_local.  bfloat16, transpose form only; other problems
 * return B200Q_ERR_UNSUPPORTED (use b200q_qmm and a collective).
 *
 * Completion across ranks uses two 32-bit words per rank that only ever grow: a flag that
 * every rank adds 1 to once per step, and a local epoch.  After b200q_qmm_sharded,
 * b200q_peer_signal (ordered after all earlier work on `stream`, system scope) adds
 * n_peers to the local epoch and 1 to the flag of every rank; b200q_peer_wait makes
 * `stream` wait until the local flag has reached the local epoch, i.e. until every
 * rank's block of this step has landed.  Both values live on the device, so a captured
 * sequence can be replayed.  The wait is bounded (about one second): when it runs out,
 * code 6 is stored in status[0] (device memory, 4 words, e.g. the status word of the
 * workspace) and the stream continues.  Flag and epoch must start at zero.
 */
int b200q_qmm_sharded(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                      void* const* y_peers, int n_peers, int64_t ld, int64_t col0, int dtype,
                      int64_t M, int64_t N_local, int64_t K, int group_size, int bits, void* ws,
                      size_t ws_bytes, void* stream);
/*
 * Expert-parallel gather_qmm: the E_total weight matrices are spread over the ranks in
 * contiguous blocks (this rank holds experts [e_lo, e_lo + E_local) in wq_local /
 * scales_local / biases_local), x and the index pairs are the same on every rank.  Every
 * rank multiplies only the pairs of its own experts and stores each result row into the
 * [n_idx * M, N] output buffer of EVERY rank (y_peers, self = index of this rank's own
 * buffer), so after b200q_peer_signal / b200q_peer_wait all ranks hold the complete
 * output: a variable-size all_gather without padding or a collective.  Replaces
 * GatherQMM::eval_gpu (mlx/backend/cuda/quantized/quantized.cpp:154-278) followed by the
 * exchange of the rows in an expert-parallel layer.  bfloat16, transpose form, K a multiple
 * of 128 only (B200Q_ERR_UNSUPPORTED otherwise).  Workspace as b200q_gather_qmm with E =
 * E_total.  Out-of-range indices: as b200q_gather_qmm, zeroed in this rank's own buffer.
 */
int b200q_gather_qmm_sharded(const void* x, const uint32_t* wq_local, const void* scales_local,
                             const void* biases_local, const uint32_t* lhs_idx, const uint32_t* rhs_idx,
                             int64_t n_idx, void* const* y_peers, int n_peers, int self, int dtype,
                             int64_t x_batch, int64_t E_total, int64_t e_lo, int64_t E_local, int64_t M,
                             int64_t N, int64_t K, int group_size, int bits, void* ws, size_t ws_bytes,
                             void* stream);
int b200q_peer_signal(uint32_t* const* flag_peers, int n_peers, uint32_t* epoch_local, void* stream);
int b200q_peer_wait(const uint32_t* flag_local, const uint32_t* epoch_local, uint32_t* status, void* stream);
/*
 * The same two operators with b200q_peer_signal folded into the matmul: the last thread block
 * to finish its peer stores fences at system scope, adds n_peers to the local epoch and 1 to
 * every rank's flag, so a step is two launches (matmul, wait) instead of three.
 * counter_local is one more device word of this rank (starts at zero, left at zero) that counts
 * finished thread blocks.  Where the selected kernel has no such epilogue (the register-path
 * decode kernel for 3-, 5- and 6-bit weights) the signal is launched separately, as before.
 * wait_flag_local (b200q_qmm_sharded_signal only; may be NULL) moves the wait to the consumer:
 * when given (this rank's own flag), the call does not read x nor store y before the flag has
 * reached the epoch the previous step left, i.e. before every rank has finished the previous
 * exchange step - what a kernel needs whose x is the gathered output of that step.  The decode
 * kernel waits inside (its weight stream starts meanwhile, so a chain of sharded layers costs
 * one launch per layer); in front of the other kernels the wait is launched on its own.  The
 * last step of a chain still needs b200q_peer_wait before its result is used.  Same bound and
 * status code as b200q_peer_wait.  wait_before_x = 1 when x is the gathered output of the previous
 * step (a stack of sharded layers feeding each other); 0 when x comes from elsewhere (replicated
 * input, the output of another exchange that was waited for): then only the stores into the
 * exchange buffers wait, which guards the reuse of a buffer the other ranks' consumers of the
 * step before may still read, and the kernel's loads and products overlap the previous exchange.
 * self = index of this rank's own buffer in y_peers, or -1 if unknown.  When known, a prefill-size
 * result over more than four ranks is stored locally by the product and moved to the other ranks by
 * a copy kernel with 16-byte accesses (the tensor-core epilogue's peer stores are 64-byte warp
 * stores per destination and take longer than the product there); the copy kernel signals.
 * The exchange these replace: AllGather::eval_gpu (mlx/backend/cuda/distributed.cu:57-83).
 */
int b200q_qmm_sharded_signal(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                             void* const* y_peers, int n_peers, int64_t ld, int64_t col0, int dtype,
                             int64_t M, int64_t N_local, int64_t K, int group_size, int bits,
                             uint32_t* const* flag_peers, uint32_t* epoch_local, uint32_t* counter_local,
                             const uint32_t* wait_flag_local, int wait_before_x, int self, void* ws,
                             size_t ws_bytes, void* stream);
int b200q_gather_qmm_sharded_signal(const void* x, const uint32_t* wq_local, const void* scales_local,
                                    const void* biases_local, const uint32_t* lhs_idx, const uint32_t* rhs_idx,
                                    int64_t n_idx, void* const* y_peers, int n_peers, int self, int dtype,
                                    int64_t x_batch, int64_t E_total, int64_t e_lo, int64_t E_local, int64_t M,
                                    int64_t N, int64_t K, int group_size, int bits,
                                    uint32_t* const* flag_peers, uint32_t* epoch_local, uint32_t* counter_local,
                                    void* ws, size_t ws_bytes, void* stream);
/*
 * Bound of b200q_peer_wait in milliseconds (process-wide, default about 1000; <= 0 restores the
 * default).  When the bound runs out the wait stores code 6 in status[0] and the stream goes on
 * with an incomplete buffer: the caller must read the status (b200q_read_status) before it uses
 * a result whose peers may lag by more than the bound.  No counterpart in the reference, whose
 * NCCL calls block without a bound (mlx/distributed/nccl/nccl.cpp:346-358).
 */
void b200q_set_peer_wait_limit_ms(int ms);

/*
 * K-sharded linear with the all_reduce fused into the exchange (QuantizedShardedToAllLinear of
 * the reference, python/mlx/nn/layers/distributed.py:490-588: matmul over this rank's slice of
 * the input dimension, then all_sum, mlx/distributed/nccl/nccl.cpp:389-406).  Every rank calls
 * b200q_qmm_sharded with y_peers[q] = slot `rank` of rank q's buffer (ld = N, col0 = 0), so its
 * partial [M, N] lands in every rank; after b200q_peer_signal / b200q_peer_wait,
 * b200q_peer_reduce adds this rank's n_slots slots (each `stride` elements apart, n = M * N
 * used) in fp32, in slot order, and rounds once to the output type: all ranks get identical
 * results.
 */
int b200q_peer_reduce(const void* slots, int n_slots, int64_t stride, int64_t n, void* y, int dtype, void* stream);

/*
 * Set-up helpers for the peer buffers (not capture-safe, they allocate): a buffer that
 * other processes on the same machine can map (cudaMalloc + cudaIpcGetMemHandle), and
 * the mapping of another process's buffer into this one (cudaIpcOpenMemHandle with lazy
 * peer access).  `handle` is the 64-byte CUDA IPC handle, to be exchanged by the caller
 * (e.g. torch.distributed.all_gather_object).
 */
int b200q_ipc_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
int b200q_ipc_open(const unsigned char handle[64], void** ptr);
int b200q_ipc_close(void* ptr);
int b200q_ipc_free(void* ptr);

/*
 * GGUF quantized tensors -> this library's affine layout, on the device (group size 32;
 * 4-bit for Q4_0 / Q4_1, 8-bit for Q8_0; float16 scales and biases).  Replaces the host-side
 * repack of the reference's loader (mlx/io/gguf_quants.cpp:11-102).  `blocks` is the tensor's
 * raw block data (n_blocks blocks of 18 / 20 / 34 bytes, 2-byte aligned), gguf_type the GGUF
 * type id (2 = Q4_0, 3 = Q4_1, 8 = Q8_0).  Outputs: wq n_blocks*4 (4-bit) or n_blocks*8 (8-bit)
 * words, scales and biases n_blocks float16 each; a [rows, K] tensor has K/32 consecutive
 * blocks per row, so the outputs are already [rows, K*bits/32] and [rows, K/32].
 */
int b200q_gguf_repack(const void* blocks, int gguf_type, int64_t n_blocks, uint32_t* wq, void* scales,
                      void* biases, void* stream);

/*
 * Introspection for tests and benchmarks: name of the kernel family b200q_qmm would
 * launch for this problem ("qmv_rows", "qmv_mma", "qmm_tcgen05", "qvm",
 * "qmm_generic").
 */
const char* b200q_qmm_kernel_name(int dtype, int64_t batch, int64_t M, int64_t N, int64_t K,
                                  int group_size, int bits, int transpose);

/*
 * Process-wide promise about the stream order around matmul calls: on != 0 says that the packed
 * weights, scales and biases passed to b200q_qmm / b200q_qmm_sharded are never written by the
 * operation that directly precedes the call on its stream (the normal case in inference: they
 * are constants).  The decode kernel then requests them while the previous kernel of the stream
 * is still finishing (programmatic dependent launch) instead of after it; x, y and the workspace
 * are always touched only after the previous kernel has completed.  Default 0 (or the
 * environment variable B200Q_WEIGHTS_CONSTANT=1).  With the promise broken (e.g. b200q_quantize
 * directly followed by b200q_qmm on the same buffers) the matmul may read stale weights.
 * The reference has no counterpart: its command encoder orders whole kernels
 * (mlx/backend/cuda/device.cpp:243-359).
 */
void b200q_set_weights_constant(int on);

/* Number of kernel launches issued by this library on the calling thread so far. */
uint64_t b200q_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
