// Non-transposed decode: y[M<=4, N] = x[M, K] * dequant(W[K, N]), W packed along N
// (reference _qmm, mlx/backend/cpu/quantized.cpp:96-152; on the reference's CUDA backend this
// shape only has the naive kernel, quantized/qmm/qmm.cu).  It is the vector-Jacobian product of
// the transposed form and streams W once: HBM-bound, CUDA cores, fp32 accumulation.
//
//  * A lane owns 16 consecutive output columns (2*bits bytes of every packed row, one vector
//    load), a warp 512 columns (256..1024 contiguous bytes per row and request), the 8 warps
//    of a CTA take every 8th row of the CTA's slab of K, and gridDim.y slabs split K so that
//    about two CTAs per SM exist whatever N is.
//  * Fields become floats without a conversion instruction: q in the top `bits` mantissa bits
//    of the float 2^bits is 2^bits + q, so acc += (x s)(2^bits + q) and 2^bits * sum(x s) is taken
//    off at the end,
//    together with sum(x b) for the biases (one scale and bias per lane and row: 16 columns
//    never straddle a group).
//  * The warps of a CTA add their columns in a shared tile; with one slab the tile is rounded
//    and written, otherwise it goes to the slab's scratch slot and the last CTA to arrive
//    (arrival counter) adds the slots in slab order and leaves slots and counter zeroed.
//    No CTA waits on another.
#include "common.cuh"
#include "kernels.h"

namespace b200q {
namespace {

constexpr int kQvmWarps = 8;
constexpr int kQvmThreads = kQvmWarps * 32;
constexpr int kQvmCols = 512;        // columns per CTA (16 per lane)
constexpr int kQvmMaxM = 4;
constexpr int kQvmMaxSlab = 2048;    // rows of K per CTA (x slab in shared memory: 4 * 2048 floats)
constexpr int kQvmTargetCtas = 296;

struct QvmPlan {
  bool ok;
  int blocks_n, slabs, slab;
};
QvmPlan qvm_plan(int64_t N, int64_t K) {
  QvmPlan p{};
  p.blocks_n = (int)((N + kQvmCols - 1) / kQvmCols);
  int want = (kQvmTargetCtas + p.blocks_n - 1) / p.blocks_n;
  const int max_slabs = (int)((K + 63) / 64);
  want = want < 1 ? 1 : (want > max_slabs ? max_slabs : want);
  int slab = (int)((K + want - 1) / want);
  slab = (slab + 7) / 8 * 8;
  if (slab > kQvmMaxSlab) slab = kQvmMaxSlab;
  p.slab = slab;
  p.slabs = (int)((K + slab - 1) / slab);
  p.ok = true;
  return p;
}

template <typename T, int BITS, int MM>
__global__ void __launch_bounds__(kQvmThreads)
qvm_kernel(const T* __restrict__ x, const uint32_t* __restrict__ wq, const T* __restrict__ scales,
           const T* __restrict__ biases, T* __restrict__ y, float* __restrict__ partial, uint32_t* __restrict__ counters,
           int M, int N, int K, int group, int slab) {
  constexpr int NW = BITS / 2;              // 32-bit words holding a lane's 16 fields
  // 2^BITS as a float with the field in the top BITS mantissa bits is the float 2^BITS + q; the
  // smallest offset that works keeps the cancellation against sum(x s) * 2^BITS small.
  constexpr int kPos = 23 - BITS;                                    // field goes to bits [kPos, 23)
  constexpr uint32_t kMagic = (uint32_t)(127 + BITS) << 23;          // 2^BITS
  constexpr float kOffset = (float)(1 << BITS);
  constexpr uint32_t kMask = ((1u << BITS) - 1u) << kPos;
  extern __shared__ float smem[];
  float* xs = smem;                          // [kQvmMaxM][slab]
  float* tile = smem + kQvmMaxM * slab;      // [kQvmMaxM][kQvmCols]
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k0 = blockIdx.y * slab;
  const int k1 = min(K, k0 + slab);
  const int n0 = blockIdx.x * kQvmCols + lane * 16;
  const bool cols = n0 < N;                 // N is a multiple of 32: a lane is all in or all out

  for (int i = tid; i < kQvmMaxM * slab; i += kQvmThreads) {
    const int m = i / slab, k = k0 + (i - m * slab);
    xs[i] = (m < M && k < k1) ? Elem<T>::to_float(x[(int64_t)m * K + k]) : 0.0f;
  }
  for (int i = tid; i < kQvmMaxM * kQvmCols; i += kQvmThreads) tile[i] = 0.0f;
  __syncthreads();

  float acc[MM][16];
  float sum_xs[MM], sum_xb[MM];
#pragma unroll
  for (int m = 0; m < MM; ++m) {
    sum_xs[m] = sum_xb[m] = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[m][j] = 0.0f;
  }
  if (cols) {
    const int64_t row_words = (int64_t)N * BITS / 32;
    const int row_groups = N / group;
    const int gcol = n0 / group;
    const uint32_t* wp = wq + (int64_t)(k0 + warp) * row_words + (int64_t)lane * NW;
    wp += (int64_t)blockIdx.x * (kQvmCols * BITS / 32);
    // Two rows per iteration: both rows' loads are issued before either is used.
    constexpr int RB = 2;
    for (int k = k0 + warp; k < k1; k += RB * kQvmWarps, wp += (int64_t)RB * kQvmWarps * row_words) {
      uint32_t w[RB][NW];
      float sv[RB], bv[RB];
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        const int ku = k + u * kQvmWarps;
        const bool on = ku < k1;
        const uint32_t* wpu = wp + (int64_t)u * kQvmWarps * row_words;
        if constexpr (NW == 4) {
          const uint4 v = on ? __ldg(reinterpret_cast<const uint4*>(wpu)) : make_uint4(0, 0, 0, 0);
          w[u][0] = v.x; w[u][1] = v.y; w[u][2] = v.z; w[u][3] = v.w;
        } else if constexpr (NW == 2) {
          const uint2 v = on ? __ldg(reinterpret_cast<const uint2*>(wpu)) : make_uint2(0, 0);
          w[u][0] = v.x; w[u][1] = v.y;
        } else {
          w[u][0] = on ? __ldg(wpu) : 0u;
        }
        sv[u] = on ? Elem<T>::to_float(scales[(int64_t)ku * row_groups + gcol]) : 0.0f;
        bv[u] = on ? Elem<T>::to_float(biases[(int64_t)ku * row_groups + gcol]) : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        const int ku = k + u * kQvmWarps;
        const int kx = ku < k1 ? ku - k0 : 0;   // rows past the slab have s = b = 0: they add nothing
        float q[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          constexpr int per_word = 32 / BITS;
          const uint32_t word = w[u][j / per_word];
          const int sh = (j % per_word) * BITS;          // field at bits [sh, sh + BITS)
          const uint32_t moved = sh >= kPos ? (word >> (sh - kPos)) : (word << (kPos - sh));
          q[j] = __uint_as_float((moved & kMask) | kMagic);
        }
#pragma unroll
        for (int m = 0; m < MM; ++m) {
          const float xv = xs[m * slab + kx];
          const float xsc = xv * sv[u];
          sum_xs[m] += xsc;
          sum_xb[m] = fmaf(xv, bv[u], sum_xb[m]);
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[m][j] = fmaf(xsc, q[j], acc[m][j]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MM; ++m) {
      const float fix = fmaf(-kOffset, sum_xs[m], sum_xb[m]);
#pragma unroll
      for (int j = 0; j < 16; ++j) atomicAdd(&tile[m * kQvmCols + lane * 16 + j], acc[m][j] + fix);
    }
  }
  __syncthreads();

  const int slabs = gridDim.y;
  const int nb = blockIdx.x * kQvmCols;
  if (slabs == 1) {
    for (int i = tid; i < M * kQvmCols; i += kQvmThreads) {
      const int m = i / kQvmCols, c = i - m * kQvmCols;
      if (nb + c < N) y[(int64_t)m * N + nb + c] = Elem<T>::from_float(tile[i]);
    }
    return;
  }
  // several slabs: this CTA's tile goes to its slot; the last CTA of the column block adds them
  float* slot = partial + ((size_t)blockIdx.x * slabs + blockIdx.y) * (kQvmMaxM * kQvmCols);
  for (int i = tid; i < M * kQvmCols; i += kQvmThreads) __stcg(slot + i, tile[i]);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned old = atomicAdd(&counters[blockIdx.x], 1u);
    s_last = old == (unsigned)(slabs - 1);
    if (s_last) counters[blockIdx.x] = 0;
    __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  float* base = partial + (size_t)blockIdx.x * slabs * (kQvmMaxM * kQvmCols);
  for (int i = tid; i < M * kQvmCols; i += kQvmThreads) {
    float v = 0.0f;
    for (int sidx = 0; sidx < slabs; ++sidx) {
      float* sp = base + (size_t)sidx * (kQvmMaxM * kQvmCols) + i;
      v += __ldcg(sp);
      __stcg(sp, 0.0f);
    }
    const int m = i / kQvmCols, c = i - m * kQvmCols;
    if (nb + c < N) y[(int64_t)m * N + nb + c] = Elem<T>::from_float(v);
  }
}

size_t qvm_counters_bytes(int blocks_n) { return (size_t)((blocks_n * 4 + 255) / 256 * 256); }

template <typename T>
int launch_qvm(const QmmArgs& a, const QvmPlan& pl, cudaStream_t st) {
  const size_t smem = (size_t)(kQvmMaxM * pl.slab + kQvmMaxM * kQvmCols) * sizeof(float);
  uint32_t* counters = reinterpret_cast<uint32_t*>(a.ws);
  float* partial = reinterpret_cast<float*>(static_cast<char*>(a.ws) + qvm_counters_bytes(pl.blocks_n));
  const dim3 grid(pl.blocks_n, pl.slabs);
  int rc = B200Q_ERR_UNSUPPORTED;
#define B200Q_QVM_LAUNCH2(BITS_, MM_)                                                                             \
  {                                                                                                               \
    cudaError_t e = cudaFuncSetAttribute(qvm_kernel<T, BITS_, MM_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));   \
    qvm_kernel<T, BITS_, MM_><<<grid, kQvmThreads, smem, st>>>((const T*)a.x, a.wq, (const T*)a.scales,           \
                                                               (const T*)a.biases, (T*)a.y, partial, counters,    \
                                                               (int)a.M, (int)a.N, (int)a.K, a.group, pl.slab);   \
    rc = B200Q_OK;                                                                                                 \
  }
#define B200Q_QVM_LAUNCH(BITS_)                        \
  {                                                    \
    if (a.M == 1) B200Q_QVM_LAUNCH2(BITS_, 1)          \
    else if (a.M == 2) B200Q_QVM_LAUNCH2(BITS_, 2)     \
    else B200Q_QVM_LAUNCH2(BITS_, 4)                   \
  }
  if (a.bits == 2) B200Q_QVM_LAUNCH(2)
  else if (a.bits == 4) B200Q_QVM_LAUNCH(4)
  else if (a.bits == 8) B200Q_QVM_LAUNCH(8)
#undef B200Q_QVM_LAUNCH2
#undef B200Q_QVM_LAUNCH
  if (rc != B200Q_OK) return fail(rc, "[quantized_matmul] qvm: unsupported bits %d", a.bits);
  B200Q_LAUNCH_OK("qvm_kernel");
  return B200Q_OK;
}

}  // namespace

bool qvm_supported(const QmmArgs& a) {
  if (a.transpose || a.w_batched || a.batch != 1) return false;
  if (a.M < 1 || a.M > kQvmMaxM || a.N < 32 || a.K < 1) return false;
  if (a.bits != 2 && a.bits != 4 && a.bits != 8) return false;
  if (a.N % a.group != 0 || a.N % 32 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.wq) & 15) || (reinterpret_cast<uintptr_t>(a.ws) & 15)) return false;
  return true;
}

size_t qvm_workspace_bytes(const QmmArgs& a) {
  if (a.N < 1 || a.K < 1) return kStatusBytes;
  const QvmPlan pl = qvm_plan(a.N, a.K);
  return qvm_counters_bytes(pl.blocks_n) + (size_t)pl.blocks_n * pl.slabs * kQvmMaxM * kQvmCols * sizeof(float) + kStatusBytes;
}

int qvm(const QmmArgs& a, cudaStream_t st) {
  const QvmPlan pl = qvm_plan(a.N, a.K);
  const size_t need = qvm_workspace_bytes(a);
  if (!a.ws || a.ws_bytes < need)
    return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul] workspace of %zu bytes required, %zu given", need, a.ws_bytes);
  switch (a.dtype) {
    case B200Q_F32: return launch_qvm<float>(a, pl, st);
    case B200Q_F16: return launch_qvm<__half>(a, pl, st);
    default: return launch_qvm<__nv_bfloat16>(a, pl, st);
  }
}

}  // namespace b200q
