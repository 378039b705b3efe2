// Shape-agnostic quantized matmul (CUDA cores, fp32 accumulation).
//
// Covers everything the specialised kernels do not: transpose == false
// (reference _qmm, mlx/backend/cpu/quantized.cpp:96-152), float32/float16 element
// types, and ragged M/N/K.  One CTA computes a 64 x 64 output tile; W is dequantised
// into shared memory as float once per 32-wide K slab and re-used by all 64 rows of x.
#include "common.cuh"
#include "kernels.h"

namespace b200q {
namespace {

constexpr int GBM = 64, GBN = 64, GBK = 32;

template <typename T, bool TRANSPOSE>
__global__ void __launch_bounds__(256)
qmm_generic_kernel(const T* __restrict__ x, const uint32_t* __restrict__ wq,
                   const T* __restrict__ scales, const T* __restrict__ biases, T* __restrict__ y,
                   int M, int N, int K, int group, int bits, int64_t w_words_per_mat,
                   int64_t g_per_mat, const uint32_t* __restrict__ lhs_idx,
                   const uint32_t* __restrict__ rhs_idx, uint32_t x_batch, uint32_t n_mats,
                   uint32_t* __restrict__ status) {
  __shared__ float xs[GBK][GBM + 1];
  __shared__ float ws[GBK][GBN + 1];
  const int b = blockIdx.z;
  int64_t xb = b, wb = b;
  if (lhs_idx != nullptr) {
    // gather form: problem b multiplies x[lhs_idx[b]] with w[rhs_idx[b]]
    const uint32_t li = lhs_idx[b], ri = rhs_idx[b];
    if (li >= x_batch || ri >= n_mats) {
      // out-of-range index: record it, leave zeros, touch no memory through it
      if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
        atomicMax(&status[0], 1u);
        status[1] = (uint32_t)b;
      }
      for (int i = threadIdx.x; i < GBM * GBN; i += 256) {
        const int m = blockIdx.y * GBM + i / GBN, n = blockIdx.x * GBN + i % GBN;
        if (m < M && n < N) y[((int64_t)b * M + m) * N + n] = Elem<T>::from_float(0.0f);
      }
      return;
    }
    xb = li;
    wb = ri;
  }
  x += xb * M * K;
  y += (int64_t)b * M * N;
  wq += wb * w_words_per_mat;
  scales += wb * g_per_mat;
  biases += wb * g_per_mat;

  const int m0 = blockIdx.y * GBM, n0 = blockIdx.x * GBN;
  const int tid = threadIdx.x;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};

  // words per packed row and groups per row of W in its stored orientation
  const int64_t row_words = TRANSPOSE ? (int64_t)K * bits / 32 : (int64_t)N * bits / 32;
  const int64_t row_groups = TRANSPOSE ? K / group : N / group;

  for (int k0 = 0; k0 < K; k0 += GBK) {
    for (int i = tid; i < GBK * GBM; i += 256) {
      const int kk = i % GBK, mm = i / GBK;
      const int m = m0 + mm, k = k0 + kk;
      xs[kk][mm] = (m < M && k < K) ? Elem<T>::to_float(x[(int64_t)m * K + k]) : 0.0f;
    }
    for (int i = tid; i < GBK * GBN; i += 256) {
      int kk, nn;
      if (TRANSPOSE) { kk = i % GBK; nn = i / GBK; } else { nn = i % GBN; kk = i / GBN; }
      const int n = n0 + nn, k = k0 + kk;
      float v = 0.0f;
      if (n < N && k < K) {
        const int64_t r = TRANSPOSE ? n : k;
        const int64_t c = TRANSPOSE ? k : n;
        const uint32_t q = stream_get_rt(wq + r * row_words, c, bits);
        const float s = Elem<T>::to_float(scales[r * row_groups + c / group]);
        const float bs = Elem<T>::to_float(biases[r * row_groups + c / group]);
        v = fmaf((float)q, s, bs);
      }
      ws[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < GBK; ++kk) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bb[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + tm + i, n = n0 + tn + j;
      if (m < M && n < N) y[(int64_t)m * N + n] = Elem<T>::from_float(acc[i][j]);
    }
}

template <typename T>
int launch_generic(const QmmArgs& a, const GatherIdx* gi, cudaStream_t st) {
  dim3 grid((unsigned)((a.N + GBN - 1) / GBN), (unsigned)((a.M + GBM - 1) / GBM), 1);
  if (grid.y > 65535)
    return fail(B200Q_ERR_UNSUPPORTED, "[quantized_matmul] No implementation for problem shape M=%lld",
                (long long)a.M);
  const bool per_mat = a.w_batched || gi != nullptr;
  const int64_t wpm = per_mat ? a.N * a.K * a.bits / 32 : 0;
  const int64_t gpm = per_mat ? a.N * a.K / a.group : 0;
  const size_t es = dtype_size(a.dtype);
  // grid.z is limited to 65535: walk the batch in slabs.
  for (int64_t b0 = 0; b0 < a.batch; b0 += 65535) {
    grid.z = (unsigned)((a.batch - b0) < 65535 ? (a.batch - b0) : 65535);
    const T* x = (const T*)a.x;
    const uint32_t* wq = a.wq;
    const T* sc = (const T*)a.scales;
    const T* bi = (const T*)a.biases;
    T* y = (T*)((char*)a.y + (size_t)b0 * a.M * a.N * es);
    const uint32_t *li = nullptr, *ri = nullptr;
    if (gi) {
      li = gi->lhs + b0;
      ri = gi->rhs + b0;
    } else {
      x += b0 * a.M * a.K;
      wq += b0 * wpm;
      sc += b0 * gpm;
      bi += b0 * gpm;
    }
    if (a.transpose)
      qmm_generic_kernel<T, true><<<grid, 256, 0, st>>>(x, wq, sc, bi, y, (int)a.M, (int)a.N, (int)a.K, a.group,
                                                        a.bits, wpm, gpm, li, ri, gi ? gi->x_batch : 0,
                                                        gi ? gi->n_mats : 0, gi ? gi->status : nullptr);
    else
      qmm_generic_kernel<T, false><<<grid, 256, 0, st>>>(x, wq, sc, bi, y, (int)a.M, (int)a.N, (int)a.K, a.group,
                                                         a.bits, wpm, gpm, li, ri, gi ? gi->x_batch : 0,
                                                         gi ? gi->n_mats : 0, gi ? gi->status : nullptr);
    B200Q_LAUNCH_OK("qmm_generic_kernel");
  }
  return B200Q_OK;
}

}  // namespace

int qmm_generic(const QmmArgs& a, cudaStream_t st, const GatherIdx* gi) {
  switch (a.dtype) {
    case B200Q_F32: return launch_generic<float>(a, gi, st);
    case B200Q_F16: return launch_generic<__half>(a, gi, st);
    default: return launch_generic<__nv_bfloat16>(a, gi, st);
  }
}

}  // namespace b200q
