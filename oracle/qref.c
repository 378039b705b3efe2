/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement (plain C) of the reference project's
 * affine group-wise quantization path.  It is the checker used by tests/, by the
 * smoke test and by the cpu_baseline leg of bench.py; the product library never
 * links, imports or executes it.
 *
 * Parity status: PINNED.  Every function below is compared bit-for-bit against the
 * reference's own CPU code (compiled from the reference checkout into
 * oracle/_ref/ref_oracle by oracle/Makefile) by tests/test_oracle_pin.py, and
 * against golden vectors that tool produced (tests/golden/).
 *
 * Reference functions restated (paths relative to the reference project root):
 *   qref_quantize     quantize<T,U>           mlx/backend/cpu/quantized.cpp:1148-1211
 *   qref_dequantize   affine_dequantize       mlx/ops.cpp:5285-5327 (op-composed: w*s then +b, in T)
 *   qref_qmm          _qmm_t<T,bits,g>        mlx/backend/cpu/quantized.cpp:154-212 (transpose)
 *                     _qmm<T,bits,g>          mlx/backend/cpu/quantized.cpp:96-152  (no transpose)
 *   qref_gather_qmm   _bs_qmm_dispatch_typed  mlx/backend/cpu/quantized.cpp:700-747
 *   half/bfloat round mlx/types/bf16.h:41-56, mlx/types/fp16.h:42-116 (round-to-nearest-even)
 *
 * Packed layout (mlx/backend/common/quantized.h:5-12, quantized.cpp:1184-1206): a row of
 * K values is a little-endian, LSB-first bit stream of K*bits bits; value k occupies bits
 * [k*bits, (k+1)*bits).
 *
 * Arithmetic model: the reference evaluates in the element type T.  For T = f16/bf16
 * every binary operation is done in float and rounded back to T
 * (mlx/types/bf16.h:74-90); this file reproduces that by rounding after each step.
 * No FMA contraction (build with -ffp-contract=off, no -march flags), matching the
 * reference build on x86-64.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

enum { QREF_F32 = 0, QREF_F16 = 1, QREF_BF16 = 2 };

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* float -> bfloat16 bits, round to nearest even (bf16.h:41-56). */
static inline uint16_t bf16_from_float(float x) {
  if (isnan(x)) return 0x7FC0;
  uint32_t u = f2u(x);
  u += ((u >> 16) & 1u) + 0x7FFFu;
  return (uint16_t)(u >> 16);
}
static inline float bf16_to_float(uint16_t b) { return u2f((uint32_t)b << 16); }

/* float -> IEEE half bits, round to nearest even, subnormals kept. */
static inline uint16_t f16_from_float(float x) {
  uint32_t u = f2u(x);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u); /* NaN */
  if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to inf (>= 65520) */
  if (a < 0x33000001u) return sign;                        /* rounds to zero (<= 2^-25) */
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) { /* subnormal half: value = m * 2^(e-23), unit = 2^-24 */
    shift = -e - 1; /* 13 + (-14 - e) */
    base = 0;
  } else {
    shift = 13;
    base = ((uint32_t)(e + 15) << 10) - 0x400u; /* implicit one of m adds 0x400 */
  }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q++;
  return (uint16_t)(sign | (base + q));
}
static inline float f16_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  if (e == 0) {
    float v = (float)m * 5.9604644775390625e-8f; /* m * 2^-24 */
    return u2f(f2u(v) | sign);
  }
  if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
  return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

static inline float load_t(const void* p, size_t i, int dt) {
  if (dt == QREF_F32) return ((const float*)p)[i];
  if (dt == QREF_F16) return f16_to_float(((const uint16_t*)p)[i]);
  return bf16_to_float(((const uint16_t*)p)[i]);
}
static inline void store_t(void* p, size_t i, int dt, float v) {
  if (dt == QREF_F32) ((float*)p)[i] = v;
  else if (dt == QREF_F16) ((uint16_t*)p)[i] = f16_from_float(v);
  else ((uint16_t*)p)[i] = bf16_from_float(v);
}
/* Round a float result to the element type T and return it as float. */
static inline float rnd_t(float v, int dt) {
  if (dt == QREF_F32) return v;
  if (dt == QREF_F16) return f16_to_float(f16_from_float(v));
  return bf16_to_float(bf16_from_float(v));
}

static int check_params(int group, int bits) {
  if (group != 32 && group != 64 && group != 128) return -1;
  if (bits < 2 || bits > 8 || bits == 7) return -2;
  return 0;
}

/* Value k of an LSB-first bit stream. */
static inline uint32_t get_q(const uint8_t* row, size_t k, int bits) {
  size_t o = k * (size_t)bits;
  size_t byte = o >> 3;
  unsigned sh = (unsigned)(o & 7);
  uint32_t v = row[byte];
  if (sh + (unsigned)bits > 8) v |= (uint32_t)row[byte + 1] << 8;
  return (v >> sh) & ((1u << bits) - 1u);
}
static inline void put_q(uint8_t* row, size_t k, int bits, uint32_t q) {
  size_t o = k * (size_t)bits;
  size_t byte = o >> 3;
  unsigned sh = (unsigned)(o & 7);
  uint32_t v = q << sh;
  row[byte] |= (uint8_t)(v & 0xFF);
  if (sh + (unsigned)bits > 8) row[byte + 1] |= (uint8_t)(v >> 8);
}

/*
 * quantize<T,U> (quantized.cpp:1148-1211).  n_elems = rows*K values, row-contiguous,
 * K divisible by group.  out must hold n_elems*bits/8 bytes.
 */
int qref_quantize(const void* w, int dt, size_t n_elems, int group, int bits,
                  uint8_t* out, void* scales, void* biases) {
  if (check_params(group, bits)) return -1;
  if (n_elems % (size_t)group) return -3;
  const float n_bins = (float)((1 << bits) - 1);
  const float eps = 1e-7f;
  size_t n_groups = n_elems / (size_t)group;
  size_t bytes_per_group = (size_t)group * bits / 8;
  memset(out, 0, n_elems * (size_t)bits / 8);
  for (size_t g = 0; g < n_groups; ++g) {
    size_t base = g * (size_t)group;
    float w_min = INFINITY, w_max = -INFINITY;
    for (int j = 0; j < group; ++j) {
      float v = load_t(w, base + j, dt);
      /* std::max(a,b) = (a<b)?b:a ; std::min(a,b) = (b<a)?b:a */
      w_max = (w_max < v) ? v : w_max;
      w_min = (v < w_min) ? v : w_min;
    }
    int mask = fabsf(w_min) > fabsf(w_max);
    float scale = (w_max - w_min) / n_bins;
    scale = (scale < eps) ? eps : scale; /* std::max(scale, eps) */
    scale = mask ? scale : -scale;
    float edge = mask ? w_min : w_max;
    float q0 = rintf(edge / scale);
    float bias = 0.0f;
    if (q0 != 0.0f) {
      scale = edge / q0;
      bias = edge;
    }
    uint8_t* gout = out + g * bytes_per_group;
    for (int j = 0; j < group; ++j) {
      float v = load_t(w, base + j, dt);
      v = rintf((v - bias) / scale);
      /* std::min(std::max(v, 0), n_bins) */
      v = (v < 0.0f) ? 0.0f : v;
      v = (n_bins < v) ? n_bins : v;
      put_q(gout, (size_t)j, bits, (uint32_t)(uint64_t)v);
    }
    store_t(scales, g, dt, scale);
    store_t(biases, g, dt, bias);
  }
  return 0;
}

/*
 * dequantize: the CPU reference has no kernel; it evaluates multiply(w, scales) then
 * add(., biases) on arrays of type T (ops.cpp:5320-5323).  Each op rounds to T.
 */
int qref_dequantize(const uint8_t* wq, const void* scales, const void* biases, int dt,
                    size_t n_elems, int group, int bits, void* out) {
  if (bits < 1 || bits > 8 || group <= 0) return -1;
  if (n_elems % (size_t)group) return -3;
  size_t n_groups = n_elems / (size_t)group;
  size_t bytes_per_group = (size_t)group * bits / 8;
  for (size_t g = 0; g < n_groups; ++g) {
    float s = load_t(scales, g, dt), b = load_t(biases, g, dt);
    const uint8_t* gin = wq + g * bytes_per_group;
    for (int j = 0; j < group; ++j) {
      float q = (float)get_q(gin, (size_t)j, bits);
      float v = rnd_t(q * s, dt);
      v = rnd_t(v + b, dt);
      store_t(out, g * (size_t)group + j, dt, v);
    }
  }
  return 0;
}

/* _qmm_t (quantized.cpp:154-212): y[m,n] = sum_k x[m,k]*(scale*q + bias), T arithmetic. */
static void qmm_t(void* y, const void* x, const uint8_t* w, const void* scales,
                  const void* biases, int dt, int M, int N, int K, int group, int bits) {
  size_t row_bytes = (size_t)K * bits / 8;
  size_t gpr = (size_t)K / group;
  if (dt == QREF_F32) { /* same operations, without the per-step rounding calls */
    const float* xf = (const float*)x;
    const float* sf = (const float*)scales;
    const float* bf = (const float*)biases;
    float* yf = (float*)y;
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) {
        const uint8_t* row = w + (size_t)n * row_bytes;
        const float* xr = xf + (size_t)m * K;
        float sum = 0.0f;
        for (size_t g = 0; g < gpr; ++g) {
          float scale = sf[(size_t)n * gpr + g], bias = bf[(size_t)n * gpr + g];
          for (int j = 0; j < group; ++j) {
            size_t k = g * group + j;
            sum += xr[k] * (scale * (float)get_q(row, k, bits) + bias);
          }
        }
        yf[(size_t)m * N + n] = sum;
      }
    return;
  }
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      const uint8_t* row = w + (size_t)n * row_bytes;
      float sum = 0.0f;
      for (size_t g = 0; g < gpr; ++g) {
        float scale = load_t(scales, (size_t)n * gpr + g, dt);
        float bias = load_t(biases, (size_t)n * gpr + g, dt);
        for (int j = 0; j < group; ++j) {
          size_t k = g * group + j;
          float q = (float)get_q(row, k, bits);
          float t = rnd_t(scale * q, dt);
          t = rnd_t(t + bias, dt);
          t = rnd_t(load_t(x, (size_t)m * K + k, dt) * t, dt);
          sum = rnd_t(sum + t, dt);
        }
      }
      store_t(y, (size_t)m * N + n, dt, sum);
    }
}

/* _qmm (quantized.cpp:96-152): w is [K, N*bits/32], scales/biases [K, N/group]. */
static void qmm_n(void* y, const void* x, const uint8_t* w, const void* scales,
                  const void* biases, int dt, int M, int N, int K, int group, int bits) {
  size_t row_bytes = (size_t)N * bits / 8;
  size_t gpr = (size_t)N / group;
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) store_t(y, (size_t)m * N + n, dt, 0.0f);
    for (int k = 0; k < K; ++k) {
      float xi = load_t(x, (size_t)m * K + k, dt);
      const uint8_t* row = w + (size_t)k * row_bytes;
      for (size_t g = 0; g < gpr; ++g) {
        float scale = load_t(scales, (size_t)k * gpr + g, dt);
        float bias = load_t(biases, (size_t)k * gpr + g, dt);
        for (int j = 0; j < group; ++j) {
          size_t n = g * group + j;
          float q = (float)get_q(row, n, bits);
          float t = rnd_t(scale * q, dt);
          t = rnd_t(t + bias, dt);
          t = rnd_t(xi * t, dt);
          float acc = load_t(y, (size_t)m * N + n, dt);
          store_t(y, (size_t)m * N + n, dt, rnd_t(acc + t, dt));
        }
      }
    }
  }
}

int qref_qmm(void* y, const void* x, const uint8_t* w, const void* scales, const void* biases,
             int dt, int M, int N, int K, int group, int bits, int transpose) {
  if (check_params(group, bits)) return -1;
  if (transpose) {
    if (K % group) return -3;
    qmm_t(y, x, w, scales, biases, dt, M, N, K, group, bits);
  } else {
    if (N % group) return -3;
    qmm_n(y, x, w, scales, biases, dt, M, N, K, group, bits);
  }
  return 0;
}

/*
 * _bs_qmm_dispatch_typed (quantized.cpp:700-747) for contiguous operands:
 * out[i] = x[lhs[i]] (M x K) * w[rhs[i]].
 */
int qref_gather_qmm(void* y, const void* x, const uint8_t* w, const void* scales,
                    const void* biases, const uint32_t* lhs, const uint32_t* rhs, size_t n_idx,
                    int dt, int M, int N, int K, int group, int bits, int transpose) {
  if (check_params(group, bits)) return -1;
  size_t esz = (dt == QREF_F32) ? 4 : 2;
  size_t w_bytes = (size_t)N * K * bits / 8;
  size_t g_els = (size_t)N * K / group;
  for (size_t i = 0; i < n_idx; ++i) {
    int rc = qref_qmm((char*)y + i * (size_t)M * N * esz,
                      (const char*)x + (size_t)lhs[i] * M * K * esz,
                      w + (size_t)rhs[i] * w_bytes,
                      (const char*)scales + (size_t)rhs[i] * g_els * esz,
                      (const char*)biases + (size_t)rhs[i] * g_els * esz,
                      dt, M, N, K, group, bits, transpose);
    if (rc) return rc;
  }
  return 0;
}
