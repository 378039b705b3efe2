// Decode path: y[M<=16, N] = x[M, K] * dequant(W[N, K])^T, bf16, HBM-bound.
//
// Replaces cu::qmv_kernel / the small-M use of cu::qmm_sm80_kernel of the reference
// (mlx/backend/cuda/quantized/qmm/qmv.cu:84-209, quantized.cpp:106-136).
//
// Design (one persistent CTA per SM, 16 warps):
//  * The problem is flattened into "steps" of (16*RT weight rows) x (128 k).  Every CTA
//    owns a contiguous span of steps, every warp a contiguous sub-span, so all SMs
//    stream the same number of packed-weight bytes (+-1 step) whatever N is.
//  * A lane loads 32 consecutive k of one weight row per 128-bit (4-bit) load, straight
//    from HBM into registers (no shared-memory staging of W: each byte is used once).
//    Loads are software-pipelined PIPE steps ahead.
//  * Fields are unpacked in registers to bf16 pairs with shift+lop3 ("0x4300 | q" is the
//    bf16 number 128+q), turned into s*q+b with two bf16x2 ops, and fed to
//    mma.sync.m16n8k16 as the A operand (weights = M dimension of the MMA, tokens = N),
//    accumulating in fp32.  The k order inside an MMA is permuted to suit the unpack;
//    x is staged once per CTA in shared memory in exactly the B-fragment order, so a
//    lane fetches its B fragments for 8 k-values with one conflict-free 128-bit read.
//  * Warps add their fp32 partial tiles into a per-CTA shared tile buffer; row blocks
//    that are complete inside the CTA are written directly, the (at most two) blocks
//    shared with a neighbouring CTA go through fp32 global atomics plus an arrival
//    counter, the last arriver converts and re-zeroes (no CTA ever waits on another).
//
// Scratch (caller-provided workspace, zero on first use, self-cleaning afterwards):
//   [ counters: ceil(N/16) x u32 | fp32 partial tiles: ceil(N/16)*16 rows x 16 tokens ]
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace b200q {
namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
// Steps of weight loads in flight per lane: `budget` packed words (4 bytes each) of
// registers, at least two steps.
__host__ __device__ constexpr int pipe_depth(int words_per_step, int budget) {
  int d = budget / words_per_step;
  return d < 2 ? 2 : (d > 6 ? 6 : d);
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
  return d;
}
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ldg_nc_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.b32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc_u64(const uint32_t* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_nc_u128(const uint32_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Loads the BITS words holding 32 consecutive fields (a "chunk") of one row.
template <int BITS>
__device__ __forceinline__ void load_chunk(const uint32_t* __restrict__ p, uint32_t (&w)[BITS]) {
  if constexpr (BITS == 4) {
    uint4 v = ldg_nc_u128(p);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else if constexpr (BITS == 8) {
    uint4 v = ldg_nc_u128(p), u = ldg_nc_u128(p + 4);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    w[4] = u.x; w[5] = u.y; w[6] = u.z; w[7] = u.w;
  } else if constexpr (BITS == 2) {
    uint2 v = ldg_nc_u64(p);
    w[0] = v.x; w[1] = v.y;
  } else if constexpr (BITS == 6) {
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      uint2 v = ldg_nc_u64(p + 2 * i);
      w[2 * i] = v.x; w[2 * i + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < BITS; ++i) w[i] = ldg_nc_u32(p + i);
  }
}

// Dequantises the 8 fields of block c (k = 8c..8c+7 of the chunk) into four bf16x2
// registers P[i] = (w[8c+i], w[8c+i+4]), i = 0..3, with w = s*q + b rounded once.
// s2/b2 hold the scale / bias replicated in both halves.
template <int BITS>
__device__ __forceinline__ void dequant_block(const uint32_t (&w)[BITS], int c, uint32_t s2,
                                              uint32_t b2, float sf, float bf, uint32_t (&P)[4]) {
  constexpr uint32_t kMagic = 0x43004300u;  // (128.0, 128.0)
  if constexpr (BITS == 4) {
    const uint32_t v = w[c];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t t = lop3_and_or(v >> (4 * i), 0x000F000Fu, kMagic);
      P[i] = fma_bf16x2(sub_bf16x2(t, kMagic), s2, b2);
    }
  } else if constexpr (BITS == 2) {
    // 16 fields per word: bytes (0,1) hold fields 0..7 of the even block, (2,3) the odd one.
    const uint32_t v = __byte_perm(w[c >> 1], 0u, (c & 1) ? 0x4342 : 0x4140);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t t = lop3_and_or(v >> (2 * i), 0x00030003u, kMagic);
      P[i] = fma_bf16x2(sub_bf16x2(t, kMagic), s2, b2);
    }
  } else if constexpr (BITS == 8) {
    // float route: 0x4B0000qq is 2^23 + q exactly.
    const uint32_t lo = w[2 * c], hi = w[2 * c + 1];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float a = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7540 | i)) - 8388608.0f;
      float d = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7540 | i)) - 8388608.0f;
      P[i] = pack_bf16x2(fmaf(a, sf, bf), fmaf(d, sf, bf));
    }
  } else {
    // 3/5/6-bit fields straddle words: extract each field with a funnel shift.
    constexpr uint32_t mask = (1u << BITS) - 1u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e0 = 8 * c + i, e1 = e0 + 4;
      const int w0 = (e0 * BITS) >> 5, s0 = (e0 * BITS) & 31;
      const int w1 = (e1 * BITS) >> 5, s1 = (e1 * BITS) & 31;
      uint32_t f0 = (s0 + BITS > 32) ? __funnelshift_r(w[w0], w[(w0 + 1) % BITS], s0) : (w[w0] >> s0);
      uint32_t f1 = (s1 + BITS > 32) ? __funnelshift_r(w[w1], w[(w1 + 1) % BITS], s1) : (w[w1] >> s1);
      uint32_t t = lop3_and_or(f0, mask, kMagic);
      asm("bfi.b32 %0, %1, %2, 16, %3;" : "=r"(t) : "r"(f1), "r"(t), "n"(BITS));
      P[i] = fma_bf16x2(sub_bf16x2(t, kMagic), s2, b2);
    }
  }
}

struct QmvParams {
  const __nv_bfloat16* x;
  const uint32_t* wq;
  const __nv_bfloat16* scales;
  const __nv_bfloat16* biases;
  __nv_bfloat16* y[kMaxPeers];  // output buffers (one, or one per GPU of an N-sharded layer)
  int n_out;
  long long ld, col0;  // row pitch and first column of this result inside every output buffer
  uint32_t* counters;  // [n_row_blocks]
  float* partial;      // [n_row_blocks][16*RT rows][8*MT tokens]
  int M, N, K;
  int ksteps;          // K / 128
  int n_row_blocks;    // ceil(N / (16*RT))
  long long total_steps;
  int tilebuf_blocks;  // row blocks a CTA span can touch
  int group_shift;     // log2(group_size / 32)
  int early;           // weights may be requested before the previous kernel of the stream has ended
};

template <int BITS, int MT, int RT>
__global__ void __launch_bounds__(kThreads, 1)
qmv_mma_kernel(const QmvParams p) {
  constexpr int ROWS = 16 * RT;      // weight rows per step
  constexpr int TOKS = 8 * MT;       // padded token count
  constexpr int NLD = 2 * RT;        // row halves (chunks) per lane per step
  constexpr int kPipe = pipe_depth(NLD * BITS, RT == 1 ? 48 : 32);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* xs = reinterpret_cast<uint4*>(smem_raw);  // [MT][ksteps][4][32] uint4
  float* tilebuf = reinterpret_cast<float*>(smem_raw + (size_t)MT * p.ksteps * 4 * 32 * 16);
  __shared__ int s_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  {
    // The first mma.sync of a kernel is slow (the tensor pipe wakes up): issue one now, while the
    // first loads are in flight anyway.  Its result is never used.
    float d0, d1, d2, d3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%4,%4,%4}, {%4,%4}, {%5,%5,%5,%5};"
                 : "=f"(d0), "=f"(d1), "=f"(d2), "=f"(d3) : "r"(0u), "f"(0.0f));
  }
  // let the next kernel of the stream start as soon as SMs free up (it waits before it reads x)
  asm volatile("griddepcontrol.launch_dependents;");
  const long long T = p.total_steps;  // < 2^31 (checked on the host)
  const int G = gridDim.x;
  const int ksteps = p.ksteps;
  const int cta_s0 = (int)((long long)blockIdx.x * T / G);
  const int cta_s1 = (int)((long long)(blockIdx.x + 1) * T / G);
  const int L = cta_s1 - cta_s0;
  const int s0 = cta_s0 + warp * L / kWarps;
  const int s1 = cta_s0 + (warp + 1) * L / kWarps;
  const int rb_first = cta_s0 / ksteps;

  const int64_t row_words = (int64_t)p.K * BITS / 32;
  const int row_groups = p.K >> (5 + p.group_shift);
  const unsigned short* sc_base = reinterpret_cast<const unsigned short*>(p.scales);
  const unsigned short* bi_base = reinterpret_cast<const unsigned short*>(p.biases);

  // ---- weight-load stream: state advances one step per issue() ---------------------
  uint32_t wbuf[kPipe][NLD][BITS];
  uint32_t sbuf[kPipe][NLD];  // scale | bias << 16
  const uint32_t* wp[NLD];    // this lane's chunk of each row half at the next step
  int gbase[NLD];             // first group of each row
  int irb = s0 / ksteps, ikb = s0 - irb * ksteps;
  auto set_rows = [&]() {
#pragma unroll
    for (int j = 0; j < NLD; ++j) {
      int row = irb * ROWS + j * 8 + g;
      row = row < p.N ? row : p.N - 1;  // ragged N: clamp, results are discarded later
      wp[j] = p.wq + (int64_t)row * row_words + (int64_t)(ikb * 4 + t) * BITS;
      gbase[j] = row * row_groups;
    }
  };
  set_rows();
  auto issue = [&](int slot) {
    const int grp = (ikb * 4 + t) >> p.group_shift;
#pragma unroll
    for (int j = 0; j < NLD; ++j) {
      load_chunk<BITS>(wp[j], wbuf[slot][j]);
      const uint32_t sc = __ldg(sc_base + gbase[j] + grp);
      const uint32_t bi = __ldg(bi_base + gbase[j] + grp);
      sbuf[slot][j] = sc | (bi << 16);
      wp[j] += 4 * BITS;
    }
    if (++ikb == ksteps) {
      ikb = 0;
      ++irb;
      set_rows();
    }
  };
  // Programmatic dependent launch: when the caller has promised that weights are constants
  // (b200q_set_weights_constant), the first weight loads run while the previous kernel of the
  // stream (e.g. the previous decode step) is still finishing; otherwise they too wait for it,
  // since that kernel may be the one that wrote them (a quantize, a cast, a repack).
  // Everything that kernel may produce (x) or still use (y, the workspace) is touched only after
  // the wait.  Without the launch attribute the instruction returns at once.
  if (!p.early) asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
  for (int d = 0; d < kPipe; ++d)
    if (s0 + d < s1) issue(d);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // ---- stage x in B-fragment order; zero the tile buffer -------------------------
  {
    constexpr int U = 8;  // loads in flight per thread
    const int per_mt = ksteps * 128;   // items of one 8-token half: [ksteps][4][32]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      uint4* xs_mt = xs + (size_t)mt * per_mt;
      for (int base = tid; base < per_mt; base += kThreads * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = base + u * kThreads;
          v[u] = make_uint4(0, 0, 0, 0);
          if (j < per_mt) {
            const int ln = j & 31, c = (j >> 5) & 3, kb = j >> 7;
            const int tok = mt * 8 + (ln >> 2);
            const int k8 = kb * 128 + 32 * (ln & 3) + 8 * c;
            if (tok < p.M) v[u] = __ldg(reinterpret_cast<const uint4*>(p.x + (int64_t)tok * p.K + k8));
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = base + u * kThreads;
          if (j < per_mt) {
            uint4 o;
            o.x = __byte_perm(v[u].x, v[u].z, 0x5410);  // (x0, x4)
            o.y = __byte_perm(v[u].x, v[u].z, 0x7632);  // (x1, x5)
            o.z = __byte_perm(v[u].y, v[u].w, 0x5410);  // (x2, x6)
            o.w = __byte_perm(v[u].y, v[u].w, 0x7632);  // (x3, x7)
            xs_mt[j] = o;
          }
        }
      }
    }
    const int nbuf = p.tilebuf_blocks * ROWS * TOKS;
    for (int i = tid; i < nbuf; i += kThreads) tilebuf[i] = 0.0f;
  }
  __syncthreads();

  // ---- main loop -------------------------------------------------------------------
  float acc[RT][MT][4];
#pragma unroll
  for (int a = 0; a < RT; ++a)
#pragma unroll
    for (int b = 0; b < MT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.0f;
  int prb = s0 / ksteps, pkb = s0 - prb * ksteps;
  const uint4* xs_lane = xs + lane;

  auto flush = [&](int rb) {
    float* tb = tilebuf + (size_t)(rb - rb_first) * ROWS * TOKS;
#pragma unroll
    for (int a = 0; a < RT; ++a)
#pragma unroll
      for (int b = 0; b < MT; ++b) {
        const int r = a * 16 + g, tk = b * 8 + 2 * t;
        atomicAdd(&tb[r * TOKS + tk], acc[a][b][0]);
        atomicAdd(&tb[r * TOKS + tk + 1], acc[a][b][1]);
        atomicAdd(&tb[(r + 8) * TOKS + tk], acc[a][b][2]);
        atomicAdd(&tb[(r + 8) * TOKS + tk + 1], acc[a][b][3]);
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.0f;
      }
  };

  auto process = [&](int slot) {
    uint32_t s2[NLD], b2[NLD];
    float sf[NLD], bf[NLD];
#pragma unroll
    for (int j = 0; j < NLD; ++j) {
      const uint32_t sb = sbuf[slot][j];
      s2[j] = __byte_perm(sb, sb, 0x1010);
      b2[j] = __byte_perm(sb, sb, 0x3232);
      if constexpr (BITS == 8) {
        sf[j] = __uint_as_float(sb << 16);
        bf[j] = __uint_as_float(sb & 0xFFFF0000u);
      } else {
        sf[j] = 0.0f;
        bf[j] = 0.0f;
      }
    }
    const uint4* xk = xs_lane + pkb * 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 xf[MT];
#pragma unroll
      for (int b = 0; b < MT; ++b) xf[b] = xk[(b * ksteps * 4 + c) * 32];
#pragma unroll
      for (int a = 0; a < RT; ++a) {
        uint32_t P0[4], P1[4];
        dequant_block<BITS>(wbuf[slot][2 * a], c, s2[2 * a], b2[2 * a], sf[2 * a], bf[2 * a], P0);
        dequant_block<BITS>(wbuf[slot][2 * a + 1], c, s2[2 * a + 1], b2[2 * a + 1], sf[2 * a + 1],
                            bf[2 * a + 1], P1);
#pragma unroll
        for (int b = 0; b < MT; ++b) {
          mma_bf16(acc[a][b], P0[0], P1[0], P0[1], P1[1], xf[b].x, xf[b].y);
          mma_bf16(acc[a][b], P0[2], P1[2], P0[3], P1[3], xf[b].z, xf[b].w);
        }
      }
    }
    if (++pkb == ksteps) {  // row block finished: hand the partial tile to the CTA buffer
      flush(prb);
      pkb = 0;
      ++prb;
    }
  };

  for (int s = s0; s < s1; s += kPipe) {
#pragma unroll
    for (int d = 0; d < kPipe; ++d) {
      if (s + d < s1) {
        process(d);
        if (s + d + kPipe < s1) issue(d);
      }
    }
  }
  if (s0 < s1 && pkb != 0) flush(prb);
  __syncthreads();

  // ---- write out -------------------------------------------------------------------
  if (L <= 0) return;
  const int rb_last = (cta_s1 - 1) / p.ksteps;
  for (int rb = rb_first; rb <= rb_last; ++rb) {
    const float* tb = tilebuf + (size_t)(rb - rb_first) * ROWS * TOKS;
    const long long blk_s0 = (long long)rb * p.ksteps, blk_s1 = blk_s0 + p.ksteps;
    const bool full = cta_s0 <= blk_s0 && blk_s1 <= cta_s1;
    const int n0 = rb * ROWS;
    if (full) {
      for (int i = tid; i < ROWS * TOKS; i += kThreads) {
        const int tk = i / ROWS, r = i % ROWS;
        if (tk < p.M && n0 + r < p.N) {
          const __nv_bfloat16 o = __float2bfloat16_rn(tb[r * TOKS + tk]);
          for (int q = 0; q < p.n_out; ++q) p.y[q][(int64_t)tk * p.ld + p.col0 + n0 + r] = o;
        }
      }
      continue;
    }
    // Shared with neighbouring CTAs: accumulate in global fp32, last arriver converts.
    float* gp = p.partial + (size_t)rb * ROWS * TOKS;
    for (int i = tid; i < ROWS * TOKS; i += kThreads) atomicAdd(&gp[i], tb[i]);
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      // CTAs whose span intersects this row block: owner(first step) .. owner(last step).
      const long long first_owner = ((blk_s0 + 1) * G - 1) / T;
      const long long last_owner = (blk_s1 * G - 1) / T;
      const unsigned expected = (unsigned)(last_owner - first_owner + 1);
      const unsigned old = atomicAdd(&p.counters[rb], 1u);
      s_flag = (old == expected - 1);
      if (s_flag) p.counters[rb] = 0;
    }
    __syncthreads();
    if (s_flag) {
      __threadfence();
      for (int i = tid; i < ROWS * TOKS; i += kThreads) {
        const int tk = i / ROWS, r = i % ROWS;
        const float v = __ldcg(&gp[r * TOKS + tk]);
        __stcg(&gp[r * TOKS + tk], 0.0f);
        if (tk < p.M && n0 + r < p.N) {
          const __nv_bfloat16 o = __float2bfloat16_rn(v);
          for (int q = 0; q < p.n_out; ++q) p.y[q][(int64_t)tk * p.ld + p.col0 + n0 + r] = o;
        }
      }
    }
    __syncthreads();
  }
}

struct QmvPlan {
  int mt, rt, grid;
  size_t smem;
  QmvParams prm;
  bool ok;
};

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

QmvPlan make_plan(const QmmArgs& a) {
  QmvPlan pl{};
  pl.ok = false;
  if (a.dtype != B200Q_BF16 || !a.transpose || a.w_batched || a.batch != 1) return pl;
  if (a.M < 1 || a.M > 16 || a.N < 1 || a.K < 128 || a.K % 128 != 0) return pl;
  if ((int64_t)a.N * a.K >= (1ll << 40)) return pl;  // keeps the step count below 2^31
  pl.mt = a.M > 8 ? 2 : 1;
  pl.rt = (pl.mt == 2 && a.bits <= 4 && a.N >= 4096) ? 2 : 1;
  const int rows = 16 * pl.rt;
  const int ksteps = (int)(a.K / 128);
  const int nrb = (int)((a.N + rows - 1) / rows);
  const long long T = (long long)nrb * ksteps;
  const int sms = sm_count();
  pl.grid = (int)(T < sms ? T : sms);
  const long long per_cta = (T + pl.grid - 1) / pl.grid;
  const int tb_blocks = (int)((per_cta + ksteps - 1) / ksteps + 1);
  pl.smem = (size_t)pl.mt * ksteps * 4 * 32 * 16 + (size_t)tb_blocks * rows * 8 * pl.mt * 4;
  if (pl.smem > 220 * 1024) return pl;
  QmvParams& p = pl.prm;
  p.x = (const __nv_bfloat16*)a.x;
  p.wq = a.wq;
  p.scales = (const __nv_bfloat16*)a.scales;
  p.biases = (const __nv_bfloat16*)a.biases;
  if (a.peers.n > 0) {
    p.n_out = a.peers.n; p.ld = a.peers.ld; p.col0 = a.peers.col0;
    for (int q = 0; q < a.peers.n; ++q) p.y[q] = (__nv_bfloat16*)a.peers.y[q];
  } else {
    p.n_out = 1; p.ld = a.N; p.col0 = 0; p.y[0] = (__nv_bfloat16*)a.y;
  }
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.ksteps = ksteps;
  p.n_row_blocks = nrb;
  p.total_steps = T;
  p.tilebuf_blocks = tb_blocks;
  p.group_shift = a.group == 32 ? 0 : (a.group == 64 ? 1 : 2);
  pl.ok = true;
  return pl;
}

size_t counters_bytes(int64_t N) { return (size_t)(((N + 15) / 16 * 4 + 255) / 256 * 256); }
size_t partial_bytes(int64_t N) { return (size_t)((N + 31) / 32 * 32) * 16 * 4; }

// B200Q_PDL=0 turns programmatic dependent launch off (plain stream order).
bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200Q_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <int BITS>
int launch(const QmvPlan& pl, cudaStream_t st) {
  auto go = [&](auto kern) -> int {
    if (pl.smem > 48 * 1024)
      B200Q_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    if (pdl_enabled()) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(pl.grid);
      cfg.blockDim = dim3(kThreads);
      cfg.dynamicSmemBytes = pl.smem;
      cfg.stream = st;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = at;
      cfg.numAttrs = 1;
      B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, pl.prm));
    } else {
      kern<<<pl.grid, kThreads, pl.smem, st>>>(pl.prm);
    }
    B200Q_LAUNCH_OK("qmv_mma_kernel");
    return B200Q_OK;
  };
  if (pl.mt == 1) return go(qmv_mma_kernel<BITS, 1, 1>);
  if (pl.rt == 1) return go(qmv_mma_kernel<BITS, 2, 1>);
  return go(qmv_mma_kernel<BITS, 2, 2>);
}

}  // namespace

bool qmv_mma_supported(const QmmArgs& a) {
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.wq) & 15)) return false;
  return make_plan(a).ok;
}

size_t qmv_mma_workspace_bytes(const QmmArgs& a) {
  return counters_bytes(a.N) + partial_bytes(a.N) + kStatusBytes;
}

int qmv_mma(const QmmArgs& a, cudaStream_t st) {
  QmvPlan pl = make_plan(a);
  if (!pl.ok) return fail(B200Q_ERR_UNSUPPORTED, "[quantized_matmul] qmv_mma: unsupported problem");
  const size_t need = qmv_mma_workspace_bytes(a);
  if (!a.ws || a.ws_bytes < need)
    return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul] workspace of %zu bytes required, %zu given", need, a.ws_bytes);
  if (reinterpret_cast<uintptr_t>(a.ws) & 15)
    return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul] workspace must be 16-byte aligned");
  pl.prm.counters = reinterpret_cast<uint32_t*>(a.ws);
  pl.prm.partial = reinterpret_cast<float*>(static_cast<char*>(a.ws) + counters_bytes(a.N));
  pl.prm.early = weights_constant() ? 1 : 0;
  int rc = B200Q_ERR_UNSUPPORTED;
  B200Q_DISPATCH_BITS(a.bits, BITS, { rc = launch<BITS>(pl, st); });
  return rc;
}

// ------------------------------------------------------------------------------------
// Decode without any allocation by anyone: the scratch of the kernel above lives in a
// fixed device array that is part of the loaded library image.
//
// Who needs this: code that may not call cudaMalloc at the point where it runs the
// operator - a plugin invoked inside someone else's memory-pool or capture discipline, a
// real-time serving loop that forbids allocator calls after start-up, a host that only
// hands out buffers for inputs and outputs.  Such a caller cannot provide the workspace
// b200q_qmm asks for, so this entry point brings its own.
//
// Cost and limits: every GPU that loads the library holds kStaticScratchBytes (about 2 MiB)
// until the process exits.  The array is sized for N <= B200Q_STATIC_SCRATCH_MAX_N weight
// rows; larger problems are rejected.  All calls on a device share the one array, so two
// calls that can overlap on the GPU (different streams, or graph branches) race on it:
// serialise them.  The array keeps whatever the previous call left; the part a call uses
// is cleared on the stream before the kernel runs.
constexpr size_t kStaticScratchBytes =
    ((B200Q_STATIC_SCRATCH_MAX_N + 15) / 16 * 4 + 255) / 256 * 256 +           // arrival counters
    (size_t)((B200Q_STATIC_SCRATCH_MAX_N + 31) / 32 * 32) * 16 * 4 + 256;      // fp32 partial tiles + status
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
// Device address of g_static_scratch per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel can use: the address has to be asked for,
// once per device, with that device current.
int static_scratch_ptr(void** out) {
  static void* ptrs[64] = {nullptr};
  int dev = 0;
  B200Q_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200Q_ERR_UNSUPPORTED, "[decode_static] device ordinal %d not supported", dev);
  if (!ptrs[dev]) {
    void* p = nullptr;
    B200Q_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return B200Q_OK;
}
}  // namespace

}  // namespace b200q

extern "C" int b200q_qmm_decode_static(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                                       void* y, int dtype, int64_t M, int64_t N, int64_t K, int group_size,
                                       int bits, void* stream) {
  using namespace b200q;
  if (dtype != B200Q_BF16)
    return fail(B200Q_ERR_UNSUPPORTED, "[decode_static] only bfloat16 is supported (dtype code %d)", dtype);
  if (!valid_group(group_size) || !valid_bits(bits))
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[decode_static] unsupported group_size %d / bits %d", group_size, bits);
  if (M < 1 || M > 16 || N < 1 || K < 128 || K % 128 != 0 || K % group_size != 0)
    return fail(B200Q_ERR_UNSUPPORTED,
                "[decode_static] needs 1 <= M <= 16 and K a multiple of 128 (got M=%lld N=%lld K=%lld)",
                (long long)M, (long long)N, (long long)K);
  if (N > B200Q_STATIC_SCRATCH_MAX_N)
    return fail(B200Q_ERR_UNSUPPORTED,
                "[decode_static] N=%lld exceeds the built-in scratch (at most %d weight rows); "
                "use b200q_qmm with a caller workspace", (long long)N, (int)B200Q_STATIC_SCRATCH_MAX_N);
  if (!x || !wq || !scales || !biases || !y) return fail(B200Q_ERR_INVALID_ARGUMENT, "[decode_static] null pointer");
  QmmArgs a{};
  a.x = x; a.wq = wq; a.scales = scales; a.biases = biases; a.y = y;
  a.dtype = dtype; a.batch = 1; a.M = M; a.N = N; a.K = K;
  a.group = group_size; a.bits = bits; a.transpose = true; a.w_batched = false;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15))
    return fail(B200Q_ERR_UNSUPPORTED, "[decode_static] x and wq must be 16-byte aligned");
  if (!qmv_mma_supported(a))
    return fail(B200Q_ERR_UNSUPPORTED,
                "[decode_static] the activations do not fit in shared memory: M=%lld rows of K=%lld need %lld KB "
                "of the 220 KB a thread block may use; use b200q_qmm with a caller workspace",
                (long long)M, (long long)K, (long long)((M > 8 ? 2 : 1) * (K / 128) * 2048 / 1024));
  void* scratch = nullptr;
  if (int rc = static_scratch_ptr(&scratch)) return rc;  // first call on a device: set-up (not capturable)
  const size_t used = qmv_mma_workspace_bytes(a);  // <= kStaticScratchBytes by the N check above
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200Q_CUDA_OK(cudaMemsetAsync(scratch, 0, used, st));  // counters and partial sums must start at zero
  a.ws = scratch;
  a.ws_bytes = used;
  return qmv_mma(a, st);
}
