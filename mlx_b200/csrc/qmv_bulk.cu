// Decode path, 4-bit: y[M<=16, N] = x[M, K] * dequant(W[N, K])^T, bf16, HBM-bound.
//
// Replaces cu::qmv_kernel and the small-M use of cu::qmm_sm80_kernel of the reference
// (mlx/backend/cuda/quantized/qmm/qmv.cu:84-209, quantized/quantized.cpp:106-136).
//
// Why this shape.  HBM only reaches its streaming rate when every weight row is read
// in runs of >= 256 contiguous bytes; the tensor-core fragment layout wants one lane
// to own 4-byte words of eight different rows.  The two are decoupled through shared
// memory: each warp owns a private two-stage ring and fills a stage with sixteen
// asynchronous bulk copies (cp.async.bulk, one per weight row, up to 256 B each)
// that complete on an mbarrier; fragments are then fetched with ldmatrix.
//
//  * One persistent CTA per SM, 16 independent warps.  The (row block, k) space is cut
//    into steps of 16 rows x 128 k; every CTA and every warp owns a contiguous span of
//    steps, so all SMs stream the same number of bytes whatever N is.
//  * Arithmetic is exact up to fp32 summation: the packed fields are turned into the
//    bf16 integers 128+q with shift+lop3 only ("0x4300 | q"), multiplied with x on the
//    tensor cores (mma.sync.m16n8k16, weights = M side, tokens = N side) into a
//    per-group fp32 accumulator, and folded as
//        acc += s * sum_k x_k (128+q_k) + (b - 128 s) * sum_k x_k
//    with the group sums of x precomputed once per CTA.
//  * x is staged once per CTA in shared memory in B-fragment order.  When x does not
//    fit next to the rings, K is split into KSPLIT slices owned by different CTAs.
//  * Per-warp partial tiles are added into a per-CTA shared tile buffer.  Row blocks
//    completed inside one CTA are written directly; the others are combined through
//    fp32 global atomics plus an arrival counter, the last arriver converts and
//    re-zeroes.  No CTA ever waits on another CTA.
//  * Every mbarrier wait is bounded; on expiry the warp records a status code and
//    carries on (the kernel always terminates).
//
// Scratch (caller workspace, zero on first use, self-cleaning): the same layout as
// the register-path kernel: [ counters: ceil(N/16) u32 | fp32 partial tiles ].
#include "common.cuh"
#include "kernels.h"

namespace b200q {
namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 2;        // ring depth per warp
constexpr int kStageSteps = 4;    // steps (of 128 k) per stage: 256 B per row at 4 bits
constexpr uint32_t kSpinLimit = 1u << 20;  // x ~50 ns: tens of milliseconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// Relaxed: nothing this thread wrote has to be visible to the copy engine, and the
// default release form drains the thread's outstanding loads first.
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cta.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false if the limit was hit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if (i > 4) __nanosleep(40);
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
  return d;
}
// d = a * b + c with distinct accumulator input (lets the first MMA of a group read zeros).
__device__ __forceinline__ void mma_bf16(float (&d)[4], const float (&c)[4], uint32_t a0, uint32_t a1,
                                         uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}
__device__ __forceinline__ float bf16_at(uint2 v, int i) {  // element i (0..3) of four packed bf16
  const uint32_t r = (i & 2) ? v.y : v.x;
  return __uint_as_float((i & 1) ? (r & 0xFFFF0000u) : (r << 16));
}

struct BulkParams {
  const __nv_bfloat16* x;
  const uint8_t* wq;  // packed rows, K/2 bytes each
  const __nv_bfloat16* scales;
  const __nv_bfloat16* biases;
  __nv_bfloat16* y;
  uint32_t* counters;
  float* partial;
  uint32_t* status;
  int M, N, K;
  int ksplit;          // K slices
  int kslice_steps;    // steps (128 k) per slice
  int n_row_blocks;    // ceil(N / 16)
  int ctas_per_slice;
  int tilebuf_blocks;
  int aligned;         // CTA spans are whole row blocks
};

// GROUP: quantization group size; MT: token tiles of 8.
template <int GROUP, int MT>
__global__ void __launch_bounds__(kThreads, 1)
qmv_bulk_kernel(const BulkParams p) {
  constexpr int TOKS = 8 * MT;
  constexpr int SB = 64;                         // packed bytes per row per step (128 k at 4 bits)
  constexpr int PITCH = kStageSteps * SB + 16;   // ring row pitch: +16 keeps ldmatrix conflict-free
  constexpr int STAGE_BYTES = 16 * PITCH;
  constexpr int GPS = 128 / GROUP;               // groups per step
  constexpr int CPG = GROUP / 32;                // 32-k cells per group
  constexpr int STG = GROUP == 32 ? 2 : 4;       // steps per ring stage (128 or 256 B per row)
  constexpr int NG = STG * GPS;                  // groups per stage: 8 (g32, g64) or 4 (g128)
  extern __shared__ __align__(128) unsigned char smem_raw[];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#ifdef B200Q_PROFILE
  const long long prof_entry = clock64();
#endif
#ifdef B200Q_PROFILE
  uint32_t prof_marks[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define PROF_MARK(i) prof_marks[i] = (uint32_t)((clock64() - prof_entry) >> 3)
#else
#define PROF_MARK(i)
#endif
  const int g = lane >> 2, t = lane & 3;
  const int kss = p.kslice_steps;
  const int slice = blockIdx.x / p.ctas_per_slice;
  const int cta_in_slice = blockIdx.x - slice * p.ctas_per_slice;
  const long long T = (long long)p.n_row_blocks * kss;  // steps per slice, < 2^31
  const int G = p.ctas_per_slice;
  // aligned: CTA spans start and end on row-block boundaries (no row block is shared
  // between CTAs of a slice); otherwise spans are equal step counts.
  const int cta_s0 = p.aligned ? (int)((long long)cta_in_slice * p.n_row_blocks / G) * kss
                               : (int)((long long)cta_in_slice * T / G);
  const int cta_s1 = p.aligned ? (int)((long long)(cta_in_slice + 1) * p.n_row_blocks / G) * kss
                               : (int)((long long)(cta_in_slice + 1) * T / G);
  const int L = cta_s1 - cta_s0;
  const int s0 = cta_s0 + (int)((long long)warp * L / kWarps);
  const int s1 = cta_s0 + (int)((long long)(warp + 1) * L / kWarps);
  const int rb_first = cta_s0 / kss;
  const int kb_slice0 = slice * kss;          // first absolute k-step of this slice
  const int cells = kss * 4;                  // 32-k cells per slice
  const int slice_groups = kss * GPS;

  // shared memory carve-up
  uint4* xs = reinterpret_cast<uint4*>(smem_raw);                         // [MT][cells][32]
  float* xsum = reinterpret_cast<float*>(xs + (size_t)MT * cells * 32);   // [slice_groups][TOKS]
  float* tilebuf = xsum + (size_t)slice_groups * TOKS;                    // [blocks][16][TOKS]
  unsigned char* ring0 = reinterpret_cast<unsigned char*>(tilebuf + (size_t)p.tilebuf_blocks * 16 * TOKS);
  ring0 = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ring0) + 127) & ~uintptr_t(127));
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring0 + (size_t)kWarps * kStages * STAGE_BYTES);
  __shared__ int s_last[64];

  unsigned char* ring = ring0 + (size_t)warp * kStages * STAGE_BYTES;
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t bar_u32 = smem_u32(bars + warp * kStages);

  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kStages; ++i) mbar_init(bar_u32 + 8 * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  PROF_MARK(7);

  const size_t row_bytes = (size_t)p.K / 2;
  const int row_groups = p.K / GROUP;

  // ---- span walker: the span [s0, s1) is visited in blocks of up to STG steps that never
  // cross an STG-aligned k boundary nor the end of a row block ----------------------------
  struct Walker {
    int s, rb, kbs;  // next step, its row block and k-step inside the slice
  };
  struct Block {
    int rb, kb0, lo, hi;  // row block, first (aligned) k-step, valid steps [lo, hi) of the block
  };
  auto walker_at = [&](int s) {
    Walker w;
    w.s = s;
    w.rb = s / kss;
    w.kbs = s - w.rb * kss;
    return w;
  };
  auto next_block = [&](Walker& w) {
    Block b;
    b.rb = w.rb;
    b.lo = w.kbs & (STG - 1);
    b.kb0 = w.kbs - b.lo;
    int n = STG - b.lo;
    n = n < s1 - w.s ? n : s1 - w.s;
    n = n < kss - w.kbs ? n : kss - w.kbs;
    b.hi = b.lo + n;
    w.s += n;
    w.kbs += n;
    if (w.kbs == kss) {
      w.kbs = 0;
      ++w.rb;
    }
    return b;
  };

  // ---- weight stream: bulk copies, `kStages` blocks ahead ---------------------------
  Walker wi = walker_at(s0);
  auto issue = [&](int slot) {
    if (wi.s >= s1) return;
    const Block b = next_block(wi);
    const uint32_t bytes = (uint32_t)(b.hi - b.lo) * SB;
    const uint32_t bar = bar_u32 + 8 * slot;
    if (lane == 0) mbar_expect_tx(bar, 16 * bytes);
    __syncwarp();
    if (lane < 16) {
      int row = b.rb * 16 + lane;
      row = row < p.N ? row : p.N - 1;  // ragged N: clamp, results are discarded later
      bulk_g2s(ring_u32 + slot * STAGE_BYTES + lane * PITCH + b.lo * SB,
               p.wq + (size_t)row * row_bytes + (size_t)(kb_slice0 + b.kb0 + b.lo) * SB, bytes, bar);
    }
  };
  // ---- stage x (B-fragment order), its group sums, and zero the tile buffer ---------
  // The first batch of x loads is issued before the weight stream is started: behind
  // ~100 KB of queued weight requests per SM those loads would wait several microseconds.
  {
    for (int i = tid; i < slice_groups * TOKS; i += kThreads) xsum[i] = 0.0f;
    const int nbuf = p.tilebuf_blocks * 16 * TOKS;
    for (int i = tid; i < nbuf; i += kThreads) tilebuf[i] = 0.0f;
    constexpr int U = 16;  // loads in flight per thread
    const int items = MT * cells * 32;
    uint4 v[U];
    auto load_batch = [&](int base) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * kThreads;
        v[u] = make_uint4(0, 0, 0, 0);
        if (i < items) {
          const int ln = i & 31, cell = (i >> 5) % cells, mt = (i >> 5) / cells;
          const int tok = mt * 8 + (ln >> 2);
          const int k8 = (kb_slice0 * 4 + cell) * 32 + 8 * (ln & 3);
          if (tok < p.M) v[u] = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)tok * p.K + k8));
        }
      }
    };
    auto store_batch = [&](int base) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * kThreads;
        if (i < items) {
          uint4 o;
          o.x = __byte_perm(v[u].x, v[u].z, 0x5410);  // (x0, x4)
          o.y = __byte_perm(v[u].x, v[u].z, 0x7632);  // (x1, x5)
          o.z = __byte_perm(v[u].y, v[u].w, 0x5410);  // (x2, x6)
          o.w = __byte_perm(v[u].y, v[u].w, 0x7632);  // (x3, x7)
          xs[i] = o;
          const int ln = i & 31, cell = (i >> 5) % cells, mt = (i >> 5) / cells;
          const int tok = mt * 8 + (ln >> 2);
          float sum = 0.0f;
          const uint32_t w4[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q)
            sum += __uint_as_float(w4[q] << 16) + __uint_as_float(w4[q] & 0xFFFF0000u);
          // the four lanes t of a token cover one 32-k cell: combine, then one atomic per cell
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          if ((ln & 3) == 0) atomicAdd(&xsum[(cell / CPG) * TOKS + tok], sum);
        }
      }
    };
    PROF_MARK(0);
    load_batch(tid);
    PROF_MARK(1);
#pragma unroll
    for (int i = 0; i < kStages; ++i) issue(i);
    PROF_MARK(2);
    __syncthreads();  // zero-fill done before the first shared atomics
    PROF_MARK(3);
    store_batch(tid);
    PROF_MARK(4);
    for (int base = tid + kThreads * U; base < items; base += kThreads * U) {
      load_batch(base);
      store_batch(base);
    }
    PROF_MARK(5);
  }
  __syncthreads();
  PROF_MARK(6);

  // ---- main loop -----------------------------------------------------------------------
  float acc[MT][4];
#pragma unroll
  for (int b = 0; b < MT; ++b)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[b][c] = 0.0f;
  const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};

  auto flush = [&](int rb) {
    float* tb = tilebuf + (rb - rb_first) * 16 * TOKS;
#pragma unroll
    for (int b = 0; b < MT; ++b) {
      const int tk = b * 8 + 2 * t;
      atomicAdd(&tb[g * TOKS + tk], acc[b][0]);
      atomicAdd(&tb[g * TOKS + tk + 1], acc[b][1]);
      atomicAdd(&tb[(g + 8) * TOKS + tk], acc[b][2]);
      atomicAdd(&tb[(g + 8) * TOKS + tk + 1], acc[b][3]);
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[b][c] = 0.0f;
    }
  };

  // Scales / biases of one block for rows g and g+8: NG = STG*GPS consecutive bf16 values
  // per row, fetched with one vector load each, one block ahead of their use.
  struct BlockScales {
    uint4 s[2], b[2];
  };
  const __nv_bfloat16* sc_lane = p.scales + (size_t)kb_slice0 * GPS;
  const __nv_bfloat16* bi_lane = p.biases + (size_t)kb_slice0 * GPS;
  auto load_scales = [&](const Block& blk) {
    BlockScales r;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int row = blk.rb * 16 + h * 8 + g;
      row = row < p.N ? row : p.N - 1;
      const size_t gi = (size_t)row * row_groups + blk.kb0 * GPS;
      if constexpr (NG == 8) {
        r.s[h] = __ldg(reinterpret_cast<const uint4*>(sc_lane + gi));
        r.b[h] = __ldg(reinterpret_cast<const uint4*>(bi_lane + gi));
      } else {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(sc_lane + gi));
        const uint2 c = __ldg(reinterpret_cast<const uint2*>(bi_lane + gi));
        r.s[h] = make_uint4(a.x, a.y, 0, 0);
        r.b[h] = make_uint4(c.x, c.y, 0, 0);
      }
    }
    return r;
  };
  auto bf16_of = [](const uint4& v, int e) {  // element e (compile-time) of eight packed bf16
    const uint32_t r = (e >> 1) == 0 ? v.x : ((e >> 1) == 1 ? v.y : ((e >> 1) == 2 ? v.z : v.w));
    return __uint_as_float((e & 1) ? (r & 0xFFFF0000u) : (r << 16));
  };

  bool timed_out = false;
#ifdef B200Q_PROFILE
  long long prof_wait = 0;
  const long long prof_t0 = clock64();
  if (tid == 0 && blockIdx.x == 0) {
    p.status[0] = (prof_marks[0] & 0xFFFF) | (prof_marks[1] << 16);
    p.status[2] = (prof_marks[2] & 0xFFFF) | (prof_marks[3] << 16);
    p.status[3] = (prof_marks[4] & 0xFFFF) | (prof_marks[5] << 16);
    p.status[1] = (prof_marks[6] & 0xFFFF) | (prof_marks[7] << 16);
  }
#endif
  Walker wp = walker_at(s0);   // processing cursor
  Walker wsc = walker_at(s0);  // scale-prefetch cursor, one block ahead
  BlockScales nxt;
  if (wsc.s < s1) {
    const Block b0 = next_block(wsc);
    nxt = load_scales(b0);
  }
  uint32_t it = 0;
  const uint32_t lm_lane = (lane & 7) * PITCH + (lane >> 3) * 16;
  while (wp.s < s1) {
#pragma unroll
    for (int slot = 0; slot < kStages; ++slot) {
      if (wp.s < s1) {
        const Block blk = next_block(wp);
        const BlockScales cur = nxt;
        if (wsc.s < s1) {
          const Block bn = next_block(wsc);
          nxt = load_scales(bn);
        }
#ifdef B200Q_PROFILE
        const long long tw0 = clock64();
#endif
        if (!mbar_wait(bar_u32 + 8 * slot, (it / kStages) & 1)) timed_out = true;
#ifdef B200Q_PROFILE
        prof_wait += clock64() - tw0;
#endif
        // ldmatrix row addresses: lanes 0-7 -> cell 0, 8-15 -> cell 1, ... of rows (lane & 7)
        const uint32_t lm = ring_u32 + slot * STAGE_BYTES + lm_lane;
        const uint4* xb = xs + (blk.kb0 * 4) * 32 + lane;
        const float* xsb = xsum + (blk.kb0 * GPS) * TOKS + 2 * t;
#pragma unroll
        for (int j = 0; j < STG; ++j) {
          if (j >= blk.lo && j < blk.hi) {
            uint32_t wlo[4], whi[4];
            ldmatrix_x4(wlo, lm + j * SB);
            ldmatrix_x4(whi, lm + j * SB + 8 * PITCH);
            float tmp[MT][4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 xf[MT];
#pragma unroll
              for (int b = 0; b < MT; ++b) xf[b] = xb[(b * cells + j * 4 + c) * 32];
              uint32_t P[4], Q[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                P[i] = lop3_and_or(wlo[c] >> (4 * i), 0x000F000Fu, 0x43004300u);
                Q[i] = lop3_and_or(whi[c] >> (4 * i), 0x000F000Fu, 0x43004300u);
              }
#pragma unroll
              for (int b = 0; b < MT; ++b) {
                if (c % CPG == 0) mma_bf16(tmp[b], zero4, P[0], Q[0], P[1], Q[1], xf[b].x, xf[b].y);
                else mma_bf16(tmp[b], tmp[b], P[0], Q[0], P[1], Q[1], xf[b].x, xf[b].y);
                mma_bf16(tmp[b], tmp[b], P[2], Q[2], P[3], Q[3], xf[b].z, xf[b].w);
              }
              if (c % CPG == CPG - 1) {
                const int e = j * GPS + c / CPG;  // group within the block (compile-time)
                const float s_lo = bf16_of(cur.s[0], e), s_hi = bf16_of(cur.s[1], e);
                const float c_lo = fmaf(-128.0f, s_lo, bf16_of(cur.b[0], e));
                const float c_hi = fmaf(-128.0f, s_hi, bf16_of(cur.b[1], e));
#pragma unroll
                for (int b = 0; b < MT; ++b) {
                  const float2 xv = *reinterpret_cast<const float2*>(xsb + e * TOKS + b * 8);
                  acc[b][0] = fmaf(s_lo, tmp[b][0], fmaf(c_lo, xv.x, acc[b][0]));
                  acc[b][1] = fmaf(s_lo, tmp[b][1], fmaf(c_lo, xv.y, acc[b][1]));
                  acc[b][2] = fmaf(s_hi, tmp[b][2], fmaf(c_hi, xv.x, acc[b][2]));
                  acc[b][3] = fmaf(s_hi, tmp[b][3], fmaf(c_hi, xv.y, acc[b][3]));
                }
              }
            }
          }
        }
        if (blk.kb0 + blk.hi == kss) flush(blk.rb);  // row block finished inside this slice
        __syncwarp();
        issue(slot);  // refill the stage just consumed
        ++it;
      }
    }
  }
  if (s0 < s1 && (s1 % kss) != 0) flush((s1 - 1) / kss);
#ifdef B200Q_PROFILE
  (void)prof_wait; (void)prof_t0;
#endif
  if (timed_out && lane == 0) atomicMax(&p.status[0], 2u);
  __syncthreads();

  // ---- write out -------------------------------------------------------------------
  if (L <= 0) return;
  const int rb_last = (cta_s1 - 1) / kss;
  const int nblk = rb_last - rb_first + 1;
  bool any_shared = false;
  for (int bi = 0; bi < nblk; ++bi) {
    const int rb = rb_first + bi;
    const float* tb = tilebuf + (size_t)bi * 16 * TOKS;
    const long long blk_s0 = (long long)rb * kss, blk_s1 = blk_s0 + kss;
    const bool full = p.ksplit == 1 && cta_s0 <= blk_s0 && blk_s1 <= cta_s1;
    const int n0 = rb * 16;
    if (full) {
      for (int i = tid; i < 16 * TOKS; i += kThreads) {
        const int tk = i / 16, r = i % 16;
        if (tk < p.M && n0 + r < p.N) p.y[(size_t)tk * p.N + n0 + r] = __float2bfloat16_rn(tb[r * TOKS + tk]);
      }
    } else {
      any_shared = true;
      float* gp = p.partial + (size_t)rb * 16 * 16;
      for (int i = tid; i < 16 * TOKS; i += kThreads) atomicAdd(&gp[i], tb[i]);
    }
  }
  if (!any_shared) return;  // uniform across the CTA
  __threadfence();
  __syncthreads();
  for (int bi = tid; bi < nblk; bi += kThreads) {
    const int rb = rb_first + bi;
    const long long blk_s0 = (long long)rb * kss, blk_s1 = blk_s0 + kss;
    const bool full = p.ksplit == 1 && cta_s0 <= blk_s0 && blk_s1 <= cta_s1;
    int last = 0;
    if (!full) {
      // contributors: in every slice, the CTAs from owner(first step) to owner(last step)
      const long long first_owner = ((blk_s0 + 1) * G - 1) / T;
      const long long last_owner = (blk_s1 * G - 1) / T;
      const unsigned expected =
          p.aligned ? (unsigned)p.ksplit : (unsigned)(last_owner - first_owner + 1) * (unsigned)p.ksplit;
      const unsigned old = atomicAdd(&p.counters[rb], 1u);
      last = (old == expected - 1);
      if (last) p.counters[rb] = 0;
    }
    if (bi < 64) s_last[bi] = last;
  }
  __syncthreads();
  for (int bi = 0; bi < nblk && bi < 64; ++bi) {
    if (!s_last[bi]) continue;
    __threadfence();
    const int rb = rb_first + bi, n0 = rb * 16;
    float* gp = p.partial + (size_t)rb * 16 * 16;
    for (int i = tid; i < 16 * TOKS; i += kThreads) {
      const int tk = i / 16, r = i % 16;
      const float v = __ldcg(&gp[r * TOKS + tk]);
      __stcg(&gp[r * TOKS + tk], 0.0f);
      if (tk < p.M && n0 + r < p.N) p.y[(size_t)tk * p.N + n0 + r] = __float2bfloat16_rn(v);
    }
  }
#ifdef B200Q_PROFILE

#endif
}

struct BulkPlan {
  bool ok;
  int mt, grid;
  size_t smem;
  BulkParams prm;
};

int sm_count_cached() {
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

BulkPlan make_plan(const QmmArgs& a) {
  BulkPlan pl{};
  pl.ok = false;
  if (a.dtype != B200Q_BF16 || !a.transpose || a.w_batched || a.batch != 1 || a.bits != 4) return pl;
  if (a.M < 1 || a.M > 16 || a.N < 1 || a.K < 512 || a.K % 512 != 0) return pl;
  if ((int64_t)a.N * a.K >= (1ll << 40)) return pl;  // keeps the step count below 2^31
  pl.mt = a.M > 8 ? 2 : 1;
  const int toks = 8 * pl.mt;
  const int sms = sm_count_cached();
  const int nrb = (int)((a.N + 15) / 16);
  const size_t ring_bytes = (size_t)kWarps * kStages * 16 * (kStageSteps * 64 + 16) + kWarps * kStages * 8 + 256;
  const size_t limit = 227 * 1024 - 1024;
  for (int ks = 1; ks <= 8; ks *= 2) {
    if ((a.K / 512) % ks != 0 || sms % ks != 0) continue;  // slices start on 512-k boundaries
    const int kss = (int)(a.K / 128 / ks);
    const long long T = (long long)nrb * kss;
    int cps = sms / ks;
    if (T < cps) cps = (int)T;
    if (cps < 1) continue;
    // Whole row blocks per CTA unless that costs more than 20% in balance: a row block
    // shared by two CTAs goes through the global atomics path and its round trips.
    const int rb_max = (nrb + cps - 1) / cps;
    const bool aligned = nrb >= cps && (double)rb_max * cps <= 1.2 * nrb;
    const long long per_cta = (T + cps - 1) / cps;
    const int tb_blocks = aligned ? rb_max : (int)((per_cta + kss - 1) / kss + 1);
    if (tb_blocks > 64) continue;  // s_last[] in the kernel
    const size_t smem = (size_t)pl.mt * kss * 4 * 32 * 16 + (size_t)kss * (128 / a.group) * toks * 4 +
                        (size_t)tb_blocks * 16 * toks * 4 + ring_bytes;
    if (smem > limit) continue;
    BulkParams& p = pl.prm;
    p.x = (const __nv_bfloat16*)a.x;
    p.wq = (const uint8_t*)a.wq;
    p.scales = (const __nv_bfloat16*)a.scales;
    p.biases = (const __nv_bfloat16*)a.biases;
    p.y = (__nv_bfloat16*)a.y;
    p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
    p.ksplit = ks;
    p.kslice_steps = kss;
    p.n_row_blocks = nrb;
    p.ctas_per_slice = cps;
    p.tilebuf_blocks = tb_blocks;
    p.aligned = aligned ? 1 : 0;
    pl.grid = cps * ks;
    pl.smem = smem;
    pl.ok = true;
    return pl;
  }
  return pl;
}

size_t counters_bytes(int64_t N) { return (size_t)(((N + 15) / 16 * 4 + 255) / 256 * 256); }
size_t partial_bytes(int64_t N) { return (size_t)((N + 31) / 32 * 32) * 16 * 4; }

template <int GROUP>
int launch(const BulkPlan& pl, cudaStream_t st) {
  auto go = [&](auto kern) -> int {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    kern<<<pl.grid, kThreads, pl.smem, st>>>(pl.prm);
    B200Q_LAUNCH_OK("qmv_bulk_kernel");
    return B200Q_OK;
  };
  if (pl.mt == 1) return go(qmv_bulk_kernel<GROUP, 1>);
  return go(qmv_bulk_kernel<GROUP, 2>);
}

}  // namespace

bool qmv_bulk_supported(const QmmArgs& a) {
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.wq) & 15)) return false;
  if ((reinterpret_cast<uintptr_t>(a.scales) & 7) || (reinterpret_cast<uintptr_t>(a.biases) & 7)) return false;
  return make_plan(a).ok;
}

size_t qmv_bulk_workspace_bytes(const QmmArgs& a) {
  return counters_bytes(a.N) + partial_bytes(a.N) + kStatusBytes;
}

int qmv_bulk(const QmmArgs& a, cudaStream_t st) {
  BulkPlan pl = make_plan(a);
  if (!pl.ok) return fail(B200Q_ERR_UNSUPPORTED, "[quantized_matmul] qmv_bulk: unsupported problem");
  const size_t need = qmv_bulk_workspace_bytes(a);
  if (!a.ws || a.ws_bytes < need)
    return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul] workspace of %zu bytes required, %zu given", need, a.ws_bytes);
  if (reinterpret_cast<uintptr_t>(a.ws) & 15)
    return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul] workspace must be 16-byte aligned");
  pl.prm.counters = reinterpret_cast<uint32_t*>(a.ws);
  pl.prm.partial = reinterpret_cast<float*>(static_cast<char*>(a.ws) + counters_bytes(a.N));
  pl.prm.status = reinterpret_cast<uint32_t*>(static_cast<char*>(a.ws) + a.ws_bytes - kStatusBytes);
  if (a.group == 32) return launch<32>(pl, st);
  if (a.group == 64) return launch<64>(pl, st);
  return launch<128>(pl, st);
}

}  // namespace b200q
