// Prefill path: y[M, N] = x[M, K] * dequant(W[N, K])^T on the 5th-generation tensor cores.
//
// Replaces cu::qmm_sm80_kernel / qmm_naive_kernel of the reference
// (mlx/backend/cuda/device/qmm_sm80.cuh:70-356, quantized/qmm/qmm.cu:20-185), which run
// Ampere-style mma.sync code on this GPU.
//
// Formulation (swap-AB): the MMA computes D[128 weight rows, NT tokens] so that the
// operand that has to be dequantised (W) is the 128-row A operand and is re-used by up
// to 256 tokens per instruction, and the operand that streams unchanged (x) is B.
//
//   thread A: TMA  --packed W tile [128 rows x 128 k, 16*bits bytes per row]-->  smem ring P
//   16 dequant warps (4 TMEM lane quadrants x 4 quarters of the 128-k stage): one thread per
//        weight row (= one TMEM lane) unpacks 32 k, applies s*q+b in bf16x2 (4- and 8-bit:
//        mask + one fma on the field read as a subnormal bf16; other widths shift/lop3/prmt),
//        tcgen05.st into the A ring in TMEM; scales and biases come as 16-byte chunks per row
//   thread B: TMA  --two x sub-tiles [NT tokens x 64 k], 128B-swizzled K-major-->  smem ring B
//   1 thread: tcgen05.mma.kind::f16 (A from TMEM, B from smem descriptors), fp32
//        accumulator [128 lanes x NT columns] in TMEM, tcgen05.commit on mbarriers
//   8 epilogue warps (two per TMEM lane quadrant, half of the token columns each):
//        tcgen05.ld the accumulator, round to bf16, store y (transposed; scattered through
//        a row table in grouped mode)
//
// The two TMA streams have a thread each: behind the x-tile waits the packed tiles would
// arrive late and starve the dequant warps.
//
// Grouped mode (gather_qmm): a device-side table lists (expert, first row, valid rows) for
// every NT-row slice of the expert-sorted activations; the weight tensor map spans the
// stacked experts [E*N, K*bits/8].
//
// TMEM columns (512 allocated): [0, 256) accumulator, [256, 512) A ring of 4 stages
// (128 k of bf16 = 64 columns each).  One CTA per SM (persistent), tiles are taken
// round-robin; no CTA ever waits on another CTA.
//
// A pipeline stage is 128 k: the MMA-issuing thread is blocked while the tensor pipe is busy
// (the queue behind tcgen05.mma is about one instruction deep; an M=128, K=16 instruction
// takes 128 cycles at N=256 and no less than about 100 at any smaller N) and pays about 65
// cycles for every tcgen05.commit, so every wait and commit per stage is time the tensor pipe
// idles: eight MMAs per pair of commits instead of four.
//
// Every mbarrier wait is bounded.  When a wait expires the role sets the CTA abort
// flag and the device status word, all roles leave their loops, TMEM is released and
// the kernel ends normally (its results are then invalid and the host reports it).
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace b200q {
namespace {

constexpr int kTileN = 128;       // weight rows per tile (MMA M)
constexpr int kBlockK = 64;       // k per x sub-tile (one 128-byte swizzle row of bf16)
constexpr int kStageK = 128;      // k per pipeline stage: two x sub-tiles, one packed tile, 8 MMAs
constexpr int kStagesA = 4;       // A ring in TMEM (64 columns each)
constexpr int kMaxStagesB = 6;    // x stages in shared memory: as many as fit (3 at 256 tokens)
constexpr int kMaxStagesP = 4;    // packed W tiles in shared memory
// Packed stages: 16 * bits bytes per row and stage; next to three 64 KB x stages 35 KB remain.
__host__ __device__ constexpr int stages_p(int bits) { return bits <= 4 ? 4 : (bits == 5 ? 3 : 2); }
constexpr size_t kSmemMax = 227 * 1024;
constexpr int kDoneRing = 12;
constexpr int kAccCols = 256;
constexpr int kTmemCols = 512;
constexpr int kDequantWarps = 16;   // two sets of 8: 4 TMEM lane quadrants x 2 halves (64 k) of a stage
constexpr int kDequantSet = 8;      // set 0 unpacks the even stages of a tile, set 1 the odd ones
constexpr int kEpilogueWarps = 8;   // two per TMEM lane quadrant, each drains half of the columns
constexpr int kProducerPWarp = 2 + kDequantWarps + kEpilogueWarps;  // last warp
constexpr int kThreads = 32 * (3 + kDequantWarps + kEpilogueWarps);  // 864

using namespace tc;

// Waits of the three single-thread roles.
#ifndef B200Q_TC_PARK
#define TC_WAIT1 mbar_wait_spin
#else
#define TC_WAIT1 mbar_wait
#endif
// Waits of the dequant warps.
#ifdef B200Q_TC_DQ_SPIN
#define TC_WAIT16 mbar_wait_spin
#else
#define TC_WAIT16 mbar_wait
#endif

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled operand tile whose
// rows are 128 bytes (64 bf16): 8-row groups are 1024 bytes apart (SBO), descriptor
// version 1 (sm_100), layout type 2 = SWIZZLE_128B.  `addr` may point 32*j bytes into
// the first row to select the j-th 16-element K slice.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);        // start address  [0,14)
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset [32,46)
  d |= (uint64_t)1 << 46;                        // descriptor version
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D f32, A/B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
}

// One entry per group of NT consecutive rows of the (expert-sorted) activation matrix.
struct MTile {
  int expert;     // weight matrix the rows multiply
  int row0;       // first row in the activation matrix
  int rows;       // valid rows (<= NT): the rest of the TMA box belongs to another expert
  int pad;
};

struct TcParams {
  // grouped (gather_qmm) mode: device-side tile table, else nullptr
  const MTile* mtiles;
  const int* n_mtiles;      // device scalar: entries of `mtiles`
  const int* dst_row;       // output row of every activation row
  const __nv_bfloat16* scales;
  const __nv_bfloat16* biases;
  __nv_bfloat16* y;
  // plain mode: output buffers (one, or one per GPU of an N-sharded layer), row pitch and first column
  __nv_bfloat16* y_out[kMaxPeers];
  int n_out;
  long long ld, col0;
  PeerSignal sig;    // completion signal towards the ranks that receive y (n == 0: none)
  uint32_t* status;
  int M, N, K;
  int NT;            // tokens per tile (multiple of 16, <= 256)
  int nsb;           // x stages in shared memory (2 .. kMaxStagesB)
  int n_tiles, m_tiles;
  int group_shift;   // log2(group / 32)
};

struct __align__(8) Barriers {
  uint64_t full_p[kMaxStagesP], empty_p[kMaxStagesP];
  uint64_t full_b[kMaxStagesB];
  uint64_t full_a[kStagesA];
  // One commit per stage: stage `it` (counted across tiles) arrives on done[it % kDoneRing] when its
  // MMAs have completed.  The A slot it % 4 and the x slot it % nsb are free again from then on: the
  // unpack warps and the x producer look at the entry of the stage that used their slot last.  The
  // ring length is a common multiple of both slot counts (nsb is 2, 3, 4 or 6).
  uint64_t done[kDoneRing];
  uint64_t acc_full, acc_empty;
  uint32_t tmem_base;
  int abort_flag;
};

// Unpacks 32 consecutive BITS-wide fields (BITS words, LSB-first bit stream) of one row into
// 16 bf16x2 registers in natural k order, applying w = s*q + b (one rounding).  s and b are
// the raw bf16 bit patterns.
template <int BITS>
__device__ __forceinline__ void dequant32(const uint32_t (&w)[BITS], uint32_t s_bits, uint32_t b_bits,
                                          uint32_t (&out)[16]) {
  constexpr uint32_t kMagic = 0x43004300u;  // (128.0, 128.0): 0x4300 | q == 128 + q for q < 128
  const uint32_t s2 = s_bits * 0x00010001u, b2 = b_bits * 0x00010001u;
  // Fast form for 4- and 8-bit fields: the masked field, read as bf16, is the subnormal (or
  // smallest normal) number q * 2^-133 (16 q * 2^-133 for a field at bits 4..7: bit 7 is the
  // exponent's lowest bit and continues the subnormal scale exactly).  fma.rn.bf16x2 takes
  // subnormal inputs exactly, so one fma with the scale times 2^133 (2^129) gives
  // round(q * s + b): no shift for half of the fields, no subtraction.  It needs the scaled scale
  // to stay finite and normal: biased exponent of s in [1, 121]; other scales (zero, subnormal,
  // |s| >= 2^-6 * 2, inf, nan) take the general form below.
  const uint32_t s_exp = (s_bits >> 7) & 0xFFu;
  const bool fast = s_exp >= 1u && s_exp <= 121u;
  if constexpr (BITS == 4) {
    if (fast) {
      const uint32_t sl = (s_bits + (133u << 7)) * 0x00010001u, sh = (s_bits + (129u << 7)) * 0x00010001u;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t u = w[j] >> 8;
        uint32_t p[4];   // p[i] = (w[i], w[i+4]) as bf16 pairs
        p[0] = fma_bf16x2(w[j] & 0x000F000Fu, sl, b2);
        p[1] = fma_bf16x2(w[j] & 0x00F000F0u, sh, b2);
        p[2] = fma_bf16x2(u & 0x000F000Fu, sl, b2);
        p[3] = fma_bf16x2(u & 0x00F000F0u, sh, b2);
        out[4 * j + 0] = __byte_perm(p[0], p[1], 0x5410);
        out[4 * j + 1] = __byte_perm(p[2], p[3], 0x5410);
        out[4 * j + 2] = __byte_perm(p[0], p[1], 0x7632);
        out[4 * j + 3] = __byte_perm(p[2], p[3], 0x7632);
      }
      return;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t p[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // p[i] = (q[i], q[i+4]) as bf16 pairs
        const uint32_t t = lop3_and_or(w[j] >> (4 * i), 0x000F000Fu, kMagic);
        p[i] = fma_bf16x2(sub_bf16x2(t, kMagic), s2, b2);
      }
      out[4 * j + 0] = __byte_perm(p[0], p[1], 0x5410);  // (w0, w1)
      out[4 * j + 1] = __byte_perm(p[2], p[3], 0x5410);  // (w2, w3)
      out[4 * j + 2] = __byte_perm(p[0], p[1], 0x7632);  // (w4, w5)
      out[4 * j + 3] = __byte_perm(p[2], p[3], 0x7632);  // (w6, w7)
    }
  } else if constexpr (BITS == 8) {
    if (fast) {
      const uint32_t sl = (s_bits + (133u << 7)) * 0x00010001u;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t r0 = fma_bf16x2(w[j] & 0x00FF00FFu, sl, b2);          // (w0, w2)
        const uint32_t r1 = fma_bf16x2((w[j] >> 8) & 0x00FF00FFu, sl, b2);   // (w1, w3)
        out[2 * j + 0] = __byte_perm(r0, r1, 0x5410);
        out[2 * j + 1] = __byte_perm(r0, r1, 0x7632);
      }
      return;
    }
    // 8-bit values exceed the bf16 integer trick: go through float (0x4B0000qq == 2^23 + q)
    const float sf = __uint_as_float(s_bits << 16), bf = __uint_as_float(b_bits << 16);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t word = w[j >> 1];
      const int b0 = (j & 1) * 2;
      const float q0 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540 | b0)) - 8388608.0f;
      const float q1 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540 | (b0 + 1))) - 8388608.0f;
      uint32_t d;
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(fmaf(q1, sf, bf)), "f"(fmaf(q0, sf, bf)));
      out[j] = d;
    }
  } else {
    constexpr uint32_t mask = (1u << BITS) - 1u;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      uint32_t f[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int e = 2 * j + h, wi = (e * BITS) >> 5, sh = (e * BITS) & 31;
        f[h] = (sh + BITS > 32) ? __funnelshift_r(w[wi], w[(wi + 1) % BITS], sh) : (w[wi] >> sh);
      }
      const uint32_t lo = lop3_and_or(f[0], mask, 0x4300u), hi = lop3_and_or(f[1], mask, 0x4300u);
      const uint32_t t = __byte_perm(lo, hi, 0x5410);
      out[j] = fma_bf16x2(sub_bf16x2(t, kMagic), s2, b2);
    }
  }
}

struct TileCoord {
  int w_row0;   // first row of the tile in the stacked weight tensor [E*N, ...]
  int w_rows_end;  // one past the last valid stacked row of this expert
  int n0;       // first output column
  int x_row0;   // first activation row
  int rows;     // valid activation rows
};
__device__ __forceinline__ TileCoord tile_coord(const TcParams& p, int tile) {
  TileCoord t;
  if (p.mtiles == nullptr) {
    const int tm = tile % p.m_tiles, tn = tile / p.m_tiles;
    t.w_row0 = tn * kTileN;
    t.w_rows_end = p.N;
    t.n0 = tn * kTileN;
    t.x_row0 = tm * p.NT;
    t.rows = p.M - t.x_row0 < p.NT ? p.M - t.x_row0 : p.NT;
  } else {
    const int g = tile / p.n_tiles, tn = tile - g * p.n_tiles;
    const MTile mt = p.mtiles[g];
    t.w_row0 = mt.expert * p.N + tn * kTileN;
    t.w_rows_end = mt.expert * p.N + p.N;
    t.n0 = tn * kTileN;
    t.x_row0 = mt.row0;
    t.rows = mt.rows;
  }
  return t;
}

#ifdef B200Q_PROFILE
__device__ uint32_t g_tc_prof[64];
#endif

template <int BITS>
__global__ void __launch_bounds__(kThreads, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
              const TcParams p) {
  // A packed stage holds 128 k of every row (16*BITS bytes, a multiple of 16 for every width).
  constexpr int kPRowBytes = 16 * BITS;
  constexpr int kStagesP = stages_p(BITS);
  constexpr int kPStageBytes = kTileN * kPRowBytes;
  const int kStagesB = p.nsb;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // carve-up: [B ring: nsb stages of two NT*128-byte sub-tiles (1024-aligned)] [P ring] [barriers]
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t b_sub_bytes = (uint32_t)p.NT * 128u;     // NT is a multiple of 16: a multiple of 2048
  const uint32_t b_stage_bytes = 2u * b_sub_bytes;
  const uint32_t b_stage_pitch = b_stage_bytes;
  unsigned char* ring_b = smem;
  unsigned char* ring_p = ring_b + (size_t)kStagesB * b_stage_pitch;
  Barriers* bars = reinterpret_cast<Barriers*>(ring_p + (size_t)kStagesP * kPStageBytes);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef B200Q_PROFILE
  // Tuning builds (plain mode only): thread block 0 leaves per-role wait cycles / 16 in a buffer of
  // its own (g_tc_prof), which a test harness reads back with cudaMemcpyFromSymbol.
  uint32_t* dbg = g_tc_prof;
  long long pw0 = 0, pw1 = 0, pw2 = 0, pw3 = 0, pw4 = 0, pt = 0;
  const long long prof_entry = clock64();
#define TC_T0() pt = clock64()
#define TC_ACC(v) v += clock64() - pt
#define TC_OUT(slot, v) if (blockIdx.x == 0 && lane == 0 && p.mtiles == nullptr) dbg[slot] = (uint32_t)((v) >> 4)
#else
#define TC_T0()
#define TC_ACC(v)
#define TC_OUT(slot, v)
#endif
  const int kstages = p.K / kStageK;
  const int total_tiles = p.mtiles ? *p.n_mtiles * p.n_tiles : p.n_tiles * p.m_tiles;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStagesP; ++i) { mbar_init(smem_u32(&bars->full_p[i]), 1); mbar_init(smem_u32(&bars->empty_p[i]), kDequantSet); }
    for (int i = 0; i < kStagesB; ++i) mbar_init(smem_u32(&bars->full_b[i]), 1);
    for (int i = 0; i < kStagesA; ++i) mbar_init(smem_u32(&bars->full_a[i]), kDequantSet);
    for (int i = 0; i < kDoneRing; ++i) mbar_init(smem_u32(&bars->done[i]), 1);
    mbar_init(smem_u32(&bars->acc_full), 1);
    mbar_init(smem_u32(&bars->acc_empty), kEpilogueWarps);
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tcgen05_alloc(smem_u32(&bars->tmem_base), kTmemCols);
    tcgen05_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_acc = tmem_base;
  const uint32_t tmem_a = tmem_base + kAccCols;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: x tiles (B ring)
    if (lane == 0) {
      uint32_t sb = 0, it = 0;  // slot and stage counter, running across tiles
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        const TileCoord tc_ = tile_coord(p, tile);
        bool ok = true;
        for (int ks = 0; ks < kstages; ++ks) {
          TC_T0();
          if (it >= (uint32_t)kStagesB) {   // the stage that used this slot last has been multiplied
            const uint32_t prev = it - (uint32_t)kStagesB;
            if (!TC_WAIT1(smem_u32(&bars->done[prev % kDoneRing]), (prev / kDoneRing) & 1u, abort_flag)) { ok = false; break; }
          }
          TC_ACC(pw1);
          const uint32_t bar = smem_u32(&bars->full_b[sb]);
          const uint32_t dst = smem_u32(ring_b + sb * b_stage_pitch);
          mbar_expect_tx(bar, b_stage_bytes);
          tma_load_2d(dst, &map_x, ks * kStageK, tc_.x_row0, bar);
          tma_load_2d(dst + b_sub_bytes, &map_x, ks * kStageK + kBlockK, tc_.x_row0, bar);
          ++it;
          if (++sb == (uint32_t)kStagesB) sb = 0;
        }
        if (!ok) break;
      }
      TC_OUT(1, pw1); TC_OUT(2, clock64() - prof_entry);
    }
  } else if (warp == kProducerPWarp) {
    // ------------------------------------------------------------ TMA producer: packed W tiles (P ring).
    // A separate thread: behind the x-tile waits of the other producer the packed tiles would
    // arrive late and starve the dequant warps.
    if (lane == 0) {
      uint32_t sp = 0, pp = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        const TileCoord tc_ = tile_coord(p, tile);
        bool ok = true;
        for (int ks = 0; ks < kstages; ++ks) {
          TC_T0();
          if (!TC_WAIT1(smem_u32(&bars->empty_p[sp]), pp ^ 1, abort_flag)) { ok = false; break; }
          TC_ACC(pw0);
          mbar_expect_tx(smem_u32(&bars->full_p[sp]), kPStageBytes);
          tma_load_2d(smem_u32(ring_p + sp * kPStageBytes), &map_w, ks * kPRowBytes, tc_.w_row0,
                      smem_u32(&bars->full_p[sp]));
          if (++sp == (uint32_t)kStagesP) { sp = 0; pp ^= 1; }
        }
        if (!ok) break;
      }
      TC_OUT(0, pw0);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(p.NT);
      uint32_t tcount = 0, sa = 0, pa = 0, sb = 0, pb = 0, itm = 0;
      // The commit of a stage is issued after the FIRST MMA of the next one: its 65 cycles then pass
      // while the tensor pipe works, not between two stages.  (The barrier then also covers that one
      // MMA: the stage is released 128 cycles later.)
      bool commit_due = false;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
        TC_T0();
        if (!TC_WAIT1(smem_u32(&bars->acc_empty), (tcount & 1) ^ 1, abort_flag)) break;
        TC_ACC(pw2);
        tcgen05_fence_after();
        bool ok = true;
        for (int ks = 0; ks < kstages; ++ks) {
          TC_T0();
          if (!TC_WAIT1(smem_u32(&bars->full_a[sa]), pa, abort_flag)) { ok = false; break; }
          TC_ACC(pw0);
          TC_T0();
          if (!TC_WAIT1(smem_u32(&bars->full_b[sb]), pb, abort_flag)) { ok = false; break; }
          TC_ACC(pw1);
          tcgen05_fence_after();
          const uint32_t b_addr = smem_u32(ring_b + sb * b_stage_pitch);
          TC_T0();
#pragma unroll
          for (int kk = 0; kk < kStageK / 16; ++kk) {
            tcgen05_mma_ts(tmem_acc, tmem_a + sa * 64 + kk * 8,
                           make_sw128_desc(b_addr + (kk >> 2) * b_sub_bytes + (kk & 3) * 32), idesc,
                           (ks | kk) != 0 ? 1u : 0u);
            if (kk == 0 && commit_due) {
              // one commit per stage: a stage is 128 k (eight MMAs) deep and both rings are released
              // through the same barrier
              tcgen05_commit(smem_u32(&bars->done[(itm - 1) % kDoneRing]));
              commit_due = false;
            }
          }
          TC_ACC(pw3);
          commit_due = true;
          ++itm;
          if (++sa == (uint32_t)kStagesA) { sa = 0; pa ^= 1; }
          if (++sb == (uint32_t)kStagesB) { sb = 0; pb ^= 1; }
        }
        if (!ok) break;
        if (commit_due) {
          tcgen05_commit(smem_u32(&bars->done[(itm - 1) % kDoneRing]));
          commit_due = false;
        }
        tcgen05_commit(smem_u32(&bars->acc_full));
      }
      TC_OUT(4, pw0); TC_OUT(5, pw1); TC_OUT(6, pw2); TC_OUT(7, clock64() - prof_entry); TC_OUT(14, pw3); TC_OUT(15, pw4);
    }
  } else if (warp < 2 + kDequantWarps) {
    // ------------------------------------------------------------ dequant: one thread per weight row
    // A warp's trip through one stage (wait for the packed tile, unpack, publish, wait for a free
    // A stage, store) is a chain of dependent latencies of about the length of a stage's MMAs; with
    // every warp on every stage that chain bounded the kernel.  So the warps form two sets that
    // take alternate stages, 64 k per thread and stage: each set has two stage times per trip.
    const int dq = warp - 2;
    const int dset = dq >> 3;            // stages ks = dset (mod 2) of every tile are this warp's
    const int quad = warp & 3;           // TMEM lane quadrant this warp may access
    const int half = (dq >> 2) & 1;      // which 64-k half of the 128-k stage
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
    const int row_groups = p.K >> (5 + p.group_shift);
    uint32_t tcount = 0;                 // tiles done: the stage counter of (tile, ks) is tcount * kstages + ks
    // An A stage is published as soon as its stores have completed: each set has a stage time of
    // slack, and the issuing thread gets the stage earlier than when the arrival waited for the
    // next unpack (388 -> 382 us on M=4096).
    auto publish = [&](uint32_t stage) {
      tcgen05_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->full_a[stage]));
    };
    // Scales and biases: a thread needs one 2-byte value of each per stage, from a row of its own,
    // so a warp's load touches 32 cache lines whatever its width.  Fetched per stage they kept the
    // load/store pipe busier than anything else in the kernel; fetched as 16-byte chunks (eight
    // groups of the row) there are up to eight times fewer loads.  `cur` holds the chunk in use,
    // `nxt` the next one of the sequence (tile by tile, chunk by chunk), requested one chunk early.
    const int gs5 = 5 + p.group_shift;
    const bool vec = (row_groups & 7) == 0 && ((reinterpret_cast<uintptr_t>(p.scales) | reinterpret_cast<uintptr_t>(p.biases)) & 15) == 0;
    const int nchunks = row_groups >> 3;
    uint4 s_cur4 = make_uint4(0, 0, 0, 0), b_cur4 = s_cur4, s_nxt4 = s_cur4, b_nxt4 = s_cur4;
    int pf_tile = blockIdx.x, pf_chunk = 0;   // next chunk to request
    auto row_of = [&](int tile_) {
      const TileCoord t_ = tile_coord(p, tile_);
      const int r_ = t_.w_row0 + row_in_tile;
      return r_ < t_.w_rows_end ? r_ : t_.w_rows_end - 1;   // rows past N: results are never stored
    };
    auto prefetch = [&]() {
      if (pf_tile >= total_tiles) return;
      const size_t off = (size_t)row_of(pf_tile) * row_groups + (size_t)pf_chunk * 8;
      s_nxt4 = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.scales) + off));
      b_nxt4 = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.biases) + off));
      if (++pf_chunk == nchunks) { pf_chunk = 0; pf_tile += gridDim.x; }
    };
    auto pick = [](const uint4& c, int idx) {
      const uint32_t wsel = idx < 4 ? (idx < 2 ? c.x : c.y) : (idx < 6 ? c.z : c.w);
      return (idx & 1) ? (wsel >> 16) : (wsel & 0xFFFFu);
    };
    if (vec) prefetch();
    int cur_chunk = -1;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles && !*abort_flag; tile += gridDim.x) {
      const int row = row_of(tile);
      const unsigned short* sc = reinterpret_cast<const unsigned short*>(p.scales) + (size_t)row * row_groups;
      const unsigned short* bi = reinterpret_cast<const unsigned short*>(p.biases) + (size_t)row * row_groups;
      cur_chunk = -1;
      for (int ks = dset; ks < kstages; ks += 2) {
        const uint32_t it = tcount * (uint32_t)kstages + (uint32_t)ks;
        const uint32_t sa = it % kStagesA;
        const uint32_t sp = it % kStagesP, pp = (it / kStagesP) & 1u;
        // scale and bias of the two 32-k quarters of this thread's half (one group or two)
        uint32_t s_q[2], b_q[2];
        if (vec) {
          const int g0 = (ks * kStageK + half * 64) >> gs5, g1 = (ks * kStageK + half * 64 + 32) >> gs5;
          if ((g0 >> 3) != cur_chunk) {
            s_cur4 = s_nxt4; b_cur4 = b_nxt4;
            cur_chunk = g0 >> 3;
            prefetch();
          }
          s_q[0] = pick(s_cur4, g0 & 7); b_q[0] = pick(b_cur4, g0 & 7);
          s_q[1] = g1 == g0 ? s_q[0] : pick(s_cur4, g1 & 7);
          b_q[1] = g1 == g0 ? b_q[0] : pick(b_cur4, g1 & 7);
        } else {
          const int g0 = (ks * kStageK + half * 64) >> gs5, g1 = (ks * kStageK + half * 64 + 32) >> gs5;
          s_q[0] = __ldg(sc + g0); b_q[0] = __ldg(bi + g0);
          s_q[1] = __ldg(sc + g1); b_q[1] = __ldg(bi + g1);
        }
        TC_T0();
        if (!TC_WAIT16(smem_u32(&bars->full_p[sp]), pp, abort_flag)) { ok = false; break; }
        TC_ACC(pw0);
        const unsigned char* src0 = ring_p + sp * kPStageBytes + row_in_tile * kPRowBytes + half * (8 * BITS);
        bool freed = false;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          // this thread's 32 fields of quarter 2 * half + q: BITS words of its row
          uint32_t w[BITS];
          {
            const unsigned char* src = src0 + q * (4 * BITS);
            if constexpr (BITS == 4) {
              const uint4 v = *reinterpret_cast<const uint4*>(src);
              w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
            } else if constexpr (BITS == 8) {
              const uint4 v = *reinterpret_cast<const uint4*>(src), u = *reinterpret_cast<const uint4*>(src + 16);
              w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; w[4] = u.x; w[5] = u.y; w[6] = u.z; w[7] = u.w;
            } else if constexpr (BITS == 2 || BITS == 6) {
#pragma unroll
              for (int i = 0; i < BITS / 2; ++i) {
                const uint2 v = *reinterpret_cast<const uint2*>(src + 8 * i);
                w[2 * i] = v.x; w[2 * i + 1] = v.y;
              }
            } else {
#pragma unroll
              for (int i = 0; i < BITS; ++i) w[i] = *reinterpret_cast<const uint32_t*>(src + 4 * i);
            }
          }
          uint32_t vals[16];
          TC_T0();
          dequant32<BITS>(w, s_q[q], b_q[q], vals);
#ifdef B200Q_PROFILE
          asm volatile("" ::"r"(vals[0]), "r"(vals[5]), "r"(vals[10]), "r"(vals[15]));
#endif
          TC_ACC(pw3);
          if (q == 0) {
            TC_T0();
            if (it >= (uint32_t)kStagesA) {   // the stage that used this A slot last has been multiplied
              const uint32_t prev = it - (uint32_t)kStagesA;
              if (!TC_WAIT16(smem_u32(&bars->done[prev % kDoneRing]), (prev / kDoneRing) & 1u, abort_flag)) { ok = false; break; }
            }
            TC_ACC(pw2);
            tcgen05_fence_after();
            freed = true;
          }
          TC_T0();
          tcgen05_st_x16(tmem_a + lane_field + sa * 64 + (2 * half + q) * 16, vals);
          TC_ACC(pw4);
        }
        if (!freed) break;
        TC_T0();
        publish(sa);
        TC_ACC(pw1);
        // The packed stage is released only here, after the stores that consume the unpacked
        // registers have been issued: the shared-memory reads above have then returned for every
        // lane, so the refill of the stage cannot overtake them.
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->empty_p[sp]));
      }
      ++tcount;
    }
    if (warp == 2) { TC_OUT(8, pw0); TC_OUT(9, pw1); TC_OUT(10, pw2); TC_OUT(11, clock64() - prof_entry); }
    TC_OUT(16 + dq, pw2); TC_OUT(32 + dq, pw0);
    if (warp == 2) { TC_OUT(48, pw3); TC_OUT(49, pw4); }
  } else if (warp < kProducerPWarp) {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    const int chalf = (warp - (2 + kDequantWarps)) >> 2;  // which half of the token columns
    const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
      const TileCoord tc_ = tile_coord(p, tile);
      TC_T0();
      if (!mbar_wait(smem_u32(&bars->acc_full), tcount & 1, abort_flag)) break;
      TC_ACC(pw0);
      tcgen05_fence_after();
      const int n = tc_.n0 + quad * 32 + lane;
      const int m0 = tc_.x_row0;
      const int c_begin = chalf * (p.NT / 2 / 16 * 16);            // NT is a multiple of 16
      const int c_end = chalf == 0 ? c_begin + (p.NT / 2 / 16 * 16) : p.NT;
      for (int c = c_begin; c < c_end; c += 32) {
        uint32_t v[32];
        tcgen05_ld_x32(tmem_acc + lane_field + c, v);
        tcgen05_wait_ld();
        if (c + 32 >= c_end) {
          // the last chunk is in registers: the accumulator is free for the next tile's MMAs while
          // this chunk is converted and stored
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty));
        }
        const int lim = (tc_.rows < c_end ? tc_.rows : c_end) - c;  // valid columns of this chunk
        if (n < p.N && lim > 0) {
          if (p.dst_row == nullptr) {
            for (int q = 0; q < p.n_out; ++q) {
              __nv_bfloat16* yp = p.y_out[q] + (size_t)(m0 + c) * p.ld + p.col0 + n;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (j < lim) *yp = __float2bfloat16_rn(__uint_as_float(v[j]));
                yp += p.ld;
              }
            }
          } else {
            const int* dr = p.dst_row + m0 + c;
            for (int q = 0; q < p.n_out; ++q) {
              __nv_bfloat16* yq = p.y_out[q] + n;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < lim) yq[(size_t)dr[j] * p.N] = __float2bfloat16_rn(__uint_as_float(v[j]));
            }
          }
        }
      }
      if (c_begin >= c_end) {   // no column of this tile for this warp: release at once
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty));
      }
    }
    if (warp == 2 + kDequantWarps) { TC_OUT(12, pw0); TC_OUT(13, clock64() - prof_entry); }
  }

  // ---- teardown: everyone meets, then the allocating warp returns the tensor memory
  tcgen05_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicMax(&p.status[0], 3u);
  if (threadIdx.x == 0) peer_signal_tail(p.sig);   // every store of the block precedes the barrier above
  if (warp == 1) {
    tcgen05_fence_after();
    tcgen05_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------- host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  }
  return fn;
}

int pick_nt(int64_t M) {
  int64_t nt = (M + 15) / 16 * 16;
  return (int)(nt > 256 ? 256 : nt);
}

// x stages that fit next to the packed ring (each holds 128 k of nt tokens).
int x_stages(int nt, int bits) {
  const size_t fixed = 1024 + (size_t)stages_p(bits) * kTileN * 16 * bits + sizeof(Barriers) + 64;
  const size_t n = (kSmemMax - fixed) / ((size_t)nt * 256);
  return n >= 6 ? 6 : (n >= 4 ? 4 : (n >= 3 ? 3 : 2));   // a divisor of the length of the `done` ring
}

size_t smem_bytes(int nt, int bits) {
  const size_t need = 1024 + (size_t)x_stages(nt, bits) * nt * 256 + (size_t)stages_p(bits) * kTileN * 16 * bits +
                      sizeof(Barriers) + 64;
  // More than half of an SM's shared memory: guarantees one CTA per SM, so the 512-column
  // tensor-memory allocation never has to wait for a co-resident CTA of this kernel.
  const size_t one_per_sm = 120 * 1024;
  return need > one_per_sm ? need : one_per_sm;
}

// Launches the kernel instantiated for `bits`.
int launch_tc(int bits, int grid, size_t smem, cudaStream_t st, const CUtensorMap& map_x, const CUtensorMap& map_w,
              const TcParams& p) {
  int rc = B200Q_ERR_UNSUPPORTED;
  B200Q_DISPATCH_BITS(bits, BITS, {
    cudaError_t e = cudaFuncSetAttribute(qmm_tc_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    qmm_tc_kernel<BITS><<<grid, kThreads, smem, st>>>(map_x, map_w, p);
    rc = B200Q_OK;
  });
  if (rc != B200Q_OK) return fail(rc, "[quantized_matmul] unsupported bits %d", bits);
  B200Q_LAUNCH_OK("qmm_tc_kernel");
  return B200Q_OK;
}

}  // namespace

bool qmm_tc_supported(const QmmArgs& a) {
  if (a.dtype != B200Q_BF16 || !a.transpose || a.w_batched || a.batch != 1) return false;
  if (a.M < 1 || a.N < 1 || a.K < 128 || a.K % 128 != 0) return false;  // packed stages hold 128 k
  if (a.K % a.group != 0) return false;
  // TMA: 16-byte aligned bases and row pitches (x rows: 2K bytes, packed rows: K/2 bytes)
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.wq) & 15)) return false;
  if ((a.K * 2) % 16 != 0 || (a.K * a.bits / 8) % 16 != 0) return false;
  return true;
}

size_t qmm_tc_workspace_bytes(const QmmArgs&) { return kStatusBytes; }

int qmm_tc(const QmmArgs& a, cudaStream_t st) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(B200Q_ERR_CUDA, "[quantized_matmul] cuTensorMapEncodeTiled is not available");
  if (!a.ws || a.ws_bytes < kStatusBytes)
    return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul] workspace of %zu bytes required, %zu given",
                (size_t)kStatusBytes, a.ws_bytes);
  const int nt = pick_nt(a.M);
  CUtensorMap map_x, map_w;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)nt};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.x), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_CUDA, "[quantized_matmul] tensor map for x failed (%d)", (int)r);
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)a.K * a.bits / 8, (cuuint64_t)a.N};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K * a.bits / 8};
    const cuuint32_t box[2] = {(cuuint32_t)(16 * a.bits), (cuuint32_t)kTileN};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint32_t*>(a.wq), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_CUDA, "[quantized_matmul] tensor map for w failed (%d)", (int)r);
  }
  TcParams p{};
  p.scales = (const __nv_bfloat16*)a.scales;
  p.biases = (const __nv_bfloat16*)a.biases;
  p.y = (__nv_bfloat16*)a.y;
  if (a.peers.n > 0) {
    p.n_out = a.peers.n; p.ld = a.peers.ld; p.col0 = a.peers.col0;
    for (int q = 0; q < a.peers.n; ++q) p.y_out[q] = (__nv_bfloat16*)a.peers.y[q];
    p.sig = a.peers.sig;
  } else {
    p.n_out = 1; p.ld = a.N; p.col0 = 0; p.y_out[0] = (__nv_bfloat16*)a.y;
  }
  p.status = reinterpret_cast<uint32_t*>(static_cast<char*>(a.ws) + a.ws_bytes - kStatusBytes);
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.NT = nt;
  p.nsb = x_stages(nt, (int)a.bits);
  p.n_tiles = (int)((a.N + kTileN - 1) / kTileN);
  p.m_tiles = (int)((a.M + nt - 1) / nt);
  p.group_shift = a.group == 32 ? 0 : (a.group == 64 ? 1 : 2);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = (long long)p.n_tiles * p.m_tiles;
  const int grid = (int)(tiles < sms ? tiles : sms);
  return launch_tc(a.bits, grid, smem_bytes(nt, a.bits), st, map_x, map_w, p);
}

int qmm_tc_grouped(const GroupedArgs& a, cudaStream_t st) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(B200Q_ERR_CUDA, "[gather_qmm] cuTensorMapEncodeTiled is not available");
  const int nt = a.nt;
  CUtensorMap map_x, map_w;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.n_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)nt};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.x_sorted), dims, strides, box,
                     estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_CUDA, "[gather_qmm] tensor map for x failed (%d)", (int)r);
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)a.K * a.bits / 8, (cuuint64_t)(a.E * a.N)};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K * a.bits / 8};
    const cuuint32_t box[2] = {(cuuint32_t)(16 * a.bits), (cuuint32_t)kTileN};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint32_t*>(a.wq), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_CUDA, "[gather_qmm] tensor map for w failed (%d)", (int)r);
  }
  TcParams p{};
  p.mtiles = static_cast<const MTile*>(a.mtiles);
  p.n_mtiles = a.n_mtiles;
  p.dst_row = a.dst_row;
  p.scales = (const __nv_bfloat16*)a.scales;
  p.biases = (const __nv_bfloat16*)a.biases;
  p.y = (__nv_bfloat16*)a.y;
  if (a.peers.n > 0) {
    p.n_out = a.peers.n;
    for (int q = 0; q < a.peers.n; ++q) p.y_out[q] = (__nv_bfloat16*)a.peers.y[q];
    p.sig = a.peers.sig;
  } else {
    p.n_out = 1; p.y_out[0] = (__nv_bfloat16*)a.y;
  }
  p.ld = a.N; p.col0 = 0;
  p.status = a.status;
  p.M = (int)a.n_rows; p.N = (int)a.N; p.K = (int)a.K;
  p.NT = nt;
  p.nsb = x_stages(nt, (int)a.bits);
  p.n_tiles = (int)((a.N + kTileN - 1) / kTileN);
  p.m_tiles = 0;
  p.group_shift = a.group == 32 ? 0 : (a.group == 64 ? 1 : 2);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = (long long)p.n_tiles * a.max_mtiles;  // upper bound; the kernel reads the exact count
  const int grid = (int)(tiles < sms ? tiles : sms);
  return launch_tc(a.bits, grid, smem_bytes(nt, a.bits), st, map_x, map_w, p);
}

size_t qmm_tc_mtile_bytes() { return sizeof(MTile); }

}  // namespace b200q
