// Decode path, row-owning form: y[M<=16, N] = x[M, K] * dequant(W[N, K])^T, bf16, HBM-bound.
//
// Replaces cu::qmv_kernel / the small-M use of cu::qmm_sm80_kernel of the reference
// (mlx/backend/cuda/quantized/qmm/qmv.cu:84-209, quantized.cpp:106-136).
//
// Design (one persistent CTA per SM, 16 warps, no scratch in global memory):
//  * Every CTA owns a contiguous range of 8-row blocks of W for the WHOLE of K, so no output is
//    shared between CTAs: no global atomics, no arrival counters, no workspace.
//  * Packed rows, scales and biases reach shared memory through `cp.async.bulk` (one copy per
//    row: whole rows are contiguous, so no tensor map and no descriptor fetch is needed), into
//    a ring of stages of 16 rows each with padded row pitch (bank-conflict-free reads).  All
//    stages that fit are requested at kernel entry: ~190 KB per SM are in flight from the
//    first microsecond.  A stage is refilled by whichever warp is last to finish with it.
//  * K is cut into 16 slices, one per warp.  A warp keeps the x values of its slice in
//    registers, as mma.sync B fragments in the order the unpack produces weights
//    (pairs (k, k+4) of every 8 consecutive k), for the whole kernel: x is read from L2 once per
//    CTA and never touches shared memory.  Long K runs in several phases, x is reloaded per phase.
//  * Weights are unpacked with shift + lop3 to the bf16 numbers 128+q ("0x4300 | q") and fed to
//    mma.sync.m16n8k16 as the A operand.  Scales are applied per group to the fp32 group sums,
//    the "128" offset and the biases come back through two small MMAs against the group sums of
//    x:  y = sum_g s_g * (sum_k x_k (128 + q_k))  +  sum_g (b_g - 128 s_g) * (sum_k x_k).
//    8-bit fields are treated as two 4-bit fields against (x, 16 x): same unpack, same rate
//    per byte.
//  * The 16 warps leave their fp32 partial tiles in shared memory; the last warp to arrive adds
//    them in warp order (the result does not depend on timing), converts and stores y.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace b200q {
namespace {

using tc::mbar_init;
using tc::mbar_expect_tx;
using tc::mbar_wait;
using tc::smem_u32;

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kPartialBufs = 2;
constexpr size_t kSmemLimit = 227 * 1024;

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
  return d;
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ uint4 ldg_nc_u128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// Compile-time shape of one (bits, group size, token tiles) instantiation.
template <int BITS, int G, int MT>
struct Cfg {
  static_assert(BITS == 2 || BITS == 4 || BITS == 8, "field widths handled by this kernel");
  static constexpr int GB = G * BITS / 8;            // packed bytes of one group of one row
  static constexpr int LB = GB / 4;                  // ... of which one lane of a quad reads
  static constexpr int KBLK = BITS == 8 ? 4 : 8;     // k values per unpack block (four bf16 pairs)
  static constexpr int NBLK = (G / 4) / KBLK;        // blocks per lane and group
  static constexpr int WORDS = LB >= 4 ? LB / 4 : 1; // registers holding the lane's packed bytes
  static constexpr int XG = MT * NBLK * 4;           // x registers per group
  static constexpr int NGW_RAW = 64 / XG;            // groups per warp and phase: 64 registers of x
  static constexpr int NGW = NGW_RAW > 8 ? 8 : (NGW_RAW < 1 ? 1 : NGW_RAW);
  // Row pitch padding (bytes mod 128) that makes the quad-per-row reads conflict-free.
  static constexpr int PAD = LB == 8 ? 32 : (LB == 16 ? 64 : 16);
};

struct RowsParams {
  const __nv_bfloat16* x;
  const unsigned char* wq;
  const unsigned char* scales;
  const unsigned char* biases;
  __nv_bfloat16* y[kMaxPeers];
  int n_out;
  long long ld, col0;
  int M, N, K;
  int nblk8;            // ceil(N / 8)
  int groups;           // K / G
  int nph, gph;         // phases over K, groups per (full) phase
  int nst;              // ring stages
  uint32_t rs, srs;     // shared-memory pitch of a packed row chunk / a scale row chunk
  uint32_t slot_bytes;  // 16 * rs + 32 * srs
  uint32_t off_slots, off_pbuf, off_tile, off_tileph;
  long long row_bytes;  // K * BITS / 8
  long long srow_bytes; // groups * 2
  uint32_t* status;     // may be null
  int early;            // weights, scales and biases may be read before the previous kernel ended
};

// Unpacks block `blk` of the lane's packed bytes into four bf16x2 registers (128+q_i, 128+q_{i+4}).
template <int BITS>
__device__ __forceinline__ void unpack_block(const uint32_t* w, int blk, uint32_t (&P)[4]) {
  constexpr uint32_t kMagic = 0x43004300u;
  if constexpr (BITS == 4 || BITS == 8) {
    const uint32_t v = w[blk];
#pragma unroll
    for (int i = 0; i < 4; ++i) P[i] = lop3_and_or(v >> (4 * i), 0x000F000Fu, kMagic);
  } else {
    // 16 fields per word; a block is one half word: spread its two bytes to bits 0-7 / 16-23
    const uint32_t v = __byte_perm(w[blk >> 1], 0u, (blk & 1) ? 0x4342 : 0x4140);
#pragma unroll
    for (int i = 0; i < 4; ++i) P[i] = lop3_and_or(v >> (2 * i), 0x00030003u, kMagic);
  }
}

template <int LB>
__device__ __forceinline__ void lds_lane(uint32_t addr, uint32_t* w) {
  if constexpr (LB == 2) {
    w[0] = lds_u16(addr);
  } else if constexpr (LB == 4) {
    w[0] = lds_u32(addr);
  } else if constexpr (LB == 8) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(addr));
  } else {
#pragma unroll
    for (int i = 0; i < LB / 16; ++i)
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(w[4 * i]), "=r"(w[4 * i + 1]), "=r"(w[4 * i + 2]), "=r"(w[4 * i + 3])
                   : "r"(addr + 16 * i));
  }
}

template <int BITS, int G, int MT>
__global__ void __launch_bounds__(kThreads, 1) qmv_rows_kernel(const RowsParams p) {
  using C = Cfg<BITS, G, MT>;
  constexpr int NGW = C::NGW, NBLK = C::NBLK, GB = C::GB, LB = C::LB;
  extern __shared__ __align__(128) unsigned char smem[];
  // header: [0, 8*nst) full barriers | 256: arrive counters | 320: partial-buffer epochs | 384: abort
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar0 = smem_base;
  volatile int* arrive = reinterpret_cast<volatile int*>(smem + 256);
  volatile int* pb_done = reinterpret_cast<volatile int*>(smem + 320);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 384);
  volatile int* tile_ph = reinterpret_cast<volatile int*>(smem + p.off_tileph);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  {
    // The first mma.sync of a kernel is slow (the tensor pipe wakes up): issue one now.
    float d0, d1, d2, d3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%4,%4,%4}, {%4,%4}, {%5,%5,%5,%5};"
                 : "=f"(d0), "=f"(d1), "=f"(d2), "=f"(d3) : "r"(0u), "f"(0.0f));
  }
  asm volatile("griddepcontrol.launch_dependents;");

  const int G_ = gridDim.x;
  const int b0 = (int)((long long)blockIdx.x * p.nblk8 / G_);
  const int b1 = (int)((long long)(blockIdx.x + 1) * p.nblk8 / G_);
  const int nrg = (b1 - b0 + 1) >> 1;           // 16-row groups of this CTA
  const int total = nrg * p.nph;                // stages
  const int row_end = min(b1 * 8, p.N);
  const int nst = p.nst;

  if (tid == 0) {
    for (int i = 0; i < nst; ++i) mbar_init(bar0 + 8 * i, 1);
    for (int i = 0; i < 16; ++i) arrive[i] = 0;
    for (int i = 0; i < kPartialBufs; ++i) pb_done[i] = 0;
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (p.nph > 1)
    for (int i = tid; i < nrg; i += kThreads) tile_ph[i] = 0;
  __syncthreads();

  // ---- producer side: one warp requests one stage ------------------------------------
  auto issue_stage = [&](int s) {
    const int ph = s / nrg, rg = s - ph * nrg;
    const int slot = s % nst;
    const int gp = min(p.gph, p.groups - ph * p.gph);
    const uint32_t wbytes = (uint32_t)gp * GB, sbytes = (uint32_t)gp * 2;
    const int row0 = (b0 + 2 * rg) * 8;
    const int nrows = min(16, row_end - row0);
    const uint32_t bar = bar0 + 8 * slot;
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)nrows * (wbytes + 2 * sbytes));
    __syncwarp();
    const uint32_t slot_base = smem_base + p.off_slots + (uint32_t)slot * p.slot_bytes;
    const int r = lane & 15;
    if (r < nrows) {
      if (lane < 16) {
        bulk_g2s(slot_base + r * p.rs, p.wq + (long long)(row0 + r) * p.row_bytes + (long long)ph * p.gph * GB, wbytes, bar);
      } else {
        const long long so = (long long)(row0 + r) * p.srow_bytes + (long long)ph * p.gph * 2;
        bulk_g2s(slot_base + 16 * p.rs + r * p.srs, p.scales + so, sbytes, bar);
        bulk_g2s(slot_base + 16 * p.rs + 16 * p.srs + r * p.srs, p.biases + so, sbytes, bar);
      }
    }
  };

  if (p.early)
    for (int s = warp; s < min(nst, total); s += kWarps) issue_stage(s);
  // Everything the previous kernel of the stream may still produce (x) or use (y) is touched only
  // after this point.  Without the launch attribute the instruction returns at once.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (!p.early)
    for (int s = warp; s < min(nst, total); s += kWarps) issue_stage(s);

  // ---- per-phase state of this warp -----------------------------------------------------
  uint32_t X[NGW][NBLK][MT][4];   // B fragments of this warp's K slice
  uint32_t sx_hi[MT], sx_lo[MT];  // group sums of x for groups 2t, 2t+1 of the slice (bf16 hi / lo parts)
  int cnt = 0, g0 = 0, nact = 0;
  int ph = 0, rg = 0, slot = 0, use = 0, pbi = 0, pbe = 0;

  auto setup_phase = [&]() {
    const int gp = min(p.gph, p.groups - ph * p.gph);
    const int base = gp / kWarps, rem = gp - base * kWarps;
    cnt = base + (warp < rem ? 1 : 0);
    g0 = warp * base + min(warp, rem);
    nact = gp < kWarps ? gp : kWarps;
    float sx[NGW][MT];
#pragma unroll
    for (int gi = 0; gi < NGW; ++gi) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        sx[gi][mt] = 0.0f;
        const int tok = mt * 8 + g;
        const bool live = gi < cnt && tok < p.M;
        const __nv_bfloat16* xp = p.x + (long long)tok * p.K + (long long)(ph * p.gph + g0 + gi) * G + t * (G / 4);
        if constexpr (BITS == 8) {
          // two blocks of 4 k per 16-byte load; pairs (x0,x2), 16(x0,x2), (x1,x3), 16(x1,x3)
#pragma unroll
          for (int j = 0; j < NBLK / 2; ++j) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (live) v = ldg_nc_u128(xp + 8 * j);
            sx[gi][mt] += (bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y)) + (bf16lo(v.z) + bf16hi(v.z)) +
                          (bf16lo(v.w) + bf16hi(v.w));
            const uint32_t a = __byte_perm(v.x, v.y, 0x5410), b = __byte_perm(v.x, v.y, 0x7632);
            const uint32_t c = __byte_perm(v.z, v.w, 0x5410), d = __byte_perm(v.z, v.w, 0x7632);
            X[gi][2 * j][mt][0] = a; X[gi][2 * j][mt][1] = mul_bf16x2(a, 0x41804180u);
            X[gi][2 * j][mt][2] = b; X[gi][2 * j][mt][3] = mul_bf16x2(b, 0x41804180u);
            X[gi][2 * j + 1][mt][0] = c; X[gi][2 * j + 1][mt][1] = mul_bf16x2(c, 0x41804180u);
            X[gi][2 * j + 1][mt][2] = d; X[gi][2 * j + 1][mt][3] = mul_bf16x2(d, 0x41804180u);
          }
        } else {
#pragma unroll
          for (int j = 0; j < NBLK; ++j) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (live) v = ldg_nc_u128(xp + 8 * j);
            sx[gi][mt] += (bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y)) + (bf16lo(v.z) + bf16hi(v.z)) +
                          (bf16lo(v.w) + bf16hi(v.w));
            X[gi][j][mt][0] = __byte_perm(v.x, v.z, 0x5410);  // (x0, x4)
            X[gi][j][mt][1] = __byte_perm(v.x, v.z, 0x7632);  // (x1, x5)
            X[gi][j][mt][2] = __byte_perm(v.y, v.w, 0x5410);  // (x2, x6)
            X[gi][j][mt][3] = __byte_perm(v.y, v.w, 0x7632);  // (x3, x7)
          }
        }
      }
    }
    // group sums over the quad, then lane t keeps groups 2t and 2t+1 (the k slots it feeds)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float e0 = 0.0f, e1 = 0.0f;
#pragma unroll
      for (int gi = 0; gi < NGW; ++gi) {
        float v = sx[gi][mt];
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
        if ((gi >> 1) == t) {
          if (gi & 1) e1 = v; else e0 = v;
        }
      }
      const uint32_t hi = pack_bf16x2(e0, e1);
      sx_hi[mt] = hi;
      sx_lo[mt] = pack_bf16x2(e0 - bf16lo(hi), e1 - bf16hi(hi));
    }
  };
  setup_phase();

  // ---- main loop over stages -------------------------------------------------------------
  for (int s = 0; s < total; ++s) {
    if (cnt > 0) {
      const uint32_t slot_base = smem_base + p.off_slots + (uint32_t)slot * p.slot_bytes;
      if (!mbar_wait(bar0 + 8 * slot, use & 1, abort_flag)) break;
      float out[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) out[mt][c] = 0.0f;
      const uint32_t w_lo = slot_base + g * p.rs + g0 * GB + t * LB;
      const uint32_t w_hi = w_lo + 8 * p.rs;
      const uint32_t sc_lo = slot_base + 16 * p.rs + g * p.srs + g0 * 2;
      const uint32_t sc_hi = sc_lo + 8 * p.srs;
#pragma unroll
      for (int gi = 0; gi < NGW; ++gi) {
        if (gi < cnt) {
          uint32_t wl[C::WORDS], wh[C::WORDS];
          lds_lane<LB>(w_lo + gi * GB, wl);
          lds_lane<LB>(w_hi + gi * GB, wh);
          const float s_l = __uint_as_float(lds_u16(sc_lo + gi * 2) << 16);
          const float s_h = __uint_as_float(lds_u16(sc_hi + gi * 2) << 16);
          float acc[MT][4];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[mt][c] = 0.0f;
#pragma unroll
          for (int j = 0; j < NBLK; ++j) {
            uint32_t Pl[4], Ph[4];
            unpack_block<BITS>(wl, j, Pl);
            unpack_block<BITS>(wh, j, Ph);
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
                mma_bf16(acc[mt], Pl[2 * h], Ph[2 * h], Pl[2 * h + 1], Ph[2 * h + 1], X[gi][j][mt][2 * h],
                         X[gi][j][mt][2 * h + 1]);
          }
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            out[mt][0] = fmaf(s_l, acc[mt][0], out[mt][0]);
            out[mt][1] = fmaf(s_l, acc[mt][1], out[mt][1]);
            out[mt][2] = fmaf(s_h, acc[mt][2], out[mt][2]);
            out[mt][3] = fmaf(s_h, acc[mt][3], out[mt][3]);
          }
        }
      }
      // biases and the unpack offset: (b_g - OFFSET * s_g) * sum_k x_k, k slots 2t, 2t+1 (hi) / +8 (lo)
      {
        uint32_t bl = 0, bh = 0, sl = 0, sh = 0;
        if (2 * t < cnt) {
          const uint32_t bi_lo = sc_lo + 16 * p.srs, bi_hi = sc_hi + 16 * p.srs;
          const bool two = 2 * t + 1 < cnt;
          bl = lds_u16(bi_lo + 4 * t) | (two ? lds_u16(bi_lo + 4 * t + 2) << 16 : 0u);
          bh = lds_u16(bi_hi + 4 * t) | (two ? lds_u16(bi_hi + 4 * t + 2) << 16 : 0u);
          sl = lds_u16(sc_lo + 4 * t) | (two ? lds_u16(sc_lo + 4 * t + 2) << 16 : 0u);
          sh = lds_u16(sc_hi + 4 * t) | (two ? lds_u16(sc_hi + 4 * t + 2) << 16 : 0u);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(out[mt], bl, bh, bl, bh, sx_hi[mt], sx_lo[mt]);
          mma_bf16(out[mt], sl, sh, sl, sh, mul_bf16x2(sx_hi[mt], 0xC300C300u), mul_bf16x2(sx_lo[mt], 0xC300C300u));
          if constexpr (BITS == 8)
            mma_bf16(out[mt], sl, sh, sl, sh, mul_bf16x2(sx_hi[mt], 0xC500C500u), mul_bf16x2(sx_lo[mt], 0xC500C500u));
        }
      }
      // hand the partial tile over
      if (pbe > 0 && lane == 0) {
        uint32_t spins = 0;
        while (pb_done[pbi] < pbe) {
          if (++spins > tc::kSpinLimit) { *abort_flag = 1; break; }
          __nanosleep(20);
        }
      }
      __syncwarp();
      if (*abort_flag) break;
      const uint32_t pb = smem_base + p.off_pbuf + (uint32_t)pbi * (kWarps * MT * 512);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
        sts_f4(pb + (warp * MT + mt) * 512 + lane * 16, out[mt][0], out[mt][1], out[mt][2], out[mt][3]);
      __syncwarp();
      int last = 0;
      if (lane == 0) {
        __threadfence_block();
        const int old = atomicAdd(const_cast<int*>(&arrive[slot]), 1);
        last = (old == nact - 1);
      }
      last = __shfl_sync(0xFFFFFFFFu, last, 0);
      if (last) {
        __threadfence_block();
        float sum[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) sum[mt][c] = 0.0f;
        for (int w = 0; w < nact; ++w) {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const float4 v = lds_f4(pb + (w * MT + mt) * 512 + lane * 16);
            sum[mt][0] += v.x; sum[mt][1] += v.y; sum[mt][2] += v.z; sum[mt][3] += v.w;
          }
        }
        __syncwarp();
        if (lane == 0) {
          arrive[slot] = 0;
          __threadfence_block();
          pb_done[pbi] = pbe + 1;
        }
        bool final_phase = true;
        if (p.nph > 1) {
          const uint32_t tl = smem_base + p.off_tile + (uint32_t)rg * (MT * 512);
          if (ph > 0) {
            if (lane == 0) {
              uint32_t spins = 0;
              while (tile_ph[rg] < ph) {
                if (++spins > tc::kSpinLimit) { *abort_flag = 1; break; }
                __nanosleep(20);
              }
            }
            __syncwarp();
            __threadfence_block();
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const float4 v = lds_f4(tl + mt * 512 + lane * 16);
              sum[mt][0] += v.x; sum[mt][1] += v.y; sum[mt][2] += v.z; sum[mt][3] += v.w;
            }
          }
          final_phase = ph == p.nph - 1;
          if (!final_phase) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) sts_f4(tl + mt * 512 + lane * 16, sum[mt][0], sum[mt][1], sum[mt][2], sum[mt][3]);
            __syncwarp();
            if (lane == 0) {
              __threadfence_block();
              tile_ph[rg] = ph + 1;
            }
          }
        }
        if (final_phase) {
          const int row0 = (b0 + 2 * rg) * 8;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int row = row0 + g + (c >> 1) * 8;
              const int tok = mt * 8 + 2 * t + (c & 1);
              if (row < row_end && tok < p.M) {
                const __nv_bfloat16 o = __float2bfloat16_rn(sum[mt][c]);
                for (int q = 0; q < p.n_out; ++q) p.y[q][(long long)tok * p.ld + p.col0 + row] = o;
              }
            }
          }
        }
        if (s + nst < total) {
          // the refill overwrites bytes every warp has finished reading (they all arrived above)
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          issue_stage(s + nst);
        }
      }
    }
    // advance to the next stage
    if (++slot == nst) { slot = 0; ++use; }
    if (++pbi == kPartialBufs) { pbi = 0; ++pbe; }
    if (++rg == nrg) {
      rg = 0;
      ++ph;
      if (ph < p.nph) setup_phase();
    }
  }
  if (*abort_flag && tid == 0 && p.status) atomicMax(&p.status[0], 7u);
}

struct RowsPlan {
  bool ok;
  int grid, mt;
  size_t smem;
  RowsParams prm;
};

int sm_count_rows() {
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

template <int BITS, int G, int MT>
bool fill_plan(const QmmArgs& a, RowsPlan& pl) {
  using C = Cfg<BITS, G, MT>;
  RowsParams& p = pl.prm;
  const int groups = (int)(a.K / G);
  const int cap = kWarps * C::NGW;
  p.nph = (groups + cap - 1) / cap;
  p.gph = ((groups + p.nph - 1) / p.nph + 7) / 8 * 8;
  if (p.gph > cap) return false;
  p.groups = groups;
  p.rs = (uint32_t)((p.gph * C::GB + 127) / 128 * 128 + C::PAD);
  p.srs = (uint32_t)((p.gph * 2 + 127) / 128 * 128 + 16);
  p.slot_bytes = 16 * p.rs + 32 * p.srs;
  p.nblk8 = (int)((a.N + 7) / 8);
  const int sms = sm_count_rows();
  pl.grid = p.nblk8 < sms ? p.nblk8 : sms;
  const int max_blk = (p.nblk8 + pl.grid - 1) / pl.grid;
  const int max_rg = (max_blk + 1) / 2 + 1;
  size_t off = 512;
  p.off_tileph = (uint32_t)off;
  if (p.nph > 1) off += (size_t)(max_rg * 4 + 127) / 128 * 128;
  p.off_pbuf = (uint32_t)off;
  off += (size_t)kPartialBufs * kWarps * MT * 512;
  p.off_tile = (uint32_t)off;
  if (p.nph > 1) off += (size_t)max_rg * MT * 512;
  p.off_slots = (uint32_t)off;
  if (off + 2 * (size_t)p.slot_bytes > kSmemLimit) return false;
  const long long stages = (long long)max_rg * p.nph;
  long long nst = (long long)((kSmemLimit - off) / p.slot_bytes);
  if (nst > 16) nst = 16;
  if (nst > stages) nst = stages;
  if (nst < 1) nst = 1;
  p.nst = (int)nst;
  pl.smem = off + (size_t)p.nst * p.slot_bytes;
  p.row_bytes = a.K * BITS / 8;
  p.srow_bytes = (long long)groups * 2;
  pl.mt = MT;
  return true;
}

RowsPlan make_plan(const QmmArgs& a) {
  RowsPlan pl{};
  pl.ok = false;
  if (a.dtype != B200Q_BF16 || !a.transpose || a.w_batched || a.batch != 1) return pl;
  if (a.M < 1 || a.M > 16 || a.N < 1 || a.K < 1) return pl;
  if (a.bits != 2 && a.bits != 4 && a.bits != 8) return pl;
  if (a.K % (8 * a.group) != 0) return pl;   // scale rows of whole 16-byte pieces
  if (a.N > (1ll << 30)) return pl;
  const int mt = a.M > 8 ? 2 : 1;
  bool ok = false;
#define B200Q_ROWS_CASE(BITS_, G_)                                                          \
  if (a.bits == BITS_ && a.group == G_)                                                     \
    ok = mt == 2 ? fill_plan<BITS_, G_, 2>(a, pl) : fill_plan<BITS_, G_, 1>(a, pl);
  B200Q_ROWS_CASE(2, 32) B200Q_ROWS_CASE(2, 64) B200Q_ROWS_CASE(2, 128)
  B200Q_ROWS_CASE(4, 32) B200Q_ROWS_CASE(4, 64) B200Q_ROWS_CASE(4, 128)
  B200Q_ROWS_CASE(8, 32) B200Q_ROWS_CASE(8, 64) B200Q_ROWS_CASE(8, 128)
#undef B200Q_ROWS_CASE
  if (!ok) return pl;
  RowsParams& p = pl.prm;
  p.x = (const __nv_bfloat16*)a.x;
  p.wq = (const unsigned char*)a.wq;
  p.scales = (const unsigned char*)a.scales;
  p.biases = (const unsigned char*)a.biases;
  if (a.peers.n > 0) {
    p.n_out = a.peers.n; p.ld = a.peers.ld; p.col0 = a.peers.col0;
    for (int q = 0; q < a.peers.n; ++q) p.y[q] = (__nv_bfloat16*)a.peers.y[q];
  } else {
    p.n_out = 1; p.ld = a.N; p.col0 = 0; p.y[0] = (__nv_bfloat16*)a.y;
  }
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.status = nullptr;
  pl.ok = true;
  return pl;
}

bool pdl_enabled_rows() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200Q_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <int BITS, int G, int MT>
int launch_rows(const RowsPlan& pl, cudaStream_t st) {
  auto kern = qmv_rows_kernel<BITS, G, MT>;
  if (pl.smem > 48 * 1024)
    B200Q_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled_rows() ? 1 : 0;
  B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, pl.prm));
  B200Q_LAUNCH_OK("qmv_rows_kernel");
  return B200Q_OK;
}

}  // namespace

// Process-wide promise that packed weights, scales and biases are not written by the
// operation that precedes a matmul on its stream (set by b200q_set_weights_constant or
// B200Q_WEIGHTS_CONSTANT=1).  Only then may the decode kernel request them before the
// previous kernel has finished (programmatic dependent launch).
static int g_weights_constant = -1;
bool weights_constant() {
  if (g_weights_constant < 0) {
    const char* e = getenv("B200Q_WEIGHTS_CONSTANT");
    g_weights_constant = (e && e[0] == '1') ? 1 : 0;
  }
  return g_weights_constant == 1;
}
void set_weights_constant(int on) { g_weights_constant = on ? 1 : 0; }

bool qmv_rows_supported(const QmmArgs& a) {
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.wq) |
                       reinterpret_cast<uintptr_t>(a.scales) | reinterpret_cast<uintptr_t>(a.biases);
  if (al & 15) return false;
  return make_plan(a).ok;
}

int qmv_rows(const QmmArgs& a, cudaStream_t st) {
  RowsPlan pl = make_plan(a);
  if (!pl.ok) return fail(B200Q_ERR_UNSUPPORTED, "[quantized_matmul] qmv_rows: unsupported problem");
  pl.prm.early = weights_constant() ? 1 : 0;
  if (a.ws && a.ws_bytes >= kStatusBytes)
    pl.prm.status = reinterpret_cast<uint32_t*>(static_cast<char*>(a.ws) + a.ws_bytes - kStatusBytes);
  int rc = B200Q_ERR_UNSUPPORTED;
#define B200Q_ROWS_CASE(BITS_, G_)                                                                  \
  if (a.bits == BITS_ && a.group == G_)                                                             \
    rc = pl.mt == 2 ? launch_rows<BITS_, G_, 2>(pl, st) : launch_rows<BITS_, G_, 1>(pl, st);
  B200Q_ROWS_CASE(2, 32) B200Q_ROWS_CASE(2, 64) B200Q_ROWS_CASE(2, 128)
  B200Q_ROWS_CASE(4, 32) B200Q_ROWS_CASE(4, 64) B200Q_ROWS_CASE(4, 128)
  B200Q_ROWS_CASE(8, 32) B200Q_ROWS_CASE(8, 64) B200Q_ROWS_CASE(8, 128)
#undef B200Q_ROWS_CASE
  return rc;
}

}  // namespace b200q
