// Decode path, row-owning form: y[M<=16, N] = x[M, K] * dequant(W[N, K])^T, bf16, HBM-bound.
//
// Replaces cu::qmv_kernel / the small-M use of cu::qmm_sm80_kernel of the reference
// (mlx/backend/cuda/quantized/qmm/qmv.cu:84-209, quantized.cpp:106-136).
//
// Design (one persistent CTA per SM; 16 consumer warps, one loader warp, one reducer warp; no
// scratch in global memory):
//  * Every CTA owns a contiguous range of 8-row blocks of W for the WHOLE of K, so no output is
//    shared between CTAs: no global atomics, no arrival counters, no workspace.
//  * A stage is 16 weight rows x one K phase.  The loader warp brings it in with one tiled TMA
//    load (cp.async.bulk.tensor.3d, box 128 B x 16 rows x up to 32 chunks, 128-byte swizzle) plus
//    one or two boxes each for the rows' scales and biases: a handful of large copies per stage,
//    because every bulk-copy instruction costs the SM's copy engine about 60 cycles whatever its
//    size.  At most `inflight` stages are outstanding, so the first one is not diluted by the rest
//    and lands early; a ring slot is requested again as soon as all consumers are done with it.
//  * K is cut into 16 slices, one per consumer warp.  A warp keeps the x values of its slice in
//    registers for the whole phase, as mma.sync B fragments in the order the unpack produces the
//    weights: x is read from L2 once per CTA and never touches shared memory.
//  * Packed words come out of shared memory with ldmatrix (conflict-free on the swizzled tile:
//    lane (g, t) receives word t of a 16-byte unit of rows g and g+8) and become mma.sync.m16n8k16
//    A operands with one AND per register: a bf16 whose high byte is zero is the subnormal number
//    (low byte) * 2^-133, exactly, and the tensor cores take subnormal inputs exactly, so
//    "w & 0x000F000F" IS the pair (q_0, q_4) * 2^-133 and "w & 0x00F000F0" the pair (16 q_1, 16 q_5)
//    * 2^-133; one shift by 8 brings the other two bytes down.  The integer processing pipe that
//    does the unpacking is what bounds this kernel, and this form needs 5 operations per 8 four-bit
//    weights (3 per 4 eight-bit weights, 9 per 16 two-bit weights) and no offset correction.
//    To keep the products inside fp32's range whatever the magnitude of x, every token row of a
//    warp's K slice is multiplied by a power of two that brings its largest element to about 2^64
//    (less where the field sits some bits up) when it is put into registers, and the warp's sums
//    are multiplied back by the matching power of two before they leave the warp: exact.
//    Scales are applied per group to fp32 group sums, the biases come back through one small MMA
//    against the group sums of x:  y = sum_g s_g * (sum_k x_k q_k) + sum_g b_g * (sum_k x_k).
//    Four independent accumulation chains per warp hide the mma.sync latency.
//  * The consumer warps leave fp32 partial tiles in shared memory; the reducer warp adds them in
//    warp order (the result does not depend on timing), converts and stores y.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace b200q {
namespace {

using tc::mbar_init;
using tc::mbar_expect_tx;
using tc::mbar_wait;
using tc::mbar_test;   // non-blocking look at a barrier phase (try_wait may park the thread before it says no)
using tc::smem_u32;

constexpr int kConsumers = 16;                   // warps that multiply; one K slice each
// Registers are handed out per group of four warps: the loader and the reducer warp come with two
// idle companions, and the two kinds of warps re-balance their register budgets at entry.
constexpr int kThreads = (kConsumers + 4) * 32;
constexpr int kRegsConsumer = 112, kRegsService = 32;
// setmaxnreg only moves registers inside what the block was launched with (96 per thread at this
// block size): a request beyond that pool would wait forever.
static_assert(kRegsConsumer * kConsumers * 32 + kRegsService * 4 * 32 <= 96 * kThreads,
              "register budgets exceed the launch allocation");
constexpr int kPartialBufs = 2;                  // fp32 partial tiles of the stages being reduced
constexpr size_t kSmemLimit = 227 * 1024;

// Clock marks for tuning builds only (-DB200Q_ROWS_PROFILE): cycles since kernel entry per CTA and
// warp, in a buffer of their own that a test harness reads back with cudaMemcpyFromSymbol.
#ifdef B200Q_ROWS_PROFILE
__device__ uint32_t g_rows_prof[160][kConsumers + 4][32];
__device__ unsigned long long g_rows_t[64][4];   // per launch (mod 64): first CTA start, last CTA start, first end, last end (globaltimer)
__device__ unsigned int g_rows_launch_in, g_rows_launch_out;
#define RP_MARK(i)                                                                            \
  do {                                                                                        \
    if (lane == 0 && (i) < 32 && blockIdx.x < 160)                                            \
      g_rows_prof[blockIdx.x][warp][(i)] = (uint32_t)(clock64() - rp_entry);                  \
  } while (0)
#else
#define RP_MARK(i)
#endif

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
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Four 8x8 matrices of 16-bit elements; lane l supplies the address of row l%8 of matrix l/8 and
// receives, from matrix m, the 32-bit word (l%4) of row l/4.
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint4 ldg_nc_u128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc_u64(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ float sum_bf16x2(uint32_t v) { return bf16lo(v) + bf16hi(v); }
__device__ __forceinline__ float asum_bf16x2(uint32_t v) { return fabsf(bf16lo(v)) + fabsf(bf16hi(v)); }

__host__ __device__ constexpr int cmin(int a, int b) { return a < b ? a : b; }
__host__ __device__ constexpr int cmax(int a, int b) { return a > b ? a : b; }

constexpr int kMaxPhases = 16;

// Compile-time shape of one (bits, group size, token tiles) instantiation.  A "unit" is 16 packed
// bytes of one row (what one ldmatrix row holds); lane t of a quad owns word t of every unit.
template <int BITS, int G, int MT>
struct Cfg {
  static_assert(BITS == 2 || BITS == 4 || BITS == 8, "field widths handled by this kernel");
  static constexpr int GB = G * BITS / 8;                  // packed bytes of one group of one row
  static_assert(GB >= 16, "a group must fill at least one 16-byte unit");
  static constexpr int UG = GB / 16;                       // units per group
  static constexpr int KW = 32 / BITS;                     // k values per 32-bit word
  static constexpr int NP = KW / 2;                        // bf16x2 registers a word unpacks to
  static constexpr int UW = cmax(UG, cmin(cmin(64 / (MT * NP), 8 * UG), 16));   // units per warp and phase
  static constexpr int NGW = UW / UG;                      // groups per warp and phase (2, 4 or 8)
  static_assert(NGW >= 2 && NGW <= 8, "groups are processed in pairs, eight at most feed one bias MMA");
};

struct RowsParams {
  const __nv_bfloat16* x;
  __nv_bfloat16* y[kMaxPeers];
  int n_out;
  long long ld, col0;
  PeerSignal sig;       // completion signal towards the ranks that receive y (n == 0: none)
  int M, N, K;
  int nblk8;            // ceil(N / 8)
  int nph;              // phases over K
  int ph_g0[kMaxPhases];   // first group of the phase
  int ph_cnt[kMaxPhases];  // groups per warp in the phase (1, 2, 4 or 8; 16 warps)
  int nch, nsb;         // 128-byte chunks of packed bytes / of scales per row in a TMA box
  int nst;              // ring stages
  uint32_t slot_bytes;  // (nch + 2 * nsb) * 2048
  uint32_t off_slots, off_tile, off_pbuf;
  int inflight;         // stages requested but not yet landed, at most
  uint32_t* status;     // may be null
  int early;            // weights, scales and biases may be read before the previous kernel ended
};

// One packed word -> NP registers of two bf16 subnormals each; register i holds fields (i, i + NP)
// of the word, scaled by 2^-133 and by the power of two in xscale<BITS>(i).
template <int BITS>
__device__ __forceinline__ void unpack_word(uint32_t w, uint32_t* P) {
  const uint32_t u = w >> 8;
  if constexpr (BITS == 4) {
    P[0] = w & 0x000F000Fu; P[1] = w & 0x00F000F0u; P[2] = u & 0x000F000Fu; P[3] = u & 0x00F000F0u;
  } else if constexpr (BITS == 8) {
    P[0] = w & 0x00FF00FFu; P[1] = u & 0x00FF00FFu;
  } else {
    P[0] = w & 0x00030003u; P[1] = w & 0x000C000Cu; P[2] = w & 0x00300030u; P[3] = w & 0x00C000C0u;
    P[4] = u & 0x00030003u; P[5] = u & 0x000C000Cu; P[6] = u & 0x00300030u; P[7] = u & 0x00C000C0u;
  }
}
// Binary places by which field i of a word sits above bit 0 of its byte: x pair i is scaled down by
// as many powers of two.
template <int BITS>
__host__ __device__ constexpr int field_shift(int i) {
  return BITS == 4 ? ((i & 1) ? 4 : 0) : (BITS == 8 ? 0 : 2 * (i & 3));
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

template <int BITS, int G, int MT>
__global__ void __launch_bounds__(kThreads, 1)
qmv_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                const __grid_constant__ CUtensorMap map_b, const RowsParams p) {
  using C = Cfg<BITS, G, MT>;
  constexpr int NGW = C::NGW, NP = C::NP, UG = C::UG, UW = C::UW, KW = C::KW;
  extern __shared__ __align__(1024) unsigned char smem[];
  // header: [0, 128) "stage landed" barriers | [128, 256) "stage consumed" barriers |
  //         [256, 288) "partial buffer free" barriers | 320: abort flag | [512, 1024) output tile
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full0 = smem_base, done0 = smem_base + 128, pfree0 = smem_base + 256;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 320);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
#ifdef B200Q_ROWS_PROFILE
  const long long rp_entry = clock64();
  if (lane == 0 && blockIdx.x < 160) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    g_rows_prof[blockIdx.x][warp][31] = (uint32_t)gt;
  }
#endif
#ifdef B200Q_ROWS_PROFILE
  if (tid == 0) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    const unsigned n = atomicAdd(&g_rows_launch_in, 1u);
    const unsigned id = (n / gridDim.x) & 63;
    if (n % gridDim.x == 0) g_rows_t[id][0] = gt;
    atomicMax(&g_rows_t[id][1], gt);
  }
#endif
  asm volatile("griddepcontrol.launch_dependents;");
  if (tid == kConsumers * 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_s) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }

  const int G_ = gridDim.x;
  const int b0 = (int)((long long)blockIdx.x * p.nblk8 / G_);
  const int b1 = (int)((long long)(blockIdx.x + 1) * p.nblk8 / G_);
  const int nrg = (b1 - b0 + 1) >> 1;           // 16-row groups of this CTA
  const int total = nrg * p.nph;                // stages
  const int row_end = min(b1 * 8, p.N);
  const int nst = p.nst;

  // Barriers are set up by the loader thread, which then starts requesting weights at once; the
  // other warps meet it at a named barrier (id 1) only when they first need the barriers - the
  // consumers after their x values are in registers.
  if (warp >= kConsumers) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsService));
    if (warp == kConsumers) {
      if (lane == 0) {
        for (int i = 0; i < nst; ++i) {
          mbar_init(full0 + 8 * i, 1);
          mbar_init(done0 + 8 * i, kConsumers);
        }
        for (int i = 0; i < kPartialBufs; ++i) mbar_init(pfree0 + 8 * i, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      }
      __syncwarp();
      asm volatile("bar.arrive 1, %0;" ::"n"(kThreads) : "memory");
      RP_MARK(1);
      // ================================= loader warp ==========================================
      // Without the caller's promise the weights may have been written by the previous kernel.
      if (!p.early) asm volatile("griddepcontrol.wait;" ::: "memory");
      RP_MARK(2);
      if (lane == 0) {
        // This one thread shares its scheduler with four busy consumer warps: everything it needs
        // per stage is kept incremental (no divisions, no parameter reloads).
        const uint32_t stage_bytes = p.slot_bytes, sb_off = (uint32_t)p.nch * 2048, bb_off = (uint32_t)(p.nch + p.nsb) * 2048;
#ifdef B200Q_ROWS_PROFILE
        const int dbg = p.inflight >> 8;
        const int nsb = (dbg & 1) ? 0 : p.nsb, inflight = p.inflight & 255;
        const uint32_t stage_bytes_dbg = (dbg & 1) ? (uint32_t)p.nch * 2048 : stage_bytes;
#define STAGE_TX stage_bytes_dbg
#else
        const int nsb = p.nsb, inflight = p.inflight;
#define STAGE_TX stage_bytes
#endif
        int slot = 0, use = 0;        // ring position of stage s
        int lslot = 0, luse = 0;      // ring position of the oldest stage not yet known to have landed
        int landed = 0, iph = 0, irg = 0;
        int grp0 = p.ph_g0[0];
        uint32_t dst = smem_base + p.off_slots;
        for (int s = 0; s < total; ++s) {
          // slot free: all consumer warps arrived for the stage that used it last
          if (use > 0 && !mbar_wait(done0 + 8 * slot, (use - 1) & 1, abort_flag)) break;
          // at most `inflight` stages outstanding
          while (landed < s && mbar_test(full0 + 8 * lslot, luse & 1)) {
            ++landed;
            if (++lslot == nst) { lslot = 0; ++luse; }
          }
          while (s - landed >= inflight) {
            if (!mbar_wait(full0 + 8 * lslot, luse & 1, abort_flag)) break;
            ++landed;
            if (++lslot == nst) { lslot = 0; ++luse; }
          }
          if (*abort_flag) break;
          const int row0 = (b0 + 2 * irg) * 8;
          const uint32_t bar = full0 + 8 * slot;
#ifdef B200Q_ROWS_PROFILE
          if (5 + 3 * s < 30 && blockIdx.x < 160) g_rows_prof[blockIdx.x][warp][5 + 3 * s] = (uint32_t)(clock64() - rp_entry);
#endif
          // rows past N and chunks past K are zero-filled by the copy engine and still counted
          mbar_expect_tx(bar, STAGE_TX);
          tma_load_3d(dst, &map_w, 0, row0, grp0 * (C::GB / 16) / 8, bar);
#ifdef B200Q_ROWS_PROFILE
          if (6 + 3 * s < 30 && blockIdx.x < 160) g_rows_prof[blockIdx.x][warp][6 + 3 * s] = (uint32_t)(clock64() - rp_entry);
#endif
          for (int i = 0; i < nsb; ++i) {
            tc::tma_load_2d(dst + sb_off + i * 2048, &map_s, grp0 * 2 + 128 * i, row0, bar);
            tc::tma_load_2d(dst + bb_off + i * 2048, &map_b, grp0 * 2 + 128 * i, row0, bar);
          }
#ifdef B200Q_ROWS_PROFILE
          if (7 + 3 * s < 30 && blockIdx.x < 160) g_rows_prof[blockIdx.x][warp][7 + 3 * s] = (uint32_t)(clock64() - rp_entry);
#endif
          dst += stage_bytes;
          if (++slot == nst) { slot = 0; ++use; dst = smem_base + p.off_slots; }
          if (++irg == nrg) { irg = 0; ++iph; grp0 = p.ph_g0[iph < p.nph ? iph : 0]; }
        }
      }
      RP_MARK(30);
    } else if (warp == kConsumers + 1) {
      // ================================= reducer warp =========================================
      // Adds the consumer warps' partial tiles of a finished stage in warp order, frees the
      // partial buffer, and stores y (or keeps running sums while K is walked in phases).
      asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
      asm volatile("griddepcontrol.wait;" ::: "memory");   // y may still be in use by the previous kernel
      if (lane == 0) peer_wait_previous(p.sig, p.status);  // ... or by a peer's consumer of the step before
      __syncwarp();
      int rph = 0, rrg = 0, rslot = 0, ruse = 0;
      for (int red = 0; red < total; ++red) {
        if (!mbar_wait(done0 + 8 * rslot, ruse & 1, abort_flag)) break;
        if (++rslot == nst) { rslot = 0; ++ruse; }
        RP_MARK(5 + 2 * red);
        const int pbi = red % kPartialBufs;
        const float4* pb = reinterpret_cast<const float4*>(smem + p.off_pbuf + (size_t)pbi * (kConsumers * MT * 512)) + lane;
        float sum[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int w = 0; w < kConsumers; w += 4) {   // four independent loads, then the additions in warp order
            const float4 v0 = pb[((w + 0) * MT + mt) * 32], v1 = pb[((w + 1) * MT + mt) * 32];
            const float4 v2 = pb[((w + 2) * MT + mt) * 32], v3 = pb[((w + 3) * MT + mt) * 32];
            acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
            acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
            acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
            acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
          }
          sum[mt][0] = acc.x; sum[mt][1] = acc.y; sum[mt][2] = acc.z; sum[mt][3] = acc.w;
        }
        __syncwarp();   // every lane holds its sums: the partial buffer may be written again
        if (lane == 0) tc::mbar_arrive(pfree0 + 8 * pbi);
        bool final_phase = true;
        if (p.nph > 1) {   // long K: running sums of this CTA's rows, touched by this warp only
          float4* tl = reinterpret_cast<float4*>(smem + p.off_tile + (size_t)rrg * (MT * 512)) + lane;
          final_phase = rph == p.nph - 1;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            if (rph > 0) {
              const float4 v = tl[mt * 32];
              sum[mt][0] += v.x; sum[mt][1] += v.y; sum[mt][2] += v.z; sum[mt][3] += v.w;
            }
            if (!final_phase) tl[mt * 32] = make_float4(sum[mt][0], sum[mt][1], sum[mt][2], sum[mt][3]);
          }
        }
        if (final_phase) {
          // transpose the 16 rows x 8*MT tokens through shared memory so that every lane stores 16
          // contiguous bytes of one token's row of y
          const int row0 = (b0 + 2 * rrg) * 8;
          __nv_bfloat16* yt = reinterpret_cast<__nv_bfloat16*>(smem + 512);   // [16 tokens][16 rows]
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c)
              yt[(mt * 8 + 2 * t + (c & 1)) * 16 + g + (c >> 1) * 8] = __float2bfloat16_rn(sum[mt][c]);
          __syncwarp();
          const int tok = lane >> 1, r8 = row0 + (lane & 1) * 8;
          if (tok < p.M && r8 < row_end) {
            const uint4 v = *reinterpret_cast<const uint4*>(yt + tok * 16 + (lane & 1) * 8);
            const long long at = (long long)tok * p.ld + p.col0 + r8;
            const bool vec = r8 + 8 <= row_end && ((at | p.ld) & 7) == 0;
            for (int q = 0; q < p.n_out; ++q) {
              __nv_bfloat16* dst = p.y[q] + at;
              if (vec && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                *reinterpret_cast<uint4*>(dst) = v;
              } else {
                const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
                for (int i = 0; i < 8 && r8 + i < row_end; ++i) dst[i] = e[i];
              }
            }
          }
          __syncwarp();
        }
        if (++rrg == nrg) { rrg = 0; ++rph; }
        RP_MARK(6 + 2 * red);
      }
      RP_MARK(30);
      __syncwarp();   // all of this block's stores to y were issued by this warp
      if (lane == 0) peer_signal_tail(p.sig);
#ifdef B200Q_ROWS_PROFILE
      if (lane == 0) {
        unsigned long long gt;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
        const unsigned n = atomicAdd(&g_rows_launch_out, 1u);
        const unsigned id = (n / gridDim.x) & 63;
        if (n % gridDim.x == 0) g_rows_t[id][2] = gt;
        atomicMax(&g_rows_t[id][3], gt);
      }
#endif
    } else {
      asm volatile("bar.arrive 1, %0;" ::"n"(kThreads) : "memory");   // idle companions of the service warps
    }
    if (warp == kConsumers && lane == 0 && *abort_flag && p.status) atomicMax(&p.status[0], 7u);
    return;
  }

  // ================================= consumer warps ===========================================
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsConsumer));
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (p.sig.wait_flag != nullptr && p.sig.wait_x) {   // x is the gathered output of the previous exchange step
    if (lane == 0) peer_wait_previous(p.sig, p.status);
    __syncwarp();
  }
  RP_MARK(2);
  uint32_t X[UW][MT][NP];         // B fragments of this warp's K slice, pre-scaled
  uint32_t sx_hi[MT], sx_lo[MT];  // scaled group sums of x for groups 2t, 2t+1 of the slice (bf16 hi / lo parts)
  float unscale[MT][2];           // per output token (2t, 2t+1 of tile mt): what brings the warp's sums back to true units / 2^69
  uint32_t woff[UW / 2];          // this lane's ldmatrix addresses inside a stage
  uint32_t soff = 0;              // scale of (row g, first group of the slice) inside a stage
  int cnt = 0;
  int ph = 0, rg = 0, slot = 0, use = 0, pbi = 0, pbe = 0;
  // ldmatrix roles of this lane: matrix m = lane / 8 covers rows (m & 1) * 8 .. +7 of unit (m >> 1)
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8, lm_unit = lane >> 4, lm_x = lane & 7;

  auto setup_phase = [&]() {
    cnt = p.ph_cnt[ph];
    const int g0 = warp * cnt;       // first group of this warp inside the phase
    const int u0 = g0 * UG;
#pragma unroll
    for (int j = 0; j < UW / 2; ++j) {
      const int U = u0 + 2 * j + lm_unit;
      woff[j] = (uint32_t)(U >> 3) * 2048 + lm_row * 128 + (((U & 7) ^ lm_x) << 4);
    }
    // scales: 128-byte rows, 16-byte units xor-ed with the row number mod 8; a warp's (at most 8)
    // groups lie inside one unit; the same entry of row g + 8 is 1024 bytes further on
    soff = (uint32_t)(p.nch + ((2 * g0) >> 7)) * 2048 + g * 128 + (((((2 * g0) >> 4) & 7) ^ g) << 4) + ((2 * g0) & 15);
    float sx[NGW][MT];
    float asum[MT];   // sum of |x| per token: an upper bound of the largest element that costs no integer operations
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      asum[mt] = 0.0f;
#pragma unroll
      for (int j = 0; j < NGW; ++j) sx[j][mt] = 0.0f;
    }
    // unit i of the slice: 4 * KW consecutive k, of which this lane owns KW starting at t * KW
    const long long k0 = (long long)(p.ph_g0[ph] + g0) * G + t * KW;
#pragma unroll
    for (int i = 0; i < UW; ++i) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int tok = mt * 8 + g;
        const bool live = i < cnt * UG && tok < p.M;
        const __nv_bfloat16* xp = p.x + (long long)tok * p.K + k0 + i * (4 * KW);
        // pair q = (x_q, x_{q + NP}), the order the unpack delivers the fields in
        if constexpr (BITS == 8) {
          uint2 v = make_uint2(0, 0);
          if (live) v = ldg_nc_u64(xp);
          sx[i / UG][mt] += sum_bf16x2(v.x) + sum_bf16x2(v.y);
          asum[mt] += asum_bf16x2(v.x) + asum_bf16x2(v.y);
          X[i][mt][0] = __byte_perm(v.x, v.y, 0x5410); X[i][mt][1] = __byte_perm(v.x, v.y, 0x7632);
        } else if constexpr (BITS == 4) {
          uint4 v = make_uint4(0, 0, 0, 0);
          if (live) v = ldg_nc_u128(xp);
          sx[i / UG][mt] += (sum_bf16x2(v.x) + sum_bf16x2(v.y)) + (sum_bf16x2(v.z) + sum_bf16x2(v.w));
          asum[mt] += (asum_bf16x2(v.x) + asum_bf16x2(v.y)) + (asum_bf16x2(v.z) + asum_bf16x2(v.w));
          X[i][mt][0] = __byte_perm(v.x, v.z, 0x5410); X[i][mt][1] = __byte_perm(v.x, v.z, 0x7632);
          X[i][mt][2] = __byte_perm(v.y, v.w, 0x5410); X[i][mt][3] = __byte_perm(v.y, v.w, 0x7632);
        } else {
          uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
          if (live) { a = ldg_nc_u128(xp); b = ldg_nc_u128(xp + 8); }
          sx[i / UG][mt] += (sum_bf16x2(a.x) + sum_bf16x2(a.y)) + (sum_bf16x2(a.z) + sum_bf16x2(a.w)) +
                            (sum_bf16x2(b.x) + sum_bf16x2(b.y)) + (sum_bf16x2(b.z) + sum_bf16x2(b.w));
          asum[mt] += (asum_bf16x2(a.x) + asum_bf16x2(a.y)) + (asum_bf16x2(a.z) + asum_bf16x2(a.w)) +
                      (asum_bf16x2(b.x) + asum_bf16x2(b.y)) + (asum_bf16x2(b.z) + asum_bf16x2(b.w));
          X[i][mt][0] = __byte_perm(a.x, b.x, 0x5410); X[i][mt][1] = __byte_perm(a.x, b.x, 0x7632);
          X[i][mt][2] = __byte_perm(a.y, b.y, 0x5410); X[i][mt][3] = __byte_perm(a.y, b.y, 0x7632);
          X[i][mt][4] = __byte_perm(a.z, b.z, 0x5410); X[i][mt][5] = __byte_perm(a.z, b.z, 0x7632);
          X[i][mt][6] = __byte_perm(a.w, b.w, 0x5410); X[i][mt][7] = __byte_perm(a.w, b.w, 0x7632);
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      // sum of |x| of token g over this warp's slice (lane's registers, then the quad): at least the
      // largest element, at most 128 times it
      float am = asum[mt];
      am += __shfl_xor_sync(0xFFFFFFFFu, am, 1);
      am += __shfl_xor_sync(0xFFFFFFFFu, am, 2);
      const uint32_t m = __float_as_uint(am);
      // E: x is multiplied by 2^E so that its largest element lands at or below 2^65
      int E = 191 - (int)((m >> 23) & 0xFF);
      E = E < -62 ? -62 : (E > 120 ? 120 : E);
      const uint32_t sc = (uint32_t)(127 + E) << 7;   // bf16 bits of 2^E
      const uint32_t sc2 = sc | (sc << 16);
#pragma unroll
      for (int i = 0; i < UW; ++i)
#pragma unroll
        for (int q = 0; q < NP; ++q)
          X[i][mt][q] = mul_bf16x2(X[i][mt][q], sc2 - (uint32_t)field_shift<BITS>(q) * 0x00800080u);
      // the weights come out as field * 2^-133: the sums of this token are true value * 2^(E - 133);
      // 2^(64 - E) is applied when the sums leave the warp, 2^69 with it
      const float un = __uint_as_float((uint32_t)(127 + 64 - E) << 23);
      unscale[mt][0] = __shfl_sync(0xFFFFFFFFu, un, (2 * t) * 4);
      unscale[mt][1] = __shfl_sync(0xFFFFFFFFu, un, (2 * t + 1) * 4);
      // group sums over the quad, in the same units; lane t keeps groups 2t and 2t+1 (the k slots it feeds)
      const float down = __uint_as_float((uint32_t)(127 + E - 64) << 23) * 0x1p-69f;
      float e0 = 0.0f, e1 = 0.0f;
#pragma unroll
      for (int j = 0; j < NGW; ++j) {
        float v = sx[j][mt];
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
        if ((j >> 1) == t) {
          if (j & 1) e1 = v; else e0 = v;
        }
      }
      e0 *= down; e1 *= down;
      const uint32_t hi = pack_bf16x2(e0, e1);
      sx_hi[mt] = hi;
      sx_lo[mt] = pack_bf16x2(e0 - bf16lo(hi), e1 - bf16hi(hi));
    }
  };
  setup_phase();
  asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");   // the barriers exist from here on
  {
    // The first mma.sync of a kernel is slow (the tensor pipe wakes up): issue one now, while the
    // first stage is in flight anyway.  Its result is never used.
    float d0, d1, d2, d3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%4,%4,%4}, {%4,%4}, {%5,%5,%5,%5};"
                 : "=f"(d0), "=f"(d1), "=f"(d2), "=f"(d3) : "r"(0u), "f"(0.0f));
  }
  RP_MARK(4);

  const uint32_t pb_mine = smem_base + p.off_pbuf + (uint32_t)(warp * MT * 32 + lane) * 16;
  uint32_t sb = smem_base + p.off_slots;   // stage the warp works on
  for (int s = 0; s < total; ++s) {
    if (!mbar_wait(full0 + 8 * slot, use & 1, abort_flag)) break;
    RP_MARK(5 + 3 * s);
    float out[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) out[mt][c] = 0.0f;
#ifdef B200Q_ROWS_PROFILE
    if (!((p.inflight >> 8) & 2))
#endif
    {
    // mma.sync results come back after many cycles: keep four independent accumulation chains going
    // per warp (two groups at a time, each group's k steps dealt round-robin to SPLIT accumulators,
    // MT token tiles).  A group past the warp's share (cnt < NGW) would multiply a neighbour's
    // bytes with x registers that are zero: it is skipped, pairs are whole because cnt is even or 1.
    constexpr int STEPS = UG * NP / 2;   // mma k steps per group
    constexpr int SPLIT = cmax(1, cmin(4 / (MT * 2), STEPS));
    const uint32_t sa = sb + soff;
#pragma unroll
    for (int gq = 0; gq < NGW; gq += 2) {
      if (gq < cnt) {
        // packed words: lane (g, t) gets word t of unit i for rows g (wl) and g + 8 (wh)
        uint32_t wl[2 * UG], wh[2 * UG];
#pragma unroll
        for (int i = 0; i < 2 * UG; i += 2) ldmatrix_x4(sb + woff[(gq * UG + i) / 2], wl[i], wh[i], wl[i + 1], wh[i + 1]);
        float acc[2][MT][SPLIT][4];
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int q = 0; q < SPLIT; ++q)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[u][mt][q][c] = 0.0f;
#pragma unroll
        for (int iu = 0; iu < UG; ++iu) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            uint32_t Pl[NP], Ph[NP];
            unpack_word<BITS>(wl[u * UG + iu], Pl);
            unpack_word<BITS>(wh[u * UG + iu], Ph);
#pragma unroll
            for (int st = 0; st < NP / 2; ++st)
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
                mma_bf16(acc[u][mt][(iu * (NP / 2) + st) % SPLIT], Pl[2 * st], Ph[2 * st], Pl[2 * st + 1], Ph[2 * st + 1],
                         X[(gq + u) * UG + iu][mt][2 * st], X[(gq + u) * UG + iu][mt][2 * st + 1]);
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          // a group beyond cnt (cnt == 1) contributes acc == 0 times a finite neighbour's scale
          const float s_l = __uint_as_float(lds_u16(sa + 2 * (gq + u)) << 16);
          const float s_h = __uint_as_float(lds_u16(sa + 1024 + 2 * (gq + u)) << 16);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int q = 1; q < SPLIT; ++q)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[u][mt][0][c] += acc[u][mt][q][c];
            out[mt][0] = fmaf(s_l, acc[u][mt][0][0], out[mt][0]);
            out[mt][1] = fmaf(s_l, acc[u][mt][0][1], out[mt][1]);
            out[mt][2] = fmaf(s_h, acc[u][mt][0][2], out[mt][2]);
            out[mt][3] = fmaf(s_h, acc[u][mt][0][3], out[mt][3]);
          }
        }
      }
    }
    // biases: b_g * sum_k x_k through one MMA, k slots 2t, 2t+1 (hi part of the sum) / +8 (lo part)
    {
      uint32_t bl = 0, bh = 0;
      const uint32_t ba = sa + (uint32_t)p.nsb * 2048;
      if (cnt >= 2) {
        if (2 * t < cnt) { bl = lds_u32(ba + 4 * t); bh = lds_u32(ba + 1024 + 4 * t); }
      } else if (t == 0) {
        bl = lds_u16(ba); bh = lds_u16(ba + 1024);
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) mma_bf16(out[mt], bl, bh, bl, bh, sx_hi[mt], sx_lo[mt]);
    }
    }
    RP_MARK(6 + 3 * s);
    // the partial buffer of this stage was read by the reducer kPartialBufs stages ago
    if (pbe > 0 && !mbar_wait(pfree0 + 8 * pbi, (pbe - 1) & 1, abort_flag)) break;
    {
      const uint32_t pa = pb_mine + (uint32_t)pbi * (kConsumers * MT * 512);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)   // back to true units on the way out (two exact multiplications)
        asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(pa + mt * 512),
                     "f"(out[mt][0] * 0x1p69f * unscale[mt][0]), "f"(out[mt][1] * 0x1p69f * unscale[mt][1]),
                     "f"(out[mt][2] * 0x1p69f * unscale[mt][0]), "f"(out[mt][3] * 0x1p69f * unscale[mt][1]) : "memory");
    }
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(done0 + 8 * slot);   // release: the partial tile is visible to the reducer
    RP_MARK(7 + 3 * s);
    // advance to the next stage
    sb += p.slot_bytes;
    if (++slot == nst) { slot = 0; ++use; sb = smem_base + p.off_slots; }
    if (++pbi == kPartialBufs) { pbi = 0; ++pbe; }
    if (++rg == nrg) {
      rg = 0;
      ++ph;
      if (ph < p.nph) setup_phase();
    }
  }
  RP_MARK(30);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn rows_encode_fn() {
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
  if (groups % kConsumers != 0) return false;   // every phase gives all 16 warps the same number of groups
  // phases of 16 * c groups, c a power of two: first as many full ones as fit, then the remainder
  p.nph = 0;
  for (int g0 = 0, rem = groups; rem > 0;) {
    int c = C::NGW;
    while (kConsumers * c > rem) c >>= 1;
    if (p.nph == kMaxPhases) return false;
    p.ph_g0[p.nph] = g0;
    p.ph_cnt[p.nph] = c;
    ++p.nph;
    g0 += kConsumers * c;
    rem -= kConsumers * c;
  }
  p.nch = kConsumers * C::NGW * C::GB / 128;          // box of a full phase
  p.nsb = (kConsumers * C::NGW * 2 + 127) / 128;
  if (p.nch > 256) return false;
  p.slot_bytes = (uint32_t)(p.nch + 2 * p.nsb) * 2048;
  p.nblk8 = (int)((a.N + 7) / 8);
  const int sms = sm_count_rows();
  pl.grid = p.nblk8 < sms ? p.nblk8 : sms;
  const int max_blk = (p.nblk8 + pl.grid - 1) / pl.grid;
  const int max_rg = (max_blk + 1) / 2 + 1;
  size_t off = 1024;   // barriers, abort flag, the reducer's 512-byte output tile
  p.off_tile = (uint32_t)off;
  if (p.nph > 1) off += (size_t)max_rg * MT * 512;
  p.off_pbuf = (uint32_t)off;
  off += (size_t)kPartialBufs * kConsumers * MT * 512;
  off = (off + 1023) / 1024 * 1024;   // swizzled tiles repeat every 1024 bytes
  p.off_slots = (uint32_t)off;
  if (off + 2 * (size_t)p.slot_bytes > kSmemLimit) return false;
  const long long stages = (long long)max_rg * p.nph;
  long long nst = (long long)((kSmemLimit - off) / p.slot_bytes);
  if (nst > 16) nst = 16;
  if (nst > stages) nst = stages;
  if (nst < 1) nst = 1;
  p.nst = (int)nst;
  pl.smem = off + (size_t)p.nst * p.slot_bytes;
  pl.mt = MT;
  return true;
}

RowsPlan make_plan(const QmmArgs& a) {
  RowsPlan pl{};
  pl.ok = false;
  if (a.dtype != B200Q_BF16 || !a.transpose || a.w_batched || a.batch != 1) return pl;
  if (a.M < 1 || a.M > 16 || a.N < 1 || a.K < 1) return pl;
  if (a.bits != 2 && a.bits != 4 && a.bits != 8) return pl;
  if (a.bits == 2 && a.group == 32) return pl;   // a group would be half a 16-byte unit
  if (a.K % (16 * a.group) != 0) return pl;       // 16 warps, whole groups each (implies 128-byte row chunks)
  if (a.N > (1ll << 30)) return pl;
  const int mt = a.M > 8 ? 2 : 1;
  bool ok = false;
#define B200Q_ROWS_CASE(BITS_, G_)                                                          \
  if (a.bits == BITS_ && a.group == G_)                                                     \
    ok = mt == 2 ? fill_plan<BITS_, G_, 2>(a, pl) : fill_plan<BITS_, G_, 1>(a, pl);
  B200Q_ROWS_CASE(2, 64) B200Q_ROWS_CASE(2, 128)
  B200Q_ROWS_CASE(4, 32) B200Q_ROWS_CASE(4, 64) B200Q_ROWS_CASE(4, 128)
  B200Q_ROWS_CASE(8, 32) B200Q_ROWS_CASE(8, 64) B200Q_ROWS_CASE(8, 128)
#undef B200Q_ROWS_CASE
  if (!ok) return pl;
  RowsParams& p = pl.prm;
  p.x = (const __nv_bfloat16*)a.x;
  if (a.peers.n > 0) {
    p.n_out = a.peers.n; p.ld = a.peers.ld; p.col0 = a.peers.col0;
    for (int q = 0; q < a.peers.n; ++q) p.y[q] = (__nv_bfloat16*)a.peers.y[q];
    p.sig = a.peers.sig;
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

// Stages the loader keeps in flight per SM.  More requests in flight dilute the first stage's arrival,
// which is what the kernel waits for at its start; fewer starve a stream that is bound by HBM.
// Measured (us per call, in flight = 1 / 2 / 3): M=16 14336x4096 4-bit 14.4 / 14.8 / 15.2; M=1
// 4096x14336 4-bit 15.2 / 15.8 / 15.7; M=1 8192x28672 4-bit 35.8 / 36.9 / 36.9; M=1 28672x8192 4-bit
// 28.5 / 28.5 / 28.5; M=1 28672x8192 8-bit 48.1 / 45.9 / 45.6; M=16 28672x8192 8-bit 53.5 / 52.8 / 52.7:
// one for 2- and 4-bit weights, two for 8-bit (twice the bytes per stage, the stream closest to the
// HBM bound).  B200Q_ROWS_INFLIGHT overrides (tuning).
int rows_inflight(int mt, int bits, int nph) {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200Q_ROWS_INFLIGHT");
    v = e ? atoi(e) : 0;
    if (v < 0) v = 0;
  }
  if (v > 0) return v;
  (void)mt; (void)nph;
  return bits >= 8 ? 2 : 1;
}

template <int BITS, int G, int MT>
int launch_rows(const QmmArgs& a, const RowsPlan& pl, cudaStream_t st) {
  EncodeFn enc = rows_encode_fn();
  if (!enc) return fail(B200Q_ERR_CUDA, "[quantized_matmul] cuTensorMapEncodeTiled is not available");
  const RowsParams& p = pl.prm;
  CUtensorMap map_w, map_s, map_b;
  {
    // packed rows as (128 bytes, row, 128-byte chunk of the row)
    const cuuint64_t row_bytes = (cuuint64_t)a.K * BITS / 8;
    const cuuint64_t dims[3] = {128, (cuuint64_t)a.N, row_bytes / 128};
    const cuuint64_t strides[2] = {row_bytes, 128};
    const cuuint32_t box[3] = {128, 16, (cuuint32_t)p.nch};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint32_t*>(a.wq), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_CUDA, "[quantized_matmul] tensor map for the packed weights failed (%d)", (int)r);
  }
  for (int which = 0; which < 2; ++which) {
    const cuuint64_t srow = (cuuint64_t)(a.K / G) * 2;
    const cuuint64_t dims[2] = {srow, (cuuint64_t)a.N};
    const cuuint64_t strides[1] = {srow};
    const cuuint32_t box[2] = {128, 16};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(which ? &map_b : &map_s, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(which ? a.biases : a.scales),
                     dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_CUDA, "[quantized_matmul] tensor map for scales / biases failed (%d)", (int)r);
  }
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
  B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, map_w, map_s, map_b, pl.prm));
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

// 17 to 32 token rows run as two passes of up to 16 rows each: the second pass finds the matrix
// in L2 when it fits, and both passes together stay below the tensor-memory kernel's cost of
// unpacking a 128-row tile.  Sharded output (peer buffers, completion signal) stays single-pass.
static bool two_pass(const QmmArgs& a) { return a.M > 16 && a.M <= 32 && a.peers.n == 0; }

static QmmArgs pass_args(const QmmArgs& a, int64_t row0, int64_t rows) {
  QmmArgs h = a;
  h.M = rows;
  h.x = static_cast<const char*>(a.x) + (size_t)row0 * a.K * 2;
  h.y = static_cast<char*>(a.y) + (size_t)row0 * a.N * 2;
  return h;
}

bool qmv_rows_supported(const QmmArgs& a) {
  if (two_pass(a)) {
    if ((a.K * 2) % 16 != 0 || (a.N * 2 * 16) % 16 != 0) return false;
    return qmv_rows_supported(pass_args(a, 0, 16)) && qmv_rows_supported(pass_args(a, 16, a.M - 16));
  }
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.wq) |
                       reinterpret_cast<uintptr_t>(a.scales) | reinterpret_cast<uintptr_t>(a.biases);
  if (al & 15) return false;
  return make_plan(a).ok;
}

int qmv_rows(const QmmArgs& a, cudaStream_t st) {
  if (two_pass(a)) {
    const int rc = qmv_rows(pass_args(a, 0, 16), st);
    return rc != B200Q_OK ? rc : qmv_rows(pass_args(a, 16, a.M - 16), st);
  }
  RowsPlan pl = make_plan(a);
  if (!pl.ok) return fail(B200Q_ERR_UNSUPPORTED, "[quantized_matmul] qmv_rows: unsupported problem");
  pl.prm.early = weights_constant() ? 1 : 0;
  pl.prm.inflight = rows_inflight(pl.mt, a.bits, pl.prm.nph);
  if (a.ws && a.ws_bytes >= kStatusBytes)
    pl.prm.status = reinterpret_cast<uint32_t*>(static_cast<char*>(a.ws) + a.ws_bytes - kStatusBytes);
  int rc = B200Q_ERR_UNSUPPORTED;
#define B200Q_ROWS_CASE(BITS_, G_)                                                                  \
  if (a.bits == BITS_ && a.group == G_)                                                             \
    rc = pl.mt == 2 ? launch_rows<BITS_, G_, 2>(a, pl, st) : launch_rows<BITS_, G_, 1>(a, pl, st);
  B200Q_ROWS_CASE(2, 64) B200Q_ROWS_CASE(2, 128)
  B200Q_ROWS_CASE(4, 32) B200Q_ROWS_CASE(4, 64) B200Q_ROWS_CASE(4, 128)
  B200Q_ROWS_CASE(8, 32) B200Q_ROWS_CASE(8, 64) B200Q_ROWS_CASE(8, 128)
#undef B200Q_ROWS_CASE
  return rc;
}

}  // namespace b200q
