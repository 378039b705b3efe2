// Decode path on the 5th-generation tensor cores: y[M<=16, N] = x[M, K] * dequant(W[N, K])^T,
// 4-bit weights, bf16, HBM-bound.
//
// Replaces cu::qmv_kernel and the small-M use of cu::qmm_sm80_kernel of the reference
// (mlx/backend/cuda/quantized/qmm/qmv.cu:84-209, quantized/quantized.cpp:106-136).
//
// The per-weight work of a warp-level (mma.sync) decode kernel is dominated by fragment
// plumbing.  Here the multiply-accumulate of a whole 128-row block is one instruction
// issued by one thread, and the rest of the CTA only moves bits:
//
//   producer (1 thread)   TMA boxes [128 rows x 128 B] of packed W (256 k, 128B-swizzled)
//                         into a 5-deep shared-memory ring: 80 KB in flight per SM
//   dequant (16 warps)    thread = weight row = TMEM lane: shift+lop3 turns each 4-bit field
//                         into the bf16 integer 128+q (no scale, no bias, no byte shuffles)
//                         and tcgen05.st writes one quantization group into the A ring
//   MMA (1 thread)        per group: tcgen05.mma M=128, N=16 tokens, K=16 x (group/16), into a
//                         fresh 16-column fp32 accumulator slot (16 slots)
//   fix-up (4 warps)      thread = weight row: tcgen05.ld the slot, then in fp32
//                         acc[t] += s * slot[t] + (b - 128 s) * X[group][t]
//                         where X holds the group sums of x.  Exact up to fp32 summation.
//
// x is staged once per CTA as the B operand (K-major, 128B swizzle) with the k order inside
// every 8-element chunk permuted to (0,4,1,5,2,6,3,7), the order in which the lop3 unpack
// produces bf16 pairs, so the weights never need a byte permute.
//
// Work decomposition: units of (128-row block, 256 k); every CTA owns a contiguous span of
// units (row-block major), so all SMs stream the same number of bytes whatever N is.  Row
// blocks completed inside one CTA are stored directly; for the others every contributing CTA
// stores its partial tile into its own scratch slot and bumps an arrival counter; the last
// arriver adds the slots in CTA order (deterministic) and writes y.  No CTA waits on another; every mbarrier wait is bounded.
#include "common.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace b200q {
namespace {

using namespace tc;

constexpr int kRows = 128;
constexpr int kChunkK = 256;
constexpr int kBoxBytes = kRows * 128;  // 16 KB
constexpr int kStagesW = 5;
constexpr int kTmemCols = 512;
constexpr int kACol0 = 256;             // A ring: columns [256, 512)
constexpr int kAccSlots = 16;           // accumulator slots of 16 columns: [0, 256)
constexpr int kWarps = 24;
constexpr int kThreads = kWarps * 32;
constexpr int kDequantWarp0 = 4, kDequantWarps = 16, kDequantSets = kDequantWarps / 4;
constexpr int kFixWarp0 = 20, kFixWarps = 4;

__device__ __forceinline__ void tcgen05_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
      "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tcgen05_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fix_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kFixWarps * 32) : "memory"); }

// K-major, 128-byte-swizzled B operand of 16 token rows (two 8-row groups 1024 B apart).
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D f32, A/B bf16 K-major, M = 128, N = 16.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

struct QtcParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* scales;
  const __nv_bfloat16* biases;
  __nv_bfloat16* y;
  uint32_t* counters;   // [n_tiles]
  float* partial;       // [grid][2][128][16]: per-CTA slots for row blocks shared with a neighbour
  uint32_t* status;
  int M, N, K;
  int n_tiles, chunks;  // row blocks, 256-k chunks per row
  long long total_units;
};

struct __align__(8) QtcBarriers {
  uint64_t full_w[kStagesW], empty_w[kStagesW];
  uint64_t full_a[16];                      // one per A stage (4 dequant warps arrive)
  uint64_t empty_a[8];                      // one per PAIR of A stages (one commit)
  uint64_t full_acc[kAccSlots / 2];         // one per PAIR of accumulator slots (one commit)
  uint64_t empty_acc[kAccSlots / 2];        // one per pair (4 fix-up warps arrive)
  uint32_t tmem_base;
  int abort_flag;
  int is_last[2];
};

template <int GROUP>
__global__ void __launch_bounds__(kThreads, 1)
qmv_tc_kernel(const __grid_constant__ CUtensorMap map_w, const QtcParams p) {
  constexpr int GPC = kChunkK / GROUP;     // groups per chunk: 8 / 4 / 2
  constexpr int AC = GROUP / 2;            // A columns per group: 16 / 32 / 64
  constexpr int SA = 256 / AC;             // A ring stages: 16 / 8 / 4
  constexpr int MMAS = GROUP / 16;         // K=16 MMAs per group
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int kblocks = p.K / 64;            // 64-k blocks of the B operand (2 KB each)
  const int groups_k = p.K / GROUP;
  unsigned char* xs = smem;                                           // [kblocks][16 rows][128 B] swizzled
  unsigned char* ring_w = xs + (size_t)kblocks * 2048;                // kStagesW boxes
  float* Xs = reinterpret_cast<float*>(ring_w + (size_t)kStagesW * kBoxBytes);  // [groups_k][16]
  QtcBarriers* bars = reinterpret_cast<QtcBarriers*>(Xs + (size_t)groups_k * 16);
  volatile int* abort_flag = &bars->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef B200Q_PROFILE
  const long long prof_entry = clock64();
#define QTC_MARK(slot) if (blockIdx.x == 0 && lane == 0) p.status[slot] = (uint32_t)(clock64() - prof_entry)
  uint32_t* dbg = p.status - 64;
  long long pw0 = 0, pw1 = 0, pw2 = 0, pt;
#define QTC_T0() pt = clock64()
#define QTC_ACC(v) v += clock64() - pt
#define QTC_OUT(slot, v) if (blockIdx.x == 0 && lane == 0) dbg[slot] = (uint32_t)(v)
#else
#define QTC_MARK(slot)
#define QTC_T0()
#define QTC_ACC(v)
#define QTC_OUT(slot, v)
#endif
  const long long T = p.total_units;
  const int G = gridDim.x;
  const int u0 = (int)((long long)blockIdx.x * T / G), u1 = (int)((long long)(blockIdx.x + 1) * T / G);

  if (tid == 0) {
    for (int i = 0; i < kStagesW; ++i) { mbar_init(smem_u32(&bars->full_w[i]), 1); mbar_init(smem_u32(&bars->empty_w[i]), kDequantWarps); }
    for (int i = 0; i < 16; ++i) mbar_init(smem_u32(&bars->full_a[i]), 4);
    for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&bars->empty_a[i]), 1);
    for (int i = 0; i < kAccSlots / 2; ++i) { mbar_init(smem_u32(&bars->full_acc[i]), 1); mbar_init(smem_u32(&bars->empty_acc[i]), kFixWarps); }
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
  if (warp == 0) QTC_MARK(0);

  // The weight stream starts before x is staged.
  auto issue_box = [&](int u) {
    const int sw = (u - u0) % kStagesW;
    const int tile = u / p.chunks, chunk = u - tile * p.chunks;
    mbar_expect_tx(smem_u32(&bars->full_w[sw]), kBoxBytes);
    tma_load_2d(smem_u32(ring_w + sw * kBoxBytes), &map_w, chunk * 128, tile * kRows, smem_u32(&bars->full_w[sw]));
  };
  if (warp == 0 && lane == 0)
    for (int u = u0; u < u1 && u < u0 + kStagesW; ++u) issue_box(u);

  // ---- stage x as the B operand (permuted chunks, manual 128B swizzle) and its group sums.
  // Warp w stages token w: lane = (64-k block mod 4, 16-byte chunk); the eight lanes of a block
  // reduce the block's sum with shuffles (no atomics), groups of 128 add the neighbouring block.
  {
    const int t = warp;            // token row: warps 0..15 stage the 16 rows of the B operand
    const int c = lane & 7, ob = lane >> 3;
    constexpr int XU = 8;  // loads in flight per lane
    for (int kb0 = 0; t < 16 && kb0 < kblocks; kb0 += 4 * XU) {
      uint4 v[XU];
#pragma unroll
      for (int i = 0; i < XU; ++i) {
        const int kb = kb0 + 4 * i + ob;
        v[i] = make_uint4(0, 0, 0, 0);
        if (t < p.M && kb < kblocks) v[i] = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)t * p.K + kb * 64 + c * 8));
      }
#pragma unroll
      for (int i = 0; i < XU; ++i) {
        const int kb = kb0 + 4 * i + ob;  // kblocks is a multiple of 4: uniform per warp
        if (kb0 + 4 * i >= kblocks) break;
        uint4 o;
        o.x = __byte_perm(v[i].x, v[i].z, 0x5410);  // (x0, x4)
        o.y = __byte_perm(v[i].x, v[i].z, 0x7632);  // (x1, x5)
        o.z = __byte_perm(v[i].y, v[i].w, 0x5410);  // (x2, x6)
        o.w = __byte_perm(v[i].y, v[i].w, 0x7632);  // (x3, x7)
        *reinterpret_cast<uint4*>(xs + (size_t)kb * 2048 + t * 128 + ((c ^ (t & 7)) << 4)) = o;
        float sum = 0.0f;
        const uint32_t w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) sum += __uint_as_float(w4[q] << 16) + __uint_as_float(w4[q] & 0xFFFF0000u);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);       // 32-k half block
        if (GROUP >= 64) sum += __shfl_xor_sync(0xffffffffu, sum, 4);   // 64-k block
        if (GROUP >= 128) sum += __shfl_xor_sync(0xffffffffu, sum, 8);  // blocks kb, kb^1 (lanes ob, ob^1)
        const int k = kb * 64 + c * 8;
        const bool writer = GROUP == 32 ? (c & 3) == 0 : (GROUP == 64 ? c == 0 : (c == 0 && (ob & 1) == 0));
        if (writer) Xs[(k / GROUP) * 16 + t] = sum;
      }
    }
    fence_proxy_async_smem();  // the MMA reads xs through the async proxy
  }
  __syncthreads();
  if (warp == 0) QTC_MARK(1);

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      for (int u = u0 + kStagesW; u < u1; ++u) {
        const int i = u - u0, sw = i % kStagesW;
        if (!mbar_wait(smem_u32(&bars->empty_w[sw]), ((i / kStagesW) & 1) ^ 1, abort_flag)) break;
        issue_box(u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // Accumulating MMAs on one slot are dependent and, at N = 16, far shorter than the
      // pipeline is deep: groups are therefore issued in batches, k-slice by k-slice, so
      // that consecutive instructions work on different accumulator slots.
      // Groups are issued in pairs, k-slice by k-slice (consecutive instructions work on
      // different accumulator slots), and one commit per pair releases both A stages / publishes
      // both slots.  The span always holds an even number of groups (GPC is even).
      const uint32_t xs_addr = smem_u32(xs);
      const uint32_t n_pairs = (uint32_t)(u1 - u0) * GPC / 2;
      int chunk = u0 < u1 ? u0 % p.chunks : 0, j = 0;  // position of the next group
      bool ok = true;
      for (uint32_t pi = 0; ok && pi < n_pairs; ++pi) {
        uint32_t dcol[2], acol[2];
        uint64_t bdesc[2];
        const uint32_t sa2 = pi % (SA / 2), sc2 = pi % (kAccSlots / 2);
        QTC_T0();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t gi = 2 * pi + i;
          const uint32_t sa = gi % SA, sc = gi % kAccSlots;
          dcol[i] = tmem_base + sc * 16;
          acol[i] = tmem_base + kACol0 + sa * AC;
          const int k0 = chunk * kChunkK + j * GROUP;
          bdesc[i] = make_sw128_desc(xs_addr + (k0 >> 6) * 2048 + ((k0 >> 4) & 3) * 32);
          if (++j == GPC) { j = 0; if (++chunk == p.chunks) chunk = 0; }
          if (ok && !mbar_wait(smem_u32(&bars->full_a[sa]), (gi / SA) & 1, abort_flag)) ok = false;
        }
        if (ok && !mbar_wait(smem_u32(&bars->empty_acc[sc2]), ((pi / (kAccSlots / 2)) & 1) ^ 1, abort_flag)) ok = false;
        QTC_ACC(pw0);
        if (!ok) break;
        tcgen05_fence_after();
        QTC_T0();
#pragma unroll
        for (int kk = 0; kk < MMAS; ++kk) {
          // descriptor advance: 32 bytes per 16-k slice, 2048 bytes per 64-k block (16-byte units)
          const uint64_t adv = (uint64_t)(((kk >> 2) * 2048 + (kk & 3) * 32) >> 4);
          tcgen05_mma_ts(dcol[0], acol[0] + kk * 8, bdesc[0] + adv, kIdesc, kk != 0 ? 1u : 0u);
          tcgen05_mma_ts(dcol[1], acol[1] + kk * 8, bdesc[1] + adv, kIdesc, kk != 0 ? 1u : 0u);
        }
        QTC_ACC(pw1);
        QTC_T0();
        tcgen05_commit(smem_u32(&bars->empty_a[sa2]));
        tcgen05_commit(smem_u32(&bars->full_acc[sc2]));
        QTC_ACC(pw2);
      }
      QTC_OUT(3, pw2);
      QTC_OUT(0, pw0);
      QTC_OUT(1, pw1);
      QTC_OUT(2, clock64() - prof_entry);
    }
  } else if (warp >= kDequantWarp0 && warp < kDequantWarp0 + kDequantWarps) {
    // ------------------------------------------------------------ dequant: thread = weight row
    const int quad = warp & 3, set = (warp - kDequantWarp0) >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
    const uint32_t swz = (uint32_t)(r & 7);
    bool pending = false, ok = true;
    uint32_t pending_sa = 0;
    auto publish = [&]() {
      tcgen05_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->full_a[pending_sa]));
      pending = false;
    };
    uint32_t gi = 0;
    for (int u = u0; ok && u < u1; ++u) {
      const int i = u - u0, sw = i % kStagesW;
      QTC_T0();
      if (!mbar_wait(smem_u32(&bars->full_w[sw]), (i / kStagesW) & 1, abort_flag)) { ok = false; break; }
      QTC_ACC(pw0);
      const unsigned char* row = ring_w + sw * kBoxBytes + r * 128;
#pragma unroll 1
      for (int j = 0; j < GPC; ++j, ++gi) {
        if ((int)(gi % kDequantSets) != set) continue;
        const uint32_t sa = gi % SA;
        constexpr int PIECES = GROUP > 64 ? GROUP / 64 : 1;
        constexpr int PW = (GROUP > 64 ? 64 : GROUP) / 8;  // words per piece: 4 or 8
#pragma unroll
        for (int pc = 0; pc < PIECES; ++pc) {
          uint32_t w[PW];
#pragma unroll
          for (int h = 0; h < PW / 4; ++h) {
            const uint32_t c16 = (uint32_t)(j * (GROUP / 32) + pc * 2 + h);  // 16-byte chunk of the row
            const uint4 v = *reinterpret_cast<const uint4*>(row + ((c16 ^ swz) << 4));
            w[4 * h + 0] = v.x; w[4 * h + 1] = v.y; w[4 * h + 2] = v.z; w[4 * h + 3] = v.w;
          }
          uint32_t vals[PW * 4];
#pragma unroll
          for (int q = 0; q < PW; ++q)
#pragma unroll
            for (int e = 0; e < 4; ++e) vals[4 * q + e] = lop3_and_or(w[q] >> (4 * e), 0x000F000Fu, 0x43004300u);
          if (pc == 0) {
            QTC_T0();
            if (pending) publish();
            QTC_ACC(pw1);
            QTC_T0();
            if (!mbar_wait(smem_u32(&bars->empty_a[sa >> 1]), ((gi / SA) & 1) ^ 1, abort_flag)) { ok = false; break; }
            QTC_ACC(pw2);
            tcgen05_fence_after();
          }
          const uint32_t taddr = tmem_base + lane_field + kACol0 + sa * AC + pc * 32;
          if constexpr (PW == 8) {
            tcgen05_st_x32(taddr, vals);
          } else {
            tcgen05_st_x16(taddr, vals);
          }
        }
        if (!ok) break;
        pending = true;
        pending_sa = sa;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->empty_w[sw]));
    }
    if (pending) publish();
    if (warp == kDequantWarp0) { QTC_OUT(4, pw0); QTC_OUT(5, pw1); QTC_OUT(6, pw2); QTC_OUT(7, clock64() - prof_entry); }
  } else if (warp >= kFixWarp0) {
    // ------------------------------------------------------------ fix-up / epilogue: thread = weight row
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int ftid = (warp - kFixWarp0) * 32 + lane;
    const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
    float acc[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) acc[t] = 0.0f;
    // Row blocks this CTA shares with a neighbour (known up front, identical in all threads,
    // so the named barriers below are reached by all fix-up threads whatever happens).
    int shared_tiles[2];
    int n_shared = 0;
    if (u0 < u1) {
      const int t_first = u0 / p.chunks, t_last = (u1 - 1) / p.chunks;
      if (u0 % p.chunks != 0 || u1 < (t_first + 1) * p.chunks) shared_tiles[n_shared++] = t_first;
      if (t_last != t_first && u1 % p.chunks != 0) shared_tiles[n_shared++] = t_last;
    }
    uint32_t gi = 0;
    bool ok = true;
    int seg_c0 = u0 < u1 ? u0 % p.chunks : 0;  // first chunk of the running row-block segment
    // scales / biases of one unit (GPC consecutive groups of this thread's row), one unit ahead
    struct Raw { uint32_t s[GPC], b[GPC]; };
    auto load_raw = [&](int u) {
      Raw rw;
      const int tile = u / p.chunks, chunk = u - tile * p.chunks;
      int row = tile * kRows + r;
      row = row < p.N ? row : p.N - 1;
      const size_t gidx = (size_t)row * groups_k + chunk * GPC;
      const unsigned short* sp = reinterpret_cast<const unsigned short*>(p.scales) + gidx;
      const unsigned short* bp = reinterpret_cast<const unsigned short*>(p.biases) + gidx;
      uint32_t sw_[GPC / 2], bw_[GPC / 2];
      if constexpr (GPC == 2) {
        sw_[0] = __ldg(reinterpret_cast<const uint32_t*>(sp));
        bw_[0] = __ldg(reinterpret_cast<const uint32_t*>(bp));
      } else if constexpr (GPC == 4) {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(sp)), c2 = __ldg(reinterpret_cast<const uint2*>(bp));
        sw_[0] = a.x; sw_[1] = a.y; bw_[0] = c2.x; bw_[1] = c2.y;
      } else {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(sp)), c4 = __ldg(reinterpret_cast<const uint4*>(bp));
        sw_[0] = a.x; sw_[1] = a.y; sw_[2] = a.z; sw_[3] = a.w;
        bw_[0] = c4.x; bw_[1] = c4.y; bw_[2] = c4.z; bw_[3] = c4.w;
      }
#pragma unroll
      for (int j = 0; j < GPC; ++j) {
        rw.s[j] = (j & 1) ? (sw_[j >> 1] & 0xFFFF0000u) : (sw_[j >> 1] << 16);
        rw.b[j] = (j & 1) ? (bw_[j >> 1] & 0xFFFF0000u) : (bw_[j >> 1] << 16);
      }
      return rw;
    };
    Raw nxt;
    if (u0 < u1) nxt = load_raw(u0);
    for (int u = u0; ok && u < u1; ++u) {
      const int tile = u / p.chunks, chunk = u - tile * p.chunks;
      const Raw cur = nxt;
      if (u + 1 < u1) nxt = load_raw(u + 1);
      float sv[GPC], cv[GPC];
#pragma unroll
      for (int j = 0; j < GPC; ++j) {
        sv[j] = __uint_as_float(cur.s[j]);
        cv[j] = fmaf(-128.0f, sv[j], __uint_as_float(cur.b[j]));
      }
#pragma unroll
      for (int j = 0; j < GPC; ++j, ++gi) {
        const uint32_t sc = gi % kAccSlots;
        QTC_T0();
        if ((j & 1) == 0) {  // slots are published in pairs
          if (!mbar_wait(smem_u32(&bars->full_acc[sc >> 1]), (gi / kAccSlots) & 1, abort_flag)) { ok = false; break; }
        }
        QTC_ACC(pw0);
        tcgen05_fence_after();
        uint32_t v[16];
        QTC_T0();
        tcgen05_ld_x16(tmem_base + lane_field + sc * 16, v);
        tcgen05_wait_ld();
        QTC_ACC(pw1);
        if (j & 1) {
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars->empty_acc[sc >> 1]));
        }
        const float4* xg = reinterpret_cast<const float4*>(Xs + (size_t)(chunk * GPC + j) * 16);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 xv = xg[q];
          acc[4 * q + 0] = fmaf(sv[j], __uint_as_float(v[4 * q + 0]), fmaf(cv[j], xv.x, acc[4 * q + 0]));
          acc[4 * q + 1] = fmaf(sv[j], __uint_as_float(v[4 * q + 1]), fmaf(cv[j], xv.y, acc[4 * q + 1]));
          acc[4 * q + 2] = fmaf(sv[j], __uint_as_float(v[4 * q + 2]), fmaf(cv[j], xv.z, acc[4 * q + 2]));
          acc[4 * q + 3] = fmaf(sv[j], __uint_as_float(v[4 * q + 3]), fmaf(cv[j], xv.w, acc[4 * q + 3]));
        }
      }
      if (!ok) break;
      // end of this CTA's part of the row block?
      if (chunk == p.chunks - 1 || u == u1 - 1) {
        const bool full = seg_c0 == 0 && chunk == p.chunks - 1;
        const int n = tile * kRows + r;
        if (full) {
          if (n < p.N) {
#pragma unroll
            for (int t = 0; t < 16; ++t)
              if (t < p.M) p.y[(size_t)t * p.N + n] = __float2bfloat16_rn(acc[t]);
          }
        } else {
          // partial row block: plain stores into this CTA's own slot (0 = its first row block)
          const int which = tile == u0 / p.chunks ? 0 : 1;
          float4* gp = reinterpret_cast<float4*>(p.partial + (((size_t)blockIdx.x * 2 + which) * kRows + r) * 16);
#pragma unroll
          for (int q = 0; q < 4; ++q) __stcg(gp + q, make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]));
        }
#pragma unroll
        for (int t = 0; t < 16; ++t) acc[t] = 0.0f;
        seg_c0 = 0;
      }
    }
    if (warp == kFixWarp0) { QTC_OUT(8, pw0); QTC_OUT(9, pw1); QTC_OUT(10, clock64() - prof_entry); }
    // ---- combine row blocks shared with other CTAs: every contributor has stored its partial
    // tile in its own slot; the last one to arrive (arrival counter) adds the slots in CTA order.
    if (n_shared > 0) {
      __threadfence();
      fix_barrier();
      if (ftid < n_shared) {
        const int tile = shared_tiles[ftid];
        const long long b0 = (long long)tile * p.chunks, b1 = b0 + p.chunks;
        const long long first_owner = ((b0 + 1) * G - 1) / T, last_owner = (b1 * G - 1) / T;
        const unsigned expected = (unsigned)(last_owner - first_owner + 1);
        const unsigned old = atomicAdd(&p.counters[tile], 1u);
        const int last = old == expected - 1;
        if (last) p.counters[tile] = 0;
        bars->is_last[ftid] = last;
      }
      fix_barrier();
      for (int i = 0; i < n_shared; ++i) {
        if (!bars->is_last[i]) continue;
        __threadfence();
        const int tile = shared_tiles[i];
        const int n = tile * kRows + r;
        const long long b0 = (long long)tile * p.chunks, b1 = b0 + p.chunks;
        const int first_owner = (int)(((b0 + 1) * G - 1) / T), last_owner = (int)((b1 * G - 1) / T);
        float sum[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) sum[t] = 0.0f;
        for (int c = first_owner; c <= last_owner; ++c) {
          const int cu0 = (int)((long long)c * T / G);
          const int which = tile == cu0 / p.chunks ? 0 : 1;
          float4* gp = reinterpret_cast<float4*>(p.partial + (((size_t)c * 2 + which) * kRows + r) * 16);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 v = __ldcg(gp + q);
            sum[4 * q] += v.x; sum[4 * q + 1] += v.y; sum[4 * q + 2] += v.z; sum[4 * q + 3] += v.w;
            // leave the slot zeroed: the workspace is shared with kernels whose accumulators start at zero
            __stcg(gp + q, make_float4(0.0f, 0.0f, 0.0f, 0.0f));
          }
        }
        if (n < p.N) {
#pragma unroll
          for (int t = 0; t < 16; ++t)
            if (t < p.M) p.y[(size_t)t * p.N + n] = __float2bfloat16_rn(sum[t]);
        }
      }
    }
  }

  // ---- teardown
  if (warp == kDequantWarp0) QTC_MARK(2);
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) QTC_MARK(3);
  if (tid == 0 && *abort_flag) atomicMax(&p.status[0], 4u);
  if (warp == 1) {
    tcgen05_fence_after();
    tcgen05_dealloc(tmem_base, kTmemCols);
  }
}

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

size_t qtc_smem_bytes(int64_t K, int group) {
  const size_t need =
      1024 + (size_t)(K / 64) * 2048 + (size_t)kStagesW * kBoxBytes + (size_t)(K / group) * 64 + sizeof(QtcBarriers) + 64;
  // more than half an SM's shared memory: one CTA per SM, so the 512-column TMEM allocation never waits
  return need > 120 * 1024 ? need : 120 * 1024;
}
size_t counters_bytes(int64_t N) { return (size_t)(((N + 15) / 16 * 4 + 255) / 256 * 256); }
// one slot of 128 x 16 floats per (CTA, first/last row block); the grid never exceeds kMaxCtas
constexpr int kMaxCtas = 256;
size_t partial_bytes(int64_t) { return (size_t)kMaxCtas * 2 * kRows * 16 * 4; }

}  // namespace

bool qmv_tc_supported(const QmmArgs& a) {
  if (a.dtype != B200Q_BF16 || !a.transpose || a.w_batched || a.batch != 1 || a.bits != 4) return false;
  if (a.M < 1 || a.M > 16 || a.N < 1 || a.K < kChunkK || a.K % kChunkK != 0) return false;
  if ((int64_t)((a.N + kRows - 1) / kRows) * (a.K / kChunkK) >= (1ll << 31)) return false;
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.wq) & 15)) return false;
  return qtc_smem_bytes(a.K, a.group) <= 227 * 1024;
}

size_t qmv_tc_workspace_bytes(const QmmArgs& a) { return counters_bytes(a.N) + partial_bytes(a.N) + kStatusBytes; }

int qmv_tc(const QmmArgs& a, cudaStream_t st) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(B200Q_ERR_CUDA, "[quantized_matmul] cuTensorMapEncodeTiled is not available");
  const size_t need = qmv_tc_workspace_bytes(a);
  if (!a.ws || a.ws_bytes < need)
    return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul] workspace of %zu bytes required, %zu given", need, a.ws_bytes);
  if (reinterpret_cast<uintptr_t>(a.ws) & 15)
    return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul] workspace must be 16-byte aligned");
  CUtensorMap map_w;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)a.K / 2, (cuuint64_t)a.N};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K / 2};
    const cuuint32_t box[2] = {128, (cuuint32_t)kRows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint32_t*>(a.wq), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_CUDA, "[quantized_matmul] tensor map for w failed (%d)", (int)r);
  }
  QtcParams p{};
  p.x = (const __nv_bfloat16*)a.x;
  p.scales = (const __nv_bfloat16*)a.scales;
  p.biases = (const __nv_bfloat16*)a.biases;
  p.y = (__nv_bfloat16*)a.y;
  p.counters = reinterpret_cast<uint32_t*>(a.ws);
  p.partial = reinterpret_cast<float*>(static_cast<char*>(a.ws) + counters_bytes(a.N));
  p.status = reinterpret_cast<uint32_t*>(static_cast<char*>(a.ws) + a.ws_bytes - kStatusBytes);
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.n_tiles = (int)((a.N + kRows - 1) / kRows);
  p.chunks = (int)(a.K / kChunkK);
  p.total_units = (long long)p.n_tiles * p.chunks;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms > kMaxCtas) sms = kMaxCtas;
  const int grid = (int)(p.total_units < sms ? p.total_units : sms);
  const size_t smem = qtc_smem_bytes(a.K, a.group);
  auto go = [&](auto kern) -> int {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(map_w, p);
    B200Q_LAUNCH_OK("qmv_tc_kernel");
    return B200Q_OK;
  };
  if (a.group == 32) return go(qmv_tc_kernel<32>);
  if (a.group == 64) return go(qmv_tc_kernel<64>);
  return go(qmv_tc_kernel<128>);
}

}  // namespace b200q
