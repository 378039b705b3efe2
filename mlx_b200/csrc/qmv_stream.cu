// Decode path for 4-bit weights: y[M<=16, N] = x[M, K] * dequant(W[N, K])^T, bf16, HBM-bound.
//
// Replaces cu::qmv_kernel / the small-M use of cu::qmm_sm80_kernel of the reference
// (mlx/backend/cuda/quantized/qmm/qmv.cu:84-209, quantized.cpp:106-136).
//
// One persistent CTA per SM of 16 warps; there is no producer warp: the warp that is last to
// finish with a ring stage refills it (shared arrival counter per stage).
//
//  * The packed weights stream through a ring of TMA boxes of 128 rows x 128 bytes (256 k),
//    128-byte swizzled, so that every byte leaves HBM once, in full lines, without passing
//    through the L1 tag stage, and ldmatrix reads it back without bank conflicts.  The boxes
//    of the whole problem are numbered row block by row block (k fastest); CTA i owns the
//    contiguous span [i*T/G, (i+1)*T/G), so every SM streams the same number of bytes.
//  * Warp (r, c) owns rows 32r..32r+31 and k 64c..64c+63 of every box.  ldmatrix hands lane
//    (g, t) one 32-bit word (8 fields) of rows g, g+8, g+16, g+24; shift+lop3 turn a word into
//    four bf16 pairs (128+q_i, 128+q_{i+4}) which are the A fragments of two
//    mma.sync.m16n8k16 (weights = M dimension, tokens = N dimension).  The k order inside an
//    MMA is permuted to suit the unpack; x is staged once per CTA in shared memory in exactly
//    that order, one conflict-free 128-bit read per two MMAs, shared by both row tiles.
//  * Scales never touch the weights: per group, T = sum x*(128+q) comes out of the tensor
//    core in fp32 and acc += s*T + (b - 128 s) * sum(x); the per-group sums of x are
//    produced once per CTA by MMAs against a matrix of ones.
//  * At the end of a row block the four k-slices are added in a shared fp32 tile.  A row block
//    that lies inside the CTA's span is rounded and written at once; one shared with a
//    neighbouring CTA goes to the CTA's own scratch slot and the last CTA to arrive (arrival
//    counter) adds the slots in CTA order, writes y and leaves slots and counter zeroed.
//    No CTA ever waits on another CTA.
//
// Every mbarrier wait is bounded: when one expires the CTA raises its abort flag and the
// device status word, all warps leave their loops and the kernel ends normally.
//
// Scratch (caller workspace, zero on first use, left zeroed):
//   [ counters: one u32 per row block | slots: kMaxCtas x 2 x 128 rows x 16 tokens fp32 ]
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace b200q {
namespace {

using namespace tc;

constexpr int kRows = 128;            // weight rows per box
constexpr int kBoxK = 256;            // k per box
constexpr int kBoxBytes = kRows * 128;
constexpr int kWarps = 16;            // 4 row slices x 4 k slices
constexpr int kThreads = 32 * kWarps;
constexpr int kMaxStages = 8;
constexpr int kMaxCtas = 192;
constexpr int kSmemLimit = 227 * 1024;

struct SParams {
  const __nv_bfloat16* x;
  const unsigned short* scales;
  const unsigned short* biases;
  __nv_bfloat16* y;
  uint32_t* counters;
  float* slots;
  uint32_t* status;
  int M, N, K;
  int kb;            // boxes per row block (K / 256)
  int n_rb;          // row blocks
  long long total;   // boxes
  int stages;
  int toks;          // token rows of x held in shared memory: 1, 2, 4, 8 or 16 (>= M)
};

struct __align__(8) SBarriers {
  uint64_t full[kMaxStages];
  uint64_t xbar;          // the activations have landed
  int done[kMaxStages];   // warps that have finished with the stage's current box
  int abort_flag;
  int dep[2];         // warps that have deposited into tile 0 / 1
  int last_flag[2];   // this CTA arrived last at its first / last shared row block
  int pend_rb[2];
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
}
// D = A*B + C with separate C registers (C may be the zero tile)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}
__device__ __forceinline__ void red_shared_add(float* p, float v) {
  asm volatile("red.shared.add.f32 [%0], %1;" ::"r"(smem_u32(p)), "f"(v) : "memory");
}
__device__ __forceinline__ void compute_barrier() { __syncthreads(); }

__device__ __forceinline__ void cp_async_zfill(uint32_t dst, const void* src, int bytes, int src_bytes) {
  // bytes is 4, 8 or 16; src_bytes == 0 writes zeros without reading
  if (bytes == 16)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
  else if (bytes == 8)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Arrives on the mbarrier once every cp.async this thread has issued so far has landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// Bounded wait with few instructions: the first probe usually succeeds; after that the hardware
// suspends the warp inside try_wait (time hint) instead of spinning through issue slots.
__device__ __forceinline__ bool mbar_wait_hint(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  for (uint32_t i = 0; i < (1u << 16); ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    if (done) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ uint32_t atom_shared_add(uint32_t addr, uint32_t v) {
  uint32_t old;
  asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// N consecutive 32-bit words (N = 1, 2 or 4) with one load
template <int N>
__device__ __forceinline__ void lds_words(uint32_t (&v)[N], uint32_t addr) {
  if constexpr (N == 4)
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
  else if constexpr (N == 2)
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "r"(addr));
  else
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v[0]) : "r"(addr));
}
// One bf16 half of a word -> fp32, as an instruction the compiler cannot move (see below).
__device__ __forceinline__ float bf16_half_pinned(uint32_t word, int hi) {
  uint32_t o;
  if (hi) asm volatile("and.b32 %0, %1, 0xFFFF0000;" : "=r"(o) : "r"(word));
  else asm volatile("mul.lo.u32 %0, %1, 65536;" : "=r"(o) : "r"(word));
  return __uint_as_float(o);
}
// bf16 bits -> fp32 as an instruction the compiler cannot move: it reads its operand, so it
// cannot issue before the shared-memory load that feeds it has returned.
__device__ __forceinline__ float bf16_to_float_pinned(uint32_t raw) {
  uint32_t o;
  asm volatile("mul.lo.u32 %0, %1, 65536;" : "=r"(o) : "r"(raw));   // a shift, issued to the multiply-add pipe
  return __uint_as_float(o);
}

// Shared-memory carve-up (bytes), identical on host and device.
struct Layout {
  uint32_t ring, stage_bytes, xs, xsum, tile, bars, total;
};
template <int MT, int GROUP>
__host__ __device__ inline Layout make_layout(int K, int stages, int toks) {
  constexpr int XG = GROUP < 64 ? GROUP : 64;
  constexpr int GPB = kBoxK / GROUP;                            // groups per box and row
  Layout L;
  uint32_t off = 0;
  L.stage_bytes = kBoxBytes + 2 * kRows * GPB * 2;              // packed box, scales, biases (multiple of 1024)
  L.ring = off; off += (uint32_t)stages * L.stage_bytes;
  L.xs = off;   off += (uint32_t)(K / 32) * toks * 64;          // [K/32 chunks][stored tokens][4 octets x 16 B]
  L.xsum = off; off += (uint32_t)(K / XG) * (8 * MT) * 4;       // [K/XG][tokens] fp32
  L.tile = off; off += 2u * kRows * (8 * MT) * 4;               // two tiles [128 rows][tokens] fp32
  L.bars = off; off += (uint32_t)sizeof(SBarriers);
  L.total = off + 1024;                                         // room to align the ring to 1024 bytes
  return L;
}

template <int MT, int GROUP, int NG>
__global__ void __launch_bounds__(kThreads, 1)
qmv_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const SParams p) {
  constexpr int TOK = 8 * MT;
  constexpr int XG = GROUP < 64 ? GROUP : 64;     // k covered by one scale application
  constexpr int APPLY = 64 / XG;                  // scale applications per box and warp (1 or 2)
  constexpr int GPB = kBoxK / GROUP;              // groups per box and row (8, 4, 2)
  constexpr int kScaleOff = kBoxBytes, kBiasOff = kBoxBytes + kRows * GPB * 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Layout L = make_layout<MT, GROUP>(p.K, p.stages, p.toks);
  const int TS = p.toks;   // token rows of x in shared memory; lanes whose token is not stored use zeros
  unsigned char* ring = smem + L.ring;
  unsigned char* xs = smem + L.xs;
  float* xsum = reinterpret_cast<float*>(smem + L.xsum);
  float* tile = reinterpret_cast<float*>(smem + L.tile);
  SBarriers* bars = reinterpret_cast<SBarriers*>(smem + L.bars);
  volatile int* abort_flag = &bars->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef B200Q_PROFILE
  // Profile builds: one CTA (blockIdx.x == gridDim.x / 2) leaves clock marks (cycles since entry)
  // in the 256 bytes before the status word.
  uint32_t* dbg = p.status - 64;
  const long long prof_entry = clock64();
  long long prof_wait = 0, prof_t = 0, ph_a = 0, ph_b = 0, ph_c = 0, ph_d = 0, ph_t = 0;
#define QS_PH(acc) { const long long now_ = clock64(); acc += now_ - ph_t; ph_t = now_; }
#define QS_MARK(slot) if (blockIdx.x == gridDim.x / 2 && lane == 0) dbg[slot] = (uint32_t)(clock64() - prof_entry)
#define QS_T0() prof_t = clock64()
#define QS_ACC() prof_wait += clock64() - prof_t
#define QS_OUT(slot, v) if (blockIdx.x == gridDim.x / 2 && lane == 0) dbg[slot] = (uint32_t)(v)
#else
#define QS_MARK(slot)
#define QS_T0()
#define QS_ACC()
#define QS_OUT(slot, v)
#define QS_PH(acc)
#endif
  const int G = gridDim.x;
  const long long b0 = (long long)blockIdx.x * p.total / G, b1 = (long long)(blockIdx.x + 1) * p.total / G;
  const int S = p.stages;
  const int row_groups = p.K / GROUP;

  {
    // The first mma.sync of a kernel takes a couple of thousand cycles (the tensor pipe wakes up):
    // issue one now, while nothing else can run anyway.  Its result is never used.
    float d0, d1, d2, d3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%4,%4,%4}, {%4,%4}, {%5,%5,%5,%5};"
                 : "=f"(d0), "=f"(d1), "=f"(d2), "=f"(d3) : "r"(0u), "f"(0.0f));
  }
  asm volatile("griddepcontrol.launch_dependents;");
  if (tid == 32) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  if (tid == 64) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
  if (tid == 0) {
    // full: the TMA transaction (one arrive.expect_tx) and the 32 scale-copy lanes of the producer warp
    for (int i = 0; i < S; ++i) { mbar_init(smem_u32(&bars->full[i]), 1 + 32); bars->done[i] = 0; }
    mbar_init(smem_u32(&bars->xbar), 1);
    bars->abort_flag = 0;
    bars->last_flag[0] = bars->last_flag[1] = 0;
    bars->dep[0] = bars->dep[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) QS_MARK(13);

  // Span bookkeeping in 32 bits: the span is walked with incremental (row block, k chunk, stage,
  // phase) counters, never with divisions.
  const int n_boxes = (int)(b1 - b0);
  const int rb_first = (int)(b0 / p.kb), kc_first = (int)(b0 - (long long)rb_first * p.kb);
  const uint32_t ring_u = smem_u32(ring), xs_u = smem_u32(xs), xsum_u = smem_u32(xsum);

  // Fills ring stage `st` with box (rb, kc): packed weights by TMA (lane 0), the box's scales
  // and biases by 4/8/16-byte async copies (all lanes of the calling warp).
  auto issue_box = [&](uint32_t st, int rb, int kc) {
    const uint32_t stage = ring_u + st * L.stage_bytes;
    const uint32_t full = smem_u32(&bars->full[st]);
    if (lane == 0) {
      mbar_expect_tx(full, kBoxBytes);
      tma_load_2d(stage, &map_w, kc * 128, rb * kRows, full);
    }
#pragma unroll
    for (int q = 0; q < kRows / 32; ++q) {
      const int rib = lane + 32 * q;
      int row = rb * kRows + rib;
      const int nbytes = row < p.N ? GPB * 2 : 0;
      row = row < p.N ? row : p.N - 1;
      const size_t src = (size_t)row * row_groups + (size_t)kc * GPB;
      cp_async_zfill(stage + kScaleOff + rib * GPB * 2, p.scales + src, GPB * 2, nbytes);
      cp_async_zfill(stage + kBiasOff + rib * GPB * 2, p.biases + src, GPB * 2, nbytes);
    }
    cp_async_arrive_noinc(full);
  };
  {
    const int g = lane >> 2, t = lane & 3;
    // warps w, w+4, w+8, w+12 share an SM sub-partition: give them the same row slice and
    // different box groups, so that a sub-partition always holds warps in different phases
    // NG == 4: group = warp / 4, the warp walks all four 64-k slices of its boxes.
    // NG == 2 (shallow rings): group = warp / 8, two warps share a row slice and take two 64-k slices each.
    constexpr int WPG = kWarps / NG;          // warps per group
    constexpr int CPW = NG / 1 == 4 ? 4 : 2;    // 64-k slices per warp and box
    const int r = warp & 3, gq = warp / WPG;
    const int c0 = NG == 4 ? 0 : ((warp >> 2) & 1) * 2;
    const int ctid = tid;

    // ---- stage x: one 3-D TMA box brings [M, K] bf16 in as [K/32 chunks][TOK tokens][32 k]
    //      (tokens >= M are zero-filled); it is requested before the weight stream so that it does
    //      not queue behind megabytes of weight requests.  The first boxes of the stream follow
    //      (warp i, box i).  Then every 8-k octet is permuted in place to
    //      (x0,x4),(x1,x5),(x2,x6),(x3,x7), the order the unpacked weight pairs come in.
    {
      // Only the first box is requested together with x: a deeper prefetch from every SM at once
      // would put megabytes of weight requests in front of the few kilobytes everything waits for.
      // The box is a constant: it may be requested while the previous kernel of the stream is
      // still running (programmatic dependent launch); x, y and the workspace only after the wait.
      if (warp == 0 && n_boxes > 0) issue_box(0u, rb_first, kc_first);
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (tid == 0) {
        mbar_expect_tx(smem_u32(&bars->xbar), (uint32_t)(p.K * TS * 2));
        tma_load_3d(xs_u, &map_x, 0, 0, 0, smem_u32(&bars->xbar));
      }
      if (warp == 0) QS_MARK(10);
      for (int i = ctid; i < 2 * kRows * TOK; i += kWarps * 32) tile[i] = 0.0f;
#ifdef B200Q_PROFILE
      if (warp == 1) { mbar_wait_hint(smem_u32(&bars->full[0]), 0, abort_flag); QS_MARK(14); }
#endif
      const bool x_ok = mbar_wait_hint(smem_u32(&bars->xbar), 0, abort_flag);
      if (!x_ok && tid == 0) atomicCAS(&p.status[2], 0u, 0x40000000u);
      if (warp == 0) QS_MARK(11);
      if (warp == 15) QS_MARK(22);
      if (warp > 0 && warp < S && warp < n_boxes) {
        const long long j = b0 + warp;
        const int rbw = (int)(j / p.kb);
        issue_box((uint32_t)warp, rbw, (int)(j - (long long)rbw * p.kb));
      }
      const int pieces = p.K / 8 * TS;
      if (x_ok) {
        for (int pi = ctid; pi < pieces; pi += kWarps * 32) {
          if (((pi >> 2) & (TS - 1)) < p.M) {   // TS is a power of two
            const uint32_t a = xs_u + (uint32_t)pi * 16;
            const uint4 v = lds128(a);
            uint4 w;
            w.x = __byte_perm(v.x, v.z, 0x5410);
            w.y = __byte_perm(v.x, v.z, 0x7632);
            w.z = __byte_perm(v.y, v.w, 0x5410);
            w.w = __byte_perm(v.y, v.w, 0x7632);
            sts128(a, w);
          }
        }
      }
    }
    if (warp == 0) QS_MARK(12);
    if (warp == 3) QS_MARK(20);
    if (warp == 15) QS_MARK(21);
    compute_barrier();
    if (warp == 0) QS_MARK(0);
    // B-fragment address of this lane inside a 32-k chunk: token g (+8b), octet t
    const uint32_t xlane_u = xs_u + (uint32_t)(g * 64 + t * 16);
    bool xstored[MT];
#pragma unroll
    for (int b = 0; b < MT; ++b) xstored[b] = g + 8 * b < TS;
    // ---- per-block sums of x through the tensor core: D = ones * B, all rows of D equal.
    //      Four blocks at a time so that the MMA chains overlap.
    {
      const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      constexpr uint32_t kOnes = 0x3F803F80u;
      const int nblk = p.K / XG;
      for (int blk0 = warp; blk0 < nblk; blk0 += kWarps * 4) {
        float d[4][MT][4];
#pragma unroll
        for (int h = 0; h < XG / 32; ++h)
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int blk = blk0 + kWarps * u;
            if (blk < nblk) {
#pragma unroll
              for (int b = 0; b < MT; ++b) {
                const int ch = blk * (XG / 32) + h;
                const uint4 xf = xstored[b] ? lds128(xlane_u + (uint32_t)(ch * TS + 8 * b) * 64) : make_uint4(0, 0, 0, 0);
                if (h == 0) mma_bf16(d[u][b], zero4, kOnes, kOnes, kOnes, kOnes, xf.x, xf.y);
                else mma_bf16(d[u][b], d[u][b], kOnes, kOnes, kOnes, kOnes, xf.x, xf.y);
                mma_bf16(d[u][b], d[u][b], kOnes, kOnes, kOnes, kOnes, xf.z, xf.w);
              }
            }
          }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int blk = blk0 + kWarps * u;
          if (blk < nblk && g == 0) {
#pragma unroll
            for (int b = 0; b < MT; ++b)
              *reinterpret_cast<float2*>(xsum + blk * TOK + 8 * b + 2 * t) = make_float2(d[u][b][0], d[u][b][1]);
          }
        }
      }
    }
    if (warp == 0) QS_MARK(23);
    if (warp == 15) QS_MARK(24);
    compute_barrier();
    if (warp == 0) QS_MARK(1);

    // ---- main loop over this CTA's boxes
    float acc[2][MT][4];
#pragma unroll
    for (int rt = 0; rt < 2; ++rt)
#pragma unroll
      for (int b = 0; b < MT; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[rt][b][i] = 0.0f;
    const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};

    constexpr int F4 = kRows * TOK / 4;           // float4 elements of a tile
    constexpr int TQ = TOK / 4;                   // float4 per row
    auto store_rows = [&](int rb, int idx, const float4& v) {
      const int n = rb * kRows + idx / TQ, tok0 = (idx % TQ) * 4;
      if (n < p.N) {
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (tok0 + q < p.M) p.y[(size_t)(tok0 + q) * p.N + n] = __float2bfloat16_rn(vv[q]);
      }
    };
    const int rb_last = (int)((b1 - 1) / p.kb);
    // Every warp calls this once per row block of the span, in order, when it has no more boxes
    // in that row block: its accumulators are added into the block's shared tile (two tiles
    // alternate) and the last of the 16 warps to do so writes the block out: rounded to y when
    // the CTA owns the whole row block, else to this CTA's slot, with a bump of the arrival
    // counter; whether this CTA arrived last is looked at after the main loop (combine()).
    auto deposit = [&](int rb) {
      float* tl = tile + (rb & 1) * (kRows * TOK);
#pragma unroll
      for (int rt = 0; rt < 2; ++rt)
#pragma unroll
        for (int b = 0; b < MT; ++b)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            red_shared_add(tl + (32 * r + 16 * rt + g + 8 * (i >> 1)) * TOK + 8 * b + 2 * t + (i & 1), acc[rt][b][i]);
            acc[rt][b][i] = 0.0f;
          }
      __syncwarp();
      int last = 0;
      if (lane == 0) {
        __threadfence_block();
        last = atom_shared_add(smem_u32(&bars->dep[rb & 1]), 1u) == (uint32_t)(kWarps - 1);
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (!last) return;
      __threadfence_block();
      const long long rb0 = (long long)rb * p.kb, rb1 = rb0 + p.kb;
      const bool owned = rb0 >= b0 && rb1 <= b1;
      const int which = rb == rb_first ? 0 : 1;
      float4* slot = reinterpret_cast<float4*>(p.slots) + ((size_t)blockIdx.x * 2 + which) * F4;
      for (int idx = lane; idx < F4; idx += 32) {
        const float4 v = reinterpret_cast<float4*>(tl)[idx];
        reinterpret_cast<float4*>(tl)[idx] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (owned) store_rows(rb, idx, v);
        else __stcg(slot + idx, v);
      }
      __syncwarp();
      if (lane == 0) {
        bars->dep[rb & 1] = 0;
        if (!owned) {
          // one fence for the warp: the warp barrier orders every lane's slot stores before it
          __threadfence();
          const int first_owner = (int)(((rb0 + 1) * G - 1) / p.total), last_owner = (int)((rb1 * G - 1) / p.total);
          const unsigned old = atomicAdd(&p.counters[rb], 1u);
          const int lastc = old == (unsigned)(last_owner - first_owner);
          if (lastc) p.counters[rb] = 0;
          __threadfence();
          bars->pend_rb[which] = rb;
          bars->last_flag[which] = lastc;
        }
      }
    };
    // The CTA that arrived last at a shared row block adds the slots in CTA order, writes y and
    // leaves the slots zeroed (all threads).
    auto combine = [&](int rb) {
      const long long rb0 = (long long)rb * p.kb, rb1 = rb0 + p.kb;
      const int first_owner = (int)(((rb0 + 1) * G - 1) / p.total), last_owner = (int)((rb1 * G - 1) / p.total);
      if (ctid < F4) {
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int cta = first_owner; cta <= last_owner; ++cta) {
          const int wh = rb == (int)(((long long)cta * p.total / G) / p.kb) ? 0 : 1;
          float4* sp = reinterpret_cast<float4*>(p.slots) + ((size_t)cta * 2 + wh) * F4 + ctid;
          const float4 u = __ldcg(sp);
          v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
          __stcg(sp, make_float4(0.0f, 0.0f, 0.0f, 0.0f));
        }
        store_rows(rb, ctid, v);
      }
    };

    // per-lane constant offsets inside a stage
    const uint32_t ldsm_row = (uint32_t)((32 * r + lane) * 128);
    const uint32_t ldsm_sw = (uint32_t)(lane & 7);
    const uint32_t sc_lane = (uint32_t)((32 * r + g) * GPB * 2);   // + q * 16 * GPB: rows g, g+8, g+16, g+24
    const uint32_t xsum_lane = xsum_u + (uint32_t)(2 * t * 4);

    // Box i of the span is handled by the four warps with (warp >> 2) == i % 4, one per 32-row
    // slice, each walking the four 64-k slices of the box.  The four groups work on four
    // consecutive boxes at a time, out of phase with each other, so that the load, unpack and
    // tensor pipes of an SM sub-partition are busy with different warps at the same time.
    int rb = rb_first, kc = kc_first + gq;
    while (kc >= p.kb) { kc -= p.kb; ++rb; }
    int cur_rb = rb_first;
    uint32_t s = (uint32_t)gq % (uint32_t)S, ph = ((uint32_t)gq / (uint32_t)S) & 1u;
    bool ok = true;
    for (int i = gq; i < n_boxes; i += NG) {
      while (cur_rb < rb) { deposit(cur_rb); ++cur_rb; }
      // After a failed wait the warp keeps walking its boxes without touching the ring, so that
      // the row-block bookkeeping still completes.
      QS_T0();
      if (ok && !mbar_wait_hint(smem_u32(&bars->full[s]), ph, abort_flag)) {
        ok = false;
        // where the wait gave up: box index within the span, stage, warp
        if (lane == 0 && atomicCAS(&p.status[2], 0u, 0x80000000u | (uint32_t)i) == 0u) p.status[3] = (s << 8) | (uint32_t)warp;
      }
      QS_ACC();
      if (i == gq && warp == 0) QS_MARK(2);
      if (ok) {
#ifdef B200Q_PROFILE
        ph_t = clock64();
#endif
        const uint32_t stage = ring_u + s * L.stage_bytes;
        // raw scales / biases of this lane's four rows: all GPB groups of the box in one load
        uint32_t s_raw[4][GPB / 2], b_raw[4][GPB / 2];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          lds_words<GPB / 2>(s_raw[q], stage + kScaleOff + sc_lane + (uint32_t)(q * 16 * GPB));
          lds_words<GPB / 2>(b_raw[q], stage + kBiasOff + sc_lane + (uint32_t)(q * 16 * GPB));
        }
        QS_PH(ph_a);
        // The slice index must be a compile-time value (it selects registers): the loop body is
        // instantiated once per possible first slice of a warp.
        auto slices = [&](auto c0c) {
        constexpr int C0 = decltype(c0c)::value;
#pragma unroll
        for (int cc = 0; cc < CPW; ++cc) {
          const int c = C0 + cc;
          uint32_t w[2][4];
          uint4 xf[2][MT];
          const uint32_t xa = xlane_u + (uint32_t)((kc * 8 + 2 * c) * TS) * 64;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            ldmatrix_x4(w[h], stage + ldsm_row + ((((uint32_t)(2 * c + h)) ^ ldsm_sw) << 4));
#pragma unroll
            for (int b = 0; b < MT; ++b)
              xf[h][b] = xstored[b] ? lds128(xa + (uint32_t)((h * TS + b * 8) * 64)) : make_uint4(0, 0, 0, 0);
          }
          float2 xv[APPLY][MT];
          const uint32_t xb = xsum_lane + (uint32_t)(((kc * kBoxK + c * 64) / XG) * TOK) * 4;
#pragma unroll
          for (int a = 0; a < APPLY; ++a)
#pragma unroll
            for (int b = 0; b < MT; ++b) xv[a][b] = lds64f(xb + (uint32_t)((a * TOK + b * 8) * 4));
          // ---- unpack and multiply: T[a] = sum over the scale block of x * (128 + q)
          float tmp[APPLY][2][MT][4];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int a = (h * 32) / XG;
            const bool fresh = (h * 32) % XG == 0;   // first 32 k of a scale block
#pragma unroll
            for (int rt = 0; rt < 2; ++rt) {
              uint32_t P[4], Q[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                P[q] = lop3_and_or(w[h][2 * rt] >> (4 * q), 0x000F000Fu, 0x43004300u);
                Q[q] = lop3_and_or(w[h][2 * rt + 1] >> (4 * q), 0x000F000Fu, 0x43004300u);
              }
#pragma unroll
              for (int b = 0; b < MT; ++b) {
                if (fresh) mma_bf16(tmp[a][rt][b], zero4, P[0], Q[0], P[1], Q[1], xf[h][b].x, xf[h][b].y);
                else mma_bf16(tmp[a][rt][b], tmp[a][rt][b], P[0], Q[0], P[1], Q[1], xf[h][b].x, xf[h][b].y);
                mma_bf16(tmp[a][rt][b], tmp[a][rt][b], P[2], Q[2], P[3], Q[3], xf[h][b].z, xf[h][b].w);
              }
            }
          }
          // ---- acc += s * T + c * sum(x); the conversions are real instructions on the loaded
          //      words, so they cannot issue before the loads have returned
#pragma unroll
          for (int a = 0; a < APPLY; ++a) {
            const int gib = (c * 64 + a * XG) / GROUP;   // group of the box this scale block lies in
            float sf[4], cf[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              sf[q] = bf16_half_pinned(s_raw[q][gib >> 1], gib & 1);
              cf[q] = fmaf(-128.0f, sf[q], bf16_half_pinned(b_raw[q][gib >> 1], gib & 1));
            }
#pragma unroll
            for (int b = 0; b < MT; ++b)
#pragma unroll
              for (int rt = 0; rt < 2; ++rt) {
                acc[rt][b][0] = fmaf(sf[2 * rt], tmp[a][rt][b][0], fmaf(cf[2 * rt], xv[a][b].x, acc[rt][b][0]));
                acc[rt][b][1] = fmaf(sf[2 * rt], tmp[a][rt][b][1], fmaf(cf[2 * rt], xv[a][b].y, acc[rt][b][1]));
                acc[rt][b][2] = fmaf(sf[2 * rt + 1], tmp[a][rt][b][2], fmaf(cf[2 * rt + 1], xv[a][b].x, acc[rt][b][2]));
                acc[rt][b][3] = fmaf(sf[2 * rt + 1], tmp[a][rt][b][3], fmaf(cf[2 * rt + 1], xv[a][b].y, acc[rt][b][3]));
              }
          }
        }
        };
        if (NG == 4 || c0 == 0) slices(std::integral_constant<int, 0>{});
        else slices(std::integral_constant<int, 2>{});
        QS_PH(ph_b);
        // ---- release the stage: everything read from it has been consumed by instructions that
        //      had to wait for it (the MMAs for the packed words, the conversions for the scales).
        //      The last of the group's four warps refills the stage with the box S places ahead.
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atom_shared_add(smem_u32(&bars->done[s]), 1u) == (uint32_t)(WPG - 1);
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          if (lane == 0) bars->done[s] = 0;
          if (i + S < n_boxes) {
            int rb_n = rb, kc_n = kc + S;
            while (kc_n >= p.kb) { kc_n -= p.kb; ++rb_n; }
            issue_box(s, rb_n, kc_n);
          }
        }
        QS_PH(ph_c);
      }
      s += NG;
      while (s >= (uint32_t)S) { s -= (uint32_t)S; ph ^= 1u; }
      kc += NG;
      while (kc >= p.kb) { kc -= p.kb; ++rb; }
    }
    if (warp == 0) { QS_MARK(3); QS_OUT(5, prof_wait); QS_OUT(6, (uint32_t)n_boxes); }
    while (cur_rb <= rb_last) { deposit(cur_rb); ++cur_rb; }
    if (warp == 0) { QS_MARK(4); QS_OUT(16, ph_a); QS_OUT(17, ph_b); QS_OUT(18, ph_c); QS_OUT(19, ph_d); }
    compute_barrier();
#pragma unroll
    for (int wh = 0; wh < 2; ++wh)
      if (bars->last_flag[wh]) combine(bars->pend_rb[wh]);
    if (warp == 0) QS_MARK(7);
  }

  __syncthreads();
  if (tid == 0 && *abort_flag) atomicMax(&p.status[0], 5u);
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

int stored_tokens(int64_t M) { return M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : (M <= 8 ? 8 : 16))); }
// Ring depth: a multiple of the number of box groups, so that a stage is always consumed by the
// same group (no warp can then be two barrier phases away from the one it waits for).  Eight or
// more stages: four groups; a ring of four to seven stages runs two groups on four or six stages,
// which leaves two or four boxes in flight while two are being worked on.
template <int MT, int GROUP>
int max_stages(int K, int toks) {
  for (int s = kMaxStages; s >= 1; --s)
    if (make_layout<MT, GROUP>(K, s, toks).total <= (uint32_t)kSmemLimit) return s;
  return 0;
}
struct RingPlan { int stages, groups; };
RingPlan plan_ring(const QmmArgs& a) {
  const int K = (int)a.K, ts = stored_tokens(a.M);
  int m;
  if (a.M <= 8) m = a.group == 32 ? max_stages<1, 32>(K, ts) : (a.group == 64 ? max_stages<1, 64>(K, ts) : max_stages<1, 128>(K, ts));
  else m = a.group == 32 ? max_stages<2, 32>(K, ts) : (a.group == 64 ? max_stages<2, 64>(K, ts) : max_stages<2, 128>(K, ts));
  if (m >= 8) return {8, 4};
  if (m >= 4) return {m & ~1, 2};
  return {0, 0};
}
int stages_for(const QmmArgs& a) { return plan_ring(a).stages; }

size_t counters_bytes(int64_t N) { return (size_t)(((N + kRows - 1) / kRows * 4 + 255) / 256 * 256); }
size_t slots_bytes() { return (size_t)kMaxCtas * 2 * kRows * 16 * 4; }

template <int MT, int GROUP, int NG>
int launch(const QmmArgs& a, const CUtensorMap& map_w, EncodeFn enc, SParams& p, int grid, cudaStream_t st) {
  // activations as a 3-D tensor (32 k, token, 32-k chunk): one box = all of x in staging order
  CUtensorMap map_x;
  {
    const cuuint64_t dims[3] = {32, (cuuint64_t)a.M, (cuuint64_t)a.K / 32};
    const cuuint64_t strides[2] = {(cuuint64_t)a.K * 2, 64};
    const cuuint32_t box[3] = {32, (cuuint32_t)p.toks, (cuuint32_t)(a.K / 32)};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(a.x), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_CUDA, "[quantized_matmul] tensor map for x failed (%d)", (int)r);
  }
  const Layout L = make_layout<MT, GROUP>((int)a.K, p.stages, p.toks);
  cudaError_t e = cudaFuncSetAttribute(qmv_stream_kernel<MT, GROUP, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total);
  if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
  {
    const char* e = getenv("B200Q_PDL");
    if (e && e[0] == '0') {
      qmv_stream_kernel<MT, GROUP, NG><<<grid, kThreads, L.total, st>>>(map_w, map_x, p);
    } else {
      // programmatic dependent launch: see the griddepcontrol instructions in the kernel
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(grid);
      cfg.blockDim = dim3(kThreads);
      cfg.dynamicSmemBytes = L.total;
      cfg.stream = st;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = at;
      cfg.numAttrs = 1;
      B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, qmv_stream_kernel<MT, GROUP, NG>, map_w, map_x, p));
    }
  }
  B200Q_LAUNCH_OK("qmv_stream_kernel");
  return B200Q_OK;
}

}  // namespace

bool qmv_stream_supported(const QmmArgs& a) {
  if (a.dtype != B200Q_BF16 || !a.transpose || a.w_batched || a.batch != 1 || a.bits != 4) return false;
  if (a.M < 1 || a.M > 16 || a.N < 1 || a.K < kBoxK || a.K % kBoxK != 0) return false;
  if (a.K > 8192) return false;   // one TMA box holds all of x: at most 256 chunks of 32 k
  if ((a.N + kRows - 1) / kRows * (a.K / kBoxK) >= (1ll << 40)) return false;
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.wq) & 15)) return false;
  return stages_for(a) >= 4;
}

// The kernel pays a fixed start-up (staging x, first boxes) and a cross-CTA combination at the
// end; it wins over the register-path kernel once every SM streams enough boxes.
bool qmv_stream_profitable(const QmmArgs& a) {
  // ... and the ring is deep enough to keep HBM busy while four boxes are being worked on.
  const long long boxes = (long long)((a.N + kRows - 1) / kRows) * (a.K / kBoxK);
  return boxes >= 24ll * 148 && stages_for(a) >= 8;
}

size_t qmv_stream_workspace_bytes(const QmmArgs& a) { return counters_bytes(a.N) + slots_bytes() + kStatusBytes; }

int qmv_stream(const QmmArgs& a, cudaStream_t st) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(B200Q_ERR_CUDA, "[quantized_matmul] cuTensorMapEncodeTiled is not available");
  const size_t need = qmv_stream_workspace_bytes(a);
  if (!a.ws || a.ws_bytes < need)
    return fail(B200Q_ERR_WORKSPACE, "[quantized_matmul] workspace of %zu bytes required, %zu given", need, a.ws_bytes);
  if (reinterpret_cast<uintptr_t>(a.ws) & 15)
    return fail(B200Q_ERR_INVALID_ARGUMENT, "[quantized_matmul] workspace must be 16-byte aligned");
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
  SParams p{};
  p.x = (const __nv_bfloat16*)a.x;
  p.scales = (const unsigned short*)a.scales;
  p.biases = (const unsigned short*)a.biases;
  p.y = (__nv_bfloat16*)a.y;
  p.counters = reinterpret_cast<uint32_t*>(a.ws);
  p.slots = reinterpret_cast<float*>(static_cast<char*>(a.ws) + counters_bytes(a.N));
  p.status = reinterpret_cast<uint32_t*>(static_cast<char*>(a.ws) + a.ws_bytes - kStatusBytes);
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.kb = (int)(a.K / kBoxK);
  p.n_rb = (int)((a.N + kRows - 1) / kRows);
  p.total = (long long)p.n_rb * p.kb;
  p.stages = stages_for(a);
  p.toks = stored_tokens(a.M);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long grid = p.total < sms ? p.total : sms;
  if (grid > kMaxCtas) grid = kMaxCtas;
  const bool mt2 = a.M > 8;
  const bool g4 = plan_ring(a).groups == 4;
#define B200Q_STREAM_LAUNCH(MT_, G_) \
  (g4 ? launch<MT_, G_, 4>(a, map_w, enc, p, (int)grid, st) : launch<MT_, G_, 2>(a, map_w, enc, p, (int)grid, st))
  if (a.group == 32) return mt2 ? B200Q_STREAM_LAUNCH(2, 32) : B200Q_STREAM_LAUNCH(1, 32);
  if (a.group == 64) return mt2 ? B200Q_STREAM_LAUNCH(2, 64) : B200Q_STREAM_LAUNCH(1, 64);
  return mt2 ? B200Q_STREAM_LAUNCH(2, 128) : B200Q_STREAM_LAUNCH(1, 128);
#undef B200Q_STREAM_LAUNCH
}

}  // namespace b200q
