// Persistent decode kernel for quantized linears at small batch (M <= 8), Q4_K and Q4_0.
//
// Roofline: HBM.  One CTA per SM, NG groups of eight warps.  Every compute warp owns a private ring of shared-memory stages that it fills
// itself with 2-D tensor TMA copies (cp.async.bulk.tensor.2d, one box of 8 rows x 288 bytes
// per half tile, completion on an mbarrier) and drains itself, so nothing inside the stream
// waits on another warp and the copy costs one instruction per stage.  A 16-row weight tile's K range is split over the eight warps of a group;
// each leaves its partial sums in a shared-memory slot and bumps the slot's counter; the warp
// that arrives last adds the eight partials in warp order (deterministic) and runs the
// epilogue and the split-K fix-up, so nobody waits for anybody.
// (Measured and dropped: one-dimensional cp.async.bulk copies of a few hundred bytes -- an SM
// keeps only a handful in flight, 0.5 TB/s in total; 16-byte cp.async -- the LSU needs ~14
// cycles per 18-lane instruction, which caps the stream at 4.4 TB/s and delays every other
// load of the SM behind the prefetch burst.)
//
// Arithmetic: the 4-bit codes go to the tensor cores as they are.  A 32-bit word of eight
// nibbles is split with two masks into two u8x4 registers, which are the A fragments of
// mma.sync.m16n8k32 (u8 x s8 -> s32; the 16 MMA rows are 16 weight rows).  The activations
// are held as 16-bit fixed point per 256-element block (x ~ delta * xi, |xi| <= 32000),
// split into a high and a low signed byte that sit in two adjacent MMA columns, so one MMA
// yields sum(q * x_hi) and sum(q * x_lo) exactly and 256*hi + lo is the exact integer dot
// product.  Sub-block scales multiply the converted sums in fp32; the "-8" offset and the
// Q4_K min term are linear in sum(x) per sub-block and go through one fp16 k8 MMA per
// 256-block against a table built in the prologue.
//
// Fused around it:
//   prologue   RMSNorm of x (optional), rounding to the activation dtype, fixed-point split
//   epilogue   plain (+bias) | SiLU(gate)*up on interleaved gate/up rows | RoPE on q/k rows
//   split-K    K-slices of different CTAs meet in a global scratch; the CTA that arrives
//              last reduces them in slice order and runs the epilogue
//   two phases gate/up -> down in ONE launch without a grid barrier: the first phase publishes h
//              as 8-byte words {payload, launch sequence number}; the second phase's prologue
//              polls the words it needs, and every warp keeps its ring full with the second
//              phase's weights meanwhile
//   exchange   tensor-parallel block: the last phase stores its fp32 sums into every rank's
//              exchange buffer (peer stores), raises a flag per CTA and ends with the reduction
// Every wait (mbarrier, slot flag, hand-over words, peer flag) is bounded by a time limit read from
// %globaltimer (Params::wait_ns); on expiry a status word is set and the kernel carries on without
// blocking.
#pragma once
#include <cuda.h>   // CUtensorMap (type only; the encoder is fetched at run time)

#include "common.cuh"
#include "kernels.h"

namespace mlxr {
namespace decode {

constexpr int kGroupWarps = 8;                          // compute warps per group
constexpr int kTileRows = 16;
constexpr int kStageSegs = 2;                           // 256-element segments per stage and row
constexpr int kSegBytes = 144;                          // Q4_K super-block = 8 Q4_0 blocks
constexpr int kRowStride = kStageSegs * kSegBytes;      // 288 B: TMA boxes are dense
constexpr int kStageBytes = kTileRows * kRowStride;     // 4608 = 36 x 128
constexpr int kSlots = 3;                               // tiles in flight per group
constexpr int kMaxStages = 6;

enum Epilogue { kEpiPlain = 0, kEpiRope = 2, kEpiF32 = 3 };   // kEpiF32: fp32 store (partial sums of a sharded linear)

struct Phase {
  // weights: up to three packed matrices stacked along N, or gate/up interleaved in tiles
  const uint8_t* w[3];
  int rows[3];
  int nmat;
  int interleave;        // 1: tile t = rows [8t, 8t+8) of w[0] (gate) and of w[1] (up)
  int n_total;           // rows covered by tiles (interleave: rows of one matrix)
  int K;
  int row_bytes;
  int ntiles;
  int S;                 // K-slices handled by different CTAs: a power of two dividing gridDim.x
  int s_shift;           // log2(S)
  int lane_step;         // (gridDim.x / S) * groups: (CTA, group) pairs sharing the tiles of a slice
  int lane_q, lane_r;    // ntiles - 1 = lane_q * lane_step + lane_r (host-side division)
  int segs_base, segs_extra;  // slice s has segs_base + (s < segs_extra) segments
  int max_slice_segs;
  // activations
  const void* x;         // [M, K] activation dtype
  const void* gamma;     // RMSNorm weight [K] or null
  float eps;
  // outputs
  void* y[3];            // per matrix [M, rows[i]]; interleave: y[0] = h [M, n_total]
  const void* bias[3];
  int epi[3];
  // rope
  const __half* cos_t;
  const __half* sin_t;
  const int32_t* positions;
  int head_dim, max_seq, pos_offset;
  // split-K scratch
  float* partials;       // [S][ntiles][16][MB]
  uint32_t* counters;    // [ntiles], zero between launches
  // hand-over between chained phases without a grid barrier: every 8-byte word carries its
  // payload (two 16-bit activations or one float) and the launch's sequence number, so a consumer
  // that sees the number knows the payload is this launch's (a single store publishes both)
  unsigned long long* y_tagged;   // interleave epilogue writes h here instead of y[0] (null: plain store)
  int x_tagged;                   // x points at such words: [M][K / per_word]
  int reverse;                    // tile lanes are numbered from the last (CTA, group) pair downwards
};

struct Params {
  // per phase and matrix: [rows][row_bytes / 8] of 8-byte elements, box 36 x 8 (288 B x 8 rows)
  alignas(64) CUtensorMap tmap[2][3];
  Phase ph[2];
  int nphases;
  int M;
  uint32_t* seq_ctl;     // [0] sequence number of the last complete launch, [1] CTAs finished (null: single phase)
  uint32_t flags;        // bit 0: request x before the weight stream (no overlap with the previous kernel's tail)
  unsigned long long wait_ns;   // limit of every device-side wait, in nanoseconds of %globaltimer
  int* status;
  unsigned long long* trace;  // optional: 16 globaltimer stamps per CTA (null = off)
  // tensor-parallel exchange fused into the last phase (world <= 1: off)
  char* tp_peer[kTpMaxWorld];
  int tp_rank, tp_world;
  uint32_t* tp_ctl;
  void* tp_y;
};

__device__ __forceinline__ float* tp_slot(char* base, int parity, int src) {
  return reinterpret_cast<float*>(base + kTpFlagBytes) + ((size_t)parity * kTpMaxWorld + src) * kTpSlotElems;
}
__device__ __forceinline__ uint32_t* tp_flag(char* base, int src, int idx) {
  return reinterpret_cast<uint32_t*>(base) + src * kTpFlagsPerRank + idx;
}

// Shared-memory plan (bytes), identical on host and device.
struct SmemPlan {
  int stages;        // per compute warp
  int x_stride;      // bytes per (batch, part) row of the int8 x slice
  int aux_stride;    // words per batch column of the sum table
  int seg_stride;    // floats per batch column of the delta table
  int off_ring, off_x, off_aux, off_delta, off_slots, off_tile, off_params, off_misc, total;
};
// aux words per segment: Q4_K 4 (pair sums hi|lo), Q4_0 8 (4 hi words + 4 lo words)
// Two int8 rows (hi, lo) per batch row in both fragment mappings.  pairs: the rows are padded so
// that hi and lo sit 16 bytes apart modulo 128 (the batch <= 2 mapping reads 16 bytes per thread).
__host__ __device__ inline SmemPlan make_plan(int ng, int stages, int max_slice_segs, int M, int MB, int aux_per_seg, int pairs) {
  SmemPlan p;
  p.stages = stages;
  p.x_stride = max_slice_segs * 256 + (pairs ? 16 : 32);
  p.aux_stride = max_slice_segs * aux_per_seg + 4;
  p.seg_stride = max_slice_segs;
  p.off_ring = 0;
  p.off_x = ng * kGroupWarps * stages * kStageBytes;
  p.off_aux = p.off_x + 2 * M * p.x_stride;
  p.off_delta = p.off_aux + M * p.aux_stride * 4;
  p.off_slots = (p.off_delta + M * p.seg_stride * 4 + 15) & ~15;
  p.off_tile = p.off_slots + ng * kSlots * kGroupWarps * kTileRows * MB * 4;
  p.off_params = (p.off_tile + ng * kSlots * kTileRows * MB * 4 + 127) & ~127;
  p.off_misc = (p.off_params + (int)sizeof(Params) + 127) & ~127;
  p.total = p.off_misc + 2048;
  return p;
}

struct Misc {
  unsigned long long full[2 * kGroupWarps][kMaxStages];   // one mbarrier per compute warp and stage
  float redbuf[2 * kGroupWarps * 8];   // per-warp, per-batch-row partial sums of squares
  int slot_free[2][kSlots];   // highest tile number that may write into the slot
  int slot_cnt[2][kSlots];    // warps that have delivered their partial sums for the slot's tile
  float rinv[8];              // 1 / rms of each batch row (x prologue, batch > 2)
  int dead;
};
static_assert(sizeof(Misc) <= 2048, "Misc must fit its smem slot");

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Every device-side wait goes through here: polls `ready` until it holds or limit_ns nanoseconds
// have passed (the clock is only read after the first 64 polls failed).  False = gave up.
template <typename F>
__device__ __forceinline__ bool bounded_wait(F&& ready, unsigned long long limit_ns) {
#pragma unroll 1
  for (int i = 0; i < 64; i++)
    if (ready()) return true;
  const unsigned long long t0 = global_ns();
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; i++)
      if (ready()) return true;
    if (global_ns() - t0 > limit_ns) return false;
  }
}
// Bounded wait: false (and *dead set) when the limit is reached.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* dead, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  if (bounded_wait([&] { return mbar_try_wait(bar, parity); }, limit_ns)) return true;
  *dead = 1;
  return false;
}
// One box of the 2-D tensor map: x in 8-byte elements (even: 16-byte rule), y in rows.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// The MMAs are pure functions of their register operands: not volatile, so the compiler may
// schedule them among the loads and the logic of neighbouring sub-blocks.
__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t pack_half2(__half lo, __half hi) {
  return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

__device__ __forceinline__ int slice_segs(const Phase& ph, int ks) { return ph.segs_base + (ks < ph.segs_extra ? 1 : 0); }
__device__ __forceinline__ int slice_seg0(const Phase& ph, int ks) {
  return ks * ph.segs_base + (ks < ph.segs_extra ? ks : ph.segs_extra);
}

// Pointer to the packed row r (0..15) of tile t.
__device__ __forceinline__ const uint8_t* tile_row(const Phase& ph, int t, int r) {
  if (ph.interleave) {
    int row = 8 * t + (r & 7);
    if (row >= ph.n_total) row = ph.n_total - 1;
    return ph.w[r >> 3] + (size_t)row * ph.row_bytes;
  }
  int R = kTileRows * t + r;
  if (R >= ph.n_total) R = ph.n_total - 1;
  int m = 0;
  if (ph.nmat > 1 && R >= ph.rows[0]) { R -= ph.rows[0]; m = 1; if (ph.nmat > 2 && R >= ph.rows[1]) { R -= ph.rows[1]; m = 2; } }
  return ph.w[m] + (size_t)R * ph.row_bytes;
}

// Tiles of one (CTA, group) in a phase: t = first + i * step, i = 0 .. count-1.  The CTA
// works on K-slice cta % S; the gridDim.x / S CTAs of a slice, times NG groups, share the tiles.
struct TileLane { int first, step, count; };
__device__ __forceinline__ TileLane tile_lane(const Phase& ph, int cta, int G, int group, int ng) {
  TileLane tl;
  tl.step = ph.lane_step;
  tl.first = (cta >> ph.s_shift) * ng + group;
  if (ph.reverse) tl.first = tl.step - 1 - tl.first;
  // floor((ntiles - 1 - first) / step) + 1 without a division (first < step)
  tl.count = tl.first <= ph.lane_r ? ph.lane_q + 1 : ph.lane_q;
  return tl;
}

// Eight consecutive activations -> fp32 (16-byte vector loads when aligned), L2-coherent.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
      const uint4 u = __ldcg(reinterpret_cast<const uint4*>(p));
      const T* h = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = Act<T>::to_f(h[i]);
      return;
    }
  } else {
    if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
      const float4 a = __ldcg(reinterpret_cast<const float4*>(p)), b = __ldcg(reinterpret_cast<const float4*>(p) + 1);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; i++) v[i] = Act<T>::to_f(__ldcg(p + i));
}

// ---- x prologue --------------------------------------------------------------------------
// The CTA's K-slice of x -> [RMSNorm, round to T] -> 16-bit fixed point per 256-element
// segment, stored as hi / lo signed bytes in MMA k order, plus the per-segment scale and the
// per-sub-block sums the offset / min term needs.  One warp per segment, 8 consecutive
// elements per lane; with a segment per warp the slice is read from L2 exactly once.
// PAIRS: the batch <= 2 mapping (see segment_mma_pairs) shares the layout of x (a hi row and a
// lo row per batch row) and keeps the pair sums as plain floats.  pre / gpre: x and gamma of (batch 0, segment = warp) loaded by the caller
// before it queued the weight prefetch (loads issued later wait behind it in the LSU).
template <int QT, typename T, bool PAIRS>
__device__ __forceinline__ void x_prologue(const Phase& ph, const SmemPlan& plan, uint8_t* smem, Misc* misc,
                                           int M, int nseg, int seg0, int nwarps, bool have_pre,
                                           const float (&pre)[8], const float (&gpre)[8], unsigned long long* tr,
                                           uint32_t seq, unsigned long long wait_ns) {
  auto tstamp = [&](int i) { if (tr && threadIdx.x == 0) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); tr[i] = t; } };
  constexpr int AUXW = (QT == MLXR_Q4_K) ? 4 : 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k0 = seg0 * 256;
  const T* xg = reinterpret_cast<const T*>(ph.x);
  const T* gam = reinterpret_cast<const T*>(ph.gamma);
  uint32_t* aux = reinterpret_cast<uint32_t*>(smem + plan.off_aux);
  float* delta = reinterpret_cast<float*>(smem + plan.off_delta);
  const bool whole_row = (nseg * 256 == ph.K);
  // Fixed-point conversion and stores of one (batch row, segment): v holds the segment's eight
  // activations of this lane, already normalised and rounded to T.
  auto emit = [&](int m, int sg, float (&v)[8]) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
    // warp-wide maximum in one instruction: non-negative floats order like their bit patterns
    // (NaN and Inf sort above every finite value)
    amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));
    // x ~ dl * xi with |xi| <= 32000; a non-finite block poisons its outputs with NaN
    float dl = 1.0f, inv = 0.0f;
    if (!(amax <= 3.0e38f)) { dl = __int_as_float(0x7fc00000); }
    else if (amax > 0.0f) { dl = amax * (1.0f / 32000.0f); inv = 32000.0f / amax; }
    int ssum = 0;
    uint32_t hi_e = 0, hi_o = 0, lo_e = 0, lo_o = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      int q16 = __float2int_rn(v[i] * inv);
      q16 = max(-32000, min(32000, q16));
      ssum += q16;
      const int h8 = (q16 + 128) >> 8, l8 = q16 - (h8 << 8);   // q16 = 256*h8 + l8, both in [-128,127]
      const uint32_t hb = (uint32_t)(h8 & 0xFF), lb = (uint32_t)(l8 & 0xFF);
      if (i & 1) { hi_o |= hb << (8 * (i >> 1)); lo_o |= lb << (8 * (i >> 1)); }
      else       { hi_e |= hb << (8 * (i >> 1)); lo_e |= lb << (8 * (i >> 1)); }
    }
    // bytes of an 8-group are stored as (e0,e2,e4,e6 | e1,e3,e5,e7): the MMA k order
    {
      uint8_t* xrow = smem + plan.off_x + (size_t)(2 * m) * plan.x_stride + sg * 256 + lane * 8;
      *reinterpret_cast<uint2*>(xrow) = make_uint2(hi_e, hi_o);
      *reinterpret_cast<uint2*>(xrow + plan.x_stride) = make_uint2(lo_e, lo_o);
    }
    // sums of xi per 32-element sub-block (this lane's eight elements lie in sub-block lane / 4):
    // one warp-wide integer reduction per sub-block
    int sb[8];
#pragma unroll
    for (int j = 0; j < 8; j++) sb[j] = __reduce_add_sync(0xffffffffu, (lane >> 2) == j ? ssum : 0);
    if (lane == 0) delta[m * plan.seg_stride + sg] = dl;
    uint32_t* arow = aux + (size_t)m * plan.aux_stride + sg * AUXW;
    if (lane < 4) {
      if constexpr (PAIRS) {
        // exact integer sums over the sub-blocks of each (scale, min) pair, as floats
        const int ps = lane == 0 ? sb[0] + sb[2] + sb[3] : lane == 1 ? sb[1] : lane == 2 ? sb[4] + sb[6] + sb[7] : sb[5];
        arow[lane] = __float_as_uint((float)ps);
      } else if constexpr (QT == MLXR_Q4_K) {
        // sums over the sub-blocks that share a (scale, min) pair, in units of 2^10
        const int ps = lane == 0 ? sb[0] + sb[2] + sb[3] : lane == 1 ? sb[1] : lane == 2 ? sb[4] + sb[6] + sb[7] : sb[5];
        const float f = (float)ps * (1.0f / 1024.0f);
        const __half h = __float2half_rn(f);
        arow[lane] = pack_half2(h, __float2half_rn(f - __half2float(h)));
      } else {
        // -8 * sum per sub-block in units of 2^10: word j = sub-blocks (2j, 2j+1); hi words, then lo words
        const int a = lane == 0 ? sb[0] : lane == 1 ? sb[2] : lane == 2 ? sb[4] : sb[6];
        const int b = lane == 0 ? sb[1] : lane == 1 ? sb[3] : lane == 2 ? sb[5] : sb[7];
        const float fa = (float)a * (-8.0f / 1024.0f), fb = (float)b * (-8.0f / 1024.0f);
        const __half ha = __float2half_rn(fa), hb2 = __float2half_rn(fb);
        arow[lane] = pack_half2(ha, hb2);
        arow[4 + lane] = pack_half2(__float2half_rn(fa - __half2float(ha)), __float2half_rn(fb - __half2float(hb2)));
      }
    }
  };
  if (ph.x_tagged) {
    // ---- x is the previous phase's output in tagged words: poll until every word carries this
    // launch's sequence number (the producer may still be running on another SM), no barrier ----
    constexpr int PW = sizeof(T) == 2 ? 2 : 1;   // activations per tagged word
    constexpr int NV = 8 / PW / 2;               // 16-byte loads (two words each) per lane and segment
    const unsigned long long* xt = reinterpret_cast<const unsigned long long*>(ph.x);
    const int nitems = M * nseg;
    auto ld16 = [](const uint4* p) {
      uint4 r;
      asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
      return r;
    };
    for (int base = warp; base < nitems; base += 4 * nwarps) {
      uint4 raw[4][NV];
      // request up to four segments before looking at any of them
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int item = base + u * nwarps;
        if (item < nitems) {
          const int m = item / nseg, sg = item - m * nseg;
          const uint4* p = reinterpret_cast<const uint4*>(xt + ((size_t)m * ph.K + k0 + sg * 256 + lane * 8) / PW);
#pragma unroll
          for (int q = 0; q < NV; q++) raw[u][q] = ld16(p + q);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int item = base + u * nwarps;
        if (item >= nitems) break;   // uniform per warp
        const int m = item / nseg, sg = item - m * nseg;
        const uint4* p = reinterpret_cast<const uint4*>(xt + ((size_t)m * ph.K + k0 + sg * 256 + lane * 8) / PW);
        auto tagged = [&] {
          bool good = true;
#pragma unroll
          for (int q = 0; q < NV; q++) good = good && raw[u][q].y == seq && raw[u][q].w == seq;
          return good;
        };
        if (!tagged()) {
          const bool ok = bounded_wait([&] {
#pragma unroll
            for (int q = 0; q < NV; q++) raw[u][q] = ld16(p + q);
            return tagged();
          }, wait_ns);
          if (!ok) misc->dead = 1;
        }
        __syncwarp();
        float v[8];
#pragma unroll
        for (int q = 0; q < NV; q++) {
          if constexpr (PW == 2) {
            const T* a = reinterpret_cast<const T*>(&raw[u][q].x);
            const T* b = reinterpret_cast<const T*>(&raw[u][q].z);
            v[4 * q + 0] = Act<T>::to_f(a[0]); v[4 * q + 1] = Act<T>::to_f(a[1]);
            v[4 * q + 2] = Act<T>::to_f(b[0]); v[4 * q + 3] = Act<T>::to_f(b[1]);
          } else {
            v[2 * q + 0] = __uint_as_float(raw[u][q].x);
            v[2 * q + 1] = __uint_as_float(raw[u][q].z);
          }
        }
        emit(m, sg, v);
      }
    }
    return;
  }
  if (M > 2) {
    // ---- batch rows in parallel: (row, segment) items are dealt to the warps round-robin ----
    if (gam) {
      const int nrow = ph.K >> 8;
      float part[8];
#pragma unroll
      for (int mm = 0; mm < 8; mm++) part[mm] = 0.0f;
      for (int item = warp; item < M * nrow; item += nwarps) {
        const int m = item / nrow, sgw = item - m * nrow;
        float v[8];
        load8(xg + (size_t)m * ph.K + sgw * 256 + lane * 8, v);
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) q = fmaf(v[i], v[i], q);
#pragma unroll
        for (int mm = 0; mm < 8; mm++) part[mm] += (mm == m) ? q : 0.0f;
      }
#pragma unroll
      for (int mm = 0; mm < 8; mm++) {
        const float t = warp_sum(part[mm]);
        if (lane == 0) misc->redbuf[warp * 8 + mm] = t;
      }
      __syncthreads();
      if (tid < M) {
        float tot = 0.0f;
        for (int w = 0; w < nwarps; w++) tot += misc->redbuf[w * 8 + tid];
        misc->rinv[tid] = 1.0f / sqrtf(tot / (float)ph.K + ph.eps);
      }
      __syncthreads();
      tstamp(13);
    }
    for (int item = warp; item < M * nseg; item += nwarps) {
      const int m = item / nseg, sg = item - m * nseg;
      float v[8];
      load8(xg + (size_t)m * ph.K + k0 + sg * 256 + lane * 8, v);
      if (gam) {
        float gv[8];
        load8(gam + k0 + sg * 256 + lane * 8, gv);
        const float rinv = misc->rinv[m];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = Act<T>::to_f(Act<T>::from_f(__fmul_rn(__fmul_rn(v[i], rinv), gv[i])));
      }
      emit(m, sg, v);
    }
    return;
  }
  for (int m = 0; m < M; m++) {
    const T* xrow_g = xg + (size_t)m * ph.K;
    float v0[8];            // first segment of this warp, kept across the reduction
    bool have0 = false;
    const bool use_pre = have_pre && m == 0 && warp < nseg;
    if (use_pre) {
#pragma unroll
      for (int i = 0; i < 8; i++) v0[i] = pre[i];
      have0 = true;
    }
    float rinv = 1.0f;
    if (gam) {
      float ss = 0.0f;
      if (whole_row) {
        for (int sg = warp; sg < nseg; sg += nwarps) {
          float v[8];
          if (use_pre && sg == warp) {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = v0[i];
          } else {
            load8(xrow_g + sg * 256 + lane * 8, v);
          }
#pragma unroll
          for (int i = 0; i < 8; i++) ss = fmaf(v[i], v[i], ss);
          if (sg == warp) {
#pragma unroll
            for (int i = 0; i < 8; i++) v0[i] = v[i];
            have0 = true;
          }
        }
      } else {
        for (int k = tid * 8; k < ph.K; k += blockDim.x * 8) {
          float v[8];
          load8(xrow_g + k, v);
#pragma unroll
          for (int i = 0; i < 8; i++) ss = fmaf(v[i], v[i], ss);
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) misc->redbuf[warp] = ss;
      __syncthreads();
      float tot = 0.0f;
      for (int i = 0; i < nwarps; i++) tot += misc->redbuf[i];
      rinv = 1.0f / sqrtf(tot / (float)ph.K + ph.eps);
      __syncthreads();
      tstamp(13);
    }
    for (int sg = warp; sg < nseg; sg += nwarps) {
      float v[8];
      if (have0 && sg == warp) {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v0[i];
      } else {
        load8(xrow_g + k0 + sg * 256 + lane * 8, v);
      }
      if (gam) {
        float gv[8];
        if (use_pre && sg == warp) {
#pragma unroll
          for (int i = 0; i < 8; i++) gv[i] = gpre[i];
        } else {
          load8(gam + k0 + sg * 256 + lane * 8, gv);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = Act<T>::to_f(Act<T>::from_f(__fmul_rn(__fmul_rn(v[i], rinv), gv[i])));
      }
      emit(m, sg, v);
    }
  }
}

// ---- one 256-element segment of 16 rows ---------------------------------------------------
// rl / rh: this thread's two rows (g and g+8) of the stage, at the segment's first byte.
// xb[j]: this thread's B-fragment bytes of n-tile j for the segment (null when the MMA column
// has no batch row behind it); auxp[j]: its word of the sum table (null likewise);
// dl[j]: fixed-point scale of batch column c + 4j for this segment.
template <int QT, int NT>
__device__ __forceinline__ void segment_mma(const uint8_t* rl, const uint8_t* rh, const uint8_t* const (&xb)[NT],
                                            const uint32_t* const (&auxp)[NT], const float (&dl)[NT], int lane,
                                            float (&total)[NT][2]) {
  const int c = lane & 3;
  float segacc[NT][2];
  float minacc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++) {
    segacc[j][0] = segacc[j][1] = 0.0f;
    minacc[j][0] = minacc[j][1] = minacc[j][2] = minacc[j][3] = 0.0f;
  }
  if constexpr (QT == MLXR_Q4_K) {
    const uint4 hl = *reinterpret_cast<const uint4*>(rl), hh = *reinterpret_cast<const uint4*>(rh);
    // this thread decodes (scale, min) pair c of both rows (q_gemm_dequant.metal:222-242, fields
    // read straight from the packed words); the quad shares the four scales by shuffle
    float ssl[4], ssh[4];
    uint32_t amin_lo, amin_hi;
    {
      const __half2 dl2 = *reinterpret_cast<const __half2*>(&hl.x), dh2 = *reinterpret_cast<const __half2*>(&hh.x);
      const uint32_t w2 = hl.y, w3 = hl.z, v2 = hh.y, v3 = hh.z;
      const uint32_t scl = c == 0 ? w2 : c == 1 ? (w2 >> 12) : c == 2 ? (w2 >> 24) : (w3 >> 4);
      const uint32_t sch = c == 0 ? v2 : c == 1 ? (v2 >> 12) : c == 2 ? (v2 >> 24) : (v3 >> 4);
      const uint32_t mnl = c == 0 ? (w2 >> 6) : c == 1 ? (w2 >> 18) : c == 2 ? ((w2 >> 30) | ((w3 & 15u) << 2)) : (w3 >> 10);
      const uint32_t mnh = c == 0 ? (v2 >> 6) : c == 1 ? (v2 >> 18) : c == 2 ? ((v2 >> 30) | ((v3 & 15u) << 2)) : (v3 >> 10);
      const float my_sl = __half2float(__hmul(__int2half_rn((int)(scl & 63u)), __low2half(dl2)));
      const float my_sh = __half2float(__hmul(__int2half_rn((int)(sch & 63u)), __low2half(dh2)));
      const float my_ml = __half2float(__hmul(__int2half_rn((int)(mnl & 63u)), __high2half(dl2)));
      const float my_mh = __half2float(__hmul(__int2half_rn((int)(mnh & 63u)), __high2half(dh2)));
      // w = (q - 8) * ss + sm = q * ss + (sm - 8 ss): the second term times sum(x)
      const __half ol = __float2half_rn(fmaf(-8.0f, my_sl, my_ml));
      const __half oh = __float2half_rn(fmaf(-8.0f, my_sh, my_mh));
      amin_lo = pack_half2(ol, ol);
      amin_hi = pack_half2(oh, oh);
#pragma unroll
      for (int p = 0; p < 4; p++) {
        ssl[p] = __shfl_sync(0xffffffffu, my_sl, (lane & ~3) | p);
        ssh[p] = __shfl_sync(0xffffffffu, my_sh, (lane & ~3) | p);
      }
    }
    // sub-blocks in the order that keeps those sharing a (scale, min) pair together
    constexpr int order[8] = {0, 2, 3, 1, 4, 6, 7, 5};
    constexpr int pair_of[8] = {0, 0, 0, 1, 2, 2, 2, 3};
    constexpr bool last_of_pair[8] = {false, false, true, true, false, false, true, true};
    const uint32_t* ql = reinterpret_cast<const uint32_t*>(rl + 16) + c;
    const uint32_t* qh = reinterpret_cast<const uint32_t*>(rh + 16) + c;
    uint32_t wl[8], wh[8];
#pragma unroll
    for (int s = 0; s < 8; s++) { wl[s] = ql[4 * s]; wh[s] = qh[4 * s]; }
    int acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int s = order[i];
      // even nibbles (elements 8c+0,2,4,6) and odd nibbles (8c+1,3,5,7) as u8x4
      const uint32_t a0 = wl[s] & 0x0f0f0f0fu, a2 = (wl[s] >> 4) & 0x0f0f0f0fu;
      const uint32_t a1 = wh[s] & 0x0f0f0f0fu, a3 = (wh[s] >> 4) & 0x0f0f0f0fu;
#pragma unroll
      for (int j = 0; j < NT; j++) {
        uint2 b = make_uint2(0u, 0u);
        if (xb[j]) b = *reinterpret_cast<const uint2*>(xb[j] + 32 * s);
        imma16832(acc[j], a0, a1, a2, a3, b.x, b.y);
      }
      if (last_of_pair[i]) {
        const int p = pair_of[i];
#pragma unroll
        for (int j = 0; j < NT; j++) {
          // columns 2c, 2c+1 of this thread = hi and lo byte sums of batch c (+4j)
          segacc[j][0] = fmaf(ssl[p], (float)(acc[j][0] * 256 + acc[j][1]), segacc[j][0]);
          segacc[j][1] = fmaf(ssh[p], (float)(acc[j][2] * 256 + acc[j][3]), segacc[j][1]);
          acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0;
        }
      }
    }
    // offset + min term: sum_p (sm_p - 8 ss_p) * Sx_p, Sx_p as hi + lo halves in column 2*batch
#pragma unroll
    for (int j = 0; j < NT; j++) {
      const uint32_t b = auxp[j] ? auxp[j][c] : 0u;
      mma1688(minacc[j], amin_lo, amin_hi, b);
    }
  } else {  // Q4_0: 8 blocks of 18 B; scale at +18s, nibbles at +18s+2
    const uint16_t* hl16 = reinterpret_cast<const uint16_t*>(rl);
    const uint16_t* hh16 = reinterpret_cast<const uint16_t*>(rh);
#pragma unroll
    for (int s = 0; s < 8; s++) {
      uint32_t wl, wh;
      if (s & 1) {  // 18s+2 is 4-byte aligned
        wl = *reinterpret_cast<const uint32_t*>(rl + 18 * s + 2 + 4 * c);
        wh = *reinterpret_cast<const uint32_t*>(rh + 18 * s + 2 + 4 * c);
      } else {      // straddles two words
        const uint32_t* pl = reinterpret_cast<const uint32_t*>(rl + 18 * s + 4 * c);
        const uint32_t* ph = reinterpret_cast<const uint32_t*>(rh + 18 * s + 4 * c);
        wl = __funnelshift_r(pl[0], pl[1], 16);
        wh = __funnelshift_r(ph[0], ph[1], 16);
      }
      const float fl = __half2float(__ushort_as_half(hl16[9 * s]));
      const float fh = __half2float(__ushort_as_half(hh16[9 * s]));
      const uint32_t a0 = wl & 0x0f0f0f0fu, a2 = (wl >> 4) & 0x0f0f0f0fu;
      const uint32_t a1 = wh & 0x0f0f0f0fu, a3 = (wh >> 4) & 0x0f0f0f0fu;
#pragma unroll
      for (int j = 0; j < NT; j++) {
        int acc[4] = {0, 0, 0, 0};
        uint2 b = make_uint2(0u, 0u);
        if (xb[j]) b = *reinterpret_cast<const uint2*>(xb[j] + 32 * s);
        imma16832(acc, a0, a1, a2, a3, b.x, b.y);
        segacc[j][0] = fmaf(fl, (float)(acc[0] * 256 + acc[1]), segacc[j][0]);
        segacc[j][1] = fmaf(fh, (float)(acc[2] * 256 + acc[3]), segacc[j][1]);
      }
    }
    // -8 * sum_s d_s * Sx_s: A = the scales of sub-blocks 2c, 2c+1 (exact in half)
    const uint32_t al = (uint32_t)hl16[18 * c] | ((uint32_t)hl16[18 * c + 9] << 16);
    const uint32_t ah = (uint32_t)hh16[18 * c] | ((uint32_t)hh16[18 * c + 9] << 16);
#pragma unroll
    for (int j = 0; j < NT; j++) {
      const uint32_t bh = auxp[j] ? auxp[j][c] : 0u, bl = auxp[j] ? auxp[j][4 + c] : 0u;
      mma1688(minacc[j], al, ah, bh);
      mma1688(minacc[j], al, ah, bl);
    }
  }
  // fold the segment: units are delta (per batch column and segment)
#pragma unroll
  for (int j = 0; j < NT; j++) {
    total[j][0] = fmaf(dl[j], fmaf(1024.0f, minacc[j][0], segacc[j][0]), total[j][0]);
    total[j][1] = fmaf(dl[j], fmaf(1024.0f, minacc[j][2], segacc[j][1]), total[j][1]);
  }
}

// ---- the same for batch <= 2: pairs in the MMA columns (Q4_K) -----------------------------------
// MMA column 2p + part of n-tile j stands for batch j's x restricted to the sub-blocks of (scale,
// min) pair p, so one accumulation runs over the whole 256-block with no reset, and thread (g, c)
// ends up with the hi / lo sums of pair c for rows g and g+8: it scales them with the pair it
// decoded itself -- no shuffles.  Thread c feeds the words of sub-block c (then 4+c), which lets
// weights and x come in 128-bit loads.  The restriction costs nothing: a thread's B fragment for
// column g covers exactly sub-block c (or 4+c), so it is either that sub-block's x bytes or zero,
// decided by two per-thread constants (keep0 / keep1); x is stored once (hi row, lo row).
// The two halves of the block accumulate independently (two short MMA chains instead of one).
// The four threads of a quad hold different pairs' partial sums; the epilogue warp adds them.
// x0: this lane's x row (part g & 1) of batch 0 at the segment, + 32 c; sx0: pair sums of batch 0
// at the segment, + c; dl0: delta of batch 0 at the segment.
template <int NT>
__device__ __forceinline__ void segment_mma_pairs(const uint8_t* rl, const uint8_t* rh, const uint8_t* x0, int x_batch_stride,
                                                  const float* sx0, int aux_stride, const float* dl0, int seg_stride,
                                                  int c, int sh1, int sh2, bool keep0, bool keep1, float (&total)[NT][2]) {
  const uint4 hl = *reinterpret_cast<const uint4*>(rl), hh = *reinterpret_cast<const uint4*>(rh);
  uint4 wl[2], wh[2];
  wl[0] = *reinterpret_cast<const uint4*>(rl + 16 + 16 * c);
  wl[1] = *reinterpret_cast<const uint4*>(rl + 80 + 16 * c);
  wh[0] = *reinterpret_cast<const uint4*>(rh + 16 + 16 * c);
  wh[1] = *reinterpret_cast<const uint4*>(rh + 80 + 16 * c);
  int acc[2][NT][4];
#pragma unroll
  for (int h = 0; h < 2; h++)
#pragma unroll
    for (int j = 0; j < NT; j++) acc[h][j][0] = acc[h][j][1] = acc[h][j][2] = acc[h][j][3] = 0;
#pragma unroll
  for (int h = 0; h < 2; h++) {
    const bool keep = h ? keep1 : keep0;
    uint4 xa[NT], xb[NT];
#pragma unroll
    for (int j = 0; j < NT; j++) {
      xa[j] = make_uint4(0u, 0u, 0u, 0u);
      xb[j] = make_uint4(0u, 0u, 0u, 0u);
      if (keep) {
        xa[j] = *reinterpret_cast<const uint4*>(x0 + (size_t)j * x_batch_stride + 128 * h);
        xb[j] = *reinterpret_cast<const uint4*>(x0 + (size_t)j * x_batch_stride + 128 * h + 16);
      }
    }
    const uint32_t wlw[4] = {wl[h].x, wl[h].y, wl[h].z, wl[h].w}, whw[4] = {wh[h].x, wh[h].y, wh[h].z, wh[h].w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t a0 = wlw[i] & 0x0f0f0f0fu, a2 = (wlw[i] >> 4) & 0x0f0f0f0fu;
      const uint32_t a1 = whw[i] & 0x0f0f0f0fu, a3 = (whw[i] >> 4) & 0x0f0f0f0fu;
#pragma unroll
      for (int j = 0; j < NT; j++) {
        const uint32_t b0 = i == 0 ? xa[j].x : i == 1 ? xa[j].z : i == 2 ? xb[j].x : xb[j].z;
        const uint32_t b1 = i == 0 ? xa[j].y : i == 1 ? xa[j].w : i == 2 ? xb[j].y : xb[j].w;
        imma16832(acc[h][j], a0, a1, a2, a3, b0, b1);
      }
    }
  }
  // (scale, min) pair c of both rows: 6-bit fields at bit 12c (scale) and 12c + 6 (min) of the
  // 48 packed bits scales[0..5] (q_gemm_dequant.metal:222-242)
  const uint32_t ul = __funnelshift_r(hl.y, hl.z, sh1) >> sh2, uh = __funnelshift_r(hh.y, hh.z, sh1) >> sh2;
  const __half2 dl2 = *reinterpret_cast<const __half2*>(&hl.x), dh2 = *reinterpret_cast<const __half2*>(&hh.x);
  const float ss_l = __half2float(__hmul(__int2half_rn((int)(ul & 63u)), __low2half(dl2)));
  const float ss_h = __half2float(__hmul(__int2half_rn((int)(uh & 63u)), __low2half(dh2)));
  const float sm_l = __half2float(__hmul(__int2half_rn((int)((ul >> 6) & 63u)), __high2half(dl2)));
  const float sm_h = __half2float(__hmul(__int2half_rn((int)((uh >> 6) & 63u)), __high2half(dh2)));
  // w = (q - 8) * ss + sm = q * ss + (sm - 8 ss); the second term multiplies sum(x) of the pair
  const float of_l = fmaf(-8.0f, ss_l, sm_l), of_h = fmaf(-8.0f, ss_h, sm_h);
#pragma unroll
  for (int j = 0; j < NT; j++) {
    const float sx = sx0[(size_t)j * aux_stride];
    const float dl = dl0[(size_t)j * seg_stride];
    const float v0 = (float)((acc[0][j][0] + acc[1][j][0]) * 256 + (acc[0][j][1] + acc[1][j][1]));
    const float v1 = (float)((acc[0][j][2] + acc[1][j][2]) * 256 + (acc[0][j][3] + acc[1][j][3]));
    total[j][0] = fmaf(dl, fmaf(ss_l, v0, of_l * sx), total[j][0]);
    total[j][1] = fmaf(dl, fmaf(ss_h, v1, of_h * sx), total[j][1]);
  }
}

// ---- tile epilogue (one warp) --------------------------------------------------------------
// tile[row][col] holds the complete sums of this CTA's K-slice for 16 rows x MB batch columns.
template <typename T, int MB>
__device__ __forceinline__ void tile_epilogue(const Params& P, const Phase& ph, float* tile, int t, int ks, int lane,
                                              uint32_t tp_seq, uint32_t seq) {
  const int M = P.M;
  bool do_epilogue = true;
  if (ph.S > 1) {
    // split-K over CTAs: park the partial; the last slice to arrive reduces all of them
    const size_t slab = (size_t)ph.ntiles * kTileRows * MB;
    float* gm = ph.partials + (size_t)ks * slab + (size_t)t * kTileRows * MB;
    for (int e = lane; e < kTileRows * MB; e += 32) __stcg(&gm[e], tile[e]);
    __threadfence();
    __syncwarp();
    int lastk = 0;
    if (lane == 0) {
      const uint32_t prev = atomicAdd(&ph.counters[t], 1u);
      lastk = (prev == (uint32_t)ph.S - 1u);
      if (lastk) ph.counters[t] = 0u;   // self-cleaning for the next launch
      __threadfence();
    }
    lastk = __shfl_sync(0xffffffffu, lastk, 0);
    do_epilogue = lastk != 0;
    if (do_epilogue) {
      for (int e = lane; e < kTileRows * MB; e += 32) {
        float v = 0.0f;
        for (int s2 = 0; s2 < ph.S; s2++) v += __ldcg(&ph.partials[(size_t)s2 * slab + (size_t)t * kTileRows * MB + e]);
        tile[e] = v;
      }
      __syncwarp();
    }
  }
  if (!do_epilogue) return;
  if (ph.interleave && ph.y_tagged) {
    // the same, published as tagged words {payload, sequence number}: one 8-byte store makes the
    // values and their validity visible together, so the next phase needs neither fence nor barrier
    auto hval = [&](int r, int m) {
      const float gv = Act<T>::to_f(Act<T>::from_f(tile[r * MB + m]));
      const float uv = Act<T>::to_f(Act<T>::from_f(tile[(r + 8) * MB + m]));
      return Act<T>::from_f(swish_f(gv) * uv);
    };
    if constexpr (sizeof(T) == 2) {
      for (int e = lane; e < 4 * MB; e += 32) {
        const int rp = e / MB, m = e % MB;
        const int col = 8 * t + 2 * rp;
        if (m < M && col < ph.n_total) {
          const T h0 = hval(2 * rp, m), h1 = hval(2 * rp + 1, m);
          const uint32_t payload = (uint32_t)*reinterpret_cast<const uint16_t*>(&h0) | ((uint32_t)*reinterpret_cast<const uint16_t*>(&h1) << 16);
          const unsigned long long word = (unsigned long long)payload | ((unsigned long long)seq << 32);
          asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(ph.y_tagged + ((size_t)m * ph.n_total + col) / 2), "l"(word) : "memory");
        }
      }
    } else {
      for (int e = lane; e < 8 * MB; e += 32) {
        const int r = e / MB, m = e % MB;
        const int col = 8 * t + r;
        if (m < M && col < ph.n_total) {
          const float h0 = Act<float>::to_f(hval(r, m));
          const unsigned long long word = (unsigned long long)__float_as_uint(h0) | ((unsigned long long)seq << 32);
          asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(ph.y_tagged + (size_t)m * ph.n_total + col), "l"(word) : "memory");
        }
      }
    }
  } else if (ph.interleave) {
    // rows 0..7 gate, 8..15 up of the same 8 intermediate indices: h = SiLU(g) * u
    for (int e = lane; e < 8 * MB; e += 32) {
      const int r = e / MB, m = e % MB;
      const int col = 8 * t + r;
      if (m < M && col < ph.n_total) {
        const float gv = Act<T>::to_f(Act<T>::from_f(tile[r * MB + m]));
        const float uv = Act<T>::to_f(Act<T>::from_f(tile[(r + 8) * MB + m]));
        reinterpret_cast<T*>(ph.y[0])[(size_t)m * ph.n_total + col] = Act<T>::from_f(swish_f(gv) * uv);
      }
    }
  } else {
    // pairs of adjacent rows (2j, 2j+1): plain store or RoPE rotation
    for (int e = lane; e < 8 * MB; e += 32) {
      const int jj = e / MB, m = e % MB;
      int R = kTileRows * t + 2 * jj;
      if (m >= M || R >= ph.n_total) continue;
      int mat = 0;
      if (ph.nmat > 1 && R >= ph.rows[0]) { R -= ph.rows[0]; mat = 1; if (ph.nmat > 2 && R >= ph.rows[1]) { R -= ph.rows[1]; mat = 2; } }
      const bool has_odd = R + 1 < ph.rows[mat];
      float ve = tile[(2 * jj) * MB + m], vo = tile[(2 * jj + 1) * MB + m];
      const T* bias = reinterpret_cast<const T*>(ph.bias[mat]);
      if (bias) { ve += Act<T>::to_f(bias[R]); if (has_odd) vo += Act<T>::to_f(bias[R + 1]); }
      if (ph.epi[mat] == kEpiF32) {
        const size_t off = (size_t)m * ph.rows[mat] + R;
        if (P.tp_world > 1) {
          // straight into slot `rank` of every rank's exchange buffer (plain peer stores)
          for (int pr = 0; pr < P.tp_world; pr++) {
            float* of = tp_slot(P.tp_peer[(P.tp_rank + 1 + pr) % P.tp_world], (int)(tp_seq & 1u), P.tp_rank) + off;
            of[0] = ve;
            if (has_odd) of[1] = vo;
          }
        } else {
          float* of = reinterpret_cast<float*>(ph.y[mat]) + off;
          of[0] = ve;
          if (has_odd) of[1] = vo;
        }
        continue;
      }
      T* out = reinterpret_cast<T*>(ph.y[mat]) + (size_t)m * ph.rows[mat] + R;
      if (ph.epi[mat] == kEpiRope) {
        const float qe = Act<T>::to_f(Act<T>::from_f(ve)), qo = Act<T>::to_f(Act<T>::from_f(vo));
        const long long pos = (long long)ph.positions[m] + ph.pos_offset;
        if (pos < 0 || pos >= ph.max_seq) { atomicExch(P.status, MLXR_ERR_SHAPE); continue; }
        const int pairs = ph.head_dim >> 1, pi = (R % ph.head_dim) >> 1;
        const float cs = __half2float(ph.cos_t[(size_t)pos * pairs + pi]);
        const float sn = __half2float(ph.sin_t[(size_t)pos * pairs + pi]);
        out[0] = Act<T>::from_f(__fsub_rn(__fmul_rn(qe, cs), __fmul_rn(qo, sn)));
        out[1] = Act<T>::from_f(__fadd_rn(__fmul_rn(qo, cs), __fmul_rn(qe, sn)));
      } else {
        out[0] = Act<T>::from_f(ve);
        if (has_odd) out[1] = Act<T>::from_f(vo);
      }
    }
    if (P.tp_world > 1 && ph.epi[0] == kEpiF32 && ph.S > 1) {
      // K split over CTAs: which CTA finishes a tile differs from rank to rank, so the flag is
      // per tile: the warp's stores to the peers, then this tile's flag there (release at system scope)
      __syncwarp();
      if (lane < P.tp_world) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(tp_flag(P.tp_peer[lane], P.tp_rank, t)), "r"(tp_seq) : "memory");
      }
    }
  }
}

// ---- the kernel ------------------------------------------------------------------------------
// PAIRS: the batch <= 2 fragment mapping (Q4_K only, NT = batch); otherwise batch x {hi, lo}
// in the MMA columns, four batch rows per n-tile.
template <int QT, typename T, int NT, int NG, bool PAIRS>
__global__ void __launch_bounds__(NG * kGroupWarps * 32, 1)
decode_kernel(const __grid_constant__ Params Pg, const __grid_constant__ SmemPlan plan) {
  extern __shared__ __align__(128) uint8_t smem[];
  // the TMA unit fetches a tensor map on first use: ask for them before anything else
  if (threadIdx.x < 6) {
    const int pi = threadIdx.x / 3, mi = threadIdx.x % 3;
    if (pi < Pg.nphases && mi < Pg.ph[pi].nmat)
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&Pg.tmap[pi][mi])) : "memory");
  }
  // Warm the TLB and L2 for the activations of every phase (a prefetch only: the data itself is
  // read after griddepcontrol.wait) and for the norm weight; first-touch page walks otherwise
  // cost each phase's prologue about a microsecond.
  {
    const int t = (int)threadIdx.x - 32;
    if (t >= 0 && t < 64 * 2 * Pg.nphases) {
      const int pi = t / 128, which = (t / 64) & 1, line = t % 64;
      const char* base = reinterpret_cast<const char*>(which ? Pg.ph[pi].gamma : Pg.ph[pi].x);
      const size_t bytes = (size_t)(which ? 1 : Pg.M) * Pg.ph[pi].K * sizeof(T);
      if (base && (size_t)line * 128 < bytes) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (size_t)line * 128));
    }
  }
  // The parameter block is copied to shared memory by all threads at once: read piecemeal from
  // the constant bank, its ~20 cache lines miss one after another (measured: 2.8 us of set-up).
  // Only the tensor maps are used in place (the TMA unit reads them through their address).
  {
    uint32_t* dst = reinterpret_cast<uint32_t*>(smem + plan.off_params);
    const uint32_t* src = reinterpret_cast<const uint32_t*>(&Pg);
    for (int i = threadIdx.x; i < (int)(sizeof(Params) / 4); i += blockDim.x) dst[i] = src[i];
  }
  __syncthreads();
  const Params& P = *reinterpret_cast<const Params*>(smem + plan.off_params);
  constexpr int MB = 4 * NT;                       // batch columns held (two MMA columns each)
  constexpr int AUXW = (QT == MLXR_Q4_K) ? 4 : 8;
  constexpr int kComputeWarps = NG * kGroupWarps;
  constexpr int kAllWarps = kComputeWarps;
  Misc* misc = reinterpret_cast<Misc*>(smem + plan.off_misc);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  // MMA row g is fed from tile row rg = g with its two low bits swapped: the two row groups of a
  // quarter warp then sit 2 rows = 576 bytes = 16 banks apart in the dense TMA box, which makes
  // the 128-bit weight loads conflict-free (adjacent rows, 288 bytes apart, would collide)
  const int rg = (g & 4) | ((g & 1) << 1) | ((g >> 1) & 1);
  const int G = gridDim.x, cta = blockIdx.x;
  const int M = P.M;
  const int D = plan.stages;
  const int group = warp / kGroupWarps;
  const int wg = warp % kGroupWarps;               // compute warp's index in its group

  if (tid == 0) {
    misc->dead = 0;
    for (int gi = 0; gi < 2; gi++)
      for (int sl = 0; sl < kSlots; sl++) { misc->slot_free[gi][sl] = kSlots - 1; misc->slot_cnt[gi][sl] = 0; }
    for (int w = 0; w < kComputeWarps; w++)
      for (int st = 0; st < D; st++) mbar_init(smem_u32(&misc->full[w][st]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  auto stamp = [&](int i) {
    if (P.trace && tid == 0) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
      P.trace[(size_t)cta * 16 + i] = t;
    }
  };
  stamp(0);

  float* slots = reinterpret_cast<float*>(smem + plan.off_slots) + (size_t)group * kSlots * kGroupWarps * kTileRows * MB;
  float* tiles = reinterpret_cast<float*>(smem + plan.off_tile) + (size_t)group * kSlots * kTileRows * MB;
  const uint32_t* aux = reinterpret_cast<const uint32_t*>(smem + plan.off_aux);
  const float* delta = reinterpret_cast<const float*>(smem + plan.off_delta);

  // tiles this group handles over the whole launch (slot hand-back is skipped at the end)
  int total_q = 0;
  for (int p = 0; p < P.nphases; p++) total_q += tile_lane(P.ph[p], cta, G, group, NG).count;

  // ---- this compute warp's private copy stream: (phase, tile, chunk) in consumption order ----
  const uint32_t ring = smem_u32(smem + plan.off_ring) + warp * D * kStageBytes;
  const uint8_t* ring_g = smem + plan.off_ring + (size_t)warp * D * kStageBytes;
  int i_phs = 0, i_tile = 0, i_ch = 0, i_nch = 0, i_seg_first = 0, i_nsw = 0;
  TileLane i_tl = {0, 1, 0};
  auto enter_phase = [&]() {   // first phase >= i_phs with work for this warp
    while (i_phs < P.nphases) {
      const Phase& ph = P.ph[i_phs];
      const int ks = (cta & (ph.S - 1)), nseg = slice_segs(ph, ks);
      const int s0 = (wg * nseg) / kGroupWarps, s1 = ((wg + 1) * nseg) / kGroupWarps;
      i_nsw = s1 - s0;
      i_seg_first = slice_seg0(ph, ks) + s0;
      i_nch = (i_nsw + kStageSegs - 1) / kStageSegs;
      i_tl = tile_lane(ph, cta, G, group, NG);
      i_tile = 0;
      i_ch = 0;
      if (i_tl.count > 0 && i_nch > 0) return;
      i_phs++;
    }
  };
  int st_issue = 0, st_cons = 0;      // ring positions (no runtime division in the stream)
  uint32_t par_cons = 0;
  // One stage = two TMA boxes (rows 0-7 and 8-15 of the tile, 288 bytes wide) signalling the
  // stage's mbarrier; issued by lane 0.  Rows past the end of a matrix and bytes past the end
  // of a row are zero-filled by the TMA unit (and still counted in the transaction bytes).
  auto issue = [&]() {
    if (i_phs >= P.nphases) return;
    const Phase& ph = P.ph[i_phs];
    if (lane == 0) {
      const int t = i_tl.first + i_tile * i_tl.step;
      const uint32_t bar = smem_u32(&misc->full[warp][st_issue]);
      const uint32_t dst = ring + st_issue * kStageBytes;
      const int x = (i_seg_first + i_ch * kStageSegs) * (kSegBytes / 8);
      int m0 = 0, y0, m1, y1;
      if (ph.interleave) { y0 = 8 * t; m1 = 1; y1 = 8 * t; }
      else {
        y0 = kTileRows * t; m1 = 0; y1 = y0 + 8;
        // stacked matrices: row counts are multiples of 8, so a half tile never straddles two
        if (ph.nmat > 1) {
          if (y0 >= ph.rows[0]) { y0 -= ph.rows[0]; m0 = 1; if (ph.nmat > 2 && y0 >= ph.rows[1]) { y0 -= ph.rows[1]; m0 = 2; } }
          if (y1 >= ph.rows[0]) { y1 -= ph.rows[0]; m1 = 1; if (ph.nmat > 2 && y1 >= ph.rows[1]) { y1 -= ph.rows[1]; m1 = 2; } }
        }
      }
      mbar_arrive_expect_tx(bar, kStageBytes);
      tma_load_2d(dst, &Pg.tmap[i_phs][m0], x, y0, bar);
      tma_load_2d(dst + 8 * kRowStride, &Pg.tmap[i_phs][m1], x, y1, bar);
    }
    if (++st_issue == D) st_issue = 0;
    if (++i_ch >= i_nch) {
      i_ch = 0;
      if (++i_tile >= i_tl.count) { i_phs++; enter_phase(); }
    }
  };
  // The weight stream starts before anything else: weights are constants of the model, so under
  // programmatic overlap their copies may run while the previous kernel of the stream drains.
  const bool x_first = (P.flags & 1u) != 0;
  enter_phase();
  if (!x_first) for (int i = 0; i < D; i++) issue();
  // Everything below may read what earlier kernels wrote (activations, barrier words, status).
  // Without the programmatic-overlap launch attribute both instructions are no-ops.
  stamp(11);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  stamp(12);
  // tensor-parallel exchange: this launch's sequence number (stable: the previous launch is complete)
  uint32_t tp_seq = 0;
  if (P.tp_world > 1) tp_seq = *reinterpret_cast<volatile uint32_t*>(P.tp_ctl) + 1u;
  // the same for the hand-over between chained phases
  uint32_t seq = 0;
  if (P.seq_ctl) seq = *reinterpret_cast<volatile uint32_t*>(P.seq_ctl) + 1u;
  const unsigned long long wait_ns = P.wait_ns;
  // x (and gamma) of batch 0 for this warp's first segment are requested up front so that
  // their latency overlaps the set-up below
  float pre[8] = {0, 0, 0, 0, 0, 0, 0, 0}, gpre[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  bool have_pre = false;
  {
    const Phase& ph0 = P.ph[0];
    const int ks0 = (cta & (ph0.S - 1)), nseg0 = slice_segs(ph0, ks0);
    if (warp < nseg0 && tile_lane(ph0, cta, G, 0, NG).count > 0) {
      const size_t k = (size_t)(slice_seg0(ph0, ks0) + warp) * 256 + lane * 8;
      load8(reinterpret_cast<const T*>(ph0.x) + k, pre);
      if (ph0.gamma) load8(reinterpret_cast<const T*>(ph0.gamma) + k, gpre);
    }
    have_pre = true;
  }
  if (x_first) for (int i = 0; i < D; i++) issue();
  const int sh1 = c < 2 ? 12 * c : 24, sh2 = c == 3 ? 12 : 0;   // bit position of (scale, min) pair c
  // sub-block s belongs to (scale, min) pair {0,1,0,0,2,3,2,2}[s]; this thread's MMA column g stands
  // for pair g >> 1 and its B fragment covers sub-block c (first half of a block) or 4 + c (second)
  const bool keep0 = (int)((0x22320010u >> (4 * c)) & 7u) == (g >> 1);
  const bool keep1 = (int)((0x22320010u >> (4 * (c + 4))) & 7u) == (g >> 1);

  int qg = 0;  // sequence number of the tile within this group (indexes the hand-over slots)

  for (int phs = 0; phs < P.nphases; phs++) {
    const Phase& ph = P.ph[phs];
    if (phs > 0) {
      // No grid barrier: the previous phase's output arrives as tagged words that the prologue
      // below polls.  The CTA barrier only protects this CTA's own x slice in shared memory,
      // which warps still working on the previous phase are reading.
      if (warp == 0) stamp(8);
      __syncthreads();
      stamp(9);
    }
    // no tile for any group of this CTA: no work in this phase (uniform per CTA)
    if (tile_lane(ph, cta, G, 0, NG).count + tile_lane(ph, cta, G, NG - 1, NG).count == 0) continue;

    const int ks = (cta & (ph.S - 1));
    const int nseg = slice_segs(ph, ks), seg0 = slice_seg0(ph, ks);
    x_prologue<QT, T, PAIRS>(ph, plan, smem, misc, M, nseg, seg0, kAllWarps, have_pre && phs == 0, pre, gpre,
                             (P.trace && phs == 0) ? P.trace + (size_t)cta * 16 : nullptr, seq, wait_ns);

    __syncthreads();
    stamp(1 + 4 * phs);

    const TileLane tl = tile_lane(ph, cta, G, group, NG);
    {
      // this warp's K part of the slice
      const int s0w = (wg * nseg) / kGroupWarps, nsw = ((wg + 1) * nseg) / kGroupWarps - s0w;
      const int nch = (nsw + kStageSegs - 1) / kStageSegs;
      for (int it = 0; it < tl.count; it++, qg++) {
        float total[NT][2];
#pragma unroll
        for (int j = 0; j < NT; j++) total[j][0] = total[j][1] = 0.0f;
        for (int ch = 0; ch < nch; ch++) {
          const int csegs = min(kStageSegs, nsw - ch * kStageSegs);
          const uint8_t* st = ring_g + (size_t)st_cons * kStageBytes + rg * kRowStride;
          mbar_wait(smem_u32(&misc->full[warp][st_cons]), par_cons, &misc->dead, wait_ns);
          if (it == 0 && ch == 0 && warp == 0) stamp(2 + 4 * phs);
          for (int sl = 0; sl < csegs; sl++) {
            const int sg = s0w + ch * kStageSegs + sl;  // segment index within the slice
            if constexpr (PAIRS) {
              segment_mma_pairs<NT>(st + sl * kSegBytes, st + sl * kSegBytes + 8 * kRowStride,
                                    smem + plan.off_x + (size_t)(g & 1) * plan.x_stride + sg * 256 + 32 * c, 2 * plan.x_stride,
                                    reinterpret_cast<const float*>(aux) + sg * 4 + c, plan.aux_stride,
                                    delta + sg, plan.seg_stride, c, sh1, sh2, keep0, keep1, total);
            } else {
              const uint8_t* xb[NT];
              const uint32_t* auxp[NT];
              float dl[NT];
#pragma unroll
              for (int j = 0; j < NT; j++) {
                const int b = (g >> 1) + 4 * j;    // MMA column g = (batch b, part g & 1)
                xb[j] = b < M ? smem + plan.off_x + (size_t)(2 * b + (g & 1)) * plan.x_stride + sg * 256 + c * 8 : nullptr;
                auxp[j] = (b < M && !(g & 1)) ? aux + (size_t)b * plan.aux_stride + sg * AUXW : nullptr;
                dl[j] = (c + 4 * j) < M ? delta[(c + 4 * j) * plan.seg_stride + sg] : 0.0f;
              }
              segment_mma<QT, NT>(st + sl * kSegBytes, st + sl * kSegBytes + 8 * kRowStride, xb, auxp, dl, lane, total);
            }
          }
          if (++st_cons == D) { st_cons = 0; par_cons ^= 1u; }
          __syncwarp();
          issue();   // refill the stage that was just drained
        }
        if (it == 0 && warp == 0) stamp(3 + 4 * phs);
        // hand the partial sums to the epilogue warp through the tile's slot
        const int slot = qg % kSlots;
        // the slot must have been read out by the duty warp of tile qg - kSlots: a flag, not a
        // barrier, so that the eight writers do not have to meet (bounded poll)
        {
          volatile int* fr = &misc->slot_free[group][slot];
          if (!bounded_wait([&] { return *fr >= qg; }, wait_ns)) misc->dead = 1;
        }
        float* mine = slots + ((size_t)slot * kGroupWarps + wg) * kTileRows * MB;
        if constexpr (PAIRS) {
          // the four lanes of a quad hold the four pairs' parts of (row, batch): add them here so
          // that the epilogue warp has 16 x NT values per warp to read instead of 16 x 4 NT
#pragma unroll
          for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
              float v = total[j][h];
              v += __shfl_xor_sync(0xffffffffu, v, 1);
              v += __shfl_xor_sync(0xffffffffu, v, 2);
              if (c == 0) mine[(rg + 8 * h) * NT + j] = v;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < NT; j++) {
            mine[rg * MB + 4 * j + c] = total[j][0];
            mine[(rg + 8) * MB + 4 * j + c] = total[j][1];
          }
        }
        // the warp that delivers last finishes the tile: nobody waits.  Shared-memory stores of
        // a warp are ordered before its later shared-memory atomic (fence for the memory model)
        __threadfence_block();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = (atomicAdd(&misc->slot_cnt[group][slot], 1) == kGroupWarps - 1);
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          // ===== this warp finishes the tile =====
          __threadfence_block();
          const int t = tl.first + it * tl.step;
          float* tile = tiles + (size_t)slot * kTileRows * MB;
          const float* sl0 = slots + (size_t)slot * kGroupWarps * kTileRows * MB;
          if constexpr (PAIRS) {
            // slot rows are [16][NT]; the tile buffer stays [16][MB] for the common epilogue
            for (int e = lane; e < kTileRows * NT; e += 32) {
              float v = 0.0f;
#pragma unroll
              for (int w8 = 0; w8 < kGroupWarps; w8++) v += sl0[w8 * kTileRows * MB + e];
              tile[(e / NT) * MB + (e % NT)] = v;
            }
          } else {
            for (int e = lane; e < kTileRows * MB; e += 32) {
              float v = 0.0f;
#pragma unroll
              for (int w8 = 0; w8 < kGroupWarps; w8++) v += sl0[w8 * kTileRows * MB + e];
              tile[e] = v;
            }
          }
          __syncwarp();
          if (lane == 0) {   // hand the slot back
            misc->slot_cnt[group][slot] = 0;
            __threadfence_block();
            *reinterpret_cast<volatile int*>(&misc->slot_free[group][slot]) = qg + kSlots;
          }
          tile_epilogue<T, MB>(P, ph, tile, t, ks, lane, tp_seq, seq);
          __syncwarp();
        }
      }
    }
  }
  stamp(15);
  if (P.tp_world > 1) {
    // ---- reduction of the tensor-parallel block: output tile t is summed by CTA t mod G, one warp
    // per tile, once every rank's flag for the tile has arrived (bounded wait); ranks are added
    // in rank order, so all ranks store bit-identical results ----
    const Phase& ph = P.ph[P.nphases - 1];
    char* mine = P.tp_peer[P.tp_rank];
    const int parity = (int)(tp_seq & 1u);
    // Without a K split the tile -> CTA map is the same on every rank: one flag per CTA, raised
    // once after all of its tiles (a single system-scope fence, after the rings have drained),
    // and a CTA reduces exactly the tiles it produced.  Flag indices: CTA c, or tile t when split.
    const bool per_cta = ph.S == 1;
    if (per_cta) {
      __syncthreads();
      if (tid < P.tp_world) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(tp_flag(P.tp_peer[tid], P.tp_rank, cta)), "r"(tp_seq) : "memory");
      }
    }
    // tiles this CTA reduces: its own (both groups' lanes) without a K split, else t = cta, cta + G, ..
    const int n_mine = per_cta ? tile_lane(ph, cta, G, 0, NG).count + (NG > 1 ? tile_lane(ph, cta, G, NG - 1, NG).count : 0)
                               : (ph.ntiles > cta ? (ph.ntiles - cta + G - 1) / G : 0);
    for (int k = 0; k < n_mine; k++) {
      int t;
      if (per_cta) {
        const int c0 = tile_lane(ph, cta, G, 0, NG).count;
        const TileLane tl = tile_lane(ph, cta, G, k < c0 ? 0 : NG - 1, NG);
        t = tl.first + (k < c0 ? k : k - c0) * tl.step;
      } else {
        t = cta + k * G;
      }
      if (k % kAllWarps != warp) continue;
      bool ok = true;
      if (lane < P.tp_world) {
        const uint32_t* f = tp_flag(mine, lane, per_cta ? cta : t);
        ok = bounded_wait([&] {
          uint32_t v;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
          return (int32_t)(v - tp_seq) >= 0;
        }, wait_ns);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { misc->dead = 1; continue; }
      T* yf = reinterpret_cast<T*>(P.tp_y);
      for (int e = lane; e < kTileRows * M; e += 32) {
        const int r = e % kTileRows, m = e / kTileRows;
        const int R = kTileRows * t + r;
        if (R >= ph.n_total) continue;
        const size_t off = (size_t)m * ph.n_total + R;
        float acc = 0.0f;
        for (int src = 0; src < P.tp_world; src++) acc += __ldcg(tp_slot(mine, parity, src) + off);
        yf[off] = Act<T>::from_f(acc);
      }
    }
  }
  __syncthreads();
  if (tid == 0 && misc->dead) atomicExch(P.status, MLXR_ERR_TIMEOUT);
  if (P.seq_ctl && tid == 0) {
    // the last CTA to finish publishes this launch's sequence number for the next launch to read
    __threadfence();
    if (atomicAdd(P.seq_ctl + 1, 1u) == (uint32_t)G - 1u) {
      P.seq_ctl[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(P.seq_ctl) = seq;
    }
  }
  if (P.tp_world > 1 && tid == 0) {
    // the last CTA to finish advances the sequence number for the next launch
    __threadfence();
    if (atomicAdd(P.tp_ctl + 1, 1u) == (uint32_t)G - 1u) {
      P.tp_ctl[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(P.tp_ctl) = tp_seq;
    }
  }
}

}  // namespace decode
}  // namespace mlxr
