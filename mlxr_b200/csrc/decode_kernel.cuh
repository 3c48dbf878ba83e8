// Persistent decode kernel for quantized linears at small batch (M <= 16).
//
// Roofline: HBM.  One CTA per SM streams packed weight rows through a ring of shared-
// memory stages filled by bulk async copies (cp.async.bulk, one per row segment, completion
// on an mbarrier); eight consumer warps dequantize nibbles in registers with the
// (x & mask) | magic half-precision trick and feed warp-level tensor-core MMAs
// (m16n8k16, fp16 x fp16 -> fp32) in which the 16 MMA rows are 16 weight rows and the 8 MMA
// columns are the batch.  Sub-block scales are applied to the fp32 accumulators, the
// Q4_K min term goes through one extra k8 MMA per super-block.  Fused around it:
//   prologue   RMSNorm of x (optional), rounding to the activation dtype, power-of-two
//              normalisation into fp16, k-permutation into shared memory
//   epilogue   plain (+bias) | SiLU(gate)*up on interleaved gate/up rows | RoPE on q/k rows
//   split-K    partial sums of K-slices meet in a global scratch; the CTA that arrives last
//              for a tile reduces them in slice order (deterministic) and runs the epilogue
//   two phases gate/up -> grid barrier -> down in ONE launch: the producer warp keeps
//              streaming the next phase's weights while consumers wait at the barrier
// Every wait (mbarrier, grid barrier) is bounded; on expiry a status word is set and the
// kernel carries on without blocking.
#pragma once
#include "common.cuh"

namespace mlxr {
namespace decode {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;   // + 1 producer warp
constexpr int kTileRows = 16;
constexpr int kMaxChunkSegs = 8;                      // segments (256 k) per stage and row
constexpr int kSegBytes = 144;                        // Q4_K super-block = 8 Q4_0 blocks
constexpr int kRowStride = kMaxChunkSegs * kSegBytes + 16;  // 1168 B: 292 words = 4 mod 32
constexpr int kStageBytes = kTileRows * kRowStride;   // 18688
constexpr uint32_t kSpinLimit = 1u << 20;

enum Epilogue { kEpiPlain = 0, kEpiSwiglu = 1, kEpiRope = 2 };

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
  int S;                 // K-slices
  int segs_base, segs_extra;  // slice s has segs_base + (s < segs_extra) segments
  int max_slice_segs;
  // activations
  const void* x;         // [M, K] activation dtype
  const void* gamma;     // RMSNorm weight [K] or null
  float eps;
  // outputs
  void* y[3];            // per matrix [M, rows[i]]; swiglu: y[0] = h [M, n_total]
  const void* bias[3];
  int epi[3];
  // rope
  const __half* cos_t;
  const __half* sin_t;
  const int32_t* positions;
  int head_dim, max_seq, pos_offset;
  // split-K scratch
  float* partials;       // [S][M_pad][n_pad]
  uint32_t* counters;    // [ntiles], zero between launches
};

struct Params {
  Phase ph[2];
  int nphases;
  int M;
  uint32_t* gridbar;     // monotonically increasing arrival counter
  uint32_t bar_base;     // value of *gridbar before this launch
  int* status;
};

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait: false (and *dead set) when the limit is reached.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* dead) {
  if (*dead) return false;
  for (uint32_t i = 0; i < kSpinLimit; i++)
    if (mbar_try_wait(bar, parity)) return true;
  *dead = 1;
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & b) | c
  return r;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// 8 nibbles of one 32-bit word -> four half2 registers holding (q - 8) exactly:
// out[0] = (n0, n4), out[1] = (n1, n5), out[2] = (n2, n6), out[3] = (n3, n7).
__device__ __forceinline__ void nibbles_to_half2(uint32_t w, uint32_t (&out)[4]) {
  const uint32_t ws = w >> 8;
  out[0] = hsub2_u32(lop3_and_or(w, 0x000f000fu, 0x64006400u), 0x64086408u);   // 1024 + q - 1032
  out[1] = hsub2_u32(lop3_and_or(w, 0x00f000f0u, 0x54005400u), 0x54805480u);   // 64 + q - 72
  out[2] = hsub2_u32(lop3_and_or(ws, 0x000f000fu, 0x64006400u), 0x64086408u);
  out[3] = hsub2_u32(lop3_and_or(ws, 0x00f000f0u, 0x54005400u), 0x54805480u);
}

// position of element e (0..7) of an 8-group in the permuted x layout (0,4,1,5,2,6,3,7)
__host__ __device__ inline int perm8(int e) { return ((e & 3) << 1) | (e >> 2); }

// Shared-memory plan (bytes), identical on host and device.
struct SmemPlan {
  int stages;
  int x_stride;      // bytes per batch column of the fp16 x slice
  int sxp_stride;    // words per batch column of the pair-sum table
  int off_ring, off_x, off_sxp, off_red, off_tile, off_misc, total;
};
__host__ __device__ inline SmemPlan make_plan(int stages, int max_slice_k, int max_slice_segs, int mcols, int xcols) {
  SmemPlan p;
  p.stages = stages;
  p.x_stride = max_slice_k * 2 + 64;
  int w = max_slice_segs * 4;
  p.sxp_stride = w + ((4 - (w & 31)) & 31);          // = 4 (mod 32)
  p.off_ring = 0;
  p.off_x = p.off_ring + stages * kStageBytes;
  p.off_sxp = p.off_x + xcols * p.x_stride;
  p.off_red = p.off_sxp + xcols * p.sxp_stride * 4;
  p.off_tile = p.off_red + kConsumerWarps * kTileRows * mcols * 4;
  p.off_misc = p.off_tile + kTileRows * mcols * 4;
  p.total = p.off_misc + 1024;
  return p;
}

struct Misc {
  unsigned long long full[16];
  unsigned long long empty[16];
  float colscale[16];    // 2^e per batch column (x16 = x * 2^-e)
  float colrinv[16];
  float redbuf[kConsumerWarps * 16];
  int dead;
  int last_flag;
};
static_assert(sizeof(Misc) <= 1024, "Misc must fit its smem slot");

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

template <int QT, typename T, int NT>
__global__ void __launch_bounds__(kThreads, 1) decode_kernel(const __grid_constant__ Params P, const __grid_constant__ SmemPlan plan) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int MC = 8 * NT;  // batch columns held
  Misc* misc = reinterpret_cast<Misc*>(smem + plan.off_misc);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int M = P.M;
  volatile int* dead = &misc->dead;

  if (tid == 0) {
    misc->dead = 0;
    for (int s = 0; s < plan.stages; s++) {
      mbar_init(smem_u32(&misc->full[s]), 1);
      mbar_init(smem_u32(&misc->empty[s]), kConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  const uint32_t ring = smem_u32(smem + plan.off_ring);

  if (warp == kConsumerWarps) {
    // ================= producer warp =================
    uint32_t n = 0;  // chunks issued so far
    for (int phs = 0; phs < P.nphases; phs++) {
      const Phase& ph = P.ph[phs];
      const int nitems = ph.ntiles * ph.S;
      for (int item = cta; item < nitems; item += G) {
        const int t = item / ph.S, ks = item - t * ph.S;
        const int nseg = slice_segs(ph, ks), seg0 = slice_seg0(ph, ks);
        const int nchunks = (nseg + kMaxChunkSegs - 1) / kMaxChunkSegs;
        const int cb = nseg / nchunks, ce = nseg - cb * nchunks;   // balanced chunk sizes
        const uint8_t* src = lane < kTileRows ? tile_row(ph, t, lane) + (size_t)seg0 * kSegBytes : nullptr;
        int done = 0;
        for (int ch = 0; ch < nchunks; ch++) {
          const int csegs = cb + (ch < ce ? 1 : 0);
          const int stage = n % plan.stages;
          const uint32_t par = ((n / plan.stages) & 1) ^ 1;
          const uint32_t fullb = smem_u32(&misc->full[stage]);
          bool ok = true;
          if (lane == 0) ok = mbar_wait(smem_u32(&misc->empty[stage]), par, dead);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (ok) {
            const uint32_t bytes = (uint32_t)csegs * kSegBytes;
            if (lane == 0) mbar_arrive_expect_tx(fullb, bytes * kTileRows);
            __syncwarp();
            if (lane < kTileRows)
              bulk_g2s(ring + stage * kStageBytes + lane * kRowStride, src + (size_t)done * kSegBytes, bytes, fullb);
          }
          done += csegs;
          n++;
        }
      }
    }
    // If a wait gave up, copies may still be in flight: give them a bounded time to land
    // before the CTA's shared memory is released.
    if (*dead && lane == 0) {
      for (int s = 0; s < plan.stages; s++)
        for (uint32_t i = 0; i < (1u << 16); i++)
          if (mbar_try_wait(smem_u32(&misc->full[s]), 0) || mbar_try_wait(smem_u32(&misc->full[s]), 1)) break;
    }
    return;
  }

  // ================= consumer warps =================
  const int g = lane >> 2, c = lane & 3;
  uint8_t* xs = smem + plan.off_x;
  uint32_t* sxp = reinterpret_cast<uint32_t*>(smem + plan.off_sxp);
  float* red = reinterpret_cast<float*>(smem + plan.off_red);
  float* tilebuf = reinterpret_cast<float*>(smem + plan.off_tile);
  const int ctid = tid;  // 0..255
  uint32_t n = 0;

  for (int phs = 0; phs < P.nphases; phs++) {
    const Phase& ph = P.ph[phs];
    const int nitems = ph.ntiles * ph.S;

    if (phs > 0) {
      // ---- grid barrier: every CTA has finished (and made visible) the previous phase ----
      __threadfence();
      consumer_sync();
      if (ctid == 0) {
        const uint32_t target = P.bar_base + (uint32_t)phs * (uint32_t)G;
        atomicAdd(P.gridbar, 1u);
        bool ok = false;
        for (uint32_t i = 0; i < (kSpinLimit << 2) && !*dead; i++) {
          const uint32_t v = *reinterpret_cast<volatile uint32_t*>(P.gridbar);
          if ((int32_t)(v - target) >= 0) { ok = true; break; }
          __nanosleep(32);
        }
        if (!ok) { *dead = 1; }
        __threadfence();
      }
      consumer_sync();
    }
    if (cta >= nitems) continue;  // nothing to do in this phase (uniform per CTA)

    // ---- x prologue: this CTA's K-slice of x -> fp16, normalised, permuted ----------------
    const int ks_mine = cta % ph.S;   // G % S == 0, so every item of this CTA has this slice
    const int nseg = slice_segs(ph, ks_mine), seg0 = slice_seg0(ph, ks_mine);
    const int k0 = seg0 * 256, kn = nseg * 256;
    const T* xg = reinterpret_cast<const T*>(ph.x);
    const T* gam = reinterpret_cast<const T*>(ph.gamma);
    if (ctid < MC) misc->colscale[ctid] = 1.0f;
    consumer_sync();
    for (int m = 0; m < M; m++) {
      float rinv = 1.0f;
      if (gam) {
        float ss = 0.0f;
        for (int k = ctid; k < ph.K; k += kConsumerWarps * 32) {
          const float v = Act<T>::to_f(__ldcg(&xg[(size_t)m * ph.K + k]));
          ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) misc->redbuf[warp] = ss;
        consumer_sync();
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < kConsumerWarps; i++) tot += misc->redbuf[i];
        rinv = 1.0f / sqrtf(tot / (float)ph.K + ph.eps);
        consumer_sync();
      }
      // pass 1: values of the slice (rounded to the activation dtype) and their max
      float amax = 0.0f;
      for (int k = ctid; k < kn; k += kConsumerWarps * 32) {
        float v = Act<T>::to_f(__ldcg(&xg[(size_t)m * ph.K + k0 + k]));
        if (gam) v = Act<T>::to_f(Act<T>::from_f(__fmul_rn(__fmul_rn(v, rinv), Act<T>::to_f(gam[k0 + k]))));
        amax = fmaxf(amax, fabsf(v));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (lane == 0) misc->redbuf[warp] = amax;
      consumer_sync();
      amax = 0.0f;
#pragma unroll
      for (int i = 0; i < kConsumerWarps; i++) amax = fmaxf(amax, misc->redbuf[i]);
      // power of two that brings amax into [16, 32): sums of 96 values stay below 65504
      int e = 0;
      if (amax > 0.0f && amax < 3.0e38f) { (void)frexpf(amax, &e); e -= 5; }
      const float down = ldexpf(1.0f, -e);
      if (ctid == 0) misc->colscale[m] = ldexpf(1.0f, e);
      // pass 2: store fp16(v * 2^-e) at the permuted position
      __half* xcol = reinterpret_cast<__half*>(xs + (size_t)m * plan.x_stride);
      for (int k = ctid; k < kn; k += kConsumerWarps * 32) {
        float v = Act<T>::to_f(__ldcg(&xg[(size_t)m * ph.K + k0 + k]));
        if (gam) v = Act<T>::to_f(Act<T>::from_f(__fmul_rn(__fmul_rn(v, rinv), Act<T>::to_f(gam[k0 + k]))));
        xcol[(k & ~7) | perm8(k & 7)] = __float2half_rn(v * down);
      }
      consumer_sync();
      // pair sums for the Q4_K min term: sub-blocks {0,2,3}, {1}, {4,6,7}, {5} of every segment
      if constexpr (QT == MLXR_Q4_K) {
        for (int task = ctid; task < nseg * 4; task += kConsumerWarps * 32) {
          const int sg = task >> 2, p = task & 3;
          const int subs[4][3] = {{0, 2, 3}, {1, -1, -1}, {4, 6, 7}, {5, -1, -1}};
          float s = 0.0f;
          for (int j = 0; j < 3; j++) {
            const int sb = subs[p][j];
            if (sb < 0) continue;
            const __half* q = xcol + sg * 256 + sb * 32;
            for (int i = 0; i < 32; i++) s += __half2float(q[i]);
          }
          const __half hi = __float2half_rn(s);
          const __half lo = __float2half_rn(s - __half2float(hi));
          sxp[(size_t)m * plan.sxp_stride + sg * 4 + p] = (uint32_t)__half_as_ushort(hi) | ((uint32_t)__half_as_ushort(lo) << 16);
        }
      }
    }
    consumer_sync();

    // ---- items -------------------------------------------------------------------------
    for (int item = cta; item < nitems; item += G) {
      const int t = item / ph.S, ks = item - t * ph.S;
      const int nchunks = (nseg + kMaxChunkSegs - 1) / kMaxChunkSegs;
      const int cb = nseg / nchunks, ce = nseg - cb * nchunks;
      float total[NT][4];
#pragma unroll
      for (int j = 0; j < NT; j++) total[j][0] = total[j][1] = total[j][2] = total[j][3] = 0.0f;
      int segdone = 0;
      for (int ch = 0; ch < nchunks; ch++) {
        const int csegs = cb + (ch < ce ? 1 : 0);
        const int stage = n % plan.stages;
        const uint32_t par = (n / plan.stages) & 1;
        const bool ok = mbar_wait(smem_u32(&misc->full[stage]), par, dead);
        if (ok && warp < csegs) {
          const int sg = segdone + warp;  // segment index within the slice
          const uint32_t r_lo = ring + stage * kStageBytes + g * kRowStride + warp * kSegBytes;
          const uint32_t r_hi = r_lo + 8 * kRowStride;
          const uint32_t xaddr = smem_u32(xs) + sg * 512 + c * 16;

          if constexpr (QT == MLXR_Q4_K) {
            const uint4 hl = lds128(r_lo), hh = lds128(r_hi);
            // 6-bit fields (q_gemm_dequant.metal:222-242) straight from the packed words
            float ssl[4], ssh[4];
            uint32_t amin_lo, amin_hi;
            {
              const __half2 dl = *reinterpret_cast<const __half2*>(&hl.x), dh = *reinterpret_cast<const __half2*>(&hh.x);
              const uint32_t w2 = hl.y, w3 = hl.z, v2 = hh.y, v3 = hh.z;
              const int scl[4] = {(int)(w2 & 63u), (int)((w2 >> 12) & 63u), (int)((w2 >> 24) & 63u), (int)((w3 >> 4) & 63u)};
              const int sch[4] = {(int)(v2 & 63u), (int)((v2 >> 12) & 63u), (int)((v2 >> 24) & 63u), (int)((v3 >> 4) & 63u)};
#pragma unroll
              for (int p = 0; p < 4; p++) {
                ssl[p] = __half2float(__hmul(__int2half_rn(scl[p]), __low2half(dl)));
                ssh[p] = __half2float(__hmul(__int2half_rn(sch[p]), __low2half(dh)));
              }
              // this thread supplies the min of pair c (k-slots 2c, 2c+1 of the k8 MMA)
              const uint32_t mnl = c == 0 ? (w2 >> 6) : c == 1 ? (w2 >> 18) : c == 2 ? ((w2 >> 30) | ((w3 & 15u) << 2)) : (w3 >> 10);
              const uint32_t mnh = c == 0 ? (v2 >> 6) : c == 1 ? (v2 >> 18) : c == 2 ? ((v2 >> 30) | ((v3 & 15u) << 2)) : (v3 >> 10);
              const __half sml = __hmul(__int2half_rn((int)(mnl & 63u)), __high2half(dl));
              const __half smh = __hmul(__int2half_rn((int)(mnh & 63u)), __high2half(dh));
              amin_lo = (uint32_t)__half_as_ushort(sml) * 0x00010001u;
              amin_hi = (uint32_t)__half_as_ushort(smh) * 0x00010001u;
            }
            constexpr int order[8] = {0, 2, 3, 1, 4, 6, 7, 5};
            constexpr int pair_of[8] = {0, 0, 0, 1, 2, 2, 2, 3};
            constexpr bool last_of_pair[8] = {false, false, true, true, false, false, true, true};
            float acc[NT][4];
#pragma unroll
            for (int j = 0; j < NT; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const int s = order[i];
              uint32_t al[4], ah[4];
              nibbles_to_half2(lds32(r_lo + 16 + 16 * s + 4 * c), al);
              nibbles_to_half2(lds32(r_hi + 16 + 16 * s + 4 * c), ah);
#pragma unroll
              for (int j = 0; j < NT; j++) {
                uint4 b = make_uint4(0u, 0u, 0u, 0u);
                if (g + 8 * j < M) b = lds128(xaddr + (uint32_t)(g + 8 * j) * plan.x_stride + 64 * s);
                mma16816(acc[j], al[0], ah[0], al[1], ah[1], b.x, b.y);
                mma16816(acc[j], al[2], ah[2], al[3], ah[3], b.z, b.w);
              }
              if (last_of_pair[i]) {
                const int p = pair_of[i];
#pragma unroll
                for (int j = 0; j < NT; j++) {
                  total[j][0] = fmaf(ssl[p], acc[j][0], total[j][0]);
                  total[j][1] = fmaf(ssl[p], acc[j][1], total[j][1]);
                  total[j][2] = fmaf(ssh[p], acc[j][2], total[j][2]);
                  total[j][3] = fmaf(ssh[p], acc[j][3], total[j][3]);
                  acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
                }
              }
            }
            // min term: sum_p sm_p * Sx_p, Sx_p as hi + lo halves
#pragma unroll
            for (int j = 0; j < NT; j++) {
              uint32_t b = 0u;
              if (g + 8 * j < M) b = sxp[(size_t)(g + 8 * j) * plan.sxp_stride + sg * 4 + c];
              mma1688(total[j], amin_lo, amin_hi, b);
            }
          } else {  // Q4_0: 8 blocks of 18 B; scale at +18s, nibbles at +18s+2
#pragma unroll
            for (int s = 0; s < 8; s++) {
              uint32_t wl, wh;
              if (s & 1) {  // 18s+2 is 4-byte aligned
                wl = lds32(r_lo + 18 * s + 2 + 4 * c);
                wh = lds32(r_hi + 18 * s + 2 + 4 * c);
              } else {      // straddles two words
                wl = __funnelshift_r(lds32(r_lo + 18 * s + 4 * c), lds32(r_lo + 18 * s + 4 * c + 4), 16);
                wh = __funnelshift_r(lds32(r_hi + 18 * s + 4 * c), lds32(r_hi + 18 * s + 4 * c + 4), 16);
              }
              uint32_t sl, sh;
              asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sl) : "r"(r_lo + 18 * s));
              asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sh) : "r"(r_hi + 18 * s));
              const float fl = __half2float(__ushort_as_half((unsigned short)sl));
              const float fh = __half2float(__ushort_as_half((unsigned short)sh));
              uint32_t al[4], ah[4];
              nibbles_to_half2(wl, al);
              nibbles_to_half2(wh, ah);
#pragma unroll
              for (int j = 0; j < NT; j++) {
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                uint4 b = make_uint4(0u, 0u, 0u, 0u);
                if (g + 8 * j < M) b = lds128(xaddr + (uint32_t)(g + 8 * j) * plan.x_stride + 64 * s);
                mma16816(acc, al[0], ah[0], al[1], ah[1], b.x, b.y);
                mma16816(acc, al[2], ah[2], al[3], ah[3], b.z, b.w);
                total[j][0] = fmaf(fl, acc[0], total[j][0]);
                total[j][1] = fmaf(fl, acc[1], total[j][1]);
                total[j][2] = fmaf(fh, acc[2], total[j][2]);
                total[j][3] = fmaf(fh, acc[3], total[j][3]);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&misc->empty[stage]));
        segdone += csegs;
        n++;
      }

      // ---- reduce the eight warps' partial sums: tilebuf[row][col] in true units ---------
#pragma unroll
      for (int j = 0; j < NT; j++) {
        float* rw = red + (size_t)warp * kTileRows * MC;
        *reinterpret_cast<float2*>(&rw[g * MC + 8 * j + 2 * c]) = make_float2(total[j][0], total[j][1]);
        *reinterpret_cast<float2*>(&rw[(g + 8) * MC + 8 * j + 2 * c]) = make_float2(total[j][2], total[j][3]);
      }
      consumer_sync();
      for (int e = ctid; e < kTileRows * MC; e += kConsumerWarps * 32) {
        float v = 0.0f;
#pragma unroll
        for (int w8 = 0; w8 < kConsumerWarps; w8++) v += red[(size_t)w8 * kTileRows * MC + e];
        tilebuf[e] = v * misc->colscale[e % MC];
      }
      consumer_sync();

      // ---- split-K: park the partial, the last slice to arrive reduces all of them -------
      bool do_epilogue = true;
      if (ph.S > 1) {
        const size_t slab = (size_t)ph.ntiles * kTileRows * MC;
        float* mine = ph.partials + (size_t)ks * slab + (size_t)t * kTileRows * MC;
        for (int e = ctid; e < kTileRows * MC; e += kConsumerWarps * 32) __stcg(&mine[e], tilebuf[e]);
        __threadfence();
        consumer_sync();
        if (ctid == 0) {
          const uint32_t prev = atomicAdd(&ph.counters[t], 1u);
          misc->last_flag = (prev == (uint32_t)ph.S - 1u);
          if (misc->last_flag) ph.counters[t] = 0u;   // self-cleaning for the next launch
          __threadfence();
        }
        consumer_sync();
        do_epilogue = misc->last_flag != 0;
        if (do_epilogue) {
          for (int e = ctid; e < kTileRows * MC; e += kConsumerWarps * 32) {
            float v = 0.0f;
            for (int s2 = 0; s2 < ph.S; s2++) v += __ldcg(&ph.partials[(size_t)s2 * slab + (size_t)t * kTileRows * MC + e]);
            tilebuf[e] = v;
          }
          consumer_sync();
        }
      }

      // ---- epilogue ----------------------------------------------------------------------
      if (do_epilogue) {
        if (ph.interleave) {
          // rows 0..7 gate, 8..15 up of the same 8 intermediate indices: h = SiLU(g) * u
          for (int e = ctid; e < 8 * MC; e += kConsumerWarps * 32) {
            const int r = e / MC, m = e % MC;
            const int col = 8 * t + r;
            if (m < M && col < ph.n_total) {
              const float gv = Act<T>::to_f(Act<T>::from_f(tilebuf[r * MC + m]));
              const float uv = Act<T>::to_f(Act<T>::from_f(tilebuf[(r + 8) * MC + m]));
              reinterpret_cast<T*>(ph.y[0])[(size_t)m * ph.n_total + col] = Act<T>::from_f(swish_f(gv) * uv);
            }
          }
        } else {
          // pairs of adjacent rows (2j, 2j+1): plain store or RoPE rotation
          for (int e = ctid; e < 8 * MC; e += kConsumerWarps * 32) {
            const int j = e / MC, m = e % MC;
            int R = kTileRows * t + 2 * j;
            if (m >= M || R >= ph.n_total) continue;
            int mat = 0;
            if (ph.nmat > 1 && R >= ph.rows[0]) { R -= ph.rows[0]; mat = 1; if (ph.nmat > 2 && R >= ph.rows[1]) { R -= ph.rows[1]; mat = 2; } }
            const bool has_odd = R + 1 < ph.rows[mat];
            float ve = tilebuf[(2 * j) * MC + m], vo = tilebuf[(2 * j + 1) * MC + m];
            const T* bias = reinterpret_cast<const T*>(ph.bias[mat]);
            if (bias) { ve += Act<T>::to_f(bias[R]); if (has_odd) vo += Act<T>::to_f(bias[R + 1]); }
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
        }
      }
      consumer_sync();  // tilebuf / red are reused by the next item
    }
  }
  if (ctid == 0 && *dead) atomicExch(P.status, MLXR_ERR_TIMEOUT);
}

}  // namespace decode
}  // namespace mlxr
