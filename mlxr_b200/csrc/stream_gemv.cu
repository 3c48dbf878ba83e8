// Streaming decode linear for Q4_K at batch 1 and 2: many small CTAs, weights straight from
// global memory into tensor-core fragments, L2 as the prefetch buffer.
//
// Roofline: HBM.  The persistent decode kernel (decode_kernel.cuh) keeps 16 warps per SM busy with
// long dependent instruction chains and has shared memory (~150 KB per SM) as its only prefetch
// buffer, so every wait - for the previous kernel, for the activations - stops the stream after
// that much data.  This kernel turns both around:
//   * 24 warps per SM (three CTAs of eight warps): latency is hidden by thread-level parallelism;
//     a warp loads its 16 weight rows x 256-element segment straight into the registers that are
//     the A fragments of mma.sync.m16n8k32 (u8 x s8), two segments in flight;
//   * the next tiles' rows are requested with bulk L2 prefetches (cp.async.bulk.prefetch.L2, one
//     instruction per row, fire and forget): the 126 MB L2 is the prefetch buffer, so the copies of
//     a launch run while the previous kernel of the stream drains (programmatic stream
//     serialization: weights are constants, only the activations wait for griddepcontrol.wait)
//     and whole-row requests reach DRAM as long contiguous bursts;
//   * gate/up with the SiLU(gate)*up epilogue and the down projection are two launches chained by
//     programmatic serialization: the kernel boundary is the hand-over of h, no grid barrier.
// Arithmetic is that of the persistent kernel (see decode_kernel.cuh): activations as 16-bit fixed
// point per 256-element block, split in a high and a low signed byte; raw nibbles multiplied as
// unsigned bytes; (scale, min) pairs of the Q4_K super-block in the MMA columns, so one
// accumulation runs over a whole block; results are deterministic (fixed reduction order).
#include <atomic>
#include <mutex>

#include "decode_kernel.cuh"
#include "kernels.h"

namespace mlxr {
namespace sgemv {

using decode::imma16832;
using decode::load8;
using decode::kSegBytes;
using decode::kTileRows;

constexpr int kWarps = 8;            // per CTA: the K range of a 16-row tile is split over them
constexpr int kThreads = kWarps * 32;
#ifndef MLXR_SGEMV_CTAS
#define MLXR_SGEMV_CTAS 2
#endif
constexpr int kCtasPerSm = MLXR_SGEMV_CTAS;

struct Params {
  const uint8_t* w[3];   // up to three packed matrices stacked along N, or gate/up interleaved
  int rows[3];
  int nmat;
  int interleave;        // tile t = rows [8t, 8t+8) of w[0] (gate) and of w[1] (up); y[0] = h [M, rows[0]]
  int n_total;
  int K, row_bytes, nseg, ntiles;
  int M;
  const void* x;         // [M, K]
  const void* gamma;     // RMSNorm weight or null
  float eps;
  void* y[3];
  const void* bias[3];
  int epi[3];            // decode::Epilogue
  const __half* cos_t;
  const __half* sin_t;
  const int32_t* positions;
  int head_dim, max_seq, pos_offset;
  int* status;
  // shared-memory layout
  unsigned long long* trace;   // optional: 16 globaltimer stamps per CTA (tuning builds)
  const uint8_t* next_w;       // packed weights of the launch that follows this one (prefetch hint) or null
  size_t next_bytes;
  int x_stride;          // bytes per int8 row of x (hi row, lo row per batch row)
  int off_aux, off_delta, off_slots, off_red;
};

// Pointer to packed row r (0..15) of tile t; rows past the end are clamped (their sums are dropped).
__device__ __forceinline__ const uint8_t* tile_row(const Params& P, int t, int r) {
  if (P.interleave) {
    int row = 8 * t + (r & 7);
    if (row >= P.n_total) row = P.n_total - 1;
    return P.w[r >> 3] + (size_t)row * P.row_bytes;
  }
  int R = kTileRows * t + r;
  if (R >= P.n_total) R = P.n_total - 1;
  int m = 0;
  if (P.nmat > 1 && R >= P.rows[0]) { R -= P.rows[0]; m = 1; if (P.nmat > 2 && R >= P.rows[1]) { R -= P.rows[1]; m = 2; } }
  return P.w[m] + (size_t)R * P.row_bytes;
}

__device__ __forceinline__ uint4 ldg16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// Fixed-point conversion of one (batch row, segment): v holds this lane's eight activations.
// x ~ delta * xi with |xi| <= 32000, xi = 256 hi + lo stored as two signed-byte rows in MMA k
// order; per (scale, min) pair of the block the exact integer sum of xi (the offset / min term is
// linear in it).  Warp-wide maxima and sums use the redux instructions (one instruction each).
__device__ __forceinline__ void emit_segment(uint8_t* smem, const Params& P, int m, int sg, int lane, float (&v)[8]) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
  // non-negative floats order like their bit patterns (NaN and Inf sort above every finite value)
  amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));
  float dl = 1.0f, inv = 0.0f;
  if (!(amax <= 3.0e38f)) { dl = __int_as_float(0x7fc00000); }   // a non-finite block poisons its outputs
  else if (amax > 0.0f) { dl = amax * (1.0f / 32000.0f); inv = __fdividef(32000.0f, amax); }
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
  uint8_t* xrow = smem + (size_t)(2 * m) * P.x_stride + sg * 256 + lane * 8;
  *reinterpret_cast<uint2*>(xrow) = make_uint2(hi_e, hi_o);
  *reinterpret_cast<uint2*>(xrow + P.x_stride) = make_uint2(lo_e, lo_o);
  // sums of xi per (scale, min) pair: sub-blocks {0,2,3}, {1}, {4,6,7}, {5} share a pair
  // (q_gemm_dequant.metal:222-242); this lane's eight elements lie in sub-block lane / 4
  const int myp = (int)((0x22320010u >> (4 * (lane >> 2))) & 7u);
  const int p0 = __reduce_add_sync(0xffffffffu, myp == 0 ? ssum : 0), p1 = __reduce_add_sync(0xffffffffu, myp == 1 ? ssum : 0);
  const int p2 = __reduce_add_sync(0xffffffffu, myp == 2 ? ssum : 0), p3 = __reduce_add_sync(0xffffffffu, myp == 3 ? ssum : 0);
  float* aux = reinterpret_cast<float*>(smem + P.off_aux) + ((size_t)m * P.nseg + sg) * 4;
  if (lane == 0) {
    reinterpret_cast<float*>(smem + P.off_delta)[m * P.nseg + sg] = dl;
    *reinterpret_cast<float4*>(aux) = make_float4((float)p0, (float)p1, (float)p2, (float)p3);
  }
}

// One 256-element segment of 16 rows: rl / rh = this thread's two rows (g and g+8) at the
// segment's first byte in global memory.  MMA column 2p + part of n-tile j stands for batch j's x
// restricted to the sub-blocks of (scale, min) pair p; thread (g, c) feeds the words of sub-block
// c (then 4 + c), so its B fragment is either that sub-block's x bytes or zero (keep0 / keep1) and
// it ends up with the sums of pair c, which it scales with the pair it decodes itself.  Low
// nibbles go to the tensor cores as they are (w & 0x0f0f0f0f); high nibbles stay in place
// (w & 0xf0f0f0f0 = 16 x nibble) and accumulate separately (two logic operations per word, two
// independent MMA chains).
struct SegRegs { uint4 hl, hh, wl0, wl1, wh0, wh1; };
__device__ __forceinline__ void seg_load(SegRegs& r, const uint8_t* rl, const uint8_t* rh, int c) {
  r.hl = ldg16(rl);
  r.hh = ldg16(rh);
  r.wl0 = ldg16(rl + 16 + 16 * c);
  r.wl1 = ldg16(rl + 80 + 16 * c);
  r.wh0 = ldg16(rh + 16 + 16 * c);
  r.wh1 = ldg16(rh + 80 + 16 * c);
}
template <int NT>
__device__ __forceinline__ void seg_math(const SegRegs& r, const uint8_t* x0, int x_batch_stride, const float* sx0,
                                         int aux_batch_stride, const float* dl0, int dl_batch_stride, int sh1, int sh2,
                                         bool keep0, bool keep1, float (&total)[NT][2]) {
  int acc_lo[NT][4], acc_hi[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++) {
    acc_lo[j][0] = acc_lo[j][1] = acc_lo[j][2] = acc_lo[j][3] = 0;
    acc_hi[j][0] = acc_hi[j][1] = acc_hi[j][2] = acc_hi[j][3] = 0;
  }
#pragma unroll
  for (int h = 0; h < 2; h++) {
    const bool keep = h ? keep1 : keep0;
    const uint4 wl = h ? r.wl1 : r.wl0, wh = h ? r.wh1 : r.wh0;
    uint4 xa[NT], xb[NT];   // (even, odd) x bytes of 8-element groups 0, 1 and of groups 2, 3
#pragma unroll
    for (int j = 0; j < NT; j++) {
      xa[j] = make_uint4(0u, 0u, 0u, 0u);
      xb[j] = make_uint4(0u, 0u, 0u, 0u);
      if (keep) {
        xa[j] = *reinterpret_cast<const uint4*>(x0 + (size_t)j * x_batch_stride + 128 * h);
        xb[j] = *reinterpret_cast<const uint4*>(x0 + (size_t)j * x_batch_stride + 128 * h + 16);
      }
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const uint32_t wa = i == 0 ? wl.x : wl.z, wb = i == 0 ? wl.y : wl.w;   // words 2i, 2i+1 of row g
      const uint32_t va = i == 0 ? wh.x : wh.z, vb = i == 0 ? wh.y : wh.w;   // ... of row g+8
      const uint32_t l0 = wa & 0x0f0f0f0fu, l1 = va & 0x0f0f0f0fu, l2 = wb & 0x0f0f0f0fu, l3 = vb & 0x0f0f0f0fu;
      const uint32_t h0 = wa & 0xf0f0f0f0u, h1 = va & 0xf0f0f0f0u, h2 = wb & 0xf0f0f0f0u, h3 = vb & 0xf0f0f0f0u;
#pragma unroll
      for (int j = 0; j < NT; j++) {
        const uint4 xv = i == 0 ? xa[j] : xb[j];
        imma16832(acc_lo[j], l0, l1, l2, l3, xv.x, xv.z);
        imma16832(acc_hi[j], h0, h1, h2, h3, xv.y, xv.w);
      }
    }
  }
  // (scale, min) pair c of both rows: 6-bit fields at bit 12c (scale) and 12c + 6 (min) of the 48
  // packed bits scales[0..5] (q_gemm_dequant.metal:222-242); sub-block scale = rn16(sc * d),
  // sub-block min = rn16(m * dmin) as the shader computes them
  const uint32_t ul = __funnelshift_r(r.hl.y, r.hl.z, sh1) >> sh2, uh = __funnelshift_r(r.hh.y, r.hh.z, sh1) >> sh2;
  const __half2 dl2 = *reinterpret_cast<const __half2*>(&r.hl.x), dh2 = *reinterpret_cast<const __half2*>(&r.hh.x);
  const float ss_l = __half2float(__hmul(__int2half_rn((int)(ul & 63u)), __low2half(dl2)));
  const float ss_h = __half2float(__hmul(__int2half_rn((int)(uh & 63u)), __low2half(dh2)));
  const float sm_l = __half2float(__hmul(__int2half_rn((int)((ul >> 6) & 63u)), __high2half(dl2)));
  const float sm_h = __half2float(__hmul(__int2half_rn((int)((uh >> 6) & 63u)), __high2half(dh2)));
  // w = (q - 8) * ss + sm = q * ss + (sm - 8 ss); the second term multiplies sum(x) of the pair
  const float of_l = fmaf(-8.0f, ss_l, sm_l), of_h = fmaf(-8.0f, ss_h, sm_h);
#pragma unroll
  for (int j = 0; j < NT; j++) {
    const float sx = sx0[(size_t)j * aux_batch_stride];
    const float dl = dl0[(size_t)j * dl_batch_stride];
    // the high-nibble sums are exact multiples of 16
    const float v0 = (float)((acc_lo[j][0] + (acc_hi[j][0] >> 4)) * 256 + (acc_lo[j][1] + (acc_hi[j][1] >> 4)));
    const float v1 = (float)((acc_lo[j][2] + (acc_hi[j][2] >> 4)) * 256 + (acc_lo[j][3] + (acc_hi[j][3] >> 4)));
    total[j][0] = fmaf(dl, fmaf(ss_l, v0, of_l * sx), total[j][0]);
    total[j][1] = fmaf(dl, fmaf(ss_h, v1, of_h * sx), total[j][1]);
  }
}

// The 16 rows of tile t into L2: one prefetch instruction per 128-byte line, spread over the
// CTA's threads (fire and forget; a 16 x 2304-byte tile is 288 lines, a 16 x 8064-byte tile 1008).
__device__ __forceinline__ void prefetch_tile(const Params& P, int t, int tid) {
  if (t >= P.ntiles) return;
  const int lines_per_row = (P.row_bytes + 127) >> 7;
  for (int i = tid; i < kTileRows * lines_per_row; i += kThreads) {
    const int r = i / lines_per_row, l = i - r * lines_per_row;
    const uint8_t* p = tile_row(P, t, r) + ((size_t)l << 7);
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
  }
}

template <typename T, int NT>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) stream_gemv_kernel(const __grid_constant__ Params P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int M = P.M;
#ifdef MLXR_TUNING
  auto stamp = [&](int i) {
    if (P.trace && tid == 0) P.trace[(size_t)blockIdx.x * 16 + i] = decode::global_ns();
  };
#else
  auto stamp = [&](int) {};
#endif
  stamp(0);
  // Weights are constants of the model: their first tiles are requested before this launch waits
  // for the previous kernel of the stream.
  prefetch_tile(P, blockIdx.x, tid);
  prefetch_tile(P, blockIdx.x + gridDim.x, tid);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // this warp's part of the K range; it converts exactly the activations it multiplies
  const int s_begin = (warp * P.nseg) / kWarps, s_end = ((warp + 1) * P.nseg) / kWarps;
  const int n = s_end - s_begin;
  const int sh1 = c < 2 ? 12 * c : 24, sh2 = c == 3 ? 12 : 0;   // bit position of (scale, min) pair c
  // sub-block s belongs to pair {0,1,0,0,2,3,2,2}[s]; MMA column g stands for pair g >> 1
  const bool keep0 = (int)((0x22320010u >> (4 * c)) & 7u) == (g >> 1);
  const bool keep1 = (int)((0x22320010u >> (4 * (c + 4))) & 7u) == (g >> 1);
  const uint8_t* xbase = smem + (size_t)(g & 1) * P.x_stride + 32 * c;
  const float* sxbase = reinterpret_cast<const float*>(smem + P.off_aux) + c;
  const float* dlbase = reinterpret_cast<const float*>(smem + P.off_delta);
  float* slots = reinterpret_cast<float*>(smem + P.off_slots);   // [2][kWarps][16][NT]
  float* red = reinterpret_cast<float*>(smem + P.off_red);       // [kWarps][NT] sums of squares

  // the first weight segment is requested before the activations: it is independent of them
  int t = blockIdx.x;
  SegRegs ra, rb;
  const uint8_t *rl = nullptr, *rh = nullptr;
  if (t < P.ntiles && n > 0) {
    rl = tile_row(P, t, g) + (size_t)s_begin * kSegBytes;
    rh = tile_row(P, t, g + 8) + (size_t)s_begin * kSegBytes;
    seg_load(ra, rl, rh, c);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  stamp(1);

  // ---- activations of this warp's K part: [x * gamma,] fixed-point split into shared memory.
  // With RMSNorm the factor 1 / rms(x) is a scalar per batch row: the block scaling of the fixed-
  // point format makes the conversion independent of it, so it multiplies the sums in the epilogue
  // and the conversion does not wait for the reduction over the whole row.
  {
    const T* xg = reinterpret_cast<const T*>(P.x);
    const T* gam = reinterpret_cast<const T*>(P.gamma);
    for (int m = 0; m < M; m++) {
      const T* xrow = xg + (size_t)m * P.K;
      float ss = 0.0f;
      for (int s0 = s_begin; s0 < s_end; s0 += 4) {
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; u++)
          if (s0 + u < s_end) load8(xrow + (s0 + u) * 256 + lane * 8, v[u]);
#pragma unroll
        for (int u = 0; u < 4; u++) {
          if (s0 + u >= s_end) break;
          if (gam) {
            float gv[8];
            load8(gam + (s0 + u) * 256 + lane * 8, gv);
#pragma unroll
            for (int i = 0; i < 8; i++) { ss = fmaf(v[u][i], v[u][i], ss); v[u][i] *= gv[i]; }
          }
          emit_segment(smem, P, m, s0 + u, lane, v[u]);
        }
      }
      if (gam) {
        ss = warp_sum(ss);
        if (lane == 0) red[warp * NT + m] = ss;
      }
    }
  }
  __syncwarp();
  stamp(2);

  int it = 0;
  for (; t < P.ntiles; t += gridDim.x, it++) {
    prefetch_tile(P, t + 2 * gridDim.x, tid);
    // rows of the next tile: its first segment is requested before this tile's sums are handed over
    const int tn = t + gridDim.x;
    const uint8_t *nl = nullptr, *nh = nullptr;
    if (tn < P.ntiles) {
      nl = tile_row(P, tn, g) + (size_t)s_begin * kSegBytes;
      nh = tile_row(P, tn, g + 8) + (size_t)s_begin * kSegBytes;
    }
    float total[NT][2];
#pragma unroll
    for (int j = 0; j < NT; j++) total[j][0] = total[j][1] = 0.0f;
    // two segments in flight: the loads of the next one are issued before the math of this one
    for (int s = 0; s < n; s += 2) {
      if (s + 1 < n) seg_load(rb, rl + (size_t)(s + 1) * kSegBytes, rh + (size_t)(s + 1) * kSegBytes, c);
      else if (nl) seg_load(rb, nl, nh, c);
      {
        const int sg = s_begin + s;
        seg_math<NT>(ra, xbase + sg * 256, 2 * P.x_stride, sxbase + sg * 4, P.nseg * 4, dlbase + sg, P.nseg, sh1, sh2, keep0, keep1, total);
      }
      if (s + 1 < n) {
        if (s + 2 < n) seg_load(ra, rl + (size_t)(s + 2) * kSegBytes, rh + (size_t)(s + 2) * kSegBytes, c);
        else if (nl) seg_load(ra, nl, nh, c);
        const int sg = s_begin + s + 1;
        seg_math<NT>(rb, xbase + sg * 256, 2 * P.x_stride, sxbase + sg * 4, P.nseg * 4, dlbase + sg, P.nseg, sh1, sh2, keep0, keep1, total);
      } else {
        ra = rb;   // odd number of segments: the next tile's first segment arrived in the other set
      }
    }
    rl = nl;
    rh = nh;
    // the four lanes of a quad hold the four pairs' parts of (row, batch): add them, then the
    // eight warps' K parts meet in shared memory (double-buffered: one CTA barrier per tile)
    float* mine = slots + ((size_t)(it & 1) * kWarps + warp) * kTileRows * NT;
#pragma unroll
    for (int j = 0; j < NT; j++) {
#pragma unroll
      for (int h = 0; h < 2; h++) {
        float v = total[j][h];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if (c == 0) mine[(g + 8 * h) * NT + j] = v;
      }
    }
    __syncthreads();
    if (it == 0) stamp(3);
    if (warp == (it & (kWarps - 1))) {
      // ===== this warp finishes the tile: fixed warp order, so results are deterministic =====
      const float* sl0 = slots + (size_t)(it & 1) * kWarps * kTileRows * NT;
      float val = 0.0f;   // lane -> (row = lane / NT, batch = lane % NT) for lane < 16 NT
      const int r = lane / NT, m = lane % NT;
      if (lane < kTileRows * NT) {
#pragma unroll
        for (int w8 = 0; w8 < kWarps; w8++) val += sl0[w8 * kTileRows * NT + lane];
        if (P.gamma) {
          float tot = 0.0f;
#pragma unroll
          for (int w8 = 0; w8 < kWarps; w8++) tot += red[w8 * NT + m];
          val *= 1.0f / sqrtf(tot / (float)P.K + P.eps);
        }
      }
      if (P.interleave) {
        // rows 0..7 gate, 8..15 up of the same 8 intermediate indices: h = SiLU(g) * u
        const float up = __shfl_sync(0xffffffffu, val, (lane + 8 * NT) & 31);
        const int col = 8 * t + r;
        if (lane < 8 * NT && m < M && col < P.n_total) {
          const float gv = Act<T>::to_f(Act<T>::from_f(val)), uv = Act<T>::to_f(Act<T>::from_f(up));
          reinterpret_cast<T*>(P.y[0])[(size_t)m * P.n_total + col] = Act<T>::from_f(swish_f(gv) * uv);
        }
      } else {
        // pairs of adjacent rows (2j, 2j+1): plain store or RoPE rotation by the even row's lane
        const float vo = __shfl_sync(0xffffffffu, val, (lane + NT) & 31);
        int R = kTileRows * t + r;
        if (lane < kTileRows * NT && !(r & 1) && m < M && R < P.n_total) {
          int mat = 0;
          if (P.nmat > 1 && R >= P.rows[0]) { R -= P.rows[0]; mat = 1; if (P.nmat > 2 && R >= P.rows[1]) { R -= P.rows[1]; mat = 2; } }
          const bool has_odd = R + 1 < P.rows[mat];
          float ve = val, vod = vo;
          const T* bias = reinterpret_cast<const T*>(P.bias[mat]);
          if (bias) { ve += Act<T>::to_f(bias[R]); if (has_odd) vod += Act<T>::to_f(bias[R + 1]); }
          if (P.epi[mat] == decode::kEpiF32) {
            float* of = reinterpret_cast<float*>(P.y[mat]) + (size_t)m * P.rows[mat] + R;
            of[0] = ve;
            if (has_odd) of[1] = vod;
          } else {
            T* out = reinterpret_cast<T*>(P.y[mat]) + (size_t)m * P.rows[mat] + R;
            if (P.epi[mat] == decode::kEpiRope) {
              const float qe = Act<T>::to_f(Act<T>::from_f(ve)), qo = Act<T>::to_f(Act<T>::from_f(vod));
              const long long pos = (long long)P.positions[m] + P.pos_offset;
              if (pos < 0 || pos >= P.max_seq) { atomicExch(P.status, MLXR_ERR_SHAPE); }
              else {
                const int pairs = P.head_dim >> 1, pi = (R % P.head_dim) >> 1;
                const float cs = __half2float(P.cos_t[(size_t)pos * pairs + pi]);
                const float sn = __half2float(P.sin_t[(size_t)pos * pairs + pi]);
                out[0] = Act<T>::from_f(__fsub_rn(__fmul_rn(qe, cs), __fmul_rn(qo, sn)));
                out[1] = Act<T>::from_f(__fadd_rn(__fmul_rn(qo, cs), __fmul_rn(qe, sn)));
              }
            } else {
              out[0] = Act<T>::from_f(ve);
              if (has_odd) out[1] = Act<T>::from_f(vod);
            }
          }
        }
      }
    }
  }
  stamp(4);
}

}  // namespace sgemv

using namespace sgemv;

bool stream_gemv_supported(int qt, int M, int K, const void* const* w, int nmat) {
  if (qt != MLXR_Q4_K) return false;
  if (M < 1 || M > 2 || K < 256 || K % 256 != 0 || K > 32768) return false;
  for (int i = 0; i < nmat; i++)
    if (((uintptr_t)w[i]) & 15u) return false;
  return true;
}

template <typename T, int NT>
static int launch_inst(const sgemv::Params& P, int grid, size_t smem, cudaStream_t st) {
  auto kern = stream_gemv_kernel<T, NT>;
  static std::mutex mu;
  static size_t smem_set[64] = {};
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  if (smem > 48 * 1024) {
    std::lock_guard<std::mutex> lk(mu);
    if (smem_set[dev & 63] < smem) {
      MLXR_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      smem_set[dev & 63] = smem;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  MLXR_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, P));
  count_launch();
  return MLXR_OK;
}

int launch_stream_gemv(const DecodeLinear& L, int M, int dtype, int* status, cudaStream_t st, const void* next_w, size_t next_bytes) {
  static std::atomic<int> sms[64];
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  int nsm = sms[dev & 63].load();
  if (!nsm) {
    MLXR_CUDA_TRY(cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, dev));
    sms[dev & 63].store(nsm);
  }
  sgemv::Params P;
  memset(&P, 0, sizeof(P));
  int total_rows = 0;
  for (int j = 0; j < 3; j++) {
    P.w[j] = (const uint8_t*)L.w[j];
    P.rows[j] = j < L.nmat ? L.rows[j] : 0;
    P.y[j] = L.y[j];
    P.bias[j] = L.bias[j];
    P.epi[j] = L.epi[j];
    if (j < L.nmat) total_rows += L.rows[j];
    if (j < L.nmat && L.nmat > 1 && !L.interleave && L.rows[j] % 2 != 0) {
      set_error("stream gemv: stacked matrices need even row counts");
      return MLXR_ERR_UNSUPPORTED;
    }
  }
  P.nmat = L.nmat;
  P.interleave = L.interleave;
  P.n_total = L.interleave ? L.rows[0] : total_rows;
  P.K = L.K;
  P.nseg = L.K / 256;
  P.row_bytes = P.nseg * kSegBytes;
  P.ntiles = L.interleave ? (P.n_total + 7) / 8 : (P.n_total + kTileRows - 1) / kTileRows;
  P.M = M;
  P.x = L.x;
  P.gamma = L.gamma;
  P.eps = L.eps;
  P.cos_t = (const __half*)L.cos_t;
  P.sin_t = (const __half*)L.sin_t;
  P.positions = L.positions;
  P.head_dim = L.head_dim;
  P.max_seq = L.max_seq;
  P.pos_offset = L.pos_offset;
  P.status = status;
  P.next_w = (const uint8_t*)next_w;
  P.next_bytes = next_w ? next_bytes : 0;
  P.trace = (unsigned long long*)get_decode_trace();
  if (P.trace && L.x_tagged == 0 && !L.interleave) P.trace += 1024 * 16;   // second launch of a block: its own region
  // shared memory: x as hi / lo int8 rows (16 bytes of padding put the two rows of a batch row 16
  // bytes apart modulo 128: conflict-free 128-bit reads), pair sums, block scales, reduction slots
  P.x_stride = L.K + 16;
  P.off_aux = 2 * M * P.x_stride;
  P.off_delta = P.off_aux + M * P.nseg * 16;
  P.off_slots = (P.off_delta + M * P.nseg * 4 + 15) & ~15;
  P.off_red = P.off_slots + 2 * kWarps * kTileRows * M * 4;
  const size_t smem = (size_t)P.off_red + kWarps * 2 * 4;
  if (P.ntiles < 1) return MLXR_OK;
  // as few waves as the resident CTAs allow, then as few CTAs as that number of waves needs:
  // every CTA gets the same number of tiles (1792 tiles on 296 slots: 256 CTAs x 7)
  const int waves = (P.ntiles + kCtasPerSm * nsm - 1) / (kCtasPerSm * nsm);
  const int grid = (P.ntiles + waves - 1) / waves;
#define BY_NT(T) (M == 1 ? launch_inst<T, 1>(P, grid, smem, st) : launch_inst<T, 2>(P, grid, smem, st))
  if (dtype == MLXR_F16) return BY_NT(__half);
  if (dtype == MLXR_BF16) return BY_NT(__nv_bfloat16);
  return BY_NT(float);
#undef BY_NT
}

}  // namespace mlxr
