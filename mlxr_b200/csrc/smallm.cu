// Small-batch Q4_K / Q4_0 linear (3 <= M <= 64 rows of X) on the 5th-generation tensor cores.
//
//   Y[M, N] = X[M, K] * dequant(W)[N, K]^T (+ bias),  X, Y fp16 or bf16, W in MLXR's Q4_K or Q4_0
//   layout (q_gemm_dequant.metal:205-260 and 142-161; q_gemm_dequant_primitive.mm:186-203 for the
//   host contract).  Both formats spend 144 bytes per 256 weights of a row, so the staging is the
//   same and only the producers' reading of the bytes differs.
//
// At these batch sizes the linear is bound by the stream of packed weights from HBM, and the
// work per byte is the conversion of the weights, not the product.  The roles of the operands
// are therefore swapped against the prefill kernel: 128 WEIGHT rows are the M side of a
// tcgen05.mma (the TMEM lanes), the batch (padded to 16, 32 or 64) is its N side, so the
// product costs almost nothing and every weight is converted exactly once.
//
// * Work units are (tile of 128 weight rows, 256-wide super-block of K).  All units of the
//   linear, tile-major, are dealt to the CTAs in equal contiguous ranges (one CTA per SM), so
//   every SM streams the same number of bytes whatever N and K are.  A CTA's range may cover
//   the end of one tile, whole tiles and the start of another; the sums of a tile that several
//   CTAs share are parked as fp32 partials and added, in CTA order, by whichever of them
//   arrives last (a counter per tile, nobody waits).
// * One TMA box per unit brings the tile's 128 x 144 bytes of one super-block (a ring three or
//   four deep: 54-72 KB in flight per SM); 16 producer warps, thread (row, k-block), convert
//   them into the 128-byte-swizzled K-major operand tiles of the unit's four 64-wide k-blocks
//   (a six-deep ring); a second copy warp brings the X tiles a unit at a time (their own ring,
//   two to four units ahead: fetched per k-block behind the MMAs, their L2 round trip was the
//   kernel's pace); four issuer warps, one per k-block, issue the MMAs into accumulators of
//   their own (one issuer for all four needed 0.4 us per k-block and set the pace); four
//   epilogue warps add the four accumulators and drain them, double-buffered in tensor memory
//   so that the next tile's MMAs do not wait for them.
// * Gate/up form: a tile holds 16 gate rows and 16 up rows per TMEM lane quarter (eight TMA
//   boxes from two tensor maps) and the epilogue stores SiLU(gate) * up.
// * Launched with programmatic stream serialization: set-up, the weight stream and the
//   conversion start while the previous kernel of the stream drains; the X loads and everything
//   the epilogue reads or writes wait for griddepcontrol.wait.
// * Every wait is bounded (tc::mbar_wait); a role that gives up sets a flag that the others
//   poll, copies in flight are awaited, tensor memory is freed, and the status word reports
//   MLXR_ERR_TIMEOUT.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <atomic>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace mlxr {
namespace smallm {

using namespace tc;

constexpr int kRows = 128;                 // weight rows per tile (MMA M, TMEM lanes)
constexpr int kBK = 64;                    // K per operand tile: one 128-byte swizzle row
constexpr int kStages = 6;                 // converted operand tiles (one 64-wide k-block each) in flight
constexpr int kMaxXStages = 4, kMaxRawStages = 5;
#ifndef MLXR_SM_RAW16
#define MLXR_SM_RAW16 4      // packed super-blocks in flight at the narrowest batch width
#endif
constexpr int kRawBytes = kRows * 144;     // 18432
constexpr int kATile = kRows * kBK * 2;    // 16 KB
constexpr int kProducerWarps = 16;
constexpr int kWarpEpi0 = 16;              // four epilogue warps: warp % 4 = TMEM lane quarter
constexpr int kWarpMma0 = 20;              // four MMA issuer warps, one per k-block group
constexpr int kWarpRaw = 24, kWarpX = 25;
constexpr int kThreads = 26 * 32;

struct Params {
  const void* bias;
  void* y;
  int M, N, K;
  int nsb;             // super-blocks per row = K / 256
  int ntiles;          // ceil(N / 128)
  int maxc;            // most CTAs that share one tile
  long long U;         // units = ntiles * nsb
  int* status;
  float* partials;     // [ntiles][maxc][NPAD][128] fp32
  uint32_t* counters;  // one per tile, self-clearing
  unsigned long long* trace;   // tuning: 32 time stamps per CTA
  int debug;           // tuning probes (builds with MLXR_TUNING): 1 no conversion math, 2 no weight copies, 4 no MMAs, 8 plain arrives, 16 no X copies after the first ring fill
};

struct Shared {
  // Operand tile s is used alternately by two k-block groups (k-block 4 i + j sits in stage
  // (4 i + j) % 6).  Its n-th use signals through barrier pair [s][n & 1], so that each barrier
  // belongs to one group and every waiter sees consecutive phases of the barrier it polls: with
  // one barrier per stage, a group running two uses ahead of the other would read the parity of
  // the use before last as completion.
  uint64_t full_a[kStages][2];    // the four producer warps of a group have written the tile
  uint64_t x_full[kMaxXStages];   // the four X tiles of a unit have landed
  uint64_t x_empty[kMaxXStages];  // the MMAs that read them are done
  uint64_t empty[kStages][2];     // the MMAs that read it are done
  uint64_t raw_full[kMaxRawStages];
  uint64_t raw_empty[kMaxRawStages];
  uint64_t acc_full[2];         // all MMAs of a tile part are done
  uint64_t acc_empty[2];        // the epilogue has read the accumulator out
  uint32_t tmem_base;
  int dead;
  int last;
  int epi_fail;
};

// first unit of CTA c, and the CTA that owns unit u, when U units are dealt to G CTAs
__host__ __device__ inline long long unit_begin(long long U, int G, int c) { return (U * c) / G; }
__host__ __device__ inline int unit_owner(long long U, int G, long long u) { return (int)(((u + 1) * G - 1) / U); }

// 16 columns of 32 TMEM lanes: thread i of the warp receives lane (base + i)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// SiLU with the sign-split sigmoid of swiglu_mlp_fused.metal:92-99, on the fast exponential and
// reciprocal (relative error about 1e-6, far below the rounding to the activation dtype that
// follows): the epilogue applies it to every batch row in turn, one thread per output column, and
// the exact expf and division made that serial chain several times longer than the tile's MMAs.
__device__ __forceinline__ float swish_fast(float x) {
  const float e = __expf(-fabsf(x));
  const float s = __fdividef(1.0f, 1.0f + e);      // sigmoid(|x|)
  return x * (x >= 0.0f ? s : e * s);
}

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Eight consecutive weights (one word of nibbles) as four bf16 pairs, bf16 arithmetic throughout:
// 0x4300 | n is the bf16 number 128 + n; subtracting 136 gives n - 8 exactly; one fused
// multiply-add with the sub-block's scale and min (both rounded to bf16) rounds once.
__device__ __forceinline__ uint4 dequant8_bf16x2(uint32_t v, __nv_bfloat162 ss, __nv_bfloat162 sm) {
  const uint32_t lo = v & 0x0F0F0F0Fu, hi = (v >> 4) & 0x0F0F0F0Fu;
  const uint32_t w01 = __byte_perm(lo, hi, 0x5140), w23 = __byte_perm(lo, hi, 0x7362);   // (l0,h0,l1,h1), (l2,h2,l3,h3)
  uint32_t b[4] = {__byte_perm(w01, 0x43434343u, 0x4140), __byte_perm(w01, 0x43434343u, 0x4342),
                   __byte_perm(w23, 0x43434343u, 0x4140), __byte_perm(w23, 0x43434343u, 0x4342)};
  uint32_t k136 = 0x43084308u;
  const __nv_bfloat162 off = *reinterpret_cast<__nv_bfloat162*>(&k136);
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const __nv_bfloat162 q = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&b[j]), off);
    const __nv_bfloat162 r = __hfma2(q, ss, sm);
    out[j] = *reinterpret_cast<const uint32_t*>(&r);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

template <int NPAD> struct Rings {
  // shared memory: 96 KB of converted tiles + X + packed weights must stay under 227 KB
  static constexpr int kXStages = NPAD == 64 ? 2 : NPAD == 32 ? 3 : 4;      // X tiles of whole units in flight
  static constexpr int kRawStages = NPAD == 64 ? 3 : NPAD == 16 ? MLXR_SM_RAW16 : 4;   // packed super-blocks in flight
  static constexpr int kXTile = NPAD * kBK * 2;                             // one k-block of X
  static constexpr int kXUnit = 4 * kXTile;                                 // the four k-blocks of a unit
  static constexpr size_t kBytes = (size_t)kStages * kATile + (size_t)kXStages * kXUnit + (size_t)kRawStages * kRawBytes;
};

// SWIGLU: the tile's rows are 16 gate rows and 16 up rows per TMEM lane quarter (from two weight
// matrices, wmap and wmap2), Y = SiLU(gate) * up with gate and up rounded to T first, N = the
// number of gate rows; a tile then covers 64 output columns.
template <int QT, typename T, int NPAD, int BF, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_smallm_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                    const __grid_constant__ CUtensorMap wmap2, const Params P) {
  extern __shared__ uint8_t smem_raw[];
#ifdef MLXR_TUNING
  if (threadIdx.x == 0 && P.trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    P.trace[(size_t)blockIdx.x * 32] = t;
  }
#endif
  // the TMA unit fetches a tensor map on first use: ask for both before anything else
  if (threadIdx.x == kWarpRaw * 32) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&wmap)) : "memory");
  if (threadIdx.x == kWarpX * 32) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&xmap)) : "memory");
  if (SWIGLU && threadIdx.x == kWarpRaw * 32 + 1) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&wmap2)) : "memory");
  using R = Rings<NPAD>;
  constexpr int kXStages = R::kXStages, kRawStages = R::kRawStages, kXTile = R::kXTile, kXUnit = R::kXUnit;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;     // operand tiles need 1024-byte alignment (128-byte swizzle)
  uint8_t* smem = smem_raw + pad;
  uint8_t* aring = smem;
  uint8_t* xring = aring + (size_t)kStages * kATile;
  uint8_t* rawring = xring + (size_t)kXStages * kXUnit;
  Shared* sh = reinterpret_cast<Shared*>(rawring + (size_t)kRawStages * kRawBytes);
  volatile int* dead = &sh->dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  // accumulators: [2 buffers][4 k-block groups][NPAD columns]
  constexpr uint32_t kCols = 8 * NPAD;

  if (tid == 0) {
    sh->dead = 0;
    sh->epi_fail = 0;
    for (int s = 0; s < kStages; s++)
      for (int u = 0; u < 2; u++) {
        mbar_init(smem_u32(&sh->full_a[s][u]), 4);
        mbar_init(smem_u32(&sh->empty[s][u]), 1);
      }
    for (int r = 0; r < kXStages; r++) {
      mbar_init(smem_u32(&sh->x_full[r]), 1);
      mbar_init(smem_u32(&sh->x_empty[r]), 4);       // one commit per k-block group
    }
    for (int r = 0; r < kRawStages; r++) {
      mbar_init(smem_u32(&sh->raw_full[r]), 1);
      mbar_init(smem_u32(&sh->raw_empty[r]), kProducerWarps);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(smem_u32(&sh->acc_full[a]), 4);      // one commit per k-block group
      mbar_init(smem_u32(&sh->acc_empty[a]), 4);     // the four epilogue warps
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kWarpRaw) tmem_alloc(smem_u32(&sh->tmem_base), kCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);
#ifdef MLXR_TUNING
  auto stamp = [&](int i) {
    if (P.trace) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
      P.trace[(size_t)cta * 32 + i] = t;
    }
  };
  if (tid == 0) stamp(1);
#else
  auto stamp = [&](int) {};
#endif

  // Under a programmatic-overlap launch the next kernel of the stream may start its set-up and its
  // weight stream now; whatever it reads or writes that this launch produces waits below
  // (griddepcontrol.wait).  Without the launch attribute both instructions do nothing.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // this CTA's units [u0, u1): unit u = (tile u / nsb, super-block u % nsb)
  const long long u0 = unit_begin(P.U, G, cta), u1 = unit_begin(P.U, G, cta + 1);
  const int nunits = (int)(u1 - u0);
  const int t_first = (int)(u0 / P.nsb), sb_first = (int)(u0 - (long long)t_first * P.nsb);

  if (warp < kProducerWarps) {
    // ===== producers: thread (row p, k-block j of the super-block); the four warps of group j
    // convert k-block j of every unit =====
    const int p = tid & (kRows - 1), j = tid >> 7;
    int s = j;                 // stage of k-block 4 i + j
    int use = 0;               // which use of that stage this is: (4 i + j) / 6
    int r = 0;
    uint32_t rpar = 0;
    const uint32_t a_row0 = smem_u32(aring) + (uint32_t)p * 128u + (uint32_t)((p & 7) << 4);
    for (int i = 0; i < nunits; i++) {
#ifdef MLXR_TUNING
      if (!(P.debug & 2))
#endif
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->raw_full[r]), rpar, dead))) break;   // warp-uniform
      if (tid == 0 && i == 0) stamp(2);
      const uint8_t* rowp = rawring + (size_t)r * kRawBytes + (size_t)p * 144;
      // this thread's 64 weights (two sub-blocks) as eight words of nibbles, element order = nibble
      // order in both formats, and each sub-block's scale and min in fp16
      uint32_t wa[4], wb[4];
      __half ss0, sm0, ss1, sm1;
      if constexpr (QT == MLXR_Q4_K) {
        const uint4 ch = *reinterpret_cast<const uint4*>(rowp);
        const uint4 qa = *reinterpret_cast<const uint4*>(rowp + 16 + 32 * j);
        const uint4 qb = *reinterpret_cast<const uint4*>(rowp + 32 + 32 * j);
        wa[0] = qa.x; wa[1] = qa.y; wa[2] = qa.z; wa[3] = qa.w;
        wb[0] = qb.x; wb[1] = qb.y; wb[2] = qb.z; wb[3] = qb.w;
        // header: d, dmin (fp16), scales[12]; group j >> 1 reads scales[3 (j >> 1) ..] as one 24-bit
        // value.  Sub-block 2 j + hb has offset (2 j + hb) & 3 in its group: offset 1 takes the
        // second (scale, min) pair, offsets 0, 2 and 3 the first (q_gemm_dequant.metal:222-242)
        const __half d = __ushort_as_half((unsigned short)(ch.x & 0xFFFFu));
        const __half dmin = __ushort_as_half((unsigned short)(ch.x >> 16));
        // The three bytes hold four consecutive 6-bit fields: scale and min of the first pair, then of
        // the second (the shader's byte-wise extraction, (b0 & 63), (b0 >> 6 | (b1 & 15) << 2),
        // (b1 >> 4 | (b2 & 3) << 4), (b2 >> 2), reads exactly bits 0-5, 6-11, 12-17, 18-23)
        const uint32_t t24 = __funnelshift_r(ch.y, ch.z, (j & 2) ? 24 : 0);
        const int sc_a = (int)(t24 & 0x3Fu), mn_a = (int)((t24 >> 6) & 0x3Fu);
        const int sc_b = (int)((t24 >> 12) & 0x3Fu), mn_b = (int)((t24 >> 18) & 0x3Fu);
        const bool second = (j & 1) == 0;      // sub-block 2 j + 1 has offset 1 only for even j
        ss0 = __hmul_rn(__int2half_rn(sc_a), d); sm0 = __hmul_rn(__int2half_rn(mn_a), dmin);
        ss1 = __hmul_rn(__int2half_rn(second ? sc_b : sc_a), d); sm1 = __hmul_rn(__int2half_rn(second ? mn_b : mn_a), dmin);
      } else {
        // Q4_0 (q_gemm_dequant.metal:142-161): eight 18-byte blocks {fp16 d, 16 bytes of nibbles} fill
        // the same 144 bytes per 256 weights.  Blocks 2 j and 2 j + 1 are the 36 bytes from 36 j:
        // d0 | 16 nibble bytes (2 bytes off a word boundary) | d1 | 16 nibble bytes (aligned)
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(rowp + 36 * j);
        uint32_t W[9];
#pragma unroll
        for (int q = 0; q < 9; q++) W[q] = wp[q];
#pragma unroll
        for (int q = 0; q < 4; q++) { wa[q] = __funnelshift_r(W[q], W[q + 1], 16); wb[q] = W[5 + q]; }
        ss0 = __ushort_as_half((unsigned short)(W[0] & 0xFFFFu));
        ss1 = __ushort_as_half((unsigned short)(W[4] >> 16));
        sm0 = sm1 = __ushort_as_half((unsigned short)0);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->raw_empty[r]));
      if (++r == kRawStages) { r = 0; rpar ^= 1u; }

      // the MMAs of the stage's previous use (the other group's) must be done
      if (use > 0 && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->empty[s][(use - 1) & 1]), ((use - 1) >> 1) & 1, dead))) break;   // warp-uniform
      // 16-byte chunk c of row p sits at chunk position c ^ (p & 7) (128-byte swizzle): with the row
      // base 128-byte aligned, its shared-memory address is (row base + 16 (p & 7)) ^ 16 c
      const uint32_t arow = a_row0 + (uint32_t)s * kATile;
#ifdef MLXR_TUNING
      if (P.debug & 1) {
#pragma unroll
        for (int c = 0; c < 4; c++) sts128(arow ^ (uint32_t)(c << 4), make_uint4(wa[0], wa[1], wa[2], wa[3]));
#pragma unroll
        for (int c = 0; c < 4; c++) sts128(arow ^ (uint32_t)((4 + c) << 4), make_uint4(wb[0], wb[1], wb[2], wb[3]));
      } else
#endif
      if constexpr (BF == 0) {
        const __half2 s0 = __half2half2(ss0), m0 = __half2half2(sm0), s1 = __half2half2(ss1), m1 = __half2half2(sm1);
#pragma unroll
        for (int c = 0; c < 4; c++) sts128(arow ^ (uint32_t)(c << 4), dequant8_f16(wa[c], s0, m0));
#pragma unroll
        for (int c = 0; c < 4; c++) sts128(arow ^ (uint32_t)((4 + c) << 4), dequant8_f16(wb[c], s1, m1));
      } else {
        const __nv_bfloat162 s0 = __float2bfloat162_rn(__half2float(ss0)), m0 = __float2bfloat162_rn(__half2float(sm0));
        const __nv_bfloat162 s1 = __float2bfloat162_rn(__half2float(ss1)), m1 = __float2bfloat162_rn(__half2float(sm1));
#pragma unroll
        for (int c = 0; c < 4; c++) sts128(arow ^ (uint32_t)(c << 4), dequant8_bf16x2(wa[c], s0, m0));
#pragma unroll
        for (int c = 0; c < 4; c++) sts128(arow ^ (uint32_t)((4 + c) << 4), dequant8_bf16x2(wb[c], s1, m1));
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->full_a[s][use & 1]));
      if (tid == 0 && i < 12) stamp(8 + i);
      s += 4;
      if (s >= kStages) { s -= kStages; use++; }
    }
  } else if (warp >= kWarpMma0 && warp < kWarpMma0 + 4) {
    // ===== MMA issuers: warp j (lane 0) multiplies k-block j of every unit into group j's own
    // accumulator (the epilogue adds the four), so that the four issue streams run side by side =====
    if (lane == 0) {
      const int j = warp - kWarpMma0;
      constexpr uint32_t idesc = instr_desc(Fmt<T>::v, BF, kRows, NPAD);
      // shared-memory descriptors differ only in their start-address field (bits 0-13, in 16-byte units)
      const uint64_t desc_hi = smem_desc_sw128(0);
      const uint32_t a_lo0 = (smem_u32(aring) & 0x3FFFFu) >> 4, x_lo0 = ((smem_u32(xring) + (uint32_t)j * kXTile) & 0x3FFFFu) >> 4;
      int s = j, use = 0, xs = 0, g = 0, sb = sb_first;
      uint32_t xpar = 0;
      bool first = true;
      for (int i = 0; i < nunits; i++) {
        const int ab = g & 1;
        bool ok = true;
        if (first) ok = mbar_wait(smem_u32(&sh->acc_empty[ab]), ((g >> 1) & 1) ^ 1u, dead);
        ok = ok && mbar_wait(smem_u32(&sh->x_full[xs]), xpar, dead) &&
             mbar_wait(smem_u32(&sh->full_a[s][use & 1]), (use >> 1) & 1, dead);
        if (!ok) break;
        tc_fence_after();
        const uint32_t dcol = tmem + (uint32_t)((ab * 4 + j) * NPAD);
        const uint64_t adesc = desc_hi | (uint64_t)(a_lo0 + (uint32_t)s * (kATile >> 4));
        const uint64_t xdesc = desc_hi | (uint64_t)(x_lo0 + (uint32_t)xs * (kXUnit >> 4));
#ifdef MLXR_TUNING
        if (!(P.debug & 4))
#endif
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; k++)
          umma_f16(dcol, adesc + (uint64_t)(k * (kUmmaK * 2 >> 4)), xdesc + (uint64_t)(k * (kUmmaK * 2 >> 4)), idesc, (!first || k > 0) ? 1u : 0u);
        umma_commit(smem_u32(&sh->empty[s][use & 1]));
        umma_commit(smem_u32(&sh->x_empty[xs]));
        const bool last_of_part = (sb + 1 == P.nsb) || (i + 1 == nunits);
        if (last_of_part) umma_commit(smem_u32(&sh->acc_full[ab]));
        first = false;
        if (last_of_part) { first = true; g++; }
        if (++sb == P.nsb) sb = 0;
        if (++xs == kXStages) { xs = 0; xpar ^= 1u; }
        s += 4;
        if (s >= kStages) { s -= kStages; use++; }
      }
    }
  } else if (warp == kWarpRaw) {
    // ===== packed weights: one box of 128 rows x 144 bytes per unit; for gate/up eight boxes of
    // 16 rows, issued by eight lanes at once (one thread issuing eight copies per unit was the
    // kernel's pace).  The whole warp walks the loop. =====
    {
      int issued = 0, t = t_first, sb = sb_first;
      for (int i = 0; i < nunits; i++) {
        const int r = i % kRawStages, rit = i / kRawStages;
#ifdef MLXR_TUNING
        if (P.debug & 2) { issued = 0; continue; }
#endif
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->raw_empty[r]), (rit & 1) ^ 1, dead))) break;
        const uint32_t bar = smem_u32(&sh->raw_full[r]);
        if (lane == 0) mbar_expect_tx(bar, kRawBytes);
        __syncwarp();
        if constexpr (SWIGLU) {
          // lane q < 4: gate rows 64 t + 16 q .. + 15 -> tile rows 32 q ..; lane 4 + q: the same rows of up -> 32 q + 16 ..
          const int q = lane & 3;
          const uint32_t dst = smem_u32(rawring + (size_t)r * kRawBytes + (size_t)(32 * q + (lane < 4 ? 0 : 16)) * 144);
          if (lane < 4) tma_load_2d(dst, &wmap, 18 * sb, 64 * t + 16 * q, bar);
          else if (lane < 8) tma_load_2d(dst, &wmap2, 18 * sb, 64 * t + 16 * q, bar);
        } else {
          if (lane == 0) tma_load_2d(smem_u32(rawring + (size_t)r * kRawBytes), &wmap, 18 * sb, t * kRows, bar);
        }
        __syncwarp();
        issued = i + 1;
        if (++sb == P.nsb) { sb = 0; t++; }
      }
      if (*dead && lane == 0) {   // copies in flight must land before the CTA may exit (bounded)
        for (int i = max(0, issued - kRawStages); i < issued; i++) {
          const uint32_t bar = smem_u32(&sh->raw_full[i % kRawStages]);
          for (uint32_t sp = 0; sp < kSpin; sp++) if (mbar_try(bar, (i / kRawStages) & 1)) break;
        }
      }
    }
  } else if (warp == kWarpX) {
    // ===== activations: per unit the four X tiles [NPAD rows, 64 columns] of its super-block =====
    if (lane == 0) {
      int issued = 0, sb = sb_first, xs = 0;
      uint32_t par = 0;
      asm volatile("griddepcontrol.wait;" ::: "memory");      // X may be the previous kernel's output
      for (int i = 0; i < nunits; i++) {
        if (!mbar_wait(smem_u32(&sh->x_empty[xs]), par ^ 1u, dead)) break;
        const uint32_t bar = smem_u32(&sh->x_full[xs]);
#ifdef MLXR_TUNING
        if ((P.debug & 16) && i >= kXStages) {      // probe: reuse the tiles already in the ring
          mbar_arrive(bar);
          if (++sb == P.nsb) sb = 0;
          if (++xs == kXStages) { xs = 0; par ^= 1u; }
          continue;
        }
#endif
        mbar_expect_tx(bar, kXUnit);
#pragma unroll
        for (int jj = 0; jj < 4; jj++)
          tma_load_2d(smem_u32(xring + (size_t)xs * kXUnit + (size_t)jj * kXTile), &xmap, (4 * sb + jj) * kBK, 0, bar);
        issued = i + 1;
        if (++sb == P.nsb) sb = 0;
        if (++xs == kXStages) { xs = 0; par ^= 1u; }
      }
      if (*dead) {
        for (int i = max(0, issued - kXStages); i < issued; i++) {
          const uint32_t bar = smem_u32(&sh->x_full[i % kXStages]);
          for (uint32_t sp = 0; sp < kSpin; sp++) if (mbar_try(bar, (i / kXStages) & 1)) break;
        }
      }
    }
  } else if (warp >= kWarpEpi0 && warp < kWarpEpi0 + 4) {
    // ===== epilogue: warp quarter q owns TMEM lanes 32 q .. 32 q + 31 = weight rows of the tile =====
    const int quarter = warp & 3, et = tid - kWarpEpi0 * 32;
    const int rt = quarter * 32 + lane;      // row within the tile
    const T* bias = reinterpret_cast<const T*>(P.bias);
    int t = t_first, sb = sb_first, g = 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");        // Y, the partial sums and the tile counters
    for (int i = 0; i < nunits; g++) {
      const int cnt = min(P.nsb - sb, nunits - i);
      const int ab = g & 1;
      const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->acc_full[ab]), (g >> 1) & 1, dead));
      if (!ok) sh->epi_fail = 1;
      epi_barrier();                         // the four warps leave together or not at all
      if (*reinterpret_cast<volatile int*>(&sh->epi_fail)) break;
      tc_fence_after();
      if (et == 0) stamp(g == 0 ? 6 : 24);
      const bool whole = cnt == P.nsb;       // this CTA summed the tile's whole K: store Y directly
      // output column of this lane: its weight row, or for SWIGLU the gate row that lanes l and l + 16 share
      const int n = SWIGLU ? 64 * t + 16 * quarter + (lane & 15) : t * kRows + rt;
      const bool writer = (!SWIGLU || lane < 16) && n < P.N;
      // sums of one batch row -> Y: plain (+ bias), or SiLU(gate) * up across the lane pair
      auto finish = [&](float v, float bv) -> T {
        if constexpr (SWIGLU) {
          const float o = __shfl_xor_sync(0xffffffffu, v, 16);        // lanes < 16: v = gate, o = up
          const float gv = Act<T>::to_f(Act<T>::from_f(v)), uv = Act<T>::to_f(Act<T>::from_f(o));
          return Act<T>::from_f(swish_fast(gv) * uv);
        } else {
          return Act<T>::from_f(v + bv);
        }
      };
      const int slot = whole ? 0 : cta - unit_owner(P.U, G, (long long)t * P.nsb);
      float* part = P.partials + (((size_t)t * P.maxc + slot) * NPAD) * kRows + rt;
      const float bv = (!SWIGLU && bias && n < P.N) ? Act<T>::to_f(bias[n]) : 0.0f;
#pragma unroll 1
      for (int c0 = 0; c0 < NPAD; c0 += 16) {
        // the four groups' sums of these 16 batch columns, added in group order
        uint32_t r[16], q[16];
        const uint32_t base = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * 4 * NPAD + c0);
        tmem_ld16(base, r);
#pragma unroll 1
        for (int jj = 1; jj < 4; jj++) {
          tmem_ld16(base + (uint32_t)(jj * NPAD), q);
#pragma unroll
          for (int c = 0; c < 16; c++) r[c] = __float_as_uint(__uint_as_float(r[c]) + __uint_as_float(q[c]));
        }
        if (whole) {
#pragma unroll
          for (int c = 0; c < 16; c++) {
            if (c0 + c < P.M) {             // uniform: every lane takes part in the exchange
              const T o = finish(__uint_as_float(r[c]), bv);
              if (writer) reinterpret_cast<T*>(P.y)[(size_t)(c0 + c) * P.N + n] = o;
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < 16; c++)
            if (c0 + c < P.M) __stcg(part + (size_t)(c0 + c) * kRows, __uint_as_float(r[c]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[ab]));
      if (!whole) {
        // the last CTA to deliver its part of tile t adds the parts in CTA order and stores Y
        __threadfence();
        epi_barrier();
        if (et == 0) {
          const int nc = unit_owner(P.U, G, (long long)(t + 1) * P.nsb - 1) - unit_owner(P.U, G, (long long)t * P.nsb) + 1;
          const uint32_t prev = atomicAdd(P.counters + t, 1u);
          const int last = prev == (uint32_t)nc - 1u;
          if (last) P.counters[t] = 0u;       // self-clearing for the next launch
          __threadfence();
          sh->last = last ? nc : 0;
        }
        epi_barrier();
        const int nc = *reinterpret_cast<volatile int*>(&sh->last);
        if (nc) {
          const float* src = P.partials + ((size_t)t * P.maxc * NPAD) * kRows + rt;
          // sixteen batch rows and two parts at a time: 32 loads in flight per thread (one load
          // after the other, each L2 round trip would be paid M * nc times)
          for (int m0 = 0; m0 < P.M; m0 += 16) {
            float v[16];
#pragma unroll
            for (int e = 0; e < 16; e++) v[e] = 0.0f;
            for (int z = 0; z < nc; z += 2) {
              float a[16], b[16];
              const bool two = z + 1 < nc;
#pragma unroll
              for (int e = 0; e < 16; e++) a[e] = (m0 + e < P.M) ? __ldcg(src + ((size_t)z * NPAD + m0 + e) * kRows) : 0.0f;
#pragma unroll
              for (int e = 0; e < 16; e++) b[e] = (two && m0 + e < P.M) ? __ldcg(src + ((size_t)(z + 1) * NPAD + m0 + e) * kRows) : 0.0f;
#pragma unroll
              for (int e = 0; e < 16; e++) { v[e] += a[e]; v[e] += b[e]; }
            }
#pragma unroll
            for (int e = 0; e < 16; e++) {
              if (m0 + e < P.M) {
                const T o = finish(v[e], bv);
                if (writer) reinterpret_cast<T*>(P.y)[(size_t)(m0 + e) * P.N + n] = o;
              }
            }
          }
        }
      }
      i += cnt;
      sb = 0;
      t++;
      if (et == 0) stamp(7);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kWarpRaw) {
    tc_fence_after();
    tmem_dealloc(tmem, kCols);
  }
  if (tid == 0 && sh->dead) atomicExch(P.status, MLXR_ERR_TIMEOUT);
  if (tid == 0) stamp(3);
}

}  // namespace smallm

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int tensor_map_encoder(EncodeTiledFn* out) {
  static std::mutex mu;
  static EncodeTiledFn encode = nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    MLXR_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess) { set_error("cuTensorMapEncodeTiled is not available in this driver"); return MLXR_ERR_CUDA; }
    encode = (EncodeTiledFn)fn;
  }
  *out = encode;
  return MLXR_OK;
}

static int device_sms(int* out) {
  static std::atomic<int> sms[64];
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  int n = sms[dev & 63].load();
  if (!n) {
    MLXR_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    sms[dev & 63].store(n);
  }
  *out = n;
  return MLXR_OK;
}

static int smallm_npad(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }

void smallm_partition(long long units, int ctas, int cta, long long unit, long long* begin, long long* end, int* owner) {
  if (begin) *begin = smallm::unit_begin(units, ctas, cta);
  if (end) *end = smallm::unit_begin(units, ctas, cta + 1);
  if (owner) *owner = smallm::unit_owner(units, ctas, unit);
}

bool smallm_supported(int qt, int M, int N, int K, int dtype, const void* x, const void* w) {
  if ((qt != MLXR_Q4_K && qt != MLXR_Q4_0) || (dtype != MLXR_F16 && dtype != MLXR_BF16)) return false;
  if (M < 1 || M > 64 || N < 1 || K < 256 || K % 256 != 0) return false;
  if ((((uintptr_t)x) | ((uintptr_t)w)) & 15u) return false;
  if ((N + smallm::kRows - 1) / smallm::kRows > kSyncWords - 16) return false;   // one counter per tile
  return true;
}

int smallm_plan(int M, int rows, int K, int* grid, int* maxc, size_t* partial_bytes) {
  const int N = rows;
  int sms = 0;
  if (int r = device_sms(&sms)) return r;
  const int nsb = K / 256, ntiles = (N + smallm::kRows - 1) / smallm::kRows;
  const long long U = (long long)ntiles * nsb;
  int G = (int)std::min<long long>(sms, U);
  // Equal ranges make most tiles shared, and a shared tile costs its CTAs an epilogue whose length
  // grows with the padded batch width (partial sums stored, counted, re-read by the last arriver:
  // measured about 3 us at width 16 and 7 to 15 us at width 64).  When there is at most one tile
  // per SM, one whole tile per CTA needs no fix-up at all and only lengthens the loop from U / G
  // units to K / 256: taken when that difference (about 1 us per unit) is below 0.13 us per
  // column of the padded width (measured at N = 14336, K = 4096: batch 32 23.1 -> 19.4 us,
  // batch 64 29.4 -> 21.5 us; at width 16 the equal ranges stay ahead, 19.1 us).
  if (ntiles <= sms && (double)nsb - (double)U / G < 0.13 * smallm_npad(M)) G = ntiles;
  int mc = 1;
  for (int t = 0; t < ntiles; t++)
    mc = std::max(mc, smallm::unit_owner(U, G, (long long)(t + 1) * nsb - 1) - smallm::unit_owner(U, G, (long long)t * nsb) + 1);
  *grid = G;
  *maxc = mc;
  *partial_bytes = (size_t)ntiles * mc * smallm_npad(M) * smallm::kRows * sizeof(float);
  return MLXR_OK;
}

template <int QT, typename T, int NPAD, int BF, bool SWIGLU>
static int launch_inst(const CUtensorMap& xmap, const CUtensorMap& wmap, const CUtensorMap& wmap2, const smallm::Params& P, int grid,
                       cudaStream_t st) {
  using namespace smallm;
  auto kern = qgemm_smallm_kernel<QT, T, NPAD, BF, SWIGLU>;
  constexpr size_t smem = Rings<NPAD>::kBytes + sizeof(Shared) + 1024;
  static std::atomic<bool> attr_done[64] = {};
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_done[dev & 63].load(std::memory_order_acquire)) {
    MLXR_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done[dev & 63].store(true, std::memory_order_release);
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
  MLXR_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, xmap, wmap, wmap2, P));
  count_launch();
  return MLXR_OK;
}

// Packed rows as 8-byte elements, boxes of one super-block (18 elements) x `box_rows` rows; rows past N read as zero.
static int weight_map(EncodeTiledFn encode, const void* w, int N, int K, int box_rows, CUtensorMap* out) {
  const size_t row_bytes = (size_t)(K / 256) * 144;
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)N};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {18, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(w), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d) for W [%d rows of %zu bytes]", (int)r, N, row_bytes); return MLXR_ERR_CUDA; }
  return MLXR_OK;
}

// w2 == nullptr: Y[M, N] = X W^T (+ bias).  Otherwise w = gate, w2 = up (both [N, K]) and
// Y[M, N] = SiLU(X gate^T) * (X up^T), the two products rounded to the activation dtype first.
int launch_smallm(const void* x, const void* w, const void* w2, const void* bias, void* y, int M, int N, int K, int qt, int dtype,
                  int* status, float* partials, uint32_t* counters, int grid, int maxc, cudaStream_t st) {
  EncodeTiledFn encode = nullptr;
  if (int r = tensor_map_encoder(&encode)) return r;
  const int npad = smallm_npad(M);
  const bool swiglu = w2 != nullptr;
  CUtensorMap xmap, wmap, wmap2;
  {
    // X [M, K] of a 16-bit type (K inner), boxes of 64 x NPAD with the 128-byte swizzle; rows past M read as zero
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)smallm::kBK, (cuuint32_t)npad};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(&xmap, dtype == MLXR_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                              const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d) for X [%d, %d]", (int)r, M, K); return MLXR_ERR_CUDA; }
  }
  if (int r = weight_map(encode, w, N, K, swiglu ? 16 : smallm::kRows, &wmap)) return r;
  if (int r = weight_map(encode, swiglu ? w2 : w, N, K, swiglu ? 16 : smallm::kRows, &wmap2)) return r;
  smallm::Params P;
  memset(&P, 0, sizeof(P));
  P.bias = bias;
  P.y = y;
  P.M = M; P.N = N; P.K = K;
  P.nsb = K / 256;
  P.ntiles = ((swiglu ? 2 * N : N) + smallm::kRows - 1) / smallm::kRows;
  P.maxc = maxc;
  P.U = (long long)P.ntiles * P.nsb;
  P.status = status;
  P.partials = partials;
  P.counters = counters;
  if (const char* e = tune_env("MLXR_SM_DEBUG")) P.debug = atoi(e);   // tuning probe
#ifdef MLXR_TUNING
  P.trace = (unsigned long long*)get_decode_trace();
  if (P.trace && swiglu) P.trace += 256 * 32;
#endif
  int rc = MLXR_ERR_UNSUPPORTED;
#define MLXR_SMALLM_BY_NPAD(QTV, T, BF, SW)                                                    \
  do {                                                                                         \
    if (npad == 16) rc = launch_inst<QTV, T, 16, BF, SW>(xmap, wmap, wmap2, P, grid, st);      \
    else if (npad == 32) rc = launch_inst<QTV, T, 32, BF, SW>(xmap, wmap, wmap2, P, grid, st); \
    else rc = launch_inst<QTV, T, 64, BF, SW>(xmap, wmap, wmap2, P, grid, st);                 \
  } while (0)
#define MLXR_SMALLM_BY_DTYPE(QTV)                                                                          \
  do {                                                                                                     \
    if (dtype == MLXR_F16) { if (swiglu) MLXR_SMALLM_BY_NPAD(QTV, __half, 0, true); else MLXR_SMALLM_BY_NPAD(QTV, __half, 0, false); } \
    else { if (swiglu) MLXR_SMALLM_BY_NPAD(QTV, __nv_bfloat16, 1, true); else MLXR_SMALLM_BY_NPAD(QTV, __nv_bfloat16, 1, false); }     \
  } while (0)
  if (qt == MLXR_Q4_K) MLXR_SMALLM_BY_DTYPE(MLXR_Q4_K);
  else if (qt == MLXR_Q4_0) MLXR_SMALLM_BY_DTYPE(MLXR_Q4_0);
  else set_error("small-batch kernel: no producer for %s", mlxr_quant_type_name(qt));
#undef MLXR_SMALLM_BY_DTYPE
#undef MLXR_SMALLM_BY_NPAD
  return rc;
}

}  // namespace mlxr
