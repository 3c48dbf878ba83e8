// Prefill / large-batch quantized GEMM on the 5th-generation tensor cores:
//   Y[M, N] = X[M, K] * dequant(W[N, K])^T (+ bias),  W packed Q4_K, X and Y fp16 or bf16.
//
// One CTA computes a (MT x 128) x 256 output tile over the whole K:
//   * X tiles (128 rows x 64 K, 16 KB each) arrive by 2-D tensor TMA with the 128-byte swizzle;
//   * sixteen producer warps read the packed Q4_K rows (one weight row and 32-weight sub-block
//     per thread and stage), dequantize (fp16 activations: the reference shader's half
//     arithmetic, q_gemm_dequant.metal:214-259, bit-exact; bf16 activations: one fp32
//     multiply-add from the exact fp16 scale and min, rounded once to bf16) and store the
//     K-major, 128-byte swizzled B tile (256 rows x 64 K, 32 KB);
//   * one thread issues tcgen05.mma (cta_group::1, 128 x 256 x 16, fp32 accumulators in tensor
//     memory); the same B tile feeds MT accumulators (MT x 256 columns of TMEM), which halves
//     the dequantization work per flop at MT = 2;
//   * the producer warps drain the accumulators with tcgen05.ld and store Y.
// Stages are recycled through mbarriers; tcgen05.commit releases a stage when the MMAs that
// read it have finished.  Every wait is bounded: when one gives up, a flag makes all roles leave
// their loops, the TMA thread waits (bounded) for its copies in flight, tensor memory is freed
// and the stream's status word reports MLXR_ERR_TIMEOUT.
#include <cuda.h>
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace mlxr {
namespace prefill {

constexpr int kBM = 128;          // rows of X per accumulator (MMA M)
constexpr int kBN = 256;          // weight rows per tile (MMA N)
constexpr int kBK = 64;           // K per stage: one 128-byte swizzle row of 16-bit elements
constexpr int kProducerWarps = 16; // one (weight row, 32-weight sub-block) per producer thread and stage
constexpr int kThreads = (2 + kProducerWarps) * 32;   // MMA warp, producers, copy warp
constexpr int kRawStages = 3;             // packed Q4_K nibbles staged by TMA: k-blocks in flight
constexpr int kRawBytes = 2 * kBN * 16;   // per k-block: 256 rows x 16 bytes for each of the two sub-blocks
constexpr int kHdrStages = 2;             // super-block headers (256 rows x 16 bytes) in flight
constexpr int kHdrBytes = kBN * 16;
constexpr int kRawRing = kRawStages * kRawBytes + kHdrStages * kHdrBytes;   // 32 KB
constexpr int kATile = kBM * kBK * 2;     // 16 KB
constexpr int kBTile = kBN * kBK * 2;     // 32 KB

struct Params {
  const uint8_t* w;
  const void* bias;
  void* y;
  int M, N, K;
  size_t row_bytes;
  int* status;
  float* partials;    // split-K: [S][M][N] float partial sums (null when S == 1)
  uint32_t* counters; // split-K: one arrival counter per output tile (self-clearing)
  int S;              // K-slices = gridDim.z
  int vec_loads;      // packed buffer is 16-byte aligned and a multiple of 16 bytes long: vector loads allowed
  int debug;          // tuning probes: 1 skip the conversion math, 2 skip the weight loads
};

using namespace tc;


// NW consecutive 32-bit words starting at a 2-byte aligned address, fetched with 16-byte aligned
// read-only loads and funnel shifts (the 18- and 34-byte blocks never line up with vector loads;
// one two-byte load per half word would cost 8 to 16 load instructions per thread and stage).
// Only vectors that contain wanted bytes are read, so the reads stay inside a 16-byte aligned
// buffer whose size is a multiple of 16.
template <int NW>
__device__ __forceinline__ void load_words_2b(const uint8_t* p, uint32_t (&out)[NW]) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint4* base = reinterpret_cast<const uint4*>(a & ~(uintptr_t)15);
  const int off = (int)(a & 15);                    // even
  constexpr int NV = (14 + NW * 4 - 1) / 16 + 1;    // vectors a worst-case offset can touch
  uint32_t w[NV * 4 + 1];
#pragma unroll
  for (int v = 0; v < NV; v++) {
    uint4 q = make_uint4(0u, 0u, 0u, 0u);
    if (v * 16 < off + NW * 4) q = __ldg(base + v);
    w[4 * v] = q.x; w[4 * v + 1] = q.y; w[4 * v + 2] = q.z; w[4 * v + 3] = q.w;
  }
  w[NV * 4] = 0u;
  const int wo = off >> 2;
  const uint32_t sh = (uint32_t)(off & 3) * 8u;     // 0 or 16
#pragma unroll
  for (int c = 0; c < 4; c++) {
    if (wo == c) {
#pragma unroll
      for (int i = 0; i < NW; i++) out[i] = (c + i + 1 <= NV * 4) ? __funnelshift_r(w[c + i], w[c + i + 1], sh) : 0u;
    }
  }
}

// 32 weights (group hb of k-block kb) of a Q4_0 / Q8_0 / NF4 row -> four 16-byte chunks of the
// activation dtype.  Blocks of these formats are only 2-byte aligned.  fp16 activations get the
// reference's value rounded to fp16 (rn16 of the exact product); bf16 one rounding to bf16.
template <int QT, int BF>
__device__ __forceinline__ void dequant32_other(const uint8_t* rowp, int kb, int hb, const float* nf4, bool vec, uint4 (&o)[4]) {
  if constexpr (QT == MLXR_Q4_0) {
    const uint8_t* blk = rowp + (size_t)(2 * kb + hb) * 18;          // q_gemm_dequant.metal:142-161
    const __half d = h_from_bits(ld_u16(blk));
    uint32_t qw[4];
    if (vec) load_words_2b<4>(blk + 2, qw);
    else {
#pragma unroll
      for (int i = 0; i < 4; i++) qw[i] = (uint32_t)ld_u16(blk + 2 + 4 * i) | ((uint32_t)ld_u16(blk + 4 + 4 * i) << 16);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t v = qw[i];
      if constexpr (BF == 0) o[i] = dequant8_f16(v, __half2half2(d), __half2half2(__ushort_as_half((unsigned short)0)));
      else { const float ss = __half2float(d); o[i] = dequant8_bf16(v, ss, -136.0f * ss); }
    }
  } else if constexpr (QT == MLXR_Q8_0) {
    const uint8_t* blk = rowp + (size_t)(2 * kb + hb) * 34;          // q_gemm_dequant.metal:190-201
    const __half d = h_from_bits(ld_u16(blk));
    const float df = __half2float(d);
    uint32_t qw[8];
    if (vec) load_words_2b<8>(blk + 2, qw);
    else {
#pragma unroll
      for (int i = 0; i < 8; i++) qw[i] = (uint32_t)ld_u16(blk + 2 + 4 * i) | ((uint32_t)ld_u16(blk + 4 + 4 * i) << 16);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint32_t out[4];
#pragma unroll
      for (int h2 = 0; h2 < 2; h2++) {
        const int wi = 2 * i + h2;
        const uint32_t u = qw[wi] ^ 0x80808080u;  // bytes q + 128
#pragma unroll
        for (int j = 0; j < 2; j++) {
          if constexpr (BF == 0) {
            // 1024 + (q + 128) as fp16 is 0x6400 | byte; minus 1152 gives q exactly; then one rounding of q * d
            const uint32_t sel = (uint32_t)(2 * j) | ((uint32_t)(2 * j) << 4) | ((uint32_t)(2 * j + 1) << 8) | ((uint32_t)(2 * j + 1) << 12);
            uint32_t bits = (__byte_perm(u, u, sel) & 0x00FF00FFu) | 0x64006400u;
            const __half2 q = __hsub2(*reinterpret_cast<__half2*>(&bits), __half2half2(__ushort_as_half((unsigned short)0x6480)));
            const __half2 r = __hmul2_rn(q, __half2half2(d));
            out[2 * h2 + j] = *reinterpret_cast<const uint32_t*>(&r);
          } else {
            // byte b placed one byte up in 0x4300'0000 is the fp32 number 128 + b / 256
            const float fe = __uint_as_float(__byte_perm(u, 0x00004300u, 0x5606u | ((uint32_t)(2 * j) << 4)));
            const float fo = __uint_as_float(__byte_perm(u, 0x00004300u, 0x5606u | ((uint32_t)(2 * j + 1) << 4)));
            const float s256 = 256.0f * df, c = -32896.0f * df;      // (128 + b/256) * 256 d - (32768 + 128) d = (b - 128) d
            __nv_bfloat162 b2 = __floats2bfloat162_rn(fmaf(fe, s256, c), fmaf(fo, s256, c));
            out[2 * h2 + j] = *reinterpret_cast<const uint32_t*>(&b2);
          }
        }
      }
      o[i] = make_uint4(out[0], out[1], out[2], out[3]);
    }
  } else {   // NF4: 64-element blocks of 34 bytes (fp16 absmax, 32 index bytes, low nibble = even element)
    const uint8_t* blk = rowp + (size_t)kb * 34;
    const float am = __half2float(h_from_bits(ld_u16(blk)));
    uint32_t qw[4];
    if (vec) load_words_2b<4>(blk + 2 + 16 * hb, qw);
    else {
#pragma unroll
      for (int i = 0; i < 4; i++) qw[i] = (uint32_t)ld_u16(blk + 2 + 16 * hb + 4 * i) | ((uint32_t)ld_u16(blk + 4 + 16 * hb + 4 * i) << 16);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t v = qw[i];
      uint32_t out[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float fe = nf4[(v >> (8 * j)) & 15u] * am, fo = nf4[(v >> (8 * j + 4)) & 15u] * am;
        if constexpr (BF == 0) { const __half2 r = __floats2half2_rn(fe, fo); out[j] = *reinterpret_cast<const uint32_t*>(&r); }
        else { __nv_bfloat162 r = __floats2bfloat162_rn(fe, fo); out[j] = *reinterpret_cast<const uint32_t*>(&r); }
      }
      o[i] = make_uint4(out[0], out[1], out[2], out[3]);
    }
  }
}

struct Shared {
  uint64_t full_a[4];
  uint64_t full_b[4];
  uint64_t empty[4];
  uint64_t raw_full[kRawStages];    // the packed nibbles (and header) of a k-block have landed
  uint64_t raw_empty[kRawStages];   // all producer warps have read them
  uint64_t acc_full;
  uint32_t tmem_base;
  int dead;
  int last;
  float nf4[16];
};

// 32 consecutive fp32 sums of output row m starting at column nc -> Y (+ bias), rounded to T
template <typename T>
__device__ __forceinline__ void store_row(const Params& P, int m, int nc, const uint32_t (&r)[32]) {
  T* dst = reinterpret_cast<T*>(P.y) + (size_t)m * P.N + nc;
  const T* bias = reinterpret_cast<const T*>(P.bias);
  if (nc + 32 <= P.N && (P.N & 7) == 0) {
#pragma unroll
    for (int v4 = 0; v4 < 4; v4++) {
      uint32_t pk[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float f0 = __uint_as_float(r[8 * v4 + 2 * e]), f1 = __uint_as_float(r[8 * v4 + 2 * e + 1]);
        if (bias) { f0 += Act<T>::to_f(bias[nc + 8 * v4 + 2 * e]); f1 += Act<T>::to_f(bias[nc + 8 * v4 + 2 * e + 1]); }
        const T t0 = Act<T>::from_f(f0), t1 = Act<T>::from_f(f1);
        pk[e] = (uint32_t)(*reinterpret_cast<const unsigned short*>(&t0)) |
                ((uint32_t)(*reinterpret_cast<const unsigned short*>(&t1)) << 16);
      }
      *reinterpret_cast<uint4*>(dst + 8 * v4) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  } else {
    for (int e = 0; e < 32; e++) {
      if (nc + e < P.N) {
        float f = __uint_as_float(r[e]);
        if (bias) f += Act<T>::to_f(bias[nc + e]);
        dst[e] = Act<T>::from_f(f);
      }
    }
  }
}

// MT accumulators (MT x 128 rows of X) per CTA, STAGES pipeline stages.
// Warp 0: tensor-memory owner and MMA issuer (lane 0).  Warps 1..16: producers; thread pp of them
// owns (weight row pp & 255, sub-block pp >> 8 of the 64-wide k-block).  Warp 17: copies (lane 0):
// the X tiles and, for Q4_K, the packed weights, which reach the producers through a small
// shared-memory ring filled by TMA boxes of 256 rows x 16 bytes (a thread's 16 bytes of nibbles
// sit 2304 or 8064 bytes from its neighbour's in global memory: fetched by the threads
// themselves, every warp-level load touched 32 different sectors and the producers waited on
// them; the TMA unit walks the rows instead and the producers read dense shared memory).
template <int QT, typename T, int MT, int STAGES, int BF>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const Params P) {
  extern __shared__ uint8_t smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  constexpr int kStageBytes = MT * kATile + kBTile;
  uint8_t* rawring = smem + (size_t)STAGES * kStageBytes;          // [kRawStages][2][256][16] then [kHdrStages][256][16]
  uint8_t* hdrring = rawring + kRawStages * kRawBytes;
  Shared* sh = reinterpret_cast<Shared*>(rawring + kRawRing);
  volatile int* dead = &sh->dead;
  constexpr bool kStaged = (QT == MLXR_Q4_K);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kBN, m0 = blockIdx.y * (MT * kBM);
  // this CTA's K-slice: k-blocks [kb0, kb0 + nkb)
  const int nkb_all = P.K / kBK;
  const int kb0 = (int)(((long long)blockIdx.z * nkb_all) / P.S);
  const int nkb = (int)(((long long)(blockIdx.z + 1) * nkb_all) / P.S) - kb0;
  constexpr uint32_t kCols = MT * kBN;        // TMEM columns (256 or 512: powers of two)

  if (tid >= 32 && tid < 48) sh->nf4[tid - 32] = kNF4[tid - 32];
  if (tid == 0) {
    sh->dead = 0;
    for (int s = 0; s < STAGES; s++) {
      mbar_init(smem_u32(&sh->full_a[s]), 1);
      mbar_init(smem_u32(&sh->full_b[s]), kProducerWarps);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int r = 0; r < kRawStages; r++) {
      mbar_init(smem_u32(&sh->raw_full[r]), 1);
      mbar_init(smem_u32(&sh->raw_empty[r]), kProducerWarps);
    }
    mbar_init(smem_u32(&sh->acc_full), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&sh->tmem_base), kCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);

  if (warp == 0) {
    // ===== MMA issuer =====
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(Fmt<T>::v, BF, kBM, kBN);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; kb++) {
        const int s = kb % STAGES, it = kb / STAGES;
        ok = mbar_wait(smem_u32(&sh->full_a[s]), it & 1, dead) && mbar_wait(smem_u32(&sh->full_b[s]), it & 1, dead);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_base = smem_u32(smem + (size_t)s * kStageBytes);
        const uint32_t b_base = a_base + MT * kATile;
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; k++) {
          const uint64_t bdesc = smem_desc_sw128(b_base + k * kUmmaK * 2);
#pragma unroll
          for (int a = 0; a < MT; a++) {
            const uint64_t adesc = smem_desc_sw128(a_base + a * kATile + k * kUmmaK * 2);
            umma_f16(tmem + a * kBN, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(&sh->empty[s]));      // the stage is free when these MMAs are done
      }
      if (ok) umma_commit(smem_u32(&sh->acc_full));
    }
  } else if (warp == 1 + kProducerWarps) {
    // ===== copies =====
    if (lane == 0) {
      int issued = 0;
      for (int i = 0; i < nkb; i++) {
        const int kb = kb0 + i;
        if constexpr (kStaged) {
          // packed nibbles of k-block kb (two boxes: sub-block 2 (kb % 4) and the next one), and the
          // header of its super-block when a new one starts; x in 8-byte elements, always even
          const int r = i % kRawStages, rit = i / kRawStages;
          if (!mbar_wait(smem_u32(&sh->raw_empty[r]), (rit & 1) ^ 1, dead)) break;
          const bool new_sb = (kb & 3) == 0 || i == 0;
          const uint32_t bar = smem_u32(&sh->raw_full[r]);
          mbar_expect_tx(bar, kRawBytes + (new_sb ? kHdrBytes : 0));
          const int xq = 18 * (kb >> 2) + 2 + 4 * (kb & 3);
          tma_load_2d(smem_u32(rawring + (size_t)r * kRawBytes), &wmap, xq, n0, bar);
          tma_load_2d(smem_u32(rawring + (size_t)r * kRawBytes + kBN * 16), &wmap, xq + 2, n0, bar);
          if (new_sb) tma_load_2d(smem_u32(hdrring + (size_t)((kb >> 2) & 1) * kHdrBytes), &wmap, 18 * (kb >> 2), n0, bar);
        }
        const int s = i % STAGES, it = i / STAGES;
        if (!mbar_wait(smem_u32(&sh->empty[s]), (it & 1) ^ 1, dead)) break;
        const uint32_t bar = smem_u32(&sh->full_a[s]);
        mbar_expect_tx(bar, MT * kATile);
#pragma unroll
        for (int a = 0; a < MT; a++)
          tma_load_2d(smem_u32(smem + (size_t)s * kStageBytes + a * kATile), &xmap, kb * kBK, m0 + a * kBM, bar);
        issued = i + 1;
      }
      if (*dead) {
        // copies in flight must land before the CTA may exit (bounded)
        for (int j = max(0, issued - STAGES); j < issued; j++) {
          const uint32_t bar = smem_u32(&sh->full_a[j % STAGES]);
          for (uint32_t sp = 0; sp < kSpin; sp++) if (mbar_try(bar, (j / STAGES) & 1)) break;
        }
        if constexpr (kStaged) {
          for (int j = max(0, issued - kRawStages); j < min(issued + 1, nkb); j++) {
            const uint32_t bar = smem_u32(&sh->raw_full[j % kRawStages]);
            for (uint32_t sp = 0; sp < kSpin; sp++) if (mbar_try(bar, (j / kRawStages) & 1)) break;
          }
        }
      }
    }
  } else {
    // ===== dequantizing producers =====
    const int pp = tid - 32;
    const int p = pp & (kBN - 1), hb = pp >> 8;          // weight row of the tile, sub-block of the k-block
    const int n = n0 + p;
    const bool live = n < P.N;
    const uint8_t* rowp = P.w + (size_t)(live ? n : 0) * P.row_bytes;
    uint4 q0 = make_uint4(0, 0, 0, 0), q1 = q0, hdr = q0;
    // k-block kb: super-block kb / 4, this thread's sub-block s = 2 * (kb % 4) + hb (16 bytes of nibbles)
    auto fetch = [&](int kb, uint4& q) {
      const uint8_t* blk = rowp + (size_t)(kb >> 2) * 144;
      if ((kb & 3) == 0 || kb == kb0) hdr = __ldg(reinterpret_cast<const uint4*>(blk));
      q = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 32 * (kb & 3) + 16 * hb));
    };
    // nibbles are requested two k-blocks ahead (q0: even, q1: odd steps); the header of a
    // super-block arrives with its first k-block and is copied out before the next one overwrites it
    (void)fetch; (void)q0; (void)q1;
    uint4 ch = make_uint4(0, 0, 0, 0);
    for (int i = 0; i < nkb; i++) {
      const int kb = kb0 + i;
      const int s = i % STAGES, it = i / STAGES;
      uint4 cq = make_uint4(0, 0, 0, 0);
      if constexpr (kStaged) {
        // this thread's 16 bytes of nibbles and its row's header from the staged copies
        const int r = i % kRawStages, rit = i / kRawStages;
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->raw_full[r]), rit & 1, dead))) break;   // warp-uniform
        cq = *reinterpret_cast<const uint4*>(rawring + (size_t)r * kRawBytes + (size_t)hb * (kBN * 16) + (size_t)p * 16);
        ch = *reinterpret_cast<const uint4*>(hdrring + (size_t)((kb >> 2) & 1) * kHdrBytes + (size_t)p * 16);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->raw_empty[r]));
      }
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->empty[s]), (it & 1) ^ 1, dead))) break;   // warp-uniform
      uint8_t* brow = smem + (size_t)s * kStageBytes + MT * kATile + (size_t)p * 128;
      uint4 o[4];
#ifdef MLXR_TUNING
      if (live && (P.debug & 1)) {
#pragma unroll
        for (int i = 0; i < 4; i++) o[i] = cq;
      } else
#endif
      if (live && QT != MLXR_Q4_K) {
        dequant32_other<QT, BF>(rowp, kb, hb, sh->nf4, P.vec_loads != 0, o);
      } else if (live) {
        // header: d, dmin (fp16), scales[12].  scales[3g .. 3g+2] of group g = (kb & 3) >> 1 as
        // one 24-bit value (only scales[0..5] are read); sub-block offset o = (2 (kb & 3) + hb) & 3:
        // only o == 1 takes the second pair (offsets 2 and 3 alias offset 0, q_gemm_dequant.metal:222-242)
        const __half d = __ushort_as_half((unsigned short)(ch.x & 0xFFFFu));
        const __half dmin = __ushort_as_half((unsigned short)(ch.x >> 16));
        // the group's three bytes are four consecutive 6-bit fields (scale, min of the first pair, then
        // of the second): the shader's byte-wise extraction reads exactly bits 0-5, 6-11, 12-17, 18-23
        const uint32_t t24 = __funnelshift_r(ch.y, ch.z, (kb & 2) ? 24 : 0);
        const uint32_t pair = (((kb & 1) == 0) && hb == 1) ? (t24 >> 12) : t24;
        const int sc = (int)(pair & 0x3Fu), mn = (int)((pair >> 6) & 0x3Fu);
        const __half ssh = __hmul_rn(__int2half_rn(sc), d), smh = __hmul_rn(__int2half_rn(mn), dmin);
        const uint32_t w4[4] = {cq.x, cq.y, cq.z, cq.w};
        if constexpr (BF == 0) {
          const __half2 ss = __half2half2(ssh), sm = __half2half2(smh);
#pragma unroll
          for (int i = 0; i < 4; i++) o[i] = dequant8_f16(w4[i], ss, sm);
        } else {
          const float ss = __half2float(ssh), c = fmaf(-136.0f, ss, __half2float(smh));
#pragma unroll
          for (int i = 0; i < 4; i++) o[i] = dequant8_bf16(w4[i], ss, c);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; i++) o[i] = make_uint4(0, 0, 0, 0);
      }
      // 16-byte chunk c of row p sits at chunk position c ^ (p & 7) (128-byte swizzle)
#pragma unroll
      for (int i = 0; i < 4; i++) *reinterpret_cast<uint4*>(brow + (((4 * hb + i) ^ (p & 7)) << 4)) = o[i];
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->full_b[s]));
    }
    __syncwarp();
    // ===== epilogue: warp (warp % 4) owns TMEM lanes 32 * (warp % 4) ..; the four producer
    // warps of a quarter share the (accumulator, 32-column chunk) units between them =====
    if (__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->acc_full), 0, dead))) {   // warp-uniform: tcgen05.ld is .aligned
      tc_fence_after();
      const int quarter = warp & 3, gi = (warp - 1) >> 2;
#pragma unroll 1
      for (int u = gi; u < MT * (kBN / 32); u += 4) {
        const int a = u / (kBN / 32), chn = u % (kBN / 32);
        const int m = m0 + a * kBM + quarter * 32 + lane;
        uint32_t r[32];
        tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * kBN + chn * 32), r);
        const int nc = n0 + chn * 32;
        if (m < P.M) {
          if (P.S == 1) {
            store_row<T>(P, m, nc, r);
          } else {
            // split-K: park this slice's sums; the last slice to arrive adds them up below
            float* dst = P.partials + ((size_t)blockIdx.z * P.M + m) * P.N + nc;
            if (nc + 32 <= P.N && (P.N & 3) == 0) {
#pragma unroll
              for (int v4 = 0; v4 < 8; v4++)
                __stcg(reinterpret_cast<float4*>(dst) + v4, make_float4(__uint_as_float(r[4 * v4]), __uint_as_float(r[4 * v4 + 1]),
                                                                       __uint_as_float(r[4 * v4 + 2]), __uint_as_float(r[4 * v4 + 3])));
            } else {
              for (int e = 0; e < 32; e++) if (nc + e < P.N) __stcg(dst + e, __uint_as_float(r[e]));
            }
          }
        }
      }
      if (P.S > 1) __threadfence();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, kCols);
  }
  if (tid == 0 && sh->dead) atomicExch(P.status, MLXR_ERR_TIMEOUT);
  if (P.S > 1) {
    // every warp's partial stores were fenced before the barrier above; the last slice of this
    // output tile adds the S slices in slice order (deterministic) and stores Y
    if (tid == 0) {
      const int tile = blockIdx.y * gridDim.x + blockIdx.x;
      const uint32_t prev = atomicAdd(P.counters + tile, 1u);
      const int last = (prev == (uint32_t)P.S - 1u) && !sh->dead;
      if (prev == (uint32_t)P.S - 1u) P.counters[tile] = 0u;     // self-clearing for the next launch
      __threadfence();
      sh->last = last;
    }
    __syncthreads();
    if (sh->last && warp >= 1 && warp <= kProducerWarps) {
      const int quarter = warp & 3, gi = (warp - 1) >> 2;
#pragma unroll 1
      for (int u = gi; u < MT * (kBN / 32); u += 4) {
        const int a = u / (kBN / 32), chn = u % (kBN / 32);
        const int m = m0 + a * kBM + quarter * 32 + lane;
        const int nc = n0 + chn * 32;
        if (m >= P.M) continue;
        uint32_t r[32];
#pragma unroll
        for (int e = 0; e < 32; e++) r[e] = 0u;
        for (int z = 0; z < P.S; z++) {
          const float* src = P.partials + ((size_t)z * P.M + m) * P.N + nc;
          if (nc + 32 <= P.N && (P.N & 3) == 0) {
#pragma unroll
            for (int v4 = 0; v4 < 8; v4++) {
              const float4 f = __ldcg(reinterpret_cast<const float4*>(src) + v4);
              r[4 * v4] = __float_as_uint(__uint_as_float(r[4 * v4]) + f.x);
              r[4 * v4 + 1] = __float_as_uint(__uint_as_float(r[4 * v4 + 1]) + f.y);
              r[4 * v4 + 2] = __float_as_uint(__uint_as_float(r[4 * v4 + 2]) + f.z);
              r[4 * v4 + 3] = __float_as_uint(__uint_as_float(r[4 * v4 + 3]) + f.w);
            }
          } else {
            for (int e = 0; e < 32; e++) if (nc + e < P.N) r[e] = __float_as_uint(__uint_as_float(r[e]) + __ldcg(src + e));
          }
        }
        store_row<T>(P, m, nc, r);
      }
    }
  }
}

}  // namespace prefill

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// X [M, K] of a 16-bit type as a 2-D tensor (K inner), boxes of 64 x 128 elements with the
// 128-byte swizzle; rows past M read as zero.
static int x_tensor_map(const void* x, int M, int K, int dtype, CUtensorMap* out) {
  static EncodeTiledFn encode = nullptr;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      MLXR_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
      if (!fn || q != cudaDriverEntryPointSuccess) { set_error("cuTensorMapEncodeTiled is not available in this driver"); return MLXR_ERR_CUDA; }
      encode = (EncodeTiledFn)fn;
    }
  }
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)prefill::kBK, (cuuint32_t)prefill::kBM};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(out, dtype == MLXR_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                            const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d) for X [%d, %d]", (int)r, M, K); return MLXR_ERR_CUDA; }
  return MLXR_OK;
}

// Packed Q4_K weights [N rows][row_bytes] as a 2-D tensor of 8-byte elements, boxes of 2 x 256
// (16 bytes of 256 consecutive rows); rows past N read as zero.
static int w_tensor_map(const void* w, int N, size_t row_bytes, CUtensorMap* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  MLXR_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
  if (!fn || q != cudaDriverEntryPointSuccess) { set_error("cuTensorMapEncodeTiled is not available in this driver"); return MLXR_ERR_CUDA; }
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)N};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {2, (cuuint32_t)prefill::kBN};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = ((EncodeTiledFn)fn)(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(w), dims, strides, box, estr,
                                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d) for W [%d rows of %zu bytes]", (int)r, N, row_bytes); return MLXR_ERR_CUDA; }
  return MLXR_OK;
}

bool prefill_supported(int qt, int M, int N, int K, int dtype, const void* x, const void* w, const void* y) {
  if (dtype != MLXR_F16 && dtype != MLXR_BF16) return false;
  if (qt == MLXR_Q4_K) { if (K % 256 != 0 || (((uintptr_t)w) & 15u)) return false; }
  else if (qt == MLXR_Q4_0 || qt == MLXR_Q8_0 || qt == MLXR_NF4) { if (K % 64 != 0 || (((uintptr_t)w) & 1u)) return false; }
  else return false;
  if (M < 9 || N < 1 || K < 64) return false;
  if ((((uintptr_t)x) | ((uintptr_t)y)) & 15u) return false;
  return true;
}

template <int QT, typename T, int MT, int STAGES, int BF>
static int launch_tc(const CUtensorMap& xmap, const CUtensorMap& wmap, const prefill::Params& P, cudaStream_t st) {
  using namespace prefill;
  auto kern = qgemm_tc_kernel<QT, T, MT, STAGES, BF>;
  constexpr size_t smem = (size_t)STAGES * (MT * kATile + kBTile) + kRawRing + sizeof(Shared) + 1024;
  // set once per device; the call is idempotent, the flags are atomic so that concurrent first
  // launches from several host threads do not race on them
  static std::atomic<bool> attr_done[64] = {};
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_done[dev & 63].load(std::memory_order_acquire)) {
    MLXR_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done[dev & 63].store(true, std::memory_order_release);
  }
  dim3 grid((P.N + kBN - 1) / kBN, (P.M + MT * kBM - 1) / (MT * kBM), P.S);
  kern<<<grid, kThreads, smem, st>>>(xmap, wmap, P);
  MLXR_LAUNCH_CHECK("qgemm_tc_kernel");
  return MLXR_OK;
}

// K-slices for a launch: only when one row of tiles (M <= 128) leaves most SMs idle.
int prefill_slices(int M, int N, int K) {
  if (M > prefill::kBM) return 1;
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int ntiles = (N + prefill::kBN - 1) / prefill::kBN, nkb = K / prefill::kBK;
  int S = 1;
  while (S < 8 && ntiles * (S * 2) <= sms && nkb / (S * 2) >= 4) S *= 2;
  return S;
}

int launch_prefill(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int qt, int dtype,
                   int* status, float* partials, uint32_t* counters, int S, cudaStream_t st) {
  CUtensorMap xmap, wmap;
  if (int r = x_tensor_map(x, M, K, dtype, &xmap)) return r;
  memset(&wmap, 0, sizeof(wmap));
  if (qt == MLXR_Q4_K) {
    if (int r = w_tensor_map(w, N, (size_t)(K / 256) * 144, &wmap)) return r;
  }
  prefill::Params P;
  P.w = (const uint8_t*)w;
  P.bias = bias;
  P.y = y;
  P.M = M; P.N = N; P.K = K;
  P.row_bytes = (size_t)(K / block_elems(qt)) * block_bytes(qt);
  P.status = status;
  P.partials = S > 1 ? partials : nullptr;
  P.counters = counters;
  P.S = S;
  P.vec_loads = ((((uintptr_t)w) & 15u) == 0 && ((size_t)N * P.row_bytes) % 16 == 0) ? 1 : 0;
  P.debug = 0;
  if (const char* e = tune_env("MLXR_TC_DEBUG")) P.debug = atoi(e);   // tuning probe
  const bool two = M > prefill::kBM;      // a second accumulator only pays when there are rows for it
  // kind::f16 needs A and B in one format: a bf16 x fp16 mix raised a CUDA error at launch, so
  // for bf16 activations the weights are rounded to bf16 as well
  int rc = MLXR_ERR_UNSUPPORTED;
#define MLXR_TC_BY_QT(QTV)                                                                                     \
  do {                                                                                                         \
    if (dtype == MLXR_F16) rc = two ? launch_tc<QTV, __half, 2, 3, 0>(xmap, wmap, P, st) : launch_tc<QTV, __half, 1, 4, 0>(xmap, wmap, P, st); \
    else rc = two ? launch_tc<QTV, __nv_bfloat16, 2, 3, 1>(xmap, wmap, P, st) : launch_tc<QTV, __nv_bfloat16, 1, 4, 1>(xmap, wmap, P, st);     \
  } while (0)
  switch (qt) {
    case MLXR_Q4_K: MLXR_TC_BY_QT(MLXR_Q4_K); break;
    case MLXR_Q4_0: MLXR_TC_BY_QT(MLXR_Q4_0); break;
    case MLXR_Q8_0: MLXR_TC_BY_QT(MLXR_Q8_0); break;
    case MLXR_NF4: MLXR_TC_BY_QT(MLXR_NF4); break;
    default: set_error("tensor-core GEMM: no producer for %s", mlxr_quant_type_name(qt)); break;
  }
#undef MLXR_TC_BY_QT
  return rc;
}

}  // namespace mlxr
