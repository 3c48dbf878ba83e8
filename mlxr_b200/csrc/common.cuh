// Shared device/host helpers for the sm_100a quantized-linear kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mlxr_b200.h"

namespace mlxr {

// ---- error plumbing (host) ----------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);  // records text, returns MLXR_ERR_CUDA
void count_launch(int n = 1);

#define MLXR_CUDA_TRY(expr)                                         \
  do {                                                              \
    cudaError_t _e = (expr);                                        \
    if (_e != cudaSuccess) return ::mlxr::cuda_fail(_e, #expr);     \
  } while (0)

// Launch check used after every <<<>>>; counts the launch.
#define MLXR_LAUNCH_CHECK(name)                                     \
  do {                                                              \
    ::mlxr::count_launch();                                         \
    cudaError_t _e = cudaGetLastError();                            \
    if (_e != cudaSuccess) return ::mlxr::cuda_fail(_e, name);      \
  } while (0)

// ---- format geometry (host + device) ------------------------------------------------
// Elements and bytes per block; 0 for a format without code.
__host__ __device__ inline int block_elems(int qt) {
  switch (qt) {
    case MLXR_Q4_0: case MLXR_Q4_1: case MLXR_Q8_0: case MLXR_GGML_Q4_0: return 32;
    case MLXR_Q4_K: case MLXR_GGML_Q4_K: return 256;
    case MLXR_NF4: return 64;
    default: return 0;
  }
}
__host__ __device__ inline int block_bytes(int qt) {
  switch (qt) {
    case MLXR_Q4_0: case MLXR_GGML_Q4_0: return 18; case MLXR_Q4_1: return 20; case MLXR_Q8_0: return 34;
    case MLXR_Q4_K: case MLXR_GGML_Q4_K: return 144; case MLXR_NF4: return 34;
    default: return 0;
  }
}

// The 16 NF4 levels (same literals as the oracle's table).
__device__ __constant__ static const float kNF4[16] = {
#include "nf4_codebook.inc"
};

// ---- activation dtype traits --------------------------------------------------------
template <typename T> struct Act;
template <> struct Act<__half> {
  static constexpr int kDtype = MLXR_F16;
  __device__ static float to_f(__half v) { return __half2float(v); }
  __device__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Act<__nv_bfloat16> {
  static constexpr int kDtype = MLXR_BF16;
  __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Act<float> {
  static constexpr int kDtype = MLXR_F32;
  __device__ static float to_f(float v) { return v; }
  __device__ static float from_f(float v) { return v; }
};

__host__ inline size_t dtype_size(int dt) { return dt == MLXR_F32 ? 4 : 2; }

// Dispatch a lambda-free macro over the activation dtype.
#define MLXR_DISPATCH_DTYPE(dt, T, ...)                                  \
  switch (dt) {                                                          \
    case MLXR_F16: { using T = __half; __VA_ARGS__; break; }             \
    case MLXR_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }     \
    case MLXR_F32: { using T = float; __VA_ARGS__; break; }              \
    default: ::mlxr::set_error("unsupported dtype %d", (int)(dt));       \
             return MLXR_ERR_INVALID_ARGUMENT;                           \
  }

// ---- small device helpers -----------------------------------------------------------
__device__ __forceinline__ uint16_t ld_u16(const uint8_t* p) {
  return __ldg(reinterpret_cast<const uint16_t*>(p));
}
__device__ __forceinline__ __half h_from_bits(uint16_t b) { return __ushort_as_half(b); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// SiLU with the sign-split sigmoid of swiglu_mlp_fused.metal:92-99.
__device__ __forceinline__ float swish_f(float x) {
  if (x >= 0.0f) return x / (1.0f + expf(-x));
  float e = expf(x);
  return x * e / (1.0f + e);
}

// The 6-bit (scale, min) pair the reference shader uses for sub-block s of a Q4_K
// super-block (q_gemm_dequant.metal:222-242): only scales[0..5] are read, and offsets 2
// and 3 inside each group of four take the branch of offset 0.
__device__ __forceinline__ void q4k_pair(const uint8_t* scales, int s, int& sc, int& mn) {
  const int g = s >> 2, o = s & 3;
  const uint32_t b0 = scales[3 * g + 0], b1 = scales[3 * g + 1], b2 = scales[3 * g + 2];
  if (o == 1) {
    sc = ((b1 >> 4) | ((b2 & 0x03u) << 4)) & 0x3F;
    mn = (b2 >> 2) & 0x3F;
  } else {
    sc = b0 & 0x3F;
    mn = ((b0 >> 6) | ((b1 & 0x0Fu) << 2)) & 0x3F;
  }
}

// Dequantize one 32-element unit (unit u of a row = elements [32u, 32u+32)) into fp32,
// with exactly the reference's values: fp32 products for Q4_0 / Q4_1 / Q8_0 / NF4, the
// shader's half arithmetic (one rounding per operation, never contracted) widened to
// fp32 for Q4_K.  `row` points at the first block of the row; only 2-byte
// alignment is assumed.  FUSED selects the single-rounding multiply-add variant of the
// half-precision formulas; HALF_MATH selects the shader's half arithmetic where it
// differs from rounding the fp32 result (Q4_1: half(v) * scale + min in half,
// q_gemm_dequant.metal:166-185).
template <int QT, bool FUSED = false, bool HALF_MATH = false>
__device__ __forceinline__ void dequant_unit(const uint8_t* __restrict__ row, int u,
                                             float (&w)[32]) {
  if constexpr (QT == MLXR_Q4_0) {
    const uint8_t* b = row + (size_t)u * 18;
    const float s = __half2float(h_from_bits(ld_u16(b)));
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t v = ld_u16(b + 2 + 2 * i);
      w[4 * i + 0] = (float)((int)(v & 15u) - 8) * s;
      w[4 * i + 1] = (float)((int)((v >> 4) & 15u) - 8) * s;
      w[4 * i + 2] = (float)((int)((v >> 8) & 15u) - 8) * s;
      w[4 * i + 3] = (float)((int)((v >> 12) & 15u) - 8) * s;
    }
  } else if constexpr (QT == MLXR_Q4_1) {
    const uint8_t* b = row + (size_t)u * 20;
    const __half sh = h_from_bits(ld_u16(b)), mh = h_from_bits(ld_u16(b + 2));
    const float s = __half2float(sh), m = __half2float(mh);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t v = ld_u16(b + 4 + 2 * i);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int q = (int)((v >> (4 * j)) & 15u);
        if constexpr (HALF_MATH) {
          const __half qh = __int2half_rn(q);
          w[4 * i + j] = __half2float(FUSED ? __hfma(qh, sh, mh) : __hadd_rn(__hmul_rn(qh, sh), mh));
        } else {
          w[4 * i + j] = __fadd_rn(__fmul_rn((float)q, s), m);  // product is exact
        }
      }
    }
  } else if constexpr (QT == MLXR_Q8_0) {
    const uint8_t* b = row + (size_t)u * 34;
    const float s = __half2float(h_from_bits(ld_u16(b)));
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const uint32_t v = ld_u16(b + 2 + 2 * i);
      w[2 * i + 0] = (float)(int)(int8_t)(v & 0xFFu) * s;
      w[2 * i + 1] = (float)(int)(int8_t)(v >> 8) * s;
    }
  } else if constexpr (QT == MLXR_NF4) {
    const uint8_t* b = row + (size_t)(u >> 1) * 34;
    const float a = __half2float(h_from_bits(ld_u16(b)));
    const uint8_t* q = b + 2 + (u & 1) * 16;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t v = ld_u16(q + 2 * i);
      w[4 * i + 0] = kNF4[v & 15u] * a;
      w[4 * i + 1] = kNF4[(v >> 4) & 15u] * a;
      w[4 * i + 2] = kNF4[(v >> 8) & 15u] * a;
      w[4 * i + 3] = kNF4[(v >> 12) & 15u] * a;
    }
  } else if constexpr (QT == MLXR_GGML_Q4_0) {
    // canonical ggml block: element i = low nibble of qs[i], element i + 16 = high nibble;
    // w = (q - 8) * d, exact in fp32 (gguf.quants Q4_0.dequantize_blocks)
    const uint8_t* b = row + (size_t)u * 18;
    const float s = __half2float(h_from_bits(ld_u16(b)));
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t v = ld_u16(b + 2 + 2 * i);
      w[2 * i + 0] = (float)((int)(v & 15u) - 8) * s;
      w[2 * i + 1] = (float)((int)((v >> 8) & 15u) - 8) * s;
      w[2 * i + 16] = (float)((int)((v >> 4) & 15u) - 8) * s;
      w[2 * i + 17] = (float)((int)((v >> 12) & 15u) - 8) * s;
    }
  } else if constexpr (QT == MLXR_GGML_Q4_K) {
    // canonical ggml super-block: sub-block s of 64-element chunk j = s / 2 takes the low (s even)
    // or high (s odd) nibbles of qs[32j .. 32j+31]; eight independent 6-bit (scale, min) pairs in
    // the get_scale_min_k4 packing; w = (d * sc) * q - dmin * m with every float32 operation
    // rounded on its own (gguf.quants Q4_K.dequantize_blocks; the products are exact)
    const uint8_t* b = row + (size_t)(u >> 3) * 144;
    const int s = u & 7;
    const float d = __half2float(h_from_bits(ld_u16(b))), dmin = __half2float(h_from_bits(ld_u16(b + 2)));
    uint8_t sc12[12];
#pragma unroll
    for (int i = 0; i < 6; i++) {
      const uint32_t v = ld_u16(b + 4 + 2 * i);
      sc12[2 * i] = (uint8_t)(v & 0xFFu);
      sc12[2 * i + 1] = (uint8_t)(v >> 8);
    }
    int sc, mn;
    if (s < 4) { sc = sc12[s] & 63; mn = sc12[s + 4] & 63; }
    else { sc = (sc12[s + 4] & 0x0F) | ((sc12[s - 4] >> 6) << 4); mn = (sc12[s + 4] >> 4) | ((sc12[s] >> 6) << 4); }
    const float ds = __fmul_rn(d, (float)sc), dm = __fmul_rn(dmin, (float)mn);
    const uint8_t* q = b + 16 + 32 * (s >> 1);
    const int shift = (s & 1) * 4;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const uint32_t v = ld_u16(q + 2 * i);
      w[2 * i + 0] = __fsub_rn(__fmul_rn(ds, (float)((v >> shift) & 15u)), dm);
      w[2 * i + 1] = __fsub_rn(__fmul_rn(ds, (float)((v >> (8 + shift)) & 15u)), dm);
    }
  } else if constexpr (QT == MLXR_Q4_K) {
    const uint8_t* b = row + (size_t)(u >> 3) * 144;
    const int s = u & 7;
    const __half d = h_from_bits(ld_u16(b)), dmin = h_from_bits(ld_u16(b + 2));
    uint8_t sc6[6];
#pragma unroll
    for (int i = 0; i < 3; i++) {
      const uint32_t v = ld_u16(b + 4 + 2 * i);
      sc6[2 * i] = (uint8_t)(v & 0xFFu);
      sc6[2 * i + 1] = (uint8_t)(v >> 8);
    }
    int sc, mn;
    q4k_pair(sc6, s, sc, mn);
    const __half ss = __hmul_rn(__int2half_rn(sc), d);
    const __half sm = __hmul_rn(__int2half_rn(mn), dmin);
    const uint8_t* q = b + 16 + 16 * s;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t v = ld_u16(q + 2 * i);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const __half qv = __int2half_rn((int)((v >> (4 * j)) & 15u) - 8);
        const __half r = FUSED ? __hfma(qv, ss, sm) : __hadd_rn(__hmul_rn(qv, ss), sm);
        w[4 * i + j] = __half2float(r);
      }
    }
  }
}

// Call `F<QT>` for a runtime format value.
#define MLXR_DISPATCH_QT(qt, QT, ...)                                               \
  switch (qt) {                                                                     \
    case MLXR_Q4_0: { constexpr int QT = MLXR_Q4_0; __VA_ARGS__; break; }           \
    case MLXR_Q4_1: { constexpr int QT = MLXR_Q4_1; __VA_ARGS__; break; }           \
    case MLXR_Q8_0: { constexpr int QT = MLXR_Q8_0; __VA_ARGS__; break; }           \
    case MLXR_Q4_K: { constexpr int QT = MLXR_Q4_K; __VA_ARGS__; break; }           \
    case MLXR_NF4: { constexpr int QT = MLXR_NF4; __VA_ARGS__; break; }             \
    case MLXR_GGML_Q4_0: { constexpr int QT = MLXR_GGML_Q4_0; __VA_ARGS__; break; } \
    case MLXR_GGML_Q4_K: { constexpr int QT = MLXR_GGML_Q4_K; __VA_ARGS__; break; } \
    default: ::mlxr::set_error("quant type %d has no implementation", (int)(qt));   \
             return MLXR_ERR_UNSUPPORTED;                                           \
  }

}  // namespace mlxr
