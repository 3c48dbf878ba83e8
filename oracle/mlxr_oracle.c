/*
 * mlxr_oracle.c -- CPU restatement of MLXR's quantized-linear path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against; nothing in the product (the CUDA library, its C ABI, the C++ primitive
 * layer) calls, links or falls back to it.
 *
 * Each function cites the reference file:line it follows (paths relative to the
 * MLXR source tree).
 *
 * Parity status
 *   Q4_0 / Q8_0 / Q4_1 dequant, fp16->fp32, the eval_cpu GEMM, RoPE and its tables:
 *       pinned against the reference's own C++ (compiled from the reference tree into
 *       oracle/_ref by oracle/Makefile) on fuzzed and hand-built blocks.
 *   Q4_K dequant: pinned against the reference's Metal shader functions compiled
 *       as plain C++ (same recipe); the shader evaluates in `half`, rounding after every
 *       operation, and this file does the same ("unfused").  A "fused" variant, one
 *       rounding for multiply-add, is also provided so the difference can be audited.
 *   NF4: the reference has no NF4 code at all -> parity unpinned.  The format here is
 *       the one the benchmark configuration spells out (64-element blocks, fp16 absmax,
 *       16-level normal-float codebook), see orc_nf4_codebook below.
 *   RMSNorm / SwiGLU / the MLP composition: the reference computes these with MLX array
 *       ops (a third-party dependency, mlx >= 0.12, not vendored); restated in fp32 with
 *       rounding to the activation dtype where the composition materialises an array.
 *       The reference's tests hold tolerances only, no golden vectors -> parity unpinned
 *       beyond those tolerances.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* QuantType values: core/kernels/primitives/q_gemm_dequant_primitive.h:18-35.
 * NF4 is not in the reference enum; 16 is the first free value. */
enum { ORC_Q4_0 = 0, ORC_Q4_1 = 1, ORC_Q8_0 = 2, ORC_Q4_K = 3, ORC_Q6_K = 4, ORC_NF4 = 16 };

/* ------------------------------------------------------------------------------------
 * IEEE binary16 helpers
 * ---------------------------------------------------------------------------------- */

/* binary16 -> binary32, exact.  Follows fp16_to_fp32,
 * core/kernels/primitives/q_gemm_dequant_primitive.mm:141-165: zero keeps its sign,
 * subnormals are mantissa/1024 * 2^-14, Inf keeps its sign and every NaN becomes the
 * canonical positive quiet NaN (sign and payload dropped, :158). */
ORC_API float orc_fp16_to_fp32(uint16_t h) {
  uint32_t sign = (h >> 15) & 1u, exponent = (h >> 10) & 0x1Fu, mantissa = h & 0x3FFu;
  float r;
  if (exponent == 0) {
    if (mantissa == 0) return sign ? -0.0f : 0.0f;
    r = ldexpf((float)mantissa, -24);
  } else if (exponent == 31) {
    if (mantissa) return NAN;
    r = INFINITY;
  } else {
    r = ldexpf((float)(mantissa | 0x400u), (int)exponent - 25);
  }
  return sign ? -r : r;
}

/* double -> binary16 with round-to-nearest-even; overflow goes to Inf, NaN to 0x7E00.
 * Every `half` operation in the shader dequantizers is "compute exactly, round once";
 * a product or a sum of two binary16 values is exact in double, so rounding the double
 * result once gives the correctly rounded binary16 result. */
static uint16_t f64_to_f16(double v) {
  uint16_t sign = signbit(v) ? 0x8000u : 0;
  if (isnan(v)) return 0x7E00u;
  double a = fabs(v);
  if (isinf(a)) return sign | 0x7C00u;
  if (a == 0.0) return sign;
  int e;
  (void)frexp(a, &e);           /* a = m * 2^e, 0.5 <= m < 1  -> unbiased exponent e-1 */
  int ue = e - 1;
  if (ue < -14) ue = -14;        /* subnormal range: fixed quantum 2^-24 */
  double q = ldexp(a, 10 - ue);  /* in units of the quantum, < 2048 */
  double r = nearbyint(q);       /* default rounding mode: to nearest, ties to even */
  if (r >= 2048.0) { r = 1024.0; ue += 1; }
  if (ue > 15) return sign | 0x7C00u;
  uint32_t ri = (uint32_t)r;
  if (ri < 1024) return sign | (uint16_t)ri;                     /* subnormal or zero */
  return sign | (uint16_t)(((uint32_t)(ue + 15) << 10) | (ri - 1024u));
}

ORC_API uint16_t orc_fp32_to_fp16(float f) { return f64_to_f16((double)f); }

static inline double h2d(uint16_t h) { return (double)orc_fp16_to_fp32(h); }
/* half(a) * half(b) and half(a) + half(b) with one rounding each */
static inline uint16_t hmul(uint16_t a, uint16_t b) { return f64_to_f16(h2d(a) * h2d(b)); }
static inline uint16_t hadd(uint16_t a, uint16_t b) { return f64_to_f16(h2d(a) + h2d(b)); }
static inline uint16_t hfma(uint16_t a, uint16_t b, uint16_t c) {
  return f64_to_f16(h2d(a) * h2d(b) + h2d(c)); /* exact in double for |a| <= 63 integers */
}
static inline uint16_t i2h(int v) { return f64_to_f16((double)v); }

/* bfloat16: round-to-nearest-even from fp32 (the conversion CUDA and MLX both use) */
ORC_API uint16_t orc_fp32_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
ORC_API float orc_bf16_to_fp32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f;
}

/* ------------------------------------------------------------------------------------
 * Block layouts: core/kernels/primitives/q_gemm_dequant_primitive.mm:29-57 and
 * core/kernels/metal/q_gemm_dequant.metal:78-131.  All are byte-packed, no padding.
 * ---------------------------------------------------------------------------------- */
#pragma pack(push, 1)
typedef struct { uint16_t scale; uint8_t data[16]; } blk_q4_0;              /* 18 B / 32  */
typedef struct { uint16_t scale; uint16_t min; uint8_t data[16]; } blk_q4_1; /* 20 B / 32  */
typedef struct { uint16_t scale; int8_t data[32]; } blk_q8_0;               /* 34 B / 32  */
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4_k; /* 144 B / 256 */
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } blk_q6_k; /* 210 B / 256 */
typedef struct { uint16_t absmax; uint8_t idx[32]; } blk_nf4;               /* 34 B / 64  */
#pragma pack(pop)

/* Elements per block and bytes per block.
 * get_default_group_size, q_gemm_dequant_primitive.mm:80-92; sizeof(Block*) :63-78. */
ORC_API int orc_block_elems(int qt) {
  switch (qt) {
    case ORC_Q4_0: case ORC_Q4_1: case ORC_Q8_0: return 32;
    case ORC_Q4_K: return 256;
    case ORC_NF4: return 64;
    default: return 0;
  }
}
ORC_API int orc_block_bytes(int qt) {
  switch (qt) {
    case ORC_Q4_0: return 18; case ORC_Q4_1: return 20; case ORC_Q8_0: return 34;
    case ORC_Q4_K: return 144; case ORC_NF4: return 34;
    default: return 0;
  }
}
/* compute_quantized_weight_size, q_gemm_dequant_primitive.mm:116-135:
 * N * ceil(K / block) * sizeof(block). Returns 0 for a format without code. */
ORC_API size_t orc_quantized_weight_size(int N, int K, int qt) {
  int be = orc_block_elems(qt);
  if (!be) return 0;
  size_t groups = (size_t)((K + be - 1) / be);
  return (size_t)N * groups * (size_t)orc_block_bytes(qt);
}

/* ------------------------------------------------------------------------------------
 * Dequantizers, one block each.  fp32 outputs follow the reference's CPU functions;
 * h16 outputs follow the shader (`half` arithmetic).
 * ---------------------------------------------------------------------------------- */

/* dequant_q4_0_cpu, q_gemm_dequant_primitive.mm:189-201: byte i holds elements 2i (low
 * nibble) and 2i+1 (high nibble), value (nibble - 8) * scale in fp32. */
static void deq_q4_0(const blk_q4_0* b, float* out) {
  float s = orc_fp16_to_fp32(b->scale);
  for (int i = 0; i < 16; i++) {
    int8_t v0 = (int8_t)((b->data[i] & 0x0F) - 8);
    int8_t v1 = (int8_t)(((b->data[i] >> 4) & 0x0F) - 8);
    out[2 * i + 0] = v0 * s;
    out[2 * i + 1] = v1 * s;
  }
}
/* dequant_q4_1_cpu, q_gemm_dequant_primitive.mm:203-216 */
static void deq_q4_1(const blk_q4_1* b, float* out) {
  float s = orc_fp16_to_fp32(b->scale), m = orc_fp16_to_fp32(b->min);
  for (int i = 0; i < 16; i++) {
    uint8_t v0 = b->data[i] & 0x0F, v1 = (b->data[i] >> 4) & 0x0F;
    /* -ffp-contract=off in the Makefile keeps these as multiply-then-add */
    out[2 * i + 0] = v0 * s + m;
    out[2 * i + 1] = v1 * s + m;
  }
}
/* Shader dequant_q4_1, q_gemm_dequant.metal:166-185: half(v) * scale + min in half. */
static void deq_q4_1_half(const blk_q4_1* b, uint16_t* out, int fused) {
  for (int i = 0; i < 16; i++) {
    int v0 = b->data[i] & 0x0F, v1 = (b->data[i] >> 4) & 0x0F;
    out[2 * i + 0] = fused ? hfma(i2h(v0), b->scale, b->min) : hadd(hmul(i2h(v0), b->scale), b->min);
    out[2 * i + 1] = fused ? hfma(i2h(v1), b->scale, b->min) : hadd(hmul(i2h(v1), b->scale), b->min);
  }
}
/* dequant_q8_0_cpu, q_gemm_dequant_primitive.mm:218-225 */
static void deq_q8_0(const blk_q8_0* b, float* out) {
  float s = orc_fp16_to_fp32(b->scale);
  for (int i = 0; i < 32; i++) out[i] = b->data[i] * s;
}

/* The 6-bit (scale, min) pair the shader uses for sub-block s of a Q4_K super-block:
 * dequant_q4_k, core/kernels/metal/q_gemm_dequant.metal:222-242.  Only scales[0..5] are
 * read; offsets 2 and 3 of each group of four take the same branch as offset 0. */
static void q4k_pair(const uint8_t* scales, int s, int* sc, int* mn) {
  int g = s / 4, o = s % 4;
  uint8_t b0 = scales[3 * g + 0], b1 = scales[3 * g + 1], b2 = scales[3 * g + 2];
  if (o == 1) {
    *sc = ((b1 >> 4) | ((b2 & 0x03) << 4)) & 0x3F;
    *mn = (b2 >> 2) & 0x3F;
  } else {
    *sc = b0 & 0x3F;
    *mn = ((b0 >> 6) | ((b1 & 0x0F) << 2)) & 0x3F;
  }
}
/* dequant_q4_k, q_gemm_dequant.metal:214-259, all arithmetic in `half`:
 *   sub_scale = half(sc) * d;  sub_min = half(mn) * dmin;
 *   w = half(nibble - 8) * sub_scale + sub_min
 * fused == 0: the product is rounded to half before the add (two roundings);
 * fused != 0: multiply-add with a single rounding (what a contracting compiler emits). */
static void deq_q4_k(const blk_q4_k* b, uint16_t* out, int fused) {
  for (int s = 0; s < 8; s++) {
    int sc, mn;
    q4k_pair(b->scales, s, &sc, &mn);
    uint16_t ss = hmul(i2h(sc), b->d), sm = hmul(i2h(mn), b->dmin);
    for (int i = 0; i < 16; i++) {
      uint8_t byte = b->qs[16 * s + i];
      int v0 = (byte & 0x0F) - 8, v1 = ((byte >> 4) & 0x0F) - 8;
      out[32 * s + 2 * i + 0] = fused ? hfma(i2h(v0), ss, sm) : hadd(hmul(i2h(v0), ss), sm);
      out[32 * s + 2 * i + 1] = fused ? hfma(i2h(v1), ss, sm) : hadd(hmul(i2h(v1), ss), sm);
    }
  }
}
/* Q6_K is deliberately absent: the shader's dequant_q6_k (q_gemm_dequant.metal:265-286)
 * indexes ql[sub_block * 16 + i] with sub_block up to 15, i.e. up to byte 255 of a
 * 210-byte block whose ql array has 128 entries -- it reads the neighbouring block and,
 * for the last block, past the buffer.  There is no well-defined result to restate. */

/* NF4 codebook (no reference counterpart).  Normal-float construction: 8 quantiles on
 * the positive side and 7 on the negative side of a standard normal, evenly spaced in
 * probability between 0.5 and the offset 0.9677083, an exact zero between them, divided
 * by the largest magnitude.  oracle/nf4_codebook.py derives the table with
 * scipy.stats.norm.ppf and prints these literals (fp32-rounded). */
static const float NF4_CODE[16] = {
#include "nf4_codebook.inc"
};
ORC_API const float* orc_nf4_codebook(void) { return NF4_CODE; }
/* NF4 block: 64 elements, byte i holds elements 2i (low nibble) and 2i+1 (high nibble),
 * the nibble order MLXR's Q4_0 uses; w = codebook[idx] * absmax in fp32. */
static void deq_nf4(const blk_nf4* b, float* out) {
  float a = orc_fp16_to_fp32(b->absmax);
  for (int i = 0; i < 32; i++) {
    out[2 * i + 0] = NF4_CODE[b->idx[i] & 0x0F] * a;
    out[2 * i + 1] = NF4_CODE[(b->idx[i] >> 4) & 0x0F] * a;
  }
}

/* Dequantize a whole [N, K] packed matrix, block index n * (K / blk) + g as at
 * q_gemm_dequant_primitive.mm:319-338 and q_gemm_dequant.metal:410-411.  K must be a
 * whole number of blocks (the reference overruns the row otherwise).
 * out_f32: fp32 values (for Q4_K the half results widened exactly).
 * out_h16 (may be NULL): binary16 bits -- for Q4_0/Q8_0/NF4 the fp32 value rounded once
 *   to half, which is what the shader's half multiply produces (the fp32 product of a
 *   small integer and a half is exact); Q4_1 in the shader's half arithmetic.
 * flags bit 0: Q4_K / Q4_1 multiply-add fused (single rounding) in the half formulas.
 * Returns 0, or -1 for an unsupported format / ragged K. */
ORC_API int orc_dequantize(int qt, const void* w, int N, int K, float* out_f32,
                           uint16_t* out_h16, int flags) {
  int be = orc_block_elems(qt);
  if (!be || K % be) return -1;
  size_t nblk = (size_t)N * (size_t)(K / be);
  const uint8_t* p = (const uint8_t*)w;
  int bb = orc_block_bytes(qt);
  float tmp[256];
  uint16_t th[256];
  for (size_t i = 0; i < nblk; i++, p += bb) {
    int is_half = 0;
    switch (qt) {
      case ORC_Q4_0: deq_q4_0((const blk_q4_0*)p, tmp); break;
      case ORC_Q4_1: deq_q4_1((const blk_q4_1*)p, tmp);
                     if (out_h16) deq_q4_1_half((const blk_q4_1*)p, out_h16 + i * be, flags & 1);
                     break;
      case ORC_Q8_0: deq_q8_0((const blk_q8_0*)p, tmp); break;
      case ORC_NF4: deq_nf4((const blk_nf4*)p, tmp); break;
      case ORC_Q4_K: deq_q4_k((const blk_q4_k*)p, th, flags & 1); is_half = 1; break;
      default: return -1;
    }
    for (int e = 0; e < be; e++) {
      if (is_half) {
        if (out_f32) out_f32[i * be + e] = orc_fp16_to_fp32(th[e]);
        if (out_h16) out_h16[i * be + e] = th[e];
      } else {
        if (out_f32) out_f32[i * be + e] = tmp[e];
        if (out_h16 && qt != ORC_Q4_1) out_h16[i * be + e] = orc_fp32_to_fp16(tmp[e]);
      }
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------------------
 * GEMM: QGemmDequantPrimitive::eval_cpu, q_gemm_dequant_primitive.mm:299-365.
 * Full dequantization to fp32, then for every (m, n) a sequential fp32 sum over k in
 * increasing order, bias added last.  The reference only does this for Q4_0/Q4_1/Q8_0
 * (:330-341); the same loop is applied here to the other formats' dequantized values.
 * ---------------------------------------------------------------------------------- */
ORC_API int orc_qgemm_cpu(const float* x, const void* w, const float* bias, float* y,
                          int M, int N, int K, int qt) {
  float* wd = (float*)malloc((size_t)N * K * sizeof(float));
  if (!wd) return -2;
  if (orc_dequantize(qt, w, N, K, wd, NULL, 0)) { free(wd); return -1; }
  for (int m = 0; m < M; m++)
    for (int n = 0; n < N; n++) {
      float acc = 0.0f;
      for (int k = 0; k < K; k++) acc += x[(size_t)m * K + k] * wd[(size_t)n * K + k];
      if (bias) acc += bias[n];
      y[(size_t)m * N + n] = acc;
    }
  free(wd);
  return 0;
}

/* Same loop over an already dequantized fp32 matrix, rows [n0, n1) only: lets the CPU
 * baseline time a bounded sample of a large workload. */
ORC_API void orc_gemm_rows_f32(const float* x, const float* wd, float* y, int M, int N,
                               int K, int n0, int n1) {
  for (int m = 0; m < M; m++)
    for (int n = n0; n < n1; n++) {
      float acc = 0.0f;
      for (int k = 0; k < K; k++) acc += x[(size_t)m * K + k] * wd[(size_t)n * K + k];
      y[(size_t)m * N + n] = acc;
    }
}

/* ------------------------------------------------------------------------------------
 * RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w.
 * Composition of MLX ops at core/graph/layers.cpp:39-55 and
 * rmsnorm_primitive.mm:122-131; kernel at core/kernels/metal/rmsnorm.metal:39-156.
 * The kernel's order is kept: per-thread strided partial sums (threads = min(1024,
 * hidden), rmsnorm_primitive.mm:210-228), power-of-two tree over the partials, mean,
 * rsqrt, then (x * rms) * w with the product rounded to the I/O dtype once at the store.
 * Inputs and outputs are fp32 here; the caller rounds to fp16/bf16.
 * ---------------------------------------------------------------------------------- */
ORC_API void orc_rmsnorm(const float* x, const float* w, float* y, int rows, int hidden,
                         float eps) {
  int threads = hidden < 1024 ? hidden : 1024;
  int p2 = 1; while (p2 * 2 <= threads) p2 *= 2;   /* the tree assumes a power of two */
  float* part = (float*)calloc((size_t)threads, sizeof(float));
  for (int r = 0; r < rows; r++) {
    const float* xr = x + (size_t)r * hidden;
    for (int t = 0; t < threads; t++) {
      float s = 0.0f;
      for (int i = t; i < hidden; i += threads) s += xr[i] * xr[i];
      part[t] = s;
    }
    /* threads beyond the largest power of two are folded in first so that no partial
     * is lost when hidden is not a power of two */
    for (int t = p2; t < threads; t++) part[t - p2] += part[t];
    for (int stride = p2 / 2; stride > 0; stride >>= 1)
      for (int t = 0; t < stride; t++) part[t] += part[t + stride];
    float mean_sq = part[0] / (float)hidden;
    float rms = 1.0f / sqrtf(mean_sq + eps);
    for (int i = 0; i < hidden; i++) {
      float normalized = xr[i] * rms;
      y[(size_t)r * hidden + i] = normalized * w[i];
    }
  }
  free(part);
}

/* ------------------------------------------------------------------------------------
 * SwiGLU: h = g * sigmoid(g) * u.
 * swish/swiglu at swiglu_mlp_primitive.mm:306-318, MLP::forward at
 * core/graph/layers.cpp:400-420; the shader's sign-split sigmoid at
 * core/kernels/metal/swiglu_mlp_fused.metal:92-99 is used so large |g| cannot overflow.
 * ---------------------------------------------------------------------------------- */
static inline float swish_f(float x) {
  if (x >= 0.0f) return x / (1.0f + expf(-x));
  float e = expf(x);
  return x * e / (1.0f + e);
}
ORC_API void orc_swiglu(const float* g, const float* u, float* h, size_t n) {
  for (size_t i = 0; i < n; i++) h[i] = swish_f(g[i]) * u[i];
}

/* ------------------------------------------------------------------------------------
 * RoPE tables: compute_rope_tables, rope_apply_primitive.mm:49-106.
 * theta = pos * base^(-2p/d) with powf/cosf/sinf in fp32, tables [max_seq, d/2] cast to
 * binary16 (:101-103).  NTK rescales the base by (scale - (scale - 1))^(d/(d-2)), which
 * is 1 (:37-47); LINEAR divides the position by scale_factor (:78-80).
 * mode: 0 BASE, 1 NTK, 2 YARN (no code in the reference: treated as BASE), 3 LINEAR.
 * ---------------------------------------------------------------------------------- */
ORC_API void orc_rope_tables(int max_seq, int head_dim, float base, int mode,
                             float scale_factor, uint16_t* cos_h, uint16_t* sin_h,
                             float* cos_f, float* sin_f) {
  int pairs = head_dim / 2;
  float eff = base;
  if (mode == 1) {
    float exponent = (float)head_dim / (float)(head_dim - 2);
    float sf = scale_factor - (scale_factor - 1);
    eff = base * powf(sf, exponent);
  }
  for (int pos = 0; pos < max_seq; pos++) {
    float position = (float)pos;
    if (mode == 3) position /= scale_factor;
    for (int p = 0; p < pairs; p++) {
      float freq_exponent = -2.0f * p / head_dim;
      float freq = powf(eff, freq_exponent);
      float theta = position * freq;
      float c = cosf(theta), s = sinf(theta);
      size_t idx = (size_t)pos * pairs + p;
      if (cos_f) cos_f[idx] = c;
      if (sin_f) sin_f[idx] = s;
      if (cos_h) cos_h[idx] = orc_fp32_to_fp16(c);
      if (sin_h) sin_h[idx] = orc_fp32_to_fp16(s);
    }
  }
}

/* RoPE application: RoPEApplyPrimitive::eval_cpu, rope_apply_primitive.mm:191-270, and
 * the kernel core/kernels/metal/rope_apply.metal:103-172.  Interleaved pairs (2p, 2p+1):
 *   y_e = x_e*c - x_o*s;  y_o = x_o*c + x_e*s;   table index (pos + offset)*(d/2) + p;
 * LINEAR mode multiplies both outputs by scale_factor (:259-262).  fp32 math; tables are
 * given as fp32 values (the caller widens the binary16 tables exactly).
 * x is [batch, seq, heads, d]; positions is [batch] when seq == 1, else [batch, seq]. */
ORC_API void orc_rope_apply(const float* x, const float* cos_t, const float* sin_t,
                            const int32_t* positions, float* y, int batch, int seq,
                            int heads, int head_dim, int mode, float scale_factor,
                            int position_offset) {
  int pairs = head_dim / 2;
  for (int b = 0; b < batch; b++)
    for (int t = 0; t < seq; t++) {
      int position = (seq == 1 ? positions[b] : positions[b * seq + t]) + position_offset;
      for (int h = 0; h < heads; h++) {
        size_t off = (((size_t)b * seq + t) * heads + h) * head_dim;
        for (int p = 0; p < pairs; p++) {
          float xe = x[off + 2 * p], xo = x[off + 2 * p + 1];
          float c = cos_t[(size_t)position * pairs + p], s = sin_t[(size_t)position * pairs + p];
          float ye = xe * c - xo * s;
          float yo = xo * c + xe * s;
          if (mode == 3) { ye *= scale_factor; yo *= scale_factor; }
          y[off + 2 * p] = ye;
          y[off + 2 * p + 1] = yo;
        }
      }
    }
}

/* RoPE of the graph layer: graph::RotaryEmbedding, core/graph/layers.cpp:113-225 ("parity
 * unpinned" beyond elementary IEEE arithmetic: the composition is made of MLX ops, and MLX is an
 * absent third-party dependency).  compute_freqs (:121-154): freq_i = 1 / pow(base, 2i/dim),
 * angle = pos * freq_i, float32 tables [max_seq, dim/2].  forward (:157-225): the head splits
 * into halves x1 | x2, positions are offset .. offset + seq,
 *   y1 = x1*cos - x2*sin;  y2 = x2*cos + x1*sin
 * where every product and every sum is a separately materialised float32 array (built without
 * contraction: the Makefile passes -ffp-contract=off). */
ORC_API void orc_rope_tables_f32(int max_seq, int dim, float base, float* cos_f, float* sin_f) {
  int half = dim / 2;
  for (int pos = 0; pos < max_seq; pos++)
    for (int i = 0; i < half; i++) {
      float freq = 1.0f / powf(base, (2.0f * i) / dim);
      float angle = (float)pos * freq;
      cos_f[(size_t)pos * half + i] = cosf(angle);
      sin_f[(size_t)pos * half + i] = sinf(angle);
    }
}
ORC_API void orc_rope_split_half(const float* x, const float* cos_t, const float* sin_t, float* y,
                                 int batch, int seq, int heads, int head_dim, int offset) {
  int half = head_dim / 2;
  for (int b = 0; b < batch; b++)
    for (int t = 0; t < seq; t++)
      for (int h = 0; h < heads; h++) {
        size_t off = (((size_t)b * seq + t) * heads + h) * head_dim;
        for (int p = 0; p < half; p++) {
          float x1 = x[off + p], x2 = x[off + half + p];
          float c = cos_t[(size_t)(offset + t) * half + p], s = sin_t[(size_t)(offset + t) * half + p];
          float x1c = x1 * c, x2s = x2 * s, x2c = x2 * c, x1s = x1 * s;
          y[off + p] = x1c - x2s;
          y[off + half + p] = x2c + x1s;
        }
      }
}

/* In-place rounding of an fp32 buffer to the activation dtype and back (0 fp16, 1 bf16,
 * anything else: unchanged): marks the points where the composition materialises an
 * fp16/bf16 array. */
ORC_API void orc_round_to(float* v, size_t n, int dtype) {
  if (dtype == 0) for (size_t i = 0; i < n; i++) v[i] = orc_fp16_to_fp32(orc_fp32_to_fp16(v[i]));
  else if (dtype == 1) for (size_t i = 0; i < n; i++) v[i] = orc_bf16_to_fp32(orc_fp32_to_bf16(v[i]));
}
