// Test oracle: C interface to the reference's own host code for this path, compiled from
// the MLXR tree (q_gemm_dequant_primitive.mm, rope_apply_primitive.mm) against the MLX
// stand-in headers built host-only.  Used to pin mlxr_oracle.c and to generate the golden
// fixtures under tests/golden/; also the "reference" CPU baseline of bench.py.
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>

#include "q_gemm_dequant_primitive.h"
#include "rope_apply_primitive.h"

// CPU dequantizers defined (with external linkage) in q_gemm_dequant_primitive.mm:189-225
namespace mlxr {
namespace kernels {
struct BlockQ4_0;
struct BlockQ4_1;
struct BlockQ8_0;
void dequant_q4_0_cpu(const BlockQ4_0* block, float* output, int offset);
void dequant_q4_1_cpu(const BlockQ4_1* block, float* output, int offset);
void dequant_q8_0_cpu(const BlockQ8_0* block, float* output, int offset);
}  // namespace kernels
}  // namespace mlxr

namespace mx = mlx::core;
using namespace mlxr::kernels;

static thread_local std::string g_err;
#define EXPORT extern "C" __attribute__((visibility("default")))

EXPORT const char* ref_last_error() { return g_err.c_str(); }

// dequant_*_cpu over nblocks consecutive blocks -> fp32
EXPORT int ref_cpu_dequant(int qt, const void* blocks, long nblocks, float* out) {
  const uint8_t* p = static_cast<const uint8_t*>(blocks);
  for (long b = 0; b < nblocks; b++) {
    switch (qt) {
      case 0: dequant_q4_0_cpu(reinterpret_cast<const BlockQ4_0*>(p + b * 18), out, (int)(b * 32)); break;
      case 1: dequant_q4_1_cpu(reinterpret_cast<const BlockQ4_1*>(p + b * 20), out, (int)(b * 32)); break;
      case 2: dequant_q8_0_cpu(reinterpret_cast<const BlockQ8_0*>(p + b * 34), out, (int)(b * 32)); break;
      default: return -1;
    }
  }
  return 0;
}

EXPORT size_t ref_weight_size(int N, int K, int qt) {
  try { return compute_quantized_weight_size(N, K, static_cast<QuantType>(qt)); }
  catch (const std::exception& e) { g_err = e.what(); return 0; }
}
EXPORT float ref_bytes_per_weight(int qt) {
  try { return QGemmDequantPrimitive::get_bytes_per_weight(static_cast<QuantType>(qt)); }
  catch (const std::exception& e) { g_err = e.what(); return -1.0f; }
}
EXPORT int ref_default_group_size(int qt) { return QGemmDequantPrimitive::get_default_group_size(static_cast<QuantType>(qt)); }
EXPORT const char* ref_quant_type_name(int qt) { return quant_type_name(static_cast<QuantType>(qt)); }
EXPORT const char* ref_rope_mode_name(int m) { return rope_scaling_mode_name(static_cast<RoPEScalingMode>(m)); }
EXPORT float ref_ntk_base(float base, float scale, int head_dim, int orig) { return compute_ntk_scaled_base(base, scale, head_dim, orig); }

// q_gemm_dequant() on the CPU device: QGemmDequantPrimitive::eval_cpu
// (q_gemm_dequant_primitive.mm:299-365), fp32 in / fp32 out.
EXPORT int ref_qgemm_cpu(const float* x, const void* w, const float* bias, float* y, int M, int N, int K,
                         int qt, int group_size) {
  try {
    const size_t wbytes = compute_quantized_weight_size(N, K, static_cast<QuantType>(qt));
    mx::array input(x, mx::Shape{M, K}, mx::float32);
    mx::array weights(static_cast<const uint8_t*>(w), mx::Shape{(int)wbytes}, mx::uint8);
    mx::array out = mx::array(0.0f);
    if (bias) {
      mx::array b(bias, mx::Shape{N}, mx::float32);
      out = q_gemm_dequant(input, weights, M, N, K, static_cast<QuantType>(qt), group_size, &b, mx::Device(mx::Device::cpu));
    } else {
      out = q_gemm_dequant(input, weights, M, N, K, static_cast<QuantType>(qt), group_size, nullptr, mx::Device(mx::Device::cpu));
    }
    std::memcpy(y, out.data<float>(), (size_t)M * N * sizeof(float));
    return 0;
  } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// compute_rope_tables (rope_apply_primitive.mm:49-106) -> binary16 bits
EXPORT int ref_rope_tables(int max_seq, int head_dim, float base, int mode, float scale, int orig_ctx,
                           uint16_t* cos_h, uint16_t* sin_h) {
  try {
    auto t = compute_rope_tables(max_seq, head_dim, base, static_cast<RoPEScalingMode>(mode), scale, orig_ctx);
    if (t.first.dtype() != mx::float16) { g_err = "tables are not float16"; return -2; }
    std::memcpy(cos_h, t.first.data<uint16_t>(), t.first.nbytes());
    std::memcpy(sin_h, t.second.data<uint16_t>(), t.second.nbytes());
    return 0;
  } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// rope_apply() on the CPU device: RoPEApplyPrimitive::eval_cpu
// (rope_apply_primitive.mm:191-270); it reads x and the tables as fp32.
// ndim 3: x [batch, heads, d], positions [batch]; ndim 4: x [batch, seq, heads, d].
EXPORT int ref_rope_apply_cpu(const float* x, const float* cos_f, const float* sin_f, const int32_t* pos, float* y,
                              int ndim, int batch, int seq, int heads, int d, int max_seq, int mode, float scale,
                              int offset, int inplace) {
  try {
    mx::Shape xs = ndim == 3 ? mx::Shape{batch, heads, d} : mx::Shape{batch, seq, heads, d};
    mx::Shape ps = ndim == 3 ? mx::Shape{batch} : mx::Shape{batch, seq};
    mx::array input(x, xs, mx::float32);
    mx::array c(cos_f, mx::Shape{max_seq, d / 2}, mx::float32), s(sin_f, mx::Shape{max_seq, d / 2}, mx::float32);
    mx::array p(pos, ps, mx::int32);
    mx::array out = rope_apply(input, c, s, p, static_cast<RoPEScalingMode>(mode), scale, offset, inplace != 0,
                               mx::Device(mx::Device::cpu));
    std::memcpy(y, out.data<float>(), out.nbytes());
    return 0;
  } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
