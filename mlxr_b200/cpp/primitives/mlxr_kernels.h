// MLXR's kernel primitives (namespace mlxr::kernels) on the B200 path.
//
// Same class names, constructor arguments, accessors, free functions, default arguments,
// primitive names and exception types as the four reference headers
//   core/kernels/primitives/q_gemm_dequant_primitive.h   (QuantType, QGemmDequantPrimitive, q_gemm_dequant, ...)
//   core/kernels/primitives/rmsnorm_primitive.h           (RMSNormPrimitive, rmsnorm_fused)
//   core/kernels/primitives/swiglu_mlp_primitive.h        (SwiGLUMLPPrimitive, swiglu_mlp, swish, swiglu)
//   core/kernels/primitives/rope_apply_primitive.h        (RoPEScalingMode, RoPEApplyPrimitive, rope_apply, ...)
// so that code written against those headers compiles unchanged.  eval_gpu hands the
// arrays' pointers to the C ABI (include/mlxr_b200.h); eval_cpu throws: this build has no
// CPU path.  Additions that MLXR does not have are marked "extension".
#pragma once

#include <utility>
#include <vector>

#include <mlx/array.h>
#include <mlx/device.h>
#include <mlx/primitives.h>
#include <mlx/stream.h>
#include <mlx/utils.h>

namespace mlxr {
namespace kernels {

namespace mx = mlx::core;

// q_gemm_dequant_primitive.h:18-35; NF4 is an extension (the first free value)
enum class QuantType {
  Q4_0 = 0, Q4_1 = 1, Q8_0 = 2, Q4_K = 3, Q6_K = 4, Q5_0 = 5, Q5_1 = 6, Q8_1 = 7,
  Q2_K = 8, Q3_K = 9, Q5_K = 10, Q8_K = 11, IQ2_XXS = 12, IQ2_XS = 13, IQ3_XXS = 14, IQ3_S = 15,
  NF4 = 16,
};

// rope_apply_primitive.h:18-23
enum class RoPEScalingMode { BASE = 0, NTK = 1, YARN = 2, LINEAR = 3 };

// Shared boilerplate of the four primitives: no CPU path, no autodiff / vmap (the
// reference throws "not yet implemented" for these as well).
class B200Primitive : public mx::Primitive {
 public:
  using mx::Primitive::Primitive;
  void eval_cpu(const std::vector<mx::array>& inputs, std::vector<mx::array>& outputs) override;
  std::pair<std::vector<mx::array>, std::vector<int>> vmap(const std::vector<mx::array>& inputs,
                                                           const std::vector<int>& axes) override;
  std::vector<mx::array> jvp(const std::vector<mx::array>& primals, const std::vector<mx::array>& tangents,
                             const std::vector<int>& argnums) override;
  std::vector<mx::array> vjp(const std::vector<mx::array>& primals, const std::vector<mx::array>& cotangents,
                             const std::vector<int>& argnums, const std::vector<mx::array>& outputs) override;
};

// ---- Y = X W^T (+ bias), W packed ------------------------------------------------------------
// q_gemm_dequant_primitive.h:78-195.  Inputs [input [M,K], weights (bytes), bias [N]?].
class QGemmDequantPrimitive : public B200Primitive {
 public:
  QGemmDequantPrimitive(mx::Stream stream, int M, int N, int K, QuantType quant_type, int group_size,
                        bool has_bias = false);
  ~QGemmDequantPrimitive() override;
  void eval_gpu(const std::vector<mx::array>& inputs, std::vector<mx::array>& outputs) override;
  std::vector<mx::Shape> output_shapes(const std::vector<mx::array>&) override { return {{M_, N_}}; }
  const char* name() const override { return "q_gemm_dequant"; }
  bool is_equivalent(const mx::Primitive& other) const override;
  int M() const { return M_; }
  int N() const { return N_; }
  int K() const { return K_; }
  QuantType quant_type() const { return quant_type_; }
  int group_size() const { return group_size_; }
  bool has_bias() const { return has_bias_; }
  static float get_bytes_per_weight(QuantType type);   // throws for a format without code
  static int get_default_group_size(QuantType type);

 private:
  int M_, N_, K_;
  QuantType quant_type_;
  int group_size_;
  bool has_bias_;
};

mx::array q_gemm_dequant(const mx::array& input, const mx::array& weights, int M, int N, int K,
                         QuantType quant_type, int group_size, const mx::array* bias = nullptr,
                         mx::StreamOrDevice s = {});
size_t compute_quantized_weight_size(int N, int K, QuantType quant_type);
const char* quant_type_name(QuantType type);
// extension: the reference's dequantizers on their own ([N, K] float16 or float32)
mx::array dequantize(const mx::array& weights, int N, int K, QuantType quant_type,
                     mx::Dtype out_dtype = mx::float16, mx::StreamOrDevice s = {});

// ---- RMSNorm ------------------------------------------------------------------------------------
// rmsnorm_primitive.h:31-126.  Lazy: rmsnorm_fused returns an unevaluated array.
class RMSNormPrimitive : public B200Primitive {
 public:
  explicit RMSNormPrimitive(mx::Stream stream, float eps);
  ~RMSNormPrimitive() override;
  void eval_gpu(const std::vector<mx::array>& inputs, std::vector<mx::array>& outputs) override;
  std::vector<mx::Shape> output_shapes(const std::vector<mx::array>& inputs) override { return {inputs[0].shape()}; }
  const char* name() const override { return "rmsnorm_fused"; }
  bool is_equivalent(const mx::Primitive& other) const override;
  float eps() const { return eps_; }

 private:
  float eps_;
};
mx::array rmsnorm_fused(const mx::array& input, const mx::array& weight, float eps = 1e-6f,
                        mx::StreamOrDevice s = {});

// ---- SwiGLU MLP ---------------------------------------------------------------------------------
// swiglu_mlp_primitive.h:57-191.  Inputs [input, w_gate, w_up, w_down, biases...], dense
// weights of the activation dtype as in the reference.
class SwiGLUMLPPrimitive : public B200Primitive {
 public:
  SwiGLUMLPPrimitive(mx::Stream stream, int M, int hidden_size, int intermediate_size, bool has_bias = false);
  ~SwiGLUMLPPrimitive() override;
  void eval_gpu(const std::vector<mx::array>& inputs, std::vector<mx::array>& outputs) override;
  std::vector<mx::Shape> output_shapes(const std::vector<mx::array>& inputs) override { return {inputs[0].shape()}; }
  const char* name() const override { return "swiglu_mlp_fused"; }
  bool is_equivalent(const mx::Primitive& other) const override;
  int M() const { return M_; }
  int hidden_size() const { return hidden_size_; }
  int intermediate_size() const { return intermediate_size_; }
  bool has_bias() const { return has_bias_; }

 private:
  int M_, hidden_size_, intermediate_size_;
  bool has_bias_;
};
mx::array swiglu_mlp(const mx::array& input, const mx::array& w_gate, const mx::array& w_up,
                     const mx::array& w_down, const mx::array* bias_gate = nullptr,
                     const mx::array* bias_up = nullptr, const mx::array* bias_down = nullptr,
                     mx::StreamOrDevice s = {});
mx::array swish(const mx::array& x, mx::StreamOrDevice s = {});
mx::array swiglu(const mx::array& gate, const mx::array& up, mx::StreamOrDevice s = {});
// extension: the block with PACKED weights (what plan/MetalKernelsPlan.md:109-117 intends)
// and an optional RMSNorm prologue: y = down(SiLU(gate(n)) * up(n)), n = rmsnorm(x).
mx::array swiglu_mlp_quantized(const mx::array& input, const mx::array& w_gate, const mx::array& w_up,
                               const mx::array& w_down, int intermediate_size, QuantType quant_type,
                               const mx::array* norm_weight = nullptr, float eps = 1e-5f,
                               mx::StreamOrDevice s = {});

// ---- RoPE ---------------------------------------------------------------------------------------
// rope_apply_primitive.h:59-230.  Inputs [input, cos_table, sin_table, positions].
class RoPEApplyPrimitive : public B200Primitive {
 public:
  RoPEApplyPrimitive(mx::Stream stream, int batch_size, int seq_len, int num_heads, int head_dim,
                     RoPEScalingMode scaling_mode = RoPEScalingMode::BASE, float scale_factor = 1.0f,
                     int position_offset = 0, bool inplace = false);
  ~RoPEApplyPrimitive() override;
  void eval_gpu(const std::vector<mx::array>& inputs, std::vector<mx::array>& outputs) override;
  std::vector<mx::Shape> output_shapes(const std::vector<mx::array>& inputs) override { return {inputs[0].shape()}; }
  const char* name() const override { return inplace_ ? "rope_apply_inplace" : "rope_apply"; }
  bool is_equivalent(const mx::Primitive& other) const override;
  int batch_size() const { return batch_size_; }
  int seq_len() const { return seq_len_; }
  int num_heads() const { return num_heads_; }
  int head_dim() const { return head_dim_; }
  RoPEScalingMode scaling_mode() const { return scaling_mode_; }
  float scale_factor() const { return scale_factor_; }
  int position_offset() const { return position_offset_; }
  bool inplace() const { return inplace_; }

 private:
  int batch_size_, seq_len_, num_heads_, head_dim_;
  RoPEScalingMode scaling_mode_;
  float scale_factor_;
  int position_offset_;
  bool inplace_;
};
mx::array rope_apply(const mx::array& input, const mx::array& cos_table, const mx::array& sin_table,
                     const mx::array& positions, RoPEScalingMode scaling_mode = RoPEScalingMode::BASE,
                     float scale_factor = 1.0f, int position_offset = 0, bool inplace = false,
                     mx::StreamOrDevice s = {});
std::pair<mx::array, mx::array> compute_rope_tables(int max_seq_len, int head_dim, float base = 10000.0f,
                                                    RoPEScalingMode scaling_mode = RoPEScalingMode::BASE,
                                                    float scale_factor = 1.0f, int orig_context = 2048);
float compute_ntk_scaled_base(float base, float scale, int head_dim, int orig_context);
const char* rope_scaling_mode_name(RoPEScalingMode mode);

}  // namespace kernels
}  // namespace mlxr
