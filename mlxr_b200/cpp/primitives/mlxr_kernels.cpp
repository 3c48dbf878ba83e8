// Implementation of MLXR's kernel primitives over the C ABI of libmlxr_b200.so.
// Shape checks, messages and exception types follow the reference's public functions
// (cited per function); the arithmetic is entirely behind mlxr_* calls.
#include "mlxr_kernels.h"

#include <cmath>
#include <stdexcept>
#include <string>

#include <mlx/ops.h>

#include "../../../include/mlxr_b200.h"

namespace mlxr {
namespace kernels {

namespace {

int act_dtype(const mx::array& a, const char* who) {
  if (a.dtype() == mx::float16) return MLXR_F16;
  if (a.dtype() == mx::bfloat16) return MLXR_BF16;
  if (a.dtype() == mx::float32) return MLXR_F32;
  throw std::invalid_argument(std::string(who) + ": activations must be float16, bfloat16 or float32");
}

// std::invalid_argument for MLXR_ERR_INVALID_ARGUMENT, std::runtime_error otherwise
[[noreturn]] void raise(int status) {
  const std::string msg = mlxr_last_error();
  if (status == MLXR_ERR_INVALID_ARGUMENT) throw std::invalid_argument(msg);
  throw std::runtime_error(msg);
}
inline void check(int status) {
  if (status != MLXR_OK) raise(status);
}

void require_gpu(const mx::Stream& s, const char* who) {
  if (s.device.type != mx::Device::gpu)
    throw std::runtime_error(std::string(who) + ": this build has no CPU path (the stream's device must be gpu)");
}

void* cuda_stream(mx::Primitive& p) { return mx::native_stream(p.stream()); }

}  // namespace

// ---- shared boilerplate ------------------------------------------------------------------------
void B200Primitive::eval_cpu(const std::vector<mx::array>&, std::vector<mx::array>&) {
  throw std::runtime_error(std::string(name()) + ": no CPU evaluation in the B200 build");
}
std::pair<std::vector<mx::array>, std::vector<int>> B200Primitive::vmap(const std::vector<mx::array>&,
                                                                         const std::vector<int>&) {
  throw std::runtime_error(std::string("vmap not yet implemented for ") + name());
}
std::vector<mx::array> B200Primitive::jvp(const std::vector<mx::array>&, const std::vector<mx::array>&,
                                          const std::vector<int>&) {
  throw std::runtime_error(std::string("jvp not yet implemented for ") + name());
}
std::vector<mx::array> B200Primitive::vjp(const std::vector<mx::array>&, const std::vector<mx::array>&,
                                          const std::vector<int>&, const std::vector<mx::array>&) {
  throw std::runtime_error(std::string("vjp not yet implemented for ") + name());
}

// ---- q_gemm_dequant ------------------------------------------------------------------------------
QGemmDequantPrimitive::QGemmDequantPrimitive(mx::Stream stream, int M, int N, int K, QuantType quant_type,
                                             int group_size, bool has_bias)
    : B200Primitive(stream), M_(M), N_(N), K_(K), quant_type_(quant_type), group_size_(group_size),
      has_bias_(has_bias) {}
QGemmDequantPrimitive::~QGemmDequantPrimitive() = default;

// get_bytes_per_weight, q_gemm_dequant_primitive.mm:63-78 (throws for formats without code)
float QGemmDequantPrimitive::get_bytes_per_weight(QuantType type) {
  const float b = mlxr_bytes_per_weight(static_cast<int>(type));
  if (b < 0) throw std::runtime_error("Unsupported quantization type");
  return b;
}
int QGemmDequantPrimitive::get_default_group_size(QuantType type) {
  return mlxr_default_group_size(static_cast<int>(type));
}
const char* quant_type_name(QuantType type) { return mlxr_quant_type_name(static_cast<int>(type)); }

// compute_quantized_weight_size, q_gemm_dequant_primitive.mm:116-135
size_t compute_quantized_weight_size(int N, int K, QuantType quant_type) {
  if (mlxr_bytes_per_weight(static_cast<int>(quant_type)) < 0)
    throw std::runtime_error("Unsupported quantization type");
  return mlxr_quantized_weight_size(N, K, static_cast<int>(quant_type));
}

bool QGemmDequantPrimitive::is_equivalent(const mx::Primitive& other) const {
  const auto* o = dynamic_cast<const QGemmDequantPrimitive*>(&other);
  return o && M_ == o->M_ && N_ == o->N_ && K_ == o->K_ && quant_type_ == o->quant_type_ &&
         group_size_ == o->group_size_ && has_bias_ == o->has_bias_;
}

// eval_gpu, q_gemm_dequant_primitive.mm:367-450: inputs [input, weights, bias?]; the output
// is a fresh [M, N] array of the input's dtype (the reference: float16).
void QGemmDequantPrimitive::eval_gpu(const std::vector<mx::array>& inputs, std::vector<mx::array>& outputs) {
  if (inputs.size() < 2 || (has_bias_ && inputs.size() < 3))
    throw std::runtime_error("QGemmDequant requires input, weights, and optional bias");
  const mx::array& input = inputs[0];
  const mx::array& weights = inputs[1];
  const mx::array* bias = has_bias_ ? &inputs[2] : nullptr;
  const size_t need = mlxr_quantized_weight_size(N_, K_, static_cast<int>(quant_type_));
  if (need && weights.nbytes() < need)
    throw std::runtime_error("QGemmDequant: weights buffer is smaller than compute_quantized_weight_size(N, K, type)");
  if (bias && bias->dtype() != input.dtype()) throw std::runtime_error("QGemmDequant: bias dtype must match input");
  mx::array out(mx::Shape{M_, N_}, input.dtype());
  check(mlxr_q_gemm_dequant(input.data<void>(), weights.data<void>(), bias ? bias->data<void>() : nullptr,
                            out.data<void>(), M_, N_, K_, static_cast<int>(quant_type_), group_size_,
                            act_dtype(input, "QGemmDequant"), cuda_stream(*this)));
  outputs[0] = out;
}

// q_gemm_dequant(), q_gemm_dequant_primitive.mm:478-522: eager, validates shapes first
mx::array q_gemm_dequant(const mx::array& input, const mx::array& weights, int M, int N, int K,
                         QuantType quant_type, int group_size, const mx::array* bias, mx::StreamOrDevice s) {
  if (input.shape().size() != 2 || input.shape(0) != M || input.shape(1) != K)
    throw std::runtime_error("Input shape must be [M, K]");
  if (bias != nullptr && (bias->shape().size() != 1 || bias->shape(0) != N))
    throw std::runtime_error("Bias shape must be [N]");
  auto stream = mx::to_stream(s);
  require_gpu(stream, "q_gemm_dequant");
  auto prim = std::make_shared<QGemmDequantPrimitive>(stream, M, N, K, quant_type, group_size, bias != nullptr);
  std::vector<mx::array> in = {input, weights};
  if (bias) in.push_back(*bias);
  for (auto& a : in) a.eval();
  std::vector<mx::array> out = {mx::array::wrap(nullptr, mx::Shape{M, N}, input.dtype())};
  prim->eval_gpu(in, out);
  return out[0];
}

mx::array dequantize(const mx::array& weights, int N, int K, QuantType quant_type, mx::Dtype out_dtype,
                     mx::StreamOrDevice s) {
  if (out_dtype != mx::float16 && out_dtype != mx::float32)
    throw std::invalid_argument("dequantize: out_dtype must be float16 or float32");
  auto stream = mx::to_stream(s);
  require_gpu(stream, "dequantize");
  mx::array w = weights;
  w.eval();
  mx::array out(mx::Shape{N, K}, out_dtype);
  check(mlxr_dequantize(w.data<void>(), out.data<void>(), N, K, static_cast<int>(quant_type),
                        out_dtype == mx::float16 ? MLXR_F16 : MLXR_F32, 0, mx::native_stream(stream)));
  return out;
}

// ---- RMSNorm -------------------------------------------------------------------------------------
RMSNormPrimitive::RMSNormPrimitive(mx::Stream stream, float eps) : B200Primitive(stream), eps_(eps) {}
RMSNormPrimitive::~RMSNormPrimitive() = default;
bool RMSNormPrimitive::is_equivalent(const mx::Primitive& other) const {
  const auto* o = dynamic_cast<const RMSNormPrimitive*>(&other);
  return o && eps_ == o->eps_;
}
// eval_gpu, rmsnorm_primitive.mm:139-231: allocate the output, one row per thread group
void RMSNormPrimitive::eval_gpu(const std::vector<mx::array>& inputs, std::vector<mx::array>& outputs) {
  if (inputs.size() != 2 || outputs.size() != 1) throw std::invalid_argument("RMSNorm takes [input, weight]");
  const mx::array& input = inputs[0];
  const mx::array& weight = inputs[1];
  mx::array& out = outputs[0];
  out.set_data(mx::allocator::malloc(out.nbytes()));
  const int hidden = input.shape(-1);
  const int rows = hidden ? (int)(input.size() / hidden) : 0;
  check(mlxr_rmsnorm(input.data<void>(), weight.data<void>(), nullptr, out.data<void>(), rows, hidden, eps_,
                     act_dtype(input, "RMSNorm"), cuda_stream(*this)));
}
// rmsnorm_fused(), rmsnorm_primitive.mm:302-359: lazy node; invalid_argument on bad shapes
mx::array rmsnorm_fused(const mx::array& input, const mx::array& weight, float eps, mx::StreamOrDevice s) {
  if (input.ndim() < 1) throw std::invalid_argument("RMSNorm input must have at least 1 dimension");
  if (weight.ndim() != 1) throw std::invalid_argument("RMSNorm weight must be 1-dimensional");
  if (weight.size() != (size_t)input.shape().back())
    throw std::invalid_argument("RMSNorm weight size must match input's last dimension");
  if (weight.dtype() != input.dtype()) throw std::invalid_argument("RMSNorm weight dtype must match input");
  auto stream = mx::to_stream(s);
  require_gpu(stream, "rmsnorm_fused");
  (void)act_dtype(input, "RMSNorm");
  auto prim = std::make_shared<RMSNormPrimitive>(stream, eps);
  // arrays of this build are always row-contiguous, so the reference's contiguity copies
  // (rmsnorm_primitive.mm:332-346) have nothing to do
  return mx::array::make_arrays({input.shape()}, {input.dtype()}, prim, {input, weight})[0];
}

// ---- SwiGLU --------------------------------------------------------------------------------------
SwiGLUMLPPrimitive::SwiGLUMLPPrimitive(mx::Stream stream, int M, int hidden_size, int intermediate_size, bool has_bias)
    : B200Primitive(stream), M_(M), hidden_size_(hidden_size), intermediate_size_(intermediate_size),
      has_bias_(has_bias) {}
SwiGLUMLPPrimitive::~SwiGLUMLPPrimitive() = default;
bool SwiGLUMLPPrimitive::is_equivalent(const mx::Primitive& other) const {
  const auto* o = dynamic_cast<const SwiGLUMLPPrimitive*>(&other);
  return o && M_ == o->M_ && hidden_size_ == o->hidden_size_ && intermediate_size_ == o->intermediate_size_ &&
         has_bias_ == o->has_bias_;
}
// The composition of eval_cpu, swiglu_mlp_primitive.mm:47-82, on the device (the reference's
// own eval_gpu cannot run: its host/shader argument structs disagree).  Biases are taken in
// the order they were pushed: gate, up, down.
void SwiGLUMLPPrimitive::eval_gpu(const std::vector<mx::array>& inputs, std::vector<mx::array>& outputs) {
  if (inputs.size() < 4) throw std::invalid_argument("SwiGLUMLP takes [input, w_gate, w_up, w_down, biases...]");
  const mx::array& x = inputs[0];
  const void* bg = (has_bias_ && inputs.size() > 4) ? inputs[4].data<void>() : nullptr;
  const void* bu = (has_bias_ && inputs.size() > 5) ? inputs[5].data<void>() : nullptr;
  const void* bd = (has_bias_ && inputs.size() > 6) ? inputs[6].data<void>() : nullptr;
  for (int i = 1; i < 4; i++)
    if (inputs[i].dtype() != x.dtype()) throw std::invalid_argument("SwiGLUMLP: weights must have the input's dtype");
  mx::array out(mx::Shape{M_, hidden_size_}, x.dtype());
  check(mlxr_mlp_block_dense(x.data<void>(), inputs[1].data<void>(), inputs[2].data<void>(), inputs[3].data<void>(),
                             bg, bu, bd, out.data<void>(), M_, hidden_size_, intermediate_size_,
                             act_dtype(x, "SwiGLUMLP"), cuda_stream(*this)));
  outputs[0] = out;
}
// swiglu_mlp(), swiglu_mlp_primitive.mm:235-304
mx::array swiglu_mlp(const mx::array& input, const mx::array& w_gate, const mx::array& w_up, const mx::array& w_down,
                     const mx::array* bias_gate, const mx::array* bias_up, const mx::array* bias_down,
                     mx::StreamOrDevice s) {
  if (input.ndim() != 2) throw std::invalid_argument("Input must be 2D [M, hidden_size]");
  const int M = input.shape(0), hidden = input.shape(1);
  if (w_gate.ndim() != 2 || w_gate.shape(1) != hidden) throw std::invalid_argument("w_gate shape mismatch");
  const int inter = w_gate.shape(0);
  if (w_up.ndim() != 2 || w_up.shape(0) != inter || w_up.shape(1) != hidden) throw std::invalid_argument("w_up shape mismatch");
  if (w_down.ndim() != 2 || w_down.shape(0) != hidden || w_down.shape(1) != inter)
    throw std::invalid_argument("w_down shape mismatch");
  std::vector<mx::array> in = {input, w_gate, w_up, w_down};
  bool has_bias = false;
  for (const mx::array* b : {bias_gate, bias_up, bias_down})
    if (b) { in.push_back(*b); has_bias = true; }
  auto stream = mx::to_stream(s);
  require_gpu(stream, "swiglu_mlp");
  for (auto& a : in) a.eval();
  auto prim = std::make_shared<SwiGLUMLPPrimitive>(stream, M, hidden, inter, has_bias);
  std::vector<mx::array> out = {mx::array::wrap(nullptr, input.shape(), input.dtype())};
  prim->eval_gpu(in, out);
  return out[0];
}
// swish() / swiglu(), swiglu_mlp_primitive.mm:306-318
mx::array swish(const mx::array& x, mx::StreamOrDevice s) {
  auto stream = mx::to_stream(s);
  require_gpu(stream, "swish");
  mx::array in = x;
  in.eval();
  mx::array out(x.shape(), x.dtype());
  check(mlxr_swiglu(in.data<void>(), nullptr, out.data<void>(), x.size(), act_dtype(x, "swish"), mx::native_stream(stream)));
  return out;
}
mx::array swiglu(const mx::array& gate, const mx::array& up, mx::StreamOrDevice s) {
  if (gate.shape() != up.shape() || gate.dtype() != up.dtype()) throw std::invalid_argument("swiglu: gate and up must match");
  auto stream = mx::to_stream(s);
  require_gpu(stream, "swiglu");
  mx::array g = gate, u = up;
  g.eval();
  u.eval();
  mx::array out(gate.shape(), gate.dtype());
  check(mlxr_swiglu(g.data<void>(), u.data<void>(), out.data<void>(), gate.size(), act_dtype(gate, "swiglu"),
                    mx::native_stream(stream)));
  return out;
}
mx::array swiglu_mlp_quantized(const mx::array& input, const mx::array& w_gate, const mx::array& w_up,
                               const mx::array& w_down, int intermediate_size, QuantType quant_type,
                               const mx::array* norm_weight, float eps, mx::StreamOrDevice s) {
  if (input.ndim() != 2) throw std::invalid_argument("Input must be 2D [M, hidden_size]");
  const int M = input.shape(0), hidden = input.shape(1), qt = static_cast<int>(quant_type);
  const size_t gu = mlxr_quantized_weight_size(intermediate_size, hidden, qt), dn = mlxr_quantized_weight_size(hidden, intermediate_size, qt);
  if (gu == 0) throw std::runtime_error("Unsupported quantization type");
  if (w_gate.nbytes() != gu) throw std::invalid_argument("w_gate shape mismatch");
  if (w_up.nbytes() != gu) throw std::invalid_argument("w_up shape mismatch");
  if (w_down.nbytes() != dn) throw std::invalid_argument("w_down shape mismatch");
  if (norm_weight && (norm_weight->ndim() != 1 || norm_weight->shape(0) != hidden || norm_weight->dtype() != input.dtype()))
    throw std::invalid_argument("RMSNorm weight size must match input's last dimension");
  auto stream = mx::to_stream(s);
  require_gpu(stream, "swiglu_mlp_quantized");
  mx::array x = input, g = w_gate, u = w_up, d = w_down;
  x.eval(); g.eval(); u.eval(); d.eval();
  const void* nw = nullptr;
  mx::array nwa = input;
  if (norm_weight) { nwa = *norm_weight; nwa.eval(); nw = nwa.data<void>(); }
  mx::array out(input.shape(), input.dtype());
  check(mlxr_mlp_block(x.data<void>(), nw, g.data<void>(), u.data<void>(), d.data<void>(), out.data<void>(), M, hidden,
                       intermediate_size, qt, eps, act_dtype(input, "swiglu_mlp_quantized"), mx::native_stream(stream)));
  return out;
}

// ---- RoPE ----------------------------------------------------------------------------------------
const char* rope_scaling_mode_name(RoPEScalingMode mode) { return mlxr_rope_scaling_mode_name(static_cast<int>(mode)); }
float compute_ntk_scaled_base(float base, float scale, int head_dim, int orig_context) {
  return mlxr_ntk_scaled_base(base, scale, head_dim, orig_context);
}
// compute_rope_tables, rope_apply_primitive.mm:49-106: host computation, float16 tables
std::pair<mx::array, mx::array> compute_rope_tables(int max_seq_len, int head_dim, float base, RoPEScalingMode scaling_mode,
                                                    float scale_factor, int orig_context) {
  if (head_dim % 2 != 0) throw std::runtime_error("head_dim must be even for RoPE");
  mx::array c(mx::Shape{max_seq_len, head_dim / 2}, mx::float16), sn(mx::Shape{max_seq_len, head_dim / 2}, mx::float16);
  check(mlxr_rope_tables_host(c.data<uint16_t>(), sn.data<uint16_t>(), max_seq_len, head_dim, base,
                              static_cast<int>(scaling_mode), scale_factor, orig_context));
  return {c, sn};
}
RoPEApplyPrimitive::RoPEApplyPrimitive(mx::Stream stream, int batch_size, int seq_len, int num_heads, int head_dim,
                                       RoPEScalingMode scaling_mode, float scale_factor, int position_offset, bool inplace)
    : B200Primitive(stream), batch_size_(batch_size), seq_len_(seq_len), num_heads_(num_heads), head_dim_(head_dim),
      scaling_mode_(scaling_mode), scale_factor_(scale_factor), position_offset_(position_offset), inplace_(inplace) {
  if (head_dim % 2 != 0) throw std::runtime_error("head_dim must be even for RoPE");
}
RoPEApplyPrimitive::~RoPEApplyPrimitive() = default;
bool RoPEApplyPrimitive::is_equivalent(const mx::Primitive& other) const {
  const auto* o = dynamic_cast<const RoPEApplyPrimitive*>(&other);
  return o && batch_size_ == o->batch_size_ && seq_len_ == o->seq_len_ && num_heads_ == o->num_heads_ &&
         head_dim_ == o->head_dim_ && scaling_mode_ == o->scaling_mode_ && scale_factor_ == o->scale_factor_ &&
         position_offset_ == o->position_offset_ && inplace_ == o->inplace_;
}
// eval_gpu, rope_apply_primitive.mm:272-370: inputs [input, cos, sin, positions]; in place
// aliases the input (:288-292).  Positions outside the table are reported, not read.
void RoPEApplyPrimitive::eval_gpu(const std::vector<mx::array>& inputs, std::vector<mx::array>& outputs) {
  if (inputs.size() != 4) throw std::runtime_error("RoPEApply requires 4 inputs: input, cos_table, sin_table, positions");
  const mx::array& input = inputs[0];
  if (inputs[1].dtype() != mx::float16 || inputs[2].dtype() != mx::float16)
    throw std::runtime_error("RoPEApply: cos/sin tables must be float16 (compute_rope_tables)");
  if (inputs[3].dtype() != mx::int32) throw std::runtime_error("RoPEApply: positions must be int32");
  mx::array out = inplace_ ? input : mx::array(input.shape(), input.dtype());
  check(mlxr_rope_apply(input.data<void>(), inputs[1].data<uint16_t>(), inputs[2].data<uint16_t>(), inputs[3].data<int32_t>(),
                        out.data<void>(), batch_size_, seq_len_, num_heads_, head_dim_, inputs[1].shape(0),
                        static_cast<int>(scaling_mode_), scale_factor_, position_offset_, act_dtype(input, "RoPEApply"),
                        /*check=*/1, cuda_stream(*this)));
  outputs[0] = out;
}
// rope_apply(), rope_apply_primitive.mm:399-475
mx::array rope_apply(const mx::array& input, const mx::array& cos_table, const mx::array& sin_table, const mx::array& positions,
                     RoPEScalingMode scaling_mode, float scale_factor, int position_offset, bool inplace, mx::StreamOrDevice s) {
  if (input.ndim() != 4 && input.ndim() != 3)
    throw std::runtime_error("Input must be 3D [tokens, num_heads, head_dim] or 4D [batch, seq_len, num_heads, head_dim]");
  int batch_size, seq_len, num_heads, head_dim;
  if (input.ndim() == 4) {
    batch_size = input.shape(0); seq_len = input.shape(1); num_heads = input.shape(2); head_dim = input.shape(3);
  } else {
    batch_size = input.shape(0); seq_len = 1; num_heads = input.shape(1); head_dim = input.shape(2);
  }
  if (head_dim % 2 != 0) throw std::runtime_error("head_dim must be even for RoPE");
  const int num_pairs = head_dim / 2;
  if (cos_table.ndim() != 2 || cos_table.shape(1) != num_pairs) throw std::runtime_error("cos_table must have shape [max_seq_len, head_dim/2]");
  if (sin_table.ndim() != 2 || sin_table.shape(1) != num_pairs) throw std::runtime_error("sin_table must have shape [max_seq_len, head_dim/2]");
  if (seq_len == 1) {
    if (positions.ndim() != 1 || positions.shape(0) != batch_size)
      throw std::runtime_error("For flattened input, positions must have shape [tokens]");
  } else if (positions.ndim() != 2 || positions.shape(0) != batch_size || positions.shape(1) != seq_len) {
    throw std::runtime_error("positions must have shape [batch, seq_len]");
  }
  auto stream = mx::to_stream(s);
  require_gpu(stream, "rope_apply");
  auto prim = std::make_shared<RoPEApplyPrimitive>(stream, batch_size, seq_len, num_heads, head_dim, scaling_mode, scale_factor,
                                                   position_offset, inplace);
  std::vector<mx::array> in = {input, cos_table, sin_table, positions};
  for (auto& a : in) a.eval();
  std::vector<mx::array> out = {inplace ? input : mx::array::wrap(nullptr, input.shape(), input.dtype())};
  prim->eval_gpu(in, out);
  return out[0];
}

}  // namespace kernels
}  // namespace mlxr
