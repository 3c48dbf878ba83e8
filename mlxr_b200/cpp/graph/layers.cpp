// Implementation of the graph layers over the kernel primitives and the C ABI.
#include "layers.h"

#include <cstring>
#include <sstream>
#include <stdexcept>

#include <mlx/ops.h>

#include "../../../include/mlxr_b200.h"

namespace mlxr {
namespace graph {

namespace mx = mlx::core;

namespace {

int act_dtype(mx::Dtype d, const char* who) {
  if (d == mx::float16) return MLXR_F16;
  if (d == mx::bfloat16) return MLXR_BF16;
  if (d == mx::float32) return MLXR_F32;
  throw std::invalid_argument(std::string(who) + ": activations must be float16, bfloat16 or float32");
}
void check(int status) {
  if (status == MLXR_OK) return;
  const std::string msg = mlxr_last_error();
  if (status == MLXR_ERR_INVALID_ARGUMENT) throw std::invalid_argument(msg);
  throw std::runtime_error(msg);
}
void* gpu_stream() { return mx::native_stream(mx::default_stream(mx::Device(mx::Device::gpu))); }
// rows of a tensor whose last dimension is `last`
int rows_of(const Tensor& x, int last, const char* who) {
  if (x.ndim() < 1 || x.shape().back() != last)
    throw std::invalid_argument(std::string(who) + ": the input's last dimension must be " + std::to_string(last));
  return (int)(x.size() / (size_t)last);
}

}  // namespace

// ---- Tensor --------------------------------------------------------------------------------
Tensor::Tensor() : array_(mx::Shape{0}, mx::float32), empty_(true) {}
Tensor::Tensor(const mx::array& array) : array_(array) {}
Tensor::Tensor(const std::vector<int>& shape, mx::Dtype dtype) : array_(to_shape(shape), dtype) {}
mx::array& Tensor::array() { return array_; }
const mx::array& Tensor::array() const { return array_; }
std::vector<int> Tensor::shape() const { return from_shape(array_.shape()); }
mx::Dtype Tensor::dtype() const { return array_.dtype(); }
int Tensor::ndim() const { return (int)array_.ndim(); }
size_t Tensor::size() const { return array_.size(); }
bool Tensor::empty() const { return empty_ || array_.size() == 0; }
Tensor Tensor::reshape(const std::vector<int>& new_shape) const { return Tensor(mx::reshape(array_, to_shape(new_shape))); }
void Tensor::eval() { array_.eval(); }
std::string Tensor::to_string() const {
  std::ostringstream os;
  os << "Tensor(shape=[";
  const auto s = shape();
  for (size_t i = 0; i < s.size(); i++) os << (i ? ", " : "") << s[i];
  os << "], dtype=" << mx::dtype_name(dtype()) << ")";
  return os.str();
}
Tensor zeros(const std::vector<int>& shape, mx::Dtype dtype) { return Tensor(mx::zeros(to_shape(shape), dtype)); }
Tensor ones(const std::vector<int>& shape, mx::Dtype dtype) { return Tensor(mx::ones(to_shape(shape), dtype)); }
Tensor from_data(const void* data, const std::vector<int>& shape, mx::Dtype dtype) {
  Tensor t(shape, dtype);
  mx::array& a = t.array();
  a.eval();
  if (a.nbytes()) std::memcpy(a.data<void>(), data, a.nbytes());
  return t;
}

// ---- RMSNorm (layers.cpp:26-59) --------------------------------------------------------------
RMSNorm::RMSNorm(int dim, float eps) : dim_(dim), eps_(eps), weight_(ones({dim})) {}
Tensor RMSNorm::forward(const Tensor& x) {
  rows_of(x, dim_, "RMSNorm");
  mx::array w = weight_.array();
  if (w.dtype() != x.dtype()) w = mx::astype(w, x.dtype());
  return Tensor(kernels::rmsnorm_fused(x.array(), w, eps_));
}
Tensor& RMSNorm::weight() { return weight_; }
const Tensor& RMSNorm::weight() const { return weight_; }

// ---- Linear (layers.cpp:65-107) --------------------------------------------------------------
Linear::Linear(int in_features, int out_features, bool bias)
    : in_features_(in_features), out_features_(out_features), has_bias_(bias),
      weight_(zeros({out_features, in_features})), bias_(bias ? zeros({out_features}) : Tensor()) {}
void Linear::set_quantized(const Tensor& packed, kernels::QuantType quant_type) {
  const size_t need = kernels::compute_quantized_weight_size(out_features_, in_features_, quant_type);
  if (packed.dtype() != mx::uint8 || packed.size() != need)
    throw std::invalid_argument("Linear::set_quantized: packed weights must be " + std::to_string(need) + " uint8 bytes");
  packed_ = packed;
  quant_type_ = quant_type;
  quantized_ = true;
}
Tensor Linear::forward(const Tensor& x) {
  const int M = rows_of(x, in_features_, "Linear");
  std::vector<int> out_shape = x.shape();
  out_shape.back() = out_features_;
  const mx::array* b = nullptr;
  mx::array bias_arr = weight_.array();
  if (has_bias_) {
    bias_arr = bias_.array();
    if (bias_arr.dtype() != x.dtype()) bias_arr = mx::astype(bias_arr, x.dtype());
    b = &bias_arr;
  }
  if (quantized_) {
    mx::array x2 = mx::reshape(x.array(), {M, in_features_});
    mx::array y = kernels::q_gemm_dequant(x2, packed_.array(), M, out_features_, in_features_, quant_type_,
                                          kernels::QGemmDequantPrimitive::get_default_group_size(quant_type_), b);
    return Tensor(mx::reshape(y, to_shape(out_shape)));
  }
  mx::array xa = x.array(), w = weight_.array();
  if (w.dtype() != x.dtype()) w = mx::astype(w, x.dtype());
  xa.eval();
  w.eval();
  if (b) bias_arr.eval();
  mx::array y(to_shape(out_shape), x.dtype());
  check(mlxr_linear_dense(xa.data<void>(), w.data<void>(), b ? bias_arr.data<void>() : nullptr, y.data<void>(), M,
                          out_features_, in_features_, act_dtype(x.dtype(), "Linear"), gpu_stream()));
  return Tensor(y);
}
Tensor& Linear::weight() { return weight_; }
const Tensor& Linear::weight() const { return weight_; }
Tensor* Linear::bias() { return has_bias_ ? &bias_ : nullptr; }
const Tensor* Linear::bias() const { return has_bias_ ? &bias_ : nullptr; }

// ---- RotaryEmbedding (layers.cpp:113-225) ----------------------------------------------------
RotaryEmbedding::RotaryEmbedding(int dim, int max_seq_len, float base) : dim_(dim), max_seq_len_(max_seq_len), base_(base) {
  if (dim % 2 != 0) throw std::invalid_argument("RotaryEmbedding dimension must be even");
  compute_freqs();
}
void RotaryEmbedding::compute_freqs() {
  cos_cached_ = Tensor({max_seq_len_, dim_ / 2}, mx::float32);
  sin_cached_ = Tensor({max_seq_len_, dim_ / 2}, mx::float32);
  cos_cached_.eval();
  sin_cached_.eval();
  check(mlxr_rope_tables_f32_host(cos_cached_.array().data<float>(), sin_cached_.array().data<float>(), max_seq_len_, dim_, base_));
}
std::pair<Tensor, Tensor> RotaryEmbedding::forward(const Tensor& q, const Tensor& k, int offset) {
  if (q.ndim() != 4 || k.ndim() != 4)
    throw std::invalid_argument("RotaryEmbedding expects 4D tensors [batch, seq_len, num_heads, head_dim]");
  if (q.shape()[3] != dim_ || k.shape()[3] != dim_) throw std::invalid_argument("head_dim must match RotaryEmbedding dim");
  auto rotate = [&](const Tensor& t) {
    const auto s = t.shape();
    mx::array in = t.array();
    in.eval();
    mx::array out(in.shape(), in.dtype());
    check(mlxr_rope_apply_split_half(in.data<void>(), cos_cached_.array().data<float>(), sin_cached_.array().data<float>(),
                                     out.data<void>(), s[0], s[1], s[2], s[3], max_seq_len_, offset,
                                     act_dtype(in.dtype(), "RotaryEmbedding"), gpu_stream()));
    return Tensor(out);
  };
  return {rotate(q), rotate(k)};
}

// ---- MLP (layers.cpp:386-426) ----------------------------------------------------------------
MLP::MLP(int hidden_size, int intermediate_size)
    : hidden_size_(hidden_size), intermediate_size_(intermediate_size),
      gate_proj_(hidden_size, intermediate_size, false), up_proj_(hidden_size, intermediate_size, false),
      down_proj_(intermediate_size, hidden_size, false) {}
Tensor MLP::forward(const Tensor& x) { return run(x, nullptr); }
Tensor MLP::forward(const Tensor& x, const RMSNorm& norm) { return run(x, &norm); }
Tensor MLP::run(const Tensor& x, const RMSNorm* norm) {
  const int M = rows_of(x, hidden_size_, "MLP");
  const bool fused = gate_proj_.quantized() && up_proj_.quantized() && down_proj_.quantized() &&
                     gate_proj_.quant_type() == up_proj_.quant_type() && gate_proj_.quant_type() == down_proj_.quant_type();
  if (fused) {
    // one call: [RMSNorm ->] gate/up -> SiLU(gate) * up -> down on packed weights
    mx::array x2 = mx::reshape(x.array(), {M, hidden_size_});
    mx::array nw = x2;
    const mx::array* nwp = nullptr;
    if (norm) {
      nw = norm->weight().array();
      if (nw.dtype() != x.dtype()) nw = mx::astype(nw, x.dtype());
      nwp = &nw;
    }
    mx::array y = kernels::swiglu_mlp_quantized(x2, gate_proj_.packed_weight().array(), up_proj_.packed_weight().array(),
                                                down_proj_.packed_weight().array(), intermediate_size_, gate_proj_.quant_type(),
                                                nwp, norm ? norm->eps() : 1e-5f);
    return Tensor(mx::reshape(y, to_shape(x.shape())));
  }
  // gate = gate_proj(n); up = up_proj(n); down_proj(SiLU(gate) * up)   (layers.cpp:400-420)
  Tensor n = x;
  if (norm) n = const_cast<RMSNorm*>(norm)->forward(x);
  Tensor gate = gate_proj_.forward(n);
  Tensor up = up_proj_.forward(n);
  Tensor h(kernels::swiglu(gate.array(), up.array()));
  return down_proj_.forward(h);
}
Linear& MLP::gate_proj() { return gate_proj_; }
Linear& MLP::up_proj() { return up_proj_; }
Linear& MLP::down_proj() { return down_proj_; }

}  // namespace graph
}  // namespace mlxr
