// MLXR's graph layers on the quantized-linear path (namespace mlxr::graph), B200 build.
//
// Same class names, constructors, forward() signatures and accessors as
// core/graph/layers.h:26-253 for RMSNorm, Linear, RotaryEmbedding and MLP, so that model code
// written against that header compiles unchanged; forward() runs the kernels of
// libmlxr_b200.so instead of chains of MLX ops:
//   RMSNorm::forward           -> rmsnorm_fused            (layers.cpp:39-55)
//   Linear::forward            -> dense linear, or q_gemm_dequant once packed weights are set
//                                                          (layers.cpp:86-99)
//   RotaryEmbedding::forward   -> split-half RoPE kernel   (layers.cpp:157-225)
//   MLP::forward               -> the fused block when its three linears are quantized in one
//                                 format, else three linears and swiglu (layers.cpp:400-420)
// Additions the reference does not have are marked "extension": Linear::set_quantized (the
// quantized Linear the reference planned but skips at load, daemon/server/model_loader.cpp:
// 236-245) and MLP::forward's optional RMSNorm prologue.  Attention, TransformerBlock and the
// KV cache are outside this path.
#pragma once
#include <memory>
#include <utility>
#include <vector>

#include "../primitives/mlxr_kernels.h"
#include "tensor.h"

namespace mlxr {
namespace graph {

class RMSNorm {
 public:
  explicit RMSNorm(int dim, float eps = 1e-6f);
  Tensor forward(const Tensor& x);
  Tensor& weight();
  const Tensor& weight() const;
  float eps() const { return eps_; }   // extension

 private:
  int dim_;
  float eps_;
  Tensor weight_;
};

class Linear {
 public:
  Linear(int in_features, int out_features, bool bias = false);
  Tensor forward(const Tensor& x);
  Tensor& weight();
  const Tensor& weight() const;
  Tensor* bias();
  const Tensor* bias() const;
  // extension: replace the dense weight by packed blocks [out_features, in_features] of
  // `quant_type` (compute_quantized_weight_size bytes, uint8); forward() then runs q_gemm_dequant
  void set_quantized(const Tensor& packed, kernels::QuantType quant_type);
  bool quantized() const { return quantized_; }
  kernels::QuantType quant_type() const { return quant_type_; }
  const Tensor& packed_weight() const { return packed_; }
  int in_features() const { return in_features_; }
  int out_features() const { return out_features_; }

 private:
  int in_features_;
  int out_features_;
  bool has_bias_;
  Tensor weight_;
  Tensor bias_;
  bool quantized_ = false;
  kernels::QuantType quant_type_ = kernels::QuantType::Q4_0;
  Tensor packed_;
};

class RotaryEmbedding {
 public:
  RotaryEmbedding(int dim, int max_seq_len, float base = 10000.0f);
  std::pair<Tensor, Tensor> forward(const Tensor& q, const Tensor& k, int offset = 0);
  const Tensor& cos_table() const { return cos_cached_; }
  const Tensor& sin_table() const { return sin_cached_; }

 private:
  void compute_freqs();
  int dim_;
  int max_seq_len_;
  float base_;
  Tensor cos_cached_;
  Tensor sin_cached_;
};

class MLP {
 public:
  MLP(int hidden_size, int intermediate_size);
  Tensor forward(const Tensor& x);
  // extension: the block with its RMSNorm prologue fused in (TransformerBlock::forward applies
  // post_attention_layernorm right before the MLP, layers.cpp:449-452)
  Tensor forward(const Tensor& x, const RMSNorm& norm);
  Linear& gate_proj();
  Linear& up_proj();
  Linear& down_proj();

 private:
  Tensor run(const Tensor& x, const RMSNorm* norm);
  int hidden_size_;
  int intermediate_size_;
  Linear gate_proj_;
  Linear up_proj_;
  Linear down_proj_;
};

}  // namespace graph
}  // namespace mlxr
