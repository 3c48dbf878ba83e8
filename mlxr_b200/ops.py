"""Host-side mirror of MLXR's kernel free functions over torch CUDA tensors.

Names, argument order and error behaviour follow the reference's public functions
(core/kernels/primitives/*.h); every function ends in a call through the C ABI.  torch is
used for device memory and the current stream only.  A CPU tensor is an error, not a
fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np
import torch

from . import _capi
from ._capi import check, lib
from .types import QuantType, RoPEScalingMode

_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT,
                                        f"unsupported activation dtype {t.dtype}") from None


def _dev(t: Optional[torch.Tensor], name: str) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise _capi.MlxrError(_capi.ERR_CUDA, f"{name} must be a CUDA tensor: there is no CPU path")
    if not t.is_contiguous():
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, f"{name} must be contiguous")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# ---- helpers -------------------------------------------------------------------------------

def compute_quantized_weight_size(N: int, K: int, quant_type: QuantType) -> int:
    """compute_quantized_weight_size, q_gemm_dequant_primitive.mm:116-135 (raises for a
    format without code, as the reference does)."""
    n = lib.mlxr_quantized_weight_size(N, K, int(quant_type))
    if n == 0 and N > 0 and K > 0:
        raise _capi.MlxrError(_capi.ERR_UNSUPPORTED, "Unsupported quantization type")
    return n


def quant_type_name(quant_type: int) -> str:
    """quant_type_name, q_gemm_dequant_primitive.mm:94-114"""
    return lib.mlxr_quant_type_name(int(quant_type)).decode()


def compute_rope_tables(max_seq_len: int, head_dim: int, base: float = 10000.0,
                        scaling_mode: RoPEScalingMode = RoPEScalingMode.BASE,
                        scale_factor: float = 1.0, orig_context: int = 2048,
                        device: Optional[torch.device] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """compute_rope_tables, rope_apply_primitive.mm:49-106: (cos, sin), fp16
    [max_seq_len, head_dim/2].  Computed on the host like the reference, then moved to
    `device` when given."""
    pairs = max(head_dim // 2, 0)
    cos = np.empty((max_seq_len, pairs), dtype=np.float16)
    sin = np.empty((max_seq_len, pairs), dtype=np.float16)
    check(lib.mlxr_rope_tables_host(cos.ctypes.data, sin.ctypes.data, max_seq_len, head_dim,
                                    base, int(scaling_mode), scale_factor, orig_context))
    tc, ts = torch.from_numpy(cos), torch.from_numpy(sin)
    if device is not None:
        tc, ts = tc.to(device), ts.to(device)
    return tc, ts


# ---- operators -----------------------------------------------------------------------------

def dequantize(weights: torch.Tensor, N: int, K: int, quant_type: QuantType,
               out_dtype: torch.dtype = torch.float16, fused: bool = False) -> torch.Tensor:
    """The reference's dequantizers, bit for bit (see mlxr_dequantize)."""
    if out_dtype not in (torch.float16, torch.float32):
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "out_dtype must be fp16 or fp32")
    out = torch.empty((N, K), dtype=out_dtype, device=weights.device)
    check(lib.mlxr_dequantize(_dev(weights, "weights"), out.data_ptr(), N, K, int(quant_type),
                              _DT[out_dtype], 1 if fused else 0, _stream()))
    return out


def repack_ggml_q4_0(ggml_blocks: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """Canonical ggml Q4_0 blocks [N, K] (device, uint8) -> MLXR Q4_0 blocks: value-preserving."""
    out = torch.empty_like(ggml_blocks)
    check(lib.mlxr_repack_ggml_q4_0(_dev(ggml_blocks, "ggml_blocks"), out.data_ptr(), N, K, _stream()))
    return out


def q_gemm_dequant(input: torch.Tensor, weights: torch.Tensor, M: int, N: int, K: int,
                   quant_type: QuantType, group_size: int, bias: Optional[torch.Tensor] = None
                   ) -> torch.Tensor:
    """q_gemm_dequant(), q_gemm_dequant_primitive.h:211-215 / .mm:478-522.
    input [M, K]; weights: packed uint8; bias [N] optional -> [M, N] of input's dtype."""
    if input.dim() != 2 or input.shape[0] != M or input.shape[1] != K:
        raise _capi.MlxrError(_capi.ERR_SHAPE, "Input shape must be [M, K]")
    if bias is not None and (bias.dim() != 1 or bias.shape[0] != N):
        raise _capi.MlxrError(_capi.ERR_SHAPE, "Bias shape must be [N]")
    need = lib.mlxr_quantized_weight_size(N, K, int(quant_type))
    if need and weights.numel() * weights.element_size() < need:
        raise _capi.MlxrError(_capi.ERR_SHAPE, f"weights buffer holds {weights.numel() * weights.element_size()} bytes, {need} needed")
    if bias is not None and bias.dtype != input.dtype:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "bias dtype must match input")
    out = torch.empty((M, N), dtype=input.dtype, device=input.device)
    check(lib.mlxr_q_gemm_dequant(_dev(input, "input"), _dev(weights, "weights"), _dev(bias, "bias"),
                                  out.data_ptr(), M, N, K, int(quant_type), group_size,
                                  _dtype_code(input), _stream()))
    return out


def rmsnorm_fused(input: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                  residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """rmsnorm_fused(), rmsnorm_primitive.h:123-126 / .mm:302-359.  A non-contiguous
    input is made contiguous first, as the reference does (:332-346)."""
    if input.dim() < 1:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "RMSNorm input must have at least 1 dimension")
    if weight.dim() != 1:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "RMSNorm weight must be 1-dimensional")
    hidden = input.shape[-1]
    if weight.numel() != hidden:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT,
                                        "RMSNorm weight size must match input's last dimension")
    if weight.dtype != input.dtype:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "RMSNorm weight dtype must match input")
    x = input.contiguous()
    w = weight.contiguous()
    r = residual.contiguous() if residual is not None else None
    out = torch.empty_like(x)
    rows = x.numel() // hidden if hidden else 0
    check(lib.mlxr_rmsnorm(_dev(x, "input"), _dev(w, "weight"), _dev(r, "residual"), out.data_ptr(),
                           rows, hidden, eps, _dtype_code(x), _stream()))
    return out


def swish(x: torch.Tensor) -> torch.Tensor:
    """swish(), swiglu_mlp_primitive.mm:306-309"""
    out = torch.empty_like(x)
    check(lib.mlxr_swiglu(_dev(x, "x"), None, out.data_ptr(), x.numel(), _dtype_code(x), _stream()))
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """swiglu(), swiglu_mlp_primitive.mm:311-318"""
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "gate and up must match")
    out = torch.empty_like(gate)
    check(lib.mlxr_swiglu(_dev(gate, "gate"), _dev(up, "up"), out.data_ptr(), gate.numel(),
                          _dtype_code(gate), _stream()))
    return out


def swiglu_mlp(input: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
               bias_gate: Optional[torch.Tensor] = None, bias_up: Optional[torch.Tensor] = None,
               bias_down: Optional[torch.Tensor] = None) -> torch.Tensor:
    """swiglu_mlp(), swiglu_mlp_primitive.h:169-176 / .mm:236-304: dense weights of the activation
    dtype, w_gate and w_up [inter, hidden], w_down [hidden, inter], optional biases."""
    if input.dim() != 2:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "Input must be 2D [M, hidden_size]")
    M, hidden = input.shape
    if w_gate.dim() != 2 or w_gate.shape[1] != hidden or w_up.shape != w_gate.shape:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "w_gate and w_up must be [intermediate_size, hidden_size]")
    inter = w_gate.shape[0]
    if tuple(w_down.shape) != (hidden, inter):
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "w_down must be [hidden_size, intermediate_size]")
    for name, t in (("w_gate", w_gate), ("w_up", w_up), ("w_down", w_down), ("bias_gate", bias_gate),
                    ("bias_up", bias_up), ("bias_down", bias_down)):
        if t is not None and t.dtype != input.dtype:
            raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, f"{name} must have the input's dtype")
    y = torch.empty_like(input)
    check(lib.mlxr_mlp_block_dense(_dev(input, "input"), _dev(w_gate, "w_gate"), _dev(w_up, "w_up"),
                                   _dev(w_down, "w_down"), _dev(bias_gate, "bias_gate"), _dev(bias_up, "bias_up"),
                                   _dev(bias_down, "bias_down"), y.data_ptr(), M, hidden, inter,
                                   _dtype_code(input), _stream()))
    return y


def rope_apply(input: torch.Tensor, cos_table: torch.Tensor, sin_table: torch.Tensor,
               positions: torch.Tensor, scaling_mode: RoPEScalingMode = RoPEScalingMode.BASE,
               scale_factor: float = 1.0, position_offset: int = 0, inplace: bool = False,
               check_positions: bool = True) -> torch.Tensor:
    """rope_apply(), rope_apply_primitive.h:192-197 / .mm:399-475.  input is
    [tokens, heads, d] or [batch, seq, heads, d]; tables fp16 [max_seq, d/2]."""
    if input.dim() not in (3, 4):
        raise _capi.MlxrError(_capi.ERR_SHAPE, "Input must be 3D [tokens, num_heads, head_dim] or 4D [batch, seq_len, num_heads, head_dim]")
    if input.dim() == 4:
        batch, seq, heads, hd = input.shape
    else:
        batch, heads, hd = input.shape
        seq = 1
    if hd % 2 != 0:
        raise _capi.MlxrError(_capi.ERR_SHAPE, "head_dim must be even for RoPE")
    pairs = hd // 2
    for name, t in (("cos_table", cos_table), ("sin_table", sin_table)):
        if t.dim() != 2 or t.shape[1] != pairs:
            raise _capi.MlxrError(_capi.ERR_SHAPE, f"{name} must have shape [max_seq_len, head_dim/2]")
        if t.dtype != torch.float16:
            raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, f"{name} must be float16")
    if seq == 1:
        if positions.dim() != 1 or positions.shape[0] != batch:
            raise _capi.MlxrError(_capi.ERR_SHAPE, "For flattened input, positions must have shape [tokens]")
    elif positions.dim() != 2 or positions.shape[0] != batch or positions.shape[1] != seq:
        raise _capi.MlxrError(_capi.ERR_SHAPE, "positions must have shape [batch, seq_len]")
    if positions.dtype != torch.int32:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "positions must be int32")
    out = input if inplace else torch.empty_like(input)
    check(lib.mlxr_rope_apply(_dev(input, "input"), _dev(cos_table, "cos_table"), _dev(sin_table, "sin_table"),
                              _dev(positions, "positions"), out.data_ptr(), batch, seq, heads, hd,
                              cos_table.shape[0], int(scaling_mode), scale_factor, position_offset,
                              _dtype_code(input), 1 if check_positions else 0, _stream()))
    return out


class RotaryEmbedding:
    """graph::RotaryEmbedding (core/graph/layers.h:67-90, layers.cpp:113-225): the split-half
    ("rotate_half") convention with float32 tables and contiguous positions offset .. offset + seq -
    not the interleaved convention of rope_apply above (the reference has both)."""

    def __init__(self, dim: int, max_seq_len: int, base: float = 10000.0):
        if dim % 2 != 0:
            raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "RotaryEmbedding dimension must be even")
        self.dim, self.max_seq_len, self.base = dim, max_seq_len, base
        cos = torch.empty((max_seq_len, dim // 2), dtype=torch.float32)
        sin = torch.empty_like(cos)
        check(lib.mlxr_rope_tables_f32_host(cos.data_ptr(), sin.data_ptr(), max_seq_len, dim, base))
        self.cos_host, self.sin_host = cos, sin
        self._dev = {}

    def cos_table(self) -> torch.Tensor:
        return self.cos_host

    def sin_table(self) -> torch.Tensor:
        return self.sin_host

    def _tables(self, device):
        if device not in self._dev:
            self._dev[device] = (self.cos_host.to(device), self.sin_host.to(device))
        return self._dev[device]

    def forward(self, q: torch.Tensor, k: torch.Tensor, offset: int = 0):
        """q, k: [batch, seq_len, num_heads, head_dim] -> (q_rotated, k_rotated)."""
        if q.dim() != 4 or k.dim() != 4:
            raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT,
                                            "RotaryEmbedding expects 4D tensors [batch, seq_len, num_heads, head_dim]")
        if q.shape[3] != self.dim or k.shape[3] != self.dim:
            raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "head_dim must match RotaryEmbedding dim")
        outs = []
        for t in (q, k):
            cos, sin = self._tables(t.device)
            out = torch.empty_like(t)
            b, sq, h, d = t.shape
            check(lib.mlxr_rope_apply_split_half(_dev(t, "input"), cos.data_ptr(), sin.data_ptr(), out.data_ptr(), b, sq, h, d,
                                                 self.max_seq_len, offset, _dtype_code(t), _stream()))
            outs.append(out)
        return outs[0], outs[1]


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """graph::Linear::forward (core/graph/layers.cpp:86-99) with a dense weight [out, in] of the
    activation dtype: x[..., in] -> [..., out]."""
    K = x.shape[-1]
    N = weight.shape[0]
    if weight.dim() != 2 or weight.shape[1] != K or weight.dtype != x.dtype:
        raise _capi.MlxrError(_capi.ERR_SHAPE, "Linear: weight must be [out_features, in_features] of the input dtype")
    M = x.numel() // K
    y = torch.empty(x.shape[:-1] + (N,), dtype=x.dtype, device=x.device)
    check(lib.mlxr_linear_dense(_dev(x, "input"), _dev(weight, "weight"), _dev(bias, "bias"), y.data_ptr(), M, N, K,
                                _dtype_code(x), _stream()))
    return y


def mlp_block(x: torch.Tensor, norm_weight: Optional[torch.Tensor], w_gate: torch.Tensor,
              w_up: torch.Tensor, w_down: torch.Tensor, inter: int, quant_type: QuantType,
              eps: float = 1e-5) -> torch.Tensor:
    """y = down(SiLU(gate(n)) * up(n)), n = rmsnorm(x) when norm_weight is given: the
    quantized form of swiglu_mlp() (swiglu_mlp_primitive.h:169-176) with the RMSNorm
    prologue of TransformerBlock::forward (core/graph/layers.cpp:451-452)."""
    if x.dim() != 2:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "Input must be 2D [M, hidden_size]")
    M, hidden = x.shape
    qt = int(quant_type)
    for name, t, n, k in (("w_gate", w_gate, inter, hidden), ("w_up", w_up, inter, hidden),
                          ("w_down", w_down, hidden, inter)):
        need = lib.mlxr_quantized_weight_size(n, k, qt)
        if need and t.numel() * t.element_size() != need:
            raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, f"{name} shape mismatch")
    if norm_weight is not None and (norm_weight.dim() != 1 or norm_weight.numel() != hidden
                                    or norm_weight.dtype != x.dtype):
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT,
                                        "RMSNorm weight size must match input's last dimension")
    y = torch.empty_like(x)
    check(lib.mlxr_mlp_block(_dev(x, "x"), _dev(norm_weight, "norm_weight"), _dev(w_gate, "w_gate"),
                             _dev(w_up, "w_up"), _dev(w_down, "w_down"), y.data_ptr(), M, hidden,
                             inter, qt, eps, _dtype_code(x), _stream()))
    return y


def mlp_block_partial(x: torch.Tensor, norm_weight: Optional[torch.Tensor], w_gate_shard: torch.Tensor,
                      w_up_shard: torch.Tensor, w_down_shard: torch.Tensor, inter_local: int,
                      quant_type: QuantType, eps: float = 1e-5) -> torch.Tensor:
    """One rank's float32 partial [M, hidden] of the tensor-parallel block (see
    mlxr_mlp_block_partial_f32): `inter_local` is the rank's share of the intermediate size."""
    if x.dim() != 2:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "Input must be 2D [M, hidden_size]")
    M, hidden = x.shape
    y = torch.empty((M, hidden), dtype=torch.float32, device=x.device)
    check(lib.mlxr_mlp_block_partial_f32(_dev(x, "x"), _dev(norm_weight, "norm_weight"),
                                         _dev(w_gate_shard, "w_gate_shard"), _dev(w_up_shard, "w_up_shard"),
                                         _dev(w_down_shard, "w_down_shard"), y.data_ptr(), M, hidden, inter_local,
                                         int(quant_type), eps, _dtype_code(x), _stream()))
    return y


def qkv_rope(x: torch.Tensor, norm_weight: Optional[torch.Tensor], wq: torch.Tensor,
             wk: torch.Tensor, wv: torch.Tensor, cos_table: torch.Tensor, sin_table: torch.Tensor,
             positions: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
             quant_type: QuantType, eps: float = 1e-5, position_offset: int = 0
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """RMSNorm -> q/k/v projections -> rope_apply on q and k (see mlxr_qkv_rope)."""
    M, hidden = x.shape
    q = torch.empty((M, q_heads, head_dim), dtype=x.dtype, device=x.device)
    k = torch.empty((M, kv_heads, head_dim), dtype=x.dtype, device=x.device)
    v = torch.empty((M, kv_heads, head_dim), dtype=x.dtype, device=x.device)
    if positions.dtype != torch.int32 or positions.numel() != M:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "positions must be int32 [M]")
    check(lib.mlxr_qkv_rope(_dev(x, "x"), _dev(norm_weight, "norm_weight"), _dev(wq, "wq"), _dev(wk, "wk"),
                            _dev(wv, "wv"), _dev(cos_table, "cos_table"), _dev(sin_table, "sin_table"),
                            _dev(positions, "positions"), q.data_ptr(), k.data_ptr(), v.data_ptr(), M,
                            hidden, q_heads, kv_heads, head_dim, cos_table.shape[0], int(quant_type),
                            eps, position_offset, _dtype_code(x), _stream()))
    return q, k, v
