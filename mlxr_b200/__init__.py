"""mlxr_b200 -- B200-native (sm_100a) implementation of MLXR's quantized-linear path.

The product is the CUDA library behind the C ABI in include/mlxr_b200.h and the C++
primitive layer in mlxr_b200/cpp (MLXR's Primitive classes and free functions).  This
Python package is a thin host-side mirror of the same operator interface over torch
tensors (torch supplies device memory and streams only).
"""
from .types import QuantType, RoPEScalingMode  # noqa: F401
from .ops import (  # noqa: F401
    compute_quantized_weight_size,
    compute_rope_tables,
    dequantize,
    mlp_block,
    q_gemm_dequant,
    qkv_rope,
    quant_type_name,
    rmsnorm_fused,
    rope_apply,
    swiglu,
    swish,
)
