"""mlxr_b200 -- B200-native (sm_100a) implementation of MLXR's quantized-linear path.

The product is the CUDA library behind the C ABI in include/mlxr_b200.h and the C++
primitive layer in mlxr_b200/cpp (MLXR's Primitive classes and free functions).  This
Python package is a thin host-side mirror of the same operator interface over torch
tensors (torch supplies device memory and streams only).

Operators are imported on first use so that ``python -m mlxr_b200.build`` can run before
the shared library exists.
"""
from .types import QuantType, RoPEScalingMode  # noqa: F401

_OPS = ("compute_quantized_weight_size", "compute_rope_tables", "dequantize", "mlp_block", "mlp_block_partial", "q_gemm_dequant",
        "qkv_rope", "quant_type_name", "rmsnorm_fused", "rope_apply", "swiglu", "swish", "swiglu_mlp", "RotaryEmbedding", "linear", "repack_ggml_q4_0")


def __getattr__(name):
    if name in _OPS:
        from . import ops
        return getattr(ops, name)
    if name in ("ops", "_capi", "quantize", "build", "build_cpp", "tp", "gguf_layout"):
        import importlib
        return importlib.import_module(f".{name}", __name__)
    raise AttributeError(f"module 'mlxr_b200' has no attribute {name!r}")
