"""Enumerations of the operator interface (values are those of the reference headers)."""
from enum import IntEnum


class QuantType(IntEnum):
    """core/kernels/primitives/q_gemm_dequant_primitive.h:18-35, plus NF4 (not in MLXR)."""
    Q4_0 = 0
    Q4_1 = 1
    Q8_0 = 2
    Q4_K = 3
    Q6_K = 4
    Q5_0 = 5
    Q5_1 = 6
    Q8_1 = 7
    Q2_K = 8
    Q3_K = 9
    Q5_K = 10
    Q8_K = 11
    IQ2_XXS = 12
    IQ2_XS = 13
    IQ3_XXS = 14
    IQ3_S = 15
    NF4 = 16
    # extension: canonical ggml layouts as stored in .gguf files (include/mlxr_b200.h)
    GGML_Q4_0 = 32
    GGML_Q4_K = 33


class RoPEScalingMode(IntEnum):
    """core/kernels/primitives/rope_apply_primitive.h:18-23"""
    BASE = 0
    NTK = 1
    YARN = 2
    LINEAR = 3


# elements per block, bytes per block
BLOCK = {
    QuantType.Q4_0: (32, 18),
    QuantType.Q4_1: (32, 20),
    QuantType.Q8_0: (32, 34),
    QuantType.Q4_K: (256, 144),
    QuantType.NF4: (64, 34),
    QuantType.GGML_Q4_0: (32, 18),
    QuantType.GGML_Q4_K: (256, 144),
}
