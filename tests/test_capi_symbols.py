"""The C-ABI library loads and exports every symbol include/*.h declares (no compute)."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"MLXR_API\s+[^;(]*?\b(mlxr_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "mlxr_q_gemm_dequant" in names and "mlxr_dequantize" in names and len(names) >= 20


def test_library_exports_every_declared_symbol():
    from mlxr_b200 import _capi
    lib = ctypes.CDLL(_capi.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_python_binding_covers_header():
    from mlxr_b200 import _capi
    base = [n for n in declared_symbols() if not n.startswith("mlxr_tp_")]
    assert sorted(set(base) - set(_capi.PROTOTYPES)) == []


def test_format_helpers_match_reference_table():
    # q_gemm_dequant_primitive.mm:63-92,116-135; tests/unit/gguf_parser_test.cpp:139-154 (Q4_0: ceil(n/32)*18)
    from mlxr_b200._capi import lib
    assert lib.mlxr_quantized_weight_size(1, 64, 0) == 2 * 18
    assert lib.mlxr_quantized_weight_size(14336, 4096, 3) == 33030144
    assert lib.mlxr_quantized_weight_size(14336, 4096, 2) == 62390272
    assert lib.mlxr_quantized_weight_size(14336, 4096, 16) == 31195136
    assert lib.mlxr_quantized_weight_size(3, 33, 0) == 3 * 2 * 18       # ceil
    assert lib.mlxr_quantized_weight_size(4, 256, 9) == 0               # no code for Q3_K
    assert abs(lib.mlxr_bytes_per_weight(0) - 0.5625) < 1e-7
    assert abs(lib.mlxr_bytes_per_weight(1) - 0.625) < 1e-7
    assert abs(lib.mlxr_bytes_per_weight(2) - 1.0625) < 1e-7
    assert abs(lib.mlxr_bytes_per_weight(3) - 0.5625) < 1e-7
    assert lib.mlxr_bytes_per_weight(9) < 0
    assert [lib.mlxr_default_group_size(q) for q in (0, 1, 2, 3, 9)] == [32, 32, 32, 256, 32]
    names = [lib.mlxr_quant_type_name(q).decode() for q in range(18)]
    assert names[:5] == ["Q4_0", "Q4_1", "Q8_0", "Q4_K", "Q6_K"] and names[15] == "IQ3_S"
    assert names[16] == "NF4" and names[17] == "Unknown"
    assert [lib.mlxr_rope_scaling_mode_name(m).decode() for m in range(5)] == ["BASE", "NTK", "YARN", "LINEAR", "Unknown"]
    assert lib.mlxr_ntk_scaled_base(10000.0, 4.0, 128, 2048) == 10000.0  # as written: a no-op


def test_argument_errors_without_gpu():
    """Validation happens before any CUDA call, so these run anywhere."""
    from mlxr_b200._capi import lib, ERR_SHAPE, ERR_UNSUPPORTED, ERR_INVALID_ARGUMENT
    one = ctypes.c_void_p(16)
    assert lib.mlxr_q_gemm_dequant(one, one, None, one, 1, 4, 48, 0, 32, 0, None) == ERR_SHAPE       # K % 32
    assert b"multiple" in lib.mlxr_last_error()
    assert lib.mlxr_q_gemm_dequant(one, one, None, one, 1, 4, 64, 9, 32, 0, None) == ERR_UNSUPPORTED  # Q3_K
    assert lib.mlxr_q_gemm_dequant(one, one, None, one, 1, 4, 64, 4, 256, 0, None) == ERR_UNSUPPORTED  # Q6_K
    assert lib.mlxr_q_gemm_dequant(one, one, None, one, 1, 4, 64, 0, 64, 0, None) == ERR_SHAPE        # group size
    assert lib.mlxr_q_gemm_dequant(one, one, None, one, 1, 4, 64, 0, 32, 7, None) == ERR_INVALID_ARGUMENT
    assert lib.mlxr_q_gemm_dequant(None, one, None, one, 1, 4, 64, 0, 32, 0, None) == ERR_INVALID_ARGUMENT
    assert lib.mlxr_rmsnorm(None, one, None, one, 2, 8, 1e-5, 0, None) == ERR_INVALID_ARGUMENT
    assert lib.mlxr_rope_apply(one, one, one, one, one, 1, 1, 1, 7, 8, 0, 1.0, 0, 0, 0, None) == ERR_SHAPE
    assert b"head_dim must be even" in lib.mlxr_last_error()
    assert lib.mlxr_dequantize(one, one, 1, 100, 3, 0, 0, None) == ERR_SHAPE
