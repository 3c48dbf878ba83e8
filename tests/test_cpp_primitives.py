"""The C++ primitive layer (MLXR's class and function names over the C ABI): it builds, exports the
reference's entry points, and its own test program - written like the reference's
tests/unit/rmsnorm_primitive_test.cpp - passes on a GPU."""
import subprocess

import pytest


@pytest.fixture(scope="module")
def built():
    from mlxr_b200 import build_cpp
    return build_cpp.build()


def test_builds_and_exports_reference_api(built):
    lib, _ = built
    out = subprocess.run(["nm", "-D", "-C", "--defined-only", lib], capture_output=True, text=True, check=True).stdout
    for sym in ("mlxr::kernels::q_gemm_dequant(", "mlxr::kernels::rmsnorm_fused(", "mlxr::kernels::swiglu_mlp(",
                "mlxr::kernels::swish(", "mlxr::kernels::swiglu(", "mlxr::kernels::rope_apply(",
                "mlxr::kernels::compute_rope_tables(", "mlxr::kernels::compute_ntk_scaled_base(",
                "mlxr::kernels::rope_scaling_mode_name(", "mlxr::kernels::compute_quantized_weight_size(",
                "mlxr::kernels::quant_type_name(", "mlxr::kernels::QGemmDequantPrimitive::eval_gpu(",
                "mlxr::kernels::RMSNormPrimitive::eval_gpu(", "mlxr::kernels::SwiGLUMLPPrimitive::eval_gpu(",
                "mlxr::kernels::RoPEApplyPrimitive::eval_gpu(",
                "mlxr::kernels::QGemmDequantPrimitive::get_bytes_per_weight("):
        assert sym in out, sym


@pytest.mark.gpu
def test_cpp_test_program(built):
    _, exe = built
    p = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "ALL PASSED" in p.stdout, p.stdout + p.stderr
