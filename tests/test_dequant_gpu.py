"""CUDA dequantizer vs the oracle: bit-exact, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import fuzz_blocks, make_weights

pytestmark = pytest.mark.gpu

FORMATS = [0, 1, 2, 3, 16]  # Q4_0 Q4_1 Q8_0 Q4_K NF4


def assert_same_half_bits(got, ref):
    """Bit-exact, except that NaN payloads are not compared: the reference canonicalises NaN
    (q_gemm_dequant_primitive.mm:158), so only NaN-ness is part of the gate."""
    nan_g = (got & 0x7FFF) > 0x7C00
    nan_r = (ref & 0x7FFF) > 0x7C00
    assert np.array_equal(nan_g, nan_r), "NaN positions differ"
    bad = (got != ref) & ~nan_r
    assert not bad.any(), f"fp16 mismatch in {np.count_nonzero(bad)} of {got.size}"


def assert_same_float_bits(got, ref):
    nan_g, nan_r = np.isnan(got), np.isnan(ref)
    assert np.array_equal(nan_g, nan_r), "NaN positions differ"
    bad = (got.view(np.uint32) != ref.view(np.uint32)) & ~nan_r
    assert not bad.any(), f"fp32 mismatch in {np.count_nonzero(bad)} of {got.size}"


def _dequant_gpu(packed, N, K, qt, out_dtype, fused=False):
    import mlxr_b200 as mx
    w = torch.from_numpy(packed).cuda()
    out = mx.dequantize(w, N, K, mx.QuantType(qt), out_dtype, fused)
    torch.cuda.synchronize()
    return out.cpu()


@pytest.mark.parametrize("qt", FORMATS)
@pytest.mark.parametrize("fused", [False, True])
def test_fuzz_bit_exact(oracle, qt, fused):
    """Random block bytes (finite scales): every output bit equals the oracle's."""
    be = oracle.block_elems(qt)
    N, K = 37, be * 12
    packed = fuzz_blocks(qt, N * (K // be), seed=1000 + qt)
    f_ref, h_ref = oracle.dequantize(packed, N, K, qt, fused)
    h = _dequant_gpu(packed, N, K, qt, torch.float16, fused).view(torch.int16).numpy().view(np.uint16)
    f = _dequant_gpu(packed, N, K, qt, torch.float32, fused).numpy()
    # finite scales can still overflow to inf and give inf * 0 or inf - inf = NaN
    assert_same_half_bits(h, h_ref)
    assert_same_float_bits(f, f_ref)


@pytest.mark.parametrize("qt", FORMATS)
def test_quantized_normal_weights(oracle, qt):
    """Weights ~N(0, 0.02) through the package quantizer (the benchmark's distribution)."""
    from mlxr_b200.quantize import quantize
    N, K = 64, 1024
    packed = quantize(make_weights(N, K, 7), qt)
    f_ref, h_ref = oracle.dequantize(packed, N, K, qt)
    h = _dequant_gpu(packed, N, K, qt, torch.float16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(h, h_ref)


@pytest.mark.parametrize("qt", FORMATS)
def test_golden_fixture(oracle, qt):
    """Committed fixture (tests/golden/dequant_*.npz: blocks + outputs of the reference's own
    code where it exists) reproduced on the GPU."""
    import os
    path = os.path.join(os.path.dirname(__file__), "golden", f"dequant_qt{qt}.npz")
    if not os.path.exists(path):
        pytest.skip("fixture not generated")
    z = np.load(path)
    N, K = int(z["N"]), int(z["K"])
    h = _dequant_gpu(z["packed"], N, K, qt, torch.float16).view(torch.int16).numpy().view(np.uint16)
    assert_same_half_bits(h, z["h16"])
    if "f32" in z:
        f = _dequant_gpu(z["packed"], N, K, qt, torch.float32).numpy()
        assert_same_float_bits(f, z["f32"])


def test_empty_and_single_block(oracle):
    import mlxr_b200 as mx
    w = torch.zeros(0, dtype=torch.uint8, device="cuda")
    assert mx.dequantize(w, 0, 256, mx.QuantType.Q4_K).shape == (0, 256)
    packed = fuzz_blocks(3, 1, 5)
    _, h_ref = oracle.dequantize(packed, 1, 256, 3)
    h = _dequant_gpu(packed, 1, 256, 3, torch.float16).view(torch.int16).numpy().view(np.uint16)
    assert_same_half_bits(h, h_ref)


def test_full_size_checksum(oracle):
    """14336 x 4096 Q4_K (the benchmark's up_proj): 58.7 M values, compared bit for bit."""
    from mlxr_b200.quantize import quantize
    N, K = 14336, 4096
    packed = quantize(make_weights(N, K, 11), 3)
    _, h_ref = oracle.dequantize(packed, N, K, 3)
    h = _dequant_gpu(packed, N, K, 3, torch.float16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(h, h_ref)
