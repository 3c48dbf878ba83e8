"""Pins the oracle (oracle/mlxr_oracle.c) before anything is compared with it:
  1. hand-derived known answers (integers and powers of two, checkable on paper);
  2. the committed golden fixtures, which hold outputs of the REFERENCE's own code
     (tests/golden/make_golden.py ran oracle/_ref);
  3. where oracle/_ref is built (the MLXR tree is present), fresh fuzz against it.
CPU only."""
import os

import numpy as np
import pytest

from conftest import fuzz_blocks, make_weights

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def h(bits):
    return np.array([bits], dtype=np.uint16).view(np.float16)[0]


# ---- 1. known answers ---------------------------------------------------------------------

def test_fp16_to_fp32_known_values(oracle):
    f = oracle.lib.orc_fp16_to_fp32
    assert f(0x3C00) == 1.0 and f(0xC000) == -2.0 and f(0x0001) == 2.0 ** -24
    assert f(0x7BFF) == 65504.0 and f(0x0400) == 2.0 ** -14 and f(0x03FF) == 1023 * 2.0 ** -24
    assert np.signbit(np.float32(f(0x8000))) and f(0x8000) == 0.0
    assert f(0x7C00) == np.inf and f(0xFC00) == -np.inf and np.isnan(f(0x7E01)) and np.isnan(f(0xFE00))
    # all finite values agree with IEEE (numpy)
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    got = np.array([f(int(v)) for v in allh], dtype=np.float32)
    fin = np.isfinite(ref)
    assert np.array_equal(got[fin].view(np.uint32), ref[fin].view(np.uint32))


def test_fp32_to_fp16_rne(oracle):
    g = oracle.lib.orc_fp32_to_fp16
    rng = np.random.default_rng(3)
    v = np.concatenate([rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-8, 5, 20000),
                        np.array([65504, 65519.99, 65520, 1e-8, 2.0 ** -25, 2.0 ** -24 * 1.5, 0.0, -0.0], dtype=np.float32)]).astype(np.float32)
    with np.errstate(over="ignore"):
        ref = v.astype(np.float16).view(np.uint16)
    got = np.array([g(float(x)) for x in v], dtype=np.uint16)
    assert np.array_equal(got, ref)


def test_q4_0_known_block(oracle):
    # scale 1.0; byte i = lo nibble i%16, hi nibble (i+1)%16 -> elements 2i, 2i+1
    blk = np.zeros(18, dtype=np.uint8)
    blk[0:2] = [0x00, 0x3C]
    for i in range(16):
        blk[2 + i] = (i % 16) | (((i + 1) % 16) << 4)
    f, hb = oracle.dequantize(blk, 1, 32, oracle.Q4_0)
    exp = np.array([[i % 16 - 8, (i + 1) % 16 - 8] for i in range(16)], dtype=np.float32).ravel()
    assert np.array_equal(f[0], exp) and np.array_equal(hb.view(np.float16)[0].astype(np.float32), exp)
    blk[0:2] = [0x00, 0xC0]  # scale -2
    f, _ = oracle.dequantize(blk, 1, 32, oracle.Q4_0)
    assert np.array_equal(f[0], -2 * exp)
    blk[0:2] = [0x01, 0x00]  # smallest subnormal
    f, hb = oracle.dequantize(blk, 1, 32, oracle.Q4_0)
    assert np.array_equal(f[0], exp * np.float32(2.0 ** -24))
    assert np.array_equal(hb.view(np.float16)[0].astype(np.float64), exp.astype(np.float64) * 2.0 ** -24)


def test_q8_0_and_q4_1_known_block(oracle):
    blk = np.zeros(34, dtype=np.uint8)
    blk[0:2] = [0x00, 0x38]  # 0.5
    vals = np.arange(-16, 16, dtype=np.int8)
    vals[0], vals[31] = -128, 127
    blk[2:] = vals.view(np.uint8)
    f, _ = oracle.dequantize(blk, 1, 32, oracle.Q8_0)
    assert np.array_equal(f[0], vals.astype(np.float32) * 0.5)
    b1 = np.zeros(20, dtype=np.uint8)
    b1[0:2] = [0x00, 0x40]   # scale 2
    b1[2:4] = [0x00, 0xBC]   # min -1
    b1[4:] = np.arange(16) | ((15 - np.arange(16)) << 4)
    f, hb = oracle.dequantize(b1, 1, 32, oracle.Q4_1)
    exp = np.array([[2 * i - 1, 2 * (15 - i) - 1] for i in range(16)], dtype=np.float32).ravel()
    assert np.array_equal(f[0], exp) and np.array_equal(hb.view(np.float16)[0].astype(np.float32), exp)


# scales bytes and the (scale, min) pairs they decode to under the shader's unpacking
# (q_gemm_dequant.metal:222-242), worked out by hand:
#   group 0: b0=0xC5 b1=0x9A b2=0x7D -> offset 0: sc=0x05=5,  mn=(3 | 0xA<<2)=43 ; offset 1: sc=(9 | 1<<4)=25, mn=0x7D>>2=31
#   group 1: b0=0x23 b1=0xF1 b2=0x08 -> offset 0: sc=35,      mn=(0 | 1<<2)=4    ; offset 1: sc=(15 | 0)=15,    mn=2
Q4K_SCALES = [0xC5, 0x9A, 0x7D, 0x23, 0xF1, 0x08, 0xFF, 0x01, 0xAA, 0x55, 0x3C, 0xE7]
Q4K_PAIRS = [(5, 43), (25, 31), (5, 43), (5, 43), (35, 4), (15, 2), (35, 4), (35, 4)]


def _q4k_block(d_bits, dmin_bits, qs):
    b = np.zeros(144, dtype=np.uint8)
    b[0:2] = [d_bits & 255, d_bits >> 8]
    b[2:4] = [dmin_bits & 255, dmin_bits >> 8]
    b[4:16] = Q4K_SCALES
    b[16:] = qs
    return b


def test_q4_k_known_block_integer_scales(oracle):
    qs = (np.arange(128) * 29 + 7).astype(np.uint8)
    lo, hi = (qs & 15).astype(np.int32), (qs >> 4).astype(np.int32)
    q = np.stack([lo, hi], axis=1).reshape(8, 32)  # byte i -> elements 2i, 2i+1
    for d_bits, dmin_bits, dv, mv in ((0x3C00, 0x3C00, 1.0, 1.0), (0x3800, 0xB400, 0.5, -0.25)):
        f, hb = oracle.dequantize(_q4k_block(d_bits, dmin_bits, qs), 1, 256, oracle.Q4_K)
        exp = np.concatenate([(q[s] - 8) * (Q4K_PAIRS[s][0] * dv) + Q4K_PAIRS[s][1] * mv for s in range(8)])
        assert np.array_equal(f[0].astype(np.float64), exp)           # all values exact in half
        assert np.array_equal(hb.view(np.float16)[0].astype(np.float64), exp)


def test_q4_k_rounding_per_operation(oracle):
    """Non-trivial d/dmin: every half operation rounds (NumPy float16 via float64 as an
    independent implementation); the fused variant differs somewhere."""
    qs = (np.arange(128) * 53 + 11).astype(np.uint8)
    blk = _q4k_block(0x2E66, 0x3266, qs)  # d ~ 0.1, dmin ~ 0.2
    _, hb = oracle.dequantize(blk, 1, 256, oracle.Q4_K)
    _, hf = oracle.dequantize(blk, 1, 256, oracle.Q4_K, fused=True)
    d, dmin = float(h(0x2E66)), float(h(0x3266))
    exp, expf = [], []
    for s in range(8):
        sc, mn = Q4K_PAIRS[s]
        ss = float(np.float16(sc * d))
        sm = float(np.float16(mn * dmin))
        for i in range(16):
            for nib in (qs[16 * s + i] & 15, qs[16 * s + i] >> 4):
                v = int(nib) - 8
                exp.append(np.float16(float(np.float16(v * ss)) + sm))
                expf.append(np.float16(v * ss + sm))
    assert np.array_equal(hb[0], np.array(exp, dtype=np.float16).view(np.uint16))
    assert np.array_equal(hf[0], np.array(expf, dtype=np.float16).view(np.uint16))
    # the two variants are not the same function: on fuzzed blocks they differ somewhere
    packed = fuzz_blocks(3, 64, 99)
    _, a = oracle.dequantize(packed, 1, 64 * 256, oracle.Q4_K)
    _, b = oracle.dequantize(packed, 1, 64 * 256, oracle.Q4_K, fused=True)
    assert 0 < np.count_nonzero(a != b) < a.size // 4


def test_nf4_known_block(oracle):
    code = oracle.nf4_codebook()
    assert code[0] == -1.0 and code[7] == 0.0 and code[15] == 1.0 and np.all(np.diff(code) > 0)
    blk = np.zeros(34, dtype=np.uint8)
    blk[0:2] = [0x00, 0x40]  # absmax 2.0
    blk[2:] = (np.arange(32) % 16) | (((np.arange(32) + 5) % 16) << 4)
    f, _ = oracle.dequantize(blk, 1, 64, oracle.NF4)
    exp = np.array([[code[i % 16], code[(i + 5) % 16]] for i in range(32)], dtype=np.float32).ravel() * 2
    assert np.array_equal(f[0], exp)


def test_weight_size_and_ragged_k(oracle):
    assert oracle.quantized_weight_size(14336, 4096, oracle.Q4_K) == 33030144
    assert oracle.quantized_weight_size(7, 100, oracle.Q4_0) == 7 * 4 * 18   # ceil(100/32)
    with pytest.raises(ValueError):
        oracle.dequantize(np.zeros(4 * 18, dtype=np.uint8), 1, 100, oracle.Q4_0)  # K not whole blocks


def test_rmsnorm_swiglu_known_values(oracle):
    x = np.array([[3.0, 4.0, 0.0, 0.0]], dtype=np.float32)           # mean sq = 6.25 -> rms = 2.5
    y = oracle.rmsnorm(x, np.array([1, 2, 3, 4], dtype=np.float32), 0.0)
    assert np.allclose(y, [[1.2, 3.2, 0.0, 0.0]], rtol=1e-6)
    # reference rmsnorm test's composition (tests/unit/rmsnorm_primitive_test.cpp:22-33) in NumPy
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 4096)).astype(np.float32)
    w = rng.standard_normal(4096).astype(np.float32)
    ref = x * (1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5)) * w
    assert np.all(np.abs(oracle.rmsnorm(x, w, 1e-5) - ref) <= 1e-5 + 1e-4 * np.abs(ref))
    g = np.array([0.0, 1.0, -1.0, 100.0, -100.0], dtype=np.float32)
    s = oracle.swiglu(g, np.ones_like(g))
    assert s[0] == 0.0 and abs(s[1] - 0.7310586) < 1e-6 and abs(s[2] + 0.2689414) < 1e-6
    assert s[3] == 100.0 and abs(s[4]) < 1e-30


def test_rope_identity_and_quarter_turn(oracle):
    # position 0 -> identity; tables cos=0, sin=1 -> (e, o) -> (-o, e)
    x = np.arange(16, dtype=np.float32).reshape(1, 1, 2, 8)
    c, s = oracle.rope_tables(4, 8)
    assert np.array_equal(oracle.rope_apply(x, c, s, np.array([0], dtype=np.int32)), x)
    cz = np.zeros((4, 4), dtype=np.float16).view(np.uint16)
    so = np.ones((4, 4), dtype=np.float16).view(np.uint16)
    y = oracle.rope_apply(x, cz, so, np.array([1], dtype=np.int32))
    assert np.array_equal(y[..., 0::2], -x[..., 1::2]) and np.array_equal(y[..., 1::2], x[..., 0::2])
    y2 = oracle.rope_apply(x, cz, so, np.array([1], dtype=np.int32), 3, 0.5, 2)  # LINEAR scales outputs
    assert np.array_equal(y2, 0.5 * y)


# ---- 2. committed golden fixtures (outputs of the reference's own code) --------------------

@pytest.mark.parametrize("qt", [0, 1, 2, 3, 16])
def test_oracle_matches_golden_dequant(oracle, qt):
    z = np.load(os.path.join(GOLD, f"dequant_qt{qt}.npz"))
    f, hb = oracle.dequantize(z["packed"], int(z["N"]), int(z["K"]), qt)
    assert np.array_equal(hb, z["h16"])
    if "f32" in z:
        a, b = f.view(np.uint32), z["f32"].view(np.uint32)
        nan = np.isnan(f) & np.isnan(z["f32"])
        assert np.array_equal(a[~nan], b[~nan])


def test_oracle_matches_golden_qgemm(oracle):
    z = np.load(os.path.join(GOLD, "qgemm_cpu.npz"))
    for qt in (0, 1, 2):
        y = oracle.qgemm_cpu(z[f"x{qt}"], z[f"w{qt}"], 20, qt)
        yb = oracle.qgemm_cpu(z[f"x{qt}"], z[f"w{qt}"], 20, qt, z[f"b{qt}"])
        assert np.array_equal(y.view(np.uint32), z[f"y{qt}"].view(np.uint32))
        assert np.array_equal(yb.view(np.uint32), z[f"yb{qt}"].view(np.uint32))


def test_oracle_matches_golden_rope(oracle):
    z = np.load(os.path.join(GOLD, "rope.npz"))
    for name, (ms, d, base, mode, scale) in dict(llama3=(256, 128, 500000.0, 0, 1.0), tiny=(64, 64, 10000.0, 0, 1.0),
                                                 linear=(64, 32, 10000.0, 3, 4.0), ntk=(32, 16, 10000.0, 1, 8.0)).items():
        c, s = oracle.rope_tables(ms, d, base, mode, scale)
        assert np.array_equal(c, z[f"cos_{name}"]) and np.array_equal(s, z[f"sin_{name}"])
    c, s = z["cos_llama3"], z["sin_llama3"]
    assert np.array_equal(oracle.rope_apply(z["x"], c, s, z["pos"]).view(np.uint32), z["y_base"].view(np.uint32))
    assert np.array_equal(oracle.rope_apply(z["x"], c, s, z["pos"], 3, 0.5, 5).view(np.uint32), z["y_linear_off"].view(np.uint32))
    y3 = oracle.rope_apply(z["x3"][:, None], c, s, z["pos3"])[:, 0]
    assert np.array_equal(y3.view(np.uint32), z["y3"].view(np.uint32))


def test_host_rope_tables_match_golden():
    """The product's own compute_rope_tables (host code in the C-ABI library) against the
    reference's tables."""
    import mlxr_b200 as mx
    z = np.load(os.path.join(GOLD, "rope.npz"))
    c, s = mx.compute_rope_tables(256, 128, 500000.0)
    assert np.array_equal(c.numpy().view(np.uint16), z["cos_llama3"]) and np.array_equal(s.numpy().view(np.uint16), z["sin_llama3"])
    c, s = mx.compute_rope_tables(64, 32, 10000.0, mx.RoPEScalingMode.LINEAR, 4.0)
    assert np.array_equal(c.numpy().view(np.uint16), z["cos_linear"]) and np.array_equal(s.numpy().view(np.uint16), z["sin_linear"])
    c, s = mx.compute_rope_tables(32, 16, 10000.0, mx.RoPEScalingMode.NTK, 8.0)
    assert np.array_equal(c.numpy().view(np.uint16), z["cos_ntk"])


# ---- 3. live comparison with the compiled reference (container only) -----------------------

def _ref():
    from oracle import ref as R
    if not R.available():
        pytest.skip("oracle/_ref not built (MLXR tree absent)")
    return R


@pytest.mark.parametrize("qt", [0, 1, 2, 3])
def test_oracle_vs_reference_fuzz(oracle, qt):
    R = _ref()
    nb = 4000
    be = oracle.block_elems(qt)
    packed = fuzz_blocks(qt, nb, 31337 + qt)
    f, hb = oracle.dequantize(packed, 1, nb * be, qt)
    assert np.array_equal(hb.ravel(), R.shader_dequant(qt, packed, nb))
    if qt != 3:
        assert np.array_equal(f.ravel().view(np.uint32), R.cpu_dequant(qt, packed, nb).view(np.uint32))


def test_reference_helpers_vs_product(oracle):
    R = _ref()
    from mlxr_b200._capi import lib
    l = R.lib()
    for qt in (0, 1, 2, 3):
        for N, K in ((1, 32), (7, 100), (14336, 4096), (4096, 14336)):
            assert l.ref_weight_size(N, K, qt) == lib.mlxr_quantized_weight_size(N, K, qt) == oracle.quantized_weight_size(N, K, qt)
        assert l.ref_bytes_per_weight(qt) == lib.mlxr_bytes_per_weight(qt)
    for qt in range(17):
        assert l.ref_default_group_size(qt) == lib.mlxr_default_group_size(qt) or qt in (4, 16)
    for qt in range(16):
        assert l.ref_quant_type_name(qt) == lib.mlxr_quant_type_name(qt)
    for m in range(5):
        assert l.ref_rope_mode_name(m) == lib.mlxr_rope_scaling_mode_name(m)
    assert l.ref_ntk_base(10000.0, 4.0, 128, 2048) == lib.mlxr_ntk_scaled_base(10000.0, 4.0, 128, 2048)


def test_reference_eval_cpu_vs_oracle(oracle):
    R = _ref()
    from mlxr_b200.quantize import quantize
    rng = np.random.default_rng(5)
    for qt in (0, 1, 2):
        M, N, K = 2, 33, 320
        packed = quantize(make_weights(N, K, qt), qt)
        x = rng.standard_normal((M, K)).astype(np.float32)
        assert np.array_equal(R.qgemm_cpu(x, packed, N, qt, 32).view(np.uint32), oracle.qgemm_cpu(x, packed, N, qt).view(np.uint32))
    with pytest.raises(RuntimeError, match="Unsupported quantization format for CPU"):
        R.qgemm_cpu(np.zeros((1, 256), np.float32), np.zeros(144, np.uint8), 1, 3, 256)
