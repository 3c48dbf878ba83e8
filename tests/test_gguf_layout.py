"""Canonical GGML blocks -> MLXR layout (host side): the repacked bytes dequantize, through the
oracle's restatement of the reference's dequantizers, to exactly what gguf.quants gives for the
canonical bytes.  CPU only."""
import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

from conftest import make_weights


@pytest.mark.parametrize("name,ggml,qt", [("Q4_0", 2, 0), ("Q4_1", 3, 1), ("Q8_0", 8, 2)])
def test_repack_is_value_preserving(oracle, name, ggml, qt):
    import gguf.quants as gq
    from gguf import GGMLQuantizationType as T
    from mlxr_b200.gguf_layout import convert
    N, K = 24, 256
    w = make_weights(N, K, 3, std=0.05)
    canon = gq.quantize(w, T(ggml))
    want = gq.dequantize(canon, T(ggml)).astype(np.float32)
    c = convert(canon, N, K, ggml)
    assert c.exact and int(c.quant_type) == qt
    got = oracle.dequantize(c.packed, N, K, qt)[0]
    np.testing.assert_array_equal(got, want)


def test_q4_k_needs_requantization(oracle):
    import gguf.quants as gq
    from gguf import GGMLQuantizationType as T
    from mlxr_b200.gguf_layout import convert, GGML_Q4_K
    N, K = 8, 512
    # gguf.quants cannot quantize Q4_K; build canonical blocks by hand: d, dmin, 12 scale bytes, 128 nibble bytes
    rng = np.random.default_rng(1)
    blocks = rng.integers(0, 256, size=(N * K // 256, 144), dtype=np.uint8)
    blocks[:, 0:2] = np.frombuffer(np.float16(0.01).tobytes(), np.uint8)
    blocks[:, 2:4] = np.frombuffer(np.float16(0.02).tobytes(), np.uint8)
    with pytest.raises(ValueError):
        convert(blocks, N, K, GGML_Q4_K)
    c = convert(blocks, N, K, GGML_Q4_K, allow_requantize=True)
    assert not c.exact and int(c.quant_type) == 3
    want = gq.dequantize(blocks.reshape(N, -1), T.Q4_K).astype(np.float32).reshape(N, K)
    got = oracle.dequantize(c.packed, N, K, 3)[0]
    # MLXR's Q4_K shares one (scale, min) pair among three sub-blocks: a coarse requantization
    assert oracle.rel_l2(got, want) < 0.35
    assert np.isfinite(got).all()


def test_read_from_gguf_file(oracle, tmp_path):
    import gguf.quants as gq
    from gguf import GGMLQuantizationType as T, GGUFWriter
    from mlxr_b200.gguf_layout import load_linear
    N, K = 16, 128
    w = make_weights(N, K, 9, std=0.05)
    canon = gq.quantize(w, T.Q4_0)
    path = str(tmp_path / "tiny.gguf")
    wr = GGUFWriter(path, "llama")
    wr.add_tensor("blk.0.ffn_up.weight", canon, raw_shape=canon.shape, raw_dtype=T.Q4_0)
    wr.write_header_to_file(); wr.write_kv_data_to_file(); wr.write_tensors_to_file(); wr.close()
    c, n, k = load_linear(path, "blk.0.ffn_up.weight")
    assert (n, k) == (N, K) and c.exact
    np.testing.assert_array_equal(oracle.dequantize(c.packed, N, K, 0)[0], gq.dequantize(canon, T.Q4_0).astype(np.float32))
    with pytest.raises(KeyError):
        load_linear(path, "missing")
