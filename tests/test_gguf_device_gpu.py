"""Canonical ggml layouts on the device: tensors written to a .gguf file and read back are
dequantized bit for bit like gguf.quants.dequantize, and the quantized linear on them stays
inside the 2e-2 gate (GEMV and GEMM).  Reference side: daemon/registry/gguf_parser.h:141-211
parses such files; daemon/server/model_loader.cpp:236-245 skips their quantized tensors."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
gguf = pytest.importorskip("gguf")


def _canonical_q4_k(N, K, seed):
    """Random canonical Q4_K super-blocks with finite, modest fp16 d / dmin (gguf.quants cannot
    quantize to Q4_K; every bit pattern of scales[] and qs[] is a valid block)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    raw = rng.integers(0, 256, size=(N * (K // 256), 144), dtype=np.uint8)
    d = (rng.random(raw.shape[0]) * 0.002 + 0.0005).astype(np.float16)
    dmin = (rng.random(raw.shape[0]) * 0.004 + 0.0005).astype(np.float16)
    raw[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    raw[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    return raw.reshape(N, -1)


@pytest.fixture(scope="module")
def gguf_file(tmp_path_factory):
    import gguf.quants as gq
    from gguf import GGMLQuantizationType as T, GGUFWriter
    path = str(tmp_path_factory.mktemp("gguf") / "linears.gguf")
    rng = np.random.Generator(np.random.PCG64(5))
    w0 = (rng.standard_normal((320, 1024)) * 0.02).astype(np.float32)
    q4_0 = gq.quantize(w0, T.Q4_0)
    q4_k = _canonical_q4_k(192, 2048, 6)
    wr = GGUFWriter(path, "llama")
    wr.add_tensor("blk.0.ffn_up.weight", q4_0, raw_dtype=T.Q4_0)
    wr.add_tensor("blk.0.ffn_down.weight", q4_k, raw_dtype=T.Q4_K)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    return path, {"blk.0.ffn_up.weight": (q4_0, T.Q4_0, 320, 1024), "blk.0.ffn_down.weight": (q4_k, T.Q4_K, 192, 2048)}


@pytest.mark.parametrize("name", ["blk.0.ffn_up.weight", "blk.0.ffn_down.weight"])
def test_dequantize_bit_exact_from_file(gguf_file, name):
    import gguf.quants as gq
    import mlxr_b200 as mx
    from mlxr_b200.gguf_layout import load_linear_raw
    path, tensors = gguf_file
    raw, qt, N, K = load_linear_raw(path, name)
    src, gtype, n0, k0 = tensors[name]
    assert (N, K) == (n0, k0) and np.array_equal(raw, src.reshape(-1))
    want = gq.dequantize(src, gtype).astype(np.float32).reshape(N, K)
    got = mx.dequantize(torch.from_numpy(raw).cuda(), N, K, qt, torch.float32)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    got16 = mx.dequantize(torch.from_numpy(raw).cuda(), N, K, qt, torch.float16)
    assert np.array_equal(got16.cpu().numpy().view(np.uint16), want.astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("name", ["blk.0.ffn_up.weight", "blk.0.ffn_down.weight"])
@pytest.mark.parametrize("M", [1, 16])
def test_linear_on_canonical_blocks(gguf_file, oracle, name, M):
    import gguf.quants as gq
    import mlxr_b200 as mx
    from mlxr_b200.gguf_layout import load_linear_raw
    path, tensors = gguf_file
    raw, qt, N, K = load_linear_raw(path, name)
    src, gtype, _, _ = tensors[name]
    w = gq.dequantize(src, gtype).astype(np.float32).reshape(N, K)
    x = torch.from_numpy(np.random.Generator(np.random.PCG64(8)).standard_normal((M, K)).astype(np.float32)).bfloat16()
    y = mx.q_gemm_dequant(x.cuda(), torch.from_numpy(raw).cuda(), M, N, K, qt, mx._capi.lib.mlxr_default_group_size(int(qt)))
    torch.cuda.synchronize()
    want = x.float().numpy() @ w.T
    assert oracle.rel_l2(y.float().cpu().numpy(), want) <= 2e-2


def test_q4_0_repack_on_device_runs_the_fast_kernels(gguf_file, oracle):
    import gguf.quants as gq
    import mlxr_b200 as mx
    from mlxr_b200.gguf_layout import convert, load_linear_raw, GGML_Q4_0
    path, tensors = gguf_file
    raw, qt, N, K = load_linear_raw(path, "blk.0.ffn_up.weight")
    dev = mx.repack_ggml_q4_0(torch.from_numpy(raw).cuda(), N, K)
    host = convert(raw, N, K, GGML_Q4_0)                      # the host-side permutation
    assert np.array_equal(dev.cpu().numpy(), host.packed)
    a = mx.dequantize(dev, N, K, mx.QuantType.Q4_0, torch.float32)
    b = mx.dequantize(torch.from_numpy(raw).cuda(), N, K, mx.QuantType.GGML_Q4_0, torch.float32)
    assert torch.equal(a, b)
    x = torch.from_numpy(np.random.Generator(np.random.PCG64(9)).standard_normal((1, K)).astype(np.float32)).half()
    y = mx.q_gemm_dequant(x.cuda(), dev, 1, N, K, mx.QuantType.Q4_0, 32)
    want = x.float().numpy() @ gq.dequantize(tensors["blk.0.ffn_up.weight"][0], tensors["blk.0.ffn_up.weight"][1]).astype(np.float32).reshape(N, K).T
    assert oracle.rel_l2(y.float().cpu().numpy(), want) <= 2e-2
