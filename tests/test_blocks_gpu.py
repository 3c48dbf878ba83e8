"""Fused decoder-layer pieces through the C ABI vs the oracle's composition.
Gate: relative L2 <= 2e-2 (the tolerance of the benchmark definition), measured against
the oracle's fp32 composition with activation-dtype rounding; the float64 chain is
checked as well so that both sides are seen to be near the truth."""
import numpy as np
import pytest
import torch

from conftest import make_acts, make_weights

pytestmark = pytest.mark.gpu
TOL = 2e-2
CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _mlp_case(oracle, M, H, I, qt, dtype, seed, norm=True, eps=1e-5):
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    wg = quantize(make_weights(I, H, seed + 1), qt)
    wu = quantize(make_weights(I, H, seed + 2), qt)
    wd = quantize(make_weights(H, I, seed + 3), qt)
    xt, xf = make_acts(M, H, seed + 4, dtype)
    gam = (1 + 0.1 * np.random.Generator(np.random.PCG64(seed + 5)).standard_normal(H)).astype(np.float32)
    gt = torch.from_numpy(gam).to(dtype)
    gf = gt.float().numpy()
    y = mx.mlp_block(xt.cuda(), gt.cuda() if norm else None, torch.from_numpy(wg).cuda(),
                     torch.from_numpy(wu).cuda(), torch.from_numpy(wd).cuda(), I, mx.QuantType(qt), eps)
    torch.cuda.synchronize()
    ref = oracle.mlp_block(xf, gf if norm else None, wg, wu, wd, I, qt, eps, CODE[dtype])
    truth = oracle.mlp_block_f64(xf, gf if norm else None, wg, wu, wd, I, qt, eps)
    yn = y.float().cpu().numpy()
    return oracle.rel_l2(yn, ref), oracle.rel_l2(yn, truth), oracle.rel_l2(ref, truth)


def test_tinyllama_mlp_q4_0_fp16(oracle):
    """TinyLlama-1.1B-shaped MLP block, decode batch 1, Q4_0, fp16, eps 1e-5."""
    e_ref, e_truth, o_truth = _mlp_case(oracle, 1, 2048, 5632, 0, torch.float16, 10)
    assert e_ref <= TOL and e_truth <= TOL, (e_ref, e_truth, o_truth)


@pytest.mark.parametrize("M", [1, 8, 32, 64])
def test_llama3_8b_mlp_q4_k_bf16(oracle, M):
    e_ref, e_truth, o_truth = _mlp_case(oracle, M, 4096, 14336, 3, torch.bfloat16, 20 + M)
    assert e_ref <= TOL and e_truth <= TOL, (e_ref, e_truth, o_truth)


@pytest.mark.parametrize("qt", [0, 2, 3, 16])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_small_mlp_formats(oracle, qt, dtype):
    e_ref, e_truth, _ = _mlp_case(oracle, 3, 512, 1024, qt, dtype, 40 + qt)
    assert e_ref <= TOL and e_truth <= TOL, (e_ref, e_truth)


def test_mlp_without_norm(oracle):
    e_ref, e_truth, _ = _mlp_case(oracle, 2, 512, 768, 3, torch.float16, 50, norm=False)
    assert e_ref <= TOL and e_truth <= TOL


@pytest.mark.parametrize("M", [1, 8, 32, 64])
def test_llama3_8b_qkv_rope(oracle, M):
    """q 4096x4096, k/v 1024x4096, Q4_K, bf16, theta 5e5, positions uniform in [0, 8192)."""
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    H, qh, kvh, d, qt = 4096, 32, 8, 128, 3
    wq = quantize(make_weights(qh * d, H, 61), qt)
    wk = quantize(make_weights(kvh * d, H, 62), qt)
    wv = quantize(make_weights(kvh * d, H, 63), qt)
    xt, xf = make_acts(M, H, 64 + M, torch.bfloat16)
    gam = torch.from_numpy((1 + 0.1 * np.random.Generator(np.random.PCG64(65)).standard_normal(H)).astype(np.float32)).bfloat16()
    pos = torch.from_numpy(np.random.Generator(np.random.PCG64(66)).integers(0, 8192, M).astype(np.int32))
    cos, sin = mx.compute_rope_tables(8192, d, 500000.0)
    q, k, v = mx.qkv_rope(xt.cuda(), gam.cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(wk).cuda(),
                          torch.from_numpy(wv).cuda(), cos.cuda(), sin.cuda(), pos.cuda(), qh, kvh, d,
                          mx.QuantType.Q4_K, 1e-5)
    torch.cuda.synchronize()
    rq, rk, rv = oracle.qkv_rope(xf, gam.float().numpy(), wq, wk, wv, cos.numpy().view(np.uint16),
                                 sin.numpy().view(np.uint16), pos.numpy(), qh, kvh, d, qt, 1e-5, 1)
    for a, b in ((q, rq), (k, rk), (v, rv)):
        assert oracle.rel_l2(a.float().cpu().numpy(), b) <= TOL


def test_host_buffer_entry_points(oracle):
    """mlxr_mlp_block_host / mlxr_q_gemm_dequant_host: x and y in (pinned) host memory."""
    import mlxr_b200 as mx
    from mlxr_b200._capi import lib, check
    from mlxr_b200.quantize import quantize
    M, H, I, qt = 2, 512, 1024, 3
    wg, wu, wd = (torch.from_numpy(quantize(make_weights(n, k, s), qt)).cuda()
                  for n, k, s in ((I, H, 71), (I, H, 72), (H, I, 73)))
    xt, _ = make_acts(M, H, 74, torch.float16)
    gam = torch.ones(H, dtype=torch.float16, device="cuda")
    xh = xt.pin_memory()
    yh = torch.empty((M, H), dtype=torch.float16).pin_memory()
    st = torch.cuda.current_stream().cuda_stream
    check(lib.mlxr_mlp_block_host(xh.data_ptr(), gam.data_ptr(), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(),
                                  yh.data_ptr(), M, H, I, qt, 1e-5, 0, st))
    y_dev = mx.mlp_block(xt.cuda(), gam, wg, wu, wd, I, mx.QuantType(qt), 1e-5)
    assert torch.equal(yh, y_dev.cpu())
    # pageable host memory takes the staged copy instead of the direct stores
    yp = torch.empty((M, H), dtype=torch.float16)
    check(lib.mlxr_mlp_block_host(xt.contiguous().data_ptr(), gam.data_ptr(), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(),
                                  yp.data_ptr(), M, H, I, qt, 1e-5, 0, st))
    assert torch.equal(yp, y_dev.cpu())
    y2 = torch.empty((M, I), dtype=torch.float16).pin_memory()
    check(lib.mlxr_q_gemm_dequant_host(xh.data_ptr(), wg.data_ptr(), None, y2.data_ptr(), M, I, H, qt, 256, 0, st))
    assert torch.equal(y2, mx.q_gemm_dequant(xt.cuda(), wg, M, I, H, mx.QuantType(qt), 256).cpu())
