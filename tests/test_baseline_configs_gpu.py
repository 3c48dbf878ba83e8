"""Full-size parity cases of the benchmark configurations that the smaller test files leave out:

* the Llama-3-70B-shaped block (hidden 8192, intermediate 28672, Q4_K, bf16) on one GPU: decode
  batches 1 and 32, and both prefill linears at M = 4096 on sampled rows;
* the Llama-3-8B prefill linears at M = 8192, both shapes, sampled rows incl. tile corners;
* the format sweep's prefill leg (14336 x 4096, M = 2048) for Q4_0, Q8_0 and NF4.

Gate 2e-2 relative L2 against the oracle composition (the tests use 1e-2 for bf16).  Where the
oracle's full product would take minutes, a sample of output rows is compared (every row of a
linear is an independent dot-product set, so sampled rows test the kernel's tiling at those
positions and the arithmetic everywhere)."""
import numpy as np
import pytest
import torch

from conftest import make_acts, make_weights

pytestmark = pytest.mark.gpu
TOL = 1e-2
H70, I70, Q4_K = 8192, 28672, 3


@pytest.fixture(scope="module")
def w70():
    """The three packed matrices of the 70B-shaped block, quantized once for the module."""
    from mlxr_b200.quantize import quantize
    wg = quantize(make_weights(I70, H70, 501), Q4_K)
    wu = quantize(make_weights(I70, H70, 502), Q4_K)
    wd = quantize(make_weights(H70, I70, 503), Q4_K)
    return wg, wu, wd


@pytest.fixture(scope="module")
def w70_dev(w70):
    return tuple(torch.from_numpy(a).cuda() for a in w70)


@pytest.mark.parametrize("M", [1, 32])
def test_llama3_70b_decode_block(oracle, w70, w70_dev, M):
    import mlxr_b200 as mx
    wg, wu, wd = w70
    xt, xf = make_acts(M, H70, 510 + M, torch.bfloat16)
    gam = (1 + 0.1 * np.random.Generator(np.random.PCG64(520)).standard_normal(H70)).astype(np.float32)
    gt = torch.from_numpy(gam).bfloat16()
    y = mx.mlp_block(xt.cuda(), gt.cuda(), *w70_dev, I70, mx.QuantType.Q4_K, 1e-5)
    torch.cuda.synchronize()
    st = torch.zeros(1, dtype=torch.int32)
    mx._capi.check(mx._capi.lib.mlxr_stream_status(torch.cuda.current_stream().cuda_stream, st.data_ptr()))
    assert int(st[0]) == 0
    ref = oracle.mlp_block(xf, gt.float().numpy(), wg, wu, wd, I70, Q4_K, 1e-5, oracle.BF16)
    assert oracle.rel_l2(y.float().cpu().numpy(), ref) <= TOL


def _linear_rows(oracle, packed, packed_dev, M, N, K, qt, rows, seed):
    import mlxr_b200 as mx
    xt, xf = make_acts(M, K, seed, torch.bfloat16)
    y = mx.q_gemm_dequant(xt.cuda(), packed_dev, M, N, K, mx.QuantType(qt), mx._capi.lib.mlxr_default_group_size(qt))
    torch.cuda.synchronize()
    st = torch.zeros(1, dtype=torch.int32)
    mx._capi.check(mx._capi.lib.mlxr_stream_status(torch.cuda.current_stream().cuda_stream, st.data_ptr()))
    assert int(st[0]) == 0
    ref = oracle.linear(xf[rows], packed, N, qt)
    return oracle.rel_l2(y[torch.from_numpy(rows).cuda()].float().cpu().numpy(), ref)


def test_llama3_70b_prefill_linears(oracle, w70, w70_dev):
    """M = 4096: [4096, 8192] x [28672, 8192]^T and [4096, 28672] x [8192, 28672]^T."""
    M = 4096
    rows = np.array([0, 1, 127, 128, 255, 256, 2051, M - 1])
    assert _linear_rows(oracle, w70[0], w70_dev[0], M, I70, H70, Q4_K, rows, 530) <= TOL
    assert _linear_rows(oracle, w70[2], w70_dev[2], M, H70, I70, Q4_K, rows, 531) <= TOL


@pytest.mark.parametrize("N,K", [(14336, 4096), (4096, 14336)])
def test_llama3_8b_prefill_m8192(oracle, N, K):
    from mlxr_b200.quantize import quantize
    M = 8192
    packed = quantize(make_weights(N, K, 540), Q4_K)
    rows = np.array([0, 127, 128, 255, 256, 4099, M - 1])
    assert _linear_rows(oracle, packed, torch.from_numpy(packed).cuda(), M, N, K, Q4_K, rows, 541) <= TOL


@pytest.mark.parametrize("qt", [0, 2, 16])
def test_format_sweep_prefill_leg(oracle, qt):
    """Q4_0, Q8_0 and NF4 on the 14336 x 4096 linear at M = 2048 (same fp32 weights per format)."""
    from mlxr_b200.quantize import quantize
    M, N, K = 2048, 14336, 4096
    packed = quantize(make_weights(N, K, 550), qt)
    rows = np.array([0, 1, 127, 128, 255, 256, 1027, M - 1])
    assert _linear_rows(oracle, packed, torch.from_numpy(packed).cuda(), M, N, K, qt, rows, 551) <= TOL
