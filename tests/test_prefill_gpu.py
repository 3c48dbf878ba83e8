"""Tensor-core (tcgen05) quantized GEMM for batch >= 9 on Q4_K, through the C ABI vs the oracle.

Gate 2e-2 relative L2 (tests use 1e-2 bf16 / 2e-3 fp16: for bf16 activations the bit-exact fp16
weight values are rounded once more to bf16 before the MMA, about 1e-3 relative)."""
import numpy as np
import pytest
import torch

from conftest import make_acts, make_weights

pytestmark = pytest.mark.gpu
DT = {"f16": torch.float16, "bf16": torch.bfloat16}
TIGHT = {"f16": 2e-3, "bf16": 1e-2}


def _run(oracle, M, N, K, dt, bias=False, seed=0, rows=None, qt=3):
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    packed = quantize(make_weights(N, K, 100 + seed), qt)
    xt, xf = make_acts(M, K, 200 + seed, DT[dt])
    bt = bf = None
    if bias:
        bt, bf = make_acts(1, N, 300 + seed, DT[dt])
        bt, bf = bt[0].contiguous(), bf[0]
    y = mx.q_gemm_dequant(xt.cuda(), torch.from_numpy(packed).cuda(), M, N, K, mx.QuantType(qt),
                          mx._capi.lib.mlxr_default_group_size(qt), bt.cuda() if bias else None)
    torch.cuda.synchronize()
    st = torch.zeros(1, dtype=torch.int32)
    mx._capi.check(mx._capi.lib.mlxr_stream_status(torch.cuda.current_stream().cuda_stream, st.data_ptr()))
    assert int(st[0]) == 0
    yn = y.float().cpu().numpy()
    if rows is not None:
        ref = oracle.linear(xf[rows], packed, N, qt, bf)
        return oracle.rel_l2(yn[rows], ref)
    return oracle.rel_l2(yn, oracle.linear(xf, packed, N, qt, bf))


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(9, 256, 256), (16, 512, 512), (128, 256, 1024), (129, 300, 768), (256, 256, 256),
                                   (300, 520, 1280), (512, 1024, 2048)])
def test_shapes(oracle, dt, M, N, K):
    assert _run(oracle, M, N, K, dt, seed=M) <= TIGHT[dt]


@pytest.mark.parametrize("qt", [0, 2, 16])
@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(16, 256, 64), (130, 300, 448), (300, 512, 1024)])
def test_other_formats(oracle, qt, dt, M, N, K):
    """Q4_0, Q8_0 and NF4 through the same tensor-core kernel (K a multiple of 64)."""
    assert _run(oracle, M, N, K, dt, seed=M + qt, qt=qt) <= TIGHT[dt]


@pytest.mark.parametrize("M,N,K", [(16, 256, 2048), (33, 1024, 4096), (128, 300, 1536), (64, 4096, 14336)])
def test_split_k_small_batches(oracle, M, N, K):
    """One row of output tiles: the K range is split over CTAs and the last slice reduces."""
    import mlxr_b200 as mx
    assert mx._capi.lib.mlxr_version()  # library loaded
    rows = np.arange(M) if M * N * K < 3e8 else np.array([0, 1, M // 2, M - 1])
    assert _run(oracle, M, N, K, "bf16", seed=3, rows=rows, bias=(N == 300)) <= TIGHT["bf16"]
    # twice in a row: the tile counters must have cleared themselves
    assert _run(oracle, M, N, K, "bf16", seed=3, rows=rows) <= TIGHT["bf16"]


def test_bias_and_ragged_edges(oracle):
    assert _run(oracle, 70, 264, 512, "f16", bias=True) <= TIGHT["f16"]
    assert _run(oracle, 257, 8, 256, "bf16", bias=True) <= TIGHT["bf16"]


@pytest.mark.parametrize("M,N,K", [(2048, 14336, 4096), (512, 4096, 14336)])
def test_baseline_sizes_sampled_rows(oracle, M, N, K):
    """Full-size prefill shapes: a sample of output rows against the oracle (tile corners and
    interior), since the scalar oracle cannot do the whole product in seconds."""
    rows = np.array([0, 1, 127, 128, 255, 256, M // 2 + 3, M - 1])
    assert _run(oracle, M, N, K, "bf16", rows=rows) <= TIGHT["bf16"]


def test_repeatable():
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    packed = torch.from_numpy(quantize(make_weights(512, 1024, 5), 3)).cuda()
    x = torch.randn(384, 1024, dtype=torch.bfloat16, device="cuda")
    a = mx.q_gemm_dequant(x, packed, 384, 512, 1024, mx.QuantType.Q4_K, 256)
    b = mx.q_gemm_dequant(x, packed, 384, 512, 1024, mx.QuantType.Q4_K, 256)
    assert torch.equal(a, b)
