"""Small-batch tensor-core linear (Q4_K and Q4_0, 3 <= M <= 64; csrc/smallm.cu) through the C ABI vs the oracle.

Gate 2e-2 relative L2.  The tests use 2e-3 for fp16 activations (the weights are converted with
the shader's own fp16 arithmetic, q_gemm_dequant.metal:244-256) and 1e-2 for bf16 (scale, min and
weight are rounded to bf16: about 3e-3 relative).  Shapes cover every padded batch width (16, 32,
64), N that is not a multiple of the 128-row tile, a single super-block of K, tiles shared by
several CTAs (more work units than one CTA's share) and tiles owned by one CTA."""
import numpy as np
import pytest
import torch

from conftest import make_acts, make_weights

pytestmark = pytest.mark.gpu
DT = {"f16": torch.float16, "bf16": torch.bfloat16}
TIGHT = {"f16": 2e-3, "bf16": 1e-2}


def _status():
    import mlxr_b200 as mx
    st = torch.zeros(1, dtype=torch.int32)
    mx._capi.check(mx._capi.lib.mlxr_stream_status(torch.cuda.current_stream().cuda_stream, st.data_ptr()))
    return int(st[0])


def _run(oracle, M, N, K, dt, bias=False, seed=0, rows=None, twice=False, qt=3):
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    packed = quantize(make_weights(N, K, 100 + seed), qt)
    xt, xf = make_acts(M, K, 200 + seed, DT[dt])
    bt = bf = None
    if bias:
        bt, bf = make_acts(1, N, 300 + seed, DT[dt])
        bt, bf = bt[0].contiguous(), bf[0]
    xd, wd, bd = xt.cuda(), torch.from_numpy(packed).cuda(), (bt.cuda() if bias else None)
    gs = mx._capi.lib.mlxr_default_group_size(qt)
    y = mx.q_gemm_dequant(xd, wd, M, N, K, mx.QuantType(qt), gs, bd)
    if twice:   # the tile counters must have cleared themselves, and the result must not depend on arrival order
        y2 = mx.q_gemm_dequant(xd, wd, M, N, K, mx.QuantType(qt), gs, bd)
        assert torch.equal(y, y2)
    torch.cuda.synchronize()
    assert _status() == 0
    yn = y.float().cpu().numpy()
    if rows is not None:
        return oracle.rel_l2(yn[rows], oracle.linear(xf[rows], packed, N, qt, bf))
    return oracle.rel_l2(yn, oracle.linear(xf, packed, N, qt, bf))


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(3, 128, 256), (4, 130, 512), (8, 1000, 768), (9, 256, 256), (16, 512, 1024),
                                   (17, 384, 1280), (32, 640, 2048), (33, 200, 512), (64, 1024, 1024)])
def test_shapes(oracle, dt, M, N, K):
    assert _run(oracle, M, N, K, dt, seed=M, twice=True) <= TIGHT[dt]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(3, 128, 256), (9, 200, 512), (16, 512, 1024), (33, 384, 1280), (64, 1000, 768)])
def test_q4_0_shapes(oracle, dt, M, N, K):
    """Q4_0: the same 144 bytes per 256 weights of a row, read as eight 18-byte blocks."""
    assert _run(oracle, M, N, K, dt, seed=M + 50, twice=True, qt=0, bias=(N == 200)) <= TIGHT[dt]


def test_q4_0_decode_shape_sampled_rows(oracle):
    assert _run(oracle, 32, 5632, 2048, "f16", rows=np.array([0, 17, 31]), seed=8, twice=True, qt=0) <= TIGHT["f16"]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_bias_and_ragged_rows(oracle, dt):
    assert _run(oracle, 5, 8, 256, dt, bias=True, seed=1) <= TIGHT[dt]
    assert _run(oracle, 48, 257, 768, dt, bias=True, seed=2, twice=True) <= TIGHT[dt]


@pytest.mark.parametrize("M,N,K", [(16, 14336, 4096), (32, 4096, 14336), (64, 28672, 4096)])
def test_decode_shapes_sampled_rows(oracle, M, N, K):
    """Llama-3-8B-shaped linears at small batch: a sample of batch rows against the oracle."""
    rows = np.array([0, M // 2, M - 1])
    assert _run(oracle, M, N, K, "bf16", rows=rows, seed=7, twice=True) <= TIGHT["bf16"]


def test_many_units_per_cta_and_shared_tiles(oracle):
    """N = 148 * 128 + 64 rows and K = 3 super-blocks: every CTA's range of work units crosses a
    tile boundary, so most tiles are summed from two CTAs' partial sums."""
    assert _run(oracle, 12, 148 * 128 + 64, 768, "f16", rows=np.array([0, 5, 11]), seed=9, twice=True) <= TIGHT["f16"]


def test_non_finite_input_propagates():
    """A NaN in one batch row reaches that row's outputs only."""
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    N, K, M = 256, 512, 6
    packed = torch.from_numpy(quantize(make_weights(N, K, 3), 3)).cuda()
    x = torch.randn(M, K).to(torch.bfloat16)
    x[2, 17] = float("nan")
    y = mx.q_gemm_dequant(x.cuda(), packed, M, N, K, mx.QuantType(3), 256, None).float().cpu()
    assert torch.isnan(y[2]).all()
    assert torch.isfinite(y[[0, 1, 3, 4, 5]]).all()


def test_bit_identical_over_many_launches():
    """Launches of different geometry back to back, many times: every result of a shape equals the
    first one bit for bit (tiles shared between CTAs are summed in CTA order, whatever the arrival
    order; a stale barrier phase or a counter left over from another shape would show here)."""
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    shapes = [(64, 1536, 2048), (32, 640, 3584), (9, 1024, 1024)]
    data = []
    for i, (M, N, K) in enumerate(shapes):
        w = torch.from_numpy(quantize(make_weights(N, K, 40 + i), 3)).cuda()
        x = torch.randn(M, K, generator=torch.Generator().manual_seed(i)).to(torch.bfloat16).cuda()
        data.append((x, w, M, N, K, mx.q_gemm_dequant(x, w, M, N, K, mx.QuantType(3), 256, None).clone()))
    for _ in range(60):
        for x, w, M, N, K, first in data:
            assert torch.equal(mx.q_gemm_dequant(x, w, M, N, K, mx.QuantType(3), 256, None), first)
    torch.cuda.synchronize()
    assert _status() == 0
