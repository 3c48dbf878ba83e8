"""Quantized GEMM / GEMV through the C ABI vs the oracle (fp32 accumulate).
Gate: relative L2 <= 2e-2 against the oracle's composition; in practice the error is the
output rounding (fp16 ~5e-4, bf16 ~4e-3)."""
import numpy as np
import pytest
import torch

from conftest import make_acts, make_weights

pytestmark = pytest.mark.gpu

TOL = 2e-2
DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
# f32 is looser than its rounding: the decode kernel carries activations as 16-bit fixed point
# per 256-element block (about 2e-4 relative), still far inside the 2e-2 gate.
DT_TIGHT = {"f16": 2e-3, "bf16": 1e-2, "f32": 1e-3}


def _run(oracle, qt, M, N, K, dt, bias=False, seed=0):
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
    ref = oracle.linear(xf, packed, N, qt, bf)
    err = oracle.rel_l2(y.float().cpu().numpy(), ref)
    return err


@pytest.mark.parametrize("qt", [0, 1, 2, 3, 16])
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("M", [1, 3, 8, 17])
def test_small_shapes(oracle, qt, dt, M):
    err = _run(oracle, qt, M, 96, 512, dt, seed=M)
    assert err <= DT_TIGHT[dt], err


@pytest.mark.parametrize("qt", [0, 2, 3, 16])
def test_bias_and_ragged_n(oracle, qt):
    assert _run(oracle, qt, 5, 67, 768, "f16", bias=True) <= DT_TIGHT["f16"]


def test_k_single_block(oracle):
    assert _run(oracle, 0, 2, 9, 32, "f16") <= DT_TIGHT["f16"]
    assert _run(oracle, 3, 2, 9, 256, "bf16") <= DT_TIGHT["bf16"]
    assert _run(oracle, 16, 2, 9, 64, "f16") <= DT_TIGHT["f16"]


def test_q4k_group_size_32_accepted(oracle):
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    packed = torch.from_numpy(quantize(make_weights(16, 256, 1), 3)).cuda()
    x = torch.randn(1, 256, dtype=torch.float16, device="cuda")
    a = mx.q_gemm_dequant(x, packed, 1, 16, 256, mx.QuantType.Q4_K, 32)
    b = mx.q_gemm_dequant(x, packed, 1, 16, 256, mx.QuantType.Q4_K, 256)
    assert torch.equal(a, b)


def test_order_faithful_cpu_loop(oracle):
    """eval_cpu's sequential-k fp32 loop (q_gemm_dequant_primitive.mm:349-364) on a small
    case: the GPU result agrees to fp32 summation-order noise.  K = 480 keeps the call on the
    generic fp32 kernel (the decode kernel, which carries activations as 16-bit fixed point,
    takes multiples of 256 only)."""
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    M, N, K = 4, 40, 480
    for qt in (0, 2):
        packed = quantize(make_weights(N, K, 5), qt)
        xt, xf = make_acts(M, K, 6, torch.float32)
        ref = oracle.qgemm_cpu(xf, packed, N, qt)
        y = mx.q_gemm_dequant(xt.cuda(), torch.from_numpy(packed).cuda(), M, N, K, mx.QuantType(qt), 32)
        assert oracle.rel_l2(y.cpu().numpy(), ref) < 1e-5


def test_empty_batch():
    import mlxr_b200 as mx
    w = torch.zeros(18 * 4, dtype=torch.uint8, device="cuda")
    x = torch.zeros((0, 32), dtype=torch.float16, device="cuda")
    assert mx.q_gemm_dequant(x, w, 0, 4, 32, mx.QuantType.Q4_0, 32).shape == (0, 4)


def test_errors():
    import mlxr_b200 as mx
    from mlxr_b200._capi import MlxrError, MlxrInvalidArgument
    w = torch.zeros(18 * 4, dtype=torch.uint8, device="cuda")
    x = torch.zeros((2, 32), dtype=torch.float16, device="cuda")
    with pytest.raises(MlxrError, match=r"Input shape must be \[M, K\]"):
        mx.q_gemm_dequant(x, w, 3, 4, 32, mx.QuantType.Q4_0, 32)
    with pytest.raises(MlxrError, match=r"Bias shape must be \[N\]"):
        mx.q_gemm_dequant(x, w, 2, 4, 32, mx.QuantType.Q4_0, 32, bias=torch.zeros(5, dtype=torch.float16, device="cuda"))
    with pytest.raises(MlxrError):
        mx.q_gemm_dequant(x, w, 2, 4, 32, mx.QuantType.Q3_K, 32)
    with pytest.raises(MlxrError, match="no CPU path"):
        mx.q_gemm_dequant(x.cpu(), w, 2, 4, 32, mx.QuantType.Q4_0, 32)


@pytest.mark.parametrize("qt", [0, 2, 3, 16])
@pytest.mark.parametrize("M", [1, 16])
def test_format_sweep_full_size(oracle, qt, M):
    """Quant-format sweep linear 14336 x 4096 at decode batch 1 and 16 (bf16)."""
    assert _run(oracle, qt, M, 14336, 4096, "bf16", seed=qt) <= TOL


def test_down_proj_shape(oracle):
    assert _run(oracle, 3, 1, 4096, 14336, "bf16", seed=9) <= TOL
