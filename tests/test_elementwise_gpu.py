"""RMSNorm, SwiGLU and RoPE through the C ABI vs the oracle.  RMSNorm uses the reference
test's own closeness rule |a-b| <= atol + rtol*|b| with its tolerances
(tests/unit/rmsnorm_primitive_test.cpp:36-52, :76, :141, :198)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def arrays_close(a, b, rtol, atol):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return bool(np.all(np.abs(a - b) <= atol + rtol * np.abs(b)))


def _rms(oracle, shape, dtype, eps, seed, scale=1.0, residual=False):
    import mlxr_b200 as mx
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(shape, generator=g) * scale).to(dtype)
    w = (1 + 0.1 * torch.randn(shape[-1], generator=g)).to(dtype)
    r = torch.randn(shape, generator=g).to(dtype) if residual else None
    y = mx.rmsnorm_fused(x.cuda(), w.cuda(), eps, r.cuda() if residual else None).float().cpu().numpy()
    ref = oracle.rmsnorm(x.float().numpy(), w.float().numpy(), eps)
    if residual:
        ref = ref + r.float().numpy()
    return y, ref


@pytest.mark.parametrize("hidden", [32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 100, 5000, 12288])
def test_rmsnorm_fp32_hidden_sizes(oracle, hidden):
    y, ref = _rms(oracle, (4, hidden), torch.float32, 1e-6, hidden)
    assert arrays_close(y, ref, 1e-4, 1e-5)


@pytest.mark.parametrize("batch", [1, 2, 4, 8, 16, 32])
def test_rmsnorm_batch_sizes(oracle, batch):
    y, ref = _rms(oracle, (batch, 16, 128), torch.float32, 1e-6, batch)
    assert arrays_close(y, ref, 1e-4, 1e-5)


@pytest.mark.parametrize("eps", [1e-8, 1e-6, 1e-5, 1e-4, 1e-2])
def test_rmsnorm_eps(oracle, eps):
    y, ref = _rms(oracle, (2, 8, 128), torch.float32, eps, 3)
    assert arrays_close(y, ref, 1e-4, 1e-5)


def test_rmsnorm_fp16_bf16(oracle):
    y, ref = _rms(oracle, (2, 8, 4096), torch.float16, 1e-5, 4)
    assert arrays_close(y, ref, 1e-2, 1e-3)
    y, ref = _rms(oracle, (2, 8, 4096), torch.bfloat16, 1e-5, 4)
    assert arrays_close(y, ref, 2e-2, 1e-2)


def test_rmsnorm_large_values_and_residual(oracle):
    y, ref = _rms(oracle, (2, 8, 128), torch.float32, 1e-6, 5, scale=100.0)
    assert arrays_close(y, ref, 1e-3, 1e-4)
    y, ref = _rms(oracle, (3, 2048), torch.float32, 1e-6, 6, residual=True)
    assert arrays_close(y, ref, 1e-4, 1e-5)


def test_rmsnorm_non_contiguous_and_errors(oracle):
    import mlxr_b200 as mx
    x = torch.randn(8, 4, 128, device="cuda").transpose(0, 1)  # non-contiguous
    w = torch.ones(128, device="cuda")
    y = mx.rmsnorm_fused(x, w, 1e-6)
    ref = oracle.rmsnorm(x.contiguous().cpu().numpy(), w.cpu().numpy(), 1e-6)
    assert arrays_close(y.cpu().numpy(), ref, 1e-4, 1e-5)
    with pytest.raises(ValueError):
        mx.rmsnorm_fused(x, torch.ones(64, device="cuda"))
    with pytest.raises(ValueError):
        mx.rmsnorm_fused(x, torch.ones(2, 64, device="cuda"))
    # [16, 512, 4096] sanity: finite, unit RMS before the weight
    big = torch.randn(16, 512, 4096, device="cuda", dtype=torch.float16)
    out = mx.rmsnorm_fused(big, torch.ones(4096, device="cuda", dtype=torch.float16), 1e-5)
    assert torch.isfinite(out).all()
    assert abs(out.float().pow(2).mean().sqrt().item() - 1.0) < 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_swiglu(oracle, dtype):
    import mlxr_b200 as mx
    g = (torch.randn(3, 5632) * 3).to(dtype)
    u = torch.randn(3, 5632).to(dtype)
    g[0, :4] = torch.tensor([-100.0, 100.0, 0.0, -20.0]).to(dtype)  # saturating sigmoid
    h = mx.swiglu(g.cuda(), u.cuda()).float().cpu().numpy()
    ref = oracle.swiglu(g.float().numpy(), u.float().numpy())
    ref = oracle.round_to(ref, {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[dtype])
    assert arrays_close(h, ref, 1e-2 if dtype != torch.float32 else 1e-5, 1e-6)
    s = mx.swish(g.cuda()).float().cpu().numpy()
    ref_s = oracle.swiglu(g.float().numpy(), np.ones_like(g.float().numpy()))
    assert arrays_close(s, ref_s, 1e-2 if dtype != torch.float32 else 1e-5, 1e-6)


def test_rope_tables_bit_exact(oracle):
    """compute_rope_tables vs the oracle (same libm, same rounding): identical bits."""
    import mlxr_b200 as mx
    for base, d in ((10000.0, 64), (500000.0, 128)):
        c, s = mx.compute_rope_tables(512, d, base)
        co, so = oracle.rope_tables(512, d, base)
        assert np.array_equal(c.numpy().view(np.uint16), co)
        assert np.array_equal(s.numpy().view(np.uint16), so)
    c, s = mx.compute_rope_tables(64, 32, 10000.0, mx.RoPEScalingMode.LINEAR, 4.0)
    co, so = oracle.rope_tables(64, 32, 10000.0, 3, 4.0)
    assert np.array_equal(c.numpy().view(np.uint16), co) and np.array_equal(s.numpy().view(np.uint16), so)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("layout", ["3d", "4d"])
def test_rope_apply(oracle, dtype, layout):
    import mlxr_b200 as mx
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[dtype]
    heads, d, max_seq = 8, 128, 8192
    cos, sin = mx.compute_rope_tables(max_seq, d, 500000.0)
    g = torch.Generator().manual_seed(1)
    if layout == "3d":
        x = torch.randn(13, heads, d, generator=g).to(dtype)
        pos = torch.randint(0, max_seq, (13,), generator=g, dtype=torch.int32)
        x4 = x.unsqueeze(1)
    else:
        x = torch.randn(3, 5, heads, d, generator=g).to(dtype)
        pos = torch.randint(0, max_seq, (3, 5), generator=g, dtype=torch.int32)
        x4 = x
    y = mx.rope_apply(x.cuda(), cos.cuda(), sin.cuda(), pos.cuda())
    ref = oracle.rope_apply(x4.float().numpy(), cos.numpy().view(np.uint16), sin.numpy().view(np.uint16), pos.numpy())
    ref = oracle.round_to(ref, code).reshape(x.shape)
    # same fp32 operations in the same order, one rounding: identical values
    assert np.array_equal(y.float().cpu().numpy(), ref)
    # in place and LINEAR scaling with an offset
    x2 = x.clone().cuda()
    out = mx.rope_apply(x2, cos.cuda(), sin.cuda(), (pos // 2).cuda(), mx.RoPEScalingMode.LINEAR, 0.5, 3, inplace=True)
    assert out.data_ptr() == x2.data_ptr()
    ref2 = oracle.rope_apply(x4.float().numpy(), cos.numpy().view(np.uint16), sin.numpy().view(np.uint16),
                             (pos // 2).numpy(), 3, 0.5, 3)
    assert np.array_equal(x2.float().cpu().numpy(), oracle.round_to(ref2, code).reshape(x.shape))


def test_rope_errors():
    import mlxr_b200 as mx
    from mlxr_b200._capi import MlxrError
    cos, sin = mx.compute_rope_tables(16, 8)
    cos, sin = cos.cuda(), sin.cuda()
    x = torch.zeros(2, 4, 8, device="cuda", dtype=torch.float16)
    with pytest.raises(MlxrError, match="positions must have shape"):
        mx.rope_apply(x, cos, sin, torch.zeros(3, dtype=torch.int32, device="cuda"))
    with pytest.raises(MlxrError, match="cos_table must have shape"):
        mx.rope_apply(x, cos[:, :2].contiguous(), sin, torch.zeros(2, dtype=torch.int32, device="cuda"))
    with pytest.raises(MlxrError, match="outside"):
        mx.rope_apply(x, cos, sin, torch.tensor([0, 16], dtype=torch.int32, device="cuda"))
    with pytest.raises(MlxrError, match="3D"):
        mx.rope_apply(x[0], cos, sin, torch.zeros(2, dtype=torch.int32, device="cuda"))


def test_swiglu_mlp_dense_matches_composition():
    """swiglu_mlp() with dense weights and biases (swiglu_mlp_primitive.mm:47-82) against the
    same chain in float64."""
    import mlxr_b200 as mx
    g = torch.Generator().manual_seed(5)
    M, H, I = 3, 96, 224
    x = torch.randn(M, H, generator=g)
    wg, wu, wd = (torch.randn(I, H, generator=g) * 0.1, torch.randn(I, H, generator=g) * 0.1,
                  torch.randn(H, I, generator=g) * 0.1)
    bg, bu, bd = torch.randn(I, generator=g) * 0.1, torch.randn(I, generator=g) * 0.1, torch.randn(H, generator=g) * 0.1
    y = mx.swiglu_mlp(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda(), bg.cuda(), bu.cuda(), bd.cuda()).cpu().double()
    xd = x.double()
    gt = xd @ wg.double().T + bg.double()
    ut = xd @ wu.double().T + bu.double()
    want = (gt * torch.sigmoid(gt) * ut) @ wd.double().T + bd.double()
    assert float((y - want).norm() / want.norm()) < 1e-5
    with pytest.raises(ValueError):
        mx.swiglu_mlp(x.cuda(), wg.cuda(), wu.cuda()[:, :8].contiguous(), wd.cuda())
