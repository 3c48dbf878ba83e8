"""graph::RotaryEmbedding (split-half convention, float32 tables) and the stand-alone dense
graph::Linear through the C ABI vs the oracle restatement of core/graph/layers.cpp:86-99, 113-225."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dim,base", [(128, 500000.0), (64, 10000.0)])
def test_tables_match_the_restatement(oracle, dim, base):
    import mlxr_b200 as mx
    rope = mx.RotaryEmbedding(dim, 512, base)
    c, s = oracle.rope_tables_f32(512, dim, base)
    # the same libm on both sides: identical floats
    assert np.array_equal(rope.cos_table().numpy(), c) and np.array_equal(rope.sin_table().numpy(), s)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 0.0), (torch.float16, 1e-3), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("offset", [0, 37])
def test_forward_matches_the_composition(oracle, dtype, tol, offset):
    import mlxr_b200 as mx
    b, seq, qh, kvh, d = 2, 9, 32, 8, 128
    rope = mx.RotaryEmbedding(d, 128, 500000.0)
    g = np.random.Generator(np.random.PCG64(7))
    q = torch.from_numpy(g.standard_normal((b, seq, qh, d)).astype(np.float32)).to(dtype)
    k = torch.from_numpy(g.standard_normal((b, seq, kvh, d)).astype(np.float32)).to(dtype)
    qr, kr = rope.forward(q.cuda(), k.cuda(), offset)
    torch.cuda.synchronize()
    c, s = oracle.rope_tables_f32(128, d, 500000.0)
    for got, x in ((qr, q), (kr, k)):
        want = oracle.rope_split_half(x.float().numpy(), c, s, offset)
        if tol == 0.0:
            assert np.array_equal(got.cpu().numpy(), want)          # float32: operation for operation
        else:
            assert oracle.rel_l2(got.float().cpu().numpy(), want) <= tol
    # not the interleaved convention of the rope_apply primitive: the two differ on the same input
    cos16, sin16 = mx.compute_rope_tables(128, d, 500000.0)
    pos = torch.arange(offset, offset + seq, dtype=torch.int32).repeat(b, 1)
    inter = mx.rope_apply(q.cuda(), cos16.cuda(), sin16.cuda(), pos.cuda())
    assert not torch.allclose(inter.float(), qr.float(), atol=1e-2)


def test_errors():
    import mlxr_b200 as mx
    from mlxr_b200 import _capi
    with pytest.raises(ValueError):
        mx.RotaryEmbedding(7, 16)
    rope = mx.RotaryEmbedding(8, 16)
    q = torch.zeros(1, 4, 2, 8, device="cuda")
    with pytest.raises(ValueError):
        rope.forward(q[0], q[0])                    # not 4-D
    with pytest.raises(_capi.MlxrError):
        rope.forward(q, q, offset=13)               # positions 13..16 leave the 16-row table


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_dense_linear(dtype, tol):
    import mlxr_b200 as mx
    g = np.random.Generator(np.random.PCG64(9))
    x = torch.from_numpy(g.standard_normal((3, 5, 320)).astype(np.float32)).to(dtype)
    w = torch.from_numpy((g.standard_normal((77, 320)) * 0.05).astype(np.float32)).to(dtype)
    bias = torch.from_numpy(g.standard_normal(77).astype(np.float32)).to(dtype)
    y = mx.linear(x.cuda(), w.cuda(), bias.cuda())
    want = x.double() @ w.double().T + bias.double()
    err = (y.double().cpu() - want).norm() / want.norm()
    assert y.shape == (3, 5, 77) and err <= tol
