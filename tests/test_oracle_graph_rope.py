"""The oracle's restatement of graph::RotaryEmbedding (core/graph/layers.cpp:113-225) against an
independent numpy statement of the same formulas.  The MLX ops the reference composes are not
available here, so this is a consistency check of the restatement, not a pin ("parity unpinned")."""
import numpy as np


def test_tables_and_rotation(oracle):
    dim, max_seq, base = 64, 96, 500000.0
    c, s = oracle.rope_tables_f32(max_seq, dim, base)
    i = np.arange(dim // 2, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(base), (np.float32(2.0) * i) / np.float32(dim))).astype(np.float32)
    ang = (np.arange(max_seq, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    assert np.allclose(c, np.cos(ang), atol=1e-4) and np.allclose(s, np.sin(ang), atol=1e-4)
    assert np.array_equal(c[0], np.ones(dim // 2, dtype=np.float32)) and np.array_equal(s[0], np.zeros(dim // 2, dtype=np.float32))
    x = np.random.Generator(np.random.PCG64(3)).standard_normal((2, 5, 3, dim)).astype(np.float32)
    y = oracle.rope_split_half(x, c, s, offset=7)
    x1, x2 = x[..., :dim // 2], x[..., dim // 2:]
    cc, ss = c[7:12][None, :, None, :], s[7:12][None, :, None, :]
    want = np.concatenate([x1 * cc - x2 * ss, x2 * cc + x1 * ss], axis=-1)
    assert np.array_equal(y, want.astype(np.float32))
    # a rotation: the norm of every (x1[p], x2[p]) pair is preserved
    assert np.allclose(y[..., :dim // 2] ** 2 + y[..., dim // 2:] ** 2, x1 ** 2 + x2 ** 2, rtol=1e-5, atol=1e-6)
    # position 0 is the identity
    assert np.array_equal(oracle.rope_split_half(x[:, :1], c, s, offset=0), x[:, :1])
