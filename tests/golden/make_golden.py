"""Generate the golden fixtures of tests/golden/ by running the REFERENCE's own code
(oracle/_ref, compiled from the MLXR tree by oracle/Makefile) on seeded inputs.

    make -C oracle && python tests/golden/make_golden.py

Needs the MLXR tree (to build oracle/_ref); the fixtures it writes are committed so that
tests can check the oracle and the CUDA path where the tree is absent.

  dequant_qt{0,1,2,3}.npz  packed blocks (fuzzed bytes with finite scales + hand-made edge
                           blocks), h16 = shader dequantizer output bits, f32 = CPU
                           dequantizer output (Q4_0/Q4_1/Q8_0 only: Q4_K has no CPU twin)
  dequant_qt16.npz         NF4: no reference code exists; outputs are the oracle's
                           (self-consistency fixture, "parity unpinned")
  qgemm_cpu.npz            eval_cpu outputs for small Q4_0/Q4_1/Q8_0 problems
  rope.npz                 compute_rope_tables + rope_apply eval_cpu outputs
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

from conftest import fuzz_blocks, make_weights  # noqa: E402
from oracle import oracle as O, ref as R  # noqa: E402
from mlxr_b200.quantize import quantize  # noqa: E402


def edge_blocks(qt):
    """Hand-made blocks: all-zero / all-0xF nibbles, scales 1.0, -2.0, smallest subnormal, 0,
    largest finite; for Q4_K distinct scales[0..5] and non-zero scales[6..11] (never read)."""
    bb = O.block_bytes(qt)
    scales = [0x3C00, 0xC000, 0x0001, 0x0000, 0x7BFF, 0x8000, 0x2E66]
    out = []
    for i, sc in enumerate(scales):
        for fill in (0x00, 0xFF, 0x80, 0x7F, 0x5A):
            b = np.full(bb, fill, dtype=np.uint8)
            b[0], b[1] = sc & 255, sc >> 8
            if qt in (O.Q4_1, O.Q4_K):
                m = scales[(i + 3) % len(scales)]
                b[2], b[3] = m & 255, m >> 8
            if qt == O.Q4_K:
                b[4:16] = np.array([0xC5, 0x9A, 0x7D, 0x23, 0xF1, 0x08, 0xFF, 0x01, 0xAA, 0x55, 0x3C, 0xE7], dtype=np.uint8)
                b[16:] = (np.arange(128) * 37 + fill) & 255
            out.append(b)
    return np.concatenate(out)


def main():
    assert R.available(), "build oracle/_ref first (make -C oracle)"
    for qt in (O.Q4_0, O.Q4_1, O.Q8_0, O.Q4_K, O.NF4):
        be, bb = O.block_elems(qt), O.block_bytes(qt)
        packed = np.concatenate([edge_blocks(qt), fuzz_blocks(qt, 93, 9000 + qt)])
        nb = packed.size // bb
        nb -= nb % 4
        packed = packed[: nb * bb]
        N, K = 4, (nb // 4) * be
        d = dict(packed=packed, N=N, K=K)
        if qt == O.NF4:
            f, h = O.dequantize(packed, N, K, qt)
            d.update(h16=h, f32=f, source="oracle (no reference code for NF4)")
        else:
            d["h16"] = R.shader_dequant(qt, packed, nb).reshape(N, K)
            d["source"] = "reference shader dequant_* compiled as C++"
            if qt != O.Q4_K:
                d["f32"] = R.cpu_dequant(qt, packed, nb).reshape(N, K)
        np.savez_compressed(os.path.join(HERE, f"dequant_qt{qt}.npz"), **d)

    g = {}
    rng = np.random.Generator(np.random.PCG64(77))
    for qt in (O.Q4_0, O.Q4_1, O.Q8_0):
        M, N, K = 3, 20, 160
        packed = quantize(make_weights(N, K, 500 + qt), qt)
        x = rng.standard_normal((M, K)).astype(np.float32)
        b = rng.standard_normal(N).astype(np.float32)
        g[f"w{qt}"], g[f"x{qt}"], g[f"b{qt}"] = packed, x, b
        g[f"y{qt}"] = R.qgemm_cpu(x, packed, N, qt, 32)
        g[f"yb{qt}"] = R.qgemm_cpu(x, packed, N, qt, 32, b)
    np.savez_compressed(os.path.join(HERE, "qgemm_cpu.npz"), **g)

    r = {}
    for name, (ms, d, base, mode, scale) in dict(llama3=(256, 128, 500000.0, 0, 1.0), tiny=(64, 64, 10000.0, 0, 1.0),
                                                 linear=(64, 32, 10000.0, 3, 4.0), ntk=(32, 16, 10000.0, 1, 8.0)).items():
        c, s = R.rope_tables(ms, d, base, mode, scale)
        r[f"cos_{name}"], r[f"sin_{name}"] = c, s
    x = rng.standard_normal((2, 3, 4, 128)).astype(np.float32)
    pos = rng.integers(0, 250, (2, 3)).astype(np.int32)
    cf = r["cos_llama3"].view(np.float16).astype(np.float32)
    sf = r["sin_llama3"].view(np.float16).astype(np.float32)
    r["x"], r["pos"] = x, pos
    r["y_base"] = R.rope_apply_cpu(x, cf, sf, pos)
    r["y_linear_off"] = R.rope_apply_cpu(x, cf, sf, pos, 3, 0.5, 5)
    x3 = rng.standard_normal((5, 2, 128)).astype(np.float32)
    p3 = rng.integers(0, 256, 5).astype(np.int32)
    r["x3"], r["pos3"] = x3, p3
    r["y3"] = R.rope_apply_cpu(x3, cf, sf, p3)
    np.savez_compressed(os.path.join(HERE, "rope.npz"), **r)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
