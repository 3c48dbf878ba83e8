"""Pack fp32 weight matrices into MLXR's block layouts (NumPy, host side).

MLXR ships no quantizer (its loader skips quantized tensors), and its layouts differ from
ggml's, so a user of this path needs one: these functions produce byte buffers that the
dequantizers of q_gemm_dequant_primitive.mm:189-225 / q_gemm_dequant.metal:142-259 read
back.  Rounding is to nearest; quality is that of a plain min/max (Q4_K), absmax (Q4_0,
Q8_0, NF4) quantizer.

All functions take w [N, K] float32 and return a uint8 array of
compute_quantized_weight_size(N, K, type) bytes.
"""
from __future__ import annotations

import numpy as np

from .types import QuantType

# the 16 NF4 levels: the table the CUDA kernels include (csrc/nf4_codebook.inc)
_NF4 = None


def nf4_levels() -> np.ndarray:
    global _NF4
    if _NF4 is None:
        import os
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "nf4_codebook.inc")
        vals = []
        with open(path) as f:
            for line in f:
                line = line.strip()
                if line.startswith(("-0x", "0x")):
                    vals.append(float.fromhex(line.split("f,")[0]))
        _NF4 = np.asarray(vals, dtype=np.float32)
        assert _NF4.shape == (16,)
    return _NF4


def _pack_nibbles(q: np.ndarray) -> np.ndarray:
    """q [..., 2n] of values 0..15 -> bytes [..., n]; byte i = q[2i] | q[2i+1] << 4
    (MLXR's interleaved order, q_gemm_dequant_primitive.mm:192-200)."""
    q = q.astype(np.uint8)
    return (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8)


def quantize_q4_0(w: np.ndarray) -> np.ndarray:
    N, K = w.shape
    assert K % 32 == 0
    b = w.reshape(N, K // 32, 32).astype(np.float32)
    amax_idx = np.abs(b).argmax(axis=-1)
    mx = np.take_along_axis(b, amax_idx[..., None], axis=-1)[..., 0]
    d = (mx / -8.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1), 0.0)
    q = np.clip(np.rint(b * inv[..., None]) + 8, 0, 15)
    out = np.empty((N, K // 32, 18), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(N, K // 32, 2)
    out[..., 2:] = _pack_nibbles(q)
    return out.reshape(-1)


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    N, K = w.shape
    assert K % 32 == 0
    b = w.reshape(N, K // 32, 32).astype(np.float32)
    d = (np.abs(b).max(axis=-1) / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1), 0.0)
    q = np.clip(np.rint(b * inv[..., None]), -127, 127).astype(np.int8)
    out = np.empty((N, K // 32, 34), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(N, K // 32, 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_1(w: np.ndarray) -> np.ndarray:
    N, K = w.shape
    assert K % 32 == 0
    b = w.reshape(N, K // 32, 32).astype(np.float32)
    lo, hi = b.min(axis=-1), b.max(axis=-1)
    d = ((hi - lo) / 15.0).astype(np.float16)
    m = lo.astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1), 0.0)
    q = np.clip(np.rint((b - m.astype(np.float32)[..., None]) * inv[..., None]), 0, 15)
    out = np.empty((N, K // 32, 20), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(N, K // 32, 2)
    out[..., 2:4] = m.view(np.uint8).reshape(N, K // 32, 2)
    out[..., 4:] = _pack_nibbles(q)
    return out.reshape(-1)


def quantize_nf4(w: np.ndarray) -> np.ndarray:
    N, K = w.shape
    assert K % 64 == 0
    lv = nf4_levels()
    b = w.reshape(N, K // 64, 64).astype(np.float32)
    a = np.abs(b).max(axis=-1).astype(np.float16)
    af = a.astype(np.float32)
    inv = np.where(af != 0, 1.0 / np.where(af != 0, af, 1), 0.0)
    xn = b * inv[..., None]
    mid = (lv[1:] + lv[:-1]) * 0.5
    idx = np.searchsorted(mid, xn)
    out = np.empty((N, K // 64, 34), dtype=np.uint8)
    out[..., 0:2] = a.view(np.uint8).reshape(N, K // 64, 2)
    out[..., 2:] = _pack_nibbles(idx)
    return out.reshape(-1)


# Sub-blocks that share one (scale, min) pair in MLXR's Q4_K dequantizer
# (q_gemm_dequant.metal:233-242: offsets 2 and 3 of each group of four reuse offset 0).
_Q4K_GROUPS = ((0, 2, 3), (1,), (4, 6, 7), (5,))


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    """MLXR-layout Q4_K: w ~ (q - 8) * (sc * d) + (m * dmin), q in 0..15, sc and m 6-bit,
    with the four (sc, m) pairs a super-block really has under MLXR's unpacking:
    pair 0 -> sub-blocks 0,2,3; pair 1 -> 1; pair 2 -> 4,6,7; pair 3 -> 5."""
    N, K = w.shape
    assert K % 256 == 0
    nb = K // 256
    b = w.reshape(N, nb, 8, 32).astype(np.float32)
    # per pair: range over the sub-blocks that share it
    lo = np.stack([b[:, :, list(g), :].min(axis=(-1, -2)) for g in _Q4K_GROUPS], axis=-1)
    hi = np.stack([b[:, :, list(g), :].max(axis=(-1, -2)) for g in _Q4K_GROUPS], axis=-1)
    ss_want = np.maximum((hi - lo) / 15.0, 1e-12)          # (q - 8) spans -8..7
    sm_want = lo + 8.0 * ss_want                            # value at q = 8
    d = (ss_want.max(axis=-1) / 63.0).astype(np.float16)
    df = np.maximum(d.astype(np.float32), 1e-12)
    sc = np.clip(np.rint(ss_want / df[..., None]), 1, 63).astype(np.uint8)
    # one dmin (with sign) for the four mins: sign of the largest |min|
    j = np.abs(sm_want).argmax(axis=-1)
    big = np.take_along_axis(sm_want, j[..., None], axis=-1)[..., 0]
    dmin = (big / 63.0).astype(np.float16)
    dmf = dmin.astype(np.float32)
    inv = np.where(dmf != 0, 1.0 / np.where(dmf != 0, dmf, 1), 0.0)
    mn = np.clip(np.rint(sm_want * inv[..., None]), 0, 63).astype(np.uint8)
    # effective half-precision sub-scale / sub-min, as the dequantizer forms them
    ss = (sc.astype(np.float16) * d[..., None]).astype(np.float32)
    sm = (mn.astype(np.float16) * dmin[..., None]).astype(np.float32)
    pair_of = np.array([0, 1, 0, 0, 2, 3, 2, 2])
    ss_s = ss[..., pair_of]                                 # [N, nb, 8]
    sm_s = sm[..., pair_of]
    q = np.clip(np.rint((b - sm_s[..., None]) / np.maximum(ss_s[..., None], 1e-12)) + 8, 0, 15)
    out = np.zeros((N, nb, 144), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(N, nb, 2)
    out[..., 2:4] = dmin.view(np.uint8).reshape(N, nb, 2)
    # 6-bit packing read by the shader: group g uses scales[3g .. 3g+2]
    for g in range(2):
        s0, m0 = sc[..., 2 * g].astype(np.uint32), mn[..., 2 * g].astype(np.uint32)
        s1, m1 = sc[..., 2 * g + 1].astype(np.uint32), mn[..., 2 * g + 1].astype(np.uint32)
        b0 = (s0 & 63) | ((m0 & 3) << 6)
        b1 = ((m0 >> 2) & 15) | ((s1 & 15) << 4)
        b2 = ((s1 >> 4) & 3) | ((m1 & 63) << 2)
        out[..., 4 + 3 * g + 0] = b0
        out[..., 4 + 3 * g + 1] = b1
        out[..., 4 + 3 * g + 2] = b2
    out[..., 16:] = _pack_nibbles(q.reshape(N, nb, 256))
    return out.reshape(-1)


def quantize(w: np.ndarray, quant_type: QuantType) -> np.ndarray:
    fn = {QuantType.Q4_0: quantize_q4_0, QuantType.Q4_1: quantize_q4_1, QuantType.Q8_0: quantize_q8_0,
          QuantType.Q4_K: quantize_q4_k, QuantType.NF4: quantize_nf4}.get(QuantType(quant_type))
    if fn is None:
        raise ValueError(f"no quantizer for {QuantType(quant_type).name}")
    return fn(np.ascontiguousarray(w, dtype=np.float32))
