"""Python face of the test oracle: ctypes wrapper of liboracle.so plus NumPy compositions.

TEST INFRASTRUCTURE ONLY -- imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs; the product never imports it.

The C side (mlxr_oracle.c) restates the reference function by function; the compositions
here restate the MLX-op chains of core/graph/layers.cpp (RMSNorm :39-55, Linear :86-99,
MLP :400-420) and swiglu_mlp_primitive.mm:47-82: every linear is x @ dequant(W)^T with
fp32 accumulation, and values are rounded to the activation dtype where the chain
materialises an array (after RMSNorm, after each linear, after SiLU(g)*u).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")

Q4_0, Q4_1, Q8_0, Q4_K, Q6_K, NF4 = 0, 1, 2, 3, 4, 16
F16, BF16, F32 = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile liboracle.so (and oracle/_ref when the MLXR tree is present)."""
    src = os.path.join(_HERE, "mlxr_oracle.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return _LIB


def _load() -> C.CDLL:
    build()
    lib = C.CDLL(_LIB)
    vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    lib.orc_fp16_to_fp32.restype = f
    lib.orc_fp16_to_fp32.argtypes = [C.c_uint16]
    lib.orc_fp32_to_fp16.restype = C.c_uint16
    lib.orc_fp32_to_fp16.argtypes = [f]
    lib.orc_block_elems.argtypes = [i]
    lib.orc_block_bytes.argtypes = [i]
    lib.orc_quantized_weight_size.restype = sz
    lib.orc_quantized_weight_size.argtypes = [i, i, i]
    lib.orc_dequantize.argtypes = [i, vp, i, i, vp, vp, i]
    lib.orc_qgemm_cpu.argtypes = [vp, vp, vp, vp, i, i, i, i]
    lib.orc_gemm_rows_f32.restype = None
    lib.orc_gemm_rows_f32.argtypes = [vp, vp, vp, i, i, i, i, i]
    lib.orc_rmsnorm.restype = None
    lib.orc_rmsnorm.argtypes = [vp, vp, vp, i, i, f]
    lib.orc_swiglu.restype = None
    lib.orc_swiglu.argtypes = [vp, vp, vp, sz]
    lib.orc_rope_tables.restype = None
    lib.orc_rope_tables.argtypes = [i, i, f, i, f, vp, vp, vp, vp]
    lib.orc_rope_apply.restype = None
    lib.orc_rope_apply.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, f, i]
    lib.orc_rope_tables_f32.restype = None
    lib.orc_rope_tables_f32.argtypes = [i, i, f, vp, vp]
    lib.orc_rope_split_half.restype = None
    lib.orc_rope_split_half.argtypes = [vp, vp, vp, vp, i, i, i, i, i]
    lib.orc_round_to.restype = None
    lib.orc_round_to.argtypes = [vp, sz, i]
    lib.orc_nf4_codebook.restype = C.POINTER(C.c_float)
    return lib


lib = _load()


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def block_elems(qt: int) -> int:
    return lib.orc_block_elems(qt)


def block_bytes(qt: int) -> int:
    return lib.orc_block_bytes(qt)


def quantized_weight_size(N: int, K: int, qt: int) -> int:
    return lib.orc_quantized_weight_size(N, K, qt)


def nf4_codebook() -> np.ndarray:
    return np.ctypeslib.as_array(lib.orc_nf4_codebook(), shape=(16,)).copy()


def dequantize(w: np.ndarray, N: int, K: int, qt: int, fused: bool = False):
    """-> (fp32 [N,K], fp16-bits uint16 [N,K]) exactly as the reference's dequantizers."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    assert w.size >= quantized_weight_size(N, K, qt), "weight buffer too small"
    f = np.empty((N, K), dtype=np.float32)
    h = np.empty((N, K), dtype=np.uint16)
    rc = lib.orc_dequantize(qt, w.ctypes.data, N, K, f.ctypes.data, h.ctypes.data, 1 if fused else 0)
    if rc:
        raise ValueError(f"oracle: cannot dequantize qt={qt} K={K}")
    return f, h


def qgemm_cpu(x: np.ndarray, w: np.ndarray, N: int, qt: int, bias=None) -> np.ndarray:
    """eval_cpu restated: full dequant then the sequential-k fp32 triple loop."""
    x = _f32(x)
    M, K = x.shape
    w = np.ascontiguousarray(w, dtype=np.uint8)
    y = np.empty((M, N), dtype=np.float32)
    b = _f32(bias) if bias is not None else None
    rc = lib.orc_qgemm_cpu(x.ctypes.data, w.ctypes.data, b.ctypes.data if b is not None else None,
                           y.ctypes.data, M, N, K, qt)
    if rc:
        raise ValueError("oracle qgemm failed")
    return y


def round_to(a: np.ndarray, dtype: int) -> np.ndarray:
    a = _f32(a).copy()
    lib.orc_round_to(a.ctypes.data, a.size, dtype)
    return a


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = _f32(x)
    hidden = x.shape[-1]
    y = np.empty_like(x)
    lib.orc_rmsnorm(x.ctypes.data, _f32(w).ctypes.data, y.ctypes.data, x.size // hidden, hidden, eps)
    return y


def swiglu(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    g, u = _f32(g), _f32(u)
    h = np.empty_like(g)
    lib.orc_swiglu(g.ctypes.data, u.ctypes.data, h.ctypes.data, g.size)
    return h


def rope_tables(max_seq: int, head_dim: int, base: float = 10000.0, mode: int = 0, scale: float = 1.0):
    """-> (cos fp16-bits, sin fp16-bits) as uint16 [max_seq, head_dim/2]"""
    c = np.empty((max_seq, head_dim // 2), dtype=np.uint16)
    s = np.empty_like(c)
    lib.orc_rope_tables(max_seq, head_dim, base, mode, scale, c.ctypes.data, s.ctypes.data, None, None)
    return c, s


def rope_apply(x: np.ndarray, cos_h: np.ndarray, sin_h: np.ndarray, positions: np.ndarray,
               mode: int = 0, scale: float = 1.0, offset: int = 0) -> np.ndarray:
    """x [batch, seq, heads, d] fp32; tables as fp16 bits (uint16) or float16."""
    x = _f32(x)
    batch, seq, heads, d = x.shape
    cf = _f32(np.asarray(cos_h).view(np.float16))
    sf = _f32(np.asarray(sin_h).view(np.float16))
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    y = np.empty_like(x)
    lib.orc_rope_apply(x.ctypes.data, cf.ctypes.data, sf.ctypes.data, pos.ctypes.data, y.ctypes.data,
                       batch, seq, heads, d, mode, scale, offset)
    return y


def rope_tables_f32(max_seq: int, dim: int, base: float = 10000.0):
    """-> (cos, sin) float32 [max_seq, dim/2] as graph::RotaryEmbedding::compute_freqs builds them."""
    c = np.empty((max_seq, dim // 2), dtype=np.float32)
    s = np.empty_like(c)
    lib.orc_rope_tables_f32(max_seq, dim, base, c.ctypes.data, s.ctypes.data)
    return c, s


def rope_split_half(x: np.ndarray, cos_f: np.ndarray, sin_f: np.ndarray, offset: int = 0) -> np.ndarray:
    """x [batch, seq, heads, d] fp32; split-half rotation of graph::RotaryEmbedding::forward."""
    x = _f32(x)
    batch, seq, heads, d = x.shape
    y = np.empty_like(x)
    lib.orc_rope_split_half(x.ctypes.data, _f32(cos_f).ctypes.data, _f32(sin_f).ctypes.data, y.ctypes.data,
                            batch, seq, heads, d, offset)
    return y


# ---- compositions (NumPy; BLAS does the fp32 matmul so full-size cases finish in seconds) ----

def linear(x: np.ndarray, w: np.ndarray, N: int, qt: int, bias=None) -> np.ndarray:
    """x @ dequant(W)^T in fp32 (summation order is BLAS's, not eval_cpu's: use
    qgemm_cpu for the order-faithful loop on small cases)."""
    x = _f32(x)
    wd, _ = dequantize(w, N, x.shape[1], qt)
    y = x @ wd.T
    if bias is not None:
        y = y + _f32(bias)
    return y.astype(np.float32)


def mlp_block(x, norm_w, wg, wu, wd, inter: int, qt: int, eps: float, dtype: int) -> np.ndarray:
    """RMSNorm -> gate/up -> SiLU(g)*u -> down, rounding to `dtype` at each materialised
    array.  x: [M, hidden] values already representable in `dtype`."""
    x = _f32(x)
    hidden = x.shape[1]
    n = round_to(rmsnorm(x, norm_w, eps), dtype) if norm_w is not None else x
    g = round_to(linear(n, wg, inter, qt), dtype)
    u = round_to(linear(n, wu, inter, qt), dtype)
    h = round_to(swiglu(g, u), dtype)
    return round_to(linear(h, wd, hidden, qt), dtype)


def mlp_block_partial(x, norm_w, wg_s, wu_s, wd_s, inter_local: int, qt: int, eps: float, dtype: int) -> np.ndarray:
    """One rank's unrounded partial of the tensor-parallel block: the shard's gate/up rows give
    its slice of h (rounded to `dtype` like the whole h), the shard of down multiplies it; the
    float32 sums are returned as they are.  Summed over ranks and rounded, this is mlp_block up
    to float32 summation order."""
    x = _f32(x)
    hidden = x.shape[1]
    n = round_to(rmsnorm(x, norm_w, eps), dtype) if norm_w is not None else x
    g = round_to(linear(n, wg_s, inter_local, qt), dtype)
    u = round_to(linear(n, wu_s, inter_local, qt), dtype)
    h = round_to(swiglu(g, u), dtype)
    return linear(h, wd_s, hidden, qt)


def mlp_block_f64(x, norm_w, wg, wu, wd, inter: int, qt: int, eps: float) -> np.ndarray:
    """Same chain in float64 with no intermediate rounding: the 'truth' both the fp32
    oracle and the GPU are measured against in the relative-L2 gate."""
    x = np.asarray(x, dtype=np.float64)
    hidden = x.shape[1]
    if norm_w is not None:
        x = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * np.asarray(norm_w, dtype=np.float64)
    dq = lambda w, N, K: dequantize(w, N, K, qt)[0].astype(np.float64)
    g = x @ dq(wg, inter, hidden).T
    u = x @ dq(wu, inter, hidden).T
    h = g / (1.0 + np.exp(-g)) * u
    return h @ dq(wd, hidden, inter).T


def qkv_rope(x, norm_w, wq, wk, wv, cos_h, sin_h, positions, q_heads, kv_heads, head_dim, qt, eps,
             dtype, offset=0):
    x = _f32(x)
    M = x.shape[0]
    n = round_to(rmsnorm(x, norm_w, eps), dtype) if norm_w is not None else x
    q = round_to(linear(n, wq, q_heads * head_dim, qt), dtype).reshape(M, 1, q_heads, head_dim)
    k = round_to(linear(n, wk, kv_heads * head_dim, qt), dtype).reshape(M, 1, kv_heads, head_dim)
    v = round_to(linear(n, wv, kv_heads * head_dim, qt), dtype).reshape(M, kv_heads, head_dim)
    q = round_to(rope_apply(q, cos_h, sin_h, positions, 0, 1.0, offset), dtype).reshape(M, q_heads, head_dim)
    k = round_to(rope_apply(k, cos_h, sin_h, positions, 0, 1.0, offset), dtype).reshape(M, kv_heads, head_dim)
    return q, k, v


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / (den if den > 0 else 1.0))
