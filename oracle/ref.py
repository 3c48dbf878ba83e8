"""ctypes wrapper of oracle/_ref/libmlxr_ref.so: the reference's own host code for this
path (q_gemm_dequant_primitive.mm, rope_apply_primitive.mm and the dequantizers of
q_gemm_dequant.metal), compiled from the MLXR tree by oracle/Makefile.

TEST INFRASTRUCTURE ONLY.  available() is False where the library was not built (the
MLXR tree is absent); callers then rely on the committed fixtures under tests/golden/.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libmlxr_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        l = C.CDLL(LIB_PATH)
        vp, i, f = C.c_void_p, C.c_int, C.c_float
        l.ref_last_error.restype = C.c_char_p
        l.ref_cpu_dequant.argtypes = [i, vp, C.c_long, vp]
        l.ref_shader_dequant.argtypes = [i, vp, C.c_long, vp]
        l.ref_weight_size.restype = C.c_size_t
        l.ref_weight_size.argtypes = [i, i, i]
        l.ref_bytes_per_weight.restype = f
        l.ref_bytes_per_weight.argtypes = [i]
        l.ref_default_group_size.argtypes = [i]
        l.ref_quant_type_name.restype = C.c_char_p
        l.ref_quant_type_name.argtypes = [i]
        l.ref_rope_mode_name.restype = C.c_char_p
        l.ref_rope_mode_name.argtypes = [i]
        l.ref_ntk_base.restype = f
        l.ref_ntk_base.argtypes = [f, f, i, i]
        l.ref_qgemm_cpu.argtypes = [vp, vp, vp, vp, i, i, i, i, i]
        l.ref_rope_tables.argtypes = [i, i, f, i, f, i, vp, vp]
        l.ref_rope_apply_cpu.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, f, i, i]
        _lib = l
    return _lib


def cpu_dequant(qt: int, packed: np.ndarray, nblocks: int) -> np.ndarray:
    """dequant_q4_0_cpu / _q4_1_cpu / _q8_0_cpu -> fp32 [nblocks*32]"""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(nblocks * 32, dtype=np.float32)
    if lib().ref_cpu_dequant(qt, packed.ctypes.data, nblocks, out.ctypes.data):
        raise ValueError("reference has no CPU dequantizer for this format")
    return out


def shader_dequant(qt: int, packed: np.ndarray, nblocks: int) -> np.ndarray:
    """shader dequant_q4_0/_q4_1/_q8_0/_q4_k -> binary16 bits"""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    per = 256 if qt == 3 else 32
    out = np.empty(nblocks * per, dtype=np.uint16)
    if lib().ref_shader_dequant(qt, packed.ctypes.data, nblocks, out.ctypes.data):
        raise ValueError("reference shader has no dequantizer for this format")
    return out


def qgemm_cpu(x: np.ndarray, packed: np.ndarray, N: int, qt: int, group_size: int, bias=None) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, K = x.shape
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    y = np.empty((M, N), dtype=np.float32)
    b = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
    rc = lib().ref_qgemm_cpu(x.ctypes.data, packed.ctypes.data, b.ctypes.data if b is not None else None,
                             y.ctypes.data, M, N, K, qt, group_size)
    if rc:
        raise RuntimeError(lib().ref_last_error().decode())
    return y


def rope_tables(max_seq: int, head_dim: int, base=10000.0, mode=0, scale=1.0, orig_ctx=2048):
    c = np.empty((max_seq, head_dim // 2), dtype=np.uint16)
    s = np.empty_like(c)
    if lib().ref_rope_tables(max_seq, head_dim, base, mode, scale, orig_ctx, c.ctypes.data, s.ctypes.data):
        raise RuntimeError(lib().ref_last_error().decode())
    return c, s


def rope_apply_cpu(x: np.ndarray, cos_f: np.ndarray, sin_f: np.ndarray, pos: np.ndarray, mode=0, scale=1.0,
                   offset=0, inplace=False) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    cos_f = np.ascontiguousarray(cos_f, dtype=np.float32)
    sin_f = np.ascontiguousarray(sin_f, dtype=np.float32)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    if x.ndim == 3:
        batch, heads, d = x.shape
        seq = 1
    else:
        batch, seq, heads, d = x.shape
    y = np.empty_like(x)
    rc = lib().ref_rope_apply_cpu(x.ctypes.data, cos_f.ctypes.data, sin_f.ctypes.data, pos.ctypes.data, y.ctypes.data,
                                  x.ndim, batch, seq, heads, d, cos_f.shape[0], mode, scale, offset, int(inplace))
    if rc:
        raise RuntimeError(lib().ref_last_error().decode())
    return y
