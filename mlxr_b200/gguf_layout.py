"""Canonical GGML / GGUF block layouts -> MLXR's block layouts (host side, numpy).

MLXR's kernels do not read canonical GGML blocks: its Q4_0 / Q4_1 pack element 2i in the low and
2i+1 in the high nibble of byte i (q_gemm_dequant.metal:142-185), where GGML puts element i in the
low and i+16 in the high nibble, and its Q4_K reads only scales[0..5] with two aliased sub-block
groups (q_gemm_dequant.metal:214-259).  The reference's own loader skips quantized tensors for that
reason (daemon/server/model_loader.cpp:236-245).  This module is the missing step between a
.gguf file (daemon/registry/gguf_parser.h:141-211) and the packed buffers the C ABI takes:

* Q8_0: identical bytes.
* Q4_0, Q4_1: a pure permutation of nibbles: value-preserving, bit-exact.
* Q4_K (and every other K-quant): not expressible in MLXR's reduced Q4_K; `convert(...,
  allow_requantize=True)` dequantizes with gguf.quants and re-quantizes into MLXR's Q4_K
  (lossy; the result says so).

The device side can also read the canonical layouts directly (QuantType.GGML_Q4_0 /
GGML_Q4_K: bit-exact dequantization and the generic quantized linear) and repack canonical Q4_0
into MLXR's Q4_0 on the GPU (ops.repack_ggml_q4_0); `load_linear_raw` hands a tensor's bytes over
unchanged for that.  Nothing in this module runs on the GPU or in the hot path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import numpy as np

from .types import QuantType

# GGML type ids (ggml.h / gguf constants): the ones this module knows
GGML_Q4_0, GGML_Q4_1, GGML_Q8_0, GGML_Q4_K = 2, 3, 8, 12
_BLOCK = {GGML_Q4_0: (32, 18), GGML_Q4_1: (32, 20), GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144)}


@dataclass
class Converted:
    packed: np.ndarray          # uint8, MLXR layout, [N * K/block * block_bytes]
    quant_type: QuantType
    exact: bool                 # True: every dequantized value is unchanged


def _nibble_repack(blocks: np.ndarray, header: int) -> np.ndarray:
    """blocks: [nblocks, header + 16] canonical (element i low nibble of qs[i], i+16 high).
    Returns the MLXR form (byte i = elements 2i low, 2i+1 high)."""
    qs = blocks[:, header:header + 16]
    elems = np.concatenate([qs & 0x0F, qs >> 4], axis=1)          # [nblocks, 32] in element order
    out = blocks.copy()
    out[:, header:header + 16] = (elems[:, 0::2] | (elems[:, 1::2] << 4)).astype(np.uint8)
    return out


def convert(raw: np.ndarray, N: int, K: int, ggml_type: int, allow_requantize: bool = False) -> Converted:
    """raw: the tensor's bytes as stored in a GGUF file (row-major [N rows][K/block blocks])."""
    ggml_type = int(ggml_type)
    if ggml_type not in _BLOCK:
        raise ValueError(f"GGML type {ggml_type} has no conversion")
    be, bb = _BLOCK[ggml_type]
    if K % be != 0:
        raise ValueError(f"K = {K} is not a multiple of the block size {be}")
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    if raw.size != N * (K // be) * bb:
        raise ValueError(f"expected {N * (K // be) * bb} bytes, got {raw.size}")
    if ggml_type == GGML_Q8_0:
        return Converted(raw.copy(), QuantType.Q8_0, True)
    if ggml_type == GGML_Q4_0:
        return Converted(_nibble_repack(raw.reshape(-1, 18), 2).reshape(-1), QuantType.Q4_0, True)
    if ggml_type == GGML_Q4_1:
        return Converted(_nibble_repack(raw.reshape(-1, 20), 4).reshape(-1), QuantType.Q4_1, True)
    # Q4_K: MLXR's reduced format cannot hold eight independent (scale, min) pairs
    if not allow_requantize:
        raise ValueError("canonical Q4_K cannot be repacked exactly into MLXR's Q4_K; pass allow_requantize=True")
    import gguf.quants as gq
    from gguf import GGMLQuantizationType
    from .quantize import quantize
    w = gq.dequantize(raw.reshape(N, -1), GGMLQuantizationType(ggml_type)).astype(np.float32).reshape(N, K)
    return Converted(quantize(w, int(QuantType.Q4_K)), QuantType.Q4_K, False)


def load_linear_raw(path: str, name: str) -> Tuple[np.ndarray, QuantType, int, int]:
    """Read tensor `name` ([N, K]) from a .gguf file WITHOUT conversion: its bytes as stored, the
    canonical-layout quant type the device kernels take for them, N and K."""
    from gguf import GGUFReader
    reader = GGUFReader(path)
    native = {GGML_Q4_0: QuantType.GGML_Q4_0, GGML_Q4_K: QuantType.GGML_Q4_K, GGML_Q8_0: QuantType.Q8_0}
    for t in reader.tensors:
        if t.name == name:
            shape = [int(d) for d in t.shape]          # GGUF stores dimensions innermost first
            if len(shape) != 2:
                raise ValueError(f"{name} is not a matrix (shape {shape})")
            K, N = shape
            gt = int(t.tensor_type)
            if gt not in native:
                raise ValueError(f"GGML type {gt} has no device-side layout")
            return np.ascontiguousarray(np.asarray(t.data)).view(np.uint8).reshape(-1).copy(), native[gt], N, K
    raise KeyError(name)


def load_linear(path: str, name: str, allow_requantize: bool = False) -> Tuple[Converted, int, int]:
    """Read tensor `name` ([N, K], quantized) from a .gguf file and convert it.  Returns
    (converted, N, K)."""
    from gguf import GGUFReader
    reader = GGUFReader(path)
    for t in reader.tensors:
        if t.name == name:
            shape = [int(d) for d in t.shape]          # GGUF stores dimensions innermost first
            if len(shape) != 2:
                raise ValueError(f"{name} is not a matrix (shape {shape})")
            K, N = shape
            return convert(np.asarray(t.data), N, K, int(t.tensor_type), allow_requantize), N, K
    raise KeyError(name)
