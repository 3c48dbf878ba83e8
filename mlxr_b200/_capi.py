"""ctypes binding of lib/libmlxr_b200.so (the C ABI declared in include/mlxr_b200.h).

There is no fallback: if the shared library is missing or does not load, importing this
module raises.  Build it with ``python -m mlxr_b200.build``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MLXR_B200_LIB", os.path.join(_HERE, "lib", "libmlxr_b200.so"))

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: the CUDA library is required (python -m mlxr_b200.build); "
        "mlxr_b200 has no CPU fallback")
lib = C.CDLL(LIB_PATH)

# status codes (mlxr_status)
OK, ERR_INVALID_ARGUMENT, ERR_SHAPE, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_NCCL, ERR_WORKSPACE = range(8)

_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes); every symbol include/mlxr_b200.h declares
PROTOTYPES = {
    "mlxr_version": (C.c_char_p, []),
    "mlxr_status_string": (C.c_char_p, [_i]),
    "mlxr_last_error": (C.c_char_p, []),
    "mlxr_launch_count": (C.c_uint64, []),
    "mlxr_quantized_weight_size": (_sz, [_i, _i, _i]),
    "mlxr_bytes_per_weight": (_f, [_i]),
    "mlxr_default_group_size": (_i, [_i]),
    "mlxr_quant_type_name": (C.c_char_p, [_i]),
    "mlxr_rope_scaling_mode_name": (C.c_char_p, [_i]),
    "mlxr_ntk_scaled_base": (_f, [_f, _f, _i, _i]),
    "mlxr_rope_tables_host": (_i, [_vp, _vp, _i, _i, _f, _i, _f, _i]),
    "mlxr_dequantize": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "mlxr_q_gemm_dequant": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "mlxr_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "mlxr_swiglu": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "mlxr_rope_apply": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp]),
    "mlxr_repack_ggml_q4_0": (_i, [_vp, _vp, _i, _i, _vp]),
    "mlxr_rope_tables_f32_host": (_i, [_vp, _vp, _i, _i, _f]),
    "mlxr_rope_apply_split_half": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "mlxr_linear_dense": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "mlxr_mlp_block": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp]),
    "mlxr_mlp_block_partial_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp]),
    "mlxr_mlp_block_dense": (_i, [_vp] * 8 + [_i, _i, _i, _i, _vp]),
    "mlxr_stream_status": (_i, [_vp, _vp]),
    "mlxr_set_wait_limit_ns": (_i, [C.c_uint64]),
    "mlxr_static_status": (_i, [_vp, _vp]),
    "mlxr_debug_set_trace_buffer": (_i, [_vp]),
    "mlxr_debug_smallm_partition": (_i, [C.c_longlong, _i, _i, C.c_longlong, _vp, _vp, _vp]),
    "mlxr_set_decode_launch_mode": (_i, [_i]),
    "mlxr_q_gemm_dequant_static": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "mlxr_qkv_rope": (_i, [_vp] * 11 + [_i] * 7 + [_f, _i, _i, _vp]),
    "mlxr_q_gemm_dequant_host": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "mlxr_mlp_block_host": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp]),
    "mlxr_release_workspaces": (_i, []),
}

# every symbol include/mlxr_b200_tp.h declares
TP_PROTOTYPES = {
    "mlxr_tp_unique_id": (_i, [_vp]),
    "mlxr_tp_create": (_i, [_vp, _i, _i, _i, C.POINTER(_vp)]),
    "mlxr_tp_destroy": (_i, [_vp]),
    "mlxr_tp_rank": (_i, [_vp]),
    "mlxr_tp_world": (_i, [_vp]),
    "mlxr_tp_shard_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "mlxr_tp_pack_shard": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i]),
    "mlxr_tp_mlp_block": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _vp]),
    "mlxr_tp_all_reduce": (_i, [_vp, _vp, _vp, _sz, _i, _i, _vp]),
    "mlxr_tp_exchange_buffer_bytes": (_sz, []),
    "mlxr_tp_all_reduce_buffers": (_i, [_vp, _vp, _sz, _i, _i, _i, _vp, _vp, _vp]),
}

for _name, (_res, _args) in list(PROTOTYPES.items()) + list(TP_PROTOTYPES.items()):
    _fn = getattr(lib, _name)  # AttributeError here = library out of date with the header
    _fn.restype = _res
    _fn.argtypes = _args


class MlxrError(RuntimeError):
    """Failure reported by the C ABI (std::runtime_error in the C++ primitive layer)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[{lib.mlxr_status_string(status).decode()}] {message}")
        self.status = status


class MlxrInvalidArgument(MlxrError, ValueError):
    """MLXR_ERR_INVALID_ARGUMENT (std::invalid_argument in the C++ primitive layer)."""


def check(status: int) -> None:
    if status == OK:
        return
    msg = lib.mlxr_last_error().decode()
    if status == ERR_INVALID_ARGUMENT:
        raise MlxrInvalidArgument(status, msg)
    raise MlxrError(status, msg)
