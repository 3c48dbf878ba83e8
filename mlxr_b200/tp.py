"""Tensor-parallel MLP block: host-side mirror of include/mlxr_b200_tp.h.

One process per GPU.  ``torch.distributed`` is used once, to hand rank 0's communicator id to
the other ranks; everything after that goes through the C ABI (NCCL or the peer exchange
kernel inside the library).  The shard geometry is the one the C packer implements:

* w_gate / w_up, packed [inter, hidden]: rank r keeps rows [r*inter/t, (r+1)*inter/t);
* w_down, packed [hidden, inter]: rank r keeps, of every row, the blocks of columns
  [r*inter/t, (r+1)*inter/t), repacked into a packed [hidden, inter/t] matrix;
* x and the RMSNorm weight are replicated, the result is replicated.

The reference has no sharded path; the block itself is MLP::forward
(core/graph/layers.cpp:400-420).
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import Optional, Tuple

import numpy as np
import torch

from . import _capi
from ._capi import check, lib
from .types import QuantType


class Exchange(enum.IntEnum):
    AUTO = 0
    NCCL_F32 = 1
    NCCL_ACT = 2
    PEER = 3


def shard_bytes(which: int, hidden: int, inter: int, quant_type: QuantType, world: int) -> int:
    n = lib.mlxr_tp_shard_bytes(which, hidden, inter, int(quant_type), world)
    if n == 0:
        raise _capi.MlxrError(_capi.ERR_SHAPE,
                              f"cannot shard [hidden {hidden}, inter {inter}] {QuantType(quant_type).name} over {world} ranks")
    return n


def pack_shard(w_full: np.ndarray, which: int, hidden: int, inter: int, quant_type: QuantType,
               rank: int, world: int) -> np.ndarray:
    """One rank's share of a packed weight matrix (host memory, bytes in, bytes out)."""
    w_full = np.ascontiguousarray(w_full).view(np.uint8).reshape(-1)
    full = lib.mlxr_quantized_weight_size(inter if which == 0 else hidden, hidden if which == 0 else inter,
                                          int(quant_type))
    if w_full.size != full:
        raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT,
                                        f"packed matrix has {w_full.size} bytes, expected {full}")
    out = np.empty(shard_bytes(which, hidden, inter, quant_type, world), dtype=np.uint8)
    check(lib.mlxr_tp_pack_shard(w_full.ctypes.data, out.ctypes.data, which, hidden, inter, int(quant_type),
                                 rank, world))
    return out


def shard_mlp_weights(w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray, hidden: int, inter: int,
                      quant_type: QuantType, rank: int, world: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    return (pack_shard(w_gate, 0, hidden, inter, quant_type, rank, world),
            pack_shard(w_up, 0, hidden, inter, quant_type, rank, world),
            pack_shard(w_down, 1, hidden, inter, quant_type, rank, world))


class TPContext:
    """Communicator of one rank.  Collective: every rank of the default process group (or of
    ``group``) constructs it at the same point.  Uses the current CUDA device."""

    def __init__(self, group=None, use_peer: bool = True):
        import torch.distributed as dist
        if not torch.cuda.is_available():
            raise _capi.MlxrError(_capi.ERR_CUDA, "tensor-parallel context needs a CUDA device: there is no CPU path")
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        ident = (C.c_char * 128)()
        if self.rank == 0:
            check(lib.mlxr_tp_unique_id(C.addressof(ident)))
        box = [bytes(ident)]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        ident = (C.c_char * 128).from_buffer_copy(box[0])
        handle = C.c_void_p()
        check(lib.mlxr_tp_create(C.addressof(ident), self.rank, self.world, int(use_peer), C.byref(handle)))
        self._h = handle

    def close(self) -> None:
        if self._h:
            check(lib.mlxr_tp_destroy(self._h))
            self._h = None

    def mlp_block(self, x: torch.Tensor, norm_weight: Optional[torch.Tensor], w_gate_shard: torch.Tensor,
                  w_up_shard: torch.Tensor, w_down_shard: torch.Tensor, inter: int, quant_type: QuantType,
                  eps: float = 1e-5, exchange: Exchange = Exchange.AUTO,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
        from .ops import _dev, _dtype_code, _stream
        if x.dim() != 2:
            raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "Input must be 2D [M, hidden_size]")
        M, hidden = x.shape
        qt = int(quant_type)
        for name, t, which in (("w_gate_shard", w_gate_shard, 0), ("w_up_shard", w_up_shard, 0),
                               ("w_down_shard", w_down_shard, 1)):
            if t.numel() * t.element_size() != shard_bytes(which, hidden, inter, quant_type, self.world):
                raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, f"{name} shape mismatch")
        y = torch.empty_like(x) if out is None else out
        check(lib.mlxr_tp_mlp_block(self._h, _dev(x, "x"), _dev(norm_weight, "norm_weight"),
                                    _dev(w_gate_shard, "w_gate_shard"), _dev(w_up_shard, "w_up_shard"),
                                    _dev(w_down_shard, "w_down_shard"), y.data_ptr(), M, hidden, inter, qt, eps,
                                    _dtype_code(x), int(exchange), _stream()))
        return y

    def all_reduce(self, partial: torch.Tensor, dtype: torch.dtype, exchange: Exchange = Exchange.AUTO) -> torch.Tensor:
        from .ops import _DT, _dev, _stream
        if partial.dtype != torch.float32:
            raise _capi.MlxrInvalidArgument(_capi.ERR_INVALID_ARGUMENT, "partial sums are float32")
        y = torch.empty(partial.shape, dtype=dtype, device=partial.device)
        check(lib.mlxr_tp_all_reduce(self._h, _dev(partial, "partial"), y.data_ptr(), partial.numel(), _DT[dtype],
                                     int(exchange), _stream()))
        return y
