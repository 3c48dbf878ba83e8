"""Tensor-parallel MLP block without a GPU: the C shard packer and the sum-of-shards identity,
on one process and as two gloo ranks (the N > 1 host logic).  The arithmetic here is the oracle's;
the library contributes only its host-side packer."""
import os
import socket

import numpy as np
import pytest
import torch

from conftest import make_acts, make_weights

BF16 = 1


def _case(qt, hidden, inter, M, seed=0):
    from mlxr_b200.quantize import quantize
    wg = quantize(make_weights(inter, hidden, 10 + seed), qt)
    wu = quantize(make_weights(inter, hidden, 20 + seed), qt)
    wd = quantize(make_weights(hidden, inter, 30 + seed), qt)
    _, x = make_acts(M, hidden, 40 + seed, torch.bfloat16)
    _, gam = make_acts(1, hidden, 50 + seed, torch.bfloat16)
    return wg, wu, wd, x, (1.0 + 0.1 * gam[0]).astype(np.float32)


@pytest.mark.parametrize("qt,hidden,inter,world", [(3, 512, 1024, 2), (3, 512, 1024, 4), (0, 256, 384, 3), (2, 128, 256, 8),
                                                    (16, 256, 512, 2)])
def test_packer_geometry(oracle, qt, hidden, inter, world):
    """Dequantized shards are exactly the row / column ranges of the dequantized full matrices."""
    import mlxr_b200.tp as tp
    wg, wu, wd, _, _ = _case(qt, hidden, inter, 1)
    full_g = oracle.dequantize(wg, inter, hidden, qt)[0]
    full_d = oracle.dequantize(wd, hidden, inter, qt)[0]
    il = inter // world
    for r in range(world):
        sg = tp.pack_shard(wg, 0, hidden, inter, qt, r, world)
        sd = tp.pack_shard(wd, 1, hidden, inter, qt, r, world)
        assert sg.size == tp.shard_bytes(0, hidden, inter, qt, world)
        assert sd.size == tp.shard_bytes(1, hidden, inter, qt, world)
        np.testing.assert_array_equal(oracle.dequantize(sg, il, hidden, qt)[0], full_g[r * il:(r + 1) * il])
        np.testing.assert_array_equal(oracle.dequantize(sd, hidden, il, qt)[0], full_d[:, r * il:(r + 1) * il])


def test_packer_rejects_bad_splits():
    import mlxr_b200.tp as tp
    from mlxr_b200 import _capi
    assert _capi.lib.mlxr_tp_shard_bytes(0, 512, 1024, 3, 8) == 0      # 1024 / 8 is not a whole 256-block
    assert _capi.lib.mlxr_tp_shard_bytes(1, 512, 1024, 4, 2) == 0      # Q6_K has no code
    with pytest.raises(_capi.MlxrError):
        tp.pack_shard(np.zeros(10, np.uint8), 0, 512, 1024, 3, 0, 2)  # wrong byte count
    w = np.zeros(_capi.lib.mlxr_quantized_weight_size(1024, 512, 3), np.uint8)
    with pytest.raises(_capi.MlxrError):
        tp.pack_shard(w, 0, 512, 1024, 3, 2, 2)                       # rank outside the world


@pytest.mark.parametrize("world", [2, 4])
def test_sum_of_shards_equals_unsharded(oracle, world):
    import mlxr_b200.tp as tp
    qt, hidden, inter, M = 3, 512, 1024, 3
    wg, wu, wd, x, gam = _case(qt, hidden, inter, M)
    whole = oracle.mlp_block_partial(x, gam, wg, wu, wd, inter, qt, 1e-5, BF16)
    acc = np.zeros_like(whole)
    for r in range(world):
        sg, su, sd = tp.shard_mlp_weights(wg, wu, wd, hidden, inter, qt, r, world)
        acc += oracle.mlp_block_partial(x, gam, sg, su, sd, inter // world, qt, 1e-5, BF16)
    assert oracle.rel_l2(acc, whole) < 1e-6      # float32 summation order only
    assert oracle.rel_l2(oracle.round_to(acc, BF16), oracle.mlp_block(x, gam, wg, wu, wd, inter, qt, 1e-5, BF16)) < 2e-3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _gloo_rank(rank, world, port, ret):
    import torch.distributed as dist
    from oracle import oracle as O
    import mlxr_b200.tp as tp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        qt, hidden, inter, M = 3, 512, 1024, 2
        wg, wu, wd, x, gam = _case(qt, hidden, inter, M, seed=7)      # same seeds on every rank: replicated inputs
        sg, su, sd = tp.shard_mlp_weights(wg, wu, wd, hidden, inter, qt, rank, world)
        part = torch.from_numpy(O.mlp_block_partial(x, gam, sg, su, sd, inter // world, qt, 1e-5, BF16))
        dist.all_reduce(part)                                          # the block's one exchange step
        whole = O.mlp_block_partial(x, gam, wg, wu, wd, inter, qt, 1e-5, BF16)
        err = O.rel_l2(part.numpy(), whole)
        # every rank must hold the same replicated result
        gathered = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(gathered, part)
        same = all(torch.equal(gathered[0], g) for g in gathered)
        ret[rank] = (err, same)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks():
    import torch.multiprocessing as mp
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_gloo_rank, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert len(ret) == world
        for r in range(world):
            err, same = ret[r]
            assert err < 1e-6 and same
