"""Tensor-parallel MLP block on the GPU, through the C ABI.

* On one GPU: each rank's share computed in turn (mlxr_mlp_block_partial_f32 on packed shards),
  summed on the host and compared with the unsharded oracle - the sharded compute and the packer
  without any exchange.
* With two or more GPUs visible: one process per GPU, every exchange mode (NCCL float, NCCL in
  the activation dtype, the peer exchange kernel), results compared with the unsharded oracle
  and required to be bit-identical on all ranks.  Skipped on a one-GPU box.
"""
import os
import socket

import numpy as np
import pytest
import torch

from conftest import make_acts, make_weights

pytestmark = pytest.mark.gpu
BF16 = 1
TOL = 2e-2


def _case(qt, hidden, inter, M, seed=0):
    from mlxr_b200.quantize import quantize
    wg = quantize(make_weights(inter, hidden, 10 + seed), qt)
    wu = quantize(make_weights(inter, hidden, 20 + seed), qt)
    wd = quantize(make_weights(hidden, inter, 30 + seed), qt)
    xt, x = make_acts(M, hidden, 40 + seed, torch.bfloat16)
    _, g = make_acts(1, hidden, 50 + seed, torch.bfloat16)
    gt = torch.from_numpy(1.0 + 0.1 * g[0]).to(torch.bfloat16)
    return wg, wu, wd, xt, x, gt, gt.float().numpy()


@pytest.mark.parametrize("qt,hidden,inter,M,world", [(3, 512, 2048, 1, 2), (3, 1024, 2048, 3, 4), (3, 512, 4096, 8, 8),
                                                      (0, 512, 1024, 2, 4), (2, 256, 512, 5, 2)])
def test_sharded_partials_sum_to_block(oracle, qt, hidden, inter, M, world):
    import mlxr_b200 as mx
    import mlxr_b200.tp as tp
    wg, wu, wd, xt, x, gt, gam = _case(qt, hidden, inter, M)
    acc = torch.zeros(M, hidden, dtype=torch.float32, device="cuda")
    for r in range(world):
        sg, su, sd = (torch.from_numpy(a).cuda() for a in tp.shard_mlp_weights(wg, wu, wd, hidden, inter, qt, r, world))
        acc += mx.mlp_block_partial(xt.cuda(), gt.cuda(), sg, su, sd, inter // world, mx.QuantType(qt), 1e-5)
    torch.cuda.synchronize()
    ref = oracle.mlp_block(x, gam, wg, wu, wd, inter, qt, 1e-5, BF16)
    assert oracle.rel_l2(acc.to(torch.bfloat16).float().cpu().numpy(), ref) <= TOL


def test_world_of_one_matches_plain_block(oracle):
    """A one-rank context: the exchange degenerates to the rounding store."""
    import torch.distributed as dist
    import mlxr_b200 as mx
    import mlxr_b200.tp as tp
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = str(_free_port())
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        ctx = tp.TPContext()
        qt, hidden, inter, M = 3, 1024, 2048, 2
        wg, wu, wd, xt, x, gt, gam = _case(qt, hidden, inter, M)
        dev = [torch.from_numpy(a).cuda() for a in (wg, wu, wd)]
        y = ctx.mlp_block(xt.cuda(), gt.cuda(), *dev, inter, mx.QuantType(qt))
        y0 = mx.mlp_block(xt.cuda(), gt.cuda(), *dev, inter, mx.QuantType(qt))
        torch.cuda.synchronize()
        assert torch.equal(y, y0)
        ctx.close()
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist
    from oracle import oracle as O
    import mlxr_b200 as mx
    import mlxr_b200.tp as tp
    from mlxr_b200 import _capi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    out = {}
    try:
        ctx = tp.TPContext()
        for (qt, hidden, inter, M) in [(3, 1024, 4096, 1), (3, 1024, 4096, 8), (3, 512, 2048, 3)]:
            wg, wu, wd, xt, x, gt, gam = _case(qt, hidden, inter, M, seed=M)
            sh = [torch.from_numpy(a).cuda() for a in tp.shard_mlp_weights(wg, wu, wd, hidden, inter, qt, rank, world)]
            ref = O.mlp_block(x, gam, wg, wu, wd, inter, qt, 1e-5, BF16)
            for mode in (tp.Exchange.NCCL_F32, tp.Exchange.NCCL_ACT, tp.Exchange.PEER, tp.Exchange.AUTO):
                ys = [ctx.mlp_block(xt.cuda(), gt.cuda(), *sh, inter, mx.QuantType(qt), exchange=mode) for _ in range(5)]
                torch.cuda.synchronize()
                st = torch.zeros(1, dtype=torch.int32)
                _capi.check(_capi.lib.mlxr_stream_status(torch.cuda.current_stream().cuda_stream, st.data_ptr()))
                err = O.rel_l2(ys[-1].float().cpu().numpy(), ref)
                rep = all(torch.equal(ys[0], y) for y in ys)
                gathered = [torch.empty_like(ys[-1].cpu()) for _ in range(world)]
                dist.all_gather(gathered, ys[-1].cpu())
                same = all(torch.equal(gathered[0], g) for g in gathered)
                out[(qt, hidden, inter, M, int(mode))] = (err, rep, same, int(st[0]))
        ctx.close()
        ret[rank] = out
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_on_separate_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_rank_main, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert len(ret) == world
        for r in range(world):
            for key, (err, rep, same, status) in ret[r].items():
                assert status == 0, (r, key, status)
                assert err <= TOL, (r, key, err)
                assert rep, (r, key, "results differ between repeated calls")
                # NCCL may order its float sums differently per rank; the peer exchange may not
                if key[-1] == 3:
                    assert same, (r, key, "ranks disagree")
