"""A bounded device-side wait that runs out: the kernel returns, the stream's status word says
MLXR_ERR_TIMEOUT, and the next call on the stream is correct.

The wait is made to run out on the host side of the test, never by a fault: the one-shot
exchange is called on one GPU with a two-rank table of exchange buffers in which nobody plays
rank 1, so the flags it waits for are never raised; the limit is a few milliseconds.  The second
call has rank 1's contribution written by the host before the launch (no kernel waits for
another kernel)."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FLAG_BYTES = 64 * 1024
SLOT_ELEMS = 256 * 1024
MAX_WORLD = 8
FLAGS_PER_RANK = 1024


def _slot(buf, parity, src):
    """float view of slot [parity][src] of an exchange buffer (layout of mlxr_b200_tp.h)."""
    off = FLAG_BYTES + ((parity * MAX_WORLD + src) * SLOT_ELEMS) * 4
    return buf[off:off + SLOT_ELEMS * 4].view(torch.float32)


def _flags(buf):
    return buf[:MAX_WORLD * FLAGS_PER_RANK * 4].view(torch.int32).view(MAX_WORLD, FLAGS_PER_RANK)


def test_peer_wait_runs_out_then_recovers():
    from mlxr_b200._capi import ERR_TIMEOUT, check, lib
    nbytes = lib.mlxr_tp_exchange_buffer_bytes()
    assert nbytes == FLAG_BYTES + 2 * MAX_WORLD * SLOT_ELEMS * 4
    n = 4096
    ncta = (n + 1023) // 1024
    dev = torch.device("cuda")
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    table = (ctypes.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    ctl = torch.zeros(16, dtype=torch.int32, device=dev)
    p0 = torch.arange(n, dtype=torch.float32, device=dev) * 0.25
    p1 = torch.full((n,), 3.0, dtype=torch.float32, device=dev)
    y = torch.full((n,), -1.0, dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    status = ctypes.c_int(-1)
    check(lib.mlxr_stream_status(st, ctypes.byref(status)))      # start from a clean status word
    check(lib.mlxr_set_wait_limit_ns(3_000_000))                 # 3 ms instead of the default 2 s
    try:
        # call 1 of rank 0: rank 1 never shows up
        check(lib.mlxr_tp_all_reduce_buffers(p0.data_ptr(), y.data_ptr(), n, 2, 0, 2, table, ctl.data_ptr(), st))
        check(lib.mlxr_stream_status(st, ctypes.byref(status)))
        assert status.value == ERR_TIMEOUT
        assert torch.all(y == -1.0), "a CTA whose wait ran out must not store a result"
        assert int(ctl[0]) == 1 and int(ctl[1]) == 0, "the sequence number advances, the CTA counter clears"
        assert torch.all(_flags(bufs[0])[0, :ncta] == 1) and torch.all(_flags(bufs[1])[0, :ncta] == 1)
        # call 2: the host plays rank 1 before the launch (slot of parity 0, flags = 2)
        _slot(bufs[0], 0, 1)[:n] = p1
        _flags(bufs[0])[1, :ncta] = 2
        torch.cuda.synchronize()
        check(lib.mlxr_tp_all_reduce_buffers(p0.data_ptr(), y.data_ptr(), n, 2, 0, 2, table, ctl.data_ptr(), st))
        check(lib.mlxr_stream_status(st, ctypes.byref(status)))
        assert status.value == 0
        assert torch.equal(y, p0 + p1)
        assert int(ctl[0]) == 2
    finally:
        check(lib.mlxr_set_wait_limit_ns(2_000_000_000))


def test_decode_block_is_clean_under_a_short_limit(oracle):
    """The same limit applies to the persistent decode kernel's own waits (copy barriers, the
    hand-over words between its phases): a normal call stays far inside a few milliseconds."""
    import mlxr_b200 as mx
    from mlxr_b200._capi import check, lib
    from mlxr_b200.quantize import quantize
    from conftest import make_acts, make_weights
    M, H, I, qt = 3, 512, 1024, 3
    wg, wu, wd = (quantize(make_weights(n, k, s), qt) for n, k, s in ((I, H, 1), (I, H, 2), (H, I, 3)))
    xt, xf = make_acts(M, H, 4, torch.bfloat16)
    gam = torch.ones(H, dtype=torch.bfloat16)
    status = ctypes.c_int(-1)
    check(lib.mlxr_set_wait_limit_ns(5_000_000))
    try:
        y = mx.mlp_block(xt.cuda(), gam.cuda(), torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda(),
                         torch.from_numpy(wd).cuda(), I, mx.QuantType(qt), 1e-5)
        check(lib.mlxr_stream_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(status)))
    finally:
        check(lib.mlxr_set_wait_limit_ns(2_000_000_000))
    assert status.value == 0
    ref = oracle.mlp_block(xf, gam.float().numpy(), wg, wu, wd, I, qt, 1e-5, 1)
    assert oracle.rel_l2(y.float().cpu().numpy(), ref) <= 2e-2


def test_wait_limit_rejects_zero():
    from mlxr_b200._capi import ERR_INVALID_ARGUMENT, lib
    assert lib.mlxr_set_wait_limit_ns(0) == ERR_INVALID_ARGUMENT
