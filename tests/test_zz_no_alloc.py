"""mlxr_q_gemm_dequant_static: the decode linear that never allocates device memory.

Collected last on purpose (file name): the entry point keeps its scratch in a fixed array of
the loaded module, so it must give the right answer both in a fresh process (this file alone)
and after every other test has used the regular workspaces.  Each case calls it twice in a
row - the second call finds the counters and barrier words as the first one left them - and
compares with the regular entry point: the two static calls must agree bit for bit (the
reduction order is fixed), and both must agree with mlxr_q_gemm_dequant within 2e-3 relative
L2 (for some shapes the regular entry point runs a different kernel of this library, whose
float sums are added in another order).  It also checks the point of the entry: no device
memory is allocated by either call, and the status word of the static array reads clean."""
import numpy as np
import pytest
import torch

from conftest import make_acts, make_weights

pytestmark = pytest.mark.gpu
DT = {"f16": (torch.float16, 0), "bf16": (torch.bfloat16, 1), "f32": (torch.float32, 2)}


def _static(x, w, bias, M, N, K, qt, dt_code):
    from mlxr_b200 import _capi
    y = torch.empty((M, N), dtype=x.dtype, device="cuda")
    _capi.check(_capi.lib.mlxr_q_gemm_dequant_static(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                                                     y.data_ptr(), M, N, K, qt, dt_code,
                                                     torch.cuda.current_stream().cuda_stream))
    return y


@pytest.mark.parametrize("qt,M,N,K,dt,bias", [(3, 1, 4096, 4096, "bf16", False),    # split-K over CTAs: partial sums + counters
                                              (3, 2, 1024, 14336, "bf16", False),
                                              (3, 8, 8192, 1024, "f16", True),      # the largest N accepted
                                              (0, 3, 1000, 512, "f16", True),       # Q4_0, ragged N
                                              (3, 5, 264, 2048, "f32", False)])
def test_matches_regular_entry_point_twice(oracle, qt, M, N, K, dt, bias):
    import mlxr_b200 as mx
    from mlxr_b200.quantize import quantize
    tdt, code = DT[dt]
    w = torch.from_numpy(quantize(make_weights(N, K, 11), qt)).cuda()
    xt, xf = make_acts(M, K, 12, tdt)
    x = xt.cuda()
    b = None
    if bias:
        b = make_acts(1, N, 13, tdt)[0][0].contiguous().cuda()
    ref = mx.q_gemm_dequant(x, w, M, N, K, mx.QuantType(qt), mx._capi.lib.mlxr_default_group_size(qt), b)
    import ctypes
    _static(x, w, b, M, N, K, qt, code)               # first call on the device: looks up the array's address
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    y1 = _static(x, w, b, M, N, K, qt, code)
    y2 = _static(x, w, b, M, N, K, qt, code)
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    # y1 / y2 come from torch's caching allocator, whose pool only grows in whole segments; the
    # library itself must not have taken anything from the device
    assert free_after >= free_before - y1.numel() * y1.element_size() * 2 - (2 << 20)
    status = ctypes.c_int(-1)
    mx._capi.check(mx._capi.lib.mlxr_static_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(status)))
    assert status.value == 0
    assert torch.equal(y1, y2)
    refn = ref.float().cpu().numpy()
    assert oracle.rel_l2(y1.float().cpu().numpy(), refn) <= 2e-3
    # and the answer itself is right (not merely equal to the other entry point)
    want = oracle.linear(xf, w.cpu().numpy(), N, qt, b.float().cpu().numpy() if bias else None)
    assert oracle.rel_l2(y2.float().cpu().numpy(), want) <= 2e-2


def test_rejects_what_does_not_fit():
    from mlxr_b200 import _capi
    x = torch.zeros(1, 512, dtype=torch.float16, device="cuda")
    w = torch.zeros(_capi.lib.mlxr_quantized_weight_size(8208, 512, 3), dtype=torch.uint8, device="cuda")
    y = torch.zeros(16, 8208, dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    call = _capi.lib.mlxr_q_gemm_dequant_static
    assert call(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 1, 8208, 512, 3, 0, st) == _capi.ERR_WORKSPACE
    assert b"8192" in _capi.lib.mlxr_last_error()
    assert call(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 9, 64, 512, 3, 0, st) == _capi.ERR_UNSUPPORTED   # batch > 8
    assert call(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 1, 64, 512, 2, 0, st) == _capi.ERR_UNSUPPORTED   # Q8_0
    assert call(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 1, 64, 256, 3, 0, st) == _capi.ERR_UNSUPPORTED   # K < 512
    assert call(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 0, 64, 512, 3, 0, st) == _capi.OK                # empty batch
    torch.cuda.synchronize()
