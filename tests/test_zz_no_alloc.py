"""dwbnq_minmaxq_fwd_static: MinMaxQuantize for callers that cannot pass scratch memory.

Such callers exist: a function object that a framework invokes with nothing but its tensor
pointers after the framework's pool has taken the whole device, or a serving loop that may
not enter the allocator once it runs. For them the library keeps the per-channel scratch in
a fixed device array of its own. This file checks, through the C ABI, that the entry point
produces exactly what dwbnq_minmaxq_fwd produces with a caller-provided workspace, and (in
fp32) what the CPU oracle computes - on two consecutive calls, because the array keeps the
previous call's contents - and that it refuses more channels than the array holds. It is named to be collected last, so a run that stops at
the first failure has already executed every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from dwbnq import _lib as L
from dwbnq import ops

pytestmark = pytest.mark.gpu


def _static_call(x, qr_min, qr_max, ql_min, ql_max, q, y):
    dev = x.device
    n, c = x.shape[0], x.shape[1]
    size2 = x.numel() // (n * c)
    mm = L.MinMaxPtrs(qr_min.data_ptr(), qr_max.data_ptr(), ql_min.data_ptr(), ql_max.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    return L.lib().dwbnq_minmaxq_fwd_static(L.F32 if x.dtype == torch.float32 else L.F16, n, c, size2,
                                            ctypes.byref(q), ctypes.c_void_p(x.data_ptr()), ctypes.byref(mm),
                                            ctypes.c_void_p(y.data_ptr()), dev.index, stream)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
def test_static_workspace_matches_caller_workspace_twice(cuda_device, oracle, dtype):
    g = torch.Generator(device="cpu").manual_seed(5)
    # two different problems back to back: the second one finds the first one's leftovers
    for shape in ((6, 192, 14, 14), (3, 37, 9, 5)):
        c = shape[1]
        x = (torch.randn(shape, generator=g) * 3).to(dtype).to(cuda_device)
        x[:, 0] = 0.5  # a constant channel exercises the range nudge
        ql_min = torch.zeros(c, dtype=dtype, device=cuda_device)
        ql_max = torch.full((c,), 255.0, dtype=dtype, device=cuda_device)
        for x_min_max, ema in ((True, False), (True, True), (False, False)):
            q = L.QuantDesc(kind=L.Q_MINMAX, decay=0.9, eps=0.01, x_min_max=int(x_min_max), ema=int(ema))
            qr0 = (torch.randn(c, generator=g) - 3).to(dtype)
            qr1 = (torch.randn(c, generator=g) + 3).to(dtype)
            want_min, want_max = qr0.to(cuda_device), qr1.to(cuda_device)
            want = ops.min_max_quantize(x, want_min, want_max, ql_min, ql_max, 0.9, x_min_max, ema, True, 0.01)
            got_min, got_max = qr0.to(cuda_device), qr1.to(cuda_device)
            got = torch.empty_like(x)
            st = _static_call(x, got_min, got_max, ql_min, ql_max, q, got)
            assert st == L.OK, L.lib().dwbnq_last_error_string()
            torch.cuda.synchronize()
            bits = torch.int32 if dtype == torch.float32 else torch.int16
            assert torch.equal(got.view(bits), want.view(bits)), (shape, x_min_max, ema)
            assert torch.equal(got_min.view(bits), want_min.view(bits))
            assert torch.equal(got_max.view(bits), want_max.view(bits))
            if dtype == torch.float32:  # and against the CPU oracle itself, not only CUDA against CUDA
                oy, omin, omax = oracle.minmaxq(x.cpu().numpy(), qr0.numpy(), qr1.numpy(), ql_min.cpu().numpy(),
                                                ql_max.cpu().numpy(), 0.9, x_min_max, ema, 0.01)
                assert np.array_equal(got.cpu().numpy().view(np.uint32), oy.view(np.uint32)), (shape, x_min_max, ema)
                np.testing.assert_array_equal(got_min.cpu().numpy(), omin)
                np.testing.assert_array_equal(got_max.cpu().numpy(), omax)
    ops.check_device_flag()


def test_static_workspace_rejects_too_many_channels(cuda_device):
    c = L.STATIC_MAX_CHANNELS + 1
    x = torch.zeros((1, c, 1, 1), device=cuda_device)
    v = torch.zeros(c, device=cuda_device)
    q = L.QuantDesc(kind=L.Q_MINMAX, decay=0.9, eps=0.01, x_min_max=1, ema=0)
    st = _static_call(x, v.clone(), v.clone(), v, v + 255, q, torch.empty_like(x))
    assert st == L.ERR_UNSUPPORTED
    assert b"4096" in L.lib().dwbnq_last_error_string()
    # the limit itself is accepted
    c = L.STATIC_MAX_CHANNELS
    x = torch.randn((2, c, 3, 1), device=cuda_device)
    lo, hi = torch.zeros(c, device=cuda_device), torch.ones(c, device=cuda_device)
    y = torch.empty_like(x)
    assert _static_call(x, lo, hi, torch.zeros_like(lo), torch.full_like(lo, 255.0), q, y) == L.OK
    want_lo, want_hi = torch.zeros(c, device=cuda_device), torch.ones(c, device=cuda_device)
    want = ops.min_max_quantize(x, want_lo, want_hi, torch.zeros_like(lo), torch.full_like(lo, 255.0), 0.9, True,
                                False, True, 0.01)
    torch.cuda.synchronize()
    assert torch.equal(y.view(torch.int32), want.view(torch.int32))
