"""The test / tuning switches of include/dwbnq_debug.h: they belong to the calling host
thread, and the bounded device wait gives up in time and reports it through the device flag."""
import ctypes
import threading
import time

import pytest


def _plan_path(dwlib, **kw):
    lib = dwlib.lib()
    base = dict(dtype=dwlib.F32, c=32, n=4, h=112, w=112, kh=3, kw=3, stride_h=1, stride_w=1, pad_h=1, pad_w=1,
                dil_h=1, dil_w=1, multiplier=1)
    base.update(kw)
    d = dwlib.ConvDesc(**base)
    path = ctypes.c_int()
    aligned = ctypes.c_void_p(4096)
    assert lib.dwbnq_fused_plan(ctypes.byref(d), aligned, aligned, ctypes.byref(path), None, None, None, None,
                                None) == dwlib.OK
    return path.value


def test_forced_path_is_per_thread(dwlib):
    """One host thread forcing a kernel family must not change what another thread gets."""
    lib = dwlib.lib()
    assert _plan_path(dwlib) == dwlib.PATH_PLANE
    seen = {}

    def other():
        assert lib.dwbnq_set_forced_path(dwlib.PATH_GENERIC) == dwlib.OK
        assert lib.dwbnq_set_tuning(3, 2, 0, 0) == dwlib.OK
        seen["other"] = _plan_path(dwlib)
        ready.set()
        release.wait(10)
        seen["other_again"] = _plan_path(dwlib)

    ready, release = threading.Event(), threading.Event()
    t = threading.Thread(target=other)
    t.start()
    assert ready.wait(10)
    seen["main_while_other_forces"] = _plan_path(dwlib)
    release.set()
    t.join()
    assert seen == {"other": dwlib.PATH_GENERIC, "main_while_other_forces": dwlib.PATH_PLANE,
                    "other_again": dwlib.PATH_GENERIC}
    # and a new thread starts from the default again
    out = []
    t = threading.Thread(target=lambda: out.append(_plan_path(dwlib)))
    t.start()
    t.join()
    assert out == [dwlib.PATH_PLANE]


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_is_reported(dwlib, cuda_device):
    """A warp waits, with the library's bounded wait, on a barrier nothing completes: the wait
    gives up after its (shortened) time limit, the kernel returns normally, the device flag
    says so once, and the context stays usable."""
    import torch
    from dwbnq import ops
    lib = dwlib.lib()
    assert lib.dwbnq_check_device_flag(0) == dwlib.OK
    t0 = time.time()
    assert lib.dwbnq_debug_expire_wait(20000, 0, None) == dwlib.OK  # 20 ms
    st = lib.dwbnq_check_device_flag(0)
    dt = time.time() - t0
    assert st == dwlib.ERR_DEVICE_FLAG and b"bounded wait" in lib.dwbnq_last_error_string()
    assert 0.015 <= dt < 1.5, dt
    assert lib.dwbnq_check_device_flag(0) == dwlib.OK  # reading the flag cleared it
    x = torch.linspace(-3, 3, 4096, device=cuda_device)
    y = ops.fixed_point_quantize(x, True, 8, 2.0 ** -4)
    assert float((y - x).abs().max()) <= 2.0 ** -5
    ops.check_device_flag()
