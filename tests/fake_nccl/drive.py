"""Child process of tests/test_comm_failures.py: drives the communicator entry points of
libdwbnq against the stand-in NCCL library (no torch in this process, so the real libnccl is
never loaded). Prints one JSON line."""
import ctypes
import json
import os
import sys
import time

lib = ctypes.CDLL(sys.argv[1])
fake = ctypes.CDLL(os.environ["DWBNQ_NCCL_LIB"], mode=ctypes.RTLD_GLOBAL)
lib.dwbnq_last_error_string.restype = ctypes.c_char_p
out = {}
uid = (ctypes.c_ubyte * 128)()
out["get_id"] = lib.dwbnq_comm_get_unique_id(uid)
comm = ctypes.c_void_p()
out["create"] = lib.dwbnq_comm_create(bytes(uid), 1, 0, 0, ctypes.byref(comm))
timeout_ms = int(sys.argv[2])
buf = ctypes.c_void_p()


class QuantDesc(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("sign", ctypes.c_int32), ("n", ctypes.c_int32),
                ("delta", ctypes.c_float), ("with_zero", ctypes.c_int32), ("m", ctypes.c_int32),
                ("decay", ctypes.c_float), ("eps", ctypes.c_float), ("x_min_max", ctypes.c_int32),
                ("ema", ctypes.c_int32)]


class MinMaxPtrs(ctypes.Structure):
    _fields_ = [("qr_min", ctypes.c_void_p), ("qr_max", ctypes.c_void_p),
                ("ql_min", ctypes.c_void_p), ("ql_max", ctypes.c_void_p)]


class ConvDesc(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("c", ctypes.c_int32), ("n", ctypes.c_int64),
                ("h", ctypes.c_int32), ("w", ctypes.c_int32), ("kh", ctypes.c_int32),
                ("kw", ctypes.c_int32), ("stride_h", ctypes.c_int32), ("stride_w", ctypes.c_int32),
                ("pad_h", ctypes.c_int32), ("pad_w", ctypes.c_int32), ("dil_h", ctypes.c_int32),
                ("dil_w", ctypes.c_int32), ("multiplier", ctypes.c_int32)]


if sys.argv[3] in ("minmaxq", "fused_empty"):
    # The operator entry points with a communicator: the deadline is the one the communicator
    # carries (dwbnq_comm_set_deadline_ms), the collective is the one they issue themselves.
    rt = ctypes.CDLL("libcudart.so")
    C, HW, N = 4, 64, 2

    def dmalloc(nbytes, fill=None):
        p = ctypes.c_void_p()
        assert rt.cudaMalloc(ctypes.byref(p), ctypes.c_size_t(nbytes)) == 0
        assert rt.cudaMemset(p, 0, ctypes.c_size_t(nbytes)) == 0
        if fill is not None:
            arr = (ctypes.c_float * len(fill))(*fill)
            assert rt.cudaMemcpy(p, arr, ctypes.c_size_t(4 * len(fill)), 1) == 0
        return p

    x = dmalloc(4 * N * C * HW, [float(i % 7) - 3.0 for i in range(N * C * HW)])
    y = dmalloc(4 * N * C * HW)
    qr_min, qr_max = dmalloc(4 * C), dmalloc(4 * C, [1.0] * C)
    ql_min, ql_max = dmalloc(4 * C), dmalloc(4 * C, [255.0] * C)
    lib.dwbnq_workspace_bytes.restype = ctypes.c_size_t
    ws = dmalloc(lib.dwbnq_workspace_bytes(C))
    mm = MinMaxPtrs(qr_min.value, qr_max.value, ql_min.value, ql_max.value)
    q = QuantDesc(kind=3, decay=0.999, eps=0.01, x_min_max=1, ema=0)
    out["set_deadline"] = lib.dwbnq_comm_set_deadline_ms(comm, timeout_ms)
    t0 = time.time()
    if sys.argv[3] == "minmaxq":
        out["call"] = lib.dwbnq_minmaxq_fwd(0, ctypes.c_int64(N), C, ctypes.c_int64(HW), ctypes.byref(q), x,
                                            ctypes.byref(mm), y, ws, comm, 0, None)
    else:
        # a rank whose shard of the batch is empty still joins the min/max all-reduce
        d = ConvDesc(dtype=0, c=C, n=0, h=8, w=8, kh=3, kw=3, stride_h=1, stride_w=1, pad_h=1, pad_w=1,
                     dil_h=1, dil_w=1, multiplier=1)
        out["call"] = lib.dwbnq_fused_fwd(ctypes.byref(d), ctypes.c_float(1e-5), ctypes.byref(q), None, None, None,
                                          None, None, None, None, ctypes.byref(mm), None, ws, comm, 0, None)
    out["seconds"] = time.time() - t0
    out["message"] = lib.dwbnq_last_error_string().decode()
    out["allreduces_after_call"] = fake.fake_nccl_allreduces()
    # without a communicator the empty batch is a no-op
    if sys.argv[3] == "fused_empty":
        out["no_comm"] = lib.dwbnq_fused_fwd(ctypes.byref(d), ctypes.c_float(1e-5), ctypes.byref(q), None, None,
                                             None, None, None, None, None, ctypes.byref(mm), None, ws, None, 0, None)
        out["allreduces_no_comm"] = fake.fake_nccl_allreduces()
        rt.cudaDeviceSynchronize()
        lo = (ctypes.c_float * C)()
        rt.cudaMemcpy(lo, qr_min, ctypes.c_size_t(4 * C), 2)
        out["qr_min"] = [float(v) for v in lo]
    out["second_call"] = lib.dwbnq_minmaxq_fwd(0, ctypes.c_int64(N), C, ctypes.c_int64(HW), ctypes.byref(q), x,
                                               ctypes.byref(mm), y, ws, comm, 0, None)
    out["second_message"] = lib.dwbnq_last_error_string().decode()
    out["aborts"] = fake.fake_nccl_aborts()
    out["allreduces"] = fake.fake_nccl_allreduces()
    out["destroy"] = lib.dwbnq_comm_destroy(comm)
    rt.cudaDeviceSynchronize()
    print(json.dumps(out))
    sys.exit(0)
if sys.argv[3] == "device":
    rt = ctypes.CDLL("libcudart.so")
    assert rt.cudaMalloc(ctypes.byref(buf), 1024) == 0
else:
    buf = ctypes.c_void_p(256)  # never dereferenced by the stand-in
t0 = time.time()
out["allreduce"] = lib.dwbnq_comm_allreduce_max_f32(comm, buf, ctypes.c_longlong(16), None, timeout_ms)
out["seconds"] = time.time() - t0
out["message"] = lib.dwbnq_last_error_string().decode()
out["second_call"] = lib.dwbnq_comm_allreduce_max_f32(comm, buf, ctypes.c_longlong(16), None, timeout_ms)
out["second_message"] = lib.dwbnq_last_error_string().decode()
out["aborts"] = fake.fake_nccl_aborts()
out["allreduces"] = fake.fake_nccl_allreduces()
out["destroy"] = lib.dwbnq_comm_destroy(comm)
if sys.argv[3] == "device":
    rt.cudaDeviceSynchronize()  # let the stalled host function finish before the process exits
print(json.dumps(out))
