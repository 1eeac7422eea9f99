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
