"""The host layer of libdwbnq under AddressSanitizer + UndefinedBehaviorSanitizer, and the
bounds-checked build's surface - both without a GPU.

`make asan` compiles the host-heavy translation units (entry points, quantizer parameters,
communicator, planner and launch code of the two convolution families) with
-fsanitize=address,undefined into libdwbnq_asan.so; tests/cabi/validate.c, built the same way,
calls every entry point with null, out-of-range and misaligned arguments and runs the host-only
helpers in full. The client runs with no device visible (CUDA_VISIBLE_DEVICES is emptied), so
nothing it passes can reach a kernel: every call has to come back with a status, and neither
sanitizer may report anything.

`make debug` compiles the kernels with -DDWBNQ_BOUNDS_CHECK (every global index is tested against
its tensor's extent; a violation skips the access and writes 2 to the device flag word) into
libdwbnq_debug.so, which must export exactly the ABI of the normal library."""
import os
import re
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, ".."))
PKG = os.path.join(ROOT, "nnabla-ext-cuda_b200")


def _make(target):
    jobs = str(max(1, min(16, os.cpu_count() or 1)))
    r = subprocess.run(["make", "-C", PKG, "-j", jobs, target], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def _exports(path):
    out = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True, check=True).stdout
    return {ln.split()[-1] for ln in out.splitlines() if re.search(r" T dwbnq_", ln)}


def test_host_layer_is_clean_under_asan_and_ubsan(dwlib):
    _make("asan")
    out_dir = os.path.join(HERE, "cabi", "_build")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "validate_asan")
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-O1", "-g", "-fsanitize=address,undefined",
           "-fno-sanitize-recover=undefined", "-I" + os.path.join(ROOT, "include"),
           os.path.join(HERE, "cabi", "validate.c"), "-L" + PKG, "-ldwbnq_asan", "-Wl,-rpath," + PKG, "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:halt_on_error=1",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
    r = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, (r.returncode, r.stdout[-1500:], r.stderr[-3000:])
    assert r.stdout.split() == ["helpers", "planner", "operators", "pointwise", "communicator", "ok"]
    assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr, r.stderr[-3000:]


def test_bounds_checked_build_exports_the_same_abi(dwlib):
    _make("debug")
    normal = _exports(os.path.join(PKG, "libdwbnq.so"))
    debug = _exports(os.path.join(PKG, "libdwbnq_debug.so"))
    assert normal and normal == debug


@pytest.mark.gpu
def test_parity_holds_and_the_flag_stays_clear_in_the_bounds_checked_build(cuda_device):
    """The parity tests of the kernels that carry index checks (the generic depthwise kernel, the
    pointwise tcgen05 and FMA kernels) and the guard-band tests, run in a child process against
    libdwbnq_debug.so: same bits as the oracle, and no index outside its tensor recorded (each of
    those tests reads the device flag, which the checked build sets to 2 on a violation)."""
    debug = os.path.join(PKG, "libdwbnq_debug.so")
    assert os.path.exists(debug), "build it with `make -C nnabla-ext-cuda_b200 debug`"
    env = dict(os.environ, DWBNQ_LIBRARY=debug)
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
           os.path.join(HERE, "test_pointwise_gpu.py"), os.path.join(HERE, "test_guard_bands_gpu.py"),
           os.path.join(HERE, "test_parity_gpu.py"), "-k",
           "pointwise or guard or generic or random_geometries or edge_shapes"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    m = re.search(r"(\d+) passed", r.stdout)
    assert m and int(m.group(1)) >= 100 and "failed" not in r.stdout, r.stdout[-500:]
