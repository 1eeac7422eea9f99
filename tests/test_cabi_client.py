"""The C ABI from plain C: tests/cabi/client.c (C99, CUDA runtime only - no Python, no torch
on its side) is built with gcc against include/dwbnq.h and libdwbnq.so. On CPU the test
checks that it compiles without warnings and links; on the GPU it runs a layer through it
and compares the file it writes with the CPU oracle bit for bit."""
import os
import subprocess

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, ".."))
PKG = os.path.join(ROOT, "nnabla-ext-cuda_b200")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


@pytest.fixture(scope="module")
def client(dwlib):
    out_dir = os.path.join(HERE, "cabi", "_build")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "client")
    src = os.path.join(HERE, "cabi", "client.c")
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-O1", "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(CUDA, "include"), src, "-L" + PKG, "-ldwbnq", "-L" + os.path.join(CUDA, "lib64"),
           "-lcudart", "-Wl,-rpath," + PKG, "-Wl,-rpath," + os.path.join(CUDA, "lib64"), "-o", exe]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def test_client_builds_as_plain_c(client):
    assert os.access(client, os.X_OK)
    # usage error path, no device needed
    assert subprocess.run([client], capture_output=True).returncode == 2


@pytest.mark.gpu
@pytest.mark.parametrize("hw,k,stride", [(14, 3, 1), (28, 3, 2), (20, 5, 1), (56, 3, 1)])
def test_client_matches_the_oracle(client, oracle, tmp_path, hw, k, stride):
    rng = np.random.default_rng(5 + hw)
    n, c, pad = 3, 10, k // 2
    x = rng.standard_normal((n, c, hw, hw)).astype(np.float32)
    w = (rng.standard_normal((c, k, k)) / k).astype(np.float32)
    vec = [rng.standard_normal(c).astype(np.float32) * 0.3 for _ in range(2)]          # b, beta
    gamma, mean, var = (rng.random(c) * 0.4 + 0.8).astype(np.float32), rng.standard_normal(c).astype(np.float32) * 0.3, \
        (rng.random(c) + 0.5).astype(np.float32)
    sign, bits, delta, eps = 1, 8, np.float32(2.0 ** -4), np.float32(1e-5)
    layer = tmp_path / "layer.bin"
    with open(layer, "wb") as f:
        np.array([n, c, hw, hw, k, stride, pad, sign, bits], np.int32).tofile(f)
        np.array([delta, eps], np.float32).tofile(f)
        for a in (x, w, vec[0], vec[1], gamma, mean, var):
            a.tofile(f)
    out = tmp_path / "out.bin"
    r = subprocess.run([client, str(layer), str(out)], capture_output=True, text=True)
    assert r.returncode == 0, (r.returncode, r.stderr)
    shape = tuple(int(v) for v in r.stdout.split())
    got = np.fromfile(out, np.float32).reshape(shape)
    want = oracle.fpq(oracle.bn_infer(oracle.dwconv(x, w, vec[0], (stride, stride), (pad, pad)), vec[1], gamma, mean, var,
                                      1e-5), True, 8, 2.0 ** -4)
    assert got.shape == want.shape
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
