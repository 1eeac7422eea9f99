"""Training side through the C ABI against the CPU oracle: the straight-through backward of
FixedPointQuantize and Pow2Quantize and the direct input-gradient kernel of
DepthwiseConvolution are compared bit for bit (same operations, same order). Two things are
compared within a tolerance scaled by the sum of the magnitudes of the terms: the weight and
bias gradients, whose fp32 sum has no fixed association (block reduction + atomic adds here, a
block tree in the reference), and the input gradient of a stride-1 "same" convolution when it
is overwritten, which runs as the forward kernels on the rotated kernel (taps summed in the
forward order, the reverse of the reference loop's)."""
import numpy as np
import pytest
import torch

from dwbnq import _lib as L
from dwbnq import ops

pytestmark = pytest.mark.gpu

import os  # noqa: E402

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def dev(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def same_bits(got, want, what):
    got, want = np.asarray(got), np.asarray(want)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan), what
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan]), what


def by_forward(k, s, p, dil, mult):
    """The case dwbnq_dwconv_bwd hands to the forward kernels (when dx is overwritten)."""
    return s == 1 and dil == 1 and mult == 1 and k % 2 == 1 and p == k // 2


def check_dx(got, want, mag, exact, what):
    if exact:
        same_bits(got, want, what)
    else:
        assert np.all(np.abs(got - want) <= 2e-6 * mag + 1e-30), what


def _x_for_quantizers(rng, n):
    x = (rng.standard_normal(n) * 6).astype(np.float32)
    x[:8] = [0.0, -0.0, np.nan, np.inf, -np.inf, 7.9375, -7.9375, 2.0]
    x[8:12] = np.array([0x3fb504f3, 0x3fb504f4, 0x403504f3, 0x403504f4], np.uint32).view(np.float32)  # sqrt2 flips
    return x


@pytest.mark.parametrize("fine", [True, False], ids=["fine", "plain"])
def test_fixed_point_quantize_backward(oracle, cuda_device, fine):
    rng = np.random.default_rng(1)
    for n_el in (100003, 4096, 5):
        x = _x_for_quantizers(rng, max(n_el, 12))[:n_el] if n_el >= 12 else rng.standard_normal(n_el).astype(np.float32)
        dy = rng.standard_normal(n_el).astype(np.float32)
        dy[: min(3, n_el)] = [np.nan, np.inf, -1.0][: min(3, n_el)]
        old = rng.standard_normal(n_el).astype(np.float32)
        for sign, n, delta in ((True, 8, 2.0 ** -4), (False, 8, 2.0 ** -3), (True, 4, 0.3)):
            want = oracle.fpq_bwd(x, dy, None, sign, n, delta, fine)
            got = ops.fixed_point_quantize_backward(dev(dy, cuda_device), dev(x, cuda_device), sign, n, delta, fine)
            same_bits(got.cpu().numpy(), want, "fpq bwd")
            want = oracle.fpq_bwd(x, dy, old, sign, n, delta, fine)
            acc = dev(old, cuda_device)
            ops.fixed_point_quantize_backward(dev(dy, cuda_device), dev(x, cuda_device), sign, n, delta, fine, dx=acc,
                                              accum=True)
            same_bits(acc.cpu().numpy(), want, "fpq bwd accum")
    # fp16 tensors: same rule on the up-cast values, one rounding of the sum
    xh, dyh = x.astype(np.float16), dy.astype(np.float16)
    want = oracle.fpq_bwd(xh.astype(np.float32), dyh.astype(np.float32), None, True, 8, 2.0 ** -4, fine).astype(np.float16)
    got = ops.fixed_point_quantize_backward(dev(dyh, cuda_device), dev(xh, cuda_device), True, 8, 2.0 ** -4, fine)
    g16 = got.cpu().numpy()
    assert np.array_equal(np.isnan(g16), np.isnan(want))
    np.testing.assert_array_equal(g16.view(np.uint16)[~np.isnan(want)], want.view(np.uint16)[~np.isnan(want)])
    ops.check_device_flag()


@pytest.mark.parametrize("fine", [True, False], ids=["fine", "plain"])
def test_pow2_quantize_backward(oracle, cuda_device, fine):
    rng = np.random.default_rng(2)
    x = _x_for_quantizers(rng, 200003)
    dy = rng.standard_normal(x.size).astype(np.float32)
    old = rng.standard_normal(x.size).astype(np.float32)
    for sign, wz, n, m in ((True, True, 8, 1), (False, True, 8, 0), (True, False, 6, 3), (False, False, 4, -2),
                           (True, True, 3, 120)):
        want = oracle.pow2q_bwd(x, dy, None, sign, wz, n, m, fine, nthreads=oracle.max_threads())
        got = ops.pow2_quantize_backward(dev(dy, cuda_device), dev(x, cuda_device), sign, wz, n, m, fine)
        same_bits(got.cpu().numpy(), want, "pow2 bwd %s" % ((sign, wz, n, m),))
        want = oracle.pow2q_bwd(x, dy, old, sign, wz, n, m, fine, nthreads=oracle.max_threads())
        acc = dev(old, cuda_device)
        ops.pow2_quantize_backward(dev(dy, cuda_device), dev(x, cuda_device), sign, wz, n, m, fine, dx=acc, accum=True)
        same_bits(acc.cpu().numpy(), want, "pow2 bwd accum")
    ops.check_device_flag()


GEOMS = [  # n, c, h, w, k, stride, pad, dil, mult
    (3, 8, 14, 14, 3, 1, 1, 1, 1), (2, 6, 28, 28, 3, 2, 1, 1, 1), (2, 5, 15, 9, 5, 1, 2, 1, 1),
    (2, 4, 16, 16, 5, 2, 2, 1, 1), (2, 3, 12, 13, 3, 1, 2, 2, 2), (1, 4, 10, 10, 4, 3, 1, 1, 1),
    (2, 3, 9, 9, 2, 2, 0, 1, 3),
    # 3x3 stride 1 pad 1: the register-window weight-gradient kernel, 16-byte rows and not, one band and
    # several, more column blocks than lanes, a plane smaller than a block, a multiplier
    (2, 5, 12, 16, 3, 1, 1, 1, 1), (2, 3, 9, 40, 3, 1, 1, 1, 2), (1, 2, 5, 132, 3, 1, 1, 1, 1), (3, 2, 3, 3, 3, 1, 1, 1, 1),
    (2, 4, 7, 7, 3, 1, 1, 1, 1), (9, 2, 28, 28, 3, 1, 1, 1, 1), (2, 2, 1, 6, 3, 1, 1, 1, 1),
    # 3x3 stride 2 pad 1: the same window over nine input columns; odd and even planes, 16-byte rows of x only /
    # of x and dy / of neither, more column blocks than lanes, a multiplier
    (2, 3, 9, 13, 3, 2, 1, 1, 1), (3, 4, 56, 56, 3, 2, 1, 1, 1), (2, 3, 14, 14, 3, 2, 1, 1, 2), (1, 2, 5, 264, 3, 2, 1, 1, 1),
    (2, 2, 1, 1, 3, 2, 1, 1, 1), (9, 2, 7, 12, 3, 2, 1, 1, 1)]


@pytest.mark.parametrize("geom", GEOMS, ids=lambda g: "x".join(str(v) for v in g))
def test_depthwise_convolution_backward(oracle, cuda_device, geom):
    n, c, h, w_, k, s, p, dil, mult = geom
    rng = np.random.default_rng(sum(geom))
    x = rng.standard_normal((n, c, h, w_)).astype(np.float32)
    w = (rng.standard_normal((c * mult, k, k)) / k).astype(np.float32)
    ho, wo = oracle.conv_out_size(h, k, s, p, dil), oracle.conv_out_size(w_, k, s, p, dil)
    dy = rng.standard_normal((n, c * mult, ho, wo)).astype(np.float32)
    wdx, wdw, wdb = oracle.dwconv_bwd(x, w, dy, (s, s), (p, p), (dil, dil), mult)
    tx, tw, tdy = dev(x, cuda_device), dev(w, cuda_device), dev(dy, cuda_device)
    dx, dw, db = ops.depthwise_convolution_backward(tx, tw, tdy, 1, (p, p), (s, s), (dil, dil), mult)
    torch.cuda.synchronize()
    # tolerance of a sum of N rounded products: a few ulps of the sum of magnitudes
    mag_x, mag_w, _ = oracle.dwconv_bwd(np.abs(x), np.abs(w), np.abs(dy), (s, s), (p, p), (dil, dil), mult)
    check_dx(dx.cpu().numpy(), wdx, mag_x, not by_forward(k, s, p, dil, mult), "dx %s" % (geom,))
    assert np.all(np.abs(dw.cpu().numpy() - wdw) <= 4e-6 * mag_w + 1e-30), geom
    assert np.all(np.abs(db.cpu().numpy() - wdb) <= 4e-6 * np.abs(dy).sum(axis=(0, 2, 3)) + 1e-30), geom
    # accumulation onto existing gradients, and gradients that are not asked for
    o_dx, o_dw, o_db = (rng.standard_normal(a.shape).astype(np.float32) for a in (x, w, wdb))
    wdx2, wdw2, wdb2 = oracle.dwconv_bwd(x, w, dy, (s, s), (p, p), (dil, dil), mult, dx=o_dx, dw=o_dw, db=o_db)
    a_dx, a_dw, a_db = dev(o_dx, cuda_device), dev(o_dw, cuda_device), dev(o_db, cuda_device)
    ops.depthwise_convolution_backward(tx, tw, tdy, 1, (p, p), (s, s), (dil, dil), mult, dx=a_dx, dw=a_dw, db=a_db,
                                       accum=(True, True, True))
    same_bits(a_dx.cpu().numpy(), wdx2, "dx accum")
    assert np.all(np.abs(a_dw.cpu().numpy() - wdw2) <= 4e-6 * (mag_w + np.abs(o_dw)) + 1e-30)
    assert np.all(np.abs(a_db.cpu().numpy() - wdb2) <= 4e-6 * (np.abs(dy).sum(axis=(0, 2, 3)) + np.abs(o_db)) + 1e-30)
    only_dx = ops.depthwise_convolution_backward(tx, tw, tdy, 1, (p, p), (s, s), (dil, dil), mult,
                                                 need=(True, False, False))
    assert only_dx[1] is None and only_dx[2] is None
    check_dx(only_dx[0].cpu().numpy(), wdx, mag_x, not by_forward(k, s, p, dil, mult), "dx alone")
    only_db = ops.depthwise_convolution_backward(tx, tw, tdy, 1, (p, p), (s, s), (dil, dil), mult,
                                                 need=(False, False, True))
    assert np.all(np.abs(only_db[2].cpu().numpy() - wdb) <= 4e-6 * np.abs(dy).sum(axis=(0, 2, 3)) + 1e-30)
    ops.check_device_flag()


def test_depthwise_convolution_backward_cfg1_layer_sizes(oracle, cuda_device):
    """Two layer shapes of the MobileNetV2 stack at 16 images: many slices per channel."""
    rng = np.random.default_rng(5)
    for c, hw, s in ((96, 112, 2), (384, 14, 1), (144, 56, 1)):
        x = rng.standard_normal((16, c, hw, hw)).astype(np.float32)
        w = (rng.standard_normal((c, 3, 3)) / 3).astype(np.float32)
        ho = oracle.conv_out_size(hw, 3, s, 1)
        dy = rng.standard_normal((16, c, ho, ho)).astype(np.float32)
        wdx, wdw, wdb = oracle.dwconv_bwd(x, w, dy, (s, s), (1, 1), nthreads=oracle.max_threads())
        dx, dw, db = ops.depthwise_convolution_backward(dev(x, cuda_device), dev(w, cuda_device), dev(dy, cuda_device),
                                                        1, (1, 1), (s, s))
        mag_x = oracle.dwconv_bwd(np.abs(x), np.abs(w), np.abs(dy), (s, s), (1, 1), nthreads=oracle.max_threads())[0]
        check_dx(dx.cpu().numpy(), wdx, mag_x, s != 1, "dx cfg1 %d" % hw)
        scale = np.sqrt(16 * ho * ho)  # random signs: the sum of magnitudes grows like N, the error like sqrt(N)
        assert np.all(np.abs(dw.cpu().numpy() - wdw) <= 2e-6 * 16 * ho * ho / scale + 1e-5 * np.abs(wdw))
        assert np.all(np.abs(db.cpu().numpy() - wdb) <= 2e-6 * 16 * ho * ho / scale + 1e-5 * np.abs(wdb))
    ops.check_device_flag()


def test_direct_input_gradient_is_bit_exact_when_forced(oracle, cuda_device):
    """DWBNQ_BWD_INPUT_DIRECT=1 (read once per process: a child process) keeps the stride-1
    input gradient on the direct kernel, whose sum runs in the reference's order."""
    import os
    import subprocess
    import sys
    code = (
        "import sys, numpy as np, torch\n"
        "sys.path[:0] = [%r, %r]\n"
        "from dwbnq import ops\n"
        "from oracle import oracle\n"
        "rng = np.random.default_rng(3)\n"
        "for k, hw in ((3, 28), (5, 14), (3, 9)):\n"
        "    x = rng.standard_normal((4, 16, hw, hw)).astype(np.float32)\n"
        "    w = rng.standard_normal((16, k, k)).astype(np.float32)\n"
        "    dy = rng.standard_normal((4, 16, hw, hw)).astype(np.float32)\n"
        "    want = oracle.dwconv_bwd(x, w, dy, (1, 1), (k // 2, k // 2))[0]\n"
        "    t = lambda a: torch.from_numpy(a).cuda()\n"
        "    got = ops.depthwise_convolution_backward(t(x), t(w), t(dy), 1, (k // 2,) * 2, (1, 1), need=(True, False, False))[0]\n"
        "    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32)), (k, hw)\n"
        "print('direct-ok')\n") % (ROOT, os.path.join(ROOT, "nnabla-ext-cuda_b200", "python"))
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, DWBNQ_BWD_INPUT_DIRECT="1"),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "direct-ok" in r.stdout, r.stderr[-2000:]


def test_backward_argument_errors(cuda_device):
    x = torch.zeros((1, 4, 8, 8), device=cuda_device)
    w = torch.zeros((4, 3, 3), device=cuda_device)
    with pytest.raises(ValueError):
        ops.depthwise_convolution_backward(x, w, torch.zeros((1, 4, 5, 5), device=cuda_device), 1, (1, 1))
    with pytest.raises(L.DwbnqError) as e:
        ops.depthwise_convolution_backward(x.half(), w.half(), torch.zeros((1, 4, 8, 8), device=cuda_device).half(), 1,
                                           (1, 1))
    assert e.value.status == L.ERR_UNSUPPORTED
    with pytest.raises(L.DwbnqError) as e:
        ops.fixed_point_quantize_backward(torch.zeros(4, device=cuda_device), None, True, 8, 0.5, True)
    assert e.value.status == L.ERR_INVALID_ARG
