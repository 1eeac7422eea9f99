"""Pins the CPU oracle to the known answers derived by hand from the nnabla-ext-cuda
sources (tests/golden/known_answers.json) and to formula-level properties of the same
sources. nnabla core is not installed, so these are the only reference-derived vectors."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
KA = json.load(open(os.path.join(HERE, "golden", "known_answers.json")))


def _vals(lst):
    out = []
    for v in lst:
        if isinstance(v, str):
            out.append(np.array([int(v, 16)], dtype=np.uint32).view(np.float32)[0])
        else:
            out.append(np.float32(v))
    return np.array(out, dtype=np.float32)


def _bits(lst):
    return np.array([0x7fc00000 if v == "nan" else int(v, 16) for v in lst], dtype=np.uint32)


def _assert_bits(got, want_bits_list):
    got_bits = np.asarray(got, np.float32).view(np.uint32)
    for g, w, gv in zip(got_bits, want_bits_list, got):
        if w == "nan":
            assert np.isnan(gv)
        else:
            assert g == int(w, 16), "got 0x%08x want %s" % (g, w)


@pytest.mark.parametrize("case", KA["fixed_point_quantize"]["cases"])
def test_fpq_known_answers(oracle, case):
    if "x" in case:
        y = oracle.fpq(_vals(case["x"]), case["sign"], case["n"], case["delta"])
        np.testing.assert_array_equal(y, _vals(case["y"]))
    else:
        x = _bits(case["x_bits"]).view(np.float32)
        _assert_bits(oracle.fpq(x, case["sign"], case["n"], case["delta"]), case["y_bits"])


def test_fpq_range_formula(oracle):
    assert oracle.fpq_params(True, 8, 2.0 ** -4) == (7.9375, -7.9375)
    assert oracle.fpq_params(False, 8, 2.0 ** -3) == (31.875, 0.0)


@pytest.mark.parametrize("case", KA["pow2_quantize"]["cases"])
def test_pow2_known_answers(oracle, case):
    args = (case["sign"], case["with_zero"], case["n"], case["m"])
    if "params" in case:
        p_max, p_min, thr = oracle.pow2q_params(*args)
        assert p_max == case["params"]["p_max"]
        assert np.float32(p_min).view(np.uint32) == int(case["params"]["p_min_bits"], 16)
        assert thr == np.float32(np.float64(p_min) * 2.0 ** -0.5)
    if "x" in case:
        np.testing.assert_array_equal(oracle.pow2q(_vals(case["x"]), *args), _vals(case["y"]))
    else:
        x = _bits(case["x_bits"]).view(np.float32)
        _assert_bits(oracle.pow2q(x, *args), case["y_bits"])


def test_pow2_unsigned_variants(oracle):
    # sign=False: negative inputs give 0 (with_zero) or p_min (without), pow2_quantize.cu:54-60
    x = np.array([-3.0, 3.0, 0.3], np.float32)
    y = oracle.pow2q(x, False, True, 8, 1)
    np.testing.assert_array_equal(y, np.array([0.0, 2.0, 0.25], np.float32))
    y = oracle.pow2q(x, False, False, 4, 0)  # n_eff = 4 -> p_min = 2^-15, p_max = 1
    np.testing.assert_array_equal(y, np.array([2.0 ** -15, 1.0, 0.25], np.float32))


@pytest.mark.parametrize("case", KA["batch_normalization"]["cases"])
def test_bn_known_answers(oracle, case):
    x = np.array(case["x"], np.float32).reshape(1, 1, -1)
    g = None if case["gamma"] is None else np.array([case["gamma"]], np.float32)
    b = None if case["beta"] is None else np.array([case["beta"]], np.float32)
    y = oracle.bn_infer(x, b, g, np.array([case["mean"]], np.float32), np.array([case["var"]], np.float32),
                        case["eps"])
    np.testing.assert_array_equal(y.ravel(), np.array(case["y"], np.float32))


def test_bn_mean_maps_to_beta_and_axis(oracle):
    rng = np.random.default_rng(0)
    C = 5
    mean = rng.standard_normal(C).astype(np.float32)
    var = (rng.random(C) + 0.5).astype(np.float32)
    gamma = (rng.random(C) + 0.5).astype(np.float32)
    beta = rng.standard_normal(C).astype(np.float32)
    x = np.broadcast_to(mean.reshape(1, C, 1, 1), (2, C, 3, 4)).copy()
    y = oracle.bn_infer(x, beta, gamma, mean, var, 1e-5)
    np.testing.assert_array_equal(y, np.broadcast_to(beta.reshape(1, C, 1, 1), y.shape))
    # op order: ((x - mean) * gamma) / sqrt(var + eps) + beta, every op rounded to float32
    x = rng.standard_normal((2, C, 3, 4)).astype(np.float32)
    want = ((x - mean.reshape(1, C, 1, 1)) * gamma.reshape(1, C, 1, 1)) / np.sqrt(
        var.reshape(1, C, 1, 1) + np.float32(1e-5)) + beta.reshape(1, C, 1, 1)
    np.testing.assert_array_equal(oracle.bn_infer(x, beta, gamma, mean, var, 1e-5), want.astype(np.float32))
    # channel-last view (axis 3)
    xl = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
    yl = oracle.bn_infer(xl, beta, gamma, mean, var, 1e-5, axis=3)
    np.testing.assert_array_equal(yl.transpose(0, 3, 1, 2), want.astype(np.float32))


@pytest.mark.parametrize("case", KA["depthwise_convolution"]["cases"])
def test_dwconv_known_answers(oracle, case):
    C = 3
    x = np.ones((2, C, case["h"], case["w"]), np.float32)
    w = np.ones((C, case["k"], case["k"]), np.float32)
    b = None if case["bias"] is None else np.full(C, case["bias"], np.float32)
    y = oracle.dwconv(x, w, b, (case["stride"],) * 2, (case["pad"],) * 2)
    want = np.array(case["y"], np.float32)
    assert y.shape == (2, C) + want.shape
    for n in range(2):
        for c in range(C):
            np.testing.assert_array_equal(y[n, c], want)


def test_dwconv_tap_order_and_multiplier(oracle):
    """ky-major / kx-minor accumulation starting from the bias, products and sums rounded
    separately (depthwise_convolution.cu:92-108), and oc -> ic = oc / multiplier (:89)."""
    rng = np.random.default_rng(1)
    N, C, H, W, mult, k = 2, 3, 6, 7, 2, 3
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = rng.standard_normal((C * mult, k, k)).astype(np.float32)
    b = rng.standard_normal(C * mult).astype(np.float32)
    y = oracle.dwconv(x, w, b, (2, 1), (1, 0), (1, 2), mult)
    Ho = (H + 2 - 2 - 1) // 2 + 1
    Wo = (W + 0 - 2 * 2 - 1) // 1 + 1
    assert y.shape == (N, C * mult, Ho, Wo)
    for n in range(N):
        for oc in range(C * mult):
            for oy in range(Ho):
                for ox in range(Wo):
                    v = np.float32(b[oc])
                    for ky in range(k):
                        for kx in range(k):
                            iy, ix = oy * 2 + ky - 1, ox + kx * 2
                            if 0 <= iy < H and 0 <= ix < W:
                                v = np.float32(v + np.float32(w[oc, ky, kx] * x[n, oc // mult, iy, ix]))
                    assert y[n, oc, oy, ox] == v


@pytest.mark.parametrize("case", KA["min_max_quantize"]["cases"])
def test_minmax_known_answers(oracle, case):
    x = np.array(case["x"], np.float32).reshape(1, 1, -1)
    one = lambda v: np.array([v], np.float32)
    y, qmin, qmax = oracle.minmaxq(x, one(7.0), one(9.0), one(case["ql_min"]), one(case["ql_max"]),
                                   x_min_max=True, ema=False, eps=case["eps"])
    np.testing.assert_array_equal(y.ravel(), np.array(case["y"], np.float32))
    assert qmin[0] == case["qr_min"] and qmax[0] == case["qr_max"]


def test_minmax_constant_channel_is_nudged(oracle):
    """qr_max - qr_min < eps -> qr_max = qr_min + eps (min_max_quantize.cu:32-35); then the
    zero point clamps to ql_min and every value lands on M' = 255 * scale."""
    f = np.float32
    x = np.full((2, 1, 3), 1.5, np.float32)
    y, qmin, qmax, scale, lo, hi = oracle.minmaxq(x, [0.0], [0.0], [0.0], [255.0], x_min_max=True, eps=0.01,
                                                  return_ranges=True)
    assert qmin[0] == f(1.5) and qmax[0] == f(1.5) + f(0.01)
    s = f(f(qmax[0] - qmin[0]) / f(255.0))
    assert scale[0] == s and lo[0] == f(0.0) and hi[0] == f(f(255.0) * s)
    want = f(f(np.round(f(hi[0] / s)) * s) + f(0.0))
    np.testing.assert_array_equal(y, np.full_like(x, want))


def test_minmax_ema_and_fixed_ranges(oracle):
    f = np.float32
    x = np.array([[-2.0, 0.0, 6.0]], np.float32).reshape(1, 1, 3)
    _, qmin, qmax = oracle.minmaxq(x, [-1.0], [1.0], [0.0], [255.0], decay=0.75, x_min_max=True, ema=True)
    assert qmin[0] == f(f(0.75) * f(-1.0) + f(0.25) * f(-2.0))
    assert qmax[0] == f(f(0.75) * f(1.0) + f(0.25) * f(6.0))
    # x_min_max=False: the given ranges are used and left untouched
    y, qmin, qmax = oracle.minmaxq(x, [0.0], [255.0], [0.0], [255.0], x_min_max=False)
    assert qmin[0] == 0.0 and qmax[0] == 255.0
    np.testing.assert_array_equal(y.ravel(), np.array([0.0, 0.0, 6.0], np.float32))


def test_threads_do_not_change_results(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 4, 9, 9)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3)).astype(np.float32)
    a = oracle.dwconv(x, w, None, (1, 1), (1, 1), nthreads=1)
    b = oracle.dwconv(x, w, None, (1, 1), (1, 1), nthreads=4)
    np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(oracle.fpq(x, nthreads=1), oracle.fpq(x, nthreads=4))


def test_quantize_linear_known_answers(oracle):
    """Worked from src/nbla/cuda/function/generic/quantize_linear.cu: round() is half away from
    zero (:33-35); half to even replaces exact .5 cases by round(x * 0.5) * 2 (:37-47); saturate
    clamps to [min_range, max_range] (:22-31); the composite is x / scale + zero_point first."""
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 0.49, 300.0, -300.0, 1.0], np.float32)
    away = oracle.quantize_linear(x, 1.0, 0, "HALF_AWAY_FROM_ZERO", -128, 127)
    np.testing.assert_array_equal(away, [1, 2, 3, -1, -2, -3, 0, 127, -128, 1])
    even = oracle.quantize_linear(x, 1.0, 0, "HALF_TO_EVEN", -128, 127)
    np.testing.assert_array_equal(even, [0, 2, 2, 0, -2, -2, 0, 127, -128, 1])
    # scale and zero point: 0.3 / 0.125 + 3 = 5.4 -> 5; unsigned range clamps negatives to 0
    np.testing.assert_array_equal(oracle.quantize_linear(np.array([0.3, -1.0], np.float32), 0.125, 3,
                                                         "HALF_AWAY_FROM_ZERO", 0, 255), [5, 0])
    np.testing.assert_array_equal(oracle.dequantize_linear(np.array([5, 0, 255]), 0.125, 3),
                                  np.array([0.25, -0.375, 31.5], np.float32))
    # FixedPointQuantize(unsigned, n = 8, delta) is the dequantized code
    v = np.array([0.03, 0.0625, 0.19, 40.0, -1.0], np.float32)
    codes = oracle.quantize_linear(v, 0.125, 0, "HALF_AWAY_FROM_ZERO", 0, 255)
    np.testing.assert_array_equal(oracle.dequantize_linear(codes, 0.125, 0), oracle.fpq(v, False, 8, 0.125))


def test_pointwise_convolution_known_answers(oracle):
    """A 1x1 convolution worked by hand: y[co][p] = sum_ci w[co][ci] x[ci][p] + b[co], the bias
    added after the sum; the double accumulation, the fp32 accumulation and sum |w||x| + |b|."""
    x = np.array([[[[1.0, -2.0]], [[0.5, 4.0]], [[3.0, 0.25]]]], dtype=np.float32)  # [1, 3, 1, 2]
    w = np.array([[2.0, -1.0, 0.5], [0.0, 0.25, -4.0]], dtype=np.float32)
    b = np.array([0.125, -1.0], dtype=np.float32)
    acc32, acc64, mag = oracle.pwconv(x, w, b)
    want = np.array([[[[2 - 0.5 + 1.5 + 0.125, -4 - 4 + 0.125 + 0.125]], [[0.125 - 12 - 1, 1 - 1 - 1]]]], dtype=np.float32)
    np.testing.assert_array_equal(acc32, want)
    np.testing.assert_array_equal(acc64, want)
    np.testing.assert_array_equal(mag[0, 0, 0], [2 + 0.5 + 1.5 + 0.125, 4 + 4 + 0.125 + 0.125])
    # the weight may come as [co, ci, 1, 1]; no bias
    a32, _, m = oracle.pwconv(x, w.reshape(2, 3, 1, 1), None)
    np.testing.assert_array_equal(a32, want - b[None, :, None, None])
    # fp32 accumulation in ascending channel order: 2^24 + 1 is lost, then -2^24 leaves 0
    xx = np.array([[[[1.0]], [[1.0]], [[1.0]]]], dtype=np.float32)
    ww = np.array([[16777216.0, 1.0, -16777216.0]], dtype=np.float32)
    a32, a64, _ = oracle.pwconv(xx, ww, None)
    assert a32.item() == 0.0 and a64.item() == 1.0


def test_activations_and_pointwise_epilogue(oracle):
    v = np.array([-1.0, -0.0, 0.5, 6.0, 7.5, np.nan, np.inf, -np.inf], dtype=np.float32)
    np.testing.assert_array_equal(oracle.act(v, "relu6"), [0, 0, 0.5, 6, 6, 0, 6, 0])
    np.testing.assert_array_equal(oracle.act(v, "relu"), [0, 0, 0.5, 6, 7.5, 0, np.inf, 0])
    np.testing.assert_array_equal(oracle.act(v, None).view(np.uint32), v.view(np.uint32))
    # BN -> ReLU6 -> unsigned FixedPointQuantize equals the three oracle functions in sequence
    rng = np.random.default_rng(0)
    conv = rng.standard_normal((2, 3, 4, 5), dtype=np.float32) * 3
    beta, gamma, mean, var = (rng.standard_normal(3, dtype=np.float32), np.array([1.5, -0.5, 1.0], np.float32),
                              rng.standard_normal(3, dtype=np.float32), np.array([0.5, 1.0, 2.0], np.float32))
    q = {"kind": "fpq", "sign": False, "n": 8, "delta": 0.125}
    want = oracle.fpq(oracle.act(oracle.bn_infer(conv, beta, gamma, mean, var, 1e-5), "relu6"), False, 8, 0.125)
    np.testing.assert_array_equal(oracle.pw_epilogue(conv, beta, gamma, mean, var, 1e-5, "relu6", q), want)
    np.testing.assert_array_equal(oracle.pw_epilogue(conv, None, None, None, None, 1e-5, None, None), conv)
