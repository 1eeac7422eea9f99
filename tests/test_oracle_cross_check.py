"""The CPU oracle against independent implementations of the same mathematics (PyTorch's CPU
operators in fp32 / fp64 and float64 NumPy formulas). These cannot pin the oracle bit for bit
- the summation order and rounding points of another library are its own - but they bound
how far the restatement can be from the functions it restates: convolution and BN agree to a
few ulps, the quantizers agree exactly with their double-precision definitions wherever
those definitions are not within rounding distance of a decision threshold."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F


@pytest.mark.parametrize("k,stride,pad,dil,mult", [(3, 1, 1, 1, 1), (3, 2, 1, 1, 1), (5, 1, 2, 1, 1), (3, 1, 2, 2, 1),
                                                  (3, 1, 0, 1, 2), (1, 1, 0, 1, 1)])
def test_dwconv_against_torch_grouped_convolution(oracle, k, stride, pad, dil, mult):
    rng = np.random.default_rng(k * 10 + stride)
    n, c, h, w = 3, 6, 19, 23
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (rng.standard_normal((c * mult, k, k)) / k).astype(np.float32)
    b = rng.standard_normal(c * mult).astype(np.float32)
    got = oracle.dwconv(x, wt, b, (stride, stride), (pad, pad), (dil, dil), mult)
    want64 = F.conv2d(torch.from_numpy(x).double(), torch.from_numpy(wt).double()[:, None], torch.from_numpy(b).double(),
                      stride=stride, padding=pad, dilation=dil, groups=c).numpy()
    assert got.shape == want64.shape
    # fp32 accumulation of at most 26 terms of magnitude ~1 against the fp64 result
    np.testing.assert_allclose(got, want64, rtol=0, atol=2e-6 * k * k)


def test_bn_against_torch_batch_norm_eval(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 9, 7, 5)).astype(np.float32)
    p = {k: (rng.random(9) + 0.5).astype(np.float32) for k in ("beta", "gamma", "mean", "var")}
    got = oracle.bn_infer(x, p["beta"], p["gamma"], p["mean"], p["var"], 1e-5)
    want64 = F.batch_norm(torch.from_numpy(x).double(), torch.from_numpy(p["mean"]).double(),
                          torch.from_numpy(p["var"]).double(), torch.from_numpy(p["gamma"]).double(),
                          torch.from_numpy(p["beta"]).double(), training=False, eps=1e-5).numpy()
    np.testing.assert_allclose(got, want64, rtol=5e-7, atol=5e-7)  # four fp32 roundings


def test_fpq_against_its_double_precision_definition(oracle):
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(200000).astype(np.float32) * 4, np.linspace(-9, 9, 2881, dtype=np.float32)])
    for sign, n, delta in ((True, 8, 2.0 ** -4), (False, 8, 2.0 ** -3), (True, 5, 0.17), (False, 3, 1.5)):
        d = np.float32(delta)
        mx = np.float32((2 ** (n - (1 if sign else 0)) - 1)) * d
        mn = -mx if sign else np.float32(0)
        # the reference kernel (fixed_point_quantize.cu:44): the quotient of two floats is a
        # float; "+ 0.5", floor and the product with delta run in double; one cast to float
        t = (np.abs(x) / d).astype(np.float32).astype(np.float64)
        q = (np.sign(x.astype(np.float64)) * np.floor(t + 0.5) * np.float64(d)).astype(np.float32)
        want = np.where(x > mx, mx, np.where(x < mn, mn, q)).astype(np.float32)
        got = oracle.fpq(x, sign, n, delta)
        assert np.array_equal(got.view(np.uint32) & 0x7fffffff, want.view(np.uint32) & 0x7fffffff), (sign, n, delta)
        nz = want != 0
        assert np.array_equal(got[nz], want[nz])


def test_pow2_against_its_definition_away_from_thresholds(oracle):
    rng = np.random.default_rng(7)
    x = (rng.standard_normal(300000) * np.exp(rng.standard_normal(300000) * 3)).astype(np.float32)
    x = x[x != 0]
    sign, with_zero, n, m = True, True, 8, 1
    l2 = np.log2(np.abs(x.astype(np.float64)))
    away = np.abs(l2 - np.floor(l2) - 0.5) > 1e-5      # not within rounding distance of a .5 exponent
    ref_exp = np.round(l2)
    p_max, p_min = 2.0 ** m, 2.0 ** (m - (2 ** (n - 2) - 1))
    q = np.exp2(ref_exp)
    q = np.where(q > p_max, p_max, q)
    q = np.where(q < p_min, np.where(np.abs(x) < p_min * 2 ** -0.5, 0.0, p_min), q)
    want = (np.sign(x) * q).astype(np.float32)
    got = oracle.pow2q(x, sign, with_zero, n, m)
    edge = np.abs(np.abs(x.astype(np.float64)) / (p_min * 2 ** -0.5) - 1) < 1e-5
    ok = away & ~edge
    assert ok.mean() > 0.99
    assert np.array_equal(got[ok], want[ok])


def test_minmax_against_its_definition(oracle):
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((4, 5, 6, 7)) * 3).astype(np.float32)
    c = 5
    y, qmin, qmax = oracle.minmaxq(x, np.zeros(c, np.float32), np.ones(c, np.float32), np.zeros(c, np.float32),
                                   np.full(c, 255, np.float32), 0.999, True, False, 0.01)
    np.testing.assert_array_equal(qmin, x.min(axis=(0, 2, 3)))
    np.testing.assert_array_equal(qmax, x.max(axis=(0, 2, 3)))
    scale = (qmax.astype(np.float64) - qmin) / 255.0
    # 256 levels per channel, each within half a step of the input, ends of the range kept to a step
    for ch in range(c):
        yc, xc = y[:, ch].astype(np.float64), x[:, ch].astype(np.float64)
        assert np.unique(y[:, ch]).size <= 256
        assert np.abs(yc - xc).max() <= scale[ch] * (1.0 + 1e-4)


def test_backward_restatements_against_autograd(oracle):
    """The oracle's DepthwiseConvolution gradients against PyTorch's autograd of the grouped
    convolution in fp64, and the STE rules against their definitions."""
    import torch
    rng = np.random.default_rng(8)
    for (n, c, h, w_, k, s, p, dil, mult) in ((2, 4, 9, 11, 3, 1, 1, 1, 1), (2, 3, 12, 12, 5, 2, 2, 1, 2),
                                              (1, 2, 10, 10, 3, 2, 0, 2, 1)):
        x = rng.standard_normal((n, c, h, w_)).astype(np.float32)
        w = rng.standard_normal((c * mult, k, k)).astype(np.float32)
        tx = torch.tensor(x, dtype=torch.float64, requires_grad=True)
        tw = torch.tensor(w, dtype=torch.float64, requires_grad=True)
        tb = torch.zeros(c * mult, dtype=torch.float64, requires_grad=True)
        y = torch.nn.functional.conv2d(tx, tw[:, None], tb, stride=s, padding=p, dilation=dil, groups=c)
        dy = rng.standard_normal(tuple(y.shape)).astype(np.float32)
        y.backward(torch.tensor(dy, dtype=torch.float64))
        dx, dw, db = oracle.dwconv_bwd(x, w, dy, (s, s), (p, p), (dil, dil), mult)
        np.testing.assert_allclose(dx, tx.grad.numpy(), rtol=2e-5, atol=2e-5)
        np.testing.assert_allclose(dw, tw.grad.numpy(), rtol=2e-5, atol=2e-5)
        np.testing.assert_allclose(db, tb.grad.numpy(), rtol=2e-5, atol=2e-5)
    x = np.array([0.0, 8.5, -8.5, 1.0, -1.0, 7.9375, np.nan], np.float32)
    dy = np.arange(1, 8, dtype=np.float32)
    # FixedPointQuantize(sign, n = 8, 2^-4): range [-7.9375, 7.9375]; clipped elements get 0
    np.testing.assert_array_equal(oracle.fpq_bwd(x, dy, None, True, 8, 2.0 ** -4, True), [1, 0, 0, 4, 5, 6, 7])
    np.testing.assert_array_equal(oracle.fpq_bwd(x, dy, None, True, 8, 2.0 ** -4, False), dy)
    np.testing.assert_array_equal(oracle.fpq_bwd(x, dy, np.ones(7, np.float32), True, 8, 2.0 ** -4, True),
                                  [2, 1, 1, 5, 6, 7, 8])
    # Pow2Quantize(sign, with_zero, n = 8, m = 1): p_max = 2; 3.0 rounds to 4 > 2 -> 0; unsigned: negatives -> 0
    xp = np.array([3.0, 2.5, -3.0, -0.3, 0.0], np.float32)
    np.testing.assert_array_equal(oracle.pow2q_bwd(xp, dy[:5], None, True, True, 8, 1, True), [0, 2, 0, 4, 5])
    np.testing.assert_array_equal(oracle.pow2q_bwd(xp, dy[:5], None, False, True, 8, 1, True), [0, 2, 0, 0, 5])
