"""Parity of the CUDA path (through the C ABI) with the CPU oracle on the same seeded
inputs. Quantized outputs and fp32 activations are compared bit for bit (the arithmetic
contract is "same operations, same order, each rounded once", so the 1e-5 relative
tolerance the path is allowed on pre-quantization activations is met with zero error);
fp16 results are compared bit for bit against the oracle's fp16 convention and, for the
pre-quantization activations, within 2e-3 relative of the fp32 oracle."""
import numpy as np
import pytest
import torch

from dwbnq import _lib as L
from dwbnq import ops, workloads

pytestmark = pytest.mark.gpu

PATHS = [L.PATH_AUTO, L.PATH_TMA, L.PATH_COOP, L.PATH_RAW, L.PATH_GENERIC]
PATH_IDS = ["auto", "tma", "coop", "raw", "generic"]


@pytest.fixture(autouse=True)
def _reset_path():
    yield
    ops.set_forced_path(L.PATH_AUTO)
    ops.set_tuning(0, 0, 0, 0)


def dev(a, device):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(device)


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a.view(np.uint16)


def assert_same_bits(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape and got.dtype == want.dtype, (got.shape, want.shape, got.dtype, want.dtype)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan), what + ": NaN positions differ"
    gb, wb = bits(got), bits(want)
    diff = (gb != wb) & ~nan
    if diff.any():
        idx = np.argwhere(diff)[:5]
        msg = "; ".join("%s got %r want %r" % (tuple(i), got[tuple(i)], want[tuple(i)]) for i in idx)
        raise AssertionError("%s: %d of %d elements differ: %s" % (what, int(diff.sum()), got.size, msg))


def run_fused(d, spec, device, quant=None, has_bn=True, dtype=torch.float32, path=L.PATH_AUTO, bias=True):
    ops.set_forced_path(path)
    t = {k: dev(v, device) for k, v in d.items()}
    if dtype == torch.float16:
        t = {k: v.half() for k, v in t.items()}
    q = dict(quant) if quant else None
    if q and q["kind"] == "minmax":
        for k in ("qr_min", "qr_max", "ql_min", "ql_max"):
            q[k] = t[k]
    y = ops.fused_dw_bn_quant(t["x"], t["w"], t["b"] if bias else None, t["beta"] if has_bn else None,
                              t["gamma"] if has_bn else None, t["mean"] if has_bn else None,
                              t["var"] if has_bn else None, spec.bn_eps, pad=(spec.pad, spec.pad),
                              stride=(spec.stride, spec.stride), quant=q)
    torch.cuda.synchronize()
    ops.check_device_flag()
    return y.cpu().numpy(), t


def oracle_fused(orc, d, spec, quant, has_bn=True, bias=True, nthreads=None):
    nthreads = nthreads or orc.max_threads()
    y = orc.dwconv(d["x"], d["w"], d["b"] if bias else None, (spec.stride,) * 2, (spec.pad,) * 2, nthreads=nthreads)
    if has_bn:
        y = orc.bn_infer(y, d["beta"], d["gamma"], d["mean"], d["var"], spec.bn_eps, nthreads=nthreads)
    pre = y
    kind = quant["kind"] if quant else "none"
    extra = None
    if kind == "fpq":
        y = orc.fpq(y, quant["sign"], quant["n"], quant["delta"], nthreads)
    elif kind == "pow2":
        y = orc.pow2q(y, quant["sign"], quant["with_zero"], quant["n"], quant["m"], nthreads)
    elif kind == "minmax":
        y, qmin, qmax = orc.minmaxq(y, d["qr_min"], d["qr_max"], d["ql_min"], d["ql_max"],
                                    quant.get("decay", 0.999), quant.get("x_min_max", True),
                                    quant.get("ema", False), quant.get("eps", 0.01), nthreads=nthreads)
        extra = (qmin, qmax)
    return y, pre, extra


def f16_inputs(d):
    """fp16-rounded tensors and their fp32 up-casts (what the oracle computes on)."""
    h = {k: v.astype(np.float16) for k, v in d.items()}
    return h, {k: v.astype(np.float32) for k, v in h.items()}


# ---- the benchmark configurations ------------------------------------------------------

@pytest.mark.parametrize("path", PATHS, ids=PATH_IDS)
def test_cfg0_single_layer_full_size(oracle, cuda_device, path):
    spec = workloads.cfg0()[0]
    d = workloads.make_layer_data(spec)
    q = workloads.quant_for_ops(spec)
    want, pre, _ = oracle_fused(oracle, d, spec, q)
    got, _ = run_fused(d, spec, cuda_device, q, path=path)
    assert_same_bits(got, want, "cfg0 quantized")
    got_pre, _ = run_fused(d, spec, cuda_device, None, path=path)
    assert_same_bits(got_pre, pre, "cfg0 pre-quantization")
    np.testing.assert_allclose(got_pre, pre, rtol=1e-5, atol=0)


@pytest.mark.parametrize("path", PATHS, ids=PATH_IDS)
def test_cfg1_every_layer_fp32(oracle, cuda_device, path):
    for spec in workloads.cfg1(n=3):
        d = workloads.make_layer_data(spec)
        q = workloads.quant_for_ops(spec)
        want, _, _ = oracle_fused(oracle, d, spec, q)
        got, _ = run_fused(d, spec, cuda_device, q, path=path)
        assert_same_bits(got, want, spec.name)


@pytest.mark.parametrize("path", PATHS, ids=PATH_IDS)
def test_cfg2_pow2_5x5(oracle, cuda_device, path):
    spec = workloads.cfg2(n=3)[0]
    d = workloads.make_layer_data(spec)
    q = workloads.quant_for_ops(spec)
    want, pre, _ = oracle_fused(oracle, d, spec, q)
    got, _ = run_fused(d, spec, cuda_device, q, path=path)
    assert_same_bits(got, want, "cfg2 pow2")
    got_pre, _ = run_fused(d, spec, cuda_device, None, path=path)
    assert_same_bits(got_pre, pre, "cfg2 pre-quantization")


@pytest.mark.parametrize("path", PATHS, ids=PATH_IDS)
def test_cfg3_minmax_stride2(oracle, cuda_device, path):
    spec = workloads.cfg3(n=16)[0]
    d = workloads.make_layer_data(spec)
    q = workloads.quant_for_ops(spec, d)
    want, _, (qmin, qmax) = oracle_fused(oracle, d, spec, q)
    got, t = run_fused(d, spec, cuda_device, q, path=path)
    assert_same_bits(got, want, "cfg3 minmax")
    np.testing.assert_array_equal(t["qr_min"].cpu().numpy(), qmin)
    np.testing.assert_array_equal(t["qr_max"].cpu().numpy(), qmax)
    # the result sits on at most 256 levels per channel
    for c in range(0, spec.c, 37):
        assert np.unique(got[:, c]).size <= 256


@pytest.mark.parametrize("path", PATHS, ids=PATH_IDS)
def test_cfg4_every_layer_fp16(oracle, cuda_device, path):
    for spec in workloads.cfg1(n=2):
        d = workloads.make_layer_data(spec)
        h, up = f16_inputs(d)
        q = workloads.quant_for_ops(spec)
        want32, pre32, _ = oracle_fused(oracle, up, spec, q)
        got, _ = run_fused(h, spec, cuda_device, q, dtype=torch.float16, path=path)
        assert got.dtype == np.float16
        assert_same_bits(got, oracle.to_f16_result(want32), spec.name + " fp16 quantized")
        got_pre, _ = run_fused(h, spec, cuda_device, None, dtype=torch.float16, path=path)
        assert_same_bits(got_pre, oracle.to_f16_result(pre32), spec.name + " fp16 pre-quantization")
        np.testing.assert_allclose(got_pre.astype(np.float32), pre32, rtol=2e-3, atol=1e-6)


def test_fp16_pow2_and_minmax(oracle, cuda_device):
    spec = workloads.cfg2(n=2)[0]
    h, up = f16_inputs(workloads.make_layer_data(spec))
    q = workloads.quant_for_ops(spec)
    want32, _, _ = oracle_fused(oracle, up, spec, q)
    got, _ = run_fused(h, spec, cuda_device, q, dtype=torch.float16)
    assert_same_bits(got, oracle.to_f16_result(want32), "cfg2 fp16")
    spec = workloads.cfg3(n=4)[0]
    h, up = f16_inputs(workloads.make_layer_data(spec))
    q = workloads.quant_for_ops(spec, up)
    want32, _, (qmin, qmax) = oracle_fused(oracle, up, spec, q)
    got, t = run_fused(h, spec, cuda_device, q, dtype=torch.float16)
    assert_same_bits(got, oracle.to_f16_result(want32), "cfg3 fp16")
    np.testing.assert_array_equal(t["qr_min"].cpu().numpy(), qmin.astype(np.float16))
    np.testing.assert_array_equal(t["qr_max"].cpu().numpy(), qmax.astype(np.float16))


# ---- shapes that exercise every code path of the tiled family ----------------------------

def _rand_layer(rng, n, c, h, w, k):
    return {"x": rng.standard_normal((n, c, h, w)).astype(np.float32),
            "w": (rng.standard_normal((c, k, k)) / k).astype(np.float32),
            "b": rng.standard_normal(c).astype(np.float32),
            "mean": rng.standard_normal(c).astype(np.float32) * 0.3,
            "var": (rng.random(c) + 0.5).astype(np.float32),
            "gamma": (rng.random(c) * 0.4 + 0.8).astype(np.float32),
            "beta": rng.standard_normal(c).astype(np.float32) * 0.3}


@pytest.mark.parametrize("path", [L.PATH_AUTO, L.PATH_COOP, L.PATH_RAW], ids=["auto", "coop", "raw"])
@pytest.mark.parametrize("k,stride", [(3, 1), (3, 2), (5, 1), (5, 2)])
def test_edge_shapes(oracle, cuda_device, path, k, stride):
    """Planes smaller than a patch, widths that are not a vector multiple, heights that are
    not a multiple of the 7-row patch, plane counts that do not fill the last CTA."""
    rng = np.random.default_rng(100 * k + stride)
    q = {"kind": "fpq", "sign": True, "n": 8, "delta": 2.0 ** -4}
    shapes = [(1, 1), (2, 3), (3, 2), (4, 4), (5, 9), (7, 7), (8, 8), (9, 5), (13, 17), (16, 16), (15, 20),
              (29, 12), (57, 8), (8, 60)]
    for (h, w) in shapes:
        if h + 2 * (k // 2) < k or w + 2 * (k // 2) < k:
            continue
        for (n, c) in ((1, 1), (2, 5), (3, 37)):
            spec = workloads.LayerSpec("edge", n, c, h, w, k, stride, k // 2, q)
            d = _rand_layer(rng, n, c, h, w, k)
            want, _, _ = oracle_fused(oracle, d, spec, q, nthreads=1)
            got, _ = run_fused(d, spec, cuda_device, q, path=path)
            assert_same_bits(got, want, "edge %dx%d n%d c%d k%d s%d" % (h, w, n, c, k, stride))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
def test_row_tiled_planes_and_tuning_overrides(oracle, cuda_device, dtype):
    """Planes tall enough to be split into several row tiles (halo rows re-read by the
    neighbouring CTA), and the planner overrides used for tuning."""
    rng = np.random.default_rng(7)
    q = {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3}
    for (h, w, k, s) in ((112, 112, 3, 1), (112, 112, 3, 2), (224, 96, 3, 1), (120, 40, 5, 2), (300, 24, 3, 1)):
        spec = workloads.LayerSpec("tall", 2, 3, h, w, k, s, k // 2, q)
        d = _rand_layer(rng, 2, 3, h, w, k)
        if dtype == torch.float16:
            hh, up = f16_inputs(d)
            want = oracle.to_f16_result(oracle_fused(oracle, up, spec, q)[0])
            inp = hh
        else:
            want = oracle_fused(oracle, d, spec, q)[0]
            inp = d
        for tune in ((0, 0, 0, 0), (1, 1, 64, 7), (2, 3, 128, 4), (1, 2, 256, 14), (1, 5, 96, 3), (3, 1, 32, 1)):
            ops.set_tuning(*tune)
            got, _ = run_fused(inp, spec, cuda_device, q, dtype=dtype)
            assert_same_bits(got, want, "tall %s tune %s" % ((h, w, k, s), tune))
        ops.set_tuning(0, 0, 0, 0)


def test_generic_geometries(oracle, cuda_device):
    """Everything the reference accepts and the tiled family does not: dilation,
    multiplier > 1, rectangular kernels / strides / pads, no padding, 1-D."""
    rng = np.random.default_rng(5)
    cases = [dict(k=(3, 3), s=(1, 1), p=(2, 2), d=(2, 2), mult=1), dict(k=(3, 3), s=(1, 1), p=(1, 1), d=(1, 1), mult=3),
             dict(k=(3, 5), s=(2, 1), p=(1, 2), d=(1, 1), mult=2), dict(k=(3, 3), s=(1, 1), p=(0, 0), d=(1, 1), mult=1),
             dict(k=(7, 7), s=(3, 3), p=(3, 3), d=(1, 1), mult=1), dict(k=(2, 2), s=(2, 2), p=(0, 1), d=(1, 1), mult=1)]
    for cs in cases:
        n, c, h, w = 2, 4, 11, 13
        oc = c * cs["mult"]
        x = rng.standard_normal((n, c, h, w)).astype(np.float32)
        wt = rng.standard_normal((oc,) + cs["k"]).astype(np.float32)
        b = rng.standard_normal(oc).astype(np.float32)
        want = oracle.dwconv(x, wt, b, cs["s"], cs["p"], cs["d"], cs["mult"])
        got = ops.depthwise_convolution(dev(x, cuda_device), dev(wt, cuda_device), dev(b, cuda_device), 1, cs["p"],
                                        cs["s"], cs["d"], cs["mult"]).cpu().numpy()
        assert_same_bits(got, want, str(cs))
        # fused with BN + Pow2 on the same geometry
        bn = {k_: (rng.random(oc) + 0.5).astype(np.float32) for k_ in ("beta", "gamma", "mean", "var")}
        q = {"kind": "pow2", "sign": True, "with_zero": True, "n": 8, "m": 1}
        want2 = oracle.pow2q(oracle.bn_infer(want, bn["beta"], bn["gamma"], bn["mean"], bn["var"], 1e-5), True, True, 8, 1)
        got2 = ops.fused_dw_bn_quant(dev(x, cuda_device), dev(wt, cuda_device), dev(b, cuda_device),
                                     dev(bn["beta"], cuda_device), dev(bn["gamma"], cuda_device),
                                     dev(bn["mean"], cuda_device), dev(bn["var"], cuda_device), 1e-5, cs["p"], cs["s"],
                                     cs["d"], cs["mult"], q).cpu().numpy()
        assert_same_bits(got2, want2, "fused " + str(cs))
    # 1-D: x [N, C, L], w [C, k]
    x = rng.standard_normal((3, 5, 33)).astype(np.float32)
    wt = rng.standard_normal((5, 3)).astype(np.float32)
    want = oracle.dwconv(x[:, :, None, :], wt[:, None, :], None, (1, 2), (0, 1), (1, 1), 1)[:, :, 0, :]
    got = ops.depthwise_convolution(dev(x, cuda_device), dev(wt, cuda_device), None, 1, (1,), (2,), (1,), 1).cpu().numpy()
    assert_same_bits(got, want, "1-D")


@pytest.mark.parametrize("path", [L.PATH_AUTO, L.PATH_COOP, L.PATH_RAW], ids=["auto", "coop", "raw"])
def test_parameters_where_zero_padding_is_not_a_skipped_tap(oracle, cuda_device, path):
    """bias == -0.0 and non-finite weights: the reference skips out-of-bounds taps, a
    zero-padded tile would add w * 0; the tiled family must fall back to exact evaluation."""
    rng = np.random.default_rng(11)
    n, c, h, w = 2, 6, 14, 14
    spec = workloads.LayerSpec("patho", n, c, h, w, 3, 1, 1, None)
    d = _rand_layer(rng, n, c, h, w, 3)
    # channel 0: x = -0.0, w > 0, bias = -0.0: every in-bounds product is -0.0 and the sum
    # stays -0.0, while a padding zero would contribute +0.0 and flip the sign at the border
    d["x"][:, 0] = -0.0
    d["w"][0] = np.abs(d["w"][0]) + np.float32(0.1)
    d["b"][0] = -0.0
    d["w"][1, 0, 0] = np.inf  # inf * padding-zero would be NaN
    d["w"][2, 2, 2] = np.nan
    d["w"][3, 1, 1] = -np.inf
    want = oracle.dwconv(d["x"], d["w"], d["b"], (1, 1), (1, 1))
    ops.set_forced_path(path)
    got = ops.depthwise_convolution(dev(d["x"], cuda_device), dev(d["w"], cuda_device), dev(d["b"], cuda_device), 1,
                                    (1, 1), (1, 1)).cpu().numpy()
    assert_same_bits(got, want, "pathological parameters")
    assert (bits(got[:, 0]) == 0x80000000).all()
    q = {"kind": "fpq", "sign": True, "n": 8, "delta": 2.0 ** -4}
    want_q, _, _ = oracle_fused(oracle, d, spec, q)
    got_q, _ = run_fused(d, spec, cuda_device, q, path=path)
    assert_same_bits(got_q, want_q, "pathological parameters, fused")


def test_unaligned_pointers_and_optional_inputs(oracle, cuda_device):
    rng = np.random.default_rng(13)
    n, c, h, w = 3, 8, 28, 28
    spec = workloads.LayerSpec("unaligned", n, c, h, w, 3, 1, 1, None)
    d = _rand_layer(rng, n, c, h, w, 3)
    q = {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3}
    want, _, _ = oracle_fused(oracle, d, spec, q)
    # x and y start 4 bytes past a 16-byte boundary
    xbuf = torch.empty(d["x"].size + 1, device=cuda_device)
    xbuf[1:] = dev(d["x"].ravel(), cuda_device)
    x = xbuf[1:].view(n, c, h, w)
    ybuf = torch.empty(want.size + 1, device=cuda_device)
    y = ybuf[1:].view(want.shape)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    ops.fused_dw_bn_quant(x, t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, (1, 1), (1, 1),
                          quant=q, out=y)
    assert_same_bits(y.cpu().numpy(), want, "unaligned x / y")
    # no bias, no gamma, no beta
    want = oracle.fpq(oracle.bn_infer(oracle.dwconv(d["x"], d["w"], None, (1, 1), (1, 1)), None, None, d["mean"],
                                      d["var"], 1e-5), False, 8, 2.0 ** -3)
    got = ops.fused_dw_bn_quant(t["x"], t["w"], None, None, None, t["mean"], t["var"], 1e-5, (1, 1), (1, 1), quant=q)
    assert_same_bits(got.cpu().numpy(), want, "optional inputs absent")
    # empty batch
    e = ops.fused_dw_bn_quant(t["x"][:0], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, (1, 1),
                              (1, 1), quant=q)
    assert e.shape == (0, c, h, w)


# ---- the small-plane kernel (7x7 and 14x14 planes, 3x3 stride 1) -------------------------

SMALL_QUANTS = [None,
                {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3},   # lean instantiation
                {"kind": "fpq", "sign": True, "n": 8, "delta": 2.0 ** -4},    # signed, fast form
                {"kind": "fpq", "sign": True, "n": 6, "delta": 0.3},          # delta not a power of two
                {"kind": "pow2", "sign": True, "with_zero": True, "n": 6, "m": 1},
                {"kind": "minmax", "x_min_max": True, "ema": False, "decay": 0.999, "eps": 0.01}]
SMALL_QUANT_IDS = ["none", "fpq_lean", "fpq_signed", "fpq_0.3", "pow2", "minmax"]


SMALL_SHAPES = [(7, 1), (14, 1), (28, 1), (56, 1), (112, 1), (14, 2), (28, 2), (56, 2), (112, 2)]
SMALL_SHAPE_IDS = ["7x7s1", "14x14s1", "28x28s1", "56x56s1", "112x112s1", "14x14s2", "28x28s2", "56x56s2", "112x112s2"]


@pytest.mark.parametrize("quant", SMALL_QUANTS, ids=SMALL_QUANT_IDS)
@pytest.mark.parametrize("hw,stride", SMALL_SHAPES, ids=SMALL_SHAPE_IDS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
def test_small_plane_kernel(oracle, cuda_device, dtype, hw, stride, quant):
    """Full tiles, a ragged last tile (37 planes: the 7x7 fp32 remainder is not a multiple of
    16 bytes, so its tile is copied by the threads) and a batch smaller than one tile."""
    rng = np.random.default_rng(100 + hw + stride)
    for n, c in (((5, 64) if hw <= 28 else (2, 24)), (1, 37), (1, 3)):
        spec = workloads.LayerSpec("small", n, c, hw, hw, 3, stride, 1, None)
        d = _rand_layer(rng, n, c, hw, hw, 3)
        if quant and quant["kind"] == "minmax":
            d.update(qr_min=np.zeros(c, np.float32), qr_max=np.ones(c, np.float32), ql_min=np.zeros(c, np.float32),
                     ql_max=np.full(c, 255, np.float32))
        h16, up = f16_inputs(d) if dtype == torch.float16 else (d, d)
        plan = ops.fused_plan(dev(h16["x"], cuda_device), dev(h16["w"], cuda_device), pad=(1, 1),
                              stride=(stride, stride))
        assert plan["path"] == L.PATH_PLANE, plan
        want, _, extra = oracle_fused(oracle, up, spec, quant)
        got, t = run_fused(h16, spec, cuda_device, quant, dtype=dtype)
        if dtype == torch.float16:
            want = oracle.to_f16_result(want)
        assert_same_bits(got, want, "%dx%d s%d n=%d c=%d" % (hw, hw, stride, n, c))
        if extra is not None and dtype == torch.float32:
            assert_same_bits(t["qr_min"].cpu().numpy(), extra[0], "qr_min")
            assert_same_bits(t["qr_max"].cpu().numpy(), extra[1], "qr_max")


@pytest.mark.parametrize("quant", [SMALL_QUANTS[1], SMALL_QUANTS[4], SMALL_QUANTS[5]], ids=["fpq_lean", "pow2", "minmax"])
@pytest.mark.parametrize("hw", [14, 28, 56, 112])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
def test_plane_kernel_5x5(oracle, cuda_device, dtype, hw, quant):
    """5x5 stride 1 pad 2 on the plane family: two halo rows / columns, four live accumulator
    rows, weight pairs in shared memory; includes a plane with bias == -0.0 (exact path)."""
    rng = np.random.default_rng(500 + hw)
    for n, c in (((3, 40) if hw <= 28 else (2, 10)), (1, 5)):
        spec = workloads.LayerSpec("p5", n, c, hw, hw, 5, 1, 2, None)
        d = _rand_layer(rng, n, c, hw, hw, 5)
        d["b"][1] = -0.0
        if quant["kind"] == "minmax":
            d.update(qr_min=np.zeros(c, np.float32), qr_max=np.ones(c, np.float32), ql_min=np.zeros(c, np.float32),
                     ql_max=np.full(c, 255, np.float32))
        h16, up = f16_inputs(d) if dtype == torch.float16 else (d, d)
        plan = ops.fused_plan(dev(h16["x"], cuda_device), dev(h16["w"], cuda_device), pad=(2, 2), stride=(1, 1))
        assert plan["path"] == L.PATH_PLANE, plan
        want, _, _ = oracle_fused(oracle, up, spec, quant)
        got, _ = run_fused(h16, spec, cuda_device, quant, dtype=dtype)
        if dtype == torch.float16:
            want = oracle.to_f16_result(want)
        assert_same_bits(got, want, "5x5 %dx%d n=%d c=%d" % (hw, hw, n, c))


@pytest.mark.parametrize("hw,stride", SMALL_SHAPES, ids=SMALL_SHAPE_IDS)
def test_small_plane_kernel_unaligned_and_optional(oracle, cuda_device, hw, stride):
    rng = np.random.default_rng(200 + hw + stride)
    n, c = 3, 40
    st = (stride, stride)
    spec = workloads.LayerSpec("small_unaligned", n, c, hw, hw, 3, stride, 1, None)
    d = _rand_layer(rng, n, c, hw, hw, 3)
    q = {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3}
    want, _, _ = oracle_fused(oracle, d, spec, q)
    xbuf = torch.empty(d["x"].size + 1, device=cuda_device)
    xbuf[1:] = dev(d["x"].ravel(), cuda_device)
    x = xbuf[1:].view(n, c, hw, hw)
    ybuf = torch.empty(want.size + 1, device=cuda_device)
    y = ybuf[1:].view(want.shape)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    ops.fused_dw_bn_quant(x, t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, (1, 1), st,
                          quant=q, out=y)
    assert_same_bits(y.cpu().numpy(), want, "unaligned x / y")
    want = oracle.fpq(oracle.dwconv(d["x"], d["w"], None, st, (1, 1)), False, 8, 2.0 ** -3)
    got = ops.fused_dw_bn_quant(t["x"], t["w"], None, None, None, None, None, 1e-5, (1, 1), st, quant=q)
    assert_same_bits(got.cpu().numpy(), want, "no bias, no BN")
    # the other families on the same planes give the same bits
    for path in (L.PATH_RAW, L.PATH_COOP, L.PATH_GENERIC):
        got_p, _ = run_fused(d, spec, cuda_device, q, path=path)
        want_p, _, _ = oracle_fused(oracle, d, spec, q)
        assert_same_bits(got_p, want_p, "path %d" % path)


@pytest.mark.parametrize("hw,stride", SMALL_SHAPES, ids=SMALL_SHAPE_IDS)
def test_small_plane_kernel_exact_evaluation_planes(oracle, cuda_device, hw, stride):
    rng = np.random.default_rng(300 + hw + stride)
    n, c = 2, 20
    st = (stride, stride)
    spec = workloads.LayerSpec("small_patho", n, c, hw, hw, 3, stride, 1, None)
    d = _rand_layer(rng, n, c, hw, hw, 3)
    d["x"][:, 0] = -0.0
    d["w"][0] = np.abs(d["w"][0]) + np.float32(0.1)
    d["b"][0] = -0.0
    d["w"][1, 0, 0] = np.inf
    d["w"][2, 2, 2] = np.nan
    d["w"][3, 1, 1] = -np.inf
    d["b"][7] = -0.0
    want = oracle.dwconv(d["x"], d["w"], d["b"], st, (1, 1))
    got = ops.depthwise_convolution(dev(d["x"], cuda_device), dev(d["w"], cuda_device), dev(d["b"], cuda_device), 1,
                                    (1, 1), st).cpu().numpy()
    assert_same_bits(got, want, "pathological parameters")
    assert (bits(got[:, 0]) == 0x80000000).all()
    for q in SMALL_QUANTS[1:5]:
        want_q, _, _ = oracle_fused(oracle, d, spec, q)
        got_q, _ = run_fused(d, spec, cuda_device, q)
        assert_same_bits(got_q, want_q, "pathological parameters, %s" % q["kind"])


GEN_SHAPES = [(6, 6), (8, 8), (10, 10), (12, 12), (16, 16), (20, 20), (24, 24), (30, 30), (40, 40), (48, 48), (64, 64),
              (96, 96), (20, 34), (15, 16), (100, 14), (9, 448), (1, 2), (57, 130)]


@pytest.mark.parametrize("quant", [SMALL_QUANTS[1], SMALL_QUANTS[3], SMALL_QUANTS[4], SMALL_QUANTS[5]],
                         ids=["fpq_lean", "fpq_0.3", "pow2", "minmax"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
def test_general_geometry_plane_kernel(oracle, cuda_device, dtype, quant):
    """3x3 stride 1 on planes of any even width: partly filled last column / row blocks, idle
    lanes, bands with halo rows, tiles the copy engine cannot take (sizes that are not
    multiples of 16 bytes), a plane with bias == -0.0, ragged plane counts."""
    rng = np.random.default_rng(900)
    for h, w in GEN_SHAPES:
        for n, c in ((2, 9), (1, 1)):
            spec = workloads.LayerSpec("gen", n, c, h, w, 3, 1, 1, None)
            d = _rand_layer(rng, n, c, h, w, 3)
            if c > 4:
                d["b"][4] = -0.0
            if quant["kind"] == "minmax":
                d.update(qr_min=np.zeros(c, np.float32), qr_max=np.ones(c, np.float32), ql_min=np.zeros(c, np.float32),
                         ql_max=np.full(c, 255, np.float32))
            h16, up = f16_inputs(d) if dtype == torch.float16 else (d, d)
            want, _, extra = oracle_fused(oracle, up, spec, quant)
            got, t = run_fused(h16, spec, cuda_device, quant, dtype=dtype, path=L.PATH_PLANE_GEN)
            plan = ops.fused_plan(dev(h16["x"], cuda_device), dev(h16["w"], cuda_device), pad=(1, 1), stride=(1, 1))
            assert plan["path"] == L.PATH_PLANE_GEN, (h, w, plan)
            if dtype == torch.float16:
                want = oracle.to_f16_result(want)
            assert_same_bits(got, want, "%dx%d n=%d c=%d" % (h, w, n, c))
            if extra is not None and dtype == torch.float32:
                assert_same_bits(t["qr_min"].cpu().numpy(), extra[0], "qr_min")
                assert_same_bits(t["qr_max"].cpu().numpy(), extra[1], "qr_max")
    # unaligned x / y
    h, w, n, c = 24, 24, 2, 5
    spec = workloads.LayerSpec("gen_unaligned", n, c, h, w, 3, 1, 1, None)
    d = _rand_layer(rng, n, c, h, w, 3)
    q = SMALL_QUANTS[1]
    want, _, _ = oracle_fused(oracle, d, spec, q)
    xbuf = torch.empty(d["x"].size + 1, device=cuda_device)
    xbuf[1:] = dev(d["x"].ravel(), cuda_device)
    ybuf = torch.empty(want.size + 1, device=cuda_device)
    y = ybuf[1:].view(want.shape)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    ops.set_forced_path(L.PATH_PLANE_GEN)
    ops.fused_dw_bn_quant(xbuf[1:].view(n, c, h, w), t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5,
                          (1, 1), (1, 1), quant=q, out=y)
    if dtype == torch.float32:
        assert_same_bits(y.cpu().numpy(), want, "unaligned x / y")


def test_random_geometries_against_the_oracle(oracle, cuda_device):
    """A seeded sweep over shapes, kernel sizes, strides, paddings, dilations, multipliers,
    dtypes and quantizers: whichever kernel family the planner picks must reproduce the
    oracle bit for bit."""
    rng = np.random.default_rng(2024)
    quants = [None, {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3},
              {"kind": "fpq", "sign": True, "n": 5, "delta": 0.17},
              {"kind": "pow2", "sign": True, "with_zero": True, "n": 6, "m": 1},
              {"kind": "pow2", "sign": False, "with_zero": False, "n": 4, "m": 0}]
    sizes = [3, 5, 6, 7, 8, 12, 13, 14, 15, 16, 20, 24, 27, 28, 30, 40, 48, 56, 57, 64, 96, 112]
    paths_seen = set()
    for case in range(120):
        k = int(rng.choice([1, 2, 3, 3, 3, 5, 5, 7]))
        h, w = int(rng.choice(sizes)), int(rng.choice(sizes))
        if rng.random() < 0.6:
            w = h
        stride = int(rng.choice([1, 1, 2, 3]))
        dil = int(rng.choice([1, 1, 1, 2]))
        pad = int(rng.choice([0, k // 2, k // 2, k // 2, k - 1]))
        mult = int(rng.choice([1, 1, 1, 2]))
        if h + 2 * pad < dil * (k - 1) + 1 or w + 2 * pad < dil * (k - 1) + 1:
            continue
        c = int(rng.choice([1, 3, 8, 17, 32]))
        n = int(rng.choice([1, 2, 5]))
        half = rng.random() < 0.3
        quant = quants[int(rng.integers(len(quants)))]
        has_bn = rng.random() < 0.8
        oc = c * mult
        d = {"x": rng.standard_normal((n, c, h, w)).astype(np.float32),
             "w": (rng.standard_normal((oc, k, k)) / k).astype(np.float32),
             "b": rng.standard_normal(oc).astype(np.float32),
             "mean": rng.standard_normal(oc).astype(np.float32) * 0.3, "var": (rng.random(oc) + 0.5).astype(np.float32),
             "gamma": (rng.random(oc) * 0.4 + 0.8).astype(np.float32), "beta": rng.standard_normal(oc).astype(np.float32) * 0.3}
        h16, up = f16_inputs(d) if half else (d, d)
        y = oracle.dwconv(up["x"], up["w"], up["b"], (stride, stride), (pad, pad), (dil, dil), mult)
        if has_bn:
            y = oracle.bn_infer(y, up["beta"], up["gamma"], up["mean"], up["var"], 1e-5)
        if quant and quant["kind"] == "fpq":
            y = oracle.fpq(y, quant["sign"], quant["n"], quant["delta"])
        elif quant:
            y = oracle.pow2q(y, quant["sign"], quant["with_zero"], quant["n"], quant["m"])
        want = oracle.to_f16_result(y) if half else y
        dt = torch.float16 if half else torch.float32
        t = {k_: dev(v, cuda_device).to(dt) for k_, v in h16.items()}
        paths_seen.add(ops.fused_plan(t["x"], t["w"], pad=(pad, pad), stride=(stride, stride), dilation=(dil, dil),
                                      multiplier=mult)["path"])
        got = ops.fused_dw_bn_quant(t["x"], t["w"], t["b"], t["beta"] if has_bn else None, t["gamma"] if has_bn else None,
                                    t["mean"] if has_bn else None, t["var"] if has_bn else None, 1e-5, pad=(pad, pad),
                                    stride=(stride, stride), dilation=(dil, dil), multiplier=mult, quant=quant)
        torch.cuda.synchronize()
        ops.check_device_flag()
        assert_same_bits(got.cpu().numpy(), want, "case %d: n=%d c=%d %dx%d k=%d s=%d p=%d d=%d m=%d half=%s bn=%s q=%s"
                         % (case, n, c, h, w, k, stride, pad, dil, mult, half, has_bn, quant and quant["kind"]))
    assert {L.PATH_GENERIC, L.PATH_PLANE, L.PATH_PLANE_GEN}.issubset(paths_seen), paths_seen


def test_concurrent_host_threads_on_their_own_streams(oracle, cuda_device):
    """The entry points are re-entrant: four host threads, each on its own stream, run
    different layers at the same time (the reference allows concurrent function calls on one
    device: test/test_multi_thread_training.cpp); every result must match the oracle."""
    import threading
    rng = np.random.default_rng(77)
    jobs = []
    for hw, k, stride, quant in ((14, 3, 1, SMALL_QUANTS[1]), (28, 3, 2, SMALL_QUANTS[4]), (24, 3, 1, SMALL_QUANTS[2]),
                                 (15, 5, 1, SMALL_QUANTS[1])):
        n, c = 4, 24
        spec = workloads.LayerSpec("mt", n, c, hw, hw, k, stride, k // 2, None)
        d = _rand_layer(rng, n, c, hw, hw, k)
        want, _, _ = oracle_fused(oracle, d, spec, quant)
        jobs.append((spec, {k_: dev(v, cuda_device) for k_, v in d.items()}, quant, want))
    results, errors = [None] * len(jobs), []

    def work(i):
        try:
            spec, t, quant, _ = jobs[i]
            stream = torch.cuda.Stream(cuda_device)
            with torch.cuda.stream(stream):
                y = None
                for _ in range(20):
                    y = ops.fused_dw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], spec.bn_eps,
                                              pad=(spec.pad, spec.pad), stride=(spec.stride, spec.stride), quant=quant)
                stream.synchronize()
                results[i] = y.cpu().numpy()
        except Exception as e:  # surfaced in the main thread
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(jobs))]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    ops.check_device_flag()
    for i, (_, _, _, want) in enumerate(jobs):
        assert_same_bits(results[i], want, "thread %d" % i)


def test_in_place_tiles_give_the_same_bits_every_time(oracle, cuda_device):
    """The plane kernels overwrite their tile in place; the rows and columns one thread reads
    and another writes are ordered by warp barriers. A missing ordering would show up as a
    timing-dependent result: every shape is run 60 times, with a second stream keeping the
    GPU busy to perturb the timing, and every run must reproduce the oracle's bits."""
    rng = np.random.default_rng(4242)
    noise = torch.empty(64 << 20, dtype=torch.float32, device=cuda_device)
    side = torch.cuda.Stream(cuda_device)
    cases = [(14, 3, 1), (28, 3, 1), (56, 3, 1), (112, 3, 1), (28, 5, 1), (56, 5, 1), (28, 3, 2), (112, 3, 2), (24, 3, 1),
             (40, 3, 1), (30, 3, 1)]
    for hw, k, stride in cases:
        n, c = 4, 24
        spec = workloads.LayerSpec("rep", n, c, hw, hw, k, stride, k // 2, None)
        d = _rand_layer(rng, n, c, hw, hw, k)
        q = SMALL_QUANTS[1]
        want, _, _ = oracle_fused(oracle, d, spec, q)
        t = {k_: dev(v, cuda_device) for k_, v in d.items()}
        ops.set_forced_path(L.PATH_PLANE_GEN if hw in (24, 40, 30) else L.PATH_AUTO)
        wb = torch.from_numpy(want).to(cuda_device)
        bad = 0
        for i in range(60):
            if i % 3 == 0:
                with torch.cuda.stream(side):
                    noise.mul_(1.0001)
            y = ops.fused_dw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5,
                                      pad=(k // 2,) * 2, stride=(stride,) * 2, quant=q)
            bad += int((y.view(torch.int32) != wb.view(torch.int32)).sum().item())
        torch.cuda.synchronize()
        ops.check_device_flag()
        assert bad == 0, (hw, k, stride, bad)


# ---- the five standalone operators -----------------------------------------------------

def test_standalone_batch_normalization(oracle, cuda_device):
    rng = np.random.default_rng(21)
    for shape, axis in (((4, 6, 14, 14), 1), ((3, 5, 7, 7), 1), ((2, 9, 1, 1), 1), ((64, 10), 1), ((2, 5, 6, 8), 3),
                        ((3, 7, 13), 1), ((2, 3, 5, 3), 2), ((1, 960, 7, 7), 1)):
        c = shape[axis]
        x = rng.standard_normal(shape).astype(np.float32)
        p = {k: (rng.random(c) + 0.5).astype(np.float32) for k in ("beta", "gamma", "mean", "var")}
        for no_scale, no_bias in ((False, False), (True, False), (False, True), (True, True)):
            g = None if no_scale else p["gamma"]
            b = None if no_bias else p["beta"]
            want = oracle.bn_infer(x, b, g, p["mean"], p["var"], 1e-5, axis)
            got = ops.batch_normalization(dev(x, cuda_device), dev(b, cuda_device), dev(g, cuda_device),
                                          dev(p["mean"], cuda_device), dev(p["var"], cuda_device), [axis], 0.9, 1e-5,
                                          False).cpu().numpy()
            assert_same_bits(got, want, "BN %s axis %d" % (shape, axis))
        xh = x.astype(np.float16)
        ph = {k: v.astype(np.float16) for k, v in p.items()}
        want = oracle.to_f16_result(oracle.bn_infer(xh.astype(np.float32), *(ph[k].astype(np.float32) for k in
                                                                            ("beta", "gamma", "mean", "var")), 1e-5, axis))
        got = ops.batch_normalization(dev(xh, cuda_device), *(dev(ph[k], cuda_device) for k in
                                                              ("beta", "gamma", "mean", "var")), [axis], 0.9, 1e-5,
                                      False).cpu().numpy()
        assert_same_bits(got, want, "BN fp16 %s" % (shape,))
    with pytest.raises(NotImplementedError):
        ops.batch_normalization(dev(x, cuda_device), None, None, None, None, batch_stat=True)


def _bit_sweep():
    """float32 bit patterns: a stride-61 walk over all 2^32 patterns, dense around the
    quantizer decision points, and the special values."""
    walk = np.arange(0, 1 << 32, 61, dtype=np.uint64).astype(np.uint32)
    around = []
    for centre in (0x3fb504f3, 0x3f3504f3, 0x40000000, 0x3d800000, 0x3d000000, 0x41ff0000, 0x40fe0000, 0x20800000,
                   0x203504f3, 0x00800000, 0x00000001, 0x7f7fffff, 0x7f800000):
        lo = max(0, centre - 2000)
        around.append(np.arange(lo, centre + 2000, dtype=np.uint32))
        around.append(np.arange(lo, centre + 2000, dtype=np.uint32) | np.uint32(0x80000000))
    return np.concatenate([walk] + around)


def test_standalone_fixed_point_quantize_bit_sweep(oracle, cuda_device):
    b = _bit_sweep()
    x = b.view(np.float32)
    xd = dev(x, cuda_device)
    for sign, n, delta in ((True, 8, 2.0 ** -4), (False, 8, 2.0 ** -3), (True, 4, 0.1), (False, 16, 0.37), (True, 24, 1.0),
                           (True, 31, 2.0 ** -10)):
        want = oracle.fpq(x, sign, n, delta, oracle.max_threads())
        got = ops.fixed_point_quantize(xd, sign, n, delta).cpu().numpy()
        assert_same_bits(got, want, "FPQ sign=%s n=%d delta=%g" % (sign, n, delta))
    # idempotent: quantized values are fixed points of the quantizer
    y = ops.fixed_point_quantize(xd, True, 8, 2.0 ** -4)
    yy = ops.fixed_point_quantize(y, True, 8, 2.0 ** -4)
    finite = ~torch.isnan(y)
    assert torch.equal(y[finite], yy[finite])
    # in place, odd length, fp16
    z = xd[:1000003].clone()
    ops.fixed_point_quantize(z, True, 8, 2.0 ** -4, out=z)
    assert_same_bits(z.cpu().numpy(), oracle.fpq(x[:1000003], True, 8, 2.0 ** -4), "FPQ in place")
    xh = np.arange(0, 1 << 16, dtype=np.uint16).view(np.float16)
    want = oracle.to_f16_result(oracle.fpq(xh.astype(np.float32), True, 8, 2.0 ** -4))
    got = ops.fixed_point_quantize(dev(xh, cuda_device), True, 8, 2.0 ** -4).cpu().numpy()
    assert_same_bits(got, want, "FPQ fp16, all 65536 patterns")


def test_standalone_pow2_quantize_bit_sweep(oracle, cuda_device):
    b = _bit_sweep()
    x = b.view(np.float32)
    xd = dev(x, cuda_device)
    for sign, wz, n, m in ((True, True, 8, 1), (False, True, 8, 0), (True, False, 6, 3), (False, False, 4, -2),
                           (False, False, 8, 0), (True, True, 3, 120)):
        want = oracle.pow2q(x, sign, wz, n, m, oracle.max_threads())
        got = ops.pow2_quantize(xd, sign, wz, n, m).cpu().numpy()
        assert_same_bits(got, want, "Pow2 sign=%s with_zero=%s n=%d m=%d" % (sign, wz, n, m))
    xh = np.arange(0, 1 << 16, dtype=np.uint16).view(np.float16)
    want = oracle.to_f16_result(oracle.pow2q(xh.astype(np.float32), True, True, 8, 1))
    got = ops.pow2_quantize(dev(xh, cuda_device), True, True, 8, 1).cpu().numpy()
    assert_same_bits(got, want, "Pow2 fp16, all 65536 patterns")


def test_standalone_min_max_quantize(oracle, cuda_device):
    rng = np.random.default_rng(31)
    for shape in ((8, 12, 14, 14), (5, 7, 7, 7), (3, 4, 1, 3), (16, 33), (2, 3, 50, 50)):
        c = shape[1]
        x = (rng.standard_normal(shape) * 3).astype(np.float32)
        x[0, 0] = 1.25  # leaves channel 0 non-constant; channel below is constant
        if shape[0] > 1 and c > 1:
            x[:, 1] = -0.75
        ql_min = np.zeros(c, np.float32)
        ql_max = np.full(c, 255.0, np.float32)
        for x_min_max, ema in ((True, False), (True, True), (False, False)):
            qr_min = (rng.standard_normal(c) - 3).astype(np.float32)
            qr_max = (rng.standard_normal(c) + 3).astype(np.float32)
            want, wmin, wmax = oracle.minmaxq(x, qr_min, qr_max, ql_min, ql_max, 0.9, x_min_max, ema, 0.01)
            tmin, tmax = dev(qr_min, cuda_device), dev(qr_max, cuda_device)
            got = ops.min_max_quantize(dev(x, cuda_device), tmin, tmax, dev(ql_min, cuda_device),
                                       dev(ql_max, cuda_device), 0.9, x_min_max, ema, True, 0.01).cpu().numpy()
            assert_same_bits(got, want, "MinMax %s x_min_max=%s ema=%s" % (shape, x_min_max, ema))
            np.testing.assert_array_equal(tmin.cpu().numpy(), wmin)
            np.testing.assert_array_equal(tmax.cpu().numpy(), wmax)


def test_standalone_chain_equals_fused(cuda_device):
    """The unfused three-call chain and the fused kernel produce identical bits."""
    spec = workloads.cfg0(n=4)[0]
    d = workloads.make_layer_data(spec)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    y = ops.depthwise_convolution(t["x"], t["w"], t["b"], 1, (1, 1), (1, 1))
    y = ops.batch_normalization(y, t["beta"], t["gamma"], t["mean"], t["var"], [1], 0.9, 1e-5, False)
    y = ops.fixed_point_quantize(y, True, 8, 2.0 ** -4)
    f = ops.fused_dw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, (1, 1), (1, 1),
                              quant=workloads.quant_for_ops(spec))
    assert torch.equal(y.view(torch.int32), f.view(torch.int32))


# ---- many tiles, every quantizer, planes that need the tap-by-tap path ------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("hw,n,c", [(14, 128, 320), (28, 32, 320), (56, 8, 400)])
def test_plane_kernels_more_tiles_than_resident_ctas(oracle, cuda_device, dtype, hw, n, c):
    """3x3 stride 1 on 14 / 28 / 56 wide planes with more tiles than the device holds CTAs
    (several waves, the last one partial): every quantizer, one plane with a -0.0 bias and one
    with an infinite weight (tap-by-tap re-evaluation)."""
    for kind in ("fpq", "pow2", "minmax", None):
        quant = {"fpq": dict(workloads.FPQ_CFG1), "pow2": dict(workloads.POW2_CFG2),
                 "minmax": dict(workloads.MINMAX_CFG3), None: None}[kind]
        spec = workloads.LayerSpec("waves", n, c, hw, hw, 3, 1, 1, quant or dict(workloads.FPQ_CFG1), seed=hw,
                                   x_dist="normal2_outliers" if kind == "minmax" else "relu6")
        d = workloads.make_layer_data(spec)
        d["b"][5] = -0.0
        d["w"][7, 1, 1] = np.inf
        h16, up = f16_inputs(d) if dtype == torch.float16 else (d, d)
        q = workloads.quant_for_ops(spec, up) if kind else None
        want, _, extra = oracle_fused(oracle, up, spec, q)
        got, t = run_fused(h16, spec, cuda_device, q, dtype=dtype)
        if dtype == torch.float16:
            want = oracle.to_f16_result(want)
        assert_same_bits(got, want, "%dx%d %s %s" % (hw, hw, kind, dtype))
        if kind == "minmax" and dtype == torch.float32:
            np.testing.assert_array_equal(t["qr_min"].cpu().numpy(), extra[0])
            np.testing.assert_array_equal(t["qr_max"].cpu().numpy(), extra[1])


# ---- full benchmark sizes: sampled parity and size-independent properties ------------------

def test_full_size_largest_layer_sampled_images(oracle, cuda_device):
    """cfg1's largest layer (96 ch, 112x112, stride 2) at batch 256: the oracle checks a few
    whole images; the rest is checked through properties of the quantizer's range."""
    spec = workloads.cfg1()[1]
    assert (spec.c, spec.h, spec.stride, spec.n) == (96, 112, 2, 256)
    small = workloads.LayerSpec(spec.name, 8, spec.c, spec.h, spec.w, 3, 2, 1, spec.quant, seed=spec.seed,
                                x_dist=spec.x_dist)
    d = workloads.make_layer_data(small)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    x = t["x"].repeat(32, 1, 1, 1)  # 256 images: 32 copies of the 8 seeded ones
    q = workloads.quant_for_ops(spec)
    y = ops.fused_dw_bn_quant(x, t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, (1, 1), (2, 2),
                              quant=q)
    want, _, _ = oracle_fused(oracle, d, small, q)
    for rep in (0, 13, 31):
        assert_same_bits(y[rep * 8:(rep + 1) * 8].cpu().numpy(), want, "images %d.." % (rep * 8))
    # every copy equals the first one, values are on the grid and inside [0, 31.875]
    assert torch.equal(y.view(32, -1), y[:8].reshape(1, -1).expand(32, -1))
    assert float(y.min()) >= 0.0 and float(y.max()) <= 31.875
    assert torch.equal(y * 8, torch.round(y * 8))
    ops.check_device_flag()


def test_full_size_cfg2_batch128(oracle, cuda_device):
    """cfg2 at its full batch of 128 (5x5 + BN + Pow2Quantize on [128,144,56,56]): the GPU runs
    the whole seeded batch, the oracle checks whole images from its start, middle and end; all
    outputs are checked through the quantizer's value set (0 or +-2^k, 2^-62 <= |y| <= 2)."""
    spec = workloads.cfg2()[0]
    assert (spec.n, spec.c, spec.h, spec.k) == (128, 144, 56, 5)
    d = workloads.make_layer_data(spec)
    q = workloads.quant_for_ops(spec)
    got, _ = run_fused(d, spec, cuda_device, q)
    for first in (0, 62, 126):
        sub = dict(d, x=d["x"][first:first + 2])
        want, _, _ = oracle_fused(oracle, sub, spec, q)
        assert_same_bits(got[first:first + 2], want, "cfg2 images %d, %d of 128" % (first, first + 1))
    a = np.abs(got)
    nz = a[a != 0]
    mant, expo = np.frexp(nz)
    assert np.all(mant == 0.5) and expo.min() - 1 >= -62 and expo.max() - 1 <= 1


def test_full_size_cfg3_batch512_every_image(oracle, cuda_device):
    """cfg3 at its full batch of 512 (3x3 stride 2 + BN + per-channel MinMaxQuantize whose
    min / max run over the whole batch): the oracle computes all 512 images on all host cores
    and every output and both range vectors are compared."""
    spec = workloads.cfg3()[0]
    assert (spec.n, spec.c, spec.h, spec.stride) == (512, 192, 28, 2)
    d = workloads.make_layer_data(spec)
    q = workloads.quant_for_ops(spec, d)
    want, _, (qmin, qmax) = oracle_fused(oracle, d, spec, q)
    got, t = run_fused(d, spec, cuda_device, q)
    assert_same_bits(got, want, "cfg3, all 512 images")
    np.testing.assert_array_equal(t["qr_min"].cpu().numpy(), qmin)
    np.testing.assert_array_equal(t["qr_max"].cpu().numpy(), qmax)
    # at most 256 levels per channel
    assert max(len(np.unique(got[:, c])) for c in (0, 95, 191)) <= 256


@pytest.mark.parametrize("layer", [4, 14], ids=["28x28x192_s1", "7x7x960_s1"])
def test_full_size_cfg4_fp16_batch256(oracle, cuda_device, layer):
    """Two cfg4 layers (fp16 storage, fp32 arithmetic) at the bench batch of 256, every output
    against the oracle's fp16 convention: a stride-1 28x28 layer and a 7x7 layer."""
    spec = workloads.cfg1()[layer]
    assert spec.n == 256 and spec.stride == 1
    d = workloads.make_layer_data(spec)
    h, up = f16_inputs(d)
    q = workloads.quant_for_ops(spec)
    want32, _, _ = oracle_fused(oracle, up, spec, q)
    got, _ = run_fused(h, spec, cuda_device, q, dtype=torch.float16)
    assert_same_bits(got, oracle.to_f16_result(want32), "cfg4 layer %d at batch 256" % layer)


def test_more_than_2_pow_31_elements(oracle, cuda_device):
    """Offsets beyond 2^31 elements (the reference indexes with int): a [1800, 96, 112, 112]
    input has 2.17e9 elements; the last images are checked against the oracle."""
    spec = workloads.LayerSpec("big", 1800, 96, 112, 112, 3, 2, 1, dict(workloads.FPQ_CFG1), seed=3, x_dist="relu6")
    small = workloads.LayerSpec("big", 2, 96, 112, 112, 3, 2, 1, spec.quant, seed=3, x_dist="relu6")
    d = workloads.make_layer_data(small)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    x = torch.zeros((spec.n, spec.c, spec.h, spec.w), device=cuda_device)
    assert x.numel() > 2 ** 31
    x[-2:] = t["x"]
    x[899:901] = t["x"]
    q = workloads.quant_for_ops(spec)
    y = ops.fused_dw_bn_quant(x, t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, (1, 1), (2, 2),
                              quant=q)
    want, _, _ = oracle_fused(oracle, d, small, q)
    assert_same_bits(y[-2:].cpu().numpy(), want, "images beyond 2^31 elements")
    assert_same_bits(y[899:901].cpu().numpy(), want, "images in the middle")
    # standalone element-wise ops on the same large tensor
    z = ops.fixed_point_quantize(x, False, 8, 2.0 ** -3)
    assert_same_bits(z[-2:].cpu().numpy(), oracle.fpq(d["x"], False, 8, 2.0 ** -3), "FPQ beyond 2^31 elements")
    del x, y, z
    torch.cuda.empty_cache()
    ops.check_device_flag()
