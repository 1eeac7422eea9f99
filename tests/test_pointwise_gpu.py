"""Pointwise (1x1) convolution with the fused BN / activation / quantizer epilogue, through the
C ABI, against the CPU oracle.

The order of a convolution's sum is the implementation's own (the reference leaves it to its
GEMM library), so the convolution is checked within a stated tolerance of the sum accumulated
in double, relative to sum |w||x|:
  * three-pass TF32 (math "fp32"): 4e-6 - 2^-21 per product from the truncated low halves
    plus the dropped lo*lo term, and the fp32 accumulation;
  * single-pass TF32: 2^-9 (both factors truncated to 11 significant bits);
  * the FMA kernel: (c_in + 4) * 2^-24, an fp32 accumulation in any order.
Everything after the sum is exact arithmetic: the fused result must equal, bit for bit, the
oracle's BN -> activation -> quantizer applied to the convolution the same kernel returns
unfused. The fused result is also bracketed by the oracle epilogue of (double sum -/+
tolerance), which ties it to the inputs without relying on the kernel's own convolution."""
import numpy as np
import pytest
import torch

from dwbnq import _lib as L
from dwbnq import ops

pytestmark = pytest.mark.gpu

FPQ_U = {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3}
FPQ_S = {"kind": "fpq", "sign": True, "n": 8, "delta": 2.0 ** -4}
FPQ_ODD = {"kind": "fpq", "sign": False, "n": 6, "delta": 0.0371}
POW2 = {"kind": "pow2", "sign": True, "with_zero": True, "n": 8, "m": 1}


def dev(a, device):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(device)


def make(rng, n, ci, co, h, w, bias=True, dtype=np.float32):
    d = {
        "x": np.minimum(np.maximum(rng.standard_normal((n, ci, h, w), dtype=np.float32) * 2, -1), 6),
        "w": (rng.standard_normal((co, ci, 1, 1), dtype=np.float32) / np.sqrt(ci)).astype(np.float32),
        "b": (rng.standard_normal(co, dtype=np.float32) * 0.3) if bias else None,
        "mean": rng.standard_normal(co, dtype=np.float32) * 0.3,
        "var": (0.5 + rng.random(co, dtype=np.float32)),
        "gamma": (0.8 + 0.4 * rng.random(co, dtype=np.float32)) * np.where(rng.random(co) < 0.1, -1, 1).astype(np.float32),
        "beta": rng.standard_normal(co, dtype=np.float32) * 0.3,
    }
    return {k: (None if v is None else v.astype(dtype)) for k, v in d.items()}


def conv_tolerance(path, math, ci):
    if path == 0:
        return (ci + 4) * 2.0 ** -24
    return 4e-6 if math == "fp32" else 2.0 ** -9


def f32(a):
    return None if a is None else np.asarray(a, dtype=np.float32)


def check_conv(oracle, got, d, tol, half=False):
    _, acc64, mag = oracle.pwconv(f32(d["x"]), f32(d["w"]), f32(d["b"]), nthreads=oracle.max_threads())
    err = np.abs(got.astype(np.float64) - acc64.astype(np.float64))
    bound = tol * mag.astype(np.float64) + 1e-30
    if half:
        bound = bound + np.abs(acc64) * 2.0 ** -11 + 2.0 ** -25
    worst = float((err / bound).max())
    assert worst <= 1.0, "convolution off by %.3g times the tolerance" % worst
    return acc64, mag


def bracket(oracle, acc64, mag, tol, d, eps, act, quant):
    lo = oracle.pw_epilogue(acc64 - (tol * mag).astype(np.float32) - 1e-30, f32(d["beta"]), f32(d["gamma"]), f32(d["mean"]),
                            f32(d["var"]), eps, act, quant)
    hi = oracle.pw_epilogue(acc64 + (tol * mag).astype(np.float32) + 1e-30, f32(d["beta"]), f32(d["gamma"]), f32(d["mean"]),
                            f32(d["var"]), eps, act, quant)
    return np.minimum(lo, hi), np.maximum(lo, hi)


SHAPES = [
    # n, ci, co, h, w
    (2, 32, 64, 16, 16),     # one k chunk, one channel tile, full tiles
    (3, 24, 144, 12, 10),    # c_in not a multiple of 32, 144 channels -> 160 columns, ragged positions
    (1, 96, 24, 28, 28),     # 24 channels in a 32-column tile
    (2, 20, 40, 6, 6),       # c_in multiple of 4 only, one partial tile
    (1, 4, 8, 2, 2),         # smallest TMA-able shape
    (2, 192, 320, 14, 14),   # two channel tiles (256 + 64), six k chunks
    (1, 960, 160, 14, 14),   # more k chunks than pipeline stages
    (2, 64, 384, 14, 14),    # 384 = 256 + 128
    (5, 16, 96, 28, 28),     # several tiles per CTA in a small grid
    # planes TMA cannot take, or that would fill the 128-row tiles badly: rows gathered across images
    (2, 32, 64, 7, 7),
    (5, 160, 70, 7, 7),
    (3, 64, 96, 14, 14),
    (2, 8, 16, 5, 9),
    (1, 4, 8, 1, 1),
    (7, 96, 160, 3, 3),
]


@pytest.mark.parametrize("math", ["fp32", "tf32"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_tensor_core_kernel(oracle, cuda_device, shape, math):
    n, ci, co, h, w = shape
    rng = np.random.default_rng(sum(shape))
    d = make(rng, *shape)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    assert ops.pwconv_plan(t["x"], t["w"], math=math) == 1
    tol = conv_tolerance(1, math, ci)
    conv = ops.pointwise_convolution(t["x"], t["w"], t["b"], math=math)
    torch.cuda.synchronize()
    ops.check_device_flag()
    got_conv = conv.cpu().numpy()
    acc64, mag = check_conv(oracle, got_conv, d, tol)
    eps = 1e-5
    for quant, act, bn in ((FPQ_U, "relu6", True), (FPQ_U, None, True), (FPQ_S, None, True), (POW2, "relu", True),
                           (None, "relu6", True), (FPQ_U, None, False), (FPQ_ODD, "relu6", True)):
        m, v, g, be = (t["mean"], t["var"], t["gamma"], t["beta"]) if bn else (None,) * 4
        y = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], be, g, m, v, eps, quant, act, math=math)
        torch.cuda.synchronize()
        ops.check_device_flag()
        got = y.cpu().numpy()
        dd = d if bn else dict(d, mean=None, var=None, gamma=None, beta=None)
        want = oracle.pw_epilogue(got_conv, dd["beta"], dd["gamma"], dd["mean"], dd["var"], eps, act, quant)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (quant, act, bn)
        lo, hi = bracket(oracle, acc64, mag, tol, dd, eps, act, quant)
        assert np.all((got >= lo) & (got <= hi)), (quant, act, bn)


def test_no_bias_and_partial_bn_vectors(oracle, cuda_device):
    rng = np.random.default_rng(5)
    d = make(rng, 2, 32, 48, 8, 8, bias=False)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    conv = ops.pointwise_convolution(t["x"], t["w"], None).cpu().numpy()
    check_conv(oracle, conv, d, 4e-6)
    for beta, gamma in ((None, t["gamma"]), (t["beta"], None), (None, None)):
        y = ops.fused_pw_bn_quant(t["x"], t["w"], None, beta, gamma, t["mean"], t["var"], 1e-3, FPQ_U, "relu6")
        want = oracle.pw_epilogue(conv, None if beta is None else d["beta"], None if gamma is None else d["gamma"],
                                  d["mean"], d["var"], 1e-3, "relu6", FPQ_U)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))
    ops.check_device_flag()


FMA_SHAPES = [(3, 30, 50, 5, 9), (1, 3, 5, 1, 1), (2, 17, 130, 14, 14), (2, 6, 16, 8, 8)]  # c_in not a multiple of 4


@pytest.mark.parametrize("shape", FMA_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_fma_kernel_takes_every_other_shape(oracle, cuda_device, shape):
    n, ci, co, h, w = shape
    rng = np.random.default_rng(sum(shape))
    d = make(rng, *shape)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    assert ops.pwconv_plan(t["x"], t["w"]) == 0
    tol = conv_tolerance(0, "fp32", ci)
    got_conv = ops.pointwise_convolution(t["x"], t["w"], t["b"]).cpu().numpy()
    acc64, mag = check_conv(oracle, got_conv, d, tol)
    for quant, act in ((FPQ_U, "relu6"), (POW2, None), (None, "relu")):
        y = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, quant, act)
        want = oracle.pw_epilogue(got_conv, d["beta"], d["gamma"], d["mean"], d["var"], 1e-5, act, quant)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32)), (quant, act)
    ops.check_device_flag()


def test_fp16_tensors(oracle, cuda_device):
    """binary16 tensors: on the tensor-core kernel (gathered rows and ONE TF32 pass - a binary16 factor
    has 11 significant bits, so every product is exact and only the fp32 accumulation rounds - or, with
    16-byte rows, TMA loads and binary16 MMAs) when c_in is a multiple of 4, else on the FMA kernel;
    fp32 epilogue, one rounding to binary16 at the store."""
    rng = np.random.default_rng(11)
    for shape, path in (((2, 32, 64, 14, 14), 1), ((1, 24, 40, 7, 7), 1), ((3, 64, 200, 28, 28), 1), ((2, 30, 24, 6, 6), 0)):
        d = make(rng, *shape, dtype=np.float16)
        t = {k: dev(v, cuda_device) for k, v in d.items()}
        assert ops.pwconv_plan(t["x"], t["w"]) == path
        tol = (shape[1] + 4) * (2.0 ** -23 if path else 2.0 ** -24)
        got = ops.pointwise_convolution(t["x"], t["w"], t["b"])
        assert got.dtype == torch.float16
        acc64, mag = check_conv(oracle, got.cpu().numpy().astype(np.float32), d, tol, half=True)
        for quant, act in ((FPQ_U, "relu6"), (FPQ_S, None), (POW2, "relu")):
            y = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, quant, act)
            assert y.dtype == torch.float16
            lo, hi = bracket(oracle, acc64, mag, tol, d, 1e-5, act, quant)
            g = y.cpu().numpy()
            assert np.all((g >= lo.astype(np.float16)) & (g <= hi.astype(np.float16))), (shape, quant, act)
        # the prepared form is the same computation
        ws = ops.pwconv_prepare(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, act="relu6")
        y2 = ops.fused_pw_bn_quant_prepared(t["x"], t["w"], ws, True, FPQ_U, "relu6")
        y1 = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, FPQ_U, "relu6")
        assert torch.equal(y1.view(torch.int16), y2.view(torch.int16))
    ops.check_device_flag()


@pytest.mark.parametrize("shape,ctas", [((2, 24, 40, 8, 16), 0), ((2, 96, 24, 56, 56), 0), ((1, 144, 320, 16, 24), 0),
                                        ((3, 32, 96, 112, 112), 0), ((2, 384, 64, 16, 8), 0), ((4, 64, 200, 28, 28), 2),
                                        ((9, 72, 16, 24, 24), 3)],
                         ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else "ctas%d" % v)
def test_fp16_tensors_through_tma_and_binary16_mmas(oracle, cuda_device, shape, ctas):
    """binary16 tensors whose rows are multiples of 16 bytes: TMA loads of x and w as they are,
    tcgen05.mma.kind::f16 (products of binary16 factors are exact in the fp32 accumulator), 64
    channels per stage - one, two and more stages per sum, a last stage of 8 to 48 channels, planes
    that end inside a tile, several tiles per CTA. Random data within the accumulation's tolerance;
    small-integer data (every sum exact) bit for bit."""
    n, ci, co, h, w = shape
    rng = np.random.default_rng(sum(shape))
    d = make(rng, *shape, dtype=np.float16)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    desc, _ = ops.pwconv_desc(t["x"], t["w"])
    assert ops.pwconv_tiling(desc, t["x"].data_ptr())["x_path"] == 0
    tol = (ci + 4) * 2.0 ** -23
    try:
        ops.set_pw_max_ctas(ctas)
        got = ops.pointwise_convolution(t["x"], t["w"], t["b"])
        acc64, mag = check_conv(oracle, got.cpu().numpy().astype(np.float32), d, tol, half=True)
        for quant, act in ((FPQ_U, "relu6"), (FPQ_S, None)):
            y = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, quant, act)
            lo, hi = bracket(oracle, acc64, mag, tol, d, 1e-5, act, quant)
            g = y.cpu().numpy()
            assert np.all((g >= lo.astype(np.float16)) & (g <= hi.astype(np.float16))), (shape, quant, act)
        # the gathered path on the same tensors (an x that starts 8 bytes into its buffer) agrees to the last bit
        # of the fp32 sums' tolerance, and exactly on exactly summable data
        xi = (rng.integers(-40, 56, (n, ci, h, w)) / 8.0).astype(np.float16)
        wi = (rng.integers(-31, 32, (co, ci, 1, 1)) / 16.0).astype(np.float16)
        bi = (rng.integers(-24, 25, co) / 8.0).astype(np.float16)
        exact = np.einsum("nchw,oc->nohw", xi.astype(np.float64), wi[:, :, 0, 0].astype(np.float64)) + \
            bi.astype(np.float64)[None, :, None, None]
        conv = ops.pointwise_convolution(dev(xi, cuda_device), dev(wi, cuda_device), dev(bi, cuda_device))
        assert np.array_equal(conv.cpu().numpy().view(np.uint16), exact.astype(np.float16).view(np.uint16))
        buf = torch.empty(xi.size + 4, dtype=torch.float16, device=cuda_device)
        shifted = buf[4:].view(xi.shape)
        shifted.copy_(dev(xi, cuda_device))
        assert ops.pwconv_tiling(desc, shifted.data_ptr())["x_path"] != 0
        conv2 = ops.pointwise_convolution(shifted, dev(wi, cuda_device), dev(bi, cuda_device))
        assert torch.equal(conv.view(torch.int16), conv2.view(torch.int16))
    finally:
        ops.set_pw_max_ctas(0)
    ops.check_device_flag()


def test_forced_kernel_choice_and_the_two_kernels_agree(oracle, cuda_device):
    rng = np.random.default_rng(2)
    d = make(rng, 2, 64, 96, 14, 14)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    try:
        ops.set_forced_pw_path(0)
        assert ops.pwconv_plan(t["x"], t["w"]) == 0
        fma = ops.pointwise_convolution(t["x"], t["w"], t["b"]).cpu().numpy()
        ops.set_forced_pw_path(1)
        tc = ops.pointwise_convolution(t["x"], t["w"], t["b"]).cpu().numpy()
        odd = dev(rng.standard_normal((1, 30, 7, 7), dtype=np.float32), cuda_device)
        with pytest.raises(L.DwbnqError) as e:
            ops.pointwise_convolution(odd, dev(rng.standard_normal((8, 30, 1, 1), dtype=np.float32), cuda_device), None)
        assert e.value.status == 2
    finally:
        ops.set_forced_pw_path(-1)
    _, acc64, mag = oracle.pwconv(d["x"], d["w"], d["b"])
    assert np.all(np.abs(fma - tc) <= (4e-6 + 68 * 2.0 ** -24) * mag)
    ops.check_device_flag()


@pytest.mark.parametrize("plane", [(36, 40), (14, 14), (7, 7)], ids=lambda s: "%dx%d" % s)
@pytest.mark.parametrize("co", [16, 96, 144, 200, 384], ids=lambda c: "co%d" % c)
@pytest.mark.parametrize("math", ["fp32", "tf32"])
def test_many_tiles_per_cta(oracle, cuda_device, co, math, plane):
    """Three CTAs walk through 60 to 120 tiles each: every pipeline stage and every accumulator
    buffer is reused many times, with the plain (fast) and the fused (slower) epilogue, for every
    buffer count the channel tile widths give (8, 4, 3, 2 buffers)."""
    rng = np.random.default_rng(co)
    # 1440 positions = 11.25 tiles per image through TMA; 14x14 planes gathered across images
    d = make(rng, 12 * 1440 // (plane[0] * plane[1]), 40, co, *plane)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    try:
        ops.set_pw_max_ctas(3)
        conv = ops.pointwise_convolution(t["x"], t["w"], t["b"], math=math).cpu().numpy()
        y = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, FPQ_U, "relu6",
                                  math=math).cpu().numpy()
    finally:
        ops.set_pw_max_ctas(0)
    ops.check_device_flag()
    check_conv(oracle, conv, d, conv_tolerance(1, math, 40))
    want = oracle.pw_epilogue(conv, d["beta"], d["gamma"], d["mean"], d["var"], 1e-5, "relu6", FPQ_U)
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))


def test_one_prepared_workspace_serves_every_batch_size(oracle, cuda_device):
    """The channel tiling is chosen per launch (160 -> 960 on 7x7: eight tiles of 128 columns for two
    images, four of 256 - 240 used - for 256 images); the workspace does not depend on it: prepared once, used at
    both batch sizes, bit-identical to the one-call form, and the small batch checked against the oracle."""
    rng = np.random.default_rng(77)
    d = make(rng, 256, 160, 960, 7, 7)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    small = t["x"][:2].contiguous()
    ws = ops.pwconv_prepare(small, t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, act="relu6")
    for x in (small, t["x"]):
        got = ops.fused_pw_bn_quant_prepared(x, t["w"], ws, True, FPQ_U, "relu6")
        want = ops.fused_pw_bn_quant(x, t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, FPQ_U, "relu6")
        torch.cuda.synchronize()
        ops.check_device_flag()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), tuple(x.shape)
    for x in (small, t["x"][:40].contiguous()):
        conv = ops.pointwise_convolution(x, t["w"], t["b"]).cpu().numpy()
        check_conv(oracle, conv, dict(d, x=x.cpu().numpy()), conv_tolerance(1, "fp32", 160))
        y = ops.fused_pw_bn_quant_prepared(x, t["w"], ws, True, FPQ_U, "relu6").cpu().numpy()
        want = oracle.pw_epilogue(conv, d["beta"], d["gamma"], d["mean"], d["var"], 1e-5, "relu6", FPQ_U)
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("shape,ctas", [((5, 256, 160, 16, 16), 2), ((3, 64, 96, 14, 14), 1), ((2, 960, 160, 7, 7), 0),
                                        ((6, 40, 200, 8, 16), 1), ((4, 320, 72, 12, 12), 1)],
                         ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else "ctas%d" % v)
def test_few_tiles_per_cta_share_the_columns(oracle, cuda_device, shape, ctas):
    """At most six tiles per CTA and 64 or more columns per tile: the four epilogue groups split every
    tile's column units (20, 12, 16 + 9, 9 units: even and ragged quarters, a group without any)
    and walk through the accumulator buffers together, more tiles than buffers (phases wrap)."""
    rng = np.random.default_rng(sum(shape))
    d = make(rng, *shape)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    try:
        ops.set_pw_max_ctas(ctas)
        for math in ("fp32", "tf32"):
            conv = ops.pointwise_convolution(t["x"], t["w"], t["b"], math=math).cpu().numpy()
            y = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, FPQ_S, None,
                                      math=math).cpu().numpy()
            ops.check_device_flag()
            check_conv(oracle, conv, d, conv_tolerance(1, math, shape[1]))
            want = oracle.pw_epilogue(conv, d["beta"], d["gamma"], d["mean"], d["var"], 1e-5, None, FPQ_S)
            assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), math
    finally:
        ops.set_pw_max_ctas(0)


@pytest.mark.parametrize("shape", [(3, 32, 96, 28, 28), (4, 384, 64, 14, 14), (5, 160, 200, 7, 7), (2, 30, 50, 5, 9)],
                         ids=lambda s: "x".join(map(str, s)))
def test_prepared_workspace_gives_the_same_result(oracle, cuda_device, shape):
    """dwbnq_pwconv_prepare once, then dwbnq_pwconv_fused_fwd_prepared on several inputs: bit-identical
    to the one-call form, which is the two in sequence; the parameters are not read again (they
    are overwritten between the calls here)."""
    rng = np.random.default_rng(sum(shape))
    d = make(rng, *shape)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    for math in ("fp32", "tf32"):
        for quant, act, bn in ((FPQ_U, "relu6", True), (FPQ_S, None, True), (POW2, "relu", False)):
            m, v, g, be = (t["mean"], t["var"], t["gamma"], t["beta"]) if bn else (None,) * 4
            want = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], be, g, m, v, 1e-4, quant, act, math=math)
            w2, b2 = t["w"].clone(), t["b"].clone()
            ws = ops.pwconv_prepare(t["x"], w2, b2, be, g, m, v, 1e-4, act=act, math=math)
            torch.cuda.synchronize()
            w2.fill_(float("nan"))
            b2.fill_(float("nan"))
            got = ops.fused_pw_bn_quant_prepared(t["x"], t["w"], ws, bn, quant, act, math=math)
            assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (math, quant, act, bn)
            x2 = (t["x"] * 0.5 + 0.25).contiguous()
            want2 = ops.fused_pw_bn_quant(x2, t["w"], t["b"], be, g, m, v, 1e-4, quant, act, math=math)
            got2 = ops.fused_pw_bn_quant_prepared(x2, t["w"], ws, bn, quant, act, math=math)
            assert torch.equal(got2.view(torch.int32), want2.view(torch.int32)), (math, quant, act, bn)
    ops.check_device_flag()


def test_argument_errors(cuda_device):
    x = torch.zeros(1, 8, 4, 4, device=cuda_device)
    w = torch.zeros(16, 8, 1, 1, device=cuda_device)
    with pytest.raises(ValueError):
        ops.pointwise_convolution(x, torch.zeros(16, 8, 3, 3, device=cuda_device))
    with pytest.raises(L.DwbnqError) as e:  # MinMaxQuantize cannot be fused here
        ops.fused_pw_bn_quant(x, w, None, None, None, None, None, quant={"kind": "minmax"})
    assert e.value.status == 2
    d, _ = ops.pwconv_desc(x, w)
    d.math = 7
    assert L.lib().dwbnq_pwconv_workspace_bytes(d) == 0
    # an empty batch is a no-op
    y = ops.pointwise_convolution(torch.zeros(0, 8, 4, 4, device=cuda_device), w)
    assert tuple(y.shape) == (0, 16, 4, 4)


@pytest.mark.parametrize("layer", [(112, 32, 16), (56, 96, 24), (28, 144, 32), (14, 384, 64), (14, 96, 576)],
                         ids=lambda l: "%dx%d_%dto%d" % (l[0], l[0], l[1], l[2]))
def test_mobilenet_layers_at_eight_images(oracle, cuda_device, layer):
    hw, ci, co = layer
    rng = np.random.default_rng(hw + ci)
    d = make(rng, 8, ci, co, hw, hw)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    ws = ops.pwconv_workspace(t["x"], t["w"])
    conv = ops.pointwise_convolution(t["x"], t["w"], t["b"], ws=ws).cpu().numpy()
    check_conv(oracle, conv, d, 4e-6)
    y = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, FPQ_U, "relu6", ws=ws)
    want = oracle.pw_epilogue(conv, d["beta"], d["gamma"], d["mean"], d["var"], 1e-5, "relu6", FPQ_U,
                              nthreads=oracle.max_threads())
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))
    ops.check_device_flag()


@pytest.mark.parametrize("index", [1, 4, 14, 21, 27, 28, 32], ids=lambda i: "pw1.l%02d" % i)
def test_full_size_layers_of_the_bench_workload(oracle, cuda_device, index):
    """The bench's own layers at its own batch (256 images: the tile widths, the shared-column
    epilogue and the number of tiles per CTA are chosen from the batch, so small batches take other
    routes): sampled images of the convolution against the oracle within the stated tolerance, and
    the whole fused output bit for bit against the library's standalone BatchNormalization ->
    ReLU6 -> FixedPointQuantize (each bit-exact against the oracle in its own tests) applied to
    the convolution the same kernel returns unfused."""
    from dwbnq import workloads
    spec = workloads.pw1(256)[index]
    d = workloads.make_pointwise_data(spec)
    t = {k: dev(v, cuda_device) for k, v in d.items()}
    conv = ops.pointwise_convolution(t["x"], t["w"], t["b"])
    y = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], spec.bn_eps, spec.quant,
                              spec.act)
    torch.cuda.synchronize()
    ops.check_device_flag()
    pick = [0, 1, 127, 255]
    sub = dict(d, x=np.ascontiguousarray(d["x"][pick]))
    check_conv(oracle, conv[pick].cpu().numpy(), sub, conv_tolerance(1, "fp32", spec.c_in))
    chain = ops.batch_normalization(conv, t["beta"], t["gamma"], t["mean"], t["var"], eps=spec.bn_eps, batch_stat=False)
    if spec.act == "relu6":
        chain = chain.clamp(0.0, 6.0)
    q = spec.quant
    chain = ops.fixed_point_quantize(chain, q["sign"], q["n"], q["delta"])
    assert torch.equal(y.view(torch.int32), chain.view(torch.int32))
    want = oracle.pw_epilogue(conv[pick].cpu().numpy(), d["beta"], d["gamma"], d["mean"], d["var"], spec.bn_eps, spec.act, q)
    assert np.array_equal(y[pick].cpu().numpy().view(np.uint32), want.view(np.uint32))
