"""The nbla registry plugin (nnabla-ext-cuda_b200/nbla_plugin) compiled against a stand-in
for nnabla core's C++ interface (tests/nbla_stub: nnabla itself cannot be installed here) and
driven end to end: registration under the reference's (function, backend) keys, class names,
the forward of each of the five functions on device buffers against the CPU oracle, the fused
function object a graph converter substitutes for a dw-conv -> BN -> quantizer chain (through
its extern "C" factory, float and half, every quantizer), the function object for the pointwise
convolution -> BN -> activation -> quantizer chain, and the refusal of backward. What this cannot show - link compatibility with a real libnnabla - stays
open until the plugin is built in an nnabla tree."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, ".."))
PKG = os.path.join(ROOT, "nnabla-ext-cuda_b200")
STUB = os.path.join(HERE, "nbla_stub")
FUNCTIONS = ["DepthwiseConvolution", "BatchNormalization", "FixedPointQuantize", "Pow2Quantize", "MinMaxQuantize"]


@pytest.fixture(scope="module")
def harness(dwlib):
    out_dir = os.path.join(STUB, "_build")
    os.makedirs(out_dir, exist_ok=True)
    so = os.path.join(out_dir, "libdwbnq_nbla_stub.so")
    srcs = [os.path.join(PKG, "nbla_plugin", "dwbnq_nbla_plugin.cpp"), os.path.join(STUB, "harness.cpp")]
    deps = srcs + [os.path.join(STUB, "nbla", "stub_core.hpp"), os.path.join(ROOT, "include", "dwbnq.h")]
    if not os.path.exists(so) or any(os.path.getmtime(d) > os.path.getmtime(so) for d in deps):
        cmd = ["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-I" + STUB, "-I" + os.path.join(ROOT, "include")] + srcs + \
              ["-L" + PKG, "-ldwbnq", "-Wl,-rpath," + PKG, "-o", so]
        subprocess.run(cmd, check=True, capture_output=True, text=True)
    lib = ctypes.CDLL(so)
    lib.stub_last_error.restype = ctypes.c_char_p
    return lib


def test_registration_and_names(harness):
    for f in FUNCTIONS:
        for backend in (b"cuda:float", b"cuda:half"):
            assert harness.stub_registered(f.encode(), backend) == 1, (f, backend)
    assert harness.stub_registered(b"Convolution", b"cuda:float") == 0
    buf = ctypes.create_string_buffer(64)
    assert harness.stub_name(b"cuda:float", 0, buf, 64) == 0
    assert buf.value == b"FixedPointQuantizeCuda"


def test_backward_raises_not_implemented(harness):
    """MinMaxQuantize (like BatchNormalization and the fused object) has no backward here."""
    rc = harness.stub_backward_is_refused(0)
    assert rc == 100 + 1, rc  # error_code::not_implemented
    assert b"forward pass only" in harness.stub_last_error()


def test_fused_function_backward_raises_not_implemented(harness):
    rc = harness.stub_fused_backward_is_refused(0)
    assert rc == 100 + 1, rc
    assert b"FusedDwBnQuantCuda" in harness.stub_last_error()


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _shape(a):
    return (ctypes.c_int64 * a.dim())(*a.shape)


@pytest.mark.gpu
@pytest.mark.parametrize("half", [0, 1], ids=["float", "half"])
def test_forward_of_the_five_functions(harness, oracle, cuda_device, half):
    import torch
    rng = np.random.default_rng(7)
    dt = torch.float16 if half else torch.float32
    n, c, hw = 3, 24, 14

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device).to(dt)

    def host(t):
        return t.float().cpu().numpy() if half else t.cpu().numpy()

    def want16(a):
        return oracle.to_f16_result(a).astype(np.float32) if half else a

    x = rng.standard_normal((n, c, hw, hw)).astype(np.float32)
    w = (rng.standard_normal((c, 3, 3)) / 3).astype(np.float32)
    vec = {k: (rng.random(c) + 0.5).astype(np.float32) for k in ("b", "beta", "gamma", "mean", "var")}
    if half:  # the oracle computes on the fp16-rounded inputs
        x, w = x.astype(np.float16).astype(np.float32), w.astype(np.float16).astype(np.float32)
        vec = {k: v.astype(np.float16).astype(np.float32) for k, v in vec.items()}
    tx, tw = dev(x), dev(w)
    tv = {k: dev(v) for k, v in vec.items()}
    dev_index = cuda_device.index or 0

    # DepthwiseConvolution, stride 2 pad 1
    y = torch.empty((n, c, 7, 7), device=cuda_device, dtype=dt)
    rc = harness.stub_dwconv(half, dev_index, _shape(tx), _shape(tw), 4, _p(tx), _p(tw), _p(tv["b"]), _p(y), 1, 2, 1, 1)
    assert rc == 0, harness.stub_last_error()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host(y), want16(oracle.dwconv(x, w, vec["b"], (2, 2), (1, 1))))

    # BatchNormalization, batch_stat=False, with and without gamma / beta
    for use_beta, use_gamma in ((True, True), (False, True), (True, False)):
        y = torch.empty_like(tx)
        rc = harness.stub_bn(half, dev_index, _shape(tx), 4, _p(tx), _p(tv["beta"] if use_beta else None),
                             _p(tv["gamma"] if use_gamma else None), _p(tv["mean"]), _p(tv["var"]), _p(y),
                             ctypes.c_float(1e-5), 0)
        assert rc == 0, harness.stub_last_error()
        torch.cuda.synchronize()
        want = oracle.bn_infer(x, vec["beta"] if use_beta else None, vec["gamma"] if use_gamma else None, vec["mean"],
                               vec["var"], 1e-5)
        np.testing.assert_array_equal(host(y), want16(want))
    # batch_stat=True is refused with not_implemented
    rc = harness.stub_bn(half, dev_index, _shape(tx), 4, _p(tx), _p(tv["beta"]), _p(tv["gamma"]), _p(tv["mean"]),
                         _p(tv["var"]), _p(y), ctypes.c_float(1e-5), 1)
    assert rc == 100 + 1

    # FixedPointQuantize / Pow2Quantize
    y = torch.empty_like(tx)
    rc = harness.stub_fpq(half, dev_index, tx.numel(), _p(tx), _p(y), 1, 8, ctypes.c_float(2.0 ** -4))
    assert rc == 0, harness.stub_last_error()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host(y), want16(oracle.fpq(x, True, 8, 2.0 ** -4)))
    rc = harness.stub_pow2(half, dev_index, tx.numel(), _p(tx), _p(y), 1, 1, 8, 1)
    assert rc == 0, harness.stub_last_error()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host(y), want16(oracle.pow2q(x, True, True, 8, 1)))

    # MinMaxQuantize, per-channel ranges [1, C, 1, 1], updated in place
    qr_min, qr_max = dev(np.zeros(c, np.float32)), dev(np.ones(c, np.float32))
    ql_min, ql_max = dev(np.zeros(c, np.float32)), dev(np.full(c, 255, np.float32))
    scratch = torch.empty(64 * c + 1024, device=cuda_device, dtype=torch.float32)
    harness.stub_set_scratch(_p(scratch))
    rc = harness.stub_minmax(half, dev_index, _shape(tx), 4, _p(tx), _p(qr_min), _p(qr_max), _p(ql_min), _p(ql_max), _p(y),
                             ctypes.c_float(0.999), 1, 0, ctypes.c_float(0.01))
    assert rc == 0, harness.stub_last_error()
    torch.cuda.synchronize()
    want, wmin, wmax = oracle.minmaxq(x, np.zeros(c, np.float32), np.ones(c, np.float32), np.zeros(c, np.float32),
                                      np.full(c, 255, np.float32), 0.999, True, False, 0.01)
    np.testing.assert_array_equal(host(y), want16(want))
    if not half:
        np.testing.assert_array_equal(qr_min.cpu().numpy(), wmin)
        np.testing.assert_array_equal(qr_max.cpu().numpy(), wmax)


@pytest.mark.gpu
@pytest.mark.parametrize("half", [0, 1], ids=["float", "half"])
def test_fused_pointwise_function_object(harness, oracle, cuda_device, half):
    """FusedPwBnQuantCuda through dwbnq_nbla_create_fused_pw: Convolution 1x1 -> BN -> activation ->
    quantizer as one function object; output shape from setup, a copy() run instead of the
    original. The result is bracketed by the oracle's epilogue of (double sum -/+ tolerance); for
    float it is also bit-identical to the oracle's epilogue of the library's own convolution."""
    import torch
    from dwbnq import ops
    rng = np.random.default_rng(17)
    dt = torch.float16 if half else torch.float32
    n, ci, co, hw = 3, 24, 40, 14
    dev_index = cuda_device.index or 0

    def rnd16(a):
        return a.astype(np.float16).astype(np.float32) if half else a

    x = rnd16(np.clip(rng.standard_normal((n, ci, hw, hw)) * 2, -1, 6).astype(np.float32))
    w = rnd16((rng.standard_normal((co, ci, 1, 1)) / np.sqrt(ci)).astype(np.float32))
    vec = {k: rnd16((rng.random(co) + 0.5).astype(np.float32)) for k in ("b", "beta", "gamma", "mean", "var")}
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device).to(dt)
    tx, tw = to(x), to(w)
    tv = {k: to(v) for k, v in vec.items()}
    scratch = torch.empty(1 << 20, device=cuda_device, dtype=torch.uint8)
    harness.stub_set_scratch(_p(scratch))
    _, acc64, mag = oracle.pwconv(x, w, vec["b"])
    tol = (ci + 4) * 2.0 ** -24 if half else 4e-6
    cases = [  # (act name, act code, quant dict, kind, allow_tf32, with b/beta/gamma)
        ("relu6", 2, {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3}, 1, 0, (True, True, True)),
        (None, 0, {"kind": "fpq", "sign": True, "n": 8, "delta": 2.0 ** -4}, 1, 0, (True, True, True)),
        ("relu", 1, {"kind": "pow2", "sign": True, "with_zero": True, "n": 8, "m": 1}, 2, 0, (True, False, True)),
        ("relu6", 2, None, 0, 1, (True, True, False)),
    ]
    for act, act_code, q, kind, tf32, (use_b, use_beta, use_gamma) in cases:
        y = torch.full((n, co, hw, hw), float("nan"), device=cuda_device, dtype=dt)
        ptrs = [tx, tw, tv["b"] if use_b else None, tv["beta"] if use_beta else None, tv["gamma"] if use_gamma else None,
                tv["mean"], tv["var"]]
        arr = (ctypes.c_void_p * 7)(*[_p(t) for t in ptrs])
        out_shape = (ctypes.c_int64 * 4)()
        n_inputs, copies_ok = ctypes.c_int(), ctypes.c_int()
        qa = q or {}
        rc = harness.stub_fused_pw(half, dev_index, _shape(tx), _shape(tw), arr, _p(y), ctypes.c_float(1e-5), act_code, kind,
                                   int(qa.get("sign", 0)), int(qa.get("with_zero", 0)), int(qa.get("n", 8)),
                                   int(qa.get("m", 0)), ctypes.c_float(qa.get("delta", 0.0)), tf32, out_shape,
                                   ctypes.byref(n_inputs), ctypes.byref(copies_ok))
        assert rc == 0, harness.stub_last_error()
        torch.cuda.synchronize()
        assert list(out_shape) == [n, co, hw, hw]
        assert n_inputs.value == 4 + use_b + use_beta + use_gamma
        assert copies_ok.value == 1
        beta = vec["beta"] if use_beta else None
        gamma = vec["gamma"] if use_gamma else None
        t = (2.0 ** -9 if tf32 else tol)
        lo = oracle.pw_epilogue(acc64 - (t * mag).astype(np.float32), beta, gamma, vec["mean"], vec["var"], 1e-5, act, q)
        hi = oracle.pw_epilogue(acc64 + (t * mag).astype(np.float32), beta, gamma, vec["mean"], vec["var"], 1e-5, act, q)
        lo, hi = np.minimum(lo, hi), np.maximum(lo, hi)
        got = y.float().cpu().numpy()
        if half:
            lo, hi = lo.astype(np.float16).astype(np.float32), hi.astype(np.float16).astype(np.float32)
        assert np.all((got >= lo) & (got <= hi)), (act, kind, half)
        if not half:
            conv = ops.pointwise_convolution(tx, tw, tv["b"], math="tf32" if tf32 else "fp32").cpu().numpy()
            want = oracle.pw_epilogue(conv, beta, gamma, vec["mean"], vec["var"], 1e-5, act, q)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (act, kind)


def test_fused_pointwise_factory_rejects_bad_arguments(harness):
    f = harness.dwbnq_nbla_create_fused_pw
    f.restype = ctypes.c_void_p
    assert f(0, 0, 1, 1, ctypes.c_float(1e-5), 0, 0, 3, 1, 0, 0, 8, 0, ctypes.c_float(0.125), 0) is None   # act
    assert f(0, 0, 1, 1, ctypes.c_float(1e-5), 0, 0, 0, 3, 0, 0, 8, 0, ctypes.c_float(0.125), 0) is None   # MinMax
    assert f(0, -1, 1, 1, ctypes.c_float(1e-5), 0, 0, 0, 1, 0, 0, 8, 0, ctypes.c_float(0.125), 0) is None  # device


@pytest.mark.gpu
@pytest.mark.parametrize("half", [0, 1], ids=["float", "half"])
def test_fused_function_object(harness, oracle, cuda_device, half):
    """FusedDwBnQuantCuda through dwbnq_nbla_create_fused: inputs in the order of the three
    functions it replaces, output shape derived in setup, a copy() of the object run instead of
    the original; result against the CPU oracle's three-function chain, bit for bit."""
    import torch
    rng = np.random.default_rng(11)
    dt = torch.float16 if half else torch.float32
    n, c, hw = 3, 24, 14
    dev_index = cuda_device.index or 0

    def rnd16(a):
        return a.astype(np.float16).astype(np.float32) if half else a

    x = rnd16(rng.standard_normal((n, c, hw, hw)).astype(np.float32))
    w = rnd16((rng.standard_normal((c, 3, 3)) / 3).astype(np.float32))
    vec = {k: rnd16((rng.random(c) + 0.5).astype(np.float32)) for k in ("b", "beta", "gamma", "mean", "var")}
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device).to(dt)
    tx, tw = to(x), to(w)
    tv = {k: to(v) for k, v in vec.items()}
    scratch = torch.empty(64 * c + 1024, device=cuda_device, dtype=torch.float32)
    harness.stub_set_scratch(_p(scratch))
    cases = [
        # (stride, quant dict for the oracle, kind, with b/beta/gamma)
        (1, {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3}, 1, (True, True, True)),
        (2, {"kind": "pow2", "sign": True, "with_zero": True, "n": 8, "m": 1}, 2, (True, True, True)),
        (1, {"kind": "fpq", "sign": True, "n": 8, "delta": 2.0 ** -4}, 1, (False, False, True)),
        (2, {"kind": "minmax", "x_min_max": True, "ema": False, "decay": 0.999, "eps": 0.01}, 3, (True, True, False)),
        (1, None, 0, (True, True, True)),
    ]
    for stride, q, kind, (use_b, use_beta, use_gamma) in cases:
        ho = (hw + 2 - 3) // stride + 1
        y = torch.full((n, c, ho, ho), float("nan"), device=cuda_device, dtype=dt)
        ranges = None
        if kind == 3:
            ranges = [to(np.zeros(c, np.float32)), to(np.ones(c, np.float32)), to(np.zeros(c, np.float32)),
                      to(np.full(c, 255, np.float32))]
            q = dict(q, qr_min=np.zeros(c, np.float32), qr_max=np.ones(c, np.float32),
                     ql_min=np.zeros(c, np.float32), ql_max=np.full(c, 255, np.float32))
        ptrs = [tx, tw, tv["b"] if use_b else None, tv["beta"] if use_beta else None,
                tv["gamma"] if use_gamma else None, tv["mean"], tv["var"]] + (ranges or [None] * 4)
        arr = (ctypes.c_void_p * 11)(*[_p(t) for t in ptrs])
        out_shape = (ctypes.c_int64 * 4)()
        n_inputs, copies_ok = ctypes.c_int(), ctypes.c_int()
        qa = q or {}
        rc = harness.stub_fused(half, dev_index, _shape(tx), _shape(tw), 4, arr, _p(y), 1, stride,
                                ctypes.c_float(1e-5), kind, int(qa.get("sign", 0)), int(qa.get("with_zero", 0)),
                                int(qa.get("n", 8)), int(qa.get("m", 0)), ctypes.c_float(qa.get("delta", 0.0)),
                                ctypes.c_float(qa.get("decay", 0.0)), int(qa.get("x_min_max", 0)), int(qa.get("ema", 0)),
                                ctypes.c_float(qa.get("eps", 0.0)), out_shape, ctypes.byref(n_inputs),
                                ctypes.byref(copies_ok))
        assert rc == 0, harness.stub_last_error()
        torch.cuda.synchronize()
        assert list(out_shape) == [n, c, ho, ho]
        assert n_inputs.value == 4 + use_b + use_beta + use_gamma + (4 if kind == 3 else 0)
        assert copies_ok.value == 1
        want = oracle.fused_layer(x, w, vec["b"] if use_b else None, vec["beta"] if use_beta else None,
                                  vec["gamma"] if use_gamma else None, vec["mean"], vec["var"], 1e-5,
                                  (stride, stride), (1, 1), q or {"kind": "none"}, nthreads=oracle.max_threads())
        if kind == 3:
            want, wmin, wmax = want
            if not half:
                np.testing.assert_array_equal(ranges[0].cpu().numpy(), wmin)
                np.testing.assert_array_equal(ranges[1].cpu().numpy(), wmax)
        if half:  # binary16 storage, fp32 arithmetic, one rounding at the store
            want = oracle.to_f16_result(want).astype(np.float32)
        got = y.float().cpu().numpy() if half else y.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (stride, kind, half)


@pytest.mark.gpu
def test_backward_of_the_registered_classes(harness, oracle, cuda_device):
    """backward_impl of FixedPointQuantizeCuda, Pow2QuantizeCuda and DepthwiseConvolutionCuda with
    the reference's propagate_down / accum flags, against the CPU oracle."""
    import torch
    rng = np.random.default_rng(13)
    dev_index = cuda_device.index or 0
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
    x = (rng.standard_normal(5000) * 5).astype(np.float32)
    dy = rng.standard_normal(5000).astype(np.float32)
    old = rng.standard_normal(5000).astype(np.float32)
    tx, tdy = to(x), to(dy)
    for accum in (0, 1):
        dx = to(old)
        rc = harness.stub_quant_bwd(0, 0, dev_index, x.size, _p(tx), _p(tdy), _p(dx), 1, 8, ctypes.c_float(2.0 ** -4), 0, 0,
                                    1, accum, 1)
        assert rc == 0, harness.stub_last_error()
        torch.cuda.synchronize()
        np.testing.assert_array_equal(dx.cpu().numpy(), oracle.fpq_bwd(x, dy, old if accum else None, True, 8, 2.0 ** -4, True))
        dx = to(old)
        rc = harness.stub_quant_bwd(1, 0, dev_index, x.size, _p(tx), _p(tdy), _p(dx), 1, 8, ctypes.c_float(0), 1, 1, 1,
                                    accum, 1)
        assert rc == 0, harness.stub_last_error()
        torch.cuda.synchronize()
        np.testing.assert_array_equal(dx.cpu().numpy(), oracle.pow2q_bwd(x, dy, old if accum else None, True, True, 8, 1, True))
    # propagate_down false: the gradient is not touched
    dx = to(old)
    assert harness.stub_quant_bwd(0, 0, dev_index, x.size, _p(tx), _p(tdy), _p(dx), 1, 8, ctypes.c_float(2.0 ** -4), 0, 0, 1,
                                  0, 0) == 0
    torch.cuda.synchronize()
    np.testing.assert_array_equal(dx.cpu().numpy(), old)

    n, c, hw = 3, 12, 14
    xc = rng.standard_normal((n, c, hw, hw)).astype(np.float32)
    w = (rng.standard_normal((c, 3, 3)) / 3).astype(np.float32)
    b = rng.standard_normal(c).astype(np.float32)
    dyc = rng.standard_normal((n, c, 7, 7)).astype(np.float32)
    wdx, wdw, wdb = oracle.dwconv_bwd(xc, w, dyc, (2, 2), (1, 1))
    txc, tw, tb, tdyc = to(xc), to(w), to(b), to(dyc)
    dx, dw, db = torch.full_like(txc, 9.0), torch.full_like(tw, 9.0), torch.full_like(tb, 9.0)
    rc = harness.stub_dwconv_bwd(0, dev_index, _shape(txc), _shape(tw), 4, _p(txc), _p(tw), _p(tb), _p(tdyc), _p(dx), _p(dw),
                                 _p(db), 1, 2, 1, 1, 0b111, 0)
    assert rc == 0, harness.stub_last_error()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(dx.cpu().numpy(), wdx)  # stride 2: the direct kernel, the reference's order
    np.testing.assert_allclose(dw.cpu().numpy(), wdw, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(db.cpu().numpy(), wdb, rtol=1e-4, atol=1e-4)
    # only the weights, accumulated
    dx2, dw2 = torch.full_like(txc, 9.0), torch.ones_like(tw)
    rc = harness.stub_dwconv_bwd(0, dev_index, _shape(txc), _shape(tw), 4, _p(txc), _p(tw), _p(tb), _p(tdyc), _p(dx2), _p(dw2),
                                 _p(db), 1, 2, 1, 1, 0b010, 0b010)
    assert rc == 0, harness.stub_last_error()
    torch.cuda.synchronize()
    assert float(dx2.min()) == 9.0 and float(dx2.max()) == 9.0
    np.testing.assert_allclose(dw2.cpu().numpy(), wdw + 1.0, rtol=1e-4, atol=1e-4)
    # half: the convolution's backward is not implemented and says so
    rc = harness.stub_dwconv_bwd(1, dev_index, _shape(txc), _shape(tw), 4, _p(txc), _p(tw), _p(tb), _p(tdyc), _p(dx), _p(dw),
                                 _p(db), 1, 2, 1, 1, 0b111, 0)
    assert rc >= 100 and b"DWBNQ_F32" in harness.stub_last_error()
