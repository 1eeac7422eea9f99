"""Out-of-bounds writes, without a memory checker: every output tensor lives in the middle of a
larger allocation whose margins (4 KiB before, 4 KiB after) hold a known pattern, every input is
copied beforehand; after each operator - every kernel family, on edge shapes where tiles are
ragged - the margins must still hold the pattern and the inputs must be unchanged. (compute-
sanitizer is not available on the test machines; a kernel that wrote one element past its
output, or scribbled on an operand, shows up here.)"""
import numpy as np
import pytest
import torch

from dwbnq import ops

pytestmark = pytest.mark.gpu

MARGIN = 4096  # bytes
PATTERN = 0x5A


class Guarded:
    """A tensor of `shape` carved out of a byte buffer with MARGIN bytes of PATTERN on both sides."""

    def __init__(self, shape, dtype, device, offset=0):
        self.nbytes = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        self.offset = offset  # extra bytes in front, to test views that are not 256-byte aligned
        self.buf = torch.full((MARGIN + offset + self.nbytes + MARGIN,), PATTERN, dtype=torch.uint8, device=device)
        self.t = self.buf[MARGIN + offset:MARGIN + offset + self.nbytes].view(dtype).view(shape)

    def check(self, what):
        head = self.buf[:MARGIN + self.offset]
        tail = self.buf[MARGIN + self.offset + self.nbytes:]
        assert bool((head == PATTERN).all()), "%s wrote before its output" % what
        assert bool((tail == PATTERN).all()), "%s wrote past its output" % what
        written = self.t.reshape(-1).view(torch.uint8)
        assert not bool((written == PATTERN).all()) or self.nbytes == 0, "%s left its output untouched" % what


def unchanged(before, after, what):
    for k in before:
        if before[k] is not None:
            assert torch.equal(before[k].view(torch.uint8), after[k].contiguous().view(torch.uint8)), "%s changed its input %s" % (what, k)


def params(rng, c, device, dtype):
    mk = lambda a: torch.from_numpy(a.astype(np.float32)).to(device).to(dtype)
    return {"b": mk(rng.standard_normal(c) * 0.3), "beta": mk(rng.standard_normal(c) * 0.3), "gamma": mk(0.8 + 0.4 * rng.random(c)),
            "mean": mk(rng.standard_normal(c) * 0.3), "var": mk(0.5 + rng.random(c))}


FPQ = {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3}
POW2 = {"kind": "pow2", "sign": True, "with_zero": True, "n": 8, "m": 1}

DW_CASES = [
    # n, c, h, w, k, stride, pad, forced family (-1 = the planner's choice)
    (3, 5, 7, 7, 3, 1, 1, -1), (2, 7, 14, 14, 3, 1, 1, -1), (2, 3, 28, 28, 3, 2, 1, -1), (1, 3, 56, 56, 3, 1, 1, -1),
    (1, 2, 112, 112, 3, 2, 1, -1), (2, 3, 14, 14, 5, 1, 2, -1), (2, 3, 9, 11, 3, 1, 1, -1), (1, 4, 13, 10, 5, 2, 2, -1),
    (2, 3, 20, 24, 3, 1, 1, 5), (2, 3, 17, 19, 3, 1, 0, 0), (2, 5, 33, 40, 3, 1, 1, 1), (2, 5, 33, 40, 3, 2, 1, 2),
    (3, 4, 15, 15, 3, 1, 1, 3),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("case", DW_CASES, ids=lambda c: "x".join(map(str, c)))
def test_fused_depthwise_layer_stays_inside_its_output(cuda_device, case, dtype):
    n, c, h, w, k, stride, pad, family = case
    rng = np.random.default_rng(sum(case) + 100)
    x = torch.from_numpy(rng.standard_normal((n, c, h, w)).astype(np.float32)).to(cuda_device).to(dtype)
    wt = torch.from_numpy((rng.standard_normal((c, k, k)) / k).astype(np.float32)).to(cuda_device).to(dtype)
    p = params(rng, c, cuda_device, dtype)
    ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    ins = dict(p, x=x, w=wt)
    before = {kk: v.clone() for kk, v in ins.items()}
    try:
        ops.set_forced_path(family)
        for quant in (FPQ, POW2, None):
            for offset in (0, 16):
                y = Guarded((n, c, ho, wo), dtype, cuda_device, offset)
                ops.fused_dw_bn_quant(x, wt, p["b"], p["beta"], p["gamma"], p["mean"], p["var"], 1e-5, pad=(pad, pad),
                                      stride=(stride, stride), quant=quant, out=y.t)
                torch.cuda.synchronize()
                y.check("fused_dw_bn_quant %s" % (case,))
    finally:
        ops.set_forced_path(-1)
    unchanged(before, ins, "fused_dw_bn_quant %s" % (case,))
    ops.check_device_flag()


def test_minmax_layer_and_standalone_operators(cuda_device):
    rng = np.random.default_rng(3)
    n, c, h, w = 3, 6, 14, 14
    x = torch.from_numpy(rng.standard_normal((n, c, h, w)).astype(np.float32)).to(cuda_device)
    wt = torch.from_numpy((rng.standard_normal((c, 3, 3)) / 3).astype(np.float32)).to(cuda_device)
    p = params(rng, c, cuda_device, torch.float32)
    rng_t = [Guarded((c,), torch.float32, cuda_device) for _ in range(2)]
    rng_t[0].t.zero_()
    rng_t[1].t.fill_(1.0)
    ql = [torch.zeros(c, device=cuda_device), torch.full((c,), 255.0, device=cuda_device)]
    q = {"kind": "minmax", "x_min_max": True, "ema": False, "decay": 0.999, "eps": 0.01, "qr_min": rng_t[0].t, "qr_max": rng_t[1].t,
         "ql_min": ql[0], "ql_max": ql[1]}
    ws = Guarded((ops.workspace(c, cuda_device).numel(),), torch.uint8, cuda_device)
    y = Guarded((n, c, h, w), torch.float32, cuda_device)
    ops.fused_dw_bn_quant(x, wt, p["b"], p["beta"], p["gamma"], p["mean"], p["var"], 1e-5, pad=(1, 1), stride=(1, 1), quant=q,
                          ws=ws.t, out=y.t)
    torch.cuda.synchronize()
    for g, name in ((y, "y"), (ws, "workspace"), (rng_t[0], "qr_min"), (rng_t[1], "qr_max")):
        g.check("fused MinMaxQuantize layer (%s)" % name)
    xin = x.clone()
    for name, fn in (
            ("depthwise_convolution", lambda o: ops.depthwise_convolution(x, wt, p["b"], 1, (1, 1), (1, 1), out=o)),
            ("batch_normalization", lambda o: ops.batch_normalization(x, p["beta"], p["gamma"], p["mean"], p["var"], out=o)),
            ("fixed_point_quantize", lambda o: ops.fixed_point_quantize(x, True, 8, 2.0 ** -4, out=o)),
            ("pow2_quantize", lambda o: ops.pow2_quantize(x, True, True, 8, 1, out=o)),
            ("min_max_quantize", lambda o: ops.min_max_quantize(x, rng_t[0].t, rng_t[1].t, ql[0], ql[1], x_min_max=True, ws=ws.t, out=o))):
        for offset in (0, 4):
            o = Guarded((n, c, h, w), torch.float32, cuda_device, offset)
            fn(o.t)
            torch.cuda.synchronize()
            o.check(name)
    assert torch.equal(x, xin)
    # a flat tensor whose size is not a multiple of the vector width
    xf = torch.from_numpy(rng.standard_normal(100003).astype(np.float32)).to(cuda_device)
    for name, fn in (("fixed_point_quantize", lambda o: ops.fixed_point_quantize(xf, True, 8, 0.0625, out=o)),
                     ("pow2_quantize", lambda o: ops.pow2_quantize(xf, True, True, 8, 1, out=o))):
        o = Guarded((100003,), torch.float32, cuda_device, 4)
        fn(o.t)
        torch.cuda.synchronize()
        o.check(name + " (flat, odd size)")
    ops.check_device_flag()


def test_backward_kernels(cuda_device):
    rng = np.random.default_rng(4)
    for n, c, h, w, k, stride, pad in ((3, 5, 14, 14, 3, 1, 1), (2, 3, 9, 11, 3, 2, 1), (2, 4, 12, 12, 5, 1, 2)):
        x = torch.from_numpy(rng.standard_normal((n, c, h, w)).astype(np.float32)).to(cuda_device)
        wt = torch.from_numpy((rng.standard_normal((c, k, k)) / k).astype(np.float32)).to(cuda_device)
        ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        dy = torch.from_numpy(rng.standard_normal((n, c, ho, wo)).astype(np.float32)).to(cuda_device)
        dx, dw, db = Guarded((n, c, h, w), torch.float32, cuda_device), Guarded((c, k, k), torch.float32, cuda_device), \
            Guarded((c,), torch.float32, cuda_device)
        ops.depthwise_convolution_backward(x, wt, dy, 1, (pad, pad), (stride, stride), dx=dx.t, dw=dw.t, db=db.t)
        torch.cuda.synchronize()
        for g, name in ((dx, "dx"), (dw, "dw"), (db, "db")):
            g.check("depthwise_convolution_backward %s" % name)
        g = Guarded((n, c, ho, wo), torch.float32, cuda_device)
        ops.fixed_point_quantize_backward(dy, dy, True, 8, 0.0625, True, dx=g.t)
        torch.cuda.synchronize()
        g.check("fixed_point_quantize_backward")
        g = Guarded((n, c, ho, wo), torch.float32, cuda_device)
        ops.pow2_quantize_backward(dy, dy, True, True, 8, 1, True, dx=g.t)
        torch.cuda.synchronize()
        g.check("pow2_quantize_backward")
    ops.check_device_flag()


def test_eight_bit_storage(cuda_device):
    rng = np.random.default_rng(5)
    n, c, h, w = 3, 6, 14, 14
    x = torch.from_numpy(np.clip(rng.standard_normal((n, c, h, w)), 0, 6).astype(np.float32)).to(cuda_device)
    wt = torch.from_numpy((rng.standard_normal((c, 3, 3)) / 3).astype(np.float32)).to(cuda_device)
    p = params(rng, c, cuda_device, torch.float32)
    codes = Guarded((n, c, h, w), torch.uint8, cuda_device, 3)
    ops.quantize_linear_code8(x, 0.125, 0, "HALF_AWAY_FROM_ZERO", False, out=codes.t)
    torch.cuda.synchronize()
    codes.check("quantize_linear_code8")
    back = Guarded((n, c, h, w), torch.float32, cuda_device)
    ops.dequantize_linear_code8(codes.t, 0.125, 0, out=back.t)
    torch.cuda.synchronize()
    back.check("dequantize_linear_code8")
    for stride in (1, 2):
        ho = (h + 2 - 3) // stride + 1
        y = Guarded((n, c, ho, ho), torch.uint8, cuda_device)
        ops.fused_dw_bn_quant_code8(codes.t, 0.125, wt, p["b"], p["beta"], p["gamma"], p["mean"], p["var"], 1e-5, pad=(1, 1),
                                    stride=(stride, stride), quant=FPQ, out=y.t)
        torch.cuda.synchronize()
        y.check("fused_dw_bn_quant_code8 stride %d" % stride)
    ops.check_device_flag()


PW_CASES = [
    # n, c_in, c_out, h, w
    (2, 32, 64, 16, 16), (3, 24, 144, 12, 10), (1, 96, 24, 28, 28), (2, 192, 320, 14, 14), (5, 160, 70, 7, 7), (2, 8, 16, 5, 9),
    (1, 4, 8, 1, 1), (3, 30, 50, 5, 9), (2, 512, 300, 6, 6),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("case", PW_CASES, ids=lambda c: "x".join(map(str, c)))
def test_pointwise_convolution_stays_inside_its_output(cuda_device, case, dtype):
    n, ci, co, h, w = case
    rng = np.random.default_rng(sum(case))
    x = torch.from_numpy(np.clip(rng.standard_normal((n, ci, h, w)) * 2, -1, 6).astype(np.float32)).to(cuda_device).to(dtype)
    wt = torch.from_numpy((rng.standard_normal((co, ci, 1, 1)) / np.sqrt(ci)).astype(np.float32)).to(cuda_device).to(dtype)
    p = params(rng, co, cuda_device, dtype)
    ins = dict(p, x=x, w=wt)
    before = {kk: v.clone() for kk, v in ins.items()}
    maths = ("fp32", "tf32") if dtype == torch.float32 else ("fp32",)
    for math in maths:
        ws = Guarded((ops.pwconv_workspace(x, wt).numel(),), torch.uint8, cuda_device)
        for offset in ((0, 4) if dtype == torch.float32 else (0, 2)):  # a y (and an x) that TMA could not take
            y = Guarded((n, co, h, w), dtype, cuda_device, offset)
            ops.pointwise_convolution(x, wt, p["b"], math=math, ws=ws.t, out=y.t)
            torch.cuda.synchronize()
            y.check("pointwise_convolution %s %s" % (case, math))
            ws.check("pointwise_convolution workspace")
            for quant, act in ((FPQ, "relu6"), (POW2, None)):
                y = Guarded((n, co, h, w), dtype, cuda_device, offset)
                ops.fused_pw_bn_quant(x, wt, p["b"], p["beta"], p["gamma"], p["mean"], p["var"], 1e-5, quant, act, math=math,
                                      ws=ws.t, out=y.t)
                torch.cuda.synchronize()
                y.check("fused_pw_bn_quant %s %s" % (case, math))
        xo = Guarded((n, ci, h, w), dtype, cuda_device, 4 if dtype == torch.float32 else 2)  # x itself off the 16-byte grid
        xo.t.copy_(x)
        y = Guarded((n, co, h, w), dtype, cuda_device)
        ops.fused_pw_bn_quant(xo.t, wt, p["b"], p["beta"], p["gamma"], p["mean"], p["var"], 1e-5, FPQ, "relu6", math=math, ws=ws.t,
                              out=y.t)
        torch.cuda.synchronize()
        y.check("fused_pw_bn_quant with an unaligned x %s" % (case,))
        xo.check("fused_pw_bn_quant (its input)")
    unchanged(before, ins, "pointwise %s" % (case,))
    ops.check_device_flag()
