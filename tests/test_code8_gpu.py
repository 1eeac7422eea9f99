"""8-bit storage of quantized activations: QuantizeLinear / DequantizeLinear with int8 / uint8
codes and the fused layer that reads and writes codes, through the C ABI, against the CPU
oracle. The fused layer's contract: y_code * delta equals the fp32 path's output value for
value, the arithmetic being the same operations in the same order on x = x_code * in_delta."""
import ctypes

import numpy as np
import pytest
import torch

from dwbnq import _lib as L
from dwbnq import ops, workloads

pytestmark = pytest.mark.gpu


def dev(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def _inputs(rng, n):
    x = (rng.standard_normal(n) * 40).astype(np.float32)
    ties = (rng.integers(-300, 300, n // 4) + 0.5).astype(np.float32)  # exact .5 cases
    x[: ties.size] = ties
    x[-4:] = [np.nan, np.inf, -np.inf, -0.0]
    return x


@pytest.mark.parametrize("mode", ["HALF_AWAY_FROM_ZERO", "HALF_TO_EVEN"])
@pytest.mark.parametrize("signed", [False, True], ids=["uint8", "int8"])
def test_quantize_and_dequantize_linear(oracle, cuda_device, mode, signed):
    rng = np.random.default_rng(3)
    for n, scale, zp in ((100003, 0.25, 0), (4096, 0.3, 7), (17, 1.0, -3)):
        x = _inputs(rng, n)
        lo, hi = (-128, 127) if signed else (0, 255)
        want = oracle.quantize_linear(x, scale, zp, mode, lo, hi)
        got = ops.quantize_linear_code8(dev(x, cuda_device), scale, zp, mode, signed)
        assert got.dtype == (torch.int8 if signed else torch.uint8)
        np.testing.assert_array_equal(got.cpu().numpy().astype(np.int32), want)
        # a narrower range, an unaligned view, fp16 input
        want = oracle.quantize_linear(x[1:], scale, zp, mode, lo + 3, hi - 5)
        got = ops.quantize_linear_code8(dev(x, cuda_device)[1:], scale, zp, mode, signed, lo + 3, hi - 5)
        np.testing.assert_array_equal(got.cpu().numpy().astype(np.int32), want)
        xh = x.astype(np.float16)
        want = oracle.quantize_linear(xh.astype(np.float32), scale, zp, mode, lo, hi)
        got = ops.quantize_linear_code8(dev(xh, cuda_device), scale, zp, mode, signed)
        np.testing.assert_array_equal(got.cpu().numpy().astype(np.int32), want)
        # back: (code - zero_point) * scale
        codes = got
        y = ops.dequantize_linear_code8(codes, scale, zp)
        want_y = oracle.dequantize_linear(codes.cpu().numpy().astype(np.int32), scale, zp)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want_y.view(np.uint32))
        yh = ops.dequantize_linear_code8(codes[3:], scale, zp, dtype=torch.float16)
        np.testing.assert_array_equal(yh.cpu().numpy(), want_y[3:].astype(np.float16))
    ops.check_device_flag()


def test_fixed_point_quantize_is_dequantize_of_quantize(oracle, cuda_device):
    """FixedPointQuantize(sign, n, delta) == DequantizeLinear(QuantizeLinear(x, delta, 0, half away,
    [min/delta, max/delta])): the codes are the quantizer's integer levels."""
    rng = np.random.default_rng(4)
    x = (rng.standard_normal(200000) * 6).astype(np.float32)
    xd = dev(x, cuda_device)
    for sign, n, delta in ((False, 8, 2.0 ** -3), (True, 8, 2.0 ** -4), (True, 5, 0.25)):
        top = 2 ** (n - (1 if sign else 0)) - 1
        codes = ops.quantize_linear_code8(xd, delta, 0, "HALF_AWAY_FROM_ZERO", sign, -top if sign else 0, top)
        back = ops.dequantize_linear_code8(codes, delta, 0).cpu().numpy()
        want = oracle.fpq(x, sign, n, delta)
        np.testing.assert_array_equal(back, want)  # value-equal (a -0.0 of the quantizer comes back as +0.0)


def _fused_case(oracle, cuda_device, spec, quant, in_signed, in_delta, rng, bias=True, offset=0):
    d = workloads.make_layer_data(spec)
    lo, hi = (-128, 127) if in_signed else (0, 255)
    xc = rng.integers(lo, hi + 1, d["x"].shape).astype(np.int8 if in_signed else np.uint8)
    x = (xc.astype(np.float32) * np.float32(in_delta)).astype(np.float32)
    t = {k: dev(v, cuda_device) for k, v in d.items() if k != "x"}
    if offset:  # a code tensor that does not start on a 16-byte boundary
        buf = torch.empty(xc.size + 64, dtype=torch.uint8, device=cuda_device)
        xt = buf[offset:offset + xc.size].view(torch.int8 if in_signed else torch.uint8).view(xc.shape)
        xt.copy_(dev(xc, cuda_device))
    else:
        xt = dev(xc, cuda_device)
    y = ops.fused_dw_bn_quant_code8(xt, in_delta, t["w"], t["b"] if bias else None, t["beta"], t["gamma"], t["mean"],
                                    t["var"], spec.bn_eps, pad=(spec.pad,) * 2, stride=(spec.stride,) * 2, quant=quant)
    torch.cuda.synchronize()
    want = oracle.fused_layer(x, d["w"], d["b"] if bias else None, d["beta"], d["gamma"], d["mean"], d["var"],
                              spec.bn_eps, (spec.stride,) * 2, (spec.pad,) * 2, quant, nthreads=oracle.max_threads())
    want_codes = np.round(want / np.float32(quant["delta"])).astype(np.int32)
    assert np.array_equal(want_codes.astype(np.float32) * np.float32(quant["delta"]), want)  # codes are exact
    assert y.dtype == (torch.int8 if quant["sign"] else torch.uint8)
    got = y.cpu().numpy().astype(np.int32)
    assert got.shape == want_codes.shape
    bad = np.argwhere(got != want_codes)
    assert bad.size == 0, "%s: %d codes differ, first at %s: got %d want %d" % (
        spec.name, len(bad), tuple(bad[0]), got[tuple(bad[0])], want_codes[tuple(bad[0])])
    # and the fp32 path on the dequantized input gives the same values
    y32 = ops.fused_dw_bn_quant(dev(x, cuda_device), t["w"], t["b"] if bias else None, t["beta"], t["gamma"], t["mean"],
                                t["var"], spec.bn_eps, pad=(spec.pad,) * 2, stride=(spec.stride,) * 2, quant=quant)
    np.testing.assert_array_equal(ops.dequantize_linear_code8(y, quant["delta"]).cpu().numpy(), y32.cpu().numpy())


@pytest.mark.parametrize("layer", range(17))
def test_fused_code8_every_cfg1_layer(oracle, cuda_device, layer):
    """Every shape of the MobileNetV2 stack (plane kernels, whole planes and bands), 3 images so
    that the last tile of the small planes is a partial one."""
    rng = np.random.default_rng(layer)
    spec = workloads.cfg1(n=3)[layer]
    q = dict(workloads.FPQ_CFG1)                      # unsigned, n = 8, delta = 2^-3
    _fused_case(oracle, cuda_device, spec, q, False, 2.0 ** -5, rng)
    ops.check_device_flag()


@pytest.mark.parametrize("hw,stride", [(7, 1), (14, 1), (28, 2), (56, 1), (112, 2)])
def test_fused_code8_signed_codes_no_bias_unaligned(oracle, cuda_device, hw, stride):
    rng = np.random.default_rng(hw)
    spec = workloads.LayerSpec("s", 2, 20, hw, hw, 3, stride, 1, dict(workloads.FPQ_CFG0), seed=hw, x_dist="normal")
    q = dict(workloads.FPQ_CFG0)                      # signed, n = 8, delta = 2^-4 -> int8 codes
    _fused_case(oracle, cuda_device, spec, q, True, 2.0 ** -6, rng, bias=False)
    _fused_case(oracle, cuda_device, spec, q, False, 2.0 ** -4, rng, offset=5)
    # input steps that are not powers of two (the output step must be one, the input step need not)
    _fused_case(oracle, cuda_device, spec, q, True, 0.0123, rng)
    _fused_case(oracle, cuda_device, spec, q, False, 0.0371, rng)
    ops.check_device_flag()


def test_fused_code8_other_geometries_run_on_the_generic_kernel(oracle, cuda_device):
    rng = np.random.default_rng(9)
    q = {"kind": "fpq", "sign": False, "n": 6, "delta": 0.25}
    for (h, w, k, stride, pad) in ((15, 9, 3, 1, 1), (20, 20, 5, 2, 2), (30, 30, 3, 1, 0)):
        spec = workloads.LayerSpec("g", 2, 6, h, w, k, stride, pad, q, seed=1)
        _fused_case(oracle, cuda_device, spec, q, False, 2.0 ** -4, rng)
    ops.check_device_flag()


def test_fused_code8_full_batch_sampled(oracle, cuda_device):
    """cfg1's largest layer (96 ch, 112x112, stride 2) at the bench batch of 256 on codes: whole
    images from the start, middle and end against the oracle."""
    rng = np.random.default_rng(21)
    spec = workloads.cfg1()[1]
    d = workloads.make_layer_data(workloads.LayerSpec(spec.name, 1, spec.c, spec.h, spec.w, 3, 2, 1, spec.quant,
                                                      seed=spec.seed, x_dist=spec.x_dist))
    xc = rng.integers(0, 256, (256, spec.c, spec.h, spec.w), dtype=np.uint8)
    t = {k: dev(v, cuda_device) for k, v in d.items() if k != "x"}
    q = dict(workloads.FPQ_CFG1)
    y = ops.fused_dw_bn_quant_code8(dev(xc, cuda_device), 2.0 ** -5, t["w"], t["b"], t["beta"], t["gamma"], t["mean"],
                                    t["var"], 1e-5, pad=(1, 1), stride=(2, 2), quant=q)
    for i in (0, 127, 255):
        x = xc[i:i + 1].astype(np.float32) * np.float32(2.0 ** -5)
        want = oracle.fused_layer(x, d["w"], d["b"], d["beta"], d["gamma"], d["mean"], d["var"], 1e-5, (2, 2), (1, 1),
                                  q, nthreads=oracle.max_threads())
        np.testing.assert_array_equal(y[i:i + 1].cpu().numpy().astype(np.float32) * np.float32(0.125), want)
    ops.check_device_flag()


def test_fused_code8_argument_errors(cuda_device):
    x = torch.zeros((1, 4, 14, 14), dtype=torch.uint8, device=cuda_device)
    w = torch.zeros((4, 3, 3), device=cuda_device)
    v = torch.ones(4, device=cuda_device)
    call = lambda q, delta=0.125: ops.fused_dw_bn_quant_code8(x, delta, w, v, v, v, v, v, pad=(1, 1), quant=q)
    with pytest.raises(L.DwbnqError) as e:
        call({"kind": "fpq", "sign": False, "n": 9, "delta": 0.125})
    assert e.value.status == L.ERR_UNSUPPORTED
    with pytest.raises(L.DwbnqError) as e:
        call({"kind": "fpq", "sign": False, "n": 8, "delta": 0.1})
    assert e.value.status == L.ERR_UNSUPPORTED and "power of two" in str(e.value)
    with pytest.raises(L.DwbnqError) as e:
        call({"kind": "fpq", "sign": False, "n": 8, "delta": 0.125}, delta=0.0)
    assert e.value.status == L.ERR_INVALID_ARG
    with pytest.raises(ValueError):
        call({"kind": "pow2", "sign": True, "with_zero": True, "n": 8, "m": 1})
