"""The five operators of the path and the fused layer, on torch CUDA tensors.

Names, argument order and argument meaning follow nnabla's functional API
(``F.depthwise_convolution``, ``F.batch_normalization``, ``F.fixed_point_quantize``,
``F.pow2_quantize``, ``F.min_max_quantize``), which is what resolves to the ``*Cuda``
classes of nnabla-ext-cuda under ``get_extension_context('cuda')``. torch is used only
for device memory and streams; every computation is a call into libdwbnq through the
C ABI with raw device pointers.
"""
import ctypes

import torch

from . import _lib as L


def _dtype_code(t):
    if t.dtype == torch.float32:
        return L.F32
    if t.dtype == torch.float16:
        return L.F16
    raise TypeError("dwbnq supports float32 and float16 tensors, got %s" % t.dtype)


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _chk_cuda(*ts):
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("dwbnq operators take CUDA tensors (there is no CPU fallback)")
        if not t.is_contiguous():
            raise ValueError("dwbnq operators take contiguous tensors")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("all tensors must live on one device")
    return dev


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _pair(v, ndim=2):
    if isinstance(v, int):
        return (v,) * ndim
    v = tuple(int(a) for a in v)
    return v


class _ShapeOf:
    """What conv_desc reads of a tensor: its shape and element type."""

    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), dtype

    def dim(self):
        return len(self.shape)


def conv_desc(x, w, base_axis=1, pad=None, stride=None, dilation=None, multiplier=1):
    """dwbnq_conv_desc for x [..., C, (H,) W] and w [C*mult, (kh,) kw]."""
    sdims = x.dim() - base_axis - 1
    if sdims not in (1, 2):
        raise ValueError("depthwise_convolution supports 1-D and 2-D convolutions")
    if w.dim() != sdims + 1:
        raise ValueError("weight rank %d does not match %d spatial dims" % (w.dim(), sdims))
    pad = _pair(0 if pad is None else pad, sdims)
    stride = _pair(1 if stride is None else stride, sdims)
    dilation = _pair(1 if dilation is None else dilation, sdims)
    n = 1
    for s in x.shape[:base_axis]:
        n *= int(s)
    c = int(x.shape[base_axis])
    if int(w.shape[0]) != c * multiplier:
        raise ValueError("weight has %d output maps, expected C*multiplier = %d" % (w.shape[0], c * multiplier))
    if sdims == 2:
        h, wd = int(x.shape[-2]), int(x.shape[-1])
        kh, kw = int(w.shape[1]), int(w.shape[2])
        (ph, pw), (sh, sw), (dh, dw) = pad, stride, dilation
    else:
        h, wd = 1, int(x.shape[-1])
        kh, kw = 1, int(w.shape[1])
        ph, sh, dh = 0, 1, 1
        pw, sw, dw = pad[0], stride[0], dilation[0]
    d = L.ConvDesc(dtype=_dtype_code(x), c=c, n=n, h=h, w=wd, kh=kh, kw=kw, stride_h=sh, stride_w=sw,
                   pad_h=ph, pad_w=pw, dil_h=dh, dil_w=dw, multiplier=multiplier)
    ho, wo = ctypes.c_int32(), ctypes.c_int32()
    L.check(L.lib().dwbnq_conv_out_shape(ctypes.byref(d), ctypes.byref(ho), ctypes.byref(wo)))
    oshape = tuple(x.shape[:base_axis]) + (c * multiplier,) + ((ho.value, wo.value) if sdims == 2 else (wo.value,))
    return d, oshape


def depthwise_convolution(x, w, b=None, base_axis=1, pad=None, stride=None, dilation=None,
                          multiplier=1, out=None):
    dev = _chk_cuda(x, w, b, out)
    d, oshape = conv_desc(x, w, base_axis, pad, stride, dilation, multiplier)
    y = out if out is not None else torch.empty(oshape, dtype=x.dtype, device=dev)
    L.check(L.lib().dwbnq_dwconv_fwd(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(b), _ptr(y), dev.index,
                                     _stream(dev)))
    return y


def _bn_view(x, axes):
    if len(axes) != 1:
        raise ValueError("batch_normalization: exactly one channel axis is supported")
    ax = axes[0] % x.dim()
    size0 = 1
    for s in x.shape[:ax]:
        size0 *= int(s)
    size2 = 1
    for s in x.shape[ax + 1:]:
        size2 *= int(s)
    return size0, int(x.shape[ax]), size2


def batch_normalization(x, beta, gamma, mean, variance, axes=(1,), decay_rate=0.9, eps=1e-5,
                        batch_stat=False, out=None):
    """Inference mode only (batch_stat=False): the training path is outside this library."""
    if batch_stat:
        raise NotImplementedError("dwbnq implements BatchNormalization with batch_stat=False only")
    dev = _chk_cuda(x, beta, gamma, mean, variance, out)
    size0, size1, size2 = _bn_view(x, list(axes))
    y = out if out is not None else torch.empty_like(x)
    L.check(L.lib().dwbnq_bn_infer_fwd(_dtype_code(x), size0, size1, size2, float(eps), _ptr(x), _ptr(beta),
                                       _ptr(gamma), _ptr(mean), _ptr(variance), _ptr(y), dev.index,
                                       _stream(dev)))
    return y


def fixed_point_quantize(x, sign=True, n=8, delta=2.0 ** -4, ste_fine_grained=True, out=None):
    dev = _chk_cuda(x, out)
    y = out if out is not None else torch.empty_like(x)
    L.check(L.lib().dwbnq_fpq_fwd(_dtype_code(x), x.numel(), int(sign), int(n), float(delta), _ptr(x),
                                  _ptr(y), dev.index, _stream(dev)))
    return y


def pow2_quantize(x, sign=True, with_zero=True, n=8, m=1, ste_fine_grained=True, out=None):
    dev = _chk_cuda(x, out)
    y = out if out is not None else torch.empty_like(x)
    L.check(L.lib().dwbnq_pow2q_fwd(_dtype_code(x), x.numel(), int(sign), int(with_zero), int(n), int(m),
                                    _ptr(x), _ptr(y), dev.index, _stream(dev)))
    return y


def workspace(channels, device):
    """Scratch for the MinMaxQuantize entry points (torch's allocator returns 512-byte aligned blocks)."""
    nbytes = int(L.lib().dwbnq_workspace_bytes(int(channels)))
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def _mm_args(x, qr_min, qr_max, ql_min, ql_max, channels):
    for t in (qr_min, qr_max, ql_min, ql_max):
        if t.numel() != channels or t.dtype != x.dtype:
            raise ValueError("MinMaxQuantize ranges must hold one %s value per channel (%d)" % (x.dtype, channels))
    return L.MinMaxPtrs(qr_min.data_ptr(), qr_max.data_ptr(), ql_min.data_ptr(), ql_max.data_ptr())


def min_max_quantize(x, qr_min, qr_max, ql_min, ql_max, decay=0.999, x_min_max=False, ema=False,
                     ste_fine_grained=True, eps=0.01, axis=1, comm=None, ws=None, out=None):
    """Per-channel MinMaxQuantize: ranges of shape [1, C, 1, 1] along ``axis``. qr_min and
    qr_max are updated in place when x_min_max is set. ``comm`` (a dwbnq.comm.Communicator)
    all-reduces the per-channel min/max across the ranks that share a sharded batch."""
    dev = _chk_cuda(x, qr_min, qr_max, ql_min, ql_max, out)
    size0, c, size2 = _bn_view(x, [axis])
    mm = _mm_args(x, qr_min, qr_max, ql_min, ql_max, c)
    q = L.QuantDesc(kind=L.Q_MINMAX, decay=float(decay), eps=float(eps), x_min_max=int(x_min_max), ema=int(ema))
    ws = ws if ws is not None else workspace(c, dev)
    y = out if out is not None else torch.empty_like(x)
    L.check(L.lib().dwbnq_minmaxq_fwd(_dtype_code(x), size0, c, size2, ctypes.byref(q), _ptr(x),
                                      ctypes.byref(mm), _ptr(y), _ptr(ws),
                                      None if comm is None else comm.handle, dev.index, _stream(dev)))
    return y


def quant_desc(quant):
    """dict {"kind": "none"|"fpq"|"pow2"|"minmax", ...} -> QuantDesc."""
    kind = quant["kind"] if quant else "none"
    if kind == "none":
        return L.QuantDesc(kind=L.Q_NONE)
    if kind == "fpq":
        return L.QuantDesc(kind=L.Q_FPQ, sign=int(quant["sign"]), n=int(quant["n"]), delta=float(quant["delta"]))
    if kind == "pow2":
        return L.QuantDesc(kind=L.Q_POW2, sign=int(quant["sign"]), with_zero=int(quant["with_zero"]),
                           n=int(quant["n"]), m=int(quant["m"]))
    if kind == "minmax":
        return L.QuantDesc(kind=L.Q_MINMAX, decay=float(quant.get("decay", 0.999)),
                           eps=float(quant.get("eps", 0.01)), x_min_max=int(quant.get("x_min_max", True)),
                           ema=int(quant.get("ema", False)))
    raise ValueError("unknown quantizer kind %r" % (kind,))


def fused_dw_bn_quant(x, w, b, beta, gamma, mean, variance, eps=1e-5, pad=None, stride=None,
                      dilation=None, multiplier=1, quant=None, base_axis=1, comm=None, ws=None, out=None):
    """The layer the graph pass produces: quantizer(BN_inference(depthwise_convolution(x))).

    ``mean is None`` skips BatchNormalization. For kind "minmax" the dict also carries the
    tensors qr_min, qr_max, ql_min, ql_max (qr_* updated in place when x_min_max)."""
    mmt = [quant[k] for k in ("qr_min", "qr_max", "ql_min", "ql_max")] if quant and quant["kind"] == "minmax" else []
    dev = _chk_cuda(x, w, b, beta, gamma, mean, variance, out, *mmt)
    d, oshape = conv_desc(x, w, base_axis, pad, stride, dilation, multiplier)
    q = quant_desc(quant)
    y = out if out is not None else torch.empty(oshape, dtype=x.dtype, device=dev)
    mm = None
    if mmt:
        oc = int(w.shape[0])
        mm = ctypes.byref(_mm_args(x, mmt[0], mmt[1], mmt[2], mmt[3], oc))
        ws = ws if ws is not None else workspace(oc, dev)
    L.check(L.lib().dwbnq_fused_fwd(ctypes.byref(d), float(eps), ctypes.byref(q), _ptr(x), _ptr(w), _ptr(b),
                                    _ptr(beta), _ptr(gamma), _ptr(mean), _ptr(variance), mm, _ptr(y),
                                    _ptr(ws) if mmt else None, None if comm is None else comm.handle,
                                    dev.index, _stream(dev)))
    return y


# ---- training side -------------------------------------------------------------------------------

def fixed_point_quantize_backward(dy, x=None, sign=True, n=8, delta=2.0 ** -4, ste_fine_grained=True, dx=None,
                                  accum=False):
    """STE backward of fixed_point_quantize: returns dx (``dx`` given and ``accum``: added onto)."""
    dev = _chk_cuda(dy, x, dx)
    out = dx if dx is not None else torch.empty_like(dy)
    L.check(L.lib().dwbnq_fpq_bwd(_dtype_code(dy), dy.numel(), int(sign), int(n), float(delta), int(ste_fine_grained),
                                  int(accum), _ptr(x), _ptr(dy), _ptr(out), dev.index, _stream(dev)))
    return out


def pow2_quantize_backward(dy, x=None, sign=True, with_zero=True, n=8, m=1, ste_fine_grained=True, dx=None,
                           accum=False):
    """STE backward of pow2_quantize."""
    dev = _chk_cuda(dy, x, dx)
    out = dx if dx is not None else torch.empty_like(dy)
    L.check(L.lib().dwbnq_pow2q_bwd(_dtype_code(dy), dy.numel(), int(sign), int(with_zero), int(n), int(m),
                                    int(ste_fine_grained), int(accum), _ptr(x), _ptr(dy), _ptr(out), dev.index,
                                    _stream(dev)))
    return out


def depthwise_convolution_backward(x, w, dy, base_axis=1, pad=None, stride=None, dilation=None, multiplier=1,
                                   dx=None, dw=None, db=None, need=(True, True, True), accum=(False, False, False)):
    """Gradients of depthwise_convolution: returns (dx, dw, db), None where ``need`` is False
    (propagate_down); ``accum[i]`` adds onto the given tensor instead of overwriting it."""
    dev = _chk_cuda(x, w, dy, dx, dw, db)
    d, oshape = conv_desc(x, w, base_axis, pad, stride, dilation, multiplier)
    if tuple(dy.shape) != tuple(oshape):
        raise ValueError("dy has shape %s, the convolution's output is %s" % (tuple(dy.shape), tuple(oshape)))
    dx = (dx if dx is not None else torch.empty_like(x)) if need[0] else None
    dw = (dw if dw is not None else torch.empty_like(w)) if need[1] else None
    db = (db if db is not None else torch.empty(w.shape[0], dtype=w.dtype, device=dev)) if need[2] else None
    mask = (1 if accum[0] else 0) | (2 if accum[1] else 0) | (4 if accum[2] else 0)
    L.check(L.lib().dwbnq_dwconv_bwd(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(dy), _ptr(dx), _ptr(dw), _ptr(db), mask,
                                     dev.index, _stream(dev)))
    return dx, dw, db


# ---- 8-bit storage of quantized activations -------------------------------------------------

def quantize_linear_code8(x, scale, zero_point=0, round_mode="HALF_AWAY_FROM_ZERO", signed=False,
                          min_range=None, max_range=None, out=None):
    """QuantizeLinear (scalar scale / zero point) with the result stored as int8 / uint8 codes:
    saturate(round(x / scale + zero_point)). The argument names are nnabla's
    ``F.quantize_linear``; ``signed`` picks the narrow type, the range defaults to all of it."""
    dev = _chk_cuda(x, out)
    lo = (-128 if signed else 0) if min_range is None else int(min_range)
    hi = (127 if signed else 255) if max_range is None else int(max_range)
    mode = {"HALF_AWAY_FROM_ZERO": L.ROUND_HALF_AWAY_FROM_ZERO, "HALF_TO_EVEN": L.ROUND_HALF_TO_EVEN}[round_mode]
    y = out if out is not None else torch.empty(x.shape, dtype=torch.int8 if lo < 0 else torch.uint8, device=dev)
    L.check(L.lib().dwbnq_quantize_linear_code8_fwd(_dtype_code(x), x.numel(), float(scale), int(zero_point), mode,
                                                    lo, hi, _ptr(x), _ptr(y), dev.index, _stream(dev)))
    return y


def dequantize_linear_code8(codes, scale, zero_point=0, dtype=torch.float32, out=None):
    """DequantizeLinear from int8 / uint8 codes: (code - zero_point) * scale."""
    dev = _chk_cuda(codes, out)
    if codes.dtype not in (torch.int8, torch.uint8):
        raise TypeError("codes must be int8 or uint8")
    y = out if out is not None else torch.empty(codes.shape, dtype=dtype, device=dev)
    L.check(L.lib().dwbnq_dequantize_linear_code8_fwd(_dtype_code(y), codes.numel(), float(scale), int(zero_point),
                                                      int(codes.dtype == torch.int8), _ptr(codes), _ptr(y), dev.index,
                                                      _stream(dev)))
    return y


def fused_dw_bn_quant_code8(x_codes, in_delta, w, b, beta, gamma, mean, variance, eps=1e-5, pad=None, stride=None,
                            dilation=None, multiplier=1, quant=None, base_axis=1, out=None):
    """The fused layer on 8-bit codes: x_codes (int8 / uint8) stands for x = code * in_delta,
    the result is the code of FixedPointQuantize(BN(conv(x))), int8 when the quantizer is
    signed, else uint8. ``quant`` is a FixedPointQuantize dict with n <= 8 and a power-of-two
    delta; w, b and the BN vectors are float32."""
    if x_codes.dtype not in (torch.int8, torch.uint8):
        raise TypeError("x_codes must be int8 or uint8")
    if not quant or quant["kind"] != "fpq":
        raise ValueError("8-bit storage needs a FixedPointQuantize quantizer")
    dev = _chk_cuda(x_codes, w, b, beta, gamma, mean, variance, out)
    # geometry from the code tensor's shape, parameter dtype from w
    d, oshape = conv_desc(_ShapeOf(x_codes.shape, w.dtype), w, base_axis, pad, stride, dilation, multiplier)
    q = quant_desc(quant)
    io = L.Code8Desc(in_signed=int(x_codes.dtype == torch.int8), in_delta=float(in_delta))
    ydt = torch.int8 if quant["sign"] else torch.uint8
    y = out if out is not None else torch.empty(oshape, dtype=ydt, device=dev)
    if y.dtype != ydt:
        raise TypeError("out must be %s for this quantizer" % ydt)
    L.check(L.lib().dwbnq_fused_fwd_code8(ctypes.byref(d), float(eps), ctypes.byref(q), ctypes.byref(io), _ptr(x_codes),
                                          _ptr(w), _ptr(b), _ptr(beta), _ptr(gamma), _ptr(mean), _ptr(variance),
                                          _ptr(y), dev.index, _stream(dev)))
    return y


_ACTS = {None: L.ACT_NONE, "none": L.ACT_NONE, "relu": L.ACT_RELU, "relu6": L.ACT_RELU6}
_MATHS = {"fp32": L.PW_MATH_FP32, "tf32": L.PW_MATH_TF32}


def pwconv_desc(x, w, base_axis=1, math="fp32", act=None):
    """PwConvDesc for x [..., c_in, h, w] and a Convolution weight w [c_out, c_in, 1, 1] (or [c_out, c_in])."""
    if x.dim() != base_axis + 3:
        raise ValueError("pointwise convolution takes [..., c_in, h, w]")
    if w.dim() not in (2, 4) or (w.dim() == 4 and tuple(w.shape[2:]) != (1, 1)) or w.shape[1] != x.shape[base_axis]:
        raise ValueError("weight %s is not a 1x1 kernel over %d input channels" % (tuple(w.shape), x.shape[base_axis]))
    if x.dtype != w.dtype:
        raise TypeError("x and w must have one dtype")
    n = 1
    for s in x.shape[:base_axis]:
        n *= int(s)
    d = L.PwConvDesc(dtype=_dtype_code(x), c_in=int(w.shape[1]), c_out=int(w.shape[0]), h=int(x.shape[base_axis + 1]),
                     w=int(x.shape[base_axis + 2]), n=n, math=_MATHS[math], act=_ACTS[act])
    return d, tuple(x.shape[:base_axis]) + (int(w.shape[0]),) + tuple(x.shape[base_axis + 1:])


def pwconv_workspace(x, w, base_axis=1):
    """A workspace tensor of the size the pointwise entry points ask for."""
    d, _ = pwconv_desc(x, w, base_axis)
    nbytes = int(L.lib().dwbnq_pwconv_workspace_bytes(ctypes.byref(d)))
    return torch.empty(nbytes, dtype=torch.uint8, device=w.device)


def pointwise_convolution(x, w, b=None, base_axis=1, math="fp32", ws=None, out=None):
    """Convolution with a 1x1 kernel (pad 0, stride 1, dilation 1, group 1): y = w * x + b."""
    dev = _chk_cuda(x, w, b, out, ws)
    d, oshape = pwconv_desc(x, w, base_axis, math)
    ws = ws if ws is not None else pwconv_workspace(x, w, base_axis)
    y = out if out is not None else torch.empty(oshape, dtype=x.dtype, device=dev)
    L.check(L.lib().dwbnq_pwconv_fwd(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(b), _ptr(y), _ptr(ws), dev.index, _stream(dev)))
    return y


def fused_pw_bn_quant(x, w, b, beta, gamma, mean, variance, eps=1e-5, quant=None, act=None, base_axis=1, math="fp32",
                      ws=None, out=None):
    """quantizer(act(BN_inference(pointwise_convolution(x)))) in one kernel. ``mean is None`` skips
    BatchNormalization; ``act`` is None, "relu" or "relu6"; ``quant`` a "fpq" / "pow2" dict or None."""
    dev = _chk_cuda(x, w, b, beta, gamma, mean, variance, out, ws)
    d, oshape = pwconv_desc(x, w, base_axis, math, act)
    q = quant_desc(quant)
    ws = ws if ws is not None else pwconv_workspace(x, w, base_axis)
    y = out if out is not None else torch.empty(oshape, dtype=x.dtype, device=dev)
    L.check(L.lib().dwbnq_pwconv_fused_fwd(ctypes.byref(d), float(eps), ctypes.byref(q), _ptr(x), _ptr(w), _ptr(b), _ptr(beta),
                                           _ptr(gamma), _ptr(mean), _ptr(variance), _ptr(y), _ptr(ws), dev.index,
                                           _stream(dev)))
    return y


def pwconv_prepare(x, w, b, beta, gamma, mean, variance, eps=1e-5, act=None, base_axis=1, math="fp32", ws=None):
    """One-time part of fused_pw_bn_quant for parameters that do not change between calls: fills
    (and returns) the workspace; ``x`` only gives the shape."""
    dev = _chk_cuda(w, b, beta, gamma, mean, variance, ws)
    d, _ = pwconv_desc(x, w, base_axis, math, act)
    ws = ws if ws is not None else pwconv_workspace(x, w, base_axis)
    L.check(L.lib().dwbnq_pwconv_prepare(ctypes.byref(d), float(eps), _ptr(w), _ptr(b), _ptr(beta), _ptr(gamma), _ptr(mean),
                                         _ptr(variance), _ptr(ws), dev.index, _stream(dev)))
    return ws


def fused_pw_bn_quant_prepared(x, w_shape_like, ws, has_bn=True, quant=None, act=None, base_axis=1, math="fp32", out=None):
    """The per-call part: one kernel launch on a workspace ``pwconv_prepare`` filled with the same
    ``act`` and ``math``. ``w_shape_like`` is the weight (or anything with its shape and dtype)."""
    dev = _chk_cuda(x, ws, out)
    d, oshape = pwconv_desc(x, w_shape_like, base_axis, math, act)
    q = quant_desc(quant)
    y = out if out is not None else torch.empty(oshape, dtype=x.dtype, device=dev)
    L.check(L.lib().dwbnq_pwconv_fused_fwd_prepared(ctypes.byref(d), ctypes.byref(q), int(bool(has_bn)), _ptr(x), _ptr(y),
                                                    _ptr(ws), dev.index, _stream(dev)))
    return y


def pwconv_plan(x, w, base_axis=1, math="fp32"):
    """1 when the tcgen05 kernel takes this call, 0 for the plain FMA kernel (diagnostic)."""
    d, _ = pwconv_desc(x, w, base_axis, math)
    path = ctypes.c_int()
    L.check(L.lib().dwbnq_pwconv_plan(ctypes.byref(d), _ptr(x), _ptr(w), ctypes.byref(path)))
    return path.value


def pwconv_tiling(desc, x_address=4096, sms=148):
    """Launch shape of the tcgen05 pointwise kernel for a PwConvDesc (host only, diagnostic)."""
    out = (ctypes.c_int * 8)()
    L.check(L.lib().dwbnq_debug_pwconv_tiling(ctypes.byref(desc), ctypes.c_void_p(x_address), int(sms), out))
    keys = ("columns", "channel_tiles", "x_path", "tiles", "ctas", "stages", "accumulators", "shared_columns")
    return dict(zip(keys, list(out)))


def set_forced_pw_path(path):
    L.check(L.lib().dwbnq_set_forced_pw_path(int(path)))


def set_pw_max_ctas(ctas):
    L.check(L.lib().dwbnq_set_pw_max_ctas(int(ctas)))


def fused_plan(x, w, y=None, base_axis=1, pad=None, stride=None, dilation=None, multiplier=1):
    """Kernel family and tile geometry the library would choose (diagnostic)."""
    d, _ = conv_desc(x, w, base_axis, pad, stride, dilation, multiplier)
    path, p, th, thr, smem = (ctypes.c_int() for _ in range(5))
    ctas = ctypes.c_int64()
    L.check(L.lib().dwbnq_fused_plan(ctypes.byref(d), _ptr(x), _ptr(y if y is not None else x), ctypes.byref(path),
                                     ctypes.byref(p), ctypes.byref(th), ctypes.byref(thr), ctypes.byref(ctas),
                                     ctypes.byref(smem)))
    return {"path": path.value, "planes_per_cta": p.value, "rows_per_tile": th.value, "threads": thr.value,
            "ctas": ctas.value, "smem_bytes": smem.value}


def set_forced_path(path):
    L.check(L.lib().dwbnq_set_forced_path(int(path)))


def set_tuning(planes_per_cta=0, row_blocks_per_tile=0, threads=0, rows_per_patch=0):
    L.check(L.lib().dwbnq_set_tuning(int(planes_per_cta), int(row_blocks_per_tile), int(threads),
                                     int(rows_per_patch)))


def check_device_flag(device=-1):
    L.check(L.lib().dwbnq_check_device_flag(int(device)))
