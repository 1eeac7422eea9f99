"""ctypes/numpy front end of the CPU oracle (``dwbnq_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by
the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` as the checker and the
timed CPU baseline. The product (the CUDA library and its host layer) never imports it.

PARITY UNPINNED: nnabla core, which owns the CPU classes these functions restate, is
not installed here, so no reference-generated vector exists; see the header of
``dwbnq_oracle.cpp``. ``tests/golden/known_answers.json`` holds the known answers
derived by hand from the nnabla-ext-cuda sources.

fp16 convention used by every ``*_f16`` helper: inputs are fp16 values, arithmetic is
the fp32 restatement on the up-cast values, and the result is rounded to fp16 once
(the product's half kernels keep fp32 accumulators; the reference's per-op half
rounding, include/nbla/cuda/half.hpp:159-193, is deliberately not reproduced).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libdwbnq_oracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_i64 = ctypes.c_int64
_int = ctypes.c_int
_flt = ctypes.c_float


def build(force=False):
    """Compile the oracle with the Makefile beside it."""
    if force or not os.path.exists(_LIB_PATH) or (
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "dwbnq_oracle.cpp"))):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libdwbnq_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_max_threads.restype = _int
    return _lib


def max_threads():
    return int(lib().oracle_max_threads())


def _p(a):
    return None if a is None else a.ctypes.data_as(_f32p)


def _c32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def conv_out_size(size, k, s, p, d=1):
    return (size + 2 * p - d * (k - 1) - 1) // s + 1


def dwconv(x, w, b, stride=(1, 1), pad=(0, 0), dilation=(1, 1), multiplier=1, nthreads=1):
    """x [N,C,H,W] fp32, w [C*mult,kh,kw], b [C*mult] or None -> y [N,C*mult,Ho,Wo]."""
    x, w, b = _c32(x), _c32(w), _c32(b)
    N, C, H, W = x.shape
    OC, kh, kw = w.shape
    assert OC == C * multiplier
    Ho = conv_out_size(H, kh, stride[0], pad[0], dilation[0])
    Wo = conv_out_size(W, kw, stride[1], pad[1], dilation[1])
    y = np.empty((N, OC, Ho, Wo), dtype=np.float32)
    lib().oracle_dwconv_f32(_p(x), _p(w), _p(b), _p(y), _i64(N), _int(C), _int(H), _int(W),
                            _int(kh), _int(kw), _int(stride[0]), _int(stride[1]),
                            _int(pad[0]), _int(pad[1]), _int(dilation[0]), _int(dilation[1]),
                            _int(multiplier), _int(nthreads))
    return y


def bn_infer(x, beta, gamma, mean, var, eps=1e-5, axis=1, nthreads=1):
    """BatchNormalization with batch_stat=False over ``axis``; beta/gamma may be None."""
    x = _c32(x)
    size0 = int(np.prod(x.shape[:axis], dtype=np.int64))
    size1 = x.shape[axis]
    size2 = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    beta, gamma, mean, var = (_c32(None if a is None else np.reshape(a, -1))
                              for a in (beta, gamma, mean, var))
    y = np.empty_like(x)
    lib().oracle_bn_infer_f32(_p(x), _p(beta), _p(gamma), _p(mean), _p(var), _p(y),
                              _i64(size0), _i64(size1), _i64(size2), _flt(eps), _int(nthreads))
    return y


def fpq_params(sign, n, delta):
    mx, mn = _flt(), _flt()
    lib().oracle_fpq_params(_int(sign), _int(n), _flt(delta), ctypes.byref(mx), ctypes.byref(mn))
    return mx.value, mn.value


def fpq(x, sign=True, n=8, delta=2.0 ** -4, nthreads=1):
    x = _c32(x)
    y = np.empty_like(x)
    lib().oracle_fpq_f32(_p(x), _p(y), _i64(x.size), _int(sign), _int(n), _flt(delta),
                         _int(nthreads))
    return y


def pow2q_params(sign, with_zero, n, m):
    a, b, c = _flt(), _flt(), _flt()
    lib().oracle_pow2q_params(_int(sign), _int(with_zero), _int(n), _int(m), ctypes.byref(a),
                              ctypes.byref(b), ctypes.byref(c))
    return a.value, b.value, c.value


def pow2q(x, sign=True, with_zero=True, n=8, m=1, nthreads=1):
    x = _c32(x)
    y = np.empty_like(x)
    lib().oracle_pow2q_f32(_p(x), _p(y), _i64(x.size), _int(sign), _int(with_zero), _int(n),
                           _int(m), _int(nthreads))
    return y


def round_log2(x, nthreads=1):
    x = _c32(x)
    k = np.empty_like(x)
    lib().oracle_round_log2(_p(x), _p(k), _i64(x.size), _int(nthreads))
    return k


def minmax_reduce(x, axis=1, nthreads=1):
    """Per-channel (min, max) of x over every axis but ``axis``."""
    x = _c32(x)
    size0 = int(np.prod(x.shape[:axis], dtype=np.int64))
    C = x.shape[axis]
    size2 = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    mn = np.empty(C, np.float32)
    mx = np.empty(C, np.float32)
    lib().oracle_minmax_reduce_f32(_p(x), _p(mn), _p(mx), _i64(size0), _int(C), _i64(size2),
                                   _int(nthreads))
    return mn, mx


def minmaxq(x, qr_min, qr_max, ql_min, ql_max, decay=0.999, x_min_max=True, ema=False,
            eps=0.01, axis=1, nthreads=1, return_ranges=False):
    """MinMaxQuantize forward with per-channel ranges along ``axis``.

    Returns (y, qr_min_new, qr_max_new); the inputs are not modified. With
    ``return_ranges`` also (scale, m_nudged, M_nudged).
    """
    x = _c32(x)
    size0 = int(np.prod(x.shape[:axis], dtype=np.int64))
    C = x.shape[axis]
    size2 = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    qr_min = np.array(np.reshape(qr_min, -1), dtype=np.float32)
    qr_max = np.array(np.reshape(qr_max, -1), dtype=np.float32)
    ql_min = _c32(np.reshape(ql_min, -1))
    ql_max = _c32(np.reshape(ql_max, -1))
    assert qr_min.size == C and qr_max.size == C and ql_min.size == C and ql_max.size == C
    y = np.empty_like(x)
    sc = np.empty(C, np.float32)
    lo = np.empty(C, np.float32)
    hi = np.empty(C, np.float32)
    lib().oracle_minmaxq_f32(_p(x), _p(qr_min), _p(qr_max), _p(ql_min), _p(ql_max), _p(y),
                             _i64(size0), _int(C), _i64(size2), _flt(decay), _int(x_min_max),
                             _int(ema), _flt(eps), _p(sc), _p(lo), _p(hi), _int(nthreads))
    if return_ranges:
        return y, qr_min, qr_max, sc, lo, hi
    return y, qr_min, qr_max


def minmaxq_from_ranges(x, qr_min, qr_max, ql_min, ql_max, eps=0.01, axis=1, nthreads=1):
    """The quantize step alone for given (already reduced) ranges: what every shard of a
    batch-sharded MinMaxQuantize applies after the min/max exchange."""
    return minmaxq(x, qr_min, qr_max, ql_min, ql_max, x_min_max=False, ema=False, eps=eps,
                   axis=axis, nthreads=nthreads)


def fused_layer(x, w, b, beta, gamma, mean, var, eps, stride, pad, quant, dilation=(1, 1),
                multiplier=1, nthreads=1, return_prequant=False):
    """The unfused three-function chain dw-conv -> BN(inference) -> quantizer, which is
    what the reference executes. ``quant`` is a dict: {"kind": "none"|"fpq"|"pow2"|"minmax", ...}.
    For "minmax" returns (y, qr_min, qr_max)."""
    y = dwconv(x, w, b, stride, pad, dilation, multiplier, nthreads)
    y = bn_infer(y, beta, gamma, mean, var, eps, 1, nthreads)
    pre = y
    kind = quant["kind"]
    if kind == "none":
        out = y
    elif kind == "fpq":
        out = fpq(y, quant["sign"], quant["n"], quant["delta"], nthreads)
    elif kind == "pow2":
        out = pow2q(y, quant["sign"], quant["with_zero"], quant["n"], quant["m"], nthreads)
    elif kind == "minmax":
        out = minmaxq(y, quant["qr_min"], quant["qr_max"], quant["ql_min"], quant["ql_max"],
                      quant.get("decay", 0.999), quant.get("x_min_max", True),
                      quant.get("ema", False), quant.get("eps", 0.01), 1, nthreads)
    else:
        raise ValueError(kind)
    if return_prequant:
        return out, pre
    return out


def to_f16_result(y32):
    """Round an fp32 oracle result to fp16 once (the fp16 convention in the module doc)."""
    return np.asarray(y32, dtype=np.float32).astype(np.float16)
