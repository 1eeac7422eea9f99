"""ctypes binding of libdwbnq.so (the C ABI declared in include/dwbnq.h).

The library is built in-tree by ``make -C nnabla-ext-cuda_b200`` and loaded from there.
There is no fallback: if the shared object is missing, importing fails.
"""
import ctypes
import os

_PKG_ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
# DWBNQ_LIBRARY selects another build of the same ABI (the bounds-checked libdwbnq_debug.so)
LIB_PATH = os.environ.get("DWBNQ_LIBRARY") or os.path.join(_PKG_ROOT, "libdwbnq.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_DEVICE_FLAG = range(7)
F32, F16 = 0, 1
Q_NONE, Q_FPQ, Q_POW2, Q_MINMAX = 0, 1, 2, 3
PATH_AUTO, PATH_GENERIC, PATH_COOP, PATH_TMA, PATH_RAW, PATH_PLANE, PATH_PLANE_GEN = -1, 0, 1, 2, 3, 4, 5
UNIQUE_ID_BYTES = 128
STATIC_MAX_CHANNELS = 4096


class ConvDesc(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("c", ctypes.c_int32), ("n", ctypes.c_int64),
                ("h", ctypes.c_int32), ("w", ctypes.c_int32), ("kh", ctypes.c_int32),
                ("kw", ctypes.c_int32), ("stride_h", ctypes.c_int32), ("stride_w", ctypes.c_int32),
                ("pad_h", ctypes.c_int32), ("pad_w", ctypes.c_int32), ("dil_h", ctypes.c_int32),
                ("dil_w", ctypes.c_int32), ("multiplier", ctypes.c_int32)]


class QuantDesc(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("sign", ctypes.c_int32), ("n", ctypes.c_int32),
                ("delta", ctypes.c_float), ("with_zero", ctypes.c_int32), ("m", ctypes.c_int32),
                ("decay", ctypes.c_float), ("eps", ctypes.c_float), ("x_min_max", ctypes.c_int32),
                ("ema", ctypes.c_int32)]


class MinMaxPtrs(ctypes.Structure):
    _fields_ = [("qr_min", ctypes.c_void_p), ("qr_max", ctypes.c_void_p),
                ("ql_min", ctypes.c_void_p), ("ql_max", ctypes.c_void_p)]


class PwConvDesc(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("c_in", ctypes.c_int32), ("c_out", ctypes.c_int32),
                ("h", ctypes.c_int32), ("w", ctypes.c_int32), ("n", ctypes.c_int64),
                ("math", ctypes.c_int32), ("act", ctypes.c_int32)]


PW_MATH_FP32, PW_MATH_TF32 = 0, 1
ACT_NONE, ACT_RELU, ACT_RELU6 = 0, 1, 2


class Code8Desc(ctypes.Structure):
    _fields_ = [("in_signed", ctypes.c_int32), ("in_delta", ctypes.c_float)]


ROUND_HALF_AWAY_FROM_ZERO, ROUND_HALF_TO_EVEN = 0, 1


class DwbnqError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("dwbnq status %d: %s" % (status, message))
        self.status = status


_vp, _int, _i64, _flt = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
_P = ctypes.POINTER

# name -> (restype, argtypes); every symbol include/dwbnq.h and include/dwbnq_debug.h declare
SIGNATURES = {
    "dwbnq_version": (_int, []),
    "dwbnq_last_error_string": (ctypes.c_char_p, []),
    "dwbnq_device_count": (_int, []),
    "dwbnq_check_device_flag": (_int, [_int]),
    "dwbnq_conv_out_shape": (_int, [_P(ConvDesc), _P(ctypes.c_int32), _P(ctypes.c_int32)]),
    "dwbnq_fpq_range": (_int, [_int, _int, _flt, _P(_flt), _P(_flt)]),
    "dwbnq_pow2q_range": (_int, [_int, _int, _int, _int, _P(_flt), _P(_flt), _P(_flt)]),
    "dwbnq_pow2q_threshold_table": (_int, [_P(ctypes.c_uint32)]),
    "dwbnq_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int32]),
    "dwbnq_dwconv_fwd": (_int, [_P(ConvDesc), _vp, _vp, _vp, _vp, _int, _vp]),
    "dwbnq_bn_infer_fwd": (_int, [_int, _i64, _i64, _i64, _flt, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "dwbnq_fpq_fwd": (_int, [_int, _i64, _int, _int, _flt, _vp, _vp, _int, _vp]),
    "dwbnq_pow2q_fwd": (_int, [_int, _i64, _int, _int, _int, _int, _vp, _vp, _int, _vp]),
    "dwbnq_minmaxq_fwd": (_int, [_int, _i64, ctypes.c_int32, _i64, _P(QuantDesc), _vp, _P(MinMaxPtrs),
                                 _vp, _vp, _vp, _int, _vp]),
    "dwbnq_minmaxq_fwd_static": (_int, [_int, _i64, ctypes.c_int32, _i64, _P(QuantDesc), _vp, _P(MinMaxPtrs),
                                        _vp, _int, _vp]),
    "dwbnq_fused_fwd": (_int, [_P(ConvDesc), _flt, _P(QuantDesc), _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                               _P(MinMaxPtrs), _vp, _vp, _vp, _int, _vp]),
    "dwbnq_fpq_bwd": (_int, [_int, _i64, _int, _int, _flt, _int, _int, _vp, _vp, _vp, _int, _vp]),
    "dwbnq_pow2q_bwd": (_int, [_int, _i64, _int, _int, _int, _int, _int, _int, _vp, _vp, _vp, _int, _vp]),
    "dwbnq_dwconv_bwd": (_int, [_P(ConvDesc), _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _vp]),
    "dwbnq_quantize_linear_code8_fwd": (_int, [_int, _i64, _flt, _int, _int, _int, _int, _vp, _vp, _int, _vp]),
    "dwbnq_dequantize_linear_code8_fwd": (_int, [_int, _i64, _flt, _int, _int, _vp, _vp, _int, _vp]),
    "dwbnq_fused_fwd_code8": (_int, [_P(ConvDesc), _flt, _P(QuantDesc), _P(Code8Desc), _vp, _vp, _vp, _vp, _vp,
                                     _vp, _vp, _vp, _int, _vp]),
    "dwbnq_pwconv_workspace_bytes": (ctypes.c_size_t, [_P(PwConvDesc)]),
    "dwbnq_pwconv_fwd": (_int, [_P(PwConvDesc), _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "dwbnq_pwconv_fused_fwd": (_int, [_P(PwConvDesc), _flt, _P(QuantDesc), _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                      _int, _vp]),
    "dwbnq_pwconv_prepare": (_int, [_P(PwConvDesc), _flt, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "dwbnq_pwconv_fused_fwd_prepared": (_int, [_P(PwConvDesc), _P(QuantDesc), _int, _vp, _vp, _vp, _int, _vp]),
    "dwbnq_pwconv_plan": (_int, [_P(PwConvDesc), _vp, _vp, _P(_int)]),
    "dwbnq_set_forced_pw_path": (_int, [_int]),
    "dwbnq_set_pw_max_ctas": (_int, [_int]),
    "dwbnq_debug_pwconv_tiling": (_int, [ctypes.POINTER(PwConvDesc), _vp, _int, ctypes.POINTER(_int)]),
    "dwbnq_fused_plan": (_int, [_P(ConvDesc), _vp, _vp, _P(_int), _P(_int), _P(_int), _P(_int),
                                _P(_i64), _P(_int)]),
    "dwbnq_set_forced_path": (_int, [_int]),
    "dwbnq_set_tuning": (_int, [_int, _int, _int, _int]),
    "dwbnq_comm_get_unique_id": (_int, [_vp]),
    "dwbnq_comm_create": (_int, [_vp, _int, _int, _int, _P(_vp)]),
    "dwbnq_comm_destroy": (_int, [_vp]),
    "dwbnq_comm_set_deadline_ms": (_int, [_vp, _int]),
    "dwbnq_debug_expire_wait": (_int, [ctypes.c_uint, _int, _vp]),
    "dwbnq_comm_allreduce_max_f32": (_int, [_vp, _vp, _i64, _vp, _int]),
}

_lib = None


def lib():
    """The loaded library with argtypes set. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s not found: build it with `make -C %s` (there is no CPU fallback)"
                              % (LIB_PATH, _PKG_ROOT))
        l = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(status):
    if status != OK:
        raise DwbnqError(status, lib().dwbnq_last_error_string().decode("utf-8", "replace"))
