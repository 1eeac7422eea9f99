"""dwbnq: B200-native DepthwiseConvolution -> BatchNormalization(inference) -> quantizer path.

Python face of libdwbnq.so for harnesses (tests, bench); the product boundary is the C ABI
in include/dwbnq.h.
"""
from . import _lib
from ._lib import DwbnqError

__all__ = ["_lib", "DwbnqError"]
