"""deep8_b200: B200 (sm_100a) kernels for the dense-contraction path of Deep8 (MatrixMultiply, Conv2d, DeConv2d,
forward and gradients) behind a C ABI (include/d8k.h).  This Python package is a thin ctypes front-end over that ABI,
used by the tests and the benchmark; device memory comes from torch tensors."""
from . import _lib
from ._lib import F16, F32, D8kError
from .ops import Context

__all__ = ["Context", "F16", "F32", "D8kError"]
