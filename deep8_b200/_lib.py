"""ctypes binding of libdeep8_b200.so (the C ABI declared in include/d8k.h).

The library is the product; there is no fallback.  Loading fails loudly when the shared object is missing, and every
call raises when the library reports an error.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# D8K_LIB_PATH selects another build of the same library (A/B measurements); there is still no fallback.
LIB_PATH = os.environ.get("D8K_LIB_PATH") or os.path.join(_HERE, "libdeep8_b200.so")

F16, F32 = 0, 1

_vp, _i, _ll, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/d8k.h one to one
SIGNATURES = {
    "d8k_ctx_create": (_i, [_i, _sz, ctypes.POINTER(_vp)]),
    "d8k_ctx_destroy": (_i, [_vp]),
    "d8k_ctx_set_stream": (_i, [_vp, _vp]),
    "d8k_ctx_status": (_i, [_vp, ctypes.POINTER(_i)]),
    "d8k_ctx_num_sms": (_i, [_vp]),
    "d8k_last_error": (ctypes.c_char_p, []),
    "d8k_launch_count": (ctypes.c_ulonglong, []),
    "d8k_last_kernel": (ctypes.c_char_p, []),
    "d8k_gemm": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _ll, _i, _ll, _vp, _ll, _i, _ll, _vp, _ll, _ll, _i, _i, _i]),
    "d8k_gemm_static": (_i, [_i, _i, _i, _i, _i, _i, _vp, _ll, _vp, _ll, _vp, _ll, _i, _vp]),
    "d8k_matmul_forward": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp]),
    "d8k_matmul_grad_x": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp]),
    "d8k_matmul_grad_y": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp]),
    "d8k_matmul_grad_x_into": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, _i]),
    "d8k_matmul_grad_y_into": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, _i]),
    "d8k_matmul_forward_relu": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, _vp]),
    "d8k_matmul_grad_x_relu": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, _i, _vp, _vp, _i]),
    "d8k_matmul_forward_bias": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, _vp]),
    "d8k_add_bias": (_i, [_vp, _i, _vp, _vp, _vp, _sz, _i]),
    "d8k_add_bias_grad": (_i, [_vp, _i, _vp, _vp, _sz, _i]),
    "d8k_conv2d_out_dim": (_i, [_i, _i, _i, _i, _i]),
    "d8k_deconv2d_out_dim": (_i, [_i, _i, _i, _i]),
    "d8k_conv2d_interim_size": (_sz, [_vp, _i, _i] + [_i] * 9),
    "d8k_deconv2d_interim_size": (_sz, [_vp, _i, _i] + [_i] * 9),
    "d8k_conv2d_forward": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz]),
    "d8k_conv2d_grad_x": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz]),
    "d8k_conv2d_grad_y": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz]),
    "d8k_deconv2d_forward": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _vp, _sz]),
    "d8k_deconv2d_grad_x": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _vp, _sz]),
    "d8k_deconv2d_grad_y": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _vp, _sz]),
    "d8k_conv2d_grad_x_into": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _i]),
    "d8k_conv2d_grad_y_into": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _i]),
    "d8k_deconv2d_grad_x_into": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _vp, _sz, _i]),
    "d8k_deconv2d_grad_y_into": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _vp, _sz, _i]),
    "d8k_linear_forward": (_i, [_vp, _i, _vp, ctypes.c_float, ctypes.c_float, _vp, _sz]),
    "d8k_linear_grad": (_i, [_vp, _i, _vp, ctypes.c_float, _vp, _sz]),
    "d8k_matmul_forward_linear": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, ctypes.c_float, ctypes.c_float, _vp]),
    "d8k_adam_update": (_i, [_vp, _i, _vp, _vp, _vp, _vp] + [ctypes.c_float] * 5 + [_ll, _sz]),
    "d8k_adam_ratio": (ctypes.c_float, [ctypes.c_float, ctypes.c_float, ctypes.c_float, _ll]),
    "d8k_sum_shards_adam": (_i, [_vp, _i, _vp, ctypes.POINTER(_vp), _i, _sz, _vp, _vp, _vp] + [ctypes.c_float] * 5 + [_ll, ctypes.POINTER(_vp), _i]),
    "d8k_relu_forward": (_i, [_vp, _i, _vp, _vp, _sz]),
    "d8k_relu_backward": (_i, [_vp, _i, _vp, _vp, _vp, _sz]),
    "d8k_zero": (_i, [_vp, _vp, _sz]),
    "d8k_peer_alloc": (_i, [_vp, _sz, ctypes.POINTER(_vp), ctypes.c_char_p]),
    "d8k_peer_free": (_i, [_vp, _vp]),
    "d8k_peer_open": (_i, [_vp, ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "d8k_peer_close": (_i, [_vp, _vp]),
    "d8k_peer_signal": (_i, [_vp, ctypes.POINTER(_vp), _i, ctypes.c_uint]),
    "d8k_peer_wait": (_i, [_vp, ctypes.POINTER(_vp), _i, ctypes.c_uint, ctypes.c_double]),
    "d8k_peer_copy": (_i, [_vp, _vp, _vp, _sz]),
    "d8k_matmul_grad_y_scatter": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, ctypes.POINTER(_vp), _i, _i]),
    "d8k_sum_shards": (_i, [_vp, _i, _vp, ctypes.POINTER(_vp), _i, _sz]),
    "d8k_sum_shards_gather": (_i, [_vp, _i, _vp, ctypes.POINTER(_vp), _i, _sz, _vp, ctypes.c_float, ctypes.c_float, ctypes.POINTER(_vp), _i]),
    "d8k_axpby": (_i, [_vp, _i, _vp, ctypes.c_float, _vp, ctypes.c_float, _sz]),
    "d8k_sum_shards_sgd": (_i, [_vp, _i, _vp, ctypes.POINTER(_vp), _i, _sz, _vp, ctypes.c_float, ctypes.c_float]),
}

IPC_HANDLE_BYTES = 64

_lib = None


class D8kError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("d8k error %d: %s" % (code, text))
        self.code = code


def load():
    """Load the shared library once and declare every entry point."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: build it with `python -m deep8_b200.build` (needs nvcc)" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            if os.environ.get("D8K_LIB_PATH") and not hasattr(lib, name):
                continue  # an older build under test may lack newer entry points
            fn = getattr(lib, name)  # AttributeError here means header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc):
    if rc != 0:
        raise D8kError(rc, load().d8k_last_error().decode())
