"""ctypes binding of libwinograd2x2_b200.so (the C ABI declared in include/winograd2x2_b200.h).

There is no CPU or PyTorch fallback: if the shared library is missing, importing this module
raises, and every call that returns a non-zero status raises Wg2x2Error.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "libwinograd2x2_b200.so")

NHWC, NCHW = 0, 1
MATH_FP32, MATH_TF32 = 0, 1

OK, ERR_BAD_ARG, ERR_WORKSPACE, ERR_LAUNCH, ERR_TIMEOUT, ERR_UNSUPPORTED = 0, -1, -2, -3, -4, -5


class Wg2x2Error(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        super().__init__("%s: status %d (%s)" % (what, status, lib.wg2x2_status_string(status).decode()))


if not os.path.exists(LIB_PATH):
    raise ImportError(
        "libwinograd2x2_b200.so not found at %s; build it with `python %s` (nvcc, sm_100a). "
        "There is no fallback path." % (LIB_PATH, os.path.join(os.path.dirname(_HERE), "build.py")))

lib = ctypes.CDLL(LIB_PATH)

_p, _i, _z = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
_SIGS = {
    "wg2x2_status_string": (ctypes.c_char_p, [_i]),
    "wg2x2_abi_version": (_i, []),
    "wg2x2_imtrans_fwd": (_i, [_p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "wg2x2_imtrans_fwd_affine": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "wg2x2_imtrans_bwd": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "wg2x2_conv_fwd": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p, _z, _p]),
    "wg2x2_conv_fwd_workspace_bytes": (_z, [_i, _i, _i, _i, _i, _i]),
    "wg2x2_prepared_weights_bytes": (_z, [_i, _i]),
    "wg2x2_weights_prepare": (_i, [_p, _i, _i, _p, _z, _p]),
    "wg2x2_conv_fwd_prepared": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p]),
    "wg2x2_conv_fwd_prepared_fused": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p]),
    "wg2x2_conv_fwd_prepared_ws": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _z, _p]),
    "wg2x2_conv_fwd_prepared_workspace_bytes": (_z, [_i, _i, _i, _i, _i]),
    "wg2x2_conv_bwd": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p, _z, _p]),
    "wg2x2_conv_bwd_workspace_bytes": (_z, [_i, _i, _i, _i, _i, _i, _i]),
    "wg2x2_conv_bwd_dw_noalloc": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "wg2x2_conv_bwd_dw_noalloc_max_bytes": (_z, []),
    "wg2x2_layer_fwd": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p, _z, _p]),
    "wg2x2_layer_fwd_workspace_bytes": (_z, [_i, _i, _i, _i, _i, _i, _i]),
    "wg2x2_layer_fwd_prepared": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p]),
    "wg2x2_layer_fwd_prepared_ws": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _z, _p]),
    "wg2x2_layer_fwd_prepared_workspace_bytes": (_z, [_i, _i, _i, _i, _i]),
    "wg2x2_layer_fwd_fused": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p]),
    "wg2x2_layer_fwd_fused_affine": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p]),
    "wg2x2_layer_fwd_fused_supported": (_i, [_i, _i, _i, _i, _i, _i]),
    "wg2x2_maxpool3x3s2_same_nhwc_in": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "wg2x2_maxpool3x3s2_same": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "wg2x2_stem_prepared_floats": (_i, []),
    "wg2x2_stem_prepare": (_i, [_p, _p, _p]),
    "wg2x2_stem7x7s2_pool": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "wg2x2_last_device_status": (_i, [_p, ctypes.POINTER(ctypes.c_uint)]),
    "wg2x2_set_wait_limit": (_i, [ctypes.c_longlong]),
    "wg2x2_test_drop_load": (_i, [_i]),
    "wg2x2_test_wait_probe": (_i, [ctypes.c_longlong, ctypes.c_uint, _p]),
}
for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTS = tuple(_SIGS)


def check(status, what):
    if status != OK:
        raise Wg2x2Error(status, what)
