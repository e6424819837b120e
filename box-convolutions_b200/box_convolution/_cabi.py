"""ctypes binding of the C ABI in ``include/boxconv_b200.h`` (``libboxconv_b200.so``).

The library is the only implementation: if it has not been built, importing this module
raises.  Build it with ``python box-convolutions_b200/build.py``.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libboxconv_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "box_convolution: %s is missing; build it with `python box-convolutions_b200/build.py` "
        "(there is no fallback implementation)" % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

_vp, _i, _i64, _f, _d, _sz = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float,
                             ctypes.c_double, ctypes.c_size_t)

SIGNATURES = {
    "bc_version": (_i, []),
    "bc_status_string": (ctypes.c_char_p, [_i]),
    "bc_last_cuda_error": (ctypes.c_char_p, []),
    "bc_integral_image": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "bc_box_convolution_forward": (_i, [_vp] * 6 + [_i] * 7 + [_vp]),
    "bc_box_convolution_backward_workspace": (_sz, [_i] * 6),
    "bc_box_convolution_backward": (_i, [_vp] * 7 + [_f, _f] + [_i] * 8 + [_vp, _vp, _vp, _sz, _vp]),
    "bc_clip_parameters": (_i, [_vp] * 4 + [_i, _d, _d, _d, _d, _i, _vp]),
    "bc_clip_parameters_packed": (_i, [_vp] * 4 + [_i, _d, _d, _d, _d, _i, _vp, _vp]),
    "bc_integral_image_f64": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "bc_box_convolution_forward_f64": (_i, [_vp] * 6 + [_i] * 7 + [_vp]),
    "bc_box_convolution_backward_workspace_f64": (_sz, [_i] * 6),
    "bc_box_convolution_backward_f64": (_i, [_vp] * 7 + [_d, _d] + [_i] * 8 + [_vp, _vp, _vp, _sz, _vp]),
    "bc_clip_parameters_f64": (_i, [_vp] * 4 + [_i, _d, _d, _d, _d, _i, _vp]),
    "bc_boxconv2d_forward_workspace": (_sz, [_i] * 5),
    "bc_boxconv2d_forward": (_i, [_vp] * 5 + [_f, _f, _vp] + [_i] * 7 + [_vp, _sz, _vp]),
    "bc_boxconv2d_forward_fused": (_i, [_vp] * 5 + [_f, _f, _vp] + [_i] * 8 + [_vp, _vp, _vp, _i, _vp, _sz, _vp]),
    "bc_boxconv2d_backward_workspace": (_sz, [_i] * 6),
    "bc_boxconv2d_backward": (_i, [_vp] * 6 + [_f, _f] + [_i] * 8 + [_vp, _vp, _vp, _sz, _vp]),
    "bc_boxconv2d_backward_static": (_i, [_vp] * 6 + [_f, _f] + [_i] * 8 + [_vp, _vp, _vp]),
    "bc_boxconv2d_narrow_supported": (_i, [_i] * 3),
    "bc_boxconv2d_forward_narrow": (_i, [_vp, _i] + [_vp] * 4 + [_f, _f, _vp] + [_i] * 7 + [_vp]),
    "bc_boxconv2d_backward_narrow": (_i, [_vp, _i] + [_vp] * 5 + [_f, _f] + [_i] * 8 + [_vp, _vp, _vp, _sz, _vp]),
    "bc_boxconv2d_host_step_workspace": (_sz, [_i] * 6),
    "bc_boxconv2d_host_step": (_i, [_vp] * 9 + [_f, _f, _d, _d] + [_i] * 9 + [_vp, _sz, _vp, _vp, _vp]),
    "bc_launch_count": (ctypes.c_uint64, []),
    "bc_wait_timeouts": (_i, [ctypes.POINTER(_i)]),
    "bc_profile_start": (_i, [_i]),
    "bc_profile_stop": (_i, []),
    "bc_profile_count": (_i, []),
    "bc_profile_get": (_i, [_i, ctypes.POINTER(_i), ctypes.POINTER(_f)]),
    "bc_kernel_name": (ctypes.c_char_p, [_i]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

BC_IO_F16, BC_IO_BF16 = 1, 2
BC_NEED_INPUT, BC_NEED_X_MIN, BC_NEED_X_MAX, BC_NEED_Y_MIN, BC_NEED_Y_MAX = 1, 2, 4, 8, 16


def check(status, what):
    """Turns a negative status into the RuntimeError the reference's TORCH_CHECKs would raise."""
    if status != 0:
        msg = lib.bc_status_string(status).decode()
        detail = lib.bc_last_cuda_error().decode()
        raise RuntimeError("%s failed: %s%s" % (what, msg, (" (" + detail + ")") if detail and status == -4 else ""))


def wait_timeouts():
    """Bounded waits that expired inside kernels on the current device (synchronises; 0 is healthy)."""
    n = ctypes.c_int(0)
    check(lib.bc_wait_timeouts(ctypes.byref(n)), "bc_wait_timeouts")
    return n.value
