"""ctypes front end of the plain-C oracle (``oracle/boxconv_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, the smoke check and the benchmark's CPU
baseline leg, never by the product package.

The wrappers take and return numpy float32 arrays (or anything ``numpy.asarray`` accepts, e.g.
CPU torch tensors) and mirror the four entry points of the reference's compiled module
(``src/bind.cpp:29-34``): ``integral_image``, ``box_convolution_forward``,
``box_convolution_backward`` and ``clip_parameters``.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "boxconv_oracle.c")
BUILD_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(BUILD_DIR, "liboracle.so")

_lib = None
_fp = ctypes.POINTER(ctypes.c_float)


def build(force=False):
    """Compile the C oracle with gcc (a second or two).  Returns the library path."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) > os.path.getmtime(SRC):
        return LIB
    os.makedirs(BUILD_DIR, exist_ok=True)
    tmp = LIB + ".tmp%d" % os.getpid()
    subprocess.check_call(
        ["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-std=c99", "-o", tmp, SRC, "-lm"]
    )
    os.replace(tmp, LIB)
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(LIB)
        i32, i64, f32, f64 = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_double
        L.orc_integral_image.argtypes = [_fp, _fp, i64, i32, i32]
        L.orc_integral_image.restype = None
        L.orc_box_convolution_forward.argtypes = [_fp] * 6 + [i32] * 7
        L.orc_box_convolution_forward.restype = None
        L.orc_box_convolution_backward.argtypes = (
            [_fp] * 7 + [f32, f32] + [i32] * 8 + [_fp, ctypes.POINTER(_fp)]
        )
        L.orc_box_convolution_backward.restype = None
        L.orc_clip_parameters.argtypes = [_fp] * 4 + [i32, f64, f64, f64, f64, i32]
        L.orc_clip_parameters.restype = None
        _lib = L
    return _lib


def _f32(a):
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(_fp)


def integral_image(x):
    x = _f32(x)
    assert x.ndim >= 2
    h, w = x.shape[-2:]
    out = np.empty(x.shape[:-2] + (h + 1, w + 1), np.float32)
    planes = x.size // (h * w) if h * w else 0
    lib().orc_integral_image(_p(x), _p(out), planes, h, w)
    return out


def box_convolution_forward(input_integrated, x_min, x_max, y_min, y_max, normalize, exact):
    I = _f32(input_integrated)
    ps = [_f32(p) for p in (x_min, x_max, y_min, y_max)]
    N, C, hp, wp = I.shape
    F = ps[0].shape[1]
    assert all(p.shape == (C, F) for p in ps)
    h, w = hp - 1, wp - 1
    out = np.empty((N, C, F, h, w), np.float32)
    lib().orc_box_convolution_forward(
        _p(I), *[_p(p) for p in ps], _p(out), N, C, F, h, w, int(bool(normalize)), int(bool(exact))
    )
    return out.reshape(N, C * F, h, w)


def box_convolution_backward(
    input_integrated, x_min, x_max, y_min, y_max, grad_output, output,
    reparametrization_h, reparametrization_w, normalize, exact,
    input_needs_grad=True, x_min_needs_grad=True, x_max_needs_grad=True,
    y_min_needs_grad=True, y_max_needs_grad=True,
):
    """Returns [grad_input, g_x_min, g_x_max, g_y_min, g_y_max]; entries not asked for are None."""
    I = _f32(input_integrated)
    ps = [_f32(p) for p in (x_min, x_max, y_min, y_max)]
    N, C, hp, wp = I.shape
    F = ps[0].shape[1]
    h, w = hp - 1, wp - 1
    g = _f32(grad_output).reshape(N, C, F, h, w)
    o = _f32(output).reshape(N, C, F, h, w) if normalize else None
    needs = [input_needs_grad, x_min_needs_grad, x_max_needs_grad, y_min_needs_grad, y_max_needs_grad]
    mask = sum(1 << i for i, b in enumerate(needs) if b)
    gin = np.zeros((N, C, h, w), np.float32)
    gps = [np.zeros((C, F), np.float32) for _ in range(4)]
    arr = (_fp * 4)(*[_p(a) for a in gps])
    lib().orc_box_convolution_backward(
        _p(I), *[_p(p) for p in ps], _p(g), _p(o) if o is not None else None,
        float(reparametrization_h), float(reparametrization_w),
        N, C, F, h, w, int(bool(normalize)), int(bool(exact)), mask, _p(gin), arr,
    )
    return [gin if needs[0] else None] + [gp if nd else None for gp, nd in zip(gps, needs[1:])]


def clip_parameters(x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w,
                    max_input_h, max_input_w, exact):
    """In place on four contiguous float32 numpy arrays of equal size."""
    for a in (x_min, x_max, y_min, y_max):
        assert isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags.c_contiguous
    lib().orc_clip_parameters(
        _p(x_min), _p(x_max), _p(y_min), _p(y_max), x_min.size,
        float(reparametrization_h), float(reparametrization_w),
        float(max_input_h), float(max_input_w), int(bool(exact)),
    )


def boxconv2d_forward_backward(x, stored_params, grad_output, reparametrization_h,
                               reparametrization_w, normalize=True, exact=True):
    """The whole module step as the reference's autograd Function runs it
    (box_convolution/box_convolution_function.py:32-65): de-reparametrize with an fp32 multiply,
    integrate, gather, then the backward call.  Returns (output, grad_input, [4 param grads])."""
    sh, sw = np.float32(reparametrization_h), np.float32(reparametrization_w)
    xm, xM, ym, yM = [_f32(p) for p in stored_params]
    actual = [xm * sh, xM * sh, ym * sw, yM * sw]
    I = integral_image(x)
    out = box_convolution_forward(I, *actual, normalize, exact)
    res = box_convolution_backward(I, *actual, grad_output, out, reparametrization_h,
                                   reparametrization_w, normalize, exact)
    return out, res[0], res[1:]
