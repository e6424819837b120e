"""The four functions of the reference's compiled module ``box_convolution_cpp_cuda``
(``src/bind.cpp:29-34``), with the same names, argument order and return values, served by the
sm_100a library.  Code written against ``box_convolution_cpp_cuda`` can import this module in
its place.  Tensors must be CUDA float32 or float64 (all arguments of one call in the same type);
there is no CPU implementation.

float16 and bfloat16 tensors are accepted as well, as storage types only: they are widened to float32
on the device, the float32 kernels run, and results are rounded back to the caller's type (the
reference runs its arithmetic in half precision, integral images included; nothing here does).
"""
import torch

from . import _cabi
from ._cabi import check, lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _require_cuda_float(t, name, dtype=None):
    """CUDA tensor of float32 or float64 (of `dtype` when given)."""
    if not isinstance(t, torch.Tensor):
        raise TypeError("%s must be a tensor" % name)
    if not t.is_cuda:
        raise RuntimeError("box_convolution: %s is not a CUDA tensor; this build has no CPU implementation" % name)
    if t.dtype not in (torch.float32, torch.float64):
        raise RuntimeError("box_convolution: %s must be float32 or float64, got %s" % (name, t.dtype))
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError("box_convolution: %s is %s but the call's other tensors are %s" % (name, t.dtype, dtype))


_NARROW = (torch.float16, torch.bfloat16)


def _widen(tensors):
    """(float32 copies of the tensors, the narrow dtype they had) if the first one is float16 or
    bfloat16, else (the tensors, None)."""
    first = next((t for t in tensors if isinstance(t, torch.Tensor)), None)
    if first is None or first.dtype not in _NARROW:
        return tensors, None
    narrow = first.dtype
    for t in tensors:
        if isinstance(t, torch.Tensor) and t.numel() and t.dtype != narrow:
            raise RuntimeError("box_convolution: tensors of one call must share a dtype, got %s and %s" % (narrow, t.dtype))
    return [t.float() if isinstance(t, torch.Tensor) and t.numel() else t for t in tensors], narrow


def _entry(name, dtype):
    """The library function `name` for `dtype`."""
    return getattr(lib, name + ("_f64" if dtype == torch.float64 else ""))


def _check_params(x_min, x_max, y_min, y_max, in_planes, prefix, dtype):
    # same conditions and wording as src/box_convolution_interface.cpp:24-34,159-170
    ps = (x_min, x_max, y_min, y_max)
    for p, n in zip(ps, ("x_min", "x_max", "y_min", "y_max")):
        _require_cuda_float(p, n, dtype)
    if not all(p.dim() == 2 for p in ps):
        raise RuntimeError(prefix + "all parameters must have 2 dimensions")
    if not all(p.size(0) == in_planes for p in ps):
        raise RuntimeError(prefix + "all parameters must have as many rows as there are input channels")
    if not all(p.size(1) == x_min.size(1) for p in ps):
        raise RuntimeError(prefix + "all parameters must have equal number of columns")
    return [p.contiguous() for p in ps]


def _workspace(nbytes, device):
    # torch's caching allocator hands out blocks aligned to 512 bytes
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)


def integral_image(input):
    """(..., h, w) -> (..., h+1, w+1) zero-padded 2-D prefix sum.
    Mirrors src/integral_image_interface.cpp:8-27."""
    (input,), narrow = _widen([input])
    if narrow is not None:
        return integral_image(input).to(narrow)
    _require_cuda_float(input, "input")
    if input.dim() < 2:
        raise RuntimeError("integral image input must have >=2 dimensions")
    input = input.contiguous()
    h, w = input.shape[-2:]
    out = torch.empty(input.shape[:-2] + (h + 1, w + 1), dtype=input.dtype, device=input.device)
    planes = input.numel() // (h * w) if h * w else (out.numel() // ((h + 1) * (w + 1)))
    with torch.cuda.device(input.device):
        check(_entry("bc_integral_image", input.dtype)(input.data_ptr(), out.data_ptr(), planes, h, w, _stream()), "integral_image")
    return out


def box_convolution_forward(input_integrated, x_min, x_max, y_min, y_max, normalize, exact):
    """Mirrors src/box_convolution_interface.cpp:13-139.  Parameters are in actual pixels."""
    wide, narrow = _widen([input_integrated, x_min, x_max, y_min, y_max])
    if narrow is not None:
        return box_convolution_forward(*wide, normalize, exact).to(narrow)
    _require_cuda_float(input_integrated, "input_integrated")
    dtype = input_integrated.dtype
    if input_integrated.device != x_min.device:
        raise RuntimeError("BoxConv2d: input and parameters are on different devices")
    input_integrated = input_integrated.contiguous()
    if input_integrated.dim() != 4:
        raise RuntimeError("BoxConv2d: input must have 4 dimensions")
    ps = _check_params(x_min, x_max, y_min, y_max, input_integrated.size(1), "BoxConv2d: ", dtype)
    N, C, hp, wp = input_integrated.shape
    F = ps[0].size(1)
    h, w = hp - 1, wp - 1
    out = torch.empty((N, C, F, h, w), dtype=dtype, device=input_integrated.device)
    with torch.cuda.device(out.device):
        check(_entry("bc_box_convolution_forward", dtype)(
            input_integrated.data_ptr(), *[p.data_ptr() for p in ps], out.data_ptr(),
            N, C, F, h, w, int(bool(normalize)), int(bool(exact)), _stream()), "box_convolution_forward")
    return out.reshape(N, C * F, h, w)


def box_convolution_backward(
        input_integrated, x_min, x_max, y_min, y_max, grad_output, output,
        reparametrization_h, reparametrization_w, normalize, exact,
        input_needs_grad, x_min_needs_grad, x_max_needs_grad, y_min_needs_grad, y_max_needs_grad):
    """Mirrors src/box_convolution_interface.cpp:141-395: returns
    [grad_input, grad_x_min, grad_x_max, grad_y_min, grad_y_max]; entries not asked for are
    0-element tensors (interface.cpp:182,394).  `output` is accepted and ignored."""
    wide, narrow = _widen([input_integrated, x_min, x_max, y_min, y_max, grad_output])
    if narrow is not None:
        grads = box_convolution_backward(
            *wide, None, reparametrization_h, reparametrization_w, normalize, exact,
            input_needs_grad, x_min_needs_grad, x_max_needs_grad, y_min_needs_grad, y_max_needs_grad)
        return [g.to(narrow) for g in grads]
    _require_cuda_float(input_integrated, "input_integrated")
    dtype = input_integrated.dtype
    _require_cuda_float(grad_output, "grad_output", dtype)
    grad_output = grad_output.contiguous()
    input_integrated = input_integrated.contiguous()
    if grad_output.dim() != 4:
        raise RuntimeError("grad_output for box_convolution must have 4 dimensions")
    if input_integrated.dim() != 4:
        raise RuntimeError("BoxConv2d: input must have 4 dimensions")
    N, C, hp, wp = input_integrated.shape
    h, w = hp - 1, wp - 1
    ps = _check_params(x_min, x_max, y_min, y_max, C, "", dtype)
    F = ps[0].size(1)
    # the reference checks the height twice and never the width (interface.cpp:157-158); both here
    if tuple(grad_output.shape) != (N, C * F, h, w):
        raise RuntimeError("box_convolution: sizes of grad_output and input_integrated don't match")
    needs = [input_needs_grad, x_min_needs_grad, x_max_needs_grad, y_min_needs_grad, y_max_needs_grad]
    mask = sum(1 << i for i, b in enumerate(needs) if b)
    dev = input_integrated.device
    null = torch.empty(0)
    grad_input = torch.empty((N, C, h, w), dtype=dtype, device=dev) if needs[0] else None
    grad_params = torch.empty((4, C, F), dtype=dtype, device=dev) if any(needs[1:]) else None
    if mask:
        with torch.cuda.device(dev):
            ws = _workspace(_entry("bc_box_convolution_backward_workspace", dtype)(N, C, F, h, w, mask), dev)
            check(_entry("bc_box_convolution_backward", dtype)(
                input_integrated.data_ptr(), *[p.data_ptr() for p in ps], grad_output.data_ptr(), None,
                float(reparametrization_h), float(reparametrization_w), N, C, F, h, w,
                int(bool(normalize)), int(bool(exact)), mask,
                grad_input.data_ptr() if grad_input is not None else None,
                grad_params.data_ptr() if grad_params is not None else None,
                ws.data_ptr(), ws.numel(), _stream()), "box_convolution_backward")
    return [grad_input if needs[0] else null] + [grad_params[i] if needs[1 + i] else null for i in range(4)]


def clip_parameters(x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w,
                    max_input_h, max_input_w, exact):
    """In place.  Mirrors src/box_convolution_interface.cpp:397-415."""
    wide, narrow = _widen([x_min, x_max, y_min, y_max])
    if narrow is not None:
        clip_parameters(*wide, reparametrization_h, reparametrization_w, max_input_h, max_input_w, exact)
        with torch.no_grad():
            for p, v in zip((x_min, x_max, y_min, y_max), wide):
                p.copy_(v)
        return
    ps = (x_min, x_max, y_min, y_max)
    for p, n in zip(ps, ("x_min", "x_max", "y_min", "y_max")):
        _require_cuda_float(p, n, x_min.dtype if isinstance(x_min, torch.Tensor) else None)
        if not p.is_contiguous():
            raise RuntimeError("%s must be contiguous" % n)
    if not all(p.numel() == x_min.numel() for p in ps):
        raise RuntimeError("box_convolution: parameter tensors differ in size")
    with torch.cuda.device(x_min.device):
        check(_entry("bc_clip_parameters", x_min.dtype)(
            *[p.data_ptr() for p in ps], x_min.numel(), float(reparametrization_h),
            float(reparametrization_w), float(max_input_h), float(max_input_w),
            int(bool(exact)), _stream()), "clip_parameters")


def clip_parameters_packed(x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w,
                           max_input_h, max_input_w, exact):
    """``clip_parameters`` for contiguous float32 CUDA tensors that also returns a packed
    ``(4,) + x_min.shape`` copy of the clipped values, written by the same launch.  The module
    hands that copy to the autograd Function as the parameter snapshot of the step."""
    ps = (x_min, x_max, y_min, y_max)
    for p, n in zip(ps, ("x_min", "x_max", "y_min", "y_max")):
        _require_cuda_float(p, n, torch.float32)
        if not p.is_contiguous():
            raise RuntimeError("%s must be contiguous" % n)
    if not all(p.shape == x_min.shape for p in ps):
        raise RuntimeError("box_convolution: parameter tensors differ in size")
    packed = torch.empty((4,) + tuple(x_min.shape), dtype=torch.float32, device=x_min.device)
    with torch.cuda.device(x_min.device):
        check(lib.bc_clip_parameters_packed(
            *[p.data_ptr() for p in ps], x_min.numel(), float(reparametrization_h),
            float(reparametrization_w), float(max_input_h), float(max_input_w),
            int(bool(exact)), packed.data_ptr(), _stream()), "clip_parameters")
    return packed
