"""``reparametrize`` and the autograd Function of the box convolution, with the reference's call
signatures (``box_convolution/box_convolution_function.py:5-65``).

Unlike the reference, the Function does not chain integral_image -> forward and does not save the
integral image or the output for the backward pass: the fused entry points work from the input
itself (integral images live on chip for planes that fit there) and the term the reference
takes from the saved output is recomputed, so only the input and the four parameter tensors are
kept alive between forward and backward.

float64 tensors (gradient checks) take the general kernels through the four extension functions,
chained as the reference chains them.  float16 / bfloat16 tensors: planes that the shared-memory
kernels hold are read and written in their 16-bit type by those kernels (float arithmetic on chip,
float parameter gradients rounded at the end); for larger planes the Function makes float copies,
runs the float kernels and rounds results and gradients back.
"""
import torch

from . import _cabi
from ._cabi import check, lib
from . import ext
from .ext import _require_cuda_float, _stream, _workspace


def reparametrize(x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w,
                  inplace=False, inverse=False):
    """Scales box parameters between pixel units and the stored, roughly [-1, 1] units.
    ``inverse=True``: stored -> pixels (multiply by the factors); otherwise pixels -> stored.
    Returns four new tensors unless ``inplace``."""
    factor_h = reparametrization_h if inverse else 1 / reparametrization_h
    factor_w = reparametrization_w if inverse else 1 / reparametrization_w
    with torch.no_grad():
        if not inplace:
            return x_min * factor_h, x_max * factor_h, y_min * factor_w, y_max * factor_w
        x_min *= factor_h
        x_max *= factor_h
        y_min *= factor_w
        y_max *= factor_w


class BoxConvolutionFunction(torch.autograd.Function):
    """apply(input, x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w,
    normalize, exact) -> output (N, C*F, h, w).  The parameters are the stored ones.

    One optional tenth argument, used by the module: ``snapshot``, a packed float32 ``(4, C, F)``
    copy of the four parameter tensors as they are at this call (``ext.clip_parameters_packed``
    makes it while clipping).  Without it the Function copies the parameters itself."""

    @staticmethod
    def forward(ctx, input, x_min, x_max, y_min, y_max,
                reparametrization_h, reparametrization_w, normalize, exact, snapshot=None):
        ctx.narrow = None
        ctx.narrow_kernels = False
        if isinstance(input, torch.Tensor) and input.dtype in ext._NARROW:
            out = BoxConvolutionFunction._forward_narrow(ctx, input, x_min, x_max, y_min, y_max, reparametrization_h,
                                                         reparametrization_w, normalize, exact)
            if out is not None:
                return out
            # planes that the shared-memory kernels do not hold: float copies, float kernels
            (input, x_min, x_max, y_min, y_max), ctx.narrow = ext._widen([input, x_min, x_max, y_min, y_max])
            snapshot = None
        out = BoxConvolutionFunction._forward_wide(ctx, input, x_min, x_max, y_min, y_max, reparametrization_h,
                                                   reparametrization_w, normalize, exact, snapshot)
        return out if ctx.narrow is None else out.to(ctx.narrow)

    @staticmethod
    def _forward_narrow(ctx, input, x_min, x_max, y_min, y_max,
                        reparametrization_h, reparametrization_w, normalize, exact):
        """float16 / bfloat16 tensors on the kernels that read and write them as they are (the
        reference's half instantiations, src/box_convolution_cuda_forward.cu:224).  Returns None when
        the shape is not served that way."""
        params = (x_min, x_max, y_min, y_max)
        if not (input.is_cuda and input.dim() == 4 and all(isinstance(p, torch.Tensor) and p.is_cuda and p.dim() == 2
                                                           and p.device == input.device for p in params)):
            return None
        N, C, h, w = input.shape
        F = x_min.size(1)
        if not all(tuple(p.shape) == (C, F) and p.dtype == input.dtype for p in params):
            return None
        if not lib.bc_boxconv2d_narrow_supported(F, h, w):
            return None
        input = input.contiguous()
        # the parameters (and later their gradients) are small: float copies of them
        wide = torch.cat([p.detach().reshape(-1) for p in params]).float().view(4, C, F)
        kind = _cabi.BC_IO_F16 if input.dtype == torch.float16 else _cabi.BC_IO_BF16
        out = torch.empty((N, C * F, h, w), dtype=input.dtype, device=input.device)
        with torch.cuda.device(input.device):
            check(lib.bc_boxconv2d_forward_narrow(
                input.data_ptr(), kind, *[wide[i].data_ptr() for i in range(4)],
                float(reparametrization_h), float(reparametrization_w), out.data_ptr(),
                N, C, F, h, w, int(bool(normalize)), int(bool(exact)), _stream()), "BoxConv2d forward")
        ctx.normalize, ctx.exact = bool(normalize), bool(exact)
        ctx.reparametrization_h, ctx.reparametrization_w = reparametrization_h, reparametrization_w
        ctx.chained = False
        ctx.narrow_kernels = True
        ctx.io_kind = kind
        ctx.save_for_backward(input, wide)
        return out

    @staticmethod
    def _backward_narrow(ctx, grad_output):
        input, wide = ctx.saved_tensors
        N, C, h, w = input.shape
        F = wide.size(2)
        needs = ctx.needs_input_grad[:5]
        mask = sum(1 << i for i, b in enumerate(needs) if b)
        grad_input = grad_params = None
        if mask:
            if grad_output.dtype != input.dtype:
                grad_output = grad_output.to(input.dtype)
            grad_output = grad_output.contiguous()
            dev = input.device
            if needs[0]:
                grad_input = torch.empty_like(input)
            if any(needs[1:]):
                grad_params = torch.empty((4, C, F), dtype=torch.float32, device=dev)
            with torch.cuda.device(dev):
                ws = _workspace(lib.bc_boxconv2d_backward_workspace(N, C, F, h, w, mask), dev)
                check(lib.bc_boxconv2d_backward_narrow(
                    input.data_ptr(), ctx.io_kind, *[wide[i].data_ptr() for i in range(4)], grad_output.data_ptr(),
                    float(ctx.reparametrization_h), float(ctx.reparametrization_w),
                    N, C, F, h, w, int(ctx.normalize), int(ctx.exact), mask,
                    grad_input.data_ptr() if grad_input is not None else None,
                    grad_params.data_ptr() if grad_params is not None else None,
                    ws.data_ptr(), ws.numel(), _stream()), "BoxConv2d backward")
            if grad_params is not None:
                grad_params = grad_params.to(input.dtype)
        grads = [grad_input] + [grad_params[i] if needs[1 + i] else None for i in range(4)]
        return tuple(grads) + BoxConvolutionFunction._no_grads(ctx)

    @staticmethod
    def _forward_wide(ctx, input, x_min, x_max, y_min, y_max,
                      reparametrization_h, reparametrization_w, normalize, exact, snapshot=None):
        _require_cuda_float(input, "input")
        if input.dim() != 4:
            raise RuntimeError("BoxConv2d: input must have 4 dimensions")
        params = (x_min, x_max, y_min, y_max)
        for p, n in zip(params, ("x_min", "x_max", "y_min", "y_max")):
            _require_cuda_float(p, n, input.dtype)
            if p.device != input.device:
                raise RuntimeError("BoxConv2d: input and parameters are on different devices")
        if not all(p.dim() == 2 for p in params):
            raise RuntimeError("BoxConv2d: all parameters must have 2 dimensions")
        N, C, h, w = input.shape
        if not all(p.size(0) == C for p in params):
            raise RuntimeError("BoxConv2d: all parameters must have as many rows as there are input channels")
        F = x_min.size(1)
        if not all(p.size(1) == F for p in params):
            raise RuntimeError("BoxConv2d: all parameters must have equal number of columns")

        input = input.contiguous()
        # The backward pass works on a snapshot of the parameters, as the reference saves fresh
        # pixel-unit copies: the module changes its parameters in place (clipping) between a forward
        # and the backward that belongs to it.  The module supplies the snapshot; otherwise one launch
        # copies the four tensors into a packed buffer.  No snapshot when nothing will be differentiated.
        if any(ctx.needs_input_grad[:5]):
            if (snapshot is None or snapshot.dtype != input.dtype or snapshot.device != input.device
                    or tuple(snapshot.shape) != (4, C, F) or not snapshot.is_contiguous()):
                snapshot = torch.cat([p.detach().reshape(-1) for p in params]).view(4, C, F)
            params = [snapshot[0], snapshot[1], snapshot[2], snapshot[3]]
        else:
            params = [p.detach().contiguous() for p in params]
        ctx.normalize, ctx.exact = bool(normalize), bool(exact)
        ctx.reparametrization_h, ctx.reparametrization_w = reparametrization_h, reparametrization_w
        ctx.chained = input.dtype == torch.float64
        if ctx.chained:
            # box_convolution_function.py:36-49 of the reference: pixels, integral image, gather
            pixels = reparametrize(*params, reparametrization_h, reparametrization_w, inverse=True)
            input_integrated = ext.integral_image(input)
            out = ext.box_convolution_forward(input_integrated, *pixels, normalize, exact)
            ctx.save_for_backward(input_integrated, *pixels)
            return out
        out = torch.empty((N, C * F, h, w), dtype=torch.float32, device=input.device)
        with torch.cuda.device(input.device):
            ws = _workspace(lib.bc_boxconv2d_forward_workspace(N, C, F, h, w), input.device)
            check(lib.bc_boxconv2d_forward(
                input.data_ptr(), *[p.data_ptr() for p in params],
                float(reparametrization_h), float(reparametrization_w), out.data_ptr(),
                N, C, F, h, w, int(bool(normalize)), int(bool(exact)),
                ws.data_ptr(), ws.numel(), _stream()), "BoxConv2d forward")
        ctx.save_for_backward(input, *params)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.narrow_kernels:
            return BoxConvolutionFunction._backward_narrow(ctx, grad_output)
        if ctx.narrow is not None:
            grads = BoxConvolutionFunction._backward_wide(ctx, grad_output.float())
            return tuple(g.to(ctx.narrow) if g is not None else None for g in grads)
        return BoxConvolutionFunction._backward_wide(ctx, grad_output)

    @staticmethod
    def _no_grads(ctx):
        """None for every argument after the five differentiable ones."""
        return (None,) * (len(ctx.needs_input_grad) - 5)

    @staticmethod
    def _backward_wide(ctx, grad_output):
        if ctx.chained:
            input_integrated, x_min, x_max, y_min, y_max = ctx.saved_tensors
            needs = ctx.needs_input_grad[:5]
            grads = ext.box_convolution_backward(
                input_integrated, x_min, x_max, y_min, y_max, grad_output, None,
                ctx.reparametrization_h, ctx.reparametrization_w, ctx.normalize, ctx.exact, *needs)
            return tuple(g if n else None for g, n in zip(grads, needs)) + BoxConvolutionFunction._no_grads(ctx)
        input, x_min, x_max, y_min, y_max = ctx.saved_tensors
        N, C, h, w = input.shape
        F = x_min.size(1)
        needs = ctx.needs_input_grad[:5]
        mask = sum(1 << i for i, b in enumerate(needs) if b)
        grad_input = grad_params = None
        if mask:
            _require_cuda_float(grad_output, "grad_output", torch.float32)
            grad_output = grad_output.contiguous()
            dev = input.device
            if needs[0]:
                grad_input = torch.empty_like(input)
            if any(needs[1:]):
                grad_params = torch.empty((4, C, F), dtype=torch.float32, device=dev)
            with torch.cuda.device(dev):
                ws = _workspace(lib.bc_boxconv2d_backward_workspace(N, C, F, h, w, mask), dev)
                check(lib.bc_boxconv2d_backward(
                    input.data_ptr(), x_min.data_ptr(), x_max.data_ptr(), y_min.data_ptr(),
                    y_max.data_ptr(), grad_output.data_ptr(),
                    float(ctx.reparametrization_h), float(ctx.reparametrization_w),
                    N, C, F, h, w, int(ctx.normalize), int(ctx.exact), mask,
                    grad_input.data_ptr() if grad_input is not None else None,
                    grad_params.data_ptr() if grad_params is not None else None,
                    ws.data_ptr(), ws.numel(), _stream()), "BoxConv2d backward")
        grads = [grad_input] + [grad_params[i] if needs[1 + i] else None for i in range(4)]
        return tuple(grads) + BoxConvolutionFunction._no_grads(ctx)
