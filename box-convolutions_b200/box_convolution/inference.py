"""Inference-only helpers for networks built from box blocks.

``fused_box_block`` runs, in one kernel pass over the data, what the reference's
``BottleneckBoxConv`` does around its ``BoxConv2d`` in eval mode as separate PyTorch operators
(``examples/Cityscapes/models/ENet.py:282-304``, ``examples/Cityscapes/models/ERFNet.py:117-137``):
the ReLU in front of it, the BatchNorm2d after it (folded to a per-channel scale and shift), the
skip connection and the final ReLU.  No gradients flow through it.

``GraphedForward`` replays a captured CUDA graph of any such forward on fixed buffers, which takes
the Python and launch overhead out of single-frame latency (the scenario of the reference's
``examples/Cityscapes/convnet-runtime-benchmark.py``).
"""
import torch

from ._cabi import check, lib
from .ext import _require_cuda_float, _stream, _workspace


def fold_batchnorm(bn):
    """(scale, shift) of an eval-mode ``nn.BatchNorm2d``: y = scale * x + shift per channel."""
    with torch.no_grad():
        inv = torch.rsqrt(bn.running_var + bn.eps)
        scale = inv * bn.weight if bn.weight is not None else inv
        shift = -bn.running_mean * scale
        if bn.bias is not None:
            shift = shift + bn.bias
    return scale.float().contiguous(), shift.float().contiguous()


def fused_box_block(module, input, *, input_relu=False, scale=None, shift=None, residual=None,
                    output_relu=False, out=None):
    """out = act(scale * module(act_in(input)) + shift + residual), per output channel.

    module    a ``BoxConv2d`` (its stored parameters are used as they are: call ``module.eval()``
              first so that they have been clipped once, as the reference does);
    scale, shift  tensors of ``in_planes * num_filters`` values or None;
    residual  tensor of the output's shape or None;
    out       where to write (may be ``residual`` for an in-place skip connection); allocated if None.
    """
    _require_cuda_float(input, "input", torch.float32)
    if input.dim() != 4 or input.size(1) != module.in_planes:
        raise RuntimeError("fused_box_block: input must be (N, %d, h, w)" % module.in_planes)
    input = input.detach().contiguous()
    N, C, h, w = input.shape
    F = module.num_filters
    dev = input.device

    def per_channel(t, name):
        if t is None:
            return None
        _require_cuda_float(t, name, torch.float32)
        if t.numel() != C * F or t.device != dev:
            raise RuntimeError("fused_box_block: %s must hold %d values on the input's device" % (name, C * F))
        return t.detach().contiguous()

    scale, shift = per_channel(scale, "scale"), per_channel(shift, "shift")
    if out is None:
        out = torch.empty((N, C * F, h, w), dtype=torch.float32, device=dev)
    for t, name in ((residual, "residual"), (out, "out")):
        if t is None:
            continue
        _require_cuda_float(t, name, torch.float32)
        if tuple(t.shape) != (N, C * F, h, w) or not t.is_contiguous() or t.device != dev:
            raise RuntimeError("fused_box_block: %s must be a contiguous (N, %d, h, w) tensor on the input's device" % (name, C * F))
    params = [p.detach().contiguous() for p in (module.x_min, module.x_max, module.y_min, module.y_max)]
    with torch.cuda.device(dev):
        ws = _workspace(lib.bc_boxconv2d_forward_workspace(N, C, F, h, w), dev)
        check(lib.bc_boxconv2d_forward_fused(
            input.data_ptr(), *[p.data_ptr() for p in params],
            float(module.reparametrization_h), float(module.reparametrization_w), out.data_ptr(),
            N, C, F, h, w, int(bool(module.normalize)), int(bool(module.exact)),
            int(bool(input_relu)), scale.data_ptr() if scale is not None else None,
            shift.data_ptr() if shift is not None else None,
            residual.detach().data_ptr() if residual is not None else None, int(bool(output_relu)),
            ws.data_ptr(), ws.numel(), _stream()), "bc_boxconv2d_forward_fused")
    return out


class GraphedForward:
    """CUDA graph of ``fn(*inputs)`` on fixed buffers.

    ``g = GraphedForward(fn, example)`` runs ``fn`` a few times on copies of the example inputs,
    captures one more run, and from then on ``g(x)`` copies ``x`` into the captured input buffer,
    replays the graph and returns the captured output tensor (overwritten by the next call).
    ``g.inputs`` / ``g.output`` give the buffers for callers that fill them in place and call
    ``g.replay()`` themselves.  ``fn`` must not allocate differently from run to run and must not
    synchronise; it runs under ``torch.no_grad()``.
    """

    def __init__(self, fn, *example_inputs, warmup=3):
        self.inputs = [t.detach().clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):
                fn(*self.inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.output = fn(*self.inputs)

    def replay(self):
        self.graph.replay()
        return self.output

    def __call__(self, *inputs):
        for dst, src in zip(self.inputs, inputs):
            dst.copy_(src, non_blocking=True)
        return self.replay()
