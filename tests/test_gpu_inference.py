"""Inference helpers: the fused box-block tail against the same steps as separate PyTorch
operators around the module (the composition the reference's BottleneckBoxConv runs in eval mode,
examples/Cityscapes/models/ENet.py:282-304), and CUDA-graph replay."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-5      # relative to the largest magnitude of the expected tensor


def _module(C, F, h, w, exact, seed):
    import random
    from box_convolution import BoxConv2d
    random.seed(seed)
    m = BoxConv2d(C, F, h, w).cuda()
    m.exact = exact
    m.eval()
    return m


def _composition(m, x, input_relu, bn, residual, output_relu):
    with torch.no_grad():
        y = m(torch.relu(x) if input_relu else x)
        if bn is not None:
            y = bn(y)
        if residual is not None:
            y = y + residual
        return torch.relu(y) if output_relu else y


# whole-plane kernel (T = 1, 2, 4; guarded and unguarded), general kernel for larger planes
SHAPES = [(2, 4, 4, 64, 128), (1, 3, 2, 37, 50), (1, 2, 4, 96, 200), (1, 2, 2, 128, 256), (1, 2, 2, 200, 300),
          (1, 1, 3, 203, 301)]


@pytest.mark.parametrize("exact", [True, False])
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_block_matches_composition(shape, exact):
    from box_convolution import fused_box_block, fold_batchnorm
    N, C, F, h, w = shape
    torch.manual_seed(h + w)
    m = _module(C, F, h, w, exact, seed=h)
    bn = torch.nn.BatchNorm2d(C * F).cuda().eval()
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5); bn.bias.uniform_(-0.5, 0.5)
        bn.running_mean.uniform_(-0.2, 0.2); bn.running_var.uniform_(0.5, 2.0)
    x = torch.randn(N, C, h, w, device="cuda")
    res = torch.randn(N, C * F, h, w, device="cuda")
    scale, shift = fold_batchnorm(bn)
    for input_relu, use_bn, use_res, output_relu in [(True, True, True, True), (False, False, False, False),
                                                     (True, False, True, False), (False, True, False, True)]:
        want = _composition(m, x, input_relu, bn if use_bn else None, res if use_res else None, output_relu)
        got = fused_box_block(m, x, input_relu=input_relu, scale=scale if use_bn else None,
                              shift=shift if use_bn else None, residual=res if use_res else None,
                              output_relu=output_relu)
        err = (got - want).abs().max().item()
        assert err <= TOL * max(1.0, want.abs().max().item()), (input_relu, use_bn, use_res, output_relu, err)


def test_fused_block_in_place_skip_connection():
    from box_convolution import fused_box_block
    m = _module(4, 4, 64, 128, True, seed=1)
    x = torch.randn(2, 4, 64, 128, device="cuda")
    skip = torch.randn(2, 16, 64, 128, device="cuda")
    want = _composition(m, x, False, None, skip, True)
    buf = skip.clone()
    got = fused_box_block(m, x, residual=buf, output_relu=True, out=buf)
    assert got.data_ptr() == buf.data_ptr()
    assert (got - want).abs().max().item() <= TOL * want.abs().max().item()


def test_plain_forward_unchanged_by_fusion_arguments():
    """All fusion steps off: bit-identical to the module's forward."""
    from box_convolution import fused_box_block
    m = _module(3, 4, 64, 128, True, seed=2)
    x = torch.randn(2, 3, 64, 128, device="cuda")
    with torch.no_grad():
        want = m(x)
    assert torch.equal(fused_box_block(m, x), want)


def test_graphed_forward_replays():
    from box_convolution import fused_box_block, GraphedForward
    m = _module(8, 4, 64, 128, False, seed=3)
    x0 = torch.randn(1, 8, 64, 128, device="cuda")
    skip0 = torch.randn(1, 32, 64, 128, device="cuda")

    def block(x, skip):
        return fused_box_block(m, x, input_relu=True, residual=skip, output_relu=True)

    g = GraphedForward(block, x0, skip0)
    for seed in range(3):
        torch.manual_seed(seed)
        x, skip = torch.randn_like(x0), torch.randn_like(skip0)
        got = g(x, skip).clone()
        assert torch.equal(got, block(x, skip))


def test_fused_block_rejects_bad_arguments():
    from box_convolution import fused_box_block
    m = _module(2, 2, 16, 16, True, seed=4)
    x = torch.randn(1, 2, 16, 16, device="cuda")
    with pytest.raises(RuntimeError):
        fused_box_block(m, x, scale=torch.ones(3, device="cuda"))
    with pytest.raises(RuntimeError):
        fused_box_block(m, x, residual=torch.zeros(1, 4, 16, 15, device="cuda"))
    with pytest.raises(RuntimeError):
        fused_box_block(m, x.cpu())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_narrow_storage_types_run_in_float32(dtype):
    """half / bfloat16 modules and tensors: same results as the float32 run of the same (rounded)
    values, up to the rounding of the stored result."""
    from box_convolution import BoxConv2d, integral_image
    import random
    random.seed(5)
    m32 = BoxConv2d(3, 2, 32, 48).cuda()
    m16 = BoxConv2d(3, 2, 32, 48).cuda().to(dtype)
    with torch.no_grad():
        for a, b in zip(m16.parameters(), m32.parameters()):
            a.copy_(b)
            b.copy_(a.float())                 # both modules hold the same (rounded) boxes
    x16 = torch.randn(2, 3, 32, 48, device="cuda").to(dtype).requires_grad_()
    x32 = x16.detach().float().requires_grad_()
    y16, y32 = m16(x16), m32(x32)
    assert y16.dtype == dtype
    assert torch.equal(y16, y32.to(dtype))
    g = torch.randn_like(y32).to(dtype)
    y16.backward(g)
    y32.backward(g.float())
    assert x16.grad.dtype == dtype and torch.equal(x16.grad, x32.grad.to(dtype))
    for a, b in zip(m16.parameters(), m32.parameters()):
        assert a.grad.dtype == dtype and torch.equal(a.grad, b.grad.to(dtype))
    ii = integral_image(x16.detach())
    assert ii.dtype == dtype and torch.equal(ii, integral_image(x32.detach()).to(dtype))
