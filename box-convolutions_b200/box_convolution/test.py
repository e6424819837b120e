"""Self-test of an installed package: ``python -m box_convolution.test`` (the command the
reference's README gives for its own ``box_convolution/test.py``).  Needs a GPU.

Same three checks as the reference's script, restated: the integral image against a float64
cumulative sum, the module's output and input gradient against a dense float64 restatement of the
box filter, and ``torch.autograd.gradcheck`` of all five gradients in float64.
"""
import random
import sys

import torch

from . import BoxConv2d, BoxConvolutionFunction, integral_image


def _axis_matrix(lo, hi, n):
    idx = torch.arange(n, dtype=lo.dtype, device=lo.device)
    off = idx[None, :] - idx[:, None]
    return (torch.minimum(off + 1, hi + 1) - torch.maximum(off, lo)).clamp(0, 1)


def _dense(x, x_min, x_max, y_min, y_max, normalize):
    """Row weights A and column weights B of a box are the lengths of [i, i+1] inside
    [lo, hi+1]; the filter's response is A @ X @ B^T."""
    outs = []
    for c in range(x.shape[1]):
        for f in range(x_min.shape[1]):
            o = _axis_matrix(x_min[c, f], x_max[c, f], x.shape[2]) @ x[:, c] @ _axis_matrix(y_min[c, f], y_max[c, f], x.shape[3]).t()
            if normalize:
                o = o / ((x_max[c, f] - x_min[c, f] + 1) * (y_max[c, f] - y_min[c, f] + 1))
            outs.append(o)
    return torch.stack(outs, 1)


def test_integral_image(device="cuda", cases=50):
    for _ in range(cases):
        shape = (random.randint(1, 3), random.randint(1, 3), random.randint(2, 10), random.randint(2, 10))
        x = torch.rand(shape, device=device)
        want = torch.zeros(shape[:2] + (shape[2] + 1, shape[3] + 1), dtype=torch.float64, device=device)
        want[..., 1:, 1:] = x.double().cumsum(2).cumsum(3)
        assert torch.allclose(integral_image(x).double(), want, rtol=1e-5, atol=1e-6)


def _away_from_integers(lo, hi):
    while True:
        v = random.uniform(lo, hi)
        if abs(v - round(v)) >= 0.012:
            return v


def test_box_convolution_module(device="cuda", cases=40):
    for _ in range(cases):
        C, F, h, w = random.randint(1, 2), random.randint(1, 3), random.randint(2, 10), random.randint(2, 10)
        normalize = random.random() < 0.5
        m = BoxConv2d(C, F, h + 1, w + 1, reparametrization_factor=random.uniform(0.5, 5.0), normalize=normalize).to(device)
        with torch.no_grad():
            for c in range(C):
                for f in range(F):
                    x_min = _away_from_integers(-h * 0.9, h * 0.4)
                    y_min = _away_from_integers(-w * 0.9, w * 0.4)
                    x_max = _away_from_integers(x_min + 1.1, x_min + 1.1 + h * 0.5)
                    y_max = _away_from_integers(y_min + 1.1, y_min + 1.1 + w * 0.5)
                    m.x_min[c, f], m.x_max[c, f] = x_min / m.reparametrization_h, min(x_max, h - 0.3) / m.reparametrization_h
                    m.y_min[c, f], m.y_max[c, f] = y_min / m.reparametrization_w, min(y_max, w - 0.3) / m.reparametrization_w
        x = torch.rand(2, C, h, w, device=device, requires_grad=True)
        go = (torch.rand(2, C * F, h, w, device=device) < 0.3).float()
        y = m(x)
        y.backward(go)
        pix = [p.detach().double() * r for p, r in zip(
            (m.x_min, m.x_max, m.y_min, m.y_max),
            (m.reparametrization_h, m.reparametrization_h, m.reparametrization_w, m.reparametrization_w))]
        xd = x.detach().double().requires_grad_()
        want = _dense(xd, *pix, normalize)
        want_gin, = torch.autograd.grad(want, xd, go.double())
        assert torch.allclose(y.detach().double(), want.detach(), rtol=3e-5, atol=1e-5)
        assert torch.allclose(x.grad.double(), want_gin, rtol=3e-5, atol=1e-5)

        # all five gradients in float64, by finite differences
        stored = [p.detach().double().requires_grad_() for p in (m.x_min, m.x_max, m.y_min, m.y_max)]
        eps = 0.004 / max(m.reparametrization_h, m.reparametrization_w)
        torch.autograd.gradcheck(
            lambda x_, a, b, c_, d: BoxConvolutionFunction.apply(
                x_, a, b, c_, d, m.reparametrization_h, m.reparametrization_w, normalize, True),
            [x.detach().double().requires_grad_()] + stored, eps=eps, atol=1e-5, rtol=1e-3, nondet_tol=1e-12)


if __name__ == "__main__":
    if not torch.cuda.is_available():
        sys.exit("box_convolution.test needs a GPU: this build has no CPU implementation")
    seed = 1546545757
    torch.manual_seed(seed)
    random.seed(seed)
    for test in (test_integral_image, test_box_convolution_module):
        print("Testing for device 'cuda'")
        test()
        print(test.__name__, "OK")
