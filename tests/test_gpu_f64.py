"""float64 instantiation of the general kernels, checked the way the reference checks its
operator (test/test_boxconv.py of the reference: a dense restatement in float64 and
torch.autograd.gradcheck), and against the float32 path of the module.

The dense restatement here: along one axis a box [lo, hi] weighs the pixel at offset i by the
length of [i, i+1] that lies inside [lo, hi+1]; the 2-D filter is the outer product of the two
axes, so the output of one (plane, filter) pair is A @ X @ B^T with banded matrices A (rows) and
B (columns).  Everything is built from differentiable torch operations, so autograd gives
reference gradients for the input and for all four parameters.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL64 = 1e-9


def _axis_matrix(lo, hi, n):
    """(n, n) matrix M[p, r] = weight of pixel r in the box sum centred at p."""
    idx = torch.arange(n, dtype=lo.dtype, device=lo.device)
    off = idx[None, :] - idx[:, None]                      # r - p
    return (torch.minimum(off + 1, hi + 1) - torch.maximum(off, lo)).clamp(0, 1)


def dense_boxconv(x, x_min, x_max, y_min, y_max, normalize):
    """x (N,C,h,w); parameters (C,F) in pixels -> (N,C*F,h,w)."""
    N, C, h, w = x.shape
    F = x_min.shape[1]
    outs = []
    for c in range(C):
        for f in range(F):
            A = _axis_matrix(x_min[c, f], x_max[c, f], h)
            B = _axis_matrix(y_min[c, f], y_max[c, f], w)
            o = A @ x[:, c] @ B.t()
            if normalize:
                o = o / ((x_max[c, f] - x_min[c, f] + 1) * (y_max[c, f] - y_min[c, f] + 1))
            outs.append(o)
    return torch.stack(outs, 1)


def _random_boxes(rng, C, F, h, w):
    """Stored-unit style random boxes in pixels, kept away from whole numbers so that finite
    differences do not straddle a kink of the piecewise-smooth operator."""
    def away(v):
        frac = v - np.floor(v)
        return np.floor(v) + np.clip(frac, 0.05, 0.95)
    x_min = away(rng.uniform(-h * 0.6, 0.0, (C, F)))
    x_max = away(x_min + rng.uniform(1.2, h * 0.8, (C, F)))
    y_min = away(rng.uniform(-w * 0.6, 0.0, (C, F)))
    y_max = away(y_min + rng.uniform(1.2, w * 0.8, (C, F)))
    return [torch.tensor(a, dtype=torch.float64, device="cuda") for a in (x_min, x_max, y_min, y_max)]


@pytest.mark.parametrize("shape", [(3, 5, 7), (2, 40, 33), (1, 9, 300)])
def test_integral_image_f64(shape):
    from box_convolution import ext
    rng = np.random.default_rng(11)
    x = rng.standard_normal(shape)
    got = ext.integral_image(torch.tensor(x, device="cuda")).cpu().numpy()
    want = np.zeros((shape[0], shape[1] + 1, shape[2] + 1))
    want[:, 1:, 1:] = x.cumsum(1).cumsum(2)
    assert got.dtype == np.float64
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-11)


@pytest.mark.parametrize("normalize", [False, True])
@pytest.mark.parametrize("N,C,F,h,w", [(2, 3, 2, 11, 13), (1, 2, 3, 37, 70)])
def test_f64_matches_dense_restatement(N, C, F, h, w, normalize):
    from box_convolution import ext
    rng = np.random.default_rng(5)
    x = torch.tensor(rng.standard_normal((N, C, h, w)), device="cuda", requires_grad=True)
    params = [p.requires_grad_() for p in _random_boxes(rng, C, F, h, w)]
    go = torch.tensor(rng.standard_normal((N, C * F, h, w)), device="cuda")

    want = dense_boxconv(x, *params, normalize)
    want_grads = torch.autograd.grad(want, [x] + params, go)

    xi = ext.integral_image(x.detach())
    got = ext.box_convolution_forward(xi, *[p.detach() for p in params], normalize, True)
    scale = want.abs().max().item()
    assert (got - want.detach()).abs().max().item() <= TOL64 * scale

    rep_h, rep_w = 1.7, 0.6   # gradients come back multiplied by these
    grads = ext.box_convolution_backward(xi, *[p.detach() for p in params], go, got, rep_h, rep_w,
                                         normalize, True, True, True, True, True, True)
    factors = [1.0, rep_h, rep_h, rep_w, rep_w]
    for g, wg, k in zip(grads, want_grads, factors):
        assert g.dtype == torch.float64
        assert (g - wg * k).abs().max().item() <= TOL64 * max(1.0, (wg * k).abs().max().item())


@pytest.mark.parametrize("normalize", [False, True])
def test_gradcheck_f64(normalize):
    """The reference's own criterion: numerical against analytical gradients in float64."""
    from box_convolution import BoxConvolutionFunction
    rng = np.random.default_rng(3)
    N, C, F, h, w = 2, 2, 2, 9, 12
    rep_h, rep_w = float(h), float(w)
    x = torch.tensor(rng.standard_normal((N, C, h, w)), device="cuda", requires_grad=True)
    pixels = _random_boxes(rng, C, F, h, w)
    stored = [(p / r).requires_grad_() for p, r in zip(pixels, (rep_h, rep_h, rep_w, rep_w))]

    def fn(x, a, b, c, d):
        return BoxConvolutionFunction.apply(x, a, b, c, d, rep_h, rep_w, normalize, True)

    assert torch.autograd.gradcheck(fn, [x] + stored, eps=1e-6, atol=1e-6, rtol=1e-5, nondet_tol=1e-12)


def test_module_in_double_matches_float():
    from box_convolution import BoxConv2d
    torch.manual_seed(2)
    m32 = BoxConv2d(4, 3, 24, 40).cuda()
    m64 = BoxConv2d(4, 3, 24, 40).cuda().double()
    with torch.no_grad():
        for a, b in zip(m64.parameters(), m32.parameters()):
            a.copy_(b.double())
    x = torch.randn(2, 4, 24, 40, device="cuda")
    y32 = m32(x)
    y64 = m64(x.double())
    assert y64.dtype == torch.float64
    assert (y32.double() - y64).abs().max().item() <= 1e-4 * y64.abs().max().item()
    g = torch.randn_like(y32)
    y32.backward(g)
    y64.backward(g.double())
    for a, b in zip(m64.parameters(), m32.parameters()):
        assert (a.grad - b.grad.double()).abs().max().item() <= 1e-3 * max(1.0, a.grad.abs().max().item())


def test_clip_f64_matches_float_rule():
    from box_convolution import ext
    rng = np.random.default_rng(9)
    ps = [torch.tensor(rng.uniform(-2.0, 2.0, (5, 7)), device="cuda") for _ in range(4)]
    ref = [p.clone() for p in ps]
    ext.clip_parameters(*ps, 32.0, 48.0, 32.0, 48.0, True)
    # the rule restated in float64 (src/box_convolution.cpp:729-763 of the reference)
    for lo, hi, rep, mx in ((ref[0], ref[1], 32.0, 32.0), (ref[2], ref[3], 48.0, 48.0)):
        inv = 1.0 / rep
        a = lo.clamp(-(mx + 1) * inv, (mx - 1) * inv)
        b = hi.clamp(-(mx + 1) * inv, (mx - 1) * inv)
        ms = float(np.float32(1.001))
        narrow = a + (ms - 0.9999) * inv > b
        mean = 0.5 * (a + b)
        a = torch.where(narrow, mean - 0.5 * (ms - 0.9999) * inv, a)
        b = torch.where(narrow, mean + 0.5 * (ms - 0.9999) * inv, b)
        lo.copy_(a)
        hi.copy_(b)
    for p, r in zip(ps, ref):
        assert (p - r).abs().max().item() <= 1e-14


def test_mixed_dtypes_are_rejected():
    from box_convolution import ext
    xi = torch.zeros(1, 1, 5, 5, device="cuda", dtype=torch.float64)
    p32 = [torch.zeros(1, 1, device="cuda") for _ in range(4)]
    with pytest.raises(RuntimeError):
        ext.box_convolution_forward(xi, *p32, False, True)


def test_reference_style_random_cases_fp32():
    """The reference's own test loop (box_convolution/test.py:186-274 of the reference), restated:
    40 random single-plane cases with h, w <= 10, 70 % exact / 30 % rounded boxes, random
    normalisation and reparametrization factor, sparse 0/1 grad_output; the float32 module against the
    dense float64 restatement with the reference's tolerances (rtol 3e-5, atol 1e-5), and the
    parameter clip must leave the test's boxes alone."""
    import random
    from box_convolution import BoxConv2d
    rnd = random.Random(1546545757)
    rng = np.random.default_rng(1546545757)
    for case in range(40):
        h, w = rnd.randint(1, 10), rnd.randint(1, 10)
        exact = rnd.random() < 0.7
        normalize = rnd.random() < 0.5
        factor = rnd.uniform(0.5, 5.0)
        m = BoxConv2d(1, 1, h + 1, w + 1, reparametrization_factor=factor, normalize=normalize).cuda()
        m.exact = exact
        # a box inside the clip range, every coordinate at least 0.012 from a whole number
        def coord(lo, hi):
            while True:
                v = rnd.uniform(lo, hi)
                if abs(v - round(v)) >= 0.012:
                    return v
        x_min = coord(-h * 0.9, h * 0.5); x_max = coord(x_min + 1.1, x_min + h)
        y_min = coord(-w * 0.9, w * 0.5); y_max = coord(y_min + 1.1, y_min + w)
        x_max, y_max = min(x_max, h - 0.5 + 0.25), min(y_max, w - 0.5 + 0.25)
        if x_max - x_min < 1.1 or y_max - y_min < 1.1 or min(abs(v - round(v)) for v in (x_max, y_max)) < 0.012:
            continue
        pixels = [x_min, x_max, y_min, y_max]
        with torch.no_grad():
            for p, v, r in zip((m.x_min, m.x_max, m.y_min, m.y_max), pixels,
                               (m.reparametrization_h, m.reparametrization_h, m.reparametrization_w, m.reparametrization_w)):
                p.fill_(v / r)
        before = [p.detach().clone() for p in m.parameters()]
        x = torch.tensor(rng.random((1, 1, h, w), dtype=np.float32), device="cuda", requires_grad=True)
        go = torch.tensor((rng.random((1, 1, h, w)) < 0.3).astype(np.float32), device="cuda")
        y = m(x)                                    # training mode: clips first
        for a, b in zip(m.parameters(), before):
            assert torch.equal(a.detach(), b), "clip altered the test's box (case %d)" % case
        y.backward(go)

        used = [p.detach().double() * r for p, r in zip(
            (m.x_min, m.x_max, m.y_min, m.y_max),
            (m.reparametrization_h, m.reparametrization_h, m.reparametrization_w, m.reparametrization_w))]
        if not exact:
            used = [torch.ceil(used[0]), torch.floor(used[1]), torch.ceil(used[2]), torch.floor(used[3])]
        xd = x.detach().double().requires_grad_()
        want = dense_boxconv(xd, *used, False)
        if normalize:
            # the reference divides by the area of the box as used (rounded boxes: of the rounded box)
            want = want / ((used[1] - used[0] + 1) * (used[3] - used[2] + 1))
        want_gin, = torch.autograd.grad(want, xd, go.double())
        assert torch.allclose(y.detach().double(), want.detach(), rtol=3e-5, atol=1e-5), case
        assert torch.allclose(x.grad.double(), want_gin, rtol=3e-5, atol=1e-5), case


def test_package_self_test_runs():
    """`python -m box_convolution.test`, the command the reference documents for its own test file."""
    import os
    import subprocess
    import sys
    from conftest import PKG_DIR
    env = dict(os.environ, PYTHONPATH=PKG_DIR + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "box_convolution.test"], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "test_box_convolution_module OK" in r.stdout
