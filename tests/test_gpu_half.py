"""float16 / bfloat16 tensors, through the C ABI entry points that read and write them as they are.

The reference instantiates its kernels for half (`src/box_convolution_cuda_forward.cu:224`,
`src/box_convolution_cuda_backward.cu:176,431`).  Here the 16-bit tensors are converted on chip and
all arithmetic is float, so the check is against the float ORACLE run on the same (already rounded)
inputs and parameters, with a tolerance derived from the one rounding the results get when they are
stored: |ours - ref| <= u |ref| + atol, u = 2^-11 for float16 and 2^-8 for bfloat16 (half an ulp of
the 11- and 8-bit significands), atol = 1e-5 max|ref| for the float noise between two orders of
summation (the bar of the float tests is 1e-4).  Parameter gradients: float sums rounded once,
u |ref| + 1e-3 max|ref|.
"""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

UNIT = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}


@pytest.fixture(scope="module")
def bc():
    import box_convolution
    assert torch.cuda.is_available()
    return box_convolution


def close(got, ref, u, noise):
    got = got.astype(np.float64)
    ref = ref.astype(np.float64)
    return bool((np.abs(got - ref) <= 1.01 * u * np.abs(ref) + noise * np.abs(ref).max() + 1e-7).all())


def rounded(a, dtype):
    """float32 numpy array -> (tensor of `dtype` on the GPU, its values back as float32 numpy)."""
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dtype)
    return t, t.float().cpu().numpy()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape,narrow", [
    ((2, 3, 4, 64, 128), True),      # the 1/8-frame block: unguarded kernels, staged planes
    ((1, 2, 3, 40, 131), True),      # odd sizes: guarded kernels
    ((1, 2, 2, 128, 256), True),     # two tiles per warp, input plane read from global memory
    ((1, 1, 2, 300, 300), False),    # too large for the shared-memory kernels: float copies
])
@pytest.mark.parametrize("normalize,exact", [(True, True), (False, False)])
def test_half_tensors_against_the_float_oracle(bc, dtype, shape, narrow, normalize, exact):
    from box_convolution import _cabi
    N, C, F, h, w = shape
    assert bool(_cabi.lib.bc_boxconv2d_narrow_supported(F, h, w)) == narrow
    rng = np.random.default_rng(h * 7 + w + int(normalize))
    x, x32 = rounded(rng.standard_normal((N, C, h, w)).astype(np.float32), dtype)
    go, go32 = rounded(rng.standard_normal((N, C * F, h, w)).astype(np.float32), dtype)
    lo = 0.3 if exact else 1.2
    cx = rng.uniform(-h / 3, h / 3, (C, F)); ex = rng.uniform(lo, h / 4 + lo, (C, F))
    cy = rng.uniform(-w / 3, w / 3, (C, F)); ey = rng.uniform(lo, w / 4 + lo, (C, F))
    params, pix = [], []
    for a in (cx - ex, cx + ex, cy - ey, cy + ey):
        t, v = rounded(a.astype(np.float32), dtype)
        params.append(t.requires_grad_())
        pix.append(v)
    xt = x.requires_grad_()
    out = bc.BoxConvolutionFunction.apply(xt, *params, 1.0, 1.0, normalize, exact)
    assert out.dtype == dtype and out.shape == (N, C * F, h, w)
    out.backward(go)
    assert xt.grad.dtype == dtype and all(p.grad.dtype == dtype for p in params)

    integ = oracle.integral_image(x32)
    ref_out = oracle.box_convolution_forward(integ, *pix, normalize, exact)
    ref = oracle.box_convolution_backward(integ, *pix, go32, ref_out, 1.0, 1.0, normalize, exact)
    u = UNIT[dtype]
    assert close(out.detach().float().cpu().numpy(), ref_out, u, 1e-5)
    assert close(xt.grad.float().cpu().numpy(), ref[0], u, 1e-5)
    for k in range(4):
        assert close(params[k].grad.float().cpu().numpy(), ref[1 + k], u, 1e-3), k


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_half_module_and_need_mask(bc, dtype):
    """`module.half()` as a user of the reference would write it; gradients only for what requires them."""
    torch.manual_seed(5)
    m = bc.BoxConv2d(4, 4, 64, 128).cuda().to(dtype)
    x = torch.randn(2, 4, 64, 128, device="cuda", dtype=dtype)
    out = m(x)                                         # input does not require grad
    assert out.dtype == dtype
    out.float().square().mean().backward()
    assert all(p.grad is not None and p.grad.dtype == dtype and torch.isfinite(p.grad).all() for p in m.parameters())
    ref = bc.BoxConv2d(4, 4, 64, 128).cuda()
    with torch.no_grad():
        for a, b in zip(ref.parameters(), m.parameters()):
            a.copy_(b.float())
    want = ref(x.float())
    u = UNIT[dtype]
    assert close(out.detach().float().cpu().numpy(), want.detach().cpu().numpy(), u, 1e-5)
    m.eval()
    with torch.no_grad():
        again = m(x)
    assert torch.equal(again, out.detach())
