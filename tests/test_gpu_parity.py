"""Parity of the CUDA library with the oracle and with the golden fixtures produced by the
reference's own CPU code.  Every call goes through the C ABI (`libboxconv_b200.so`).

Tolerances (max|ours-ref| / max|ref| per tensor): outputs and grad-input 1e-4, parameter
gradients 1e-3, integral image 1e-5 element-wise relative -- the bars of the task; the asserts
below use tighter values where the arithmetic allows.
"""
import numpy as np
import pytest
import torch

from conftest import max_rel
from oracle import oracle
from workloads import CONFIGS, make_workload

pytestmark = pytest.mark.gpu

TOL_OUT, TOL_GIN, TOL_PARAM, TOL_II = 1e-4, 1e-4, 1e-3, 1e-5


@pytest.fixture(scope="module")
def bc():
    import box_convolution
    assert torch.cuda.is_available()
    return box_convolution


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# ------------------------------------------------------------------ integral image
def test_integral_image_golden(bc, golden):
    for i in range(int(golden["ii_count"])):
        got = bc.integral_image(cuda(golden["ii%d_in" % i])).cpu().numpy()
        ref = golden["ii%d_out" % i]
        assert got.shape == ref.shape
        np.testing.assert_allclose(got, ref, rtol=TOL_II, atol=1e-8, err_msg=str(i))


@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (2, 3, 10, 10), (3, 7, 13), (5, 64, 64), (2, 2, 64, 128),
                                   (3, 129, 257), (2, 300, 1000), (1, 40, 2051), (4, 512, 1024), (9, 3)])
def test_integral_image_random(bc, shape):
    rng = np.random.default_rng(sum(shape))
    x = rng.random(shape, dtype=np.float32)
    got = bc.integral_image(cuda(x)).cpu().numpy()
    ref = oracle.integral_image(x)
    np.testing.assert_allclose(got, ref, rtol=TOL_II, atol=1e-8)
    assert (got[..., 0, :] == 0).all() and (got[..., :, 0] == 0).all()


def test_integral_image_noncontiguous_and_unaligned(bc):
    rng = np.random.default_rng(3)
    x = rng.random((4, 6, 20, 36), dtype=np.float32)
    xt = cuda(x)
    got = bc.integral_image(xt[:, ::2, 1:, 2:]).cpu().numpy()          # strided view, made contiguous
    np.testing.assert_allclose(got, oracle.integral_image(x[:, ::2, 1:, 2:]), rtol=TOL_II)
    flat = torch.empty(6 * 20 * 36 + 3, device="cuda")
    view = flat[3:].view(6, 20, 36)                                     # 4-byte aligned only
    view.copy_(xt[0])
    np.testing.assert_allclose(bc.integral_image(view).cpu().numpy(), oracle.integral_image(x[0]), rtol=TOL_II)


def test_integral_image_empty(bc):
    out = bc.integral_image(torch.empty(0, 3, 5, 7, device="cuda"))
    assert out.shape == (0, 3, 6, 8)
    out = bc.integral_image(torch.empty(2, 0, 7, device="cuda"))
    assert out.shape == (2, 1, 8) and (out == 0).all()


# ------------------------------------------------------------------ the four-function interface
def test_four_function_interface_golden(bc, golden):
    for i in range(int(golden["bc_count"])):
        pre = "bc%d_" % i
        N, C, F, h, w, normalize, exact, _ = [int(v) for v in golden[pre + "meta"]]
        rep_h, rep_w = [float(v) for v in golden[pre + "rep"]]
        params = [cuda(p) for p in golden[pre + "params"]]
        integ = bc.integral_image(cuda(golden[pre + "x"]))
        out = bc.box_convolution_forward(integ, *params, bool(normalize), bool(exact))
        assert max_rel(out.cpu().numpy(), golden[pre + "out"]) < 1e-5, i
        res = bc.box_convolution_backward(integ, *params, cuda(golden[pre + "go"]), out, rep_h, rep_w,
                                          bool(normalize), bool(exact), True, True, True, True, True)
        assert max_rel(res[0].cpu().numpy(), golden[pre + "gin"]) < 1e-5, i
        for k in range(4):
            assert max_rel(res[1 + k].cpu().numpy(), golden[pre + "gparams"][k]) < 2e-4, (i, k)


def test_backward_need_mask(bc, golden):
    pre = "bc4_"
    N, C, F, h, w, normalize, exact, _ = [int(v) for v in golden[pre + "meta"]]
    params = [cuda(p) for p in golden[pre + "params"]]
    integ = bc.integral_image(cuda(golden[pre + "x"]))
    go = cuda(golden[pre + "go"])
    rep_h, rep_w = [float(v) for v in golden[pre + "rep"]]
    full = bc.box_convolution_backward(integ, *params, go, torch.empty(0), rep_h, rep_w,
                                       bool(normalize), bool(exact), True, True, True, True, True)
    part = bc.box_convolution_backward(integ, *params, go, torch.empty(0), rep_h, rep_w,
                                       bool(normalize), bool(exact), False, False, True, False, True)
    assert part[0].numel() == 0 and part[1].numel() == 0 and part[3].numel() == 0
    assert torch.equal(part[2], full[2]) and torch.equal(part[4], full[4])
    only_in = bc.box_convolution_backward(integ, *params, go, torch.empty(0), rep_h, rep_w,
                                          bool(normalize), bool(exact), True, False, False, False, False)
    assert all(t.numel() == 0 for t in only_in[1:])
    assert max_rel(only_in[0].cpu().numpy(), full[0].cpu().numpy()) < 1e-6


def test_clip_golden_bitwise(bc, golden):
    for i in range(int(golden["clip_count"])):
        pre = "clip%d_" % i
        C, F, mh, mw, exact = [int(v) for v in golden[pre + "meta"]]
        rep_h, rep_w = [float(v) for v in golden[pre + "rep"]]
        ps = [cuda(p) for p in golden[pre + "before"]]
        bc.clip_parameters(*ps, rep_h, rep_w, mh, mw, bool(exact))
        got = np.stack([p.cpu().numpy() for p in ps])
        assert np.array_equal(got, golden[pre + "after"]), i


def test_clip_packed_equals_clip_plus_copy(bc, golden):
    from box_convolution import ext
    for i in range(int(golden["clip_count"])):
        pre = "clip%d_" % i
        C, F, mh, mw, exact = [int(v) for v in golden[pre + "meta"]]
        rep_h, rep_w = [float(v) for v in golden[pre + "rep"]]
        ps = [cuda(p) for p in golden[pre + "before"]]
        packed = ext.clip_parameters_packed(*ps, rep_h, rep_w, mh, mw, bool(exact))
        assert packed.shape == (4, C, F)
        assert np.array_equal(packed.cpu().numpy(), golden[pre + "after"]), i
        assert np.array_equal(np.stack([p.cpu().numpy() for p in ps]), golden[pre + "after"]), i


def test_backward_uses_the_parameters_of_its_own_forward(bc):
    """The reference saves copies of the parameters at forward time.  Changing the module's parameters
    between forward and backward (a second forward that clips, an optimizer step, eval()) must not
    change the gradients of the first forward."""
    wl = make_workload("cfg1", batch=2, planes=4)
    want = run_module(bc, wl.x, wl.stored, wl.grad_output, wl.max_h, wl.max_w, 8, True, True)
    for train in (True, False):
        C, F = wl.stored[0].shape
        m = bc.BoxConv2d(C, F, wl.max_h, wl.max_w, reparametrization_factor=8).cuda()
        with torch.no_grad():
            for p, v in zip((m.x_min, m.x_max, m.y_min, m.y_max), wl.stored):
                p.copy_(cuda(v))
        m.train(train)
        xt = cuda(wl.x).requires_grad_()
        out = m(xt)
        for p in (m.x_min, m.x_max, m.y_min, m.y_max):
            p.data.mul_(0.5)                                # no version bump, like the module's own clip
        out.backward(cuda(wl.grad_output))
        assert np.array_equal(xt.grad.cpu().numpy(), want[1])
        for p, g in zip((m.x_min, m.x_max, m.y_min, m.y_max), want[2]):
            assert np.array_equal(p.grad.cpu().numpy(), g)


# ------------------------------------------------------------------ module / autograd Function
def run_module(bc, x, stored, go, max_h, max_w, factor, normalize, exact, train=True):
    C, F = stored[0].shape
    m = bc.BoxConv2d(C, F, max_h, max_w, reparametrization_factor=factor, normalize=normalize).cuda()
    m.exact = exact
    with torch.no_grad():
        for p, v in zip((m.x_min, m.x_max, m.y_min, m.y_max), stored):
            p.copy_(cuda(v))
    m.train(train)
    xt = cuda(x).requires_grad_()
    out = m(xt)
    out.backward(cuda(go))
    return (out.detach().cpu().numpy(), xt.grad.cpu().numpy(),
            [p.grad.cpu().numpy() for p in (m.x_min, m.x_max, m.y_min, m.y_max)], m)


def test_function_golden(bc, golden):
    for i in range(int(golden["bc_count"])):
        pre = "bc%d_" % i
        N, C, F, h, w, normalize, exact, _ = [int(v) for v in golden[pre + "meta"]]
        rep_h, rep_w = [float(v) for v in golden[pre + "rep"]]
        # stored = pixels / rep would not round-trip bit-exactly; call the Function with rep = 1
        # on pixel parameters and scale the parameter gradients like the reference does
        params = [cuda(p).requires_grad_() for p in golden[pre + "params"]]
        x = cuda(golden[pre + "x"]).requires_grad_()
        out = bc.BoxConvolutionFunction.apply(x, *params, 1.0, 1.0, bool(normalize), bool(exact))
        out.backward(cuda(golden[pre + "go"]))
        assert max_rel(out.detach().cpu().numpy(), golden[pre + "out"]) < 1e-5, i
        assert max_rel(x.grad.cpu().numpy(), golden[pre + "gin"]) < 1e-5, i
        for k, rep in enumerate((rep_h, rep_h, rep_w, rep_w)):
            assert max_rel(params[k].grad.cpu().numpy() * np.float32(rep), golden[pre + "gparams"][k]) < 2e-4, (i, k)


def test_function_golden_border_and_integer_boxes(bc, golden):
    """The reference's own results for boxes on integer and half-integer coordinates and on the
    plane's borders (fixtures `edge*`, all four modes)."""
    assert int(golden["edge_count"]) == 4
    for i in range(int(golden["edge_count"])):
        pre = "edge%d_" % i
        N, C, F, h, w, normalize, exact = [int(v) for v in golden[pre + "meta"]]
        params = [cuda(p).requires_grad_() for p in golden[pre + "params"]]
        x = cuda(golden[pre + "x"]).requires_grad_()
        out = bc.BoxConvolutionFunction.apply(x, *params, 1.0, 1.0, bool(normalize), bool(exact))
        out.backward(cuda(golden[pre + "go"]))
        assert out.shape == (N, C * F, h, w)
        assert max_rel(out.detach().cpu().numpy(), golden[pre + "out"].reshape(N, C * F, h, w)) < 1e-5, i
        assert max_rel(x.grad.cpu().numpy(), golden[pre + "gin"]) < 1e-5, i
        for k in range(4):
            assert max_rel(params[k].grad.cpu().numpy(), golden[pre + "gparams"][k]) < 2e-4, (i, k)


@pytest.mark.parametrize("cfg", ["cfg1", "cfg2"])
def test_module_full_config_vs_oracle(bc, cfg):
    wl = make_workload(cfg)
    out, gin, gps, m = run_module(bc, wl.x, wl.stored, wl.grad_output, wl.max_h, wl.max_w, 8,
                                  True, True)
    # training-mode clip must be the identity for these boxes
    for p, v in zip((m.x_min, m.x_max, m.y_min, m.y_max), wl.stored):
        assert np.array_equal(p.detach().cpu().numpy(), v)
    ref_out, ref_gin, ref_gps = oracle.boxconv2d_forward_backward(
        wl.x, wl.stored, wl.grad_output, wl.rep_h, wl.rep_w, True, True)
    assert max_rel(out, ref_out) < TOL_OUT
    assert max_rel(gin, ref_gin) < TOL_GIN
    for k in range(4):
        assert max_rel(gps[k], ref_gps[k]) < TOL_PARAM, k


def test_module_cfg3_subset_vs_oracle(bc):
    wl = make_workload("cfg3", batch=1, planes=4)
    out, gin, gps, _ = run_module(bc, wl.x, wl.stored, wl.grad_output, wl.max_h, wl.max_w, 8, True, True)
    ref_out, ref_gin, ref_gps = oracle.boxconv2d_forward_backward(
        wl.x, wl.stored, wl.grad_output, wl.rep_h, wl.rep_w, True, True)
    assert max_rel(out, ref_out) < TOL_OUT
    assert max_rel(gin, ref_gin) < TOL_GIN
    for k in range(4):
        assert max_rel(gps[k], ref_gps[k]) < TOL_PARAM, k


@pytest.mark.parametrize("normalize,exact", [(True, True), (False, True), (True, False), (False, False)])
@pytest.mark.parametrize("shape", [(2, 3, 2, 9, 11), (1, 2, 4, 33, 70), (3, 1, 1, 1, 1), (1, 5, 3, 64, 4),
                                   (2, 2, 3, 40, 131), (1, 2, 2, 128, 128), (1, 1, 2, 96, 200),
                                   (1, 1, 1, 200, 300),
                                   # whole-plane backward with the input read from global memory
                                   (1, 2, 2, 128, 256), (1, 1, 2, 125, 250),
                                   # planes beyond the whole-plane kernels: column bands (guarded and
                                   # unguarded), bands forward with the general backward, general both
                                   (1, 2, 2, 203, 301), (2, 1, 3, 264, 96), (1, 1, 2, 600, 20), (1, 1, 1, 1100, 12)])
def test_module_random_shapes_vs_oracle(bc, shape, normalize, exact):
    N, C, F, h, w = shape
    rng = np.random.default_rng(h * 1000 + w + 7 * int(normalize) + 13 * int(exact))
    x = rng.standard_normal((N, C, h, w)).astype(np.float32)
    go = rng.standard_normal((N, C * F, h, w)).astype(np.float32)
    lo = 0.3 if exact else 1.2
    cx = rng.uniform(-h, h, (C, F)); ex = rng.uniform(lo, h / 2 + lo, (C, F))
    cy = rng.uniform(-w, w, (C, F)); ey = rng.uniform(lo, w / 2 + lo, (C, F))
    pix = [a.astype(np.float32) for a in (cx - ex, cx + ex, cy - ey, cy + ey)]
    outside = h > 1 and C * F > 1
    if outside:
        pix[0][0, 0], pix[1][0, 0] = -3.0 * h, -2.0 * h     # a box wholly outside the image
    params = [cuda(p).requires_grad_() for p in pix]
    xt = cuda(x).requires_grad_()
    out = bc.BoxConvolutionFunction.apply(xt, *params, 1.0, 1.0, normalize, exact)
    out.backward(cuda(go))
    integ = oracle.integral_image(x)
    ref_out = oracle.box_convolution_forward(integ, *pix, normalize, exact)
    ref = oracle.box_convolution_backward(integ, *pix, go, ref_out, 1.0, 1.0, normalize, exact)
    assert max_rel(out.detach().cpu().numpy(), ref_out) < TOL_OUT
    assert max_rel(xt.grad.cpu().numpy(), ref[0]) < TOL_GIN
    for k in range(4):
        assert max_rel(params[k].grad.cpu().numpy(), ref[1 + k]) < TOL_PARAM, k
    if outside:
        assert (out.detach().view(N, C, F, h, w)[:, 0, 0] == 0).all()


@pytest.mark.parametrize("normalize,exact", [(True, True), (False, True), (True, False), (False, False)])
@pytest.mark.parametrize("shape", [(2, 2, 8, 64, 128), (1, 1, 8, 40, 131), (1, 1, 8, 203, 301)])
def test_boxes_on_integer_coordinates_and_plane_borders_vs_oracle(bc, shape, normalize, exact):
    """Box edges whose fractional part is exactly zero or one half, boxes that end exactly on the
    plane's border or one pixel beyond it, one-pixel boxes, and a box as large as the clip allows:
    the cases in which ceil/floor of an edge coincide with the edge (`src/box_convolution.cpp:14-40`)
    and in which tap rows and columns are clamped on one side only."""
    N, C, F, h, w = shape
    rng = np.random.default_rng(h + w + 3 * int(normalize) + 5 * int(exact))
    x = rng.standard_normal((N, C, h, w)).astype(np.float32)
    go = rng.standard_normal((N, C * F, h, w)).astype(np.float32)
    boxes = [                                    # (x_min, x_max, y_min, y_max) in pixels
        (-2.0, 3.0, -4.0, 1.0),                  # integers
        (-1.5, 2.5, 0.5, 6.5),                   # half-integers
        (0.0, 0.0, 0.0, 0.0) if exact else (0.0, 1.0, 0.0, 1.0),     # the smallest box
        (-(h - 1.0), 0.0, -(w - 1.0), 0.0),      # reaches exactly the first row / column from the last pixel
        (0.0, h - 1.0, 0.0, w - 1.0),            # reaches exactly the last row / column from the first pixel
        (-float(h), h - 2.0, -float(w), w - 2.0),    # one pixel beyond the border on the low side
        (-(h + 1.0), h - 1.0, -(w + 1.0), w - 1.0),  # the clip's limits
        (3.0, 7.25, -9.75, -2.0),                # integer on one side, fraction on the other
    ]
    pix = [np.empty((C, F), np.float32) for _ in range(4)]
    for c in range(C):
        for f in range(F):
            for k in range(4):
                pix[k][c, f] = boxes[(f + c) % len(boxes)][k]
    params = [cuda(p).requires_grad_() for p in pix]
    xt = cuda(x).requires_grad_()
    out = bc.BoxConvolutionFunction.apply(xt, *params, 1.0, 1.0, normalize, exact)
    out.backward(cuda(go))
    integ = oracle.integral_image(x)
    ref_out = oracle.box_convolution_forward(integ, *pix, normalize, exact)
    ref = oracle.box_convolution_backward(integ, *pix, go, ref_out, 1.0, 1.0, normalize, exact)
    assert max_rel(out.detach().cpu().numpy(), ref_out) < TOL_OUT
    assert max_rel(xt.grad.cpu().numpy(), ref[0]) < TOL_GIN
    for k in range(4):
        assert max_rel(params[k].grad.cpu().numpy(), ref[1 + k]) < TOL_PARAM, k


def test_module_empty_batch_and_strided_inputs(bc):
    """A batch of zero samples gives an empty output and zero parameter gradients; inputs and
    grad_outputs that are views with strides (channel slices, transposes) give the same results as
    their contiguous copies."""
    torch.manual_seed(3)
    m = bc.BoxConv2d(3, 2, 16, 24).cuda()
    x0 = torch.empty(0, 3, 16, 24, device="cuda", requires_grad=True)
    y0 = m(x0)
    assert y0.shape == (0, 6, 16, 24)
    y0.backward(torch.empty_like(y0))
    for p in m.parameters():
        assert p.grad is not None and (p.grad == 0).all()
        p.grad = None

    big = torch.randn(2, 5, 16, 48, device="cuda")
    view = big[:, 1:4, :, ::2]                       # strided in channels and columns
    assert not view.is_contiguous()
    xa = view.detach().requires_grad_()
    xb = view.detach().contiguous().requires_grad_()
    go_big = torch.randn(2, 16, 24, 6, device="cuda")
    go = go_big.permute(0, 3, 1, 2)                  # (2, 6, 16, 24), not contiguous
    m.eval()
    ya, yb = m(xa), m(xb)
    assert torch.equal(ya, yb)
    ya.backward(go)
    ga = [p.grad.clone() for p in m.parameters()]
    for p in m.parameters():
        p.grad = None
    yb.backward(go.contiguous())
    assert torch.equal(xa.grad, xb.grad)
    for a, p in zip(ga, m.parameters()):
        assert torch.equal(a, p.grad)


def test_many_filters_take_the_general_path(bc):
    """More filters than the per-CTA tap table holds: the module falls back to the kernels that
    read integral images from global memory; results must not change."""
    rng = np.random.default_rng(4)
    N, C, F, h, w = 1, 2, 33, 16, 20
    x = rng.standard_normal((N, C, h, w)).astype(np.float32)
    go = rng.standard_normal((N, C * F, h, w)).astype(np.float32)
    cx = rng.uniform(-h / 2, h / 2, (C, F)); ex = rng.uniform(0.6, h / 3, (C, F))
    cy = rng.uniform(-w / 2, w / 2, (C, F)); ey = rng.uniform(0.6, w / 3, (C, F))
    pix = [a.astype(np.float32) for a in (cx - ex, cx + ex, cy - ey, cy + ey)]
    params = [cuda(p).requires_grad_() for p in pix]
    xt = cuda(x).requires_grad_()
    out = bc.BoxConvolutionFunction.apply(xt, *params, 1.0, 1.0, True, True)
    out.backward(cuda(go))
    integ = oracle.integral_image(x)
    ref_out = oracle.box_convolution_forward(integ, *pix, True, True)
    ref = oracle.box_convolution_backward(integ, *pix, go, ref_out, 1.0, 1.0, True, True)
    assert max_rel(out.detach().cpu().numpy(), ref_out) < TOL_OUT
    assert max_rel(xt.grad.cpu().numpy(), ref[0]) < TOL_GIN
    for k in range(4):
        assert max_rel(params[k].grad.cpu().numpy(), ref[1 + k]) < TOL_PARAM, k


def test_eval_mode_clips_once_and_matches(bc):
    wl = make_workload("cfg1", batch=2)
    m = bc.BoxConv2d(16, 4, 64, 64).cuda()
    with torch.no_grad():
        m.x_min.fill_(0.2)
        m.x_max.fill_(0.1)        # negative size: the clip must repair it
    m.eval()
    assert (m.x_max > m.x_min).all()
    with torch.no_grad():
        y = m(cuda(wl.x))
    assert y.shape == (2, 64, 64, 64) and torch.isfinite(y).all()


# ------------------------------------------------------------------ size-independent properties
@pytest.mark.parametrize("cfg", ["cfg2", "cfg3"])
def test_adjointness_and_linearity_full_size(bc, cfg):
    """<grad_output, forward(x)> == <grad_input, x> (the gather and its mirrored-box adjoint),
    forward is linear in x, and two runs are bit-identical (no atomics anywhere)."""
    wl = make_workload(cfg)
    stored = [cuda(p) for p in wl.stored]
    x = cuda(wl.x).requires_grad_()
    go = cuda(wl.grad_output)

    def fwd(t):
        return bc.BoxConvolutionFunction.apply(t, *stored, wl.rep_h, wl.rep_w, True, True)

    out = fwd(x)
    out.backward(go)
    lhs = (out.detach().double() * go.double()).sum().item()
    rhs = (x.grad.double() * x.detach().double()).sum().item()
    scale = (out.detach().double().abs() * go.double().abs()).sum().item()
    assert abs(lhs - rhs) < 1e-5 * scale
    with torch.no_grad():
        out2 = fwd(x.detach() * 2.0)
        assert max_rel(out2.cpu().numpy(), (2.0 * out.detach()).cpu().numpy()) < 1e-6
        out3 = fwd(x.detach())
        assert torch.equal(out3, out.detach())
    g1 = x.grad.clone()
    x.grad = None
    fwd(x).backward(go)
    assert torch.equal(g1, x.grad)


def test_batch_shards_reproduce_the_full_batch(bc):
    """What data-parallel ranks compute: outputs and grad-input of a shard are bitwise the slices of
    the full-batch result, and the shards' parameter gradients add up to the full-batch gradient."""
    wl = make_workload("cfg2", batch=8, planes=8)
    full_out, full_gin, full_gps, _ = run_module(bc, wl.x, wl.stored, wl.grad_output, wl.max_h, wl.max_w, 8, True, True)
    sums = [np.zeros_like(g, dtype=np.float64) for g in full_gps]
    for lo, hi in ((0, 3), (3, 8)):                     # uneven shards
        out, gin, gps, _ = run_module(bc, wl.x[lo:hi], wl.stored, wl.grad_output[lo:hi], wl.max_h, wl.max_w, 8,
                                      True, True)
        assert np.array_equal(out, full_out[lo:hi])
        assert np.array_equal(gin, full_gin[lo:hi])
        for s, g in zip(sums, gps):
            s += g
    for s, g in zip(sums, full_gps):
        assert max_rel(s, g) < 1e-5


def test_parameter_gradients_match_finite_differences(bc):
    """The method of the reference's own test (box_convolution/test.py:276-309): central
    differences of the loss w.r.t. each stored parameter, on a small smooth case."""
    rng = np.random.default_rng(11)
    N, C, F, h, w = 2, 2, 2, 9, 8
    x = cuda(rng.standard_normal((N, C, h, w)).astype(np.float32))
    go = cuda(rng.standard_normal((N, C * F, h, w)).astype(np.float32))
    pix = [np.array(a, np.float32) for a in (
        [[-2.37, -0.61], [1.44, -3.3]], [[1.58, 2.42], [3.71, 0.36]],
        [[-1.29, 0.55], [-2.63, -3.45]], [[2.31, 3.62], [0.38, 1.71]])]
    for normalize in (True, False):
        params = [cuda(p).requires_grad_() for p in pix]
        out = bc.BoxConvolutionFunction.apply(x, *params, 1.0, 1.0, normalize, True)
        out.backward(go)
        eps = 0.01
        for k in range(4):
            for idx in [(0, 0), (1, 1)]:
                vals = []
                for sgn in (+1, -1):
                    pp = [cuda(p.copy()) for p in pix]
                    pp[k][idx] += sgn * eps
                    with torch.no_grad():
                        o = bc.BoxConvolutionFunction.apply(x, *pp, 1.0, 1.0, normalize, True)
                    vals.append((o.double() * go.double()).sum().item())
                fd = (vals[0] - vals[1]) / (2 * eps)
                an = params[k].grad[idx].item()
                assert abs(fd - an) < 2e-2 * max(1.0, abs(fd)), (normalize, k, idx, fd, an)


def test_errors_are_loud(bc):
    with pytest.raises(RuntimeError):
        bc.integral_image(torch.zeros(3, 4))                      # CPU tensor: no fallback
    with pytest.raises(RuntimeError):
        bc.integral_image(torch.zeros(4, device="cuda"))          # < 2 dims
    integ = torch.zeros(1, 2, 5, 5, device="cuda")
    p = torch.zeros(3, 2, device="cuda")
    with pytest.raises(RuntimeError):
        bc.box_convolution_forward(integ, p, p, p, p, True, True)  # rows != channels
    with pytest.raises(RuntimeError):
        bc.BoxConv2d(2, 2, 8, 8)(torch.zeros(1, 2, 8, 8))          # module on CPU


@pytest.mark.parametrize("cfg,batch,planes,chunks", [("cfg2", 5, 6, 3), ("cfg1", 4, 3, 8), ("cfg3", 2, 2, 2)])
def test_host_pipeline_matches_device_step(bc, cfg, batch, planes, chunks):
    """bc_boxconv2d_host_step (pinned host buffers in and out, chunked) against the module run on
    device tensors, and against the oracle."""
    wl = make_workload(cfg, batch=batch, planes=planes)
    N, C, F, h, w = wl.shape
    out, gin, gps, m = run_module(bc, wl.x, wl.stored, wl.grad_output, wl.max_h, wl.max_w, 8, True, True)
    pipe = bc.HostPipeline(m, N, h, w, chunks=chunks)
    hx = torch.from_numpy(wl.x).pin_memory()
    hgo = torch.from_numpy(wl.grad_output).pin_memory()
    hout = torch.empty((N, C * F, h, w)).pin_memory()
    hgin = torch.empty((N, C, h, w)).pin_memory()
    hgp = torch.empty((4, C, F)).pin_memory()
    for _ in range(2):                      # the second call reuses the workspace
        hout.fill_(float("nan")); hgin.fill_(float("nan")); hgp.fill_(float("nan"))
        pipe.step(hx, hgo, hout, hgin, hgp)
        assert np.array_equal(hout.numpy(), out)          # per-sample results do not depend on chunking
        assert np.array_equal(hgin.numpy(), gin)
        for k in range(4):
            assert max_rel(hgp[k].numpy(), gps[k]) < 1e-5, k


def test_host_pipeline_batches_in_flight(bc):
    """submit/wait with two batches in flight on alternating workspaces: five different batches
    in a row, each compared with the module run on device tensors."""
    base = make_workload("cfg2", batch=4, planes=5)
    N, C, F, h, w = base.shape
    rng = np.random.default_rng(77)
    batches = [(rng.standard_normal(base.x.shape).astype(np.float32),
                rng.standard_normal(base.grad_output.shape).astype(np.float32)) for _ in range(5)]
    want = []
    m = None
    for x, go in batches:
        out, gin, gps, m = run_module(bc, x, base.stored, go, base.max_h, base.max_w, 8, True, True)
        want.append((out, gin, gps))
    pipe = bc.HostPipeline(m, N, h, w, chunks=2, depth=2)
    host_in = [(torch.from_numpy(x).pin_memory(), torch.from_numpy(go).pin_memory()) for x, go in batches]
    host_out = [(torch.empty((N, C * F, h, w)).pin_memory(), torch.empty((N, C, h, w)).pin_memory(),
                 torch.empty((4, C, F)).pin_memory()) for _ in batches]
    tickets = []
    for i, (hx, hgo) in enumerate(host_in):
        if i >= 2:
            pipe.wait(tickets[i - 2])
        tickets.append(pipe.submit(hx, hgo, *host_out[i]))
    with pytest.raises(RuntimeError):
        pipe.submit(*host_in[0], *host_out[0])            # a third batch in flight is refused
    for t in tickets:
        pipe.wait(t)
    for (hout, hgin, hgp), (out, gin, gps) in zip(host_out, want):
        assert np.array_equal(hout.numpy(), out)
        assert np.array_equal(hgin.numpy(), gin)
        for k in range(4):
            assert max_rel(hgp[k].numpy(), gps[k]) < 1e-5, k


def test_no_bounded_wait_expired(bc):
    """Runs last in this file: the asynchronous plane copies of the staged kernels all completed."""
    from box_convolution import _cabi
    wl = make_workload("cfg2", batch=2)
    run_module(bc, wl.x, wl.stored, wl.grad_output, wl.max_h, wl.max_w, 8, True, True)
    assert _cabi.wait_timeouts() == 0
