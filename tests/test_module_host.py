"""Host-side behaviour of the BoxConv2d module that needs no GPU: constructor fields, parameter
names/shapes/units (checkpoint compatibility with the reference), the initialisation draw, the
box plot, and the refusal to compute on CPU tensors."""
import random

import numpy as np
import pytest
import torch

import box_convolution as bc


def test_fields_and_state_dict_layout():
    m = bc.BoxConv2d(3, 5, 40, 60, reparametrization_factor=4, normalize=False)
    assert (m.in_planes, m.num_filters, m.max_input_h, m.max_input_w) == (3, 5, 40, 60)
    assert (m.reparametrization_h, m.reparametrization_w) == (160, 240)
    assert m.exact is True and m.normalize is False
    sd = m.state_dict()
    assert list(sd.keys()) == ["x_min", "x_max", "y_min", "y_max"]
    assert all(v.shape == (3, 5) and v.dtype == torch.float32 for v in sd.values())
    m2 = bc.BoxConv2d(3, 5, 40, 60, reparametrization_factor=4)
    m2.load_state_dict(sd)
    assert all(torch.equal(a, b) for a, b in zip(m.parameters(), m2.parameters()))
    with pytest.raises(AssertionError):
        bc.BoxConv2d(1, 1, 8, 8, stride_h=2)


def test_reset_parameters_follows_the_reference_draw(golden):
    """The stored parameters of a freshly constructed module equal, bit for bit, those of the
    reference's own BoxConv2d built under the same `random.seed` (fixtures written by
    tests/golden/make_golden.py from box_convolution/box_convolution_module.py:69-97)."""
    for i in range(int(golden["reset_count"])):
        C, F, mh, mw, seed = [int(v) for v in golden["reset%d_meta" % i]]
        random.seed(seed)
        m = bc.BoxConv2d(C, F, mh, mw, reparametrization_factor=float(golden["reset%d_factor" % i]))
        got = np.stack([p.detach().numpy() for p in (m.x_min, m.x_max, m.y_min, m.y_max)])
        assert np.array_equal(got, golden["reset%d_params" % i]), i
    random.seed(123)
    pix = bc.BoxConv2d(2, 3, 64, 128).get_actual_parameters()
    assert all((b - a >= 2.99).all() for a, b in ((pix[0], pix[1]), (pix[2], pix[3])))   # min size 2 * 1.5


def test_reparametrize_round_trip_and_inplace():
    ps = [torch.rand(2, 2) for _ in range(4)]
    scaled = bc.reparametrize(*ps, 512, 1024, inverse=True)
    assert torch.equal(scaled[0], ps[0] * 512) and torch.equal(scaled[3], ps[3] * 1024)
    back = bc.reparametrize(*scaled, 512, 1024)
    assert all(torch.allclose(a, b) for a, b in zip(back, ps))
    clones = [p.clone() for p in ps]
    assert bc.reparametrize(*clones, 512, 1024, inplace=True, inverse=True) is None
    assert torch.equal(clones[1], ps[1] * 512)


def test_draw_boxes():
    random.seed(5)
    m = bc.BoxConv2d(4, 2, 32, 32)
    img = m.draw_boxes(resolution=(200, 300))
    assert img.shape == (200, 300, 3) and img.dtype == np.uint8
    assert (img[100].max(axis=1) > 0).all() and (img[:, 150].max(axis=1) > 0).all()   # centre cross
    assert (img.reshape(-1, 3).max(axis=1) > 70).sum() > 50                    # some box outlines
    one = m.draw_boxes(channels=[1], weights=torch.tensor([[1.0, 0.0]]))
    assert one.shape == (600, 600, 3)


def test_cpu_tensors_are_refused_everywhere():
    m = bc.BoxConv2d(2, 2, 8, 8)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        m(torch.zeros(1, 2, 8, 8))
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        m.eval()
    p = torch.zeros(2, 2)
    with pytest.raises(RuntimeError):
        bc.BoxConvolutionFunction.apply(torch.zeros(1, 2, 8, 8), p, p, p, p, 8.0, 8.0, True, True)
    with pytest.raises(RuntimeError):
        bc.box_convolution_backward(torch.zeros(1, 2, 9, 9), p, p, p, p, torch.zeros(1, 4, 8, 8),
                                    torch.empty(0), 1.0, 1.0, True, True, True, True, True, True, True)
