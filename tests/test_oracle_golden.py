"""The plain-C oracle against the golden fixtures produced by the reference's own CPU code
(tests/golden/make_golden.py).  CPU only."""
import numpy as np

from conftest import max_rel
from oracle import oracle


def test_integral_image_matches_reference_bitwise(golden):
    for i in range(int(golden["ii_count"])):
        got = oracle.integral_image(golden["ii%d_in" % i])
        assert np.array_equal(got, golden["ii%d_out" % i]), i


def test_forward_matches_reference_bitwise(golden):
    for i in range(int(golden["bc_count"])):
        pre = "bc%d_" % i
        N, C, F, h, w, normalize, exact, _ = golden[pre + "meta"]
        integ = oracle.integral_image(golden[pre + "x"])
        out = oracle.box_convolution_forward(integ, *golden[pre + "params"], normalize, exact)
        assert np.array_equal(out, golden[pre + "out"]), i


def test_backward_matches_reference(golden):
    for i in range(int(golden["bc_count"])):
        pre = "bc%d_" % i
        N, C, F, h, w, normalize, exact, _ = golden[pre + "meta"]
        rep_h, rep_w = golden[pre + "rep"]
        integ = oracle.integral_image(golden[pre + "x"])
        res = oracle.box_convolution_backward(
            integ, *golden[pre + "params"], golden[pre + "go"], golden[pre + "out"],
            rep_h, rep_w, normalize, exact)
        # per-filter gathers are bit-equal; only the sum over filters / pixels differs in order
        assert max_rel(res[0], golden[pre + "gin"]) < 2e-6, i
        for k in range(4):
            assert max_rel(res[1 + k], golden[pre + "gparams"][k]) < 2e-5, (i, k)


def test_border_and_integer_boxes_match_reference(golden):
    """Boxes on integer and half-integer coordinates, on the plane's borders and at the clip's limits,
    in all four modes: outputs bit for bit, gradients up to the order of summation."""
    assert int(golden["edge_count"]) == 4
    for i in range(int(golden["edge_count"])):
        pre = "edge%d_" % i
        N, C, F, h, w, normalize, exact = golden[pre + "meta"]
        integ = oracle.integral_image(golden[pre + "x"])
        out = oracle.box_convolution_forward(integ, *golden[pre + "params"], normalize, exact)
        assert np.array_equal(out.reshape(-1), golden[pre + "out"].reshape(-1)), i
        res = oracle.box_convolution_backward(integ, *golden[pre + "params"], golden[pre + "go"],
                                              golden[pre + "out"], 1.0, 1.0, normalize, exact)
        assert max_rel(res[0], golden[pre + "gin"]) < 2e-6, i
        for k in range(4):
            assert max_rel(res[1 + k], golden[pre + "gparams"][k]) < 2e-5, (i, k)


def test_backward_respects_need_mask(golden):
    pre = "bc2_"
    N, C, F, h, w, normalize, exact, _ = golden[pre + "meta"]
    integ = oracle.integral_image(golden[pre + "x"])
    res = oracle.box_convolution_backward(
        integ, *golden[pre + "params"], golden[pre + "go"], golden[pre + "out"], 1.0, 1.0,
        normalize, exact, False, True, False, False, True)
    assert res[0] is None and res[2] is None and res[3] is None
    assert res[1] is not None and res[4] is not None


def test_clip_matches_reference_bitwise(golden):
    for i in range(int(golden["clip_count"])):
        pre = "clip%d_" % i
        C, F, mh, mw, exact = golden[pre + "meta"]
        rep_h, rep_w = golden[pre + "rep"]
        ps = [np.ascontiguousarray(p).copy() for p in golden[pre + "before"]]
        oracle.clip_parameters(*ps, rep_h, rep_w, mh, mw, exact)
        assert np.array_equal(np.stack(ps), golden[pre + "after"]), i
        assert not np.array_equal(np.stack(ps), golden[pre + "before"]), "fixture must exercise the clip"
