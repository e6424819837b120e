"""Generates the golden fixtures in this folder by running the REFERENCE's own CPU code.

The reference's compiled module (built from its sources by ``oracle/build_ref.py`` into
``oracle/_ref/``) is called here through the same four functions its autograd Function uses
(``src/bind.cpp:29-34``): ``integral_image``, ``box_convolution_forward``,
``box_convolution_backward``, ``clip_parameters``.  Inputs are seeded; inputs and the reference's
outputs are stored together in ``boxconv_golden.npz`` so the fixtures can be checked on machines
that have neither the reference checkout nor its build.

The initial box draw of the reference's ``BoxConv2d`` module (Python's ``random``, its
``reset_parameters``) is stored as well, for two seeded constructions of the reference's own class.

Run from the repository root, on a machine that has the reference checkout (its path in
BOXCONV_REFERENCE, or a folder ``reference`` beside the repository):
    python oracle/build_ref.py && python tests/golden/make_golden.py
"""
import importlib.util
import random
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import build_ref  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "boxconv_golden.npz")


def draw_boxes(rng, C, F, h, w, far_outside=False, integer_coords=False):
    """Box parameters in actual pixels; no coordinate within 0.012 of an integer unless asked
    for (the operator is not smooth there: box_convolution/test.py:223-230)."""
    def axis(size):
        centre = rng.uniform(-size / 2, size / 2, (C, F))
        half = rng.uniform(0.6, max(1.0, size / 3), (C, F))
        return centre - half, centre + half

    while True:
        x_min, x_max = axis(h)
        y_min, y_max = axis(w)
        if far_outside:
            x_min[0, 0], x_max[0, 0] = -h - 3.3, -h + 0.4          # box entirely above the image
            y_min[-1, -1], y_max[-1, -1] = w - 0.7, w + 4.2        # box almost entirely to the right
            if C * F > 2:
                x_min[0, -1], x_max[0, -1] = -2 * h - 0.5, 2 * h + 0.5  # taller than the image
        ps = [p.astype(np.float32) for p in (x_min, x_max, y_min, y_max)]
        if integer_coords:
            ps = [np.round(p) for p in ps]
            ps[1] = np.maximum(ps[1], ps[0] + 1)
            ps[3] = np.maximum(ps[3], ps[2] + 1)
            return ps
        if all((np.abs(p - np.round(p)) > 0.012).all() for p in ps):
            return ps


def border_boxes(h, w, exact):
    """(x_min, x_max, y_min, y_max) in pixels: edges with fractional part 0 or 1/2, boxes ending on
    the plane's border or one pixel beyond it, the smallest box, the largest the clip allows."""
    return [
        (-2.0, 3.0, -4.0, 1.0),
        (-1.5, 2.5, 0.5, 6.5),
        (0.0, 0.0, 0.0, 0.0) if exact else (0.0, 1.0, 0.0, 1.0),
        (-(h - 1.0), 0.0, -(w - 1.0), 0.0),
        (0.0, h - 1.0, 0.0, w - 1.0),
        (-float(h), h - 2.0, -float(w), w - 2.0),
        (-(h + 1.0), h - 1.0, -(w + 1.0), w - 1.0),
        (3.0, 7.25, -9.75, -2.0),
    ]


def reference_package(ref_ext):
    """The reference's Python package, imported under another name (ours is called the same), with
    its compiled module name bound to the CPU build."""
    root = build_ref.reference_root()
    if root is None:
        raise SystemExit("no reference checkout: set BOXCONV_REFERENCE")
    sys.modules["box_convolution_cpp_cuda"] = ref_ext
    pkg_dir = os.path.join(root, "box_convolution")
    spec = importlib.util.spec_from_file_location("reference_box_convolution", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["reference_box_convolution"] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = build_ref.load_ref()
    if ref is None:
        raise SystemExit("build the reference first: python oracle/build_ref.py")
    rng = np.random.default_rng(20240607)
    blob = {}

    # ---- integral image: shapes of the reference's own test (box_convolution/test.py:40-46) and a few wider
    ii_shapes = [(1, 1, 2, 2), (2, 3, 5, 9), (3, 1, 10, 3), (1, 2, 7, 10), (2, 2, 1, 6), (1, 1, 33, 70), (4, 17, 40)]
    blob["ii_count"] = np.int64(len(ii_shapes))
    for i, shp in enumerate(ii_shapes):
        x = rng.random(shp, dtype=np.float32)
        blob["ii%d_in" % i] = x
        blob["ii%d_out" % i] = ref.integral_image(torch.from_numpy(x)).numpy()

    # ---- the operator: (N, C, F, h, w, normalize, exact, far_outside, integer_coords)
    cases = [
        (1, 1, 1, 5, 6, True, True, False, False),
        (1, 1, 1, 9, 4, False, True, False, False),
        (2, 3, 2, 8, 11, True, True, True, False),
        (2, 3, 2, 8, 11, False, True, True, False),
        (1, 2, 4, 13, 7, True, True, True, False),
        (3, 2, 3, 2, 2, True, True, False, False),
        (1, 4, 4, 16, 24, True, True, True, False),
        (2, 2, 2, 10, 10, True, False, False, False),
        (2, 2, 2, 10, 10, False, False, True, False),
        (1, 3, 2, 12, 9, True, True, False, True),
        (1, 1, 5, 31, 33, True, True, True, False),
    ]
    blob["bc_count"] = np.int64(len(cases))
    for i, (N, C, F, h, w, normalize, exact, far, integer) in enumerate(cases):
        x = rng.standard_normal((N, C, h, w)).astype(np.float32)
        go = rng.standard_normal((N, C * F, h, w)).astype(np.float32)
        params = draw_boxes(rng, C, F, h, w, far, integer)
        rep_h, rep_w = float(rng.uniform(0.5, 5.0) * h), float(rng.uniform(0.5, 5.0) * w)
        tp = [torch.from_numpy(p) for p in params]
        integ = ref.integral_image(torch.from_numpy(x))
        out = ref.box_convolution_forward(integ, *tp, normalize, exact)
        res = ref.box_convolution_backward(
            integ, *tp, torch.from_numpy(go), out if normalize else torch.empty(0),
            rep_h, rep_w, normalize, exact, True, True, True, True, True)
        pre = "bc%d_" % i
        blob[pre + "meta"] = np.array([N, C, F, h, w, int(normalize), int(exact), int(integer)], np.int64)
        blob[pre + "rep"] = np.array([rep_h, rep_w], np.float64)
        blob[pre + "x"] = x
        blob[pre + "go"] = go
        blob[pre + "params"] = np.stack(params)
        blob[pre + "out"] = out.numpy()
        blob[pre + "gin"] = res[0].numpy()
        blob[pre + "gparams"] = np.stack([r.numpy() for r in res[1:]])

    # ---- clip_parameters, on stored (reparametrized) values, both modes
    clip_cases = [(3, 4, 16, 24, 8.0, True), (2, 5, 64, 128, 8.0, False), (4, 4, 10, 10, 0.7, True)]
    blob["clip_count"] = np.int64(len(clip_cases))
    for i, (C, F, mh, mw, factor, exact) in enumerate(clip_cases):
        rep_h, rep_w = mh * factor, mw * factor
        stored = [rng.uniform(-2.5, 2.5, (C, F)).astype(np.float32) * np.float32(s)
                  for s in (mh / rep_h, mh / rep_h, mw / rep_w, mw / rep_w)]
        stored[1][0, 0] = stored[0][0, 0] - np.float32(0.01)    # negative size
        stored[3][0, 1] = stored[2][0, 1]                       # zero size
        before = np.stack(stored)
        tp = [torch.from_numpy(p.copy()) for p in stored]
        ref.clip_parameters(*tp, rep_h, rep_w, float(mh), float(mw), exact)
        pre = "clip%d_" % i
        blob[pre + "meta"] = np.array([C, F, mh, mw, int(exact)], np.int64)
        blob[pre + "rep"] = np.array([rep_h, rep_w], np.float64)
        blob[pre + "before"] = before
        blob[pre + "after"] = np.stack([t.numpy() for t in tp])

    # ---- the module's initial draw (box_convolution/box_convolution_module.py:69-97), stored values
    pkg = reference_package(ref)
    reset_cases = [(2, 3, 64, 128, 8.0, 123), (4, 4, 32, 32, 0.86, 7)]
    blob["reset_count"] = np.int64(len(reset_cases))
    for i, (C, F, mh, mw, factor, seed) in enumerate(reset_cases):
        random.seed(seed)
        m = pkg.BoxConv2d(C, F, mh, mw, reparametrization_factor=factor)
        blob["reset%d_meta" % i] = np.array([C, F, mh, mw, seed], np.int64)
        blob["reset%d_factor" % i] = np.float64(factor)
        blob["reset%d_params" % i] = np.stack([p.detach().numpy() for p in (m.x_min, m.x_max, m.y_min, m.y_max)])

    # ---- boxes on integer and half-integer coordinates and on the plane's borders, every mode; own
    # random stream, so that the arrays above do not depend on this block
    erng = np.random.default_rng(777)
    edge_cases = [(1, 2, 8, 12, 20, n, e) for n in (True, False) for e in (True, False)]
    blob["edge_count"] = np.int64(len(edge_cases))
    for i, (N, C, F, h, w, normalize, exact) in enumerate(edge_cases):
        x = erng.standard_normal((N, C, h, w)).astype(np.float32)
        go = erng.standard_normal((N, C * F, h, w)).astype(np.float32)
        boxes = border_boxes(h, w, exact)
        params = [np.empty((C, F), np.float32) for _ in range(4)]
        for c in range(C):
            for f in range(F):
                for k in range(4):
                    params[k][c, f] = boxes[(f + c) % len(boxes)][k]
        tp = [torch.from_numpy(p) for p in params]
        integ = ref.integral_image(torch.from_numpy(x))
        out = ref.box_convolution_forward(integ, *tp, normalize, exact)
        res = ref.box_convolution_backward(
            integ, *tp, torch.from_numpy(go), out if normalize else torch.empty(0),
            1.0, 1.0, normalize, exact, True, True, True, True, True)
        pre = "edge%d_" % i
        blob[pre + "meta"] = np.array([N, C, F, h, w, int(normalize), int(exact)], np.int64)
        blob[pre + "x"] = x
        blob[pre + "go"] = go
        blob[pre + "params"] = np.stack(params)
        blob[pre + "out"] = out.numpy()
        blob[pre + "gin"] = res[0].numpy()
        blob[pre + "gparams"] = np.stack([r.numpy() for r in res[1:]])

    np.savez_compressed(OUT, **blob)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(blob), "arrays")


if __name__ == "__main__":
    main()
