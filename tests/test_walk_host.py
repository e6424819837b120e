"""The strip-walk arithmetic shared by all gather kernels (csrc/bc_taps.cuh, csrc/bc_walk.cuh),
compiled for the host and checked against the oracle and the golden fixtures.  CPU only."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from conftest import PKG_DIR, ROOT, max_rel
from oracle import oracle

_fp = ctypes.POINTER(ctypes.c_float)


def _p(a):
    return a.ctypes.data_as(_fp)


@pytest.fixture(scope="module")
def emu(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("emul") / "libemul.so")
    src = os.path.join(ROOT, "tests", "host_emulation", "emul.cpp")
    subprocess.check_call(["g++", "-O1", "-ffp-contract=off", "-std=c++17", "-fPIC", "-shared", "-x", "c++",
                           "-I", os.path.join(PKG_DIR, "csrc"), "-o", out, src])
    return ctypes.CDLL(out)


def emu_forward(emu, integ, params, normalize, exact, rows=8):
    N, C, hp, wp = integ.shape
    F = params[0].shape[1]
    out = np.empty((N, C * F, hp - 1, wp - 1), np.float32)
    ps = [np.ascontiguousarray(p, np.float32) for p in params]
    emu.emu_forward(_p(integ), *[_p(p) for p in ps], _p(out), N, C, F, hp - 1, wp - 1,
                    int(normalize), int(exact), rows)
    return out


def emu_backward(emu, x, go, params, rep_h, rep_w, normalize, exact, rows=8):
    N, C, h, w = x.shape
    F = params[0].shape[1]
    gint = oracle.integral_image(go.reshape(N, C, F, h, w))
    gin = np.empty((N, C, h, w), np.float32)
    gp = np.empty((4, C, F), np.float32)
    ps = [np.ascontiguousarray(p, np.float32) for p in params]
    emu.emu_backward(_p(np.ascontiguousarray(x)), _p(gint), *[_p(p) for p in ps],
                     ctypes.c_float(rep_h), ctypes.c_float(rep_w), N, C, F, h, w,
                     int(normalize), int(exact), rows, _p(gin), _p(gp))
    return gin, gp


def test_walk_matches_golden(emu, golden):
    for i in range(int(golden["bc_count"])):
        pre = "bc%d_" % i
        N, C, F, h, w, normalize, exact, _ = [int(v) for v in golden[pre + "meta"]]
        rep_h, rep_w = golden[pre + "rep"]
        params = golden[pre + "params"]
        integ = oracle.integral_image(golden[pre + "x"])
        for rows in (1, 3, 8):
            out = emu_forward(emu, integ, params, normalize, exact, rows)
            assert max_rel(out, golden[pre + "out"]) < 3e-6, (i, rows)
            gin, gp = emu_backward(emu, golden[pre + "x"], golden[pre + "go"], params,
                                   rep_h, rep_w, normalize, exact, rows)
            assert max_rel(gin, golden[pre + "gin"]) < 3e-6, (i, rows)
            for k in range(4):
                assert max_rel(gp[k], golden[pre + "gparams"][k]) < 3e-5, (i, rows, k)


@pytest.mark.parametrize("normalize,exact", [(True, True), (False, True), (True, False)])
def test_walk_matches_oracle_random(emu, normalize, exact):
    rng = np.random.default_rng(7)
    for trial in range(12):
        N, C, F = rng.integers(1, 3), rng.integers(1, 4), rng.integers(1, 5)
        h, w = int(rng.integers(1, 40)), int(rng.integers(1, 40))
        x = rng.standard_normal((N, C, h, w)).astype(np.float32)
        go = rng.standard_normal((N, C * F, h, w)).astype(np.float32)
        lo = 0.1 if exact else 1.1   # rounded boxes narrower than a pixel have zero area (inf/nan in the reference too)
        cx = rng.uniform(-h, h, (C, F)); ex = rng.uniform(lo, h + lo, (C, F))
        cy = rng.uniform(-w, w, (C, F)); ey = rng.uniform(lo, w + lo, (C, F))
        params = [a.astype(np.float32) for a in (cx - ex, cx + ex, cy - ey, cy + ey)]
        if trial % 3 == 0:      # whole-pixel coordinates: the one-sided conventions must agree too
            params = [np.round(p) for p in params]
            params[1] = np.maximum(params[1], params[0])
            params[3] = np.maximum(params[3], params[2])
        integ = oracle.integral_image(x)
        ref_out = oracle.box_convolution_forward(integ, *params, normalize, exact)
        ref = oracle.box_convolution_backward(integ, *params, go, ref_out, 3.0, 5.0, normalize, exact)
        out = emu_forward(emu, integ, params, normalize, exact)
        gin, gp = emu_backward(emu, x, go, params, 3.0, 5.0, normalize, exact)
        assert max_rel(out, ref_out) < 5e-6, trial
        assert max_rel(gin, ref[0]) < 5e-6, trial
        for k in range(4):
            assert max_rel(gp[k], ref[1 + k]) < 5e-5, (trial, k)
