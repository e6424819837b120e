"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations (they stand in for Cityscapes activations of the ENet box blocks: the dataset is
not available offline).  Used by the tests and by bench.py so that the CPU oracle and the CUDA
library see identical bits.

  cfg1  N8  C16 64x64    F4   boxes: centres U(+-16), half-extents U(1,16)            (CPU-sized case)
  cfg2  N16 C32 64x128   F4   centres U(+-32 rows, +-64 cols), half-extents U(1,16)/U(1,32)   (1/8 frame)
  cfg3  N8  C16 256x512  F4   centres U(+-64, +-128), half-extents U(1,64)/U(1,128)   (1/4 frame)
  cfg4  1024 planes 512x1024, U[0,1): integral image alone
  cfg5  global N256 C32 64x128 F4, boxes as cfg2: batch-sharded training step

x and grad_output ~ N(0,1).  Boxes are redrawn until no coordinate lies within 1e-3 of a whole
pixel (keeps ceil/floor decisions identical across implementations and the gradients defined)
and are stored divided by max_input * 8, as the module stores them.
"""
from dataclasses import dataclass

import numpy as np

CONFIGS = {
    #        N   C   F   h    w    a_h  a_w  b_h  b_w
    "cfg1": (8, 16, 4, 64, 64, 16, 16, 16, 16),
    "cfg2": (16, 32, 4, 64, 128, 32, 64, 16, 32),
    "cfg3": (8, 16, 4, 256, 512, 64, 128, 64, 128),
    "cfg5": (256, 32, 4, 64, 128, 32, 64, 16, 32),
}
SEEDS = {"cfg1": 1001, "cfg2": 1002, "cfg3": 1003, "cfg4": 1004, "cfg5": 1005}
REPARAMETRIZATION_FACTOR = 8


@dataclass
class Workload:
    name: str
    x: np.ndarray               # (N, C, h, w) float32
    grad_output: np.ndarray     # (N, C*F, h, w) float32
    stored: list                # x_min, x_max, y_min, y_max as the module stores them, (C, F) float32
    max_h: int
    max_w: int
    rep_h: float
    rep_w: float
    F: int

    @property
    def shape(self):
        N, C, h, w = self.x.shape
        return N, C, self.F, h, w

    @property
    def outputs(self):
        N, C, F, h, w = self.shape
        return N * C * F * h * w

    @property
    def algorithmic_bytes(self):
        """Compulsory HBM traffic of forward+backward: read x, write out, read grad_output,
        read x again, write grad_input = 4 E (2F + 3) bytes."""
        N, C, F, h, w = self.shape
        return 4 * N * C * h * w * (2 * F + 3)


def draw_boxes(rng, C, F, a_h, a_w, b_h, b_w):
    def draw(n):
        ch = rng.uniform(-a_h, a_h, n); eh = rng.uniform(1.0, b_h, n)
        cw = rng.uniform(-a_w, a_w, n); ew = rng.uniform(1.0, b_w, n)
        return np.stack([ch - eh, ch + eh, cw - ew, cw + ew]).astype(np.float32)   # (4, n)

    boxes = draw(C * F)
    for _ in range(1000):
        bad = (np.abs(boxes - np.round(boxes)) < 1e-3).any(axis=0)
        if not bad.any():
            break
        boxes[:, bad] = draw(int(bad.sum()))
    return [boxes[i].reshape(C, F) for i in range(4)]


def make_workload(name, batch=None, planes=None):
    """`batch` / `planes` shrink N / C (same seed, same distributions) for bounded CPU samples."""
    N, C, F, h, w, a_h, a_w, b_h, b_w = CONFIGS[name]
    N = batch if batch is not None else N
    C = planes if planes is not None else C
    rng = np.random.default_rng(SEEDS[name])
    pix = draw_boxes(rng, C, F, a_h, a_w, b_h, b_w)
    rep_h, rep_w = float(h * REPARAMETRIZATION_FACTOR), float(w * REPARAMETRIZATION_FACTOR)
    stored = [pix[0] / np.float32(rep_h), pix[1] / np.float32(rep_h),
              pix[2] / np.float32(rep_w), pix[3] / np.float32(rep_w)]
    x = rng.standard_normal((N, C, h, w), dtype=np.float32)
    go = rng.standard_normal((N, C * F, h, w), dtype=np.float32)
    return Workload(name, x, go, stored, h, w, rep_h, rep_w, F)


def make_integral_workload(planes=1024, h=512, w=1024):
    """cfg4: `planes` planes of h x w, U[0,1)."""
    rng = np.random.default_rng(SEEDS["cfg4"])
    return rng.random((planes, h, w), dtype=np.float32)
