"""``BoxConv2d``: depthwise convolution with learnable box (rectangular averaging) filters.
Constructor arguments, fields, parameter names, shapes and units are those of the reference's
module (``box_convolution/box_convolution_module.py:7-222``), so its checkpoints load unchanged.
"""
import random

import torch

from . import ext
from .function import BoxConvolutionFunction, reparametrize


class BoxConv2d(torch.nn.Module):
    """Input ``(N, in_planes, h, w)`` -> output ``(N, in_planes*num_filters, h, w)``: every
    input channel is filtered with ``num_filters`` boxes whose four borders are learnable and
    may lie between pixels.

    in_planes, num_filters: channel counts as in a depthwise Conv2d.
    max_input_h, max_input_w: expected largest input size; used only to decide when a box has
        grown too large or drifted too far from the image (see ``_clip_parameters``).
    reparametrization_factor: boxes are stored divided by
        ``reparametrization_factor * max_input_{h,w}`` so that optimisers see values of order 1.
    stride_h, stride_w: must be 1.
    normalize: average over the box (True) or sum over it (False).

    Fields that may be changed after construction: ``exact`` (False rounds the box to whole
    pixels: faster, coarser), ``normalize``, ``reparametrization_h`` / ``reparametrization_w``.
    """

    def __init__(self, in_planes, num_filters, max_input_h, max_input_w,
                 reparametrization_factor=8, stride_h=1, stride_w=1, normalize=True):
        super().__init__()
        assert stride_h == 1 and stride_w == 1, 'Sorry, strides are NYI'
        self.in_planes, self.num_filters = in_planes, num_filters
        self.max_input_h, self.max_input_w = max_input_h, max_input_w
        self.reparametrization_h = max_input_h * reparametrization_factor
        self.reparametrization_w = max_input_w * reparametrization_factor
        self.stride_h, self.stride_w = stride_h, stride_w
        self.normalize = normalize
        self.exact = True
        for name in ("x_min", "x_max", "y_min", "y_max"):
            setattr(self, name, torch.nn.Parameter(torch.empty(in_planes, num_filters)))
        self.reset_parameters()

    def _parameters4(self):
        return self.x_min, self.x_max, self.y_min, self.y_max

    def reset_parameters(self):
        """Random boxes as in the reference (module.py:69-97): centres inside the middle
        +-max/2.4 of the frame, sizes of at least 2 px that keep the box inside that region,
        everything then stretched by 1.5; drawn with Python's ``random`` (seed with
        ``random.seed``)."""
        rows = [[], [], [], []]
        for _ in range(self.in_planes * self.num_filters):
            # draw order of the reference: centre_h, centre_w, height, width
            reach_h, reach_w = self.max_input_h * 2 / 4.8 - 1, self.max_input_w * 2 / 4.8 - 1
            ch = random.uniform(-reach_h + 1, reach_h - 1)
            cw = random.uniform(-reach_w + 1, reach_w - 1)
            height = 2 * random.uniform(1, min(reach_h - ch, ch + reach_h))
            width = 2 * random.uniform(1, min(reach_w - cw, cw + reach_w))
            for lst, v in zip(rows, (ch - height / 2, ch + height / 2, cw - width / 2, cw + width / 2)):
                lst.append(v * 1.5)
        with torch.no_grad():
            for p, vals in zip(self._parameters4(), rows):
                p.copy_(torch.tensor(vals, dtype=torch.float32).view(self.in_planes, self.num_filters))
        reparametrize(*self._parameters4(), self.reparametrization_h, self.reparametrization_w, inplace=True)

    def get_actual_parameters(self):
        """The four parameter tensors in pixels (new tensors, no gradient)."""
        return reparametrize(*self._parameters4(), self.reparametrization_h, self.reparametrization_w,
                             inplace=False, inverse=True)

    def _clip_parameters(self):
        """Projection step of projected gradient descent: boxes that have shrunk below the
        minimum size are re-opened around their centre, and borders further than the frame size
        from the centre pixel are pulled back."""
        ext.clip_parameters(*[p.data for p in self._parameters4()],
                            self.reparametrization_h, self.reparametrization_w,
                            self.max_input_h, self.max_input_w, self.exact)

    def train(self, mode=True):
        self.training = mode
        if mode is False:
            self._clip_parameters()
        return self

    def forward(self, input):
        snapshot = None
        if self.training:
            ps = self._parameters4()
            if all(p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() for p in ps):
                # the launch that clips also leaves the copy of the parameters that backward will use
                snapshot = ext.clip_parameters_packed(
                    *[p.data for p in ps], self.reparametrization_h, self.reparametrization_w,
                    self.max_input_h, self.max_input_w, self.exact)
            else:
                self._clip_parameters()
        args = (input, self.x_min, self.x_max, self.y_min, self.y_max,
                self.reparametrization_h, self.reparametrization_w, self.normalize, self.exact)
        return BoxConvolutionFunction.apply(*args) if snapshot is None else BoxConvolutionFunction.apply(*args, snapshot)

    def draw_boxes(self, channels=None, resolution=(600, 600), weights=None):
        """Rasterises the boxes into an ``(H, W, 3)`` uint8 numpy image for debugging: the frame
        centre is marked with grey lines, every box is an outline in a per-channel colour whose
        brightness follows ``weights`` (``len(channels) x num_filters`` values in [0, 1])."""
        import numpy as np

        channels = list(range(self.in_planes)) if channels is None else list(channels)
        shape = (len(channels), self.num_filters)
        if weights is None:
            wts = np.ones(shape, np.float32)
        else:
            wts = torch.as_tensor(weights).detach().cpu().float().numpy().reshape(shape)
        wts = np.clip(wts, 0.01, 1.0)

        H, W = resolution
        img = np.zeros((H, W, 3), np.uint8)
        cy, cx = H // 2, W // 2
        img[cy, :] = 70
        img[:, cx] = 70
        palette = np.array([
            [255, 0, 0], [0, 255, 0], [0, 0, 255], [255, 255, 255], [255, 255, 0], [255, 0, 255],
            [0, 255, 255], [47, 20, 255], [255, 60, 160], [60, 170, 255], [30, 105, 210],
            [222, 196, 176], [212, 255, 127], [250, 206, 135], [50, 205, 50], [0, 165, 255],
            [60, 20, 220], [170, 178, 32]], np.float32)
        x_min, x_max, y_min, y_max = (p.detach().float().cpu().numpy() for p in self.get_actual_parameters())
        top = x_min / self.max_input_h * (H / 2) + cy
        bottom = (x_max + 1) / self.max_input_h * (H / 2) + cy
        left = y_min / self.max_input_w * (W / 2) + cx
        right = (y_max + 1) / self.max_input_w * (W / 2) + cx
        thick = max(1, int(round(H / 500 + 0.5)))

        def fill(r0, r1, c0, c1, colour):
            r0, r1 = max(0, min(H, r0)), max(0, min(H, r1))
            c0, c1 = max(0, min(W, c0)), max(0, min(W, c1))
            if r1 > r0 and c1 > c0:
                img[r0:r1, c0:c1] = colour

        for row, ch in enumerate(channels):
            for f in range(self.num_filters):
                colour = (palette[(f if len(channels) == 1 else ch) % len(palette)] * wts[row, f]).astype(np.uint8)
                t, b = int(round(float(top[ch, f]))), int(round(float(bottom[ch, f])))
                l, r = int(round(float(left[ch, f]))), int(round(float(right[ch, f])))
                if t > b or l > r:          # a box with negative size is drawn filled
                    fill(min(t, b), max(t, b) + 1, min(l, r), max(l, r) + 1, colour)
                    continue
                half = thick // 2
                fill(t - half, t - half + thick, l - half, r + half + 1, colour)
                fill(b - half, b - half + thick, l - half, r + half + 1, colour)
                fill(t - half, b + half + 1, l - half, l - half + thick, colour)
                fill(t - half, b + half + 1, r - half, r - half + thick, colour)
        return img
