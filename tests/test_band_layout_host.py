"""Index arithmetic of the column-band kernels (csrc/box_band_smem.cu), restated on the CPU: the
padded integral-image row [4 zeros | I[a][0..w] | copies of I[a][w]] read through a clamped window
start gives the same taps as clamping every tap's column to the plane, and every window of a band
lies inside the 40 columns the CTA copies, which in turn lie inside the padded row.  The constants
are read from the source so that the check follows the kernels."""
import os
import re

import numpy as np

from conftest import PKG_DIR


def _constants():
    text = open(os.path.join(PKG_DIR, "csrc", "box_band_smem.cu")).read()
    def const(name):
        return int(re.search(r"constexpr int %s = (\d+);" % name, text).group(1))
    return const("kBand"), const("kRectCols"), const("kLPad")


def _pitch(w, rect_cols, lpad):
    return (lpad + w + 1 + (rect_cols - 1) + 3) & ~3


def test_padded_rows_reproduce_per_tap_clamping():
    band, rect_cols, lpad = _constants()
    rng = np.random.default_rng(0)
    for w in (1, 3, 31, 32, 33, 100, 512, 515):
        pitch = _pitch(w, rect_cols, lpad)
        assert pitch % 4 == 0
        row = rng.standard_normal(w + 1)
        row[0] = 0.0                                     # column 0 of an integral image
        padded = np.concatenate([np.zeros(lpad), row, np.full(pitch - lpad - (w + 1), row[w])])
        for qb in range(0, w, band):
            for off in list(range(-w - 40, w + 41, 7)) + [-1, 0, 1]:     # lo_c - 1 or hi_c of a box
                start_b = min(max(qb + off, -lpad), w)
                s4 = (start_b // 4) * 4                  # what `& ~3` does to a two's complement int
                assert -lpad <= s4 and lpad + s4 + rect_cols <= pitch     # the copied band is inside the row
                for q in range(qb, min(qb + band, w)):
                    start = min(max(q + off, -lpad), w)
                    rel = start - s4
                    assert 0 <= rel and rel + 1 < rect_cols              # both taps inside the copied band
                    for m in (0, 1):
                        want = row[min(max(q + off + m, 0), w)]
                        assert padded[lpad + start + m] == want, (w, qb, off, q, m)
