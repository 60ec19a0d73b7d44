"""The oracle's restatement of the reference's image preprocessing against vectors made by the reference code itself
(tests/golden/ref_preprocess.npz, produced by tests/golden/make_preprocess_fixtures.py). Byte work: bit-exact."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import helpers as H  # noqa: E402,F401  (puts the repo root on sys.path)
from golden.make_preprocess_fixtures import CASES, MEAN, STD, case_image  # noqa: E402
from oracle import msnh_oracle as mo  # noqa: E402

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_preprocess.npz"))


@pytest.mark.parametrize("k", range(len(CASES)))
def test_oracle_preprocessing_equals_reference(k):
    name, w, h, ow, oh, mode, swap = CASES[k]
    got = mo.preprocess_u8(case_image(k, w, h), ow, oh, mode, swap, mean=MEAN, std=STD)
    assert got.dtype == np.float32 and got.shape == (3, oh, ow)
    assert np.array_equal(got, GOLD[name]), name


def test_resize_edge_rules():
    """The quirks a re-implementation must keep: same-size images pass through untouched; at the clamped last
    row/column the two weights cancel (the reference's arithmetic, not a bug of this restatement)."""
    img = np.full((4, 4, 3), 200, np.uint8)
    assert mo.resize_bilinear_u8(img, 4, 4) is img
    up = mo.resize_bilinear_u8(img, 8, 8)
    assert up[0, 0, 0] == 200 and up[3, 3, 0] == 200
    assert up[7, 7, 0] == 0 and up[7, 3, 0] == 0          # last source row and column: weights -f and +f
    wide = np.zeros((2, 6, 3), np.uint8)
    boxed = mo.letterbox_127(wide)
    assert boxed.shape == (6, 6, 3) and boxed[0, 0, 0] == 127 and boxed[2, 0, 0] == 0 and boxed[5, 5, 2] == 127
