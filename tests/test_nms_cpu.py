"""The host half of YoloOut (score sort + per-class greedy NMS, include/msnhnet_capi.h
msnhB200PostProcess) against the oracle's restatement, on seeded candidate rows. Runs on CPU."""
import numpy as np
import pytest

import helpers as H
from oracle import msnh_oracle as mo


def random_rows(rng, n, classes=5, span=200.0):
    rows = np.zeros((n, 8), np.float32)
    rows[:, 0:2] = rng.random((n, 2), dtype=np.float32) * span
    rows[:, 2:4] = rng.random((n, 2), dtype=np.float32) * 60 + 4
    rows[:, 4] = rng.random(n, dtype=np.float32) * 0.6 + 0.4
    rows[:, 5] = rng.random(n, dtype=np.float32)
    rows[:, 6] = rng.integers(0, classes, n)
    rows[:, 7] = np.arange(n)
    return rows


@pytest.mark.parametrize("n,classes,thresh", [(0, 3, 0.5), (1, 3, 0.5), (2, 1, 0.5), (50, 1, 0.3), (400, 5, 0.5), (1500, 80, 0.45), (300, 2, 0.0)])
def test_host_nms_is_identical_to_the_oracle(n, classes, thresh):
    rng = np.random.default_rng(n * 7 + classes)
    rows = random_rows(rng, n, classes)
    got = H.host_postprocess(rows, thresh)
    want = mo.nms(rows, thresh)[:, :7] if n else np.zeros((0, 7), np.float32)
    assert got.shape == want.shape
    assert np.array_equal(got, want)                  # same boxes in the same output order, bit for bit


def test_single_box_class_is_kept_and_duplicates_are_suppressed():
    rows = np.array([[50, 50, 20, 20, 0.9, 0.8, 1, 0],
                     [50, 50, 20, 20, 0.8, 0.9, 1, 1],      # same box, lower objectness: suppressed
                     [150, 150, 20, 20, 0.5, 0.5, 2, 2]], np.float32)
    got = H.host_postprocess(rows, 0.5)
    assert got.shape[0] == 2
    assert sorted(got[:, 4].tolist()) == [0.5, np.float32(0.9)]


def test_nms_is_keyed_on_objectness_not_on_score():
    # box B has the higher conf*cls score but the lower objectness; the reference keeps A
    rows = np.array([[50, 50, 20, 20, 0.9, 0.1, 0, 0],
                     [51, 50, 20, 20, 0.6, 0.9, 0, 1]], np.float32)
    got = H.host_postprocess(rows, 0.5)
    assert got.shape[0] == 1 and got[0, 4] == np.float32(0.9)


def test_idempotence():
    rng = np.random.default_rng(5)
    rows = random_rows(rng, 600, 4)
    once = H.host_postprocess(rows, 0.5)
    again_in = np.concatenate([once, np.arange(len(once), dtype=np.float32)[:, None]], 1)
    twice = H.host_postprocess(again_in, 0.5)
    assert np.array_equal(H.sort_rows(once), H.sort_rows(twice))
