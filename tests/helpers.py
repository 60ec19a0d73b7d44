"""Shared test plumbing: the product is driven through its C ABI (ctypes), the oracle is the checker."""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from msnhnet_b200 import _ffi, synth, topologies  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")

# Tolerances of the parity tests (max |a-b| over max |b| per tensor): fp32 storage with tf32
# tensor-core products and fp16 storage with fp16 products, as stated for this path.
TOL_F32 = 1e-3
TOL_F16 = 2e-2


def rel_err(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))


def net_text(name, size, **kw):
    return topologies.NETS[name](size=size, **kw)


def golden(name, size):
    """(fixture, topology kwargs) of a committed reference fixture."""
    g = np.load(os.path.join(GOLDEN, f"ref_{name}_{size}.npz"))
    conf = float(g["conf"]) if "conf" in g else -1.0
    return g, ({"conf": conf} if conf >= 0 else {})


def net_blob(name, text):
    return synth.make_blob(text, synth.load_factors(name))


from msnhnet_b200.net import Net as GpuNet, host_postprocess  # noqa: E402,F401


def sort_rows(rows):
    """Order-insensitive comparison key for box / candidate rows."""
    rows = np.asarray(rows, np.float32)
    if len(rows) == 0:
        return rows
    return rows[np.lexsort(tuple(rows[:, k] for k in range(rows.shape[1] - 1, -1, -1)))]


def match_fraction(a, b, tol, same_class=True):
    """Fraction of boxes in b that have a box (of the same class, unless same_class is False) in a whose x,y,w,h differ
    by less than tol of b's largest coordinate (order-insensitive comparison of detection sets)."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    if len(b) == 0:
        return 1.0
    if len(a) == 0:
        return 0.0
    scale = float(np.abs(b[:, :4]).max()) + 1e-30
    hit = 0
    for row in b:
        same = a[a[:, 6] == row[6]] if same_class else a
        if len(same) and (np.abs(same[:, :4] - row[:4]).max(axis=1) / scale).min() < tol:
            hit += 1
    return hit / len(b)
