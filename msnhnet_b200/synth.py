"""Seeded synthetic weights and inputs for the benchmark nets.

There are no pretrained `.msnhbin` files here, so every number is measured on random weights drawn
per layer in `.msnhbin` blob order: conv / connected weights ~ N(0, sqrt(2 / fan_in)) (He-normal),
conv bias ~ N(0, 0.01), BatchNorm gamma ~ U(0.5, 1.5), beta ~ N(0, 0.1), running mean ~ N(0, 0.1),
running variance ~ U(0.5, 1.5); inputs are uniform [0, 1) planar CHW images, the value range the
reference's preprocessing produces (src/utils/MsnhCVUtil.cpp:203-248 of the Msnhnet source tree).

Drawn exactly like that, deep nets blow up (YOLOv4's activations reach 1e6 by the heads and every
decoded box is inf), so each weight-owning layer also carries one committed scale factor
(`data/calibration.json`, made by tests/golden/make_calibration.py) that brings its pre-activation
output to RMS 1 on the calibration image: the factor multiplies gamma and beta of a BatchNorm, or
the weights and bias of a layer without one. Distribution shapes and seeds stay as stated.

Detection heads (the bias-only convs whose channel count is 3 x (5 + classes)) get an objectness
prior: a committed per-head offset (also in calibration.json) is added to the three objectness
biases, as detector training initialises and keeps them, so that about 0.5 % of the cells pass the
confidence threshold - a realistic hundred or so candidates per image - instead of the ~35 % that
zero-mean random logits would give (which would turn the benchmark into a benchmark of the
host-side NMS).

The blob layout comes from the host library (msnhB200WeightLayout), so this module holds no second
copy of the parser.
"""
import ctypes as C
import json
import os

import numpy as np

from . import _ffi

HERE = os.path.dirname(os.path.abspath(__file__))
CALIBRATION_FILE = os.path.join(HERE, "data", "calibration.json")
WEIGHT_SEED = 1234
IMAGE_SEED = 20240


def weight_layout(text):
    """[(op, slot, count, rows)] in blob order."""
    lib = _ffi.host_lib()
    msg = C.c_char_p()
    if lib.msnhB200WeightLayout(C.byref(msg), text.encode()) != 1:
        raise ValueError(msg.value.decode() if msg.value else "weight layout failed")
    out = []
    for line in msg.value.decode().strip().split("\n"):
        if line:
            op, slot, count, rows = (int(v) for v in line.split())
            out.append((op, slot, count, rows))
    return out


class Calibration(list):
    """The per-layer factors of one net (a list) plus its per-head objectness priors."""
    obj_priors = ()


def load_factors(name, size=None):
    if not os.path.exists(CALIBRATION_FILE):
        return None
    with open(CALIBRATION_FILE) as f:
        table = json.load(f)
    entry = table.get(name)
    if entry is None:
        return None
    c = Calibration(entry["factors"])
    c.obj_priors = tuple(entry.get("obj_priors", ()))
    return c


def make_blob(text, factors=None, seed=WEIGHT_SEED, obj_priors=None):
    """The float32 `.msnhbin` content for topology `text`. `factors`: one multiplier per weight-owning
    layer in blob order (None = uncalibrated); `obj_priors`: one objectness bias offset per detection
    head in blob order (default: the ones that came with `factors`)."""
    if obj_priors is None:
        obj_priors = getattr(factors, "obj_priors", ())
    head = 0
    layout = weight_layout(text)
    rng = np.random.default_rng(seed)
    total = sum(c for _, _, c, _ in layout)
    blob = np.empty(total, np.float32)
    # group consecutive slots of the same op
    groups, cur = [], []
    for item in layout:
        if cur and item[0] != cur[0][0]:
            groups.append(cur)
            cur = []
        cur.append(item)
    if cur:
        groups.append(cur)
    if factors is not None and len(factors) != len(groups):
        raise ValueError(f"calibration has {len(factors)} factors, the net has {len(groups)} weight-owning layers")
    off = 0
    for gi, grp in enumerate(groups):
        f = np.float32(1.0 if factors is None else factors[gi])
        slots = {s for _, s, _, _ in grp}
        has_bn = _ffi.W_BN_SCALE in slots
        for _, slot, count, rows in grp:
            if slot == _ffi.W_WEIGHTS:
                fan_in = count // rows
                v = rng.standard_normal(count, dtype=np.float32) * np.float32(np.sqrt(2.0 / fan_in))
                if not has_bn:
                    v = v * f
            elif slot == _ffi.W_BIAS:
                v = rng.standard_normal(count, dtype=np.float32) * np.float32(0.01) * f
                if not has_bn and count % 3 == 0 and count // 3 > 5 and any(s2 == _ffi.W_WEIGHTS and r2 == count and r2 in (255, 18, 21, 24, 27, 30, 75) for _, s2, _, r2 in grp):
                    per = count // 3
                    if head < len(obj_priors):
                        v[4::per] += np.float32(obj_priors[head])
                    head += 1
            elif slot == _ffi.W_BN_SCALE:
                v = (rng.random(count, dtype=np.float32) + np.float32(0.5)) * f
            elif slot == _ffi.W_BN_BIAS:
                v = rng.standard_normal(count, dtype=np.float32) * np.float32(0.1) * f
            elif slot == _ffi.W_BN_MEAN:
                v = rng.standard_normal(count, dtype=np.float32) * np.float32(0.1)
            else:  # W_BN_VAR
                v = rng.random(count, dtype=np.float32) + np.float32(0.5)
            blob[off:off + count] = v
            off += count
    return blob


def make_images(n, channels, height, width, seed=IMAGE_SEED):
    """n uniform [0,1) planar CHW images; image k of the stream is the same whatever n is."""
    out = np.empty((n, channels, height, width), np.float32)
    for k in range(n):
        out[k] = np.random.default_rng(seed + k).random((channels, height, width), dtype=np.float32)
    return out
