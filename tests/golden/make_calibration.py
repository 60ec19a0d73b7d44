"""Makes msnhnet_b200/data/calibration.json: one scale factor per weight-owning layer of each
benchmark net, so that every conv / connected / BatchNorm output has RMS 1 (before its activation)
on the calibration image. Run from the repo root:  python tests/golden/make_calibration.py

Uses the numpy oracle for the forward pass (test infrastructure); the product only reads the json.
The pass is single-shot: each layer's output is measured, divided by its RMS on the spot, and the
forward continues with the rescaled tensor, which is exactly what the rescaled weights produce.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from msnhnet_b200 import synth, topologies  # noqa: E402
from oracle import msnh_oracle as mo  # noqa: E402

SIZES = {"resnet18": 224, "yolov3_tiny": 416, "mobilenetv2": 224, "yolov4": 608, "yolov5m": 640, "yolov5m_silu": 640}


def calibrate(name, size):
    text = topologies.NETS[name](size=size)
    blob = synth.make_blob(text)
    net = mo.OracleNet(text)
    net.load_weights(blob)
    img = synth.make_images(1, 3, size, size)[0]
    factors = []

    def hook(d, y):
        rms = float(np.sqrt(np.mean(np.square(y, dtype=np.float64))))
        f = 1.0 / rms if rms > 0 else 1.0
        factors.append(f)
        return (y * np.float32(f)).astype(np.float32)

    net.forward(img, hook=hook)
    # check: the calibrated blob reproduces the calibrated pass
    blob2 = synth.make_blob(text, factors)
    net2 = mo.OracleNet(text)
    net2.load_weights(blob2)
    rms = []
    net2.forward(img, hook=lambda d, y: (rms.append(float(np.sqrt(np.mean(np.square(y, dtype=np.float64))))), y)[1])
    print(name, size, "layers", len(factors), "factor range %.3g..%.3g" % (min(factors), max(factors)),
          "rms after calibration %.4f..%.4f" % (min(rms), max(rms)))
    return [float(np.float32(f)) for f in factors]


def objectness_priors(name, size, factors, pass_fraction=0.005):
    """One bias offset per detection head so that `pass_fraction` of its cells exceed the net's
    confidence threshold on the calibration image (a few hundred candidates per image)."""
    text = topologies.NETS[name](size=size)
    net = mo.OracleNet(text)
    if not any(d["kind"] == "yoloout" for d in net.layers):
        return []
    conf = [d for d in net.layers if d["kind"] == "yoloout"][0]["conf"]
    thr = float(np.log(conf / (1.0 - conf)))
    net.load_weights(synth.make_blob(text, factors, obj_priors=[]))
    img = synth.make_images(1, 3, size, size)[0]
    priors = []

    def hook(d, y):
        if d["kind"] == "conv" and not d["bn"] and d["use_bias"] and d["filters"] % 3 == 0 and d["filters"] // 3 > 5:
            t = y.reshape(3, d["filters"] // 3, -1)[:, 4]
            priors.append(float(np.float32(thr - np.quantile(t, 1.0 - pass_fraction))))
        return y

    net.forward(img, hook=hook)
    print(name, "objectness priors", priors)
    return priors


def main():
    path = synth.CALIBRATION_FILE
    old = {}
    if os.path.exists(path):
        with open(path) as f:
            old = json.load(f)
    out = {}
    priors_only = "--priors-only" in sys.argv
    names = [a for a in sys.argv[1:] if not a.startswith("--")]
    for name, size in SIZES.items():
        if names and name not in names:
            continue
        if priors_only:
            out[name] = dict(old[name])
        else:
            out[name] = {"size": size, "weight_seed": synth.WEIGHT_SEED, "image_seed": synth.IMAGE_SEED, "factors": calibrate(name, size)}
        out[name]["obj_priors"] = objectness_priors(name, size, out[name]["factors"])
    old.update(out)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as f:
        json.dump(old, f)
    print("wrote", path)


if __name__ == "__main__":
    main()
