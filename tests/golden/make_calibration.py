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

SIZES = {"resnet18": 224, "yolov3_tiny": 416, "mobilenetv2": 224, "yolov4": 608, "yolov5m": 640}


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


def main():
    out = {}
    for name, size in SIZES.items():
        if len(sys.argv) > 1 and name not in sys.argv[1:]:
            continue
        out[name] = {"size": size, "weight_seed": synth.WEIGHT_SEED, "image_seed": synth.IMAGE_SEED, "factors": calibrate(name, size)}
    path = synth.CALIBRATION_FILE
    old = {}
    if os.path.exists(path):
        with open(path) as f:
            old = json.load(f)
    old.update(out)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as f:
        json.dump(old, f)
    print("wrote", path)


if __name__ == "__main__":
    main()
