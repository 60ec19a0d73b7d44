"""Golden vectors from the UNMODIFIED reference CPU path (scalar: BaseLayer::supportAvx = false).

Needs oracle/_ref/ref_driver (make -C oracle) and therefore the reference source tree; run here, the
.npz files are committed and are all that travels. Run from the repo root:
    python tests/golden/make_reference_fixtures.py [net@size ...]

Per fixture: the topology/weights/image are NOT stored (they are regenerated from seeds by
msnhnet_b200.topologies / synth); stored are, for every top-level layer, its shape, mean, standard
deviation and 256 values sampled at fixed positions, plus the complete final result (classifier
output, or the post-NMS boxes as rows x,y,w,h,conf,bestClsConf,bestClsIdx).
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from msnhnet_b200 import synth, topologies  # noqa: E402

DRIVER = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
# name@size[@confThresh]: the small detector cases lower the confidence threshold so that a few thousand
# cells pass and the candidate / NMS path is exercised; the full-size ones keep the nets' own thresholds
DEFAULT = ["resnet18@224", "yolov3_tiny@416@0.02", "mobilenetv2@224", "yolov4@160@0.02", "yolov5m@160@0.02", "yolov4@608", "yolov5m@640"]
SAMPLES = 256


def sample_positions(n):
    """Fixed pseudo-random positions (seeded by n) so the checker can recompute them."""
    return np.random.default_rng(n).integers(0, n, size=min(SAMPLES, n))


def make(name, size, conf=None):
    text = topologies.NETS[name](size=size, **({} if conf is None else {"conf": conf}))
    blob = synth.make_blob(text, synth.load_factors(name))
    img = synth.make_images(1, 3, size, size)[0]
    out = {"net": name, "size": size, "conf": np.float64(-1.0 if conf is None else conf)}
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "net.msnhnet"), "w").write(text)
        blob.tofile(os.path.join(d, "w.msnhbin"))
        img.tofile(os.path.join(d, "img.f32"))
        r = subprocess.run([DRIVER, "run", d + "/net.msnhnet", d + "/w.msnhbin", d + "/img.f32", d, "0", "1"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(r.stderr)
        i = 0
        n_layers = 0
        while True:
            p = os.path.join(d, f"layer_{i}.f32")
            if not os.path.exists(p):
                if os.path.exists(os.path.join(d, f"layer_{i + 1}.f32")):
                    i += 1
                    continue
                break
            y = np.fromfile(p, np.float32)
            out[f"l{i}_n"] = np.int64(y.size)
            out[f"l{i}_mean"] = np.float64(y.astype(np.float64).mean())
            out[f"l{i}_std"] = np.float64(y.astype(np.float64).std())
            out[f"l{i}_absmax"] = np.float64(np.abs(y).max())
            out[f"l{i}_samples"] = y[sample_positions(y.size)]
            n_layers = i + 1
            i += 1
        out["n_layers"] = n_layers
        if os.path.exists(os.path.join(d, "boxes.f32")):
            out["boxes"] = np.fromfile(os.path.join(d, "boxes.f32"), np.float32).reshape(-1, 7)
        else:
            out["final"] = np.fromfile(os.path.join(d, "final.f32"), np.float32)
    path = os.path.join(ROOT, "tests", "golden", f"ref_{name}_{size}.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes", "layers", n_layers, "boxes" if "boxes" in out else "final", len(out.get("boxes", out.get("final"))))


if __name__ == "__main__":
    for item in (sys.argv[1:] or DEFAULT):
        parts = item.split("@")
        make(parts[0], int(parts[1]), float(parts[2]) if len(parts) > 2 else None)
