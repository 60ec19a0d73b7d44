"""Golden vectors from the UNMODIFIED reference CPU path (scalar: BaseLayer::supportAvx = false).

Needs oracle/_ref/ref_driver (make -C oracle) and therefore the reference source tree; run here, the
.npz files are committed and are all that travels. Run from the repo root:
    python tests/golden/make_reference_fixtures.py [net@size ...]

Per fixture: the topology/weights/image are NOT stored (they are regenerated from seeds by
msnhnet_b200.topologies / synth); stored are, for every top-level layer, its shape, mean, standard
deviation and values sampled at fixed positions, plus the complete final result (classifier
output, or the post-NMS boxes as rows x,y,w,h,conf,bestClsConf,bestClsIdx).

Small fixtures hold 256 samples per layer of image 0 (the tests compare those nets whole, tensor by
tensor, against the oracle anyway). The full-size detector fixtures (name@size@conf@dense, or the
DEFAULT list) hold, for images 0 AND 1 of the seeded stream, 3072 random positions plus the last 128
pixels of eight channel planes per layer (keys "i1_..." for image 1): the last pixels of a plane are where
a ragged last tile of a GPU kernel would show.
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
DEFAULT = ["resnet18@224", "yolov3_tiny@416@0.02", "mobilenetv2@224", "yolov4@160@0.02", "yolov5m@160@0.02", "yolov5m_silu@160@0.02",
           "yolov4@608@-1@dense", "yolov5m@640@-1@dense", "yolov5m_silu@640"]
SAMPLES = 256
DENSE_RANDOM, DENSE_TAIL_PIXELS, DENSE_TAIL_CHANNELS = 3072, 128, 8


def sample_positions(n):
    """Fixed pseudo-random positions (seeded by n) so the checker can recompute them."""
    return np.random.default_rng(n).integers(0, n, size=min(SAMPLES, n))


def dense_positions(n, channels):
    """The dense scheme: random positions plus the last pixels of eight channel planes of a planar (C, H, W) tensor."""
    rng = np.random.default_rng(n)
    pos = [rng.integers(0, n, size=min(DENSE_RANDOM, n))]
    hw = n // channels
    tail = min(DENSE_TAIL_PIXELS, hw)
    chans = np.unique(np.concatenate([[0, channels - 1], rng.integers(0, channels, size=DENSE_TAIL_CHANNELS - 2)]))
    for c in chans:
        pos.append(c * hw + np.arange(hw - tail, hw))
    return np.concatenate(pos).astype(np.int64)


def layer_channels(path):
    """Channels of every top-level layer's output, from the reference's own shape inference."""
    r = subprocess.run([DRIVER, "layout", path], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(r.stderr)
    return {int(l.split()[0]): int(l.split()[3]) for l in r.stdout.strip().split("\n") if l and l.split()[0].isdigit()}


def make(name, size, conf=None, dense=False):
    text = topologies.NETS[name](size=size, **({} if conf is None else {"conf": conf}))
    blob = synth.make_blob(text, synth.load_factors(name))
    out = {"net": name, "size": size, "conf": np.float64(-1.0 if conf is None else conf), "dense": np.int64(1 if dense else 0)}
    for k, img in enumerate(synth.make_images(2 if dense else 1, 3, size, size)):
        one_image(text, blob, img, out, "" if k == 0 else f"i{k}_", dense)
    n_layers = int(out["n_layers"])
    path = os.path.join(ROOT, "tests", "golden", f"ref_{name}_{size}.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes", "layers", n_layers, "boxes" if "boxes" in out else "final", len(out.get("boxes", out.get("final"))))


def one_image(text, blob, img, out, prefix, dense):
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "net.msnhnet"), "w").write(text)
        blob.tofile(os.path.join(d, "w.msnhbin"))
        img.tofile(os.path.join(d, "img.f32"))
        r = subprocess.run([DRIVER, "run", d + "/net.msnhnet", d + "/w.msnhbin", d + "/img.f32", d, "0", "1"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(r.stderr)
        chans = layer_channels(d + "/net.msnhnet") if dense else {}
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
            out[f"{prefix}l{i}_n"] = np.int64(y.size)
            out[f"{prefix}l{i}_mean"] = np.float64(y.astype(np.float64).mean())
            out[f"{prefix}l{i}_std"] = np.float64(y.astype(np.float64).std())
            out[f"{prefix}l{i}_absmax"] = np.float64(np.abs(y).max())
            if dense:
                out[f"{prefix}l{i}_c"] = np.int64(chans[i])
                out[f"{prefix}l{i}_samples"] = y[dense_positions(y.size, chans[i])]
            else:
                out[f"{prefix}l{i}_samples"] = y[sample_positions(y.size)]
            n_layers = i + 1
            i += 1
        out["n_layers"] = n_layers
        if os.path.exists(os.path.join(d, "boxes.f32")):
            out[prefix + "boxes"] = np.fromfile(os.path.join(d, "boxes.f32"), np.float32).reshape(-1, 7)
        else:
            out[prefix + "final"] = np.fromfile(os.path.join(d, "final.f32"), np.float32)


def fixture_positions(gold, prefix, i, n):
    """Positions of the stored samples of layer i (whichever scheme the fixture was made with)."""
    if int(gold["dense"]) if "dense" in gold else 0:
        return dense_positions(n, int(gold[f"{prefix}l{i}_c"]))
    return sample_positions(n)


if __name__ == "__main__":
    for item in (sys.argv[1:] or DEFAULT):
        parts = item.split("@")
        conf = float(parts[2]) if len(parts) > 2 and float(parts[2]) >= 0 else None
        make(parts[0], int(parts[1]), conf, dense=len(parts) > 3 and parts[3] == "dense")
