"""Golden vectors for the image preprocessing in front of the net, made by the UNMODIFIED reference code
(oracle/_ref/ref_prep: the reference's Mat / MatOp::resize / CVUtil sources compiled by oracle/Makefile).
Writes tests/golden/ref_preprocess.npz. Run from the repo root in a container that has the reference:
    make -C oracle && python tests/golden/make_preprocess_fixtures.py
Inputs are seeded random 8-bit images (no dataset items)."""
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
PREP = os.path.join(ROOT, "oracle", "_ref", "ref_prep")
MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
# (name, width, height, out_w, out_h, mode, swapRGB)
CASES = [
    ("yolo_wide", 53, 37, 64, 64, "yolo", 1),
    ("yolo_tall_swap0", 31, 58, 64, 64, "yolo", 0),
    ("yolo_square_same", 64, 64, 64, 64, "yolo", 1),
    ("yolo_down", 210, 97, 96, 96, "yolo", 1),
    ("c3_up", 37, 53, 64, 48, "c3", 1),
    ("c3_down_swap0", 150, 101, 56, 56, "c3", 0),
    ("googlenet", 41, 29, 48, 48, "googlenet", 1),
    ("caffe", 29, 41, 48, 48, "caffe", 0),
    ("transformed", 45, 45, 32, 32, "transformed", 1),
    ("padzero_classify", 80, 33, 56, 56, "padzero", 0),
]


def case_image(k, w, h):
    return np.random.default_rng(9100 + k).integers(0, 256, (h, w, 3), dtype=np.uint8)


def main():
    if not os.path.exists(PREP):
        sys.exit("oracle/_ref/ref_prep is missing: make -C oracle first")
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for k, (name, w, h, ow, oh, mode, swap) in enumerate(CASES):
            img = case_image(k, w, h)
            src, dst = os.path.join(tmp, "in.u8"), os.path.join(tmp, "out.f32")
            img.tofile(src)
            cmd = [PREP, mode, src, str(w), str(h), "3", str(ow), str(oh), str(swap), dst]
            if mode == "transformed":
                cmd += [str(v) for v in MEAN + STD]
            subprocess.run(cmd, check=True, capture_output=True)
            out[name] = np.fromfile(dst, np.float32).reshape(3, oh, ow)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "ref_preprocess.npz"), **out)
    print("wrote", len(out), "cases")


if __name__ == "__main__":
    main()
