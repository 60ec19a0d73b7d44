"""Makes tests/golden/seam_ops.json: for each benchmark topology, the SHA-256 of the op list and weight-slot order that
oracle/_ref/seam_adapter derives from the UNMODIFIED reference's own layer objects (Msnhnet::NetBuilder in preview mode).
Needs the reference source tree (make -C oracle); the json is committed and is all that travels. Run from the repo root:
    python tests/golden/make_seam_fixture.py
"""
import hashlib
import json
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from msnhnet_b200 import topologies  # noqa: E402

ADAPTER = os.path.join(ROOT, "oracle", "_ref", "seam_adapter")
NETS = [("resnet18", 224), ("yolov3_tiny", 416), ("mobilenetv2", 224), ("yolov4", 608), ("yolov5m", 640), ("yolov5m_silu", 640)]


def adapter_lines(text):
    """("op ..." lines, "w op slot count" lines) the adapter prints for topology `text`."""
    with tempfile.NamedTemporaryFile("w", suffix=".msnhnet", delete=False) as f:
        f.write(text)
        path = f.name
    try:
        r = subprocess.run([ADAPTER, path], capture_output=True, text=True)
    finally:
        os.unlink(path)
    if r.returncode != 0:
        raise RuntimeError(r.stderr)
    lines = r.stdout.splitlines()
    return [l for l in lines if l.startswith("op ")], [l for l in lines if l.startswith("w ")]


def digest(ops, weights):
    return hashlib.sha256(("\n".join(ops) + "\n" + "\n".join(weights) + "\n").encode()).hexdigest()


if __name__ == "__main__":
    out = {}
    for name, size in NETS:
        ops, weights = adapter_lines(topologies.NETS[name](size=size))
        out[f"{name}@{size}"] = {"ops": len(ops), "weight_slots": len(weights), "sha256": digest(ops, weights)}
        print(name, size, out[f"{name}@{size}"])
    with open(os.path.join(ROOT, "tests", "golden", "seam_ops.json"), "w") as f:
        json.dump(out, f, indent=1)
