"""Small driver for profiler captures: builds one benchmark net and runs a few forwards.

    python -m msnhnet_b200.profile_run --workload yolov4-608 --batch 2 --steps 2 [--no-graph]

Kept apart from bench.py so a capture replays as few launches as possible.
"""
import argparse

from . import _ffi, synth, topologies
from .net import Net

SIZES = {"yolov4-608": ("yolov4", 608), "yolov5m-640": ("yolov5m", 640), "mobilenetv2-224": ("mobilenetv2", 224),
         "yolov3-tiny-416": ("yolov3_tiny", 416), "resnet18-224": ("resnet18", 224)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="yolov4-608", choices=sorted(SIZES))
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "fp32"])
    ap.add_argument("--no-graph", action="store_true")
    a = ap.parse_args()
    name, size = SIZES[a.workload]
    text = topologies.NETS[name](size=size)
    blob = synth.make_blob(text, synth.load_factors(name))
    imgs = synth.make_images(a.batch, 3, size, size)
    net = Net(text, blob, a.dtype == "fp16", batch=a.batch, flags=_ffi.PLAN_NO_GRAPH if a.no_graph else 0)
    for _ in range(a.steps):
        net.forward(imgs)
    print("ran", a.steps, "forwards of", a.workload, "batch", a.batch, "kernel ms", round(net.kernel_ms(), 3))
    net.close()


if __name__ == "__main__":
    main()
