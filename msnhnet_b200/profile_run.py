"""Small driver for profiler captures: builds one benchmark net and runs a few forwards.

    python -m msnhnet_b200.profile_run --workload yolov4-608 --batch 2 --steps 2 [--no-graph]
    python -m msnhnet_b200.profile_run --conv 64,64,304,1,mish --batch 8 --steps 3     # one conv layer: Cin,Cout,plane,k,act

Kept apart from bench.py so a capture replays as few launches as possible.
"""
import argparse

import numpy as np

from . import _ffi, synth, topologies
from .net import Net

SIZES = {"yolov4-608": ("yolov4", 608), "yolov5m-640": ("yolov5m", 640), "mobilenetv2-224": ("mobilenetv2", 224),
         "yolov3-tiny-416": ("yolov3_tiny", 416), "resnet18-224": ("resnet18", 224), "fcns-320": ("fcns", 320)}


def one_conv(a):
    """One stride-1 'same' conv layer with bias and activation through the kernel library's C ABI, no graph."""
    cin, cout, hw, k = (int(v) for v in a.conv.split(",")[:4])
    act = {"mish": _ffi.ACT_MISH, "leaky": _ffi.ACT_LEAKY, "none": _ffi.ACT_NONE}[a.conv.split(",")[4]]
    ctx = _ffi.Context(0)
    rng = np.random.default_rng(0)
    x = rng.random((a.batch, cin, hw, hw), dtype=np.float32) - np.float32(0.3)
    wt = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    op = _ffi.make_op(_ffi.OP_CONV, [_ffi.INPUT], filters=cout, k_h=k, k_w=k, pad_h=k // 2, pad_w=k // 2, has_bias=1,
                      act=act, act_param=0.1, is_output=1)
    plan = _ffi.Plan(ctx, [op], (cin, hw, hw), a.batch, _ffi.F16 if a.dtype == "fp16" else _ffi.F32, _ffi.PLAN_NO_GRAPH)
    plan.set_weights(0, _ffi.W_WEIGHTS, wt)
    plan.set_weights(0, _ffi.W_BIAS, np.zeros(cout, np.float32))
    plan.finalize()
    for _ in range(a.steps):
        plan.run(x)
    print(plan.describe().strip().split("\n")[-1][:220])
    plan.close()
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="yolov4-608", choices=sorted(SIZES))
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "fp32"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--conv", default="", help="Cin,Cout,plane,k,act (act: mish | leaky | none): a single conv layer instead of a net")
    a = ap.parse_args()
    if a.conv:
        return one_conv(a)
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
