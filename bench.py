#!/usr/bin/env python
"""Throughput of the GPU forward hot path (images/s) on the named workload, one JSON line.

    python bench.py --gpus N --steps K --warmup W          # this backend (N>1: launched by torchrun)
    python bench.py --impl reference --steps K --warmup W  # the reference's own CPU path on the host cores

A step is one forward of `per-gpu-batch` synthetic images per GPU through the whole net (input
layout change, every layer, YOLO decode and candidate collection). `value` is timed with CUDA events
on the plan's stream with the inputs resident in HBM; `e2e` is the same workload through the
reference-facing call (msnhB200RunYoloBatch / RunClassifyBatch: pinned host images in, boxes out,
host NMS included). Multi-GPU is independent replicas, images sharded by index, no collective on the
data path; torch.distributed only provides the barrier and the max over ranks of the device time.
"""
import argparse
import ctypes as C
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    # name: (net, size, images per GPU per step, dtype, conv GFLOP per image)
    "yolov4-608": ("yolov4", 608, 8, "fp16", 128.39),
    "yolov5m-640": ("yolov5m", 640, 32, "fp16", 52.19),
    "mobilenetv2-224": ("mobilenetv2", 224, 64, "fp16", 0.605),
    "yolov3-tiny-416": ("yolov3_tiny", 416, 16, "fp16", 5.57),
    "resnet18-224": ("resnet18", 224, 1, "fp32", 3.63),
    # segmentation net with five transposed convolutions (the reference's models/fcns structure); output = a 2 x 320 x 320 map
    "fcns-320": ("fcns", 320, 16, "fp16", 64.54),
}


# DRAM bytes (read + write) of the tensor-core conv launches of one step, from one ncu capture of this
# command with --cache-control none (summary under profiles/): (workload, images per GPU, dtype) -> bytes
MEASURED_CONV_DRAM_BYTES = {("yolov4-608", 8, "f16"): 2.5364e9}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops": float(p.get("bf16_tflops_sustained", p.get("bf16_tflops", 1400.0))), "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs: NVML read every 5 ms from a thread
    (the timed region of a default run lasts well under the second nvidia-smi needs to start), with the
    nvidia-smi loop of the profiling recipe as the fallback when NVML cannot be loaded. Read-only."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.sm, self.mx, self.reasons, self.stop_flag, self.thread, self.source = [], None, set(), False, None, None

    def _nvml_loop(self, nv, handle):
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                for bit, name in self.REASONS:
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:      # a failed read is a missing sample, nothing more
                pass
            time.sleep(0.005)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            handle = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.mx = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.source = "nvml"
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.source = "nvidia-smi"
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.thread:
            self.stop_flag = True
            self.thread.join(timeout=2)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.mx, "reasons": sorted(self.reasons),
                    "samples": len(self.sm), "source": self.source}
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 8 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 8:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "source": self.source}


def reference_cpu(net, size, warmup, iters, blob_factors=True):
    """The reference's own CPU path (oracle/_ref/ref_driver, AVX on, all host threads), batch 1 looped like
    the reference's batch-1 block layers demand. Falls back to the numpy oracle port when the reference
    binary is not there. Returns (images_per_s, kind, cores, sample)."""
    import tempfile
    from msnhnet_b200 import synth, topologies
    text = topologies.NETS[net](size=size)
    blob = synth.make_blob(text, synth.load_factors(net))
    img = synth.make_images(1, 3, size, size)[0]
    drv = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    cores = os.cpu_count() or 1
    if os.path.exists(drv):
        with tempfile.TemporaryDirectory() as d:
            open(os.path.join(d, "n.msnhnet"), "w").write(text)
            blob.tofile(os.path.join(d, "w.msnhbin"))
            img.tofile(os.path.join(d, "i.f32"))
            env = dict(os.environ, OMP_NUM_THREADS=str(cores))
            r = subprocess.run([drv, "time", d + "/n.msnhnet", d + "/w.msnhbin", d + "/i.f32", str(warmup), str(iters), "1"], capture_output=True, text=True, env=env)
        m = re.search(r"ms_per_image ([\d.]+) threads (\d+) iters (\d+)", r.stdout)
        if m:
            ms = float(m.group(1))
            return 1000.0 / ms, "reference", int(m.group(2)), f"{m.group(3)} images after {warmup} warm-up, batch 1 looped, reference CPU path with AVX, host NMS included"
    from oracle import msnh_oracle as mo
    o = mo.OracleNet(text)
    o.load_weights(blob)
    for _ in range(min(warmup, 1)):
        o.forward(img)
    n = max(1, min(iters, 2))
    t0 = time.time()
    for _ in range(n):
        o.forward(img)
    return n / (time.time() - t0), "port", 1, f"{n} images, numpy oracle port (reference binary not present)"


def run_reference(args, net, size, unit_workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # each step is a bounded sample: `sample` images through the reference CPU path
    sample = {"yolov4": 2, "yolov5m": 3}.get(net, 8)
    ips, kind, cores, desc = reference_cpu(net, size, max(1, min(args.warmup, 2)) , max(1, args.steps) * sample)
    line = {"impl": "reference", "metric": "images/sec", "value": ips, "unit": "images/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * sample / ips, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": unit_workload,
            "cpu_baseline": {"value": ips, "unit": "images/s", "cores": cores, "kind": kind, "sample": f"{sample} images per step; " + desc},
            "e2e": {"value": ips, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="yolov4-608", choices=sorted(WORKLOADS))
    ap.add_argument("--per-gpu-batch", type=int, default=0)
    ap.add_argument("--dtype", default="", choices=["", "fp16", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-out", default="")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    net, size, B, dtype, gflop = WORKLOADS[args.workload]
    if args.per_gpu_batch:
        B = args.per_gpu_batch
    if args.dtype:
        dtype = args.dtype
    fp16 = dtype == "fp16"
    config = {"workload": f"{net} {size}x{size}, {B} images per GPU per step, seeded uniform[0,1) images, seeded He-normal weights with per-layer RMS calibration",
              "per_gpu_batch": B, "parallelism": f"replicas x{args.gpus}, images sharded by index, no collective",
              "l2": "activation working set per step exceeds the 126 MB L2 (no flush between steps)"}
    if args.impl == "reference":
        run_reference(args, net, size, config)
        return

    rank, local_rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from msnhnet_b200 import _ffi, sharding, synth, topologies
    from msnhnet_b200.net import Net

    text = topologies.NETS[net](size=size)
    blob = synth.make_blob(text, synth.load_factors(net))
    lo, hi = sharding.weak_job(B, rank, world)
    images = synth.make_images(hi - lo, 3, size, size, seed=synth.IMAGE_SEED + lo)
    pinned = torch.empty(images.shape, dtype=torch.float32).pin_memory()
    pinned.copy_(torch.from_numpy(images))
    host_images = pinned.numpy()
    g = Net(text, blob, fp16, batch=B, device=local_rank)
    klib = _ffi.kernel_lib()
    plan = C.c_void_p(g.lib.msnhB200PlanHandle())
    ctx = C.c_void_p(g.lib.msnhB200CtxHandle())

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def kcheck(rc):
        if rc != 0:
            raise RuntimeError(klib.msnh_b200_last_error(ctx).decode())

    # ---- device-resident throughput: inputs in HBM, K forwards between two CUDA events ----
    g.forward(host_images)                      # fills the staging buffer (and is the first warm-up)
    ms = C.c_float()
    kcheck(klib.msnh_b200_plan_run_timed(plan, B, max(args.warmup - 1, 1), C.byref(ms)))
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    kcheck(klib.msnh_b200_plan_run_timed(plan, B, args.steps, C.byref(ms)))
    barrier()
    clocks = sampler.stop()
    total_ms = sharding.reduce_max(float(ms.value), dist if world > 1 else None)
    value = world * B * args.steps / (total_ms / 1000.0)

    # ---- end to end through the reference-facing call: pinned host images in, boxes / logits out ----
    # One streaming call over e2e_steps batches (msnhB200RunYoloStream / RunClassifyStream): every step
    # copies its batch from pinned host memory, runs the forward, reads the result back and (detectors)
    # runs the reference's host NMS; copy-in, forward and NMS of neighbouring steps overlap.
    e2e_steps = max(3, min(args.steps, 40))
    pinned_all = torch.empty((e2e_steps,) + images.shape, dtype=torch.float32).pin_memory()
    for k in range(e2e_steps):
        pinned_all[k].copy_(torch.from_numpy(images))
    host_all = pinned_all.numpy()
    msg = C.c_char_p()
    max_boxes = 1024
    if g.is_yolo:
        boxes = (_ffi.BBox * (e2e_steps * B * max_boxes))()
        counts = (C.c_int * (e2e_steps * B))()
        def user_call(nb):
            rc = g.lib.msnhB200RunYoloStream(C.byref(msg), host_all.ctypes.data_as(C.c_void_p), nb, boxes, max_boxes, counts)
            if rc != 1:
                raise RuntimeError(msg.value.decode())
    else:
        out = np.zeros((e2e_steps * B,) + g.last_shape, np.float32)      # touched once, like a buffer a caller reuses
        def user_call(nb):
            rc = g.lib.msnhB200RunClassifyStream(C.byref(msg), host_all.ctypes.data_as(C.c_void_p), nb, out.ctypes.data_as(C.POINTER(C.c_float)), out.size)
            if rc != 1:
                raise RuntimeError(msg.value.decode())
    user_call(min(3, e2e_steps))            # warm-up (allocates the streaming slots)
    barrier()
    t0 = time.perf_counter()
    user_call(e2e_steps)
    e2e_s = sharding.reduce_max(time.perf_counter() - t0, dist if world > 1 else None)
    barrier()
    e2e_value = world * B * e2e_steps / e2e_s
    # single synchronous call, for the latency of one batch
    t0 = time.perf_counter()
    user_call(1)
    e2e_single_ms = (time.perf_counter() - t0) * 1000.0
    # the same streaming call with the score sort + NMS on the device (only kept boxes cross PCIe)
    e2e_dev_nms = None
    if g.is_yolo:
        g.set_device_nms(True)
        user_call(min(3, e2e_steps))
        barrier()
        t0 = time.perf_counter()
        user_call(e2e_steps)
        dt = sharding.reduce_max(time.perf_counter() - t0, dist if world > 1 else None)
        barrier()
        e2e_dev_nms = {"value": world * B * e2e_steps / dt, "unit": "images/s", "boxes_first_batch": int(sum(counts[i] for i in range(B)))}
        g.set_device_nms(False)
    h2d = int(host_images.nbytes)
    if g.is_yolo:
        d2h = int(min(4096, 10 ** 9) * 32 * B + 4 * B)     # fixed-size pinned slot: up to 4096 candidate rows per image + counts
        n_boxes = int(sum(counts[i] for i in range(B)))
    else:
        d2h = int(np.prod(g.last_shape) * 4 * B)
        n_boxes = 0

    # ---- per-kernel device time of the same step (events between consecutive launches) ----
    n_launch, arena = C.c_int(), C.c_size_t()
    klib.msnh_b200_plan_stats(plan, C.byref(n_launch), C.byref(arena))
    per = (C.c_float * n_launch.value)()
    kcheck(klib.msnh_b200_plan_run_instrumented(plan, B, 5, per, n_launch.value))
    desc = klib.msnh_b200_plan_describe(plan).decode().strip().split("\n")
    by_kernel = {}
    for line, t in zip(desc, per):
        name = line.split()[1]
        fl = float(re.search(r"flops=([\d.e+-]+)", line).group(1))
        by = float(re.search(r"bytes=([\d.e+-]+)", line).group(1))
        k = by_kernel.setdefault(name, {"ms": 0.0, "launches": 0, "flops": 0.0, "bytes": 0.0})
        k["ms"] += t; k["launches"] += 1; k["flops"] += fl; k["bytes"] += by
    step_ms_sum = sum(per)
    pk = peaks()
    top = max(by_kernel.items(), key=lambda kv: kv[1]["ms"])
    conv = by_kernel.get("conv_umma")
    if conv and conv["ms"] > 0:
        # Duration of the conv launches inside the timed region: the region's own device time per step
        # (graph launches with programmatic dependent launch, CUDA events on the plan's stream) times the
        # conv kernels' share of the per-launch event timings of the same step. The per-launch timings
        # themselves run kernel by kernel (no overlap of a kernel's start-up with its predecessor's tail,
        # an event between every two launches), so their sum is larger than the step and is reported beside.
        share = conv["ms"] / step_ms_sum
        conv_ms = (total_ms / args.steps) * share
        achieved = conv["flops"] / (conv_ms / 1000.0) / 1e12
        traffic = MEASURED_CONV_DRAM_BYTES.get((args.workload, B, "f16" if fp16 else "f32"))
        roofline = {"kernel": "conv_umma_kernel", "bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                    "traffic": traffic, "traffic_note": "dram__bytes_read+write summed over the conv launches of one step (one ncu capture, profiles/); algorithmic bytes of the same launches: %.3e" % conv["bytes"],
                    "peak_source": pk["source"], "launches_per_step": conv["launches"], "ms_per_step": conv_ms,
                    "ms_per_step_launch_by_launch": conv["ms"], "achieved_launch_by_launch": conv["flops"] / (conv["ms"] / 1000.0) / 1e12,
                    "share_of_step": share, "note": "algorithmic conv FLOPs of one step / (device time of the timed step x conv share of per-launch CUDA-event timings)"}
    else:
        k = top[1]
        achieved = k["bytes"] / (k["ms"] / 1000.0) / 1e9
        roofline = {"kernel": top[0], "bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"]}
    if args.profile_out and rank == 0:
        with open(args.profile_out, "w") as f:
            f.write(f"# per-launch device time, {args.workload}, batch {B}, {dtype}; CUDA events between launches, mean of 5 steps\n")
            for line, t in zip(desc, per):
                f.write(f"{t:.4f} ms | {line}\n")
            f.write("# by kernel\n")
            for name, k in sorted(by_kernel.items(), key=lambda kv: -kv[1]["ms"]):
                f.write(f"{name}: launches {k['launches']} ms {k['ms']:.4f} share {k['ms'] / step_ms_sum:.3f} TFLOP/s {k['flops'] / max(k['ms'], 1e-9) / 1e9:.1f} GB/s {k['bytes'] / max(k['ms'], 1e-9) / 1e6:.1f}\n")

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        n_img = {"yolov4": 10, "yolov5m": 20}.get(net, 100)
        ips, kind, cores, sample = reference_cpu(net, size, 1, n_img)
        cpu = {"value": ips, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample}
    g.close()
    if rank == 0:
        line = {"metric": "images/sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16" if fp16 else "f32 (tf32 products)",
                "data": "synthetic", "config": config, "clocks": clocks,
                "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                        "single_batch_ms": e2e_single_ms, "boxes_first_batch": n_boxes,
                        "with_device_nms": e2e_dev_nms,
                        "call": "msnhB200RunYoloStream (per step: H2D of pinned CHW float images, forward, candidate D2H, host NMS; steps pipelined)" if g.is_yolo else "msnhB200RunClassifyStream"},
                "gpu_launches": int(n_launch.value) * args.steps, "launches_per_step": int(n_launch.value),
                "roofline": roofline, "cpu_baseline": cpu,
                "kernels": {k: {"launches": v["launches"], "ms": round(v["ms"], 4)} for k, v in sorted(by_kernel.items(), key=lambda kv: -kv[1]["ms"])},
                "arena_bytes": int(arena.value)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
