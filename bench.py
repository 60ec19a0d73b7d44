#!/usr/bin/env python
"""Throughput of the GPU forward hot path (images/s) on the named workload, one JSON line.

    python bench.py --gpus N --steps K --warmup W          # this backend (N>1: launched by torchrun)
    python bench.py --impl reference --steps K --warmup W  # the reference's own CPU path on the host cores

A step is one forward of `per-gpu-batch` synthetic images per GPU through the whole net (input
layout change, every layer, YOLO decode and candidate collection). `value` is timed with CUDA events
on the plan's stream with the inputs resident in HBM, over as many blocks of K steps as it takes to
fill `--min-seconds` of device time (the line's `steps` is what was timed); `e2e` is the same workload
through the reference-facing call (msnhB200RunYoloStream / RunClassifyStream: pinned host images in,
boxes out, host NMS included). Multi-GPU is independent replicas, images sharded by index, no collective
on the data path; torch.distributed only provides the barrier and the max over ranks of the device time.
The same line carries a short measurement of the other benchmark workloads (`other_workloads`), the
fixed-job readings of the multi-GPU configs (`fixed_jobs`: 64 YOLOv4 images and 256 YOLOv5m images
split over the GPUs) and the per-kernel roofline fractions (`kernels`).
"""
import argparse
import ctypes as C
import json
import math
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
HEADLINE = "yolov4-608"
# the benchmark configs besides the headline, measured briefly by the default run
OTHERS = ["yolov5m-640", "yolov3-tiny-416", "mobilenetv2-224", "resnet18-224"]
# fixed-size jobs split over the GPUs: (workload, images of the whole job)
FIXED_JOBS = [("yolov4-608", 64), ("yolov5m-640", 256)]

# DRAM bytes (read + write) of the tensor-core conv launches of one step, from one ncu capture of this
# command with --cache-control none (summary under profiles/): (workload, images per GPU, dtype) -> bytes
MEASURED_CONV_DRAM_BYTES = {("yolov4-608", 8, "f16"): 2.4707e9}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        burst = float(p.get("bf16_tflops", 1590.0))
        return {"tflops": float(p.get("bf16_tflops_sustained", burst)), "tflops_burst": burst, "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1400.0, "tflops_burst": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs: NVML read every 5 ms from a thread,
    with the nvidia-smi loop of the profiling recipe as the fallback when NVML cannot be loaded. Read-only."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.sm, self.mx, self.reasons, self.stop_flag, self.thread, self.source = [], None, set(), False, None, None
        self.power = []

    def _nvml_loop(self, nv, handle):
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                self.power.append(float(nv.nvmlDeviceGetPowerUsage(handle)) / 1000.0)
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
                    "samples": len(self.sm), "source": self.source, "power_w_max": max(self.power) if self.power else None}
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


class ClockProbe:
    """The SM cycle counter's rate against the device's nanosecond timer while the timed region runs
    (msnh_b200_clock_probe_*): the clock kernels actually see, which under load is lower than the clock NVML names."""

    def __init__(self, klib, device, max_ms):
        self.klib, self.h = klib, C.c_void_p()
        if klib.msnh_b200_clock_probe_start(device, max_ms, C.byref(self.h)) != 0:
            self.h = None

    def stop(self):
        if not self.h:
            return None
        med, lo, hi, n = C.c_double(), C.c_double(), C.c_double(), C.c_int()
        self.klib.msnh_b200_clock_probe_stop(self.h, C.byref(med), C.byref(lo), C.byref(hi), C.byref(n))
        self.h = None
        return {"sm_mhz_effective": round(med.value, 1), "min": round(lo.value, 1), "max": round(hi.value, 1), "samples": n.value,
                "how": "SM cycle counter against %globaltimer, one warp sampling once a millisecond beside the timed kernels"} if n.value else None


# ------------------------------------------------------------------------------------------------
# the reference's CPU path on the host cores
# ------------------------------------------------------------------------------------------------
def host_cpu_counts():
    """(cpus this process may run on, cpu quota of its control group or None, physical cores of the machine or None)."""
    try:
        affinity = len(os.sched_getaffinity(0))
    except AttributeError:
        affinity = os.cpu_count() or 1
    quota = None
    try:
        with open("/sys/fs/cgroup/cpu.max") as f:
            a, b = f.read().split()[:2]
            if a != "max":
                quota = max(1, int(math.ceil(float(a) / float(b))))
    except (OSError, ValueError):
        pass
    physical = None
    try:
        cores = set()
        phys = core = None
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("physical id"):
                    phys = line.split(":")[1].strip()
                elif line.startswith("core id"):
                    core = line.split(":")[1].strip()
                elif not line.strip():
                    if phys is not None and core is not None:
                        cores.add((phys, core))
                    phys = core = None
        physical = len(cores) or None
    except OSError:
        pass
    return affinity, quota, physical


def reference_cpu(net, size, warmup, iters, budget_s=60.0):
    """The reference's own CPU path (oracle/_ref/ref_driver, AVX on), batch 1 looped like the reference's batch-1
    block layers demand. The thread count is swept over {cpu quota, cpus of this process, half of them, physical
    cores} on one image each and the fastest is kept (OpenMP threads beyond what the control group grants spin
    against each other at every barrier of the reference's parallel loops). Falls back to the numpy oracle port when the
    reference binary is not there. Returns (images_per_s, kind, threads, sample, details)."""
    import tempfile
    from msnhnet_b200 import synth, topologies
    text = topologies.NETS[net](size=size)
    blob = synth.make_blob(text, synth.load_factors(net))
    img = synth.make_images(1, 3, size, size)[0]
    drv = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    affinity, quota, physical = host_cpu_counts()
    if os.path.exists(drv):
        with tempfile.TemporaryDirectory() as d:
            open(os.path.join(d, "n.msnhnet"), "w").write(text)
            blob.tofile(os.path.join(d, "w.msnhbin"))
            img.tofile(os.path.join(d, "i.f32"))

            def run(threads, warm, n):
                env = dict(os.environ, OMP_NUM_THREADS=str(threads), OMP_PROC_BIND="false")
                r = subprocess.run([drv, "time", d + "/n.msnhnet", d + "/w.msnhbin", d + "/i.f32", str(warm), str(n), "1"], capture_output=True, text=True, env=env)
                m = re.search(r"ms_per_image ([\d.]+) threads (\d+) iters (\d+)", r.stdout)
                c = re.search(r"conv_share ([\d.]+)", r.stdout)
                return (float(m.group(1)), float(c.group(1)) if c else None) if m else (None, None)

            cands = sorted({c for c in (quota, affinity, max(1, affinity // 2), physical) if c and c <= affinity}, reverse=True)
            sweep = {}
            t0 = time.time()
            for c in cands:
                ms, _ = run(c, 1 if net not in ("yolov4", "yolov5m") else 0, 1)
                if ms:
                    sweep[c] = ms
                if time.time() - t0 > budget_s * 0.5:
                    break
            if sweep:
                best = min(sweep, key=sweep.get)
                n = int(max(1, min(iters, (budget_s - (time.time() - t0)) / (sweep[best] / 1000.0))))
                ms, conv_share = run(best, warmup, n)
                if ms:
                    details = {"threads": best, "cpus_of_process": affinity, "cgroup_cpu_quota": quota, "physical_cores": physical,
                               "thread_sweep_ms_per_image": {str(k): round(v, 1) for k, v in sweep.items()}, "conv_share_of_layer_time": conv_share}
                    return 1000.0 / ms, "reference", best, f"{n} images after {warmup} warm-up, batch 1 looped, reference CPU path with AVX, host NMS included", details
    from oracle import msnh_oracle as mo
    o = mo.OracleNet(text)
    o.load_weights(blob)
    for _ in range(min(warmup, 1)):
        o.forward(img)
    n = max(1, min(iters, 2))
    t0 = time.time()
    for _ in range(n):
        o.forward(img)
    return n / (time.time() - t0), "port", 1, f"{n} images, numpy oracle port (reference binary not present)", {}


def run_reference(args, net, size, config):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # each step is a bounded sample: `sample` images, one at a time, through the reference CPU path
    sample = {"yolov4": 2, "yolov5m": 3}.get(net, 8)
    ips, kind, threads, desc, details = reference_cpu(net, size, max(1, min(args.warmup, 2)), max(1, args.steps) * sample, budget_s=120.0)
    config = dict(config, reference_arm=f"batch 1 looped, {sample} images per step (the reference's block layers are batch-1 only)")
    line = {"impl": "reference", "metric": "images/sec", "value": ips, "unit": "images/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * sample / ips, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "cpu_baseline": dict({"value": ips, "unit": "images/s", "cores": threads, "kind": kind, "sample": f"{sample} images per step; " + desc}, **details),
            "e2e": {"value": ips, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# one workload on this backend
# ------------------------------------------------------------------------------------------------
class Dist:
    def __init__(self):
        self.rank, self.local_rank, self.world = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        import torch
        self.torch = torch
        torch.cuda.set_device(self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max(self, x):
        from msnhnet_b200 import sharding
        return sharding.reduce_max(float(x), self.dist)

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def layer_table(desc, per, pk, title):
    """Markdown table of every launch of one step: its binding roof (arithmetic intensity against the ridge of the
    measured peaks), what it achieved launch by launch and the fraction of that roof."""
    ridge = pk["tflops"] * 1e12 / (pk["hbm_gbs"] * 1e9)
    out = [f"# {title}", "",
           f"Per-launch device time: CUDA events between consecutive launches, mean of 5 steps, warm (each figure carries the few microseconds of a "
           f"launch boundary that the graph replay of the timed step overlaps). Roofs: {pk['tflops']:.1f} TFLOP/s sustained dense 16-bit tensor peak and "
           f"{pk['hbm_gbs']:.1f} GB/s copy bandwidth ({pk['source']}), ridge {ridge:.0f} FLOP/B. A launch is held to the tensor roof when its unfused "
           f"arithmetic intensity (FLOPs over input + output + weight bytes) is above the ridge, to the HBM roof otherwise.", "",
           "| # | kernel | in -> out | k/s | us | FLOP/B | roof | achieved | fraction |", "|---|---|---|---|---|---|---|---|---|"]
    for line, t in zip(desc, per):
        f = line.split()
        fl = float(re.search(r"flops=([\d.e+-]+)", line).group(1))
        by = float(re.search(r"bytes=([\d.e+-]+)", line).group(1))
        io = re.search(r"in=(\S+) out=(\S+) k=(\S+) s=(\d+)", line)
        if t <= 0 or (fl == 0 and by == 0):
            continue
        ai = fl / by if by else 0.0
        if fl > 0 and ai >= ridge:
            ach, roof, frac = fl / (t * 1e-3) / 1e12, "tensor", fl / (t * 1e-3) / 1e12 / pk["tflops"]
            ach_s = f"{ach:.0f} TFLOP/s"
        else:
            ach, roof, frac = by / (t * 1e-3) / 1e9, "hbm", by / (t * 1e-3) / 1e9 / pk["hbm_gbs"]
            ach_s = f"{ach:.0f} GB/s"
        shape = re.search(r"(mm=\d+(?: \w+)* bn=\d+)", line)
        out.append(f"| {f[0]} | {f[1]}{' ' + shape.group(1) if shape else ''} | {io.group(1)} -> {io.group(2)} | {io.group(3)}/{io.group(4)} | {t * 1000:.1f} | {ai:.0f} | {roof} | {ach_s} | {frac:.2f} |")
    return "\n".join(out) + "\n"


def measure(D, workload, B, fp16, steps, warmup, min_seconds, total_images=None, e2e=True, dev_nms=False, instrument=True, profile_out="", e2e_seconds=1.0):
    """Builds the net at `B` images per GPU and measures it. `total_images`: a fixed job split over the ranks (B = its share)."""
    from msnhnet_b200 import _ffi, sharding, synth, topologies
    from msnhnet_b200.net import Net
    torch = D.torch
    net, size, _, _, gflop = WORKLOADS[workload]
    text = topologies.NETS[net](size=size)
    blob = synth.make_blob(text, synth.load_factors(net))
    lo, hi = sharding.weak_job(B, D.rank, D.world)
    images = synth.make_images(hi - lo, 3, size, size, seed=synth.IMAGE_SEED + lo)
    pinned = torch.empty(images.shape, dtype=torch.float32).pin_memory()
    pinned.copy_(torch.from_numpy(images))
    host_images = pinned.numpy()
    g = Net(text, blob, fp16, batch=B, device=D.local_rank)
    klib = _ffi.kernel_lib()
    plan = C.c_void_p(g.lib.msnhB200PlanHandle())
    ctx = C.c_void_p(g.lib.msnhB200CtxHandle())

    def kcheck(rc):
        if rc != 0:
            raise RuntimeError(klib.msnh_b200_last_error(ctx).decode())

    res = {"workload": workload, "per_gpu_batch": B, "dtype": "f16" if fp16 else "f32 (tf32 products)"}
    # ---- device-resident throughput: inputs in HBM, forwards between two CUDA events ----
    g.forward(host_images)                      # fills the staging buffer (and is the first warm-up)
    ms = C.c_float()
    kcheck(klib.msnh_b200_plan_run_timed(plan, B, max(warmup - 1, 1), C.byref(ms)))
    # how many blocks of `steps` steps fill min_seconds: from one untimed block, the same number on every rank
    kcheck(klib.msnh_b200_plan_run_timed(plan, B, steps, C.byref(ms)))
    blocks = int(D.max(max(1, math.ceil(min_seconds * 1000.0 / max(ms.value, 1e-3)))))
    blocks = min(blocks, 100000)
    total_steps = blocks * steps
    sampler = ClockSampler(D.local_rank)
    sampler.start()
    probe = ClockProbe(klib, D.local_rank, int(min(60000, max(50, min_seconds * 1500 + 500))))
    D.barrier()
    kcheck(klib.msnh_b200_plan_run_timed(plan, B, total_steps, C.byref(ms)))
    D.barrier()
    eff = probe.stop()
    clocks = sampler.stop()
    if eff:
        clocks.update(eff)
    total_ms = D.max(float(ms.value))
    res.update(value=D.world * B * total_steps / (total_ms / 1000.0), steps=total_steps, ms_per_step=total_ms / total_steps, timed_region_s=total_ms / 1000.0, clocks=clocks)

    # ---- end to end through the reference-facing call: pinned host images in, boxes / logits out ----
    # One streaming call over e2e_steps batches (msnhB200RunYoloStream / RunClassifyStream): every step copies its
    # batch from pinned host memory, runs the forward, reads the result back and (detectors) runs the reference's
    # host NMS; copy-in, forward and NMS of neighbouring steps overlap. The call is repeated until e2e_seconds have passed.
    if e2e:
        # batches per streaming call: at least 40 where the pinned copy of them stays within ~3 GB, so that the pipeline's
        # fill (the first batch's copy-in, about one step) is a small part of a call
        e2e_steps = max(3, min(max(steps, 40), 64, int(3.2e9 // max(1, images.nbytes))))
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

        def timed_calls():
            user_call(min(3, e2e_steps))            # warm-up (allocates the streaming slots)
            D.barrier()
            t0 = time.perf_counter()
            user_call(e2e_steps)
            reps = int(D.max(max(1, math.ceil(e2e_seconds / max(time.perf_counter() - t0, 1e-4)))))
            D.barrier()
            t0 = time.perf_counter()
            for _ in range(reps):
                user_call(e2e_steps)
            dt = D.max(time.perf_counter() - t0)
            D.barrier()
            return D.world * B * e2e_steps * reps / dt, reps
        e2e_value, reps = timed_calls()
        t0 = time.perf_counter()
        user_call(1)                                # single synchronous call, for the latency of one batch
        e2e_single_ms = (time.perf_counter() - t0) * 1000.0
        h2d = int(host_images.nbytes)
        if g.is_yolo:
            d2h = int(4096 * 32 * B + 4 * B)        # fixed-size pinned slot: up to 4096 candidate rows per image + counts
            n_boxes = int(sum(counts[i] for i in range(B)))
        else:
            d2h = int(np.prod(g.last_shape) * 4 * B)
            n_boxes = 0
        res["e2e"] = {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps * reps,
                      "single_batch_ms": e2e_single_ms, "boxes_first_batch": n_boxes,
                      "call": ("msnhB200RunYoloStream (per step: H2D of pinned CHW float images, forward, candidate D2H, host NMS; steps pipelined)" if g.is_yolo else "msnhB200RunClassifyStream")
                              + f", {reps} calls of {e2e_steps} steps"}
        # The same call for raw 8-bit images of the net's input size (what the reference's runYoloList / runClassifyList
        # take): a quarter of the bytes over PCIe, the preprocessing on the device.
        u8 = torch.empty((e2e_steps, hi - lo, size, size, 3), dtype=torch.uint8).pin_memory()
        u8.copy_(torch.from_numpy(np.random.default_rng(7).integers(0, 256, (1, hi - lo, size, size, 3), dtype=np.uint8)).expand(e2e_steps, -1, -1, -1, -1))
        host_u8 = u8.numpy()
        float_call = user_call
        if g.is_yolo:
            def user_call(nb):      # noqa: F811
                rc = g.lib.msnhB200RunYoloStreamU8(C.byref(msg), host_u8.ctypes.data_as(C.c_void_p), size, size, 1, nb, boxes, max_boxes, counts)
                if rc != 1:
                    raise RuntimeError(msg.value.decode())
        else:
            def user_call(nb):      # noqa: F811
                rc = g.lib.msnhB200RunClassifyStreamU8(C.byref(msg), host_u8.ctypes.data_as(C.c_void_p), size, size, _ffi.PREP_UNIT, 1, None, None, nb,
                                                       out.ctypes.data_as(C.POINTER(C.c_float)), out.size)
                if rc != 1:
                    raise RuntimeError(msg.value.decode())
        v, reps_u8 = timed_calls()
        res["e2e"]["u8_input"] = {"value": v, "unit": "images/s", "h2d_bytes_per_step": int(host_u8[0].nbytes),
                                  "call": ("msnhB200RunYoloStreamU8" if g.is_yolo else "msnhB200RunClassifyStreamU8") + f" (8-bit HWC images of {size}x{size}, preprocessing on the device), {reps_u8} calls of {e2e_steps} steps"}
        user_call = float_call
        if dev_nms and g.is_yolo:
            # the same streaming call with the score sort + NMS on the device (only kept boxes cross PCIe)
            g.set_device_nms(True)
            v, _ = timed_calls()
            res["e2e"]["with_device_nms"] = {"value": v, "unit": "images/s", "boxes_first_batch": int(sum(counts[i] for i in range(B)))}
            g.set_device_nms(False)

    # ---- per-kernel device time of the same step (events between consecutive launches) ----
    n_launch, arena = C.c_int(), C.c_size_t()
    klib.msnh_b200_plan_stats(plan, C.byref(n_launch), C.byref(arena))
    res.update(launches_per_step=int(n_launch.value), gpu_launches=int(n_launch.value) * total_steps, arena_bytes=int(arena.value))
    if instrument:
        pk = peaks()
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
        top = max(by_kernel.items(), key=lambda kv: kv[1]["ms"])
        conv = by_kernel.get("conv_umma")
        if conv and conv["ms"] > 0 and conv["ms"] >= 0.5 * top[1]["ms"]:
            # Duration of the conv launches inside the timed region: the region's own device time per step (graph
            # launches with programmatic dependent launch, CUDA events on the plan's stream) times the conv kernels'
            # share of the per-launch event timings of the same step. The per-launch timings themselves run kernel by
            # kernel (an event between every two launches), so their sum is larger than the step and is reported beside.
            share = conv["ms"] / step_ms_sum
            conv_ms = res["ms_per_step"] * share
            achieved = conv["flops"] / (conv_ms / 1000.0) / 1e12
            traffic = MEASURED_CONV_DRAM_BYTES.get((workload, B, "f16" if fp16 else "f32"))
            res["roofline"] = {"kernel": "conv_umma_kernel", "bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                               "frac_of_burst_peak": achieved / pk["tflops_burst"], "peak_burst": pk["tflops_burst"],
                               "traffic": traffic, "traffic_note": "dram__bytes_read+write summed over the conv launches of one step (one ncu capture, profiles/); algorithmic bytes of the same launches: %.3e" % conv["bytes"],
                               "peak_source": pk["source"] + " (sustained dense 16-bit tensor throughput; frac_of_burst_peak is against the burst figure)", "launches_per_step": conv["launches"], "ms_per_step": conv_ms,
                               "ms_per_step_launch_by_launch": conv["ms"], "achieved_launch_by_launch": conv["flops"] / (conv["ms"] / 1000.0) / 1e12,
                               "share_of_step": share, "note": "algorithmic conv FLOPs of one step / (device time of the timed step x conv share of per-launch CUDA-event timings)"}
        else:
            k = top[1]
            achieved = k["bytes"] / (k["ms"] / 1000.0) / 1e9
            res["roofline"] = {"kernel": top[0], "bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                               "note": "algorithmic bytes of the kernel's launches of one step / their per-launch CUDA-event time"}
        res["kernels"] = {}
        for name, v in sorted(by_kernel.items(), key=lambda kv: -kv[1]["ms"]):
            e = {"launches": v["launches"], "ms": round(v["ms"], 4)}
            if v["ms"] > 0 and v["flops"] > 0:
                e["tflops"] = round(v["flops"] / (v["ms"] * 1e-3) / 1e12, 1)
                e["tensor_frac"] = round(e["tflops"] / pk["tflops"], 3)
            if v["ms"] > 0 and v["bytes"] > 0:
                e["gbs"] = round(v["bytes"] / (v["ms"] * 1e-3) / 1e9, 1)
                e["hbm_frac"] = round(e["gbs"] / pk["hbm_gbs"], 3)
            res["kernels"][name] = e
        if profile_out and D.rank == 0:
            with open(profile_out, "w") as f:
                f.write(layer_table(desc, per, pk, f"Every launch of one step: {workload}, {B} images, {'fp16' if fp16 else 'fp32'} (python bench.py --workload {workload} --profile-out <file>)"))
                f.write("\n## By kernel\n\n| kernel | launches | ms | share | TFLOP/s | GB/s |\n|---|---|---|---|---|---|\n")
                for name, k in sorted(by_kernel.items(), key=lambda kv: -kv[1]["ms"]):
                    f.write(f"| {name} | {k['launches']} | {k['ms']:.4f} | {k['ms'] / step_ms_sum:.3f} | {k['flops'] / max(k['ms'], 1e-9) / 1e9:.1f} | {k['bytes'] / max(k['ms'], 1e-9) / 1e6:.1f} |\n")
                f.write(f"\nTimed step (graph replay): {res['ms_per_step']:.4f} ms; sum of the per-launch figures: {step_ms_sum:.4f} ms.\n")
    if total_images is not None:
        res["images_total"] = total_images
    g.close()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS))
    ap.add_argument("--per-gpu-batch", type=int, default=0)
    ap.add_argument("--dtype", default="", choices=["", "fp16", "fp32"])
    ap.add_argument("--min-seconds", type=float, default=2.0, help="device time the timed region has to fill (blocks of --steps steps)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the other workloads and the fixed-size jobs")
    ap.add_argument("--profile-out", default="", help="markdown table of every launch of one step")
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

    D = Dist()
    head = measure(D, args.workload, B, fp16, args.steps, args.warmup, args.min_seconds, e2e=True, dev_nms=True, instrument=True, profile_out=args.profile_out)
    extras = args.workload == HEADLINE and not args.no_extras and not args.per_gpu_batch and not args.dtype
    others, fixed = [], []
    if extras:
        for w in OTHERS:
            n2, s2, b2, d2, _ = WORKLOADS[w]
            r = measure(D, w, b2, d2 == "fp16", max(5, min(args.steps, 20)), 3, 0.3, e2e=True, dev_nms=False, instrument=True, e2e_seconds=0.3)
            r.pop("gpu_launches", None); r.pop("arena_bytes", None)
            others.append(r)
        for w, total in FIXED_JOBS:
            if total % D.world:
                continue
            n2, s2, b2, d2, _ = WORKLOADS[w]
            r = measure(D, w, total // D.world, d2 == "fp16", 5, 3, 0.5, total_images=total, e2e=False, instrument=False)
            fixed.append({k: r[k] for k in ("workload", "images_total", "per_gpu_batch", "value", "ms_per_step", "steps", "timed_region_s")})
    cpu = None
    if D.rank == 0 and D.world == 1 and not args.no_cpu_baseline:
        n_img = {"yolov4": 10, "yolov5m": 20}.get(net, 100)
        ips, kind, threads, sample, details = reference_cpu(net, size, 1, n_img, budget_s=45.0)
        cpu = dict({"value": ips, "unit": "images/s", "cores": threads, "kind": kind, "sample": sample}, **details)
    if D.rank == 0:
        line = {"metric": "images/sec", "value": head["value"], "unit": "images/s", "n_gpus": D.world, "steps": head["steps"], "warmup": args.warmup,
                "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": head["dtype"],
                "data": "synthetic", "config": config, "clocks": head["clocks"], "timed_region_s": head["timed_region_s"],
                "steps_note": f"{head['steps'] // args.steps} blocks of --steps {args.steps} steps in one timed region",
                "e2e": head.get("e2e"), "gpu_launches": head["gpu_launches"], "launches_per_step": head["launches_per_step"],
                "roofline": head.get("roofline"), "cpu_baseline": cpu, "kernels": head.get("kernels"), "arena_bytes": head["arena_bytes"]}
        if extras:
            line["other_workloads"] = others
            line["fixed_jobs"] = fixed
        print(json.dumps(line), flush=True)
    D.close()


if __name__ == "__main__":
    main()
