"""ctypes bindings of the two native libraries (tests, bench and smoke drive the C ABI through these).

`kernel_lib()` -> libmsnh_b200.so   (include/msnh_b200.h)
`host_lib()`   -> libmsnhnet_host.so (include/msnhnet_capi.h)

Nothing here computes anything: a missing library is an ImportError-like failure, never a fallback.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
MAX_IN = 8

# status codes / enums (include/msnh_b200.h)
OK = 0
F32, F16 = 0, 1
(ACT_NONE, ACT_LOGISTIC, ACT_LOGGY, ACT_RELU, ACT_RELU6, ACT_HARD_SWISH, ACT_ELU, ACT_SELU, ACT_RELIE, ACT_RAMP,
 ACT_LEAKY, ACT_TANH, ACT_STAIR, ACT_HARDTAN, ACT_SOFT_PLUS, ACT_PLSE, ACT_LHTAN, ACT_MISH, ACT_SWISH) = range(19)
(OP_CONV, OP_BATCHNORM, OP_ACTIVATION, OP_MAXPOOL, OP_AVGPOOL, OP_UPSAMPLE, OP_CONCAT, OP_ADD, OP_SLICE, OP_PAD,
 OP_CONNECTED, OP_SOFTMAX, OP_YOLO, OP_IDENTITY, OP_BINARY, OP_YOLO_COLLECT, OP_DECONV, OP_CLIP, OP_REMAP,
 OP_REDUCE, OP_PRELU) = range(1, 22)
UPSAMPLE_NEAREST, UPSAMPLE_BILINEAR = 0, 1
REMAP_VIEW, REMAP_PERMUTE, REMAP_PIXSHF = 0, 1, 2
W_WEIGHTS, W_BIAS, W_BN_SCALE, W_BN_BIAS, W_BN_MEAN, W_BN_VAR = range(6)
PLAN_NO_GRAPH, PLAN_NO_FUSION, PLAN_KEEP_ALL, PLAN_NO_TENSOR_CORE, PLAN_TRACE, PLAN_TF32_DETECT = 1, 2, 4, 8, 16, 32
INPUT = -1


class Op(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("n_in", C.c_int32), ("inp", C.c_int32 * MAX_IN),
        ("filters", C.c_int32),
        ("k_h", C.c_int32), ("k_w", C.c_int32), ("stride_h", C.c_int32), ("stride_w", C.c_int32),
        ("pad_h", C.c_int32), ("pad_w", C.c_int32), ("dil_h", C.c_int32), ("dil_w", C.c_int32), ("groups", C.c_int32),
        ("out_h", C.c_int32), ("out_w", C.c_int32),
        ("pad_top", C.c_int32), ("pad_down", C.c_int32), ("pad_left", C.c_int32), ("pad_right", C.c_int32),
        ("slice_start", C.c_int32 * 3), ("slice_step", C.c_int32 * 3),
        ("route_groups", C.c_int32), ("route_group_id", C.c_int32),
        ("has_bn", C.c_int32), ("has_bias", C.c_int32), ("bn_eps", C.c_float),
        ("act", C.c_int32), ("act_param", C.c_float),
        ("scale", C.c_float), ("const_val", C.c_float),
        ("binary_kind", C.c_int32), ("binary_const", C.c_int32),
        ("softmax_groups", C.c_int32), ("softmax_temperature", C.c_float),
        ("yolo_type", C.c_int32), ("yolo_classes", C.c_int32), ("yolo_anchors", C.c_float * 6),
        ("is_output", C.c_int32), ("upsample_mode", C.c_int32), ("align_corners", C.c_int32),
        ("remap_kind", C.c_int32), ("remap_dims", C.c_int32 * 3), ("out_c", C.c_int32),
    ]


def make_op(kind, inputs, **kw):
    op = Op()
    op.kind = kind
    op.n_in = len(inputs)
    for i, v in enumerate(inputs):
        op.inp[i] = v
    op.k_h = op.k_w = op.stride_h = op.stride_w = op.dil_h = op.dil_w = op.groups = 1
    op.bn_eps = 1e-5
    op.scale = 1.0
    op.route_groups = 1
    op.softmax_groups = 1
    op.softmax_temperature = 1.0
    for i in range(3):
        op.slice_step[i] = 1
    for k, v in kw.items():
        if k in ("slice_start", "slice_step", "yolo_anchors", "remap_dims"):
            arr = getattr(op, k)
            for i, x in enumerate(v):
                arr[i] = x
        else:
            if not hasattr(op, k):
                raise AttributeError(k)
            setattr(op, k, v)
    return op


_kernel = None
_host = None


def kernel_lib():
    """Loads libmsnh_b200.so and declares every entry point of include/msnh_b200.h."""
    global _kernel
    if _kernel is not None:
        return _kernel
    path = os.path.join(HERE, "libmsnh_b200.so")
    if not os.path.exists(path):
        raise RuntimeError("libmsnh_b200.so is not built: run `python -m msnhnet_b200.build`")
    lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
    vp, i32, f32p = C.c_void_p, C.c_int, C.POINTER(C.c_float)
    lib.msnh_b200_device_count.argtypes = [C.POINTER(i32)]
    lib.msnh_b200_ctx_create.argtypes = [i32, C.POINTER(vp)]
    lib.msnh_b200_ctx_destroy.argtypes = [vp]
    lib.msnh_b200_last_error.argtypes = [vp]
    lib.msnh_b200_last_error.restype = C.c_char_p
    lib.msnh_b200_host_alloc.argtypes = [vp, C.c_size_t, C.POINTER(vp)]
    lib.msnh_b200_host_free.argtypes = [vp, vp]
    lib.msnh_b200_plan_create.argtypes = [vp, C.POINTER(Op), i32, i32, i32, i32, i32, i32, C.c_uint32, C.POINTER(vp)]
    lib.msnh_b200_plan_op_shape.argtypes = [vp, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]
    lib.msnh_b200_plan_weight_count.argtypes = [vp, i32, i32, C.POINTER(C.c_size_t)]
    lib.msnh_b200_plan_set_weights.argtypes = [vp, i32, i32, f32p, C.c_size_t]
    lib.msnh_b200_plan_finalize.argtypes = [vp]
    lib.msnh_b200_plan_use_pack.argtypes = [vp, C.c_char_p, C.c_uint64, C.POINTER(i32)]
    lib.msnh_b200_plan_run.argtypes = [vp, vp, i32]
    lib.msnh_b200_plan_run_device.argtypes = [vp, vp, i32, i32]
    lib.msnh_b200_plan_run_timed.argtypes = [vp, i32, i32, f32p]
    lib.msnh_b200_plan_run_instrumented.argtypes = [vp, i32, i32, f32p, i32]
    lib.msnh_b200_plan_stream_push.argtypes = [vp, i32, vp, i32]
    lib.msnh_b200_plan_stream_pop.argtypes = [vp, f32p, C.c_size_t, i32, C.POINTER(i32), C.POINTER(i32)]
    lib.msnh_b200_plan_stream_reset.argtypes = [vp]
    lib.msnh_b200_plan_stream_push_u8.argtypes = [vp, i32, vp, i32, i32, i32, i32, i32, f32p, f32p]
    lib.msnh_b200_plan_read_output.argtypes = [vp, i32, f32p, C.c_size_t]
    lib.msnh_b200_plan_read_candidates.argtypes = [vp, i32, i32, f32p, i32, C.POINTER(i32)]
    lib.msnh_b200_plan_input_buffer.argtypes = [vp, C.POINTER(vp)]
    lib.msnh_b200_plan_last_ms.argtypes = [vp, f32p]
    lib.msnh_b200_plan_stats.argtypes = [vp, C.POINTER(i32), C.POINTER(C.c_size_t)]
    lib.msnh_b200_plan_describe.argtypes = [vp]
    lib.msnh_b200_plan_describe.restype = C.c_char_p
    lib.msnh_b200_plan_profile.argtypes = [vp, i32, f32p, i32]
    lib.msnh_b200_plan_read_trace.argtypes = [vp, i32, C.POINTER(C.c_longlong), i32, C.POINTER(i32)]
    lib.msnh_b200_plan_destroy.argtypes = [vp]
    lib.msnh_b200_yolo_collect_static.argtypes = [vp, i32, i32, i32, i32, i32, C.c_float, i32, vp, i32, vp, vp]
    lib.msnh_b200_static_last_error.restype = C.c_char_p
    f64p = C.POINTER(C.c_double)
    lib.msnh_b200_clock_probe_start.argtypes = [i32, i32, C.POINTER(vp)]
    lib.msnh_b200_clock_probe_stop.argtypes = [vp, f64p, f64p, f64p, C.POINTER(i32)]
    _kernel = lib
    return lib


PREP_UNIT, PREP_PAD_SQUARE, PREP_GOOGLENET, PREP_TRANSFORMED, PREP_CAFFE = 0, 1, 2, 3, 4   # MSNH_PREP_* of include/msnh_b200.h

KERNEL_SYMBOLS = [
    "msnh_b200_device_count", "msnh_b200_ctx_create", "msnh_b200_ctx_destroy", "msnh_b200_last_error",
    "msnh_b200_host_alloc", "msnh_b200_host_free", "msnh_b200_plan_create", "msnh_b200_plan_op_shape",
    "msnh_b200_plan_weight_count", "msnh_b200_plan_set_weights", "msnh_b200_plan_finalize", "msnh_b200_plan_use_pack", "msnh_b200_plan_run",
    "msnh_b200_plan_run_device", "msnh_b200_plan_run_timed", "msnh_b200_plan_run_instrumented", "msnh_b200_plan_stream_push", "msnh_b200_plan_stream_pop", "msnh_b200_plan_stream_reset", "msnh_b200_plan_stream_push_u8", "msnh_b200_plan_read_output", "msnh_b200_plan_read_candidates", "msnh_b200_plan_preprocess_u8", "msnh_b200_plan_nms", "msnh_b200_plan_stream_nms",
    "msnh_b200_plan_input_buffer", "msnh_b200_plan_last_ms", "msnh_b200_plan_stats", "msnh_b200_plan_describe",
    "msnh_b200_plan_profile", "msnh_b200_plan_read_trace", "msnh_b200_plan_destroy",
    "msnh_b200_yolo_collect_static", "msnh_b200_static_last_error",
    "msnh_b200_clock_probe_start", "msnh_b200_clock_probe_stop",
]


class BBox(C.Structure):
    _fields_ = [("x", C.c_float), ("y", C.c_float), ("w", C.c_float), ("h", C.c_float), ("conf", C.c_float),
                ("bestClsConf", C.c_float), ("bestClsIdx", C.c_uint32), ("angle", C.c_float)]


class BBoxContainer(C.Structure):
    _fields_ = [("boxes", BBox * 1024)]


HOST_SYMBOLS = [
    # the reference's 13 entry points
    "initMsnhnet", "buildMsnhnet", "runClassifyFile", "runClassifyList", "runClassifyNoPred", "runYoloFile", "runYoloList",
    "dispose", "withGPU", "withCUDNN", "getCpuForwardTime", "getGpuForwardTime", "getInputDim",
    # additions
    "msnhB200SetOptions", "msnhB200SetPackCache", "msnhB200LastLoadUsedPack", "msnhB200SetDeviceNms", "msnhB200BuildFromMemory", "msnhB200Inspect", "msnhB200WeightLayout", "msnhB200RunClassifyBatch",
    "msnhB200OpList", "msnhB200RunYoloBatch", "msnhB200RunYoloStream", "msnhB200RunClassifyStream", "msnhB200RunYoloStreamU8", "msnhB200RunClassifyStreamU8", "msnhB200Forward", "msnhB200ForwardResident", "msnhB200GetLayerOutput", "msnhB200GetCandidates",
    "msnhB200PostProcess", "msnhB200GetInfo", "msnhB200KernelTimeMs", "msnhB200PlanHandle", "msnhB200CtxHandle",
]


def host_lib():
    """Loads libmsnhnet_host.so (the NetBuilder mirror + C API of include/msnhnet_capi.h)."""
    global _host
    if _host is not None:
        return _host
    kernel_lib()
    path = os.path.join(HERE, "libmsnhnet_host.so")
    if not os.path.exists(path):
        raise RuntimeError("libmsnhnet_host.so is not built: run `python -m msnhnet_b200.build`")
    lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
    cpp, i32, f32p, ip = C.POINTER(C.c_char_p), C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_int)
    lib.buildMsnhnet.argtypes = [cpp, C.c_char_p, C.c_char_p, i32, i32]
    lib.runClassifyNoPred.argtypes = [cpp, f32p, i32, ip, i32]
    lib.runClassifyFile.argtypes = [cpp, C.c_char_p, ip, i32, i32, f32p, f32p]
    lib.runClassifyList.argtypes = [cpp, C.c_void_p, i32, i32, i32, ip, i32, i32, i32, f32p, f32p]
    lib.runYoloFile.argtypes = [cpp, C.c_char_p, C.POINTER(BBoxContainer), ip, i32]
    lib.runYoloList.argtypes = [cpp, C.c_void_p, i32, i32, i32, C.POINTER(BBoxContainer), ip, i32, i32]
    lib.withGPU.argtypes = [ip]
    lib.withCUDNN.argtypes = [ip]
    lib.getCpuForwardTime.argtypes = [f32p]
    lib.getGpuForwardTime.argtypes = [f32p]
    lib.getInputDim.argtypes = [ip, ip, ip]
    lib.msnhB200SetOptions.argtypes = [i32, i32, C.c_uint]
    lib.msnhB200BuildFromMemory.argtypes = [cpp, C.c_char_p, f32p, C.c_size_t, i32]
    lib.msnhB200Inspect.argtypes = [cpp, C.c_char_p, ip, C.POINTER(C.c_size_t), ip]
    lib.msnhB200WeightLayout.argtypes = [cpp, C.c_char_p]
    lib.msnhB200OpList.argtypes = [cpp, C.c_char_p]
    lib.msnhB200RunClassifyBatch.argtypes = [cpp, C.c_void_p, i32, f32p, C.c_size_t]
    lib.msnhB200RunYoloBatch.argtypes = [cpp, C.c_void_p, i32, C.POINTER(BBox), i32, ip]
    lib.msnhB200RunYoloStream.argtypes = [cpp, C.c_void_p, i32, C.POINTER(BBox), i32, ip]
    lib.msnhB200RunClassifyStream.argtypes = [cpp, C.c_void_p, i32, f32p, C.c_size_t]
    lib.msnhB200RunYoloStreamU8.argtypes = [cpp, C.c_void_p, i32, i32, i32, i32, C.POINTER(BBox), i32, ip]
    lib.msnhB200RunClassifyStreamU8.argtypes = [cpp, C.c_void_p, i32, i32, i32, i32, f32p, f32p, i32, f32p, C.c_size_t]
    lib.msnhB200Forward.argtypes = [cpp, C.c_void_p, i32]
    lib.msnhB200ForwardResident.argtypes = [cpp, i32, i32]
    lib.msnhB200GetLayerOutput.argtypes = [cpp, i32, i32, f32p, C.c_size_t, ip, ip, ip]
    lib.msnhB200GetCandidates.argtypes = [cpp, i32, f32p, i32, ip]
    lib.msnhB200PostProcess.argtypes = [f32p, i32, C.c_float, i32, C.POINTER(BBox), i32, ip]
    lib.msnhB200GetInfo.argtypes = [ip, C.POINTER(C.c_size_t), ip, ip, ip, ip, ip, f32p, f32p]
    lib.msnhB200KernelTimeMs.argtypes = [f32p]
    lib.msnhB200PlanHandle.restype = C.c_void_p
    lib.msnhB200CtxHandle.restype = C.c_void_p
    _host = lib
    return lib


class KernelError(RuntimeError):
    pass


class Context:
    """One per device (msnh_b200_ctx_*)."""

    def __init__(self, device=0):
        self.lib = kernel_lib()
        self.h = C.c_void_p()
        rc = self.lib.msnh_b200_ctx_create(device, C.byref(self.h))
        if rc != OK:
            raise KernelError(f"msnh_b200_ctx_create(device={device}) failed with status {rc}")

    def error(self):
        return self.lib.msnh_b200_last_error(self.h).decode()

    def check(self, rc):
        if rc != OK:
            raise KernelError(f"status {rc}: {self.error()}")

    def close(self):
        if self.h:
            self.lib.msnh_b200_ctx_destroy(self.h)
            self.h = C.c_void_p()


class Plan:
    """A list of primitive ops lowered to a launch plan (msnh_b200_plan_*)."""

    def __init__(self, ctx, ops, in_chw, batch, dtype, flags=0):
        self.ctx, self.lib = ctx, ctx.lib
        self.n_ops = len(ops)
        self.batch = batch
        self.in_chw = tuple(in_chw)
        arr = (Op * len(ops))(*ops)
        self.h = C.c_void_p()
        ctx.check(self.lib.msnh_b200_plan_create(ctx.h, arr, len(ops), in_chw[0], in_chw[1], in_chw[2], batch, dtype,
                                                 flags, C.byref(self.h)))

    def op_shape(self, op):
        c, h, w = C.c_int(), C.c_int(), C.c_int()
        self.ctx.check(self.lib.msnh_b200_plan_op_shape(self.h, op, C.byref(c), C.byref(h), C.byref(w)))
        return c.value, h.value, w.value

    def weight_count(self, op, slot):
        n = C.c_size_t()
        self.ctx.check(self.lib.msnh_b200_plan_weight_count(self.h, op, slot, C.byref(n)))
        return n.value

    def set_weights(self, op, slot, data):
        a = np.ascontiguousarray(data, dtype=np.float32).ravel()
        self.ctx.check(self.lib.msnh_b200_plan_set_weights(self.h, op, slot, a.ctypes.data_as(C.POINTER(C.c_float)), a.size))

    def use_pack(self, path, tag):
        """Registers a weight pack file; True when finalize will load it instead of repacking."""
        usable = C.c_int32()
        self.ctx.check(self.lib.msnh_b200_plan_use_pack(self.h, path.encode(), tag, C.byref(usable)))
        return bool(usable.value)

    def finalize(self):
        self.ctx.check(self.lib.msnh_b200_plan_finalize(self.h))

    def run(self, images):
        a = np.ascontiguousarray(images, dtype=np.float32)
        n = a.shape[0]
        self.ctx.check(self.lib.msnh_b200_plan_run(self.h, a.ctypes.data_as(C.c_void_p), n))

    def run_device(self, dev_ptr, n_images, sync=True):
        self.ctx.check(self.lib.msnh_b200_plan_run_device(self.h, C.c_void_p(dev_ptr), n_images, 1 if sync else 0))

    def input_buffer(self):
        p = C.c_void_p()
        self.ctx.check(self.lib.msnh_b200_plan_input_buffer(self.h, C.byref(p)))
        return p.value

    def preprocess_u8(self, image, slot, mode, swap_rgb, mean=None, std=None):
        """Raw HWC uint8 RGB image -> image slot of the plan's input buffer (msnh_b200_plan_preprocess_u8); run_device follows."""
        a = np.ascontiguousarray(image, dtype=np.uint8)
        h, w, c = a.shape
        assert c == 3
        m = (C.c_float * 3)(*mean) if mean is not None else None
        sd = (C.c_float * 3)(*std) if std is not None else None
        self.ctx.check(self.lib.msnh_b200_plan_preprocess_u8(self.h, a.ctypes.data_as(C.POINTER(C.c_ubyte)), w, h, slot, mode, 1 if swap_rgb else 0, m, sd))

    def read_output(self, op, n_images):
        c, h, w = self.op_shape(op)
        out = np.empty((n_images, c, h, w), dtype=np.float32)
        self.ctx.check(self.lib.msnh_b200_plan_read_output(self.h, op, out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def read_candidates(self, op, n_images, max_rows=None):
        if max_rows is None:
            max_rows = self.op_shape(op)[2]
        rows = np.zeros((n_images, max_rows, 8), dtype=np.float32)
        counts = (C.c_int * n_images)()
        self.ctx.check(self.lib.msnh_b200_plan_read_candidates(self.h, op, n_images, rows.ctypes.data_as(C.POINTER(C.c_float)),
                                                               max_rows, counts))
        return [rows[i, :counts[i]].copy() for i in range(n_images)]

    def last_ms(self):
        ms = C.c_float()
        self.ctx.check(self.lib.msnh_b200_plan_last_ms(self.h, C.byref(ms)))
        return ms.value

    def stats(self):
        n, b = C.c_int(), C.c_size_t()
        self.ctx.check(self.lib.msnh_b200_plan_stats(self.h, C.byref(n), C.byref(b)))
        return n.value, b.value

    def describe(self):
        return self.lib.msnh_b200_plan_describe(self.h).decode()

    def profile(self, iters=3):
        n, _ = self.stats()
        ms = (C.c_float * n)()
        self.ctx.check(self.lib.msnh_b200_plan_profile(self.h, iters, ms, n))
        return list(ms)

    def read_trace(self, launch):
        cap = 64 * 256
        buf = (C.c_longlong * cap)()
        n = C.c_int()
        self.ctx.check(self.lib.msnh_b200_plan_read_trace(self.h, launch, buf, cap, C.byref(n)))
        return np.frombuffer(buf, dtype=np.int64)[: n.value * 64].reshape(n.value, 64).copy()

    def close(self):
        if self.h:
            self.lib.msnh_b200_plan_destroy(self.h)
            self.h = C.c_void_p()
