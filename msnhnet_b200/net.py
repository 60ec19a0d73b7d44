"""Python face of the reference-facing C API (include/msnhnet_capi.h): the process-global net driven
through ctypes. Used by the tests, bench.py and smoke(); it holds no compute of its own."""
import ctypes as C

import numpy as np

from . import _ffi


class Net:
    """The process-global net of the C API (include/msnhnet_capi.h)."""

    def __init__(self, text, blob, fp16, batch=1, flags=0, device=0):
        self.lib = _ffi.host_lib()
        self.msg = C.c_char_p()
        assert self.lib.initMsnhnet() == 1
        self.lib.msnhB200SetOptions(device, batch, flags)
        blob = np.ascontiguousarray(blob, np.float32)
        rc = self.lib.msnhB200BuildFromMemory(C.byref(self.msg), text.encode(), blob.ctypes.data_as(C.POINTER(C.c_float)), blob.size, 1 if fp16 else 0)
        if rc != 1:
            raise RuntimeError(self.error())
        self.batch = batch
        layers, wc, isy, b, lc, lh, lw = C.c_int(), C.c_size_t(), C.c_int(), C.c_int(), C.c_int(), C.c_int(), C.c_int()
        ct, nt = C.c_float(), C.c_float()
        self.lib.msnhB200GetInfo(C.byref(layers), C.byref(wc), C.byref(isy), C.byref(b), C.byref(lc), C.byref(lh), C.byref(lw), C.byref(ct), C.byref(nt))
        self.n_layers, self.is_yolo, self.last_shape = layers.value, bool(isy.value), (lc.value, lh.value, lw.value)
        self.conf_thresh, self.nms_thresh = ct.value, nt.value

    def set_device_nms(self, on):
        """Score sort + NMS of the yolo calls on the device (msnhB200SetDeviceNms) instead of on the host."""
        assert self.lib.msnhB200SetDeviceNms(1 if on else 0) == 1

    def error(self):
        return self.msg.value.decode() if self.msg.value else "unknown error"

    def _check(self, rc):
        if rc != 1:
            raise RuntimeError(self.error())

    def classify(self, images):
        images = np.ascontiguousarray(images, np.float32)
        n = images.shape[0]
        out = np.empty((n,) + self.last_shape, np.float32)
        self._check(self.lib.msnhB200RunClassifyBatch(C.byref(self.msg), images.ctypes.data_as(C.c_void_p), n, out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def yolo(self, images, max_boxes=4096):
        images = np.ascontiguousarray(images, np.float32)
        n = images.shape[0]
        boxes = (_ffi.BBox * (n * max_boxes))()
        counts = (C.c_int * n)()
        self._check(self.lib.msnhB200RunYoloBatch(C.byref(self.msg), images.ctypes.data_as(C.c_void_p), n, boxes, max_boxes, counts))
        out = []
        for i in range(n):
            rows = np.array([[b.x, b.y, b.w, b.h, b.conf, b.bestClsConf, b.bestClsIdx] for b in boxes[i * max_boxes: i * max_boxes + counts[i]]], np.float32).reshape(-1, 7)
            out.append(rows)
        return out

    def yolo_stream(self, images, max_boxes=4096):
        """images: [n_batches * batch, C, H, W] in (ideally pinned) host memory -> per-image box rows."""
        images = np.ascontiguousarray(images, np.float32)
        n = images.shape[0]
        assert n % self.batch == 0
        boxes = (_ffi.BBox * (n * max_boxes))()
        counts = (C.c_int * n)()
        self._check(self.lib.msnhB200RunYoloStream(C.byref(self.msg), images.ctypes.data_as(C.c_void_p), n // self.batch, boxes, max_boxes, counts))
        return [np.array([[b.x, b.y, b.w, b.h, b.conf, b.bestClsConf, b.bestClsIdx] for b in boxes[i * max_boxes: i * max_boxes + counts[i]]],
                         np.float32).reshape(-1, 7) for i in range(n)]

    def yolo_stream_u8(self, images, swap_rgb=True, max_boxes=4096):
        """images: [n_batches * batch, H, W, 3] uint8 (raw RGB, any size) -> per-image box rows; preprocessing on the device."""
        images = np.ascontiguousarray(images, np.uint8)
        n, h, w = images.shape[0], images.shape[1], images.shape[2]
        assert n % self.batch == 0 and images.shape[3] == 3
        boxes = (_ffi.BBox * (n * max_boxes))()
        counts = (C.c_int * n)()
        self._check(self.lib.msnhB200RunYoloStreamU8(C.byref(self.msg), images.ctypes.data_as(C.c_void_p), w, h, 1 if swap_rgb else 0, n // self.batch,
                                                     boxes, max_boxes, counts))
        return [np.array([[b.x, b.y, b.w, b.h, b.conf, b.bestClsConf, b.bestClsIdx] for b in boxes[i * max_boxes: i * max_boxes + counts[i]]],
                         np.float32).reshape(-1, 7) for i in range(n)]

    def classify_stream_u8(self, images, prep_mode, swap_rgb=True, mean=None, std=None):
        images = np.ascontiguousarray(images, np.uint8)
        n, h, w = images.shape[0], images.shape[1], images.shape[2]
        assert n % self.batch == 0 and images.shape[3] == 3
        out = np.empty((n,) + self.last_shape, np.float32)
        f3 = lambda v: None if v is None else np.ascontiguousarray(v, np.float32).ctypes.data_as(C.POINTER(C.c_float))
        self._check(self.lib.msnhB200RunClassifyStreamU8(C.byref(self.msg), images.ctypes.data_as(C.c_void_p), w, h, prep_mode, 1 if swap_rgb else 0,
                                                         f3(mean), f3(std), n // self.batch, out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def classify_stream(self, images):
        images = np.ascontiguousarray(images, np.float32)
        n = images.shape[0]
        assert n % self.batch == 0
        out = np.empty((n,) + self.last_shape, np.float32)
        self._check(self.lib.msnhB200RunClassifyStream(C.byref(self.msg), images.ctypes.data_as(C.c_void_p), n // self.batch,
                                                       out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def forward(self, images):
        images = np.ascontiguousarray(images, np.float32)
        self._check(self.lib.msnhB200Forward(C.byref(self.msg), images.ctypes.data_as(C.c_void_p), images.shape[0]))

    def layer_output(self, layer, n_images):
        cap = 1 << 20
        while True:
            out = np.empty(cap, np.float32)
            c, h, w = C.c_int(), C.c_int(), C.c_int()
            rc = self.lib.msnhB200GetLayerOutput(C.byref(self.msg), layer, n_images, out.ctypes.data_as(C.POINTER(C.c_float)), cap, C.byref(c), C.byref(h), C.byref(w))
            if rc == 1:
                return out[: n_images * c.value * h.value * w.value].reshape(n_images, c.value, h.value, w.value).copy()
            err = self.error()
            if "need " in err:
                cap = int(err.split("need ")[1].split()[0])
                continue
            raise RuntimeError(err)

    def candidates(self, n_images, max_rows):
        rows = np.zeros((n_images, max_rows, 8), np.float32)
        counts = (C.c_int * n_images)()
        self._check(self.lib.msnhB200GetCandidates(C.byref(self.msg), n_images, rows.ctypes.data_as(C.POINTER(C.c_float)), max_rows, counts))
        return [rows[i, :counts[i]].copy() for i in range(n_images)]

    def kernel_ms(self):
        ms = C.c_float()
        self.lib.msnhB200KernelTimeMs(C.byref(ms))
        return ms.value

    def plan_describe(self):
        lib = _ffi.kernel_lib()
        return lib.msnh_b200_plan_describe(C.c_void_p(self.lib.msnhB200PlanHandle())).decode()

    def plan_profile(self, iters=3):
        lib = _ffi.kernel_lib()
        plan = C.c_void_p(self.lib.msnhB200PlanHandle())
        n, b = C.c_int(), C.c_size_t()
        lib.msnh_b200_plan_stats(plan, C.byref(n), C.byref(b))
        ms = (C.c_float * n.value)()
        rc = lib.msnh_b200_plan_profile(plan, iters, ms, n.value)
        if rc != 0:
            raise RuntimeError(lib.msnh_b200_last_error(C.c_void_p(self.lib.msnhB200CtxHandle())).decode())
        return list(ms), b.value

    def close(self):
        self.lib.dispose()


def host_postprocess(rows, nms_thresh, soft=False):
    """The host half of YoloOut on given candidate rows, through the C ABI."""
    lib = _ffi.host_lib()
    rows = np.ascontiguousarray(rows, np.float32)
    cap = max(1, len(rows))
    out = (_ffi.BBox * cap)()
    n = C.c_int()
    assert lib.msnhB200PostProcess(rows.ctypes.data_as(C.POINTER(C.c_float)), len(rows), nms_thresh, 1 if soft else 0, out, cap, C.byref(n)) == 1
    return np.array([[b.x, b.y, b.w, b.h, b.conf, b.bestClsConf, b.bestClsIdx] for b in out[: n.value]], np.float32).reshape(-1, 7)
