"""msnh_b200_yolo_collect_static: candidate collection for callers that cannot allocate.

Some users of the library run where cudaMalloc is off limits - inside a real-time loop or stream
callback, as a plugin with a fixed memory grant, or under a framework that owns all device memory.
For them the library offers one entry point whose scratch (the per-image append counters) is a
static device array instead of an allocation. This test drives it through the C ABI on buffers the
test owns (torch tensors stand in for the caller's pre-allocated memory) and checks, on two calls
in a row, that it returns exactly the rows the plan-based path (MSNH_OP_YOLO_COLLECT +
msnh_b200_plan_read_candidates) returns for the same decoded head. Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

from msnhnet_b200 import _ffi as ffi

pytestmark = pytest.mark.gpu


def plan_candidates(ctx, x, classes, thresh, anchors):
    """Decoded head (NCHW, host) and candidate rows per image from the existing plan path."""
    n, c, g, _ = x.shape
    ops = [ffi.make_op(ffi.OP_ACTIVATION, [ffi.INPUT], act=ffi.ACT_NONE),
           ffi.make_op(ffi.OP_YOLO, [0], yolo_type=40, yolo_classes=classes, yolo_anchors=anchors),
           ffi.make_op(ffi.OP_YOLO_COLLECT, [1], const_val=thresh)]
    ops[1].is_output = 1
    ops[2].is_output = 1
    plan = ffi.Plan(ctx, ops, (c, g, g), n, ffi.F32, 0)
    plan.finalize()
    plan.run(x)
    dec = plan.read_output(1, n)
    rows = plan.read_candidates(2, n)
    plan.close()
    return dec, rows


def static_candidates(lib, torch, dec_nchw, classes, thresh, max_rows):
    """The same through the allocation-free entry point, on caller-owned device buffers."""
    n, c, g, _ = dec_nchw.shape
    pitch = (c + 3) // 4 * 4
    nhwc = np.zeros((n, g, g, pitch), np.float32)
    nhwc[..., :c] = dec_nchw.transpose(0, 2, 3, 1)
    d_dec = torch.from_numpy(nhwc).cuda()
    d_rows = torch.zeros((n, max_rows, 8), dtype=torch.float32, device="cuda")
    d_counts = torch.full((n,), -1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    rc = lib.msnh_b200_yolo_collect_static(C.c_void_p(d_dec.data_ptr()), n, g, g, pitch, classes, C.c_float(thresh), 0,
                                           C.c_void_p(d_rows.data_ptr()), max_rows, C.c_void_p(d_counts.data_ptr()), None)
    assert rc == ffi.OK, lib.msnh_b200_static_last_error().decode()
    torch.cuda.synchronize()
    counts = d_counts.cpu().numpy()
    rows = d_rows.cpu().numpy()
    out = []
    for i in range(n):
        r = rows[i, :counts[i]]
        out.append(r[np.argsort(r[:, 7], kind="stable")])       # the reference's scan order
    return out


def test_static_collect_matches_plan_path_twice():
    torch = pytest.importorskip("torch")
    lib = ffi.kernel_lib()
    ctx = ffi.Context(0)
    try:
        classes, g, anchors = 4, 9, [10, 13, 16, 30, 33, 23]
        c = 3 * (5 + classes)
        rng = np.random.default_rng(21)
        # two different inputs, the second with fewer images: stale counters from the first call must not leak
        xs = [(rng.standard_normal((3, c, g, g)) * 1.5).astype(np.float32), (rng.standard_normal((2, c, g, g)) * 1.5).astype(np.float32)]
        for call, (x, thresh) in enumerate(zip(xs, (0.5, 0.3))):
            dec, want = plan_candidates(ctx, x, classes, thresh, anchors)
            got = static_candidates(lib, torch, dec, classes, thresh, max_rows=3 * g * g)
            assert len(got) == len(want)
            for i in range(len(want)):
                assert got[i].shape == want[i].shape, f"call {call} image {i}"
                assert np.array_equal(got[i], want[i])           # bit-identical rows (tolerance of the collect tests: exact)
                assert len(want[i]) > 0
    finally:
        ctx.close()


def test_static_collect_rejects_oversize_and_bad_arguments():
    torch = pytest.importorskip("torch")
    lib = ffi.kernel_lib()
    buf = torch.zeros(64, dtype=torch.float32, device="cuda")
    cnt = torch.zeros(4, dtype=torch.int32, device="cuda")
    p, q = C.c_void_p(buf.data_ptr()), C.c_void_p(cnt.data_ptr())
    assert lib.msnh_b200_yolo_collect_static(p, 1025, 1, 1, 27, 4, C.c_float(0.5), 0, p, 1, q, None) == 1
    assert b"1024" in lib.msnh_b200_static_last_error()
    assert lib.msnh_b200_yolo_collect_static(None, 1, 1, 1, 27, 4, C.c_float(0.5), 0, p, 1, q, None) == 1
    assert lib.msnh_b200_yolo_collect_static(p, 1, 1, 1, 8, 4, C.c_float(0.5), 0, p, 1, q, None) == 1      # pitch too small
