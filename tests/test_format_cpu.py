"""Host-side logic on CPU: the .msnhnet / .msnhbin readers, block lowering, blob layout and the
exported C ABI. No compute call is made, so no GPU is needed."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import helpers as H
from msnhnet_b200 import _ffi, synth, topologies

# layer count and blob length of the reference's own model files for these architectures
EXPECTED = {
    "resnet18": (224, 13, 11699112),
    "yolov3_tiny": (416, 26, 8858734),
    "mobilenetv2": (224, 21, 3538984),
    "yolov4": (608, 103, 64429405),
    "yolov5m": (640, 318, 21845757),
}


def inspect(text):
    lib = _ffi.host_lib()
    msg, layers, wc, isy = C.c_char_p(), C.c_int(), C.c_size_t(), C.c_int()
    rc = lib.msnhB200Inspect(C.byref(msg), text.encode(), C.byref(layers), C.byref(wc), C.byref(isy))
    return rc, (msg.value or b"").decode(), layers.value, wc.value, isy.value


def test_kernel_library_exports_every_declared_symbol():
    lib = _ffi.kernel_lib()
    header = open(os.path.join(H.ROOT, "include", "msnh_b200.h")).read()
    for name in _ffi.KERNEL_SYMBOLS:
        assert name in header, name
        assert getattr(lib, name) is not None
    # every function the header declares is in the list (and therefore exported)
    import re
    declared = set(re.findall(r"\b(msnh_b200_\w+)\s*\(", header))
    assert declared == set(_ffi.KERNEL_SYMBOLS)


def test_host_library_exports_the_reference_c_api():
    lib = _ffi.host_lib()
    header = open(os.path.join(H.ROOT, "include", "msnhnet_capi.h")).read()
    for name in _ffi.HOST_SYMBOLS:
        assert name in header, name
        assert getattr(lib, name) is not None


@pytest.mark.parametrize("name", sorted(EXPECTED))
def test_topologies_parse_with_reference_counts(name):
    size, layers, weights = EXPECTED[name]
    rc, detail, n_layers, n_weights, is_yolo = inspect(topologies.NETS[name](size=size))
    assert rc == 1, detail
    assert (n_layers, n_weights) == (layers, weights)
    assert is_yolo == (1 if name.startswith("yolo") else 0)


def test_shapes_follow_the_reference_rules():
    rc, detail, *_ = inspect(topologies.yolov3_tiny(416))
    lines = detail.strip().split("\n")
    assert lines[0] == "0 Conv -> 16 x 416 x 416"
    assert lines[11] == "11 Padding -> 512 x 14 x 14"      # pad down/right by one
    assert lines[12] == "12 MaxPool -> 512 x 13 x 13"      # k2 s1 ceilMode 1
    assert lines[21] == "21 Route -> 384 x 26 x 26"        # concat 128 + 256
    rc, detail, *_ = inspect(topologies.yolov4(608))
    lines = detail.strip().split("\n")
    assert lines[62] == "62 ConcatBlock -> 2048 x 19 x 19"            # SPP concatblock: 13, 9, 5, identity


def test_negative_and_absolute_route_indices():
    text = "config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\n" \
           "conv:\n  filters: 4\n  kSize: 1\nconv:\n  filters: 6\n  kSize: 1\nroute:\n  layers: -1,0\n"
    rc, detail, n_layers, n_weights, _ = inspect(text)
    assert rc == 1 and n_layers == 3
    assert detail.strip().split("\n")[2] == "2 Route -> 10 x 8 x 8"
    assert n_weights == (4 * 3 + 4) + (6 * 4 + 6)           # weights + bias (useBias defaults to 1)


@pytest.mark.parametrize("text,needle", [
    ("conv:\n  filters: 4\n", "first node must be config"),
    ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nconv:\n  filters: 4\n  bogus: 1\n", "unknown key"),
    ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nconv:\n  filters: x\n", "can't convert to int"),
    ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nroute:\n  layers: 5\n", "does not name an earlier layer"),
    ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\ndeconv:\n  filters: 4\n  groups: 2\n", "not supported"),
        ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nlstm:\n  filters: 4\n", "not supported"),
        ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nview:\n  dim0: 5\n  dim1: 5\n  dim2: 5\n", "view op params error"),
        ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\npermute:\n  dim0: 1\n  dim1: 1\n  dim2: 0\n", "dims can't equal"),
        ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\npixshf:\n  factor: 2\n", "not divisible by factor"),
        ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nclip:\n  min: 2\n  max: 1\n", "[clip] min"),
        ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nreduction:\n  axis: 3\n", "axis must be"),
        ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nupsample:\n  type: cubic\n", "is not supported"),
    ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nconv:\n  filters: 255\n  kSize: 1\nyolo:\n  anchors: 1,2,3,4,5,6\n  classNum: 3\n", "class num error"),
    ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 4\nconv:\n  filters: 6\n  groups: 3\n", "groups must divide"),
    ("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\n", "no layers"),
])
def test_parse_errors_are_reported_not_fatal(text, needle):
    rc, msg, *_ = inspect(text)
    assert rc == -1
    assert needle in msg


def test_unknown_activation_means_relu_like_the_reference():
    text = "config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nconv:\n  filters: 4\n  activation: notanactivation\n"
    assert inspect(text)[0] == 1


def test_weight_layout_order_and_synth_blob():
    text = topologies.resnet18(224)
    layout = synth.weight_layout(text)
    assert sum(c for _, _, c, _ in layout) == EXPECTED["resnet18"][2]
    # first conv: 64x3x7x7 weights, no bias, then the standalone BatchNorm's scales, biases, mean, var
    assert layout[0][1:] == (_ffi.W_WEIGHTS, 64 * 3 * 49, 64)
    assert [s for _, s, _, _ in layout[1:5]] == [_ffi.W_BN_SCALE, _ffi.W_BN_BIAS, _ffi.W_BN_MEAN, _ffi.W_BN_VAR]
    blob = synth.make_blob(text, synth.load_factors("resnet18"))
    assert blob.dtype == np.float32 and blob.size == EXPECTED["resnet18"][2]
    assert np.array_equal(blob, synth.make_blob(text, synth.load_factors("resnet18")))   # seeded
    assert np.isfinite(blob).all()


def test_calibration_covers_every_weight_layer():
    for name, (size, _, _) in EXPECTED.items():
        f = synth.load_factors(name)
        assert f is not None and all(x > 0 for x in f)
        synth.make_blob(topologies.NETS[name](size=size), f)  # raises on a count mismatch


def test_c_api_reports_errors_through_msg():
    lib = _ffi.host_lib()
    msg = C.c_char_p()
    lib.dispose()
    assert lib.msnhB200Forward(C.byref(msg), None, 1) == -1 and b"initMsnhnet" in msg.value
    assert lib.initMsnhnet() == 1
    assert lib.buildMsnhnet(C.byref(msg), b"/nonexistent/net.msnhnet", b"/nonexistent/w.msnhbin", 0, 0) == -1
    assert b"can not open" in msg.value
    best = C.c_int()
    data = (C.c_float * 4)()
    assert lib.runClassifyNoPred(C.byref(msg), data, 4, C.byref(best), 0) == -1 and b"no CPU path" in msg.value
    gpu, cudnn = C.c_int(), C.c_int()
    assert lib.withGPU(C.byref(gpu)) == 1 and gpu.value == 1
    assert lib.withCUDNN(C.byref(cudnn)) == 0 and cudnn.value == 0
    lib.dispose()


def test_msnhbin_reader_rejects_a_truncated_file(tmp_path):
    lib = _ffi.host_lib()
    net = tmp_path / "n.msnhnet"
    net.write_text("config:\n  batch: 1\n  width: 8\n  height: 8\n  channels: 3\nconv:\n  filters: 4\n")
    blob = tmp_path / "w.msnhbin"
    blob.write_bytes(b"\x00" * 7)
    msg = C.c_char_p()
    # preview mode keeps this on CPU: build + load are parsed and size-checked without a device
    assert lib.initMsnhnet() == 1
    rc = lib.buildMsnhnet(C.byref(msg), str(net).encode(), str(blob).encode(), 0, 0)
    assert rc == -1
    lib.dispose()


REFERENCE_MODELS = os.environ.get("MSNHNET_REFERENCE_MODELS", "/root/reference/models")


@pytest.mark.skipif(not os.path.isdir(REFERENCE_MODELS), reason="the reference's source tree is not on this machine")
def test_every_model_file_of_the_reference_builds():
    """Every .msnhnet file the reference ships parses, lowers and shape-checks here, except the one its own parser
    rejects too (models/yolov3_spp names a `yolov3` node kind that src/io/MsnhParser.cpp no longer knows). Blob
    lengths of the segmentation nets come from the reference's layer constructors (deconv: Cin*Cout*k*k + bias)."""
    import glob
    files = sorted(glob.glob(os.path.join(REFERENCE_MODELS, "*", "*.msnhnet")))
    assert len(files) >= 30
    for f in files:
        rc, msg, layers, wc, _ = inspect(open(f, errors="replace").read())
        if os.path.basename(f) == "yolov3_spp.msnhnet":
            assert rc == -1 and "yolov3" in msg
            continue
        assert rc == 1, (f, msg)
        assert layers > 0
    rc, _, layers, wc, _ = inspect(open(os.path.join(REFERENCE_MODELS, "fcns", "fcns.msnhnet")).read())
    assert (layers, wc) == (33, 16464610)
    rc, _, layers, wc, _ = inspect(open(os.path.join(REFERENCE_MODELS, "deeplabv3", "deeplabv3.msnhnet")).read())
    assert (layers, wc) == (376, 58739925)


# ---- the seam: reference layer objects -> MsnhB200Op list (oracle/seam_adapter.cpp) ----------------------------
def lowered_lines(text):
    """The op list and weight-slot order NetBuilder::lower (host/msnh_netbuilder.cpp) makes of topology `text`, in
    the line format oracle/seam_adapter.cpp prints."""
    lib = _ffi.host_lib()
    msg = C.c_char_p()
    assert lib.msnhB200OpList(C.byref(msg), text.encode()) == 1, msg.value
    ops = [l for l in msg.value.decode().splitlines() if l]
    assert lib.msnhB200WeightLayout(C.byref(msg), text.encode()) == 1, msg.value
    weights = ["w " + " ".join(l.split()[:3]) for l in msg.value.decode().splitlines() if l]
    return ops, weights


SEAM_NETS = sorted(json.load(open(os.path.join(H.GOLDEN, "seam_ops.json"))).items())


@pytest.mark.parametrize("key,want", SEAM_NETS, ids=[k for k, _ in SEAM_NETS])
def test_lowering_equals_what_the_reference_layer_objects_give(key, want):
    """tests/golden/seam_ops.json holds, per net, the SHA-256 of the op list and weight-slot order that
    oracle/seam_adapter.cpp derives from the UNMODIFIED reference's own layer objects (Msnhnet::NetBuilder::buildNetFromMsnhNet,
    src/net/MsnhNetBuilder.cpp:154, then one MsnhB200Op per BaseLayer from its public fields). This build's own
    parser + lowering must give the same bytes: same ops in the same order with the same geometry, fused-BN flags,
    activation codes and parameters, input indices, and the same .msnhbin consumption order."""
    from golden.make_seam_fixture import ADAPTER, adapter_lines, digest
    name, size = key.split("@")
    text = topologies.NETS[name](size=int(size))
    ops, weights = lowered_lines(text)
    assert (len(ops), len(weights)) == (want["ops"], want["weight_slots"])
    assert digest(ops, weights) == want["sha256"]
    if os.path.exists(ADAPTER):        # the reference tree was on the build machine: compare line by line too
        ref_ops, ref_weights = adapter_lines(text)
        for i, (a, b) in enumerate(zip(ops, ref_ops)):
            assert a == b, (i, a, b)
        assert weights == ref_weights
