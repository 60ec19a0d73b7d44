"""Pins the numpy oracle against golden vectors produced by the UNMODIFIED reference CPU path
(tests/golden/ref_*.npz, made by tests/golden/make_reference_fixtures.py with the reference's
scalar path). Without this the oracle would only be a restatement; with it, it is checked against
the reference's own numbers layer by layer."""
import os

import numpy as np
import pytest

import helpers as H
from msnhnet_b200 import synth
from oracle import msnh_oracle as mo
from golden.make_reference_fixtures import fixture_positions

# small enough for the CPU suite; the 608 / 640 fixtures are used by the GPU tests
CASES = [("resnet18", 224), ("yolov3_tiny", 416), ("mobilenetv2", 224), ("yolov4", 160), ("yolov5m", 160), ("yolov5m_silu", 160), ("layer_zoo", 64), ("fcns", 64)]
# The reference sums each dot product in ascending k in fp32; numpy's BLAS blocks the sum. The two
# differ at fp32 rounding level; 2e-4 of the layer's largest magnitude bounds it for these nets.
LAYER_TOL = 2e-4


@pytest.mark.parametrize("name,size", CASES)
def test_oracle_matches_reference_layer_by_layer(name, size):
    g, kw = H.golden(name, size)
    text = H.net_text(name, size, **kw)
    blob = H.net_blob(name, text)
    net = mo.OracleNet(text)
    net.load_weights(blob)
    img = synth.make_images(1, 3, size, size)[0]
    res = net.forward(img)
    checked = 0
    for i in range(int(g["n_layers"])):
        if f"l{i}_n" not in g:
            continue
        y = res["layers"][i]
        assert y is not None and y.size == int(g[f"l{i}_n"]), f"layer {i} size"
        ref = g[f"l{i}_samples"]
        got = y.ravel()[fixture_positions(g, "", i, y.size)]
        scale = float(g[f"l{i}_absmax"]) + 1e-30
        assert np.abs(got - ref).max() / scale < LAYER_TOL, f"layer {i} ({net.layers[i]['kind']})"
        assert abs(float(y.astype(np.float64).mean()) - float(g[f"l{i}_mean"])) / scale < LAYER_TOL
        checked += 1
    assert checked >= len(net.layers) - 1
    if "final" in g:
        assert H.rel_err(res["out"], g["final"]) < LAYER_TOL
        assert int(res["out"].argmax()) == int(g["final"].argmax())
    else:
        ref_boxes = g["boxes"]
        got = res["boxes"][:, :7]
        assert got.shape == ref_boxes.shape
        a, b = H.sort_rows(got), H.sort_rows(ref_boxes)
        assert np.array_equal(a[:, 6], b[:, 6])                       # same classes
        assert np.abs(a - b).max() / (np.abs(b).max() + 1e-30) < LAYER_TOL


def test_parser_matches_host_library_blob_length():
    for name, size in CASES:
        text = H.net_text(name, size)
        net = mo.OracleNet(text)
        assert net.weight_count() == sum(c for _, _, c, _ in synth.weight_layout(text))


def test_activation_definitions():
    x = np.array([-30, -25, -3.5, -1, -0.0, 0.5, 2.9, 3.1, 7, 25], np.float32)
    assert np.allclose(mo.activate(x, "leaky"), np.where(x > 0, x, 0.1 * x))
    assert np.allclose(mo.activate(x, "leaky", [0.2]), np.where(x > 0, x, 0.2 * x))
    assert np.allclose(mo.activate(x, "relu6"), np.clip(x, 0, 6))
    assert np.allclose(mo.activate(x, "hardswish"), x * np.clip(x + 3, 0, 6) / 6)
    sp = np.log1p(np.exp(np.minimum(x.astype(np.float64), 20)))
    sp = np.where(x > 20, x, np.where(x < -20, np.exp(x.astype(np.float64)), sp))
    assert np.allclose(mo.activate(x, "mish"), x * np.tanh(sp), rtol=1e-5, atol=1e-7)
    assert np.allclose(mo.activate(x, "made-up-name"), np.maximum(x, 0))          # unknown -> relu


def test_pool_out_size_rules():
    assert mo.pool_out(14, 0, 2, 1, 1) == 13          # yolov3-tiny layer 12
    assert mo.pool_out(416, 0, 2, 2, 0) == 208
    assert mo.pool_out(112, 1, 3, 2, 0) == 56         # resnet stem
    assert mo.pool_out(19, 6, 13, 1, 0) == 19         # SPP
    assert mo.pool_out(7, 0, 2, 2, 1) == 4            # ceil mode adds the ragged window


def test_maxpool_padding_never_wins():
    x = -np.ones((1, 3, 3), np.float32) * 5
    y = mo.maxpool(x, 3, 3, 1, 1, 1, 1, 0)
    assert np.array_equal(y, x)


def test_iou_uses_the_plus_one_convention():
    a = np.array([10, 10, 4, 4], np.float32)
    assert mo.iou(a, a) == 1.0
    b = np.array([14, 10, 4, 4], np.float32)          # touching boxes still overlap by one pixel column
    inter = 1 * 5
    assert abs(float(mo.iou(a, b)) - inter / (25 + 25 - inter)) < 1e-6
