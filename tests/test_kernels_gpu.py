"""Per-kernel parity on the GPU: single-op plans through the kernel library's C ABI against the numpy
oracle's layer functions, fp32 and fp16, including the edge shapes the reference's layers allow
(odd planes, channel counts that are not vector multiples, 255-channel heads, stride 2 on odd
inputs, dilation, ragged last tiles)."""
import os

import numpy as np
import pytest

import helpers as H
from msnhnet_b200 import _ffi as ffi
from oracle import msnh_oracle as mo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = ffi.Context(0)
    yield c
    c.close()


def run_plan(ctx, ops, in_chw, x, dtype, weights=(), flags=0, out_ops=None, runs=1):
    ops[-1].is_output = 1
    plan = ffi.Plan(ctx, ops, in_chw, x.shape[0], dtype, flags)
    for (op, slot, data) in weights:
        plan.set_weights(op, slot, data)
    plan.finalize()
    for _ in range(runs):
        plan.run(x)
    outs = [plan.read_output(o, x.shape[0]) for o in (out_ops or [len(ops) - 1])]
    plan.close()
    return outs[0] if out_ops is None else outs


def tol(dtype, tensor_core=True):
    if dtype == ffi.F16:
        return H.TOL_F16
    return H.TOL_F32 if tensor_core else 1e-5


def quant(x, dtype):
    """The oracle sees the inputs the device sees: fp16 storage rounds them once."""
    return x.astype(np.float16).astype(np.float32) if dtype == ffi.F16 else x


def quant_tc(x, dtype):
    """The same for operands of a tensor-core product: fp32 plans multiply tf32-rounded values (10-bit mantissa,
    round to nearest, ties away from zero), so values that are already tf32 numbers multiply exactly."""
    if dtype == ffi.F16:
        return quant(x, dtype)
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x1000)) & np.uint32(0xFFFFE000)).view(np.float32)


CONV_CASES = [
    # cin, cout, h, w, k, stride, pad, dil, groups, batch
    (64, 64, 16, 16, 1, 1, 0, 1, 1, 2),
    (128, 255, 19, 19, 1, 1, 0, 1, 1, 3),        # detection head width, bias only
    (32, 64, 20, 20, 1, 1, 0, 1, 1, 2),          # 64-byte k-blocks
    (64, 128, 19, 19, 3, 1, 1, 1, 1, 3),         # odd plane, ragged last tile
    (64, 128, 38, 38, 3, 2, 1, 1, 1, 2),
    (64, 128, 19, 19, 3, 2, 1, 1, 1, 2),         # stride 2 on an odd plane
    (3, 32, 32, 32, 3, 1, 1, 1, 1, 2),           # image input: 3 channels in an 8-channel pitch
    (3, 16, 19, 23, 3, 1, 1, 1, 1, 2),           # image input, rows that do not end on a 4-pixel strip
    (3, 32, 21, 22, 3, 2, 1, 1, 1, 2),           # image input, stride 2 (one pixel per thread)
    (48, 96, 20, 20, 3, 1, 1, 1, 1, 2),          # channels not a multiple of 64
    (3, 64, 64, 64, 7, 2, 3, 1, 1, 1),           # resnet stem
    (64, 128, 28, 28, 1, 2, 0, 1, 1, 2),         # 1x1 stride 2 projection
    (64, 64, 20, 20, 3, 1, 2, 2, 1, 2),          # dilation 2
    (24, 24, 14, 14, 3, 1, 1, 1, 24, 2),         # depthwise
    (32, 32, 15, 15, 3, 2, 1, 1, 32, 2),         # depthwise stride 2, odd plane
    (144, 144, 30, 50, 3, 1, 1, 1, 144, 2),      # depthwise: several tiles per plane, two channel groups per pixel
    (96, 96, 57, 45, 3, 2, 1, 1, 96, 2),         # depthwise stride 2: odd plane, ragged last tiles in both directions
    (960, 960, 7, 7, 3, 1, 1, 1, 960, 3),        # depthwise: a plane smaller than one tile, many channel groups
    (40, 40, 19, 33, 3, 2, 1, 1, 40, 2),         # depthwise: channel count that is no multiple of a channel group
    (24, 24, 9, 9, 3, 1, 0, 1, 24, 1),           # depthwise without padding
    (16, 32, 12, 12, 3, 1, 1, 1, 4, 2),          # grouped, not depthwise (CUDA-core kernel)
    (20, 36, 9, 11, 3, 1, 1, 1, 1, 1),           # channel counts that are not vector multiples
]


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("act", ["leaky", "mish"])
def test_conv_bn_act(ctx, case, dtype, act):
    cin, cout, h, w, k, s, p, d, g, b = case
    if act == "mish" and case not in CONV_CASES[:6]:
        pytest.skip("activation variants are covered on the first shapes")
    rng = np.random.default_rng(hash(case) % 1000)
    x = quant(rng.random((b, cin, h, w), dtype=np.float32) - 0.3, dtype)
    wt = (rng.standard_normal((cout, cin // g, k, k)) * np.sqrt(2.0 / (cin // g * k * k))).astype(np.float32)
    bn = cout != 255
    op = ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=cout, k_h=k, k_w=k, stride_h=s, stride_w=s, pad_h=p, pad_w=p, dil_h=d, dil_w=d,
                     groups=g, has_bn=int(bn), has_bias=int(not bn), act=ffi.ACT_LEAKY if act == "leaky" else ffi.ACT_MISH, act_param=0.1)
    weights = [(0, ffi.W_WEIGHTS, wt)]
    if bn:
        gam, bet = rng.random(cout, dtype=np.float32) + 0.5, rng.standard_normal(cout).astype(np.float32) * 0.1
        mu, var = rng.standard_normal(cout).astype(np.float32) * 0.1, rng.random(cout, dtype=np.float32) + 0.5
        weights += [(0, ffi.W_BN_SCALE, gam), (0, ffi.W_BN_BIAS, bet), (0, ffi.W_BN_MEAN, mu), (0, ffi.W_BN_VAR, var)]
    else:
        bias = rng.standard_normal(cout).astype(np.float32) * 0.1
        weights += [(0, ffi.W_BIAS, bias)]
    got = run_plan(ctx, [op], (cin, h, w), x, dtype, weights)
    wq = quant(wt, dtype)
    for i in range(b):
        y = mo.conv2d(x[i], wq, k, k, s, s, p, p, d, d, g)
        y = mo.batchnorm(y, gam, bet, mu, var, 1e-5) if bn else y + bias[:, None, None]
        y = mo.activate(y, act, [0.1])
        assert H.rel_err(got[i], y) < tol(dtype), f"image {i}"


# every activation code of the C ABI with the reference's name for it (include/Msnhnet/layers/MsnhActivations.h:39-168)
ACT_NAMES = ["none", "logistic", "loggy", "relu", "relu6", "hardswish", "elu", "selu", "relie", "ramp", "leaky", "tanh", "stair",
             "hardtan", "softplus", "plse", "lhtan", "mish", "swish"]


def _act_param(name):
    return {"leaky": 0.1, "softplus": 20.0}.get(name, 0.0)


def _away_from_steps(pre, name):
    """stair is a step function: a pre-activation within rounding of an integer may land on either step."""
    if name != "stair":
        return np.ones(pre.shape, bool)
    return np.abs(pre - np.round(pre)) > 0.03


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
@pytest.mark.parametrize("tensor_core", [True, False])
@pytest.mark.parametrize("code", range(len(ACT_NAMES)))
def test_conv_with_every_activation(ctx, dtype, tensor_core, code):
    """conv + bias + activation for every activation the lowering accepts, on the tensor-core epilogue (its own
    packed arithmetic for mish and leaky, the shared switch for the rest) and on the CUDA-core kernel."""
    name = ACT_NAMES[code]
    rng = np.random.default_rng(100 + code)
    cin, cout, h, w, b = 64, 96, 13, 17, 2
    x = quant_tc(rng.standard_normal((b, cin, h, w)).astype(np.float32), dtype)
    wt = quant_tc((rng.standard_normal((cout, cin, 1, 1)) * np.sqrt(8.0 / cin)).astype(np.float32), dtype)     # pre-activations of a few units: every branch of every activation
    bias = rng.standard_normal(cout).astype(np.float32)
    op = ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=cout, has_bias=1, act=code, act_param=_act_param(name))
    got = run_plan(ctx, [op], (cin, h, w), x, dtype, [(0, ffi.W_WEIGHTS, wt), (0, ffi.W_BIAS, bias)],
                   flags=0 if tensor_core else ffi.PLAN_NO_TENSOR_CORE)
    for i in range(b):
        pre = mo.conv2d(x[i], wt, 1, 1, 1, 1, 0, 0, 1, 1, 1) + bias[:, None, None]
        want = mo.activate(pre, name, [_act_param(name)] if _act_param(name) else [])
        ok = _away_from_steps(pre, name)
        # the operands multiply exactly on every path, so fp32 results differ by summation order and the device's exp / log only
        assert np.abs(got[i] - want)[ok].max() / np.abs(want).max() < (H.TOL_F16 if dtype == ffi.F16 else 2e-5), name


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
@pytest.mark.parametrize("code", range(len(ACT_NAMES)))
def test_activation_layer_with_every_activation(ctx, dtype, code):
    """The standalone activation layer (src/layers/MsnhActivationLayer.cpp:334-485 in the reference)."""
    name = ACT_NAMES[code]
    rng = np.random.default_rng(200 + code)
    x = quant((rng.standard_normal((2, 24, 9, 11)) * 3).astype(np.float32), dtype)
    x[0, 0, 0, :6] = quant(np.array([-30, -21, -4.5, 4.5, 21, 30], np.float32), dtype)        # the far branches of softplus, plse, mish
    op = ffi.make_op(ffi.OP_ACTIVATION, [ffi.INPUT], act=code, act_param=_act_param(name))
    got = run_plan(ctx, [op], (24, 9, 11), x, dtype)
    want = mo.activate(x, name, [_act_param(name)] if _act_param(name) else [])
    ok = _away_from_steps(x, name)
    assert np.abs(got - want)[ok].max() / np.abs(want).max() < (H.TOL_F16 if dtype == ffi.F16 else 2e-6), name


BIN_FORMS = [("add", lambda a, b: a + b), ("sub", lambda a, b: a - b), ("subInv", lambda a, b: b - a), ("mul", lambda a, b: a * b),
             ("div", lambda a, b: a / b), ("divInv", lambda a, b: b / a)]


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
@pytest.mark.parametrize("channels", [16, 5])         # 16-byte vectors / element by element
def test_binary_ops_of_two_layers_and_with_a_constant(ctx, dtype, channels):
    """VariableOpLayer's arithmetic forms (src/layers/MsnhVariableOpLayer.cpp:244-400, kernels src/core/cuda/MsnhBlasGPU.cu:68-140):
    A op B of two layers and A op const, including the operand-swapped 'Inv' forms."""
    rng = np.random.default_rng(31)
    x = quant((rng.random((2, channels, 7, 9)) + 0.5).astype(np.float32), dtype)
    const = 1.75
    ops = [ffi.make_op(ffi.OP_ACTIVATION, [ffi.INPUT], act=ffi.ACT_LOGISTIC)]                # 0: B, in (0.62, 0.82)
    for kind in range(6):
        ops.append(ffi.make_op(ffi.OP_BINARY, [ffi.INPUT, 0], binary_kind=kind, binary_const=0))
    for kind in range(6):
        ops.append(ffi.make_op(ffi.OP_BINARY, [ffi.INPUT], binary_kind=kind, binary_const=1, const_val=const))
    for o in ops:
        o.is_output = 1
    got = run_plan(ctx, ops, (channels, 7, 9), x, dtype, out_ops=list(range(len(ops))))
    assert H.rel_err(got[0], mo.activate(x, "logistic")) < (H.TOL_F16 if dtype == ffi.F16 else 2e-6)
    t = 1e-3 if dtype == ffi.F16 else 1e-6
    for kind, (name, fn) in enumerate(BIN_FORMS):
        assert H.rel_err(got[1 + kind], fn(x, got[0])) < t, name
        assert H.rel_err(got[7 + kind], fn(x, np.float32(const))) < t, name + "Const"


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
def test_tensor_core_and_cuda_core_convs_agree(ctx, dtype):
    rng = np.random.default_rng(3)
    x = rng.random((2, 96, 21, 23), dtype=np.float32)
    wt = (rng.standard_normal((80, 96, 3, 3)) * 0.05).astype(np.float32)
    op = lambda: ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=80, k_h=3, k_w=3, pad_h=1, pad_w=1, has_bias=1, act=ffi.ACT_RELU)
    w = [(0, ffi.W_WEIGHTS, wt), (0, ffi.W_BIAS, np.zeros(80, np.float32))]
    a = run_plan(ctx, [op()], (96, 21, 23), x, dtype, w)
    b = run_plan(ctx, [op()], (96, 21, 23), x, dtype, w, flags=ffi.PLAN_NO_TENSOR_CORE)
    assert H.rel_err(a, b) < tol(dtype)


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
@pytest.mark.parametrize("shape", [{"MSNH_B200_M_MULT": "1", "MSNH_B200_BN": "64"}, {"MSNH_B200_M_MULT": "2", "MSNH_B200_BN": "128"},
                                   {"MSNH_B200_M_MULT": "4", "MSNH_B200_BN": "64"}, {"MSNH_B200_M_MULT": "1", "MSNH_B200_BN": "256"},
                                   {"MSNH_B200_M_MULT": "3", "MSNH_B200_BN": "128"},
                                   {"MSNH_B200_PAIR": "1", "MSNH_B200_BN": "128"}, {"MSNH_B200_PAIR": "1", "MSNH_B200_BN": "256"},
                                   {"MSNH_B200_STREAM_K": "1", "MSNH_B200_M_MULT": "1", "MSNH_B200_BN": "128"},
                                   {"MSNH_B200_STREAM_K": "1", "MSNH_B200_M_MULT": "2", "MSNH_B200_BN": "128"},
                                   {"MSNH_B200_STREAM_K": "1", "MSNH_B200_M_MULT": "1", "MSNH_B200_BN": "256"},
                                   # 128-pixel tiles with several store slabs, epilogue teams alternating over whole tiles
                                   {"MSNH_B200_NO_SPLIT": "1", "MSNH_B200_M_MULT": "1", "MSNH_B200_BN": "128"},
                                   {"MSNH_B200_NO_SPLIT": "1", "MSNH_B200_M_MULT": "1", "MSNH_B200_BN": "256"},
                                   # shapes that take all of TMEM (one accumulator stage), offered only to the measured choice
                                   {"MSNH_B200_M_MULT": "4", "MSNH_B200_BN": "128"}, {"MSNH_B200_M_MULT": "2", "MSNH_B200_BN": "256"},
                                   {"MSNH_B200_M_MULT": "2", "MSNH_B200_BN": "192"}])
@pytest.mark.parametrize("k", [1, 3])
def test_every_tile_shape_of_the_tensor_core_conv(ctx, dtype, shape, k, monkeypatch):
    """Tiles of 128/256/512 pixels, 64..256 channels, the CTA-pair form and the stream-K form (normally picked by
    the plan's cost model, forced here through its environment switches) all compute what the CUDA-core kernel
    computes, including ragged last tiles in both directions, several tiles per CTA and tiles split over CTAs;
    the plan runs twice so stream-K's hand-over flags are seen to reset."""
    rng = np.random.default_rng(11)
    cin, cout, h, w, b = 96, 320, 37, 41, 9          # 13653 pixels: more 128-pixel tiles than SMs; 320 = 256 + 64 channels
    x = quant(rng.random((b, cin, h, w), dtype=np.float32) - 0.4, dtype)
    wt = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    op = lambda: ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=cout, k_h=k, k_w=k, pad_h=k // 2, pad_w=k // 2, has_bias=1, act=ffi.ACT_MISH)
    wts = [(0, ffi.W_WEIGHTS, wt), (0, ffi.W_BIAS, rng.standard_normal(cout).astype(np.float32) * 0.1)]
    ref = run_plan(ctx, [op()], (cin, h, w), x, dtype, wts, flags=ffi.PLAN_NO_TENSOR_CORE)
    for name, value in shape.items():
        monkeypatch.setenv(name, value)
    got = run_plan(ctx, [op()], (cin, h, w), x, dtype, wts, runs=2)
    assert H.rel_err(got, ref) < tol(dtype)


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
def test_conv_residual_add_is_fused_and_exact(ctx, dtype):
    """conv -> add(conv_out, earlier tensor) -> activation collapses into one launch; the result equals the unfused plan."""
    rng = np.random.default_rng(4)
    x = quant(rng.random((2, 64, 19, 19), dtype=np.float32), dtype)
    w1 = (rng.standard_normal((64, 64, 1, 1)) * 0.1).astype(np.float32)
    w2 = (rng.standard_normal((64, 64, 3, 3)) * 0.05).astype(np.float32)
    def ops():
        return [ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=64, has_bias=1, act=ffi.ACT_LEAKY, act_param=0.1),
                ffi.make_op(ffi.OP_CONV, [0], filters=64, k_h=3, k_w=3, pad_h=1, pad_w=1, has_bias=1, act=ffi.ACT_LEAKY, act_param=0.1),
                ffi.make_op(ffi.OP_ADD, [0, 1], act=ffi.ACT_RELU)]
    w = [(0, ffi.W_WEIGHTS, w1), (0, ffi.W_BIAS, np.zeros(64, np.float32)), (1, ffi.W_WEIGHTS, w2), (1, ffi.W_BIAS, np.full(64, 0.01, np.float32))]
    fused = run_plan(ctx, ops(), (64, 19, 19), x, dtype, w)
    unfused = run_plan(ctx, ops(), (64, 19, 19), x, dtype, w, flags=ffi.PLAN_NO_FUSION)
    assert H.rel_err(fused, unfused) < 2e-3     # the fused chain rounds to fp16 / tf32 once less
    for i in range(2):
        a = mo.activate(mo.conv2d(x[i], quant(w1, dtype), 1, 1, 1, 1, 0, 0, 1, 1, 1), "leaky", [0.1])
        bq = mo.activate(mo.conv2d(a, quant(w2, dtype), 3, 3, 1, 1, 1, 1, 1, 1, 1) + np.float32(0.01), "leaky", [0.1])
        assert H.rel_err(fused[i], np.maximum(a + bq, 0)) < tol(dtype)


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
def test_two_1x1_convs_over_one_tensor_run_as_one_launch(ctx, dtype):
    """The two 1x1 convs a CSP stage opens with (same input, own weights, own output tensors, one of them a slice of a
    concat buffer) are merged into one tensor-core launch; every output equals the plan that runs them separately."""
    rng = np.random.default_rng(17)
    cin, h, w, b = 128, 19, 23, 3
    x = quant(rng.standard_normal((b, cin, h, w)).astype(np.float32), dtype)
    w0 = (rng.standard_normal((128, cin, 3, 3)) * 0.03).astype(np.float32)
    wa = (rng.standard_normal((64, 128, 1, 1)) * 0.1).astype(np.float32)
    wb = (rng.standard_normal((96, 128, 1, 1)) * 0.1).astype(np.float32)
    def ops():
        o = [ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=128, k_h=3, k_w=3, pad_h=1, pad_w=1, has_bias=1, act=ffi.ACT_MISH),   # 0
             ffi.make_op(ffi.OP_CONV, [0], filters=64, has_bias=1, act=ffi.ACT_MISH),                                            # 1: route branch
             ffi.make_op(ffi.OP_CONV, [0], filters=96, has_bias=1, act=ffi.ACT_MISH),                                            # 2: main branch
             ffi.make_op(ffi.OP_ACTIVATION, [2], act=ffi.ACT_LEAKY, act_param=0.1),                                               # 3
             ffi.make_op(ffi.OP_CONCAT, [3, 1])]                                                                                 # 4: op 1 lives in this buffer
        for q in o:
            q.is_output = 1
        return o
    wts = [(0, ffi.W_WEIGHTS, w0), (0, ffi.W_BIAS, np.zeros(128, np.float32)), (1, ffi.W_WEIGHTS, wa), (1, ffi.W_BIAS, rng.standard_normal(64).astype(np.float32)),
           (2, ffi.W_WEIGHTS, wb), (2, ffi.W_BIAS, rng.standard_normal(96).astype(np.float32))]
    plan = ffi.Plan(ctx, ops(), (cin, h, w), b, dtype, 0)
    for (op, slot, data) in wts:
        plan.set_weights(op, slot, data)
    plan.finalize()
    assert "with the 1x1 conv of op 2" in plan.describe()
    plan.run(x)
    merged = [plan.read_output(o, b) for o in range(5)]
    plan.close()
    apart = run_plan(ctx, ops(), (cin, h, w), x, dtype, wts, flags=ffi.PLAN_NO_FUSION, out_ops=list(range(5)))
    for o in range(5):
        # (fp16: the unfused plan stores op 2 before the leaky; fp32: which tensors get rounded to tf32 for a
        # tensor-core reader follows the arena layout, which differs between the two plans)
        assert H.rel_err(merged[o], apart[o]) < (2e-3 if dtype == ffi.F16 else 1e-3), o


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
@pytest.mark.parametrize("k,s,p,ceil,h,w", [(2, 2, 0, 0, 26, 26), (2, 1, 0, 1, 14, 14), (3, 2, 1, 0, 112, 112), (5, 1, 2, 0, 19, 19),
                                           (9, 1, 4, 0, 19, 19), (13, 1, 6, 0, 19, 19), (2, 2, 0, 1, 7, 9)])
def test_maxpool(ctx, dtype, k, s, p, ceil, h, w):
    rng = np.random.default_rng(k * 10 + s)
    c = 24
    x = quant(rng.standard_normal((2, c, h, w)).astype(np.float32), dtype)
    oh, ow = mo.pool_out(h, p, k, s, ceil), mo.pool_out(w, p, k, s, ceil)
    op = ffi.make_op(ffi.OP_MAXPOOL, [ffi.INPUT], k_h=k, k_w=k, stride_h=s, stride_w=s, pad_h=p, pad_w=p, out_h=oh, out_w=ow)
    got = run_plan(ctx, [op], (c, h, w), x, dtype)
    for i in range(2):
        assert np.array_equal(got[i], mo.maxpool(x[i], k, k, s, s, p, p, ceil))      # exact: max of stored values


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
def test_spp_concat_is_zero_copy_and_exact(ctx, dtype):
    """conv -> {maxpool 13, 9, 5, identity} -> concat, the SPP block: pools read and write channel slices of one buffer."""
    rng = np.random.default_rng(8)
    x = quant(rng.standard_normal((2, 32, 19, 19)).astype(np.float32), dtype)
    ops = [ffi.make_op(ffi.OP_ACTIVATION, [ffi.INPUT], act=ffi.ACT_LEAKY, act_param=0.1)]
    for k in (13, 9, 5):
        ops.append(ffi.make_op(ffi.OP_MAXPOOL, [0], k_h=k, k_w=k, pad_h=k // 2, pad_w=k // 2, out_h=19, out_w=19))
    ops.append(ffi.make_op(ffi.OP_CONCAT, [1, 2, 3, 0]))
    plan = ffi.Plan(ctx, ops, (32, 19, 19), 2, dtype, 0)
    ops2 = ffi.Plan(ctx, ops, (32, 19, 19), 2, dtype, ffi.PLAN_NO_FUSION)
    ops2.close()
    plan.close()
    got = run_plan(ctx, ops, (32, 19, 19), x, dtype)
    for i in range(2):
        a = quant(mo.activate(x[i], "leaky", [0.1]), dtype)
        want = np.concatenate([mo.maxpool(a, k, k, 1, 1, k // 2, k // 2, 0) for k in (13, 9, 5)] + [a], 0)
        assert np.array_equal(got[i], want)


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
def test_upsample_route_add_slice_pad_avgpool(ctx, dtype):
    rng = np.random.default_rng(9)
    x = quant(rng.standard_normal((2, 16, 10, 12)).astype(np.float32), dtype)
    ops = [ffi.make_op(ffi.OP_UPSAMPLE, [ffi.INPUT], stride_h=2, stride_w=2),                                   # 0: 16x20x24
           ffi.make_op(ffi.OP_SLICE, [0], slice_start=[0, 1, 0], slice_step=[1, 2, 2]),                         # 1: 16x10x12
           ffi.make_op(ffi.OP_ADD, [1, ffi.INPUT], act=ffi.ACT_LEAKY, act_param=0.1),                           # 2
           ffi.make_op(ffi.OP_PAD, [2], pad_top=0, pad_down=1, pad_left=0, pad_right=1, const_val=0.0),         # 3: 16x11x13
           ffi.make_op(ffi.OP_AVGPOOL, [3], k_h=3, k_w=3, stride_h=2, stride_w=2, pad_h=1, pad_w=1, out_h=6, out_w=7),   # 4
           ffi.make_op(ffi.OP_CONCAT, [2, 1]),                                                                  # 5: 32x10x12
           ffi.make_op(ffi.OP_CONCAT, [5], route_groups=2, route_group_id=1)]                                   # 6: second half = op 1
    for o in ops:
        o.is_output = 1
    got = run_plan(ctx, ops, (16, 10, 12), x, dtype, out_ops=[0, 1, 2, 3, 4, 5, 6])
    t = H.TOL_F16 if dtype == ffi.F16 else 1e-6
    for i in range(2):
        up = mo.upsample(x[i], 2, 2)
        sl = up[:, 1::2, 0::2]
        ad = quant(mo.activate(sl + x[i], "leaky", [0.1]), dtype)
        pd = np.pad(ad, ((0, 0), (0, 1), (0, 1)))
        av = mo.avgpool(pd, 3, 3, 2, 2, 1, 1, 0)
        assert np.array_equal(got[0][i], up) and np.array_equal(got[1][i], sl)
        assert H.rel_err(got[2][i], ad) < t and H.rel_err(got[3][i], pd) < t and H.rel_err(got[4][i], av) < max(t, 1e-3 if dtype == ffi.F16 else 1e-6)
        assert H.rel_err(got[5][i], np.concatenate([ad, sl], 0)) < t
        assert np.array_equal(got[6][i], got[1][i])


DECONV_CASES = [
    # cin, cout, h, w, k, stride, pad, bias, batch
    (64, 32, 8, 8, 2, 2, 0, 1, 2),        # non-overlapping taps (the segmentation decoder's form)
    (32, 24, 9, 7, 3, 2, 1, 1, 2),        # overlapping taps, odd output plane
    (16, 8, 12, 12, 4, 2, 1, 0, 1),       # no bias
    (24, 20, 6, 6, 3, 1, 1, 1, 2),        # stride 1: a correlation with the flipped kernel
    (20, 5, 5, 6, 5, 3, 2, 1, 1),         # channel counts that are not vector multiples, stride 3
]


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
@pytest.mark.parametrize("tensor_core", [True, False])
@pytest.mark.parametrize("case", DECONV_CASES)
def test_deconv(ctx, case, dtype, tensor_core):
    cin, cout, h, w, k, s, p, bias, b = case
    rng = np.random.default_rng(sum(case))
    x = quant(rng.standard_normal((b, cin, h, w)).astype(np.float32), dtype)
    wt = (rng.standard_normal((cin, cout, k, k)) * np.sqrt(1.0 / cin)).astype(np.float32)
    bs = rng.standard_normal(cout).astype(np.float32)
    ops = [ffi.make_op(ffi.OP_DECONV, [ffi.INPUT], filters=cout, k_h=k, k_w=k, stride_h=s, stride_w=s, pad_h=p, pad_w=p,
                       has_bias=bias, act=ffi.ACT_LEAKY, act_param=0.1)]
    weights = [(0, ffi.W_WEIGHTS, wt)] + ([(0, ffi.W_BIAS, bs)] if bias else [])
    got = run_plan(ctx, ops, (cin, h, w), x, dtype, weights, flags=0 if tensor_core else ffi.PLAN_NO_TENSOR_CORE)
    for i in range(b):
        y = mo.deconv2d(x[i], quant(wt, dtype) if dtype == ffi.F16 else wt, k, k, s, s, p, p)
        if bias:
            y = y + bs[:, None, None]
        want = mo.activate(y.astype(np.float32), "leaky", [0.1])
        assert got[i].shape == want.shape
        assert H.rel_err(got[i], want) < tol(dtype, tensor_core)


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
def test_bilinear_clip_remap_reduce(ctx, dtype):
    rng = np.random.default_rng(21)
    c, h, w = 16, 9, 12
    x = quant(rng.standard_normal((2, c, h, w)).astype(np.float32), dtype)
    ops = [ffi.make_op(ffi.OP_UPSAMPLE, [ffi.INPUT], upsample_mode=ffi.UPSAMPLE_BILINEAR, align_corners=0, out_h=25, out_w=30),   # 0
           ffi.make_op(ffi.OP_UPSAMPLE, [ffi.INPUT], upsample_mode=ffi.UPSAMPLE_BILINEAR, align_corners=1, out_h=5, out_w=31),    # 1: shrinks H
           ffi.make_op(ffi.OP_CLIP, [ffi.INPUT], const_val=-0.25, scale=0.75),                                                    # 2
           ffi.make_op(ffi.OP_REMAP, [ffi.INPUT], remap_kind=ffi.REMAP_PERMUTE, remap_dims=[2, 0, 1]),                            # 3: 12x16x9
           ffi.make_op(ffi.OP_REMAP, [ffi.INPUT], remap_kind=ffi.REMAP_PIXSHF, remap_dims=[2, 0, 0]),                             # 4: 4x18x24
           ffi.make_op(ffi.OP_REMAP, [ffi.INPUT], remap_kind=ffi.REMAP_VIEW, out_c=27, out_h=8, out_w=8),                         # 5
           ffi.make_op(ffi.OP_REDUCE, [ffi.INPUT], binary_kind=0, binary_const=0),                                                # 6
           ffi.make_op(ffi.OP_REDUCE, [ffi.INPUT], binary_kind=1, binary_const=1),                                                # 7
           ffi.make_op(ffi.OP_REDUCE, [ffi.INPUT], binary_kind=2, binary_const=0),                                                # 8
           ffi.make_op(ffi.OP_REDUCE, [ffi.INPUT], binary_kind=-1, binary_const=1),                                               # 9
           ffi.make_op(ffi.OP_REMAP, [3], remap_kind=ffi.REMAP_PERMUTE, remap_dims=[1, 2, 0]),                                    # 10: back to the input
           ffi.make_op(ffi.OP_PRELU, [ffi.INPUT]),                                                                                # 11
           ffi.make_op(ffi.OP_MAXPOOL, [ffi.INPUT], filters=6),                                                                   # 12: depth pooling 16 -> 6
           ffi.make_op(ffi.OP_PRELU, [12])]                                                                                       # 13: six channels: element-wise form
    for o in ops:
        o.is_output = 1
    slopes = rng.standard_normal(c).astype(np.float32)
    got = run_plan(ctx, ops, (c, h, w), x, dtype, weights=[(11, ffi.W_WEIGHTS, slopes), (13, ffi.W_WEIGHTS, slopes[:6])], out_ops=list(range(len(ops))))
    t = H.TOL_F16 if dtype == ffi.F16 else 1e-5
    for i in range(2):
        assert H.rel_err(got[0][i], mo.bilinear_resize(x[i], 30, 25, 0)) < t
        assert H.rel_err(got[1][i], mo.bilinear_resize(x[i], 31, 5, 1)) < t
        assert np.array_equal(got[2][i], quant(np.clip(x[i], np.float32(-0.25), np.float32(0.75)), dtype))
        assert np.array_equal(got[3][i], mo.permute_chw(x[i], [2, 0, 1]))
        assert np.array_equal(got[4][i], mo.pixel_shuffle(x[i], 2))
        assert np.array_equal(got[5][i], x[i].reshape(27, 8, 8))
        assert H.rel_err(got[6][i], mo.reduction(x[i], 0, False)) < t
        assert H.rel_err(got[7][i], mo.reduction(x[i], 1, True)) < t
        assert H.rel_err(got[8][i], mo.reduction(x[i], 2, False)) < t
        assert abs(float(got[9][i].ravel()[0]) - float(mo.reduction(x[i], -1, True).ravel()[0])) < (2e-3 if dtype == ffi.F16 else 1e-5)
        assert np.array_equal(got[10][i], x[i])
        assert H.rel_err(got[11][i], np.where(x[i] > 0, x[i], slopes[:, None, None] * x[i])) < t
        depth = np.stack([x[i][j::6].max(axis=0) for j in range(6)])
        assert np.array_equal(got[12][i], depth)
        assert H.rel_err(got[13][i], np.where(depth > 0, depth, slopes[:6, None, None] * depth)) < t


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
def test_connected_softmax(ctx, dtype):
    rng = np.random.default_rng(10)
    x = quant(rng.standard_normal((3, 64, 2, 2)).astype(np.float32), dtype)
    wt = (rng.standard_normal((100, 64 * 4)) * 0.1).astype(np.float32)
    bias = rng.standard_normal(100).astype(np.float32) * 0.1
    ops = [ffi.make_op(ffi.OP_CONNECTED, [ffi.INPUT], filters=100, has_bias=1), ffi.make_op(ffi.OP_SOFTMAX, [0])]
    ops[0].is_output = 1
    logits, prob = run_plan(ctx, ops, (64, 2, 2), x, dtype, [(0, ffi.W_WEIGHTS, wt), (0, ffi.W_BIAS, bias)], out_ops=[0, 1])
    for i in range(3):
        y = quant(wt, dtype) @ x[i].reshape(-1) + bias
        assert H.rel_err(logits[i].ravel(), y) < tol(dtype)
        assert H.rel_err(prob[i].ravel(), mo.softmax(quant(y.reshape(-1, 1, 1), dtype) if dtype == ffi.F16 else y.reshape(-1, 1, 1), 1, 1.0).ravel()) < tol(dtype) * 5
        assert abs(prob[i].sum() - 1) < 1e-2


@pytest.mark.parametrize("dtype", [ffi.F32, ffi.F16])
@pytest.mark.parametrize("ytype", ["yolov3", "yolov5"])
def test_yolo_decode_and_candidates(ctx, dtype, ytype):
    rng = np.random.default_rng(11)
    classes, g = 4, 7
    c = 3 * (5 + classes)
    x = quant((rng.standard_normal((2, c, g, g)) * 1.5).astype(np.float32), dtype)
    anchors = [10, 13, 16, 30, 33, 23]
    code = {"yolov3": 30, "yolov5": 50}[ytype]
    ops = [ffi.make_op(ffi.OP_ACTIVATION, [ffi.INPUT], act=ffi.ACT_NONE),
           ffi.make_op(ffi.OP_YOLO, [0], yolo_type=code, yolo_classes=classes, yolo_anchors=anchors),
           ffi.make_op(ffi.OP_YOLO_COLLECT, [1], const_val=0.5)]
    ops[1].is_output = 1
    ops[2].is_output = 1
    plan = ffi.Plan(ctx, ops, (c, g * 8, g * 8), 2, dtype, 0)
    plan.close()
    # the head sees a g x g plane; the net input is 8x larger so the stride ratio is 8
    ops_small = ops
    plan = ffi.Plan(ctx, ops_small, (c, g, g), 2, dtype, 0)
    plan.finalize()
    plan.run(x)
    dec = plan.read_output(1, 2)
    cands = plan.read_candidates(2, 2)
    plan.close()
    for i in range(2):
        want = mo.yolo_decode(x[i], anchors, classes, ytype, g)        # ratio = net_h / grid_h = 1 here
        assert H.rel_err(dec[i], want) < 1e-5                          # decode runs in fp32 on both sides
        rows = mo.yolo_candidates([dec[i]], classes, 0.5)
        assert cands[i].shape == rows.shape
        assert np.array_equal(cands[i], rows)                           # same cells, same order, same numbers


def test_bad_arguments_return_status_codes(ctx):
    lib = ffi.kernel_lib()
    import ctypes as C
    ops = (ffi.Op * 1)(ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=8, groups=3))
    plan = C.c_void_p()
    assert lib.msnh_b200_plan_create(ctx.h, ops, 1, 4, 8, 8, 1, ffi.F16, 0, C.byref(plan)) == 1     # ERR_ARG
    assert "groups" in ctx.error()
    ops = (ffi.Op * 1)(ffi.make_op(99, [ffi.INPUT]))
    assert lib.msnh_b200_plan_create(ctx.h, ops, 1, 4, 8, 8, 1, ffi.F16, 0, C.byref(plan)) == 2     # ERR_UNSUPPORTED
    # geometry that would divide by zero or index outside a tensor is refused when the plan is created
    bad = [(ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=8, stride_h=0), "conv geometry"),
           (ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=8, k_w=0), "conv geometry"),
           (ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=8, pad_h=-1), "conv geometry"),
           (ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=8, dil_w=0), "conv geometry"),
           (ffi.make_op(ffi.OP_MAXPOOL, [ffi.INPUT], k_h=2, k_w=2, stride_w=0), "pool geometry"),
           (ffi.make_op(ffi.OP_MAXPOOL, [ffi.INPUT], k_h=0, k_w=2), "pool geometry"),
           (ffi.make_op(ffi.OP_UPSAMPLE, [ffi.INPUT], stride_h=0), "upsample stride"),
           (ffi.make_op(ffi.OP_SLICE, [ffi.INPUT], slice_step=[1, 0, 1]), "slice"),
           (ffi.make_op(ffi.OP_SLICE, [ffi.INPUT], slice_start=[0, 8, 0]), "slice"),
           (ffi.make_op(ffi.OP_SLICE, [ffi.INPUT], slice_start=[-1, 0, 0]), "slice")]
    for op, needle in bad:
        ops = (ffi.Op * 1)(op)
        assert lib.msnh_b200_plan_create(ctx.h, ops, 1, 4, 8, 8, 1, ffi.F16, 0, C.byref(plan)) == 1, needle
        assert needle in ctx.error(), (needle, ctx.error())
    op = ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=8)
    op.n_in = 99                                                                                       # checked before any input is read
    assert lib.msnh_b200_plan_create(ctx.h, (ffi.Op * 1)(op), 1, 4, 8, 8, 1, ffi.F16, 0, C.byref(plan)) == 1 and "n_in" in ctx.error()
    good = ffi.Plan(ctx, [ffi.make_op(ffi.OP_CONV, [ffi.INPUT], filters=8, has_bias=1)], (4, 8, 8), 1, ffi.F16)
    assert lib.msnh_b200_plan_finalize(good.h) == 4                                                   # weights not set: ERR_STATE
    assert lib.msnh_b200_plan_run_device(good.h, None, 1, 1) == 4                                      # not finalized
    with pytest.raises(ffi.KernelError):
        good.set_weights(0, ffi.W_WEIGHTS, np.zeros(5, np.float32))                                    # wrong length
    good.close()


PREP_MODES = {"yolo": ffi.PREP_PAD_SQUARE, "padzero": ffi.PREP_PAD_SQUARE, "c3": ffi.PREP_UNIT, "googlenet": ffi.PREP_GOOGLENET,
              "transformed": ffi.PREP_TRANSFORMED, "caffe": ffi.PREP_CAFFE}


def _prep_on_device(ctx, image, ow, oh, mode, swap, mean=None, std=None):
    """8-bit image -> plan input on the device, read back through an identity plan (1x1 max pool, fp32)."""
    op = ffi.make_op(ffi.OP_MAXPOOL, [ffi.INPUT], k_h=1, k_w=1, stride_h=1, stride_w=1)
    op.is_output = 1
    plan = ffi.Plan(ctx, [op], (3, oh, ow), 2, ffi.F32, 0)
    plan.finalize()
    try:
        plan.preprocess_u8(image, 1, PREP_MODES[mode], swap, mean, std)      # into the second image slot
        plan.preprocess_u8(image[::-1].copy(), 0, PREP_MODES[mode], swap, mean, std)
        plan.run_device(0, 2)
        return plan.read_output(0, 2)[1]
    finally:
        plan.close()


def test_image_preprocessing_on_device_is_bit_exact(ctx):
    """Against the vectors the reference code produced and, on larger seeded images, against the oracle."""
    from golden.make_preprocess_fixtures import CASES, MEAN, STD, case_image
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_preprocess.npz"))
    for k, (name, w, h, ow, oh, mode, swap) in enumerate(CASES):
        got = _prep_on_device(ctx, case_image(k, w, h), ow, oh, mode, swap, MEAN, STD)
        assert np.array_equal(got, gold[name]), name
    rng = np.random.default_rng(77)
    for (w, h, ow, oh, mode, swap) in [(640, 480, 608, 608, "yolo", 1), (333, 517, 416, 416, "yolo", 0), (1280, 720, 224, 224, "c3", 1),
                                       (97, 211, 224, 224, "transformed", 0), (608, 608, 608, 608, "yolo", 1)]:
        img = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        got = _prep_on_device(ctx, img, ow, oh, mode, swap, MEAN, STD)
        assert np.array_equal(got, mo.preprocess_u8(img, ow, oh, mode, swap, mean=MEAN, std=STD)), (w, h, mode)

