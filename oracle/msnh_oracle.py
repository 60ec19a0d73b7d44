"""CPU restatement (numpy, fp32) of Msnhnet's forward path — TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may import this
module; nothing that ships calls it. It restates, layer by layer, what the reference's CPU `forward`
computes (file:line citations are into the Msnhnet source tree) on planar NCHW fp32 tensors, one
image at a time like the reference's batch-1 block layers. Pinned against the reference itself:
tests/golden holds per-layer outputs of the unmodified reference CPU path (built by oracle/Makefile,
scalar path, BaseLayer::supportAvx = false) on seeded weights, and tests/test_oracle_pin.py checks
this restatement against them.

Differences from the reference that are deliberate and documented:
  * GEMM accumulation order: numpy/BLAS blocked sums instead of the ascending-k loop of
    Gemm::cpuGemmNN (src/core/MsnhGemm.cpp:1163-1207); differences are at fp32 rounding level.
"""
import math

import numpy as np

F32 = np.float32
FLT_MAX = np.finfo(np.float32).max


# ------------------------------------------------------------------------------------------------
# .msnhnet parser (src/io/MsnhParser.cpp:140-682): order-significant key/value tree, duplicate keys
# are distinct nodes, block nodes with size: n expand to n layers, negative layer indices are
# relative to the layer that names them (:2162-2165).
# ------------------------------------------------------------------------------------------------
def _tree(text):
    items = []
    for ln, raw in enumerate(text.split("\n"), 1):
        raw = raw.lstrip("﻿").split("#")[0].rstrip()
        if not raw.strip():
            continue
        indent = len(raw) - len(raw.lstrip(" "))
        key, _, val = raw.strip().partition(":")
        items.append((indent, key.strip(), val.strip(), ln))

    def build(pos, indent):
        out = []
        while pos < len(items) and items[pos][0] == indent:
            _, k, v, ln = items[pos]
            pos += 1
            kids = []
            if pos < len(items) and items[pos][0] > indent:
                kids, pos = build(pos, items[pos][0])
            out.append((k, v, kids, ln))
        return out, pos

    roots, _ = build(0, 0)
    return roots


def _act(value):
    parts = [p.strip() for p in value.split(",")]
    return parts[0], [float(p) for p in parts[1:]]


def _geom(kids):
    g = {}
    for k, v, _, _ in kids:
        g[k] = v
    def pick(sq, x, y, default):
        sqv = int(g[sq]) if sq in g else default
        return (int(g[x]) if x in g else sqv), (int(g[y]) if y in g else sqv)
    kx, ky = pick("kSize", "kSizeX", "kSizeY", 1)
    sx, sy = pick("stride", "strideX", "strideY", 1)
    px, py = pick("padding", "paddingX", "paddingY", 0)
    dx, dy = pick("dilation", "dilationX", "dilationY", 1)
    return dict(kx=kx, ky=ky, sx=sx, sy=sy, px=px, py=py, dx=dx, dy=dy)


def _layer(node, self_index):
    k, v, kids, ln = node
    d = {"kind": k, "line": ln}
    kv = {ck: cv for ck, cv, _, _ in kids}

    def layers_list(s):
        out = []
        for p in s.split(","):
            i = int(p.strip())
            out.append(i + self_index if i < 0 else i)
        return out

    if k == "conv":
        d.update(_geom(kids))
        d.update(bn=int(kv.get("batchNorm", 0)), filters=int(kv.get("filters", 1)), groups=int(kv.get("groups", 1)),
                 use_bias=int(kv.get("useBias", 1)), eps=float(kv.get("eps", 1e-5)))
        d["act"], d["act_p"] = _act(kv.get("activation", "none"))
    elif k == "batchnorm":
        d["eps"] = float(kv.get("eps", 1e-5))
        d["act"], d["act_p"] = _act(kv.get("activation", "none"))
    elif k == "act":
        d["act"], d["act_p"] = _act(kv.get("activation", "none"))
    elif k in ("maxpool", "localavgpool"):
        d.update(_geom(kids))
        d["ceil"] = int(kv.get("ceilMode", 0))
        d["depth"] = int(kv.get("maxPoolDepth", 0)) if k == "maxpool" else 0
        d["out_channels"] = int(kv.get("outChannels", 1))
    elif k == "globalavgpool":
        pass
    elif k == "padding":
        d.update(top=int(kv.get("top", 0)), down=int(kv.get("down", 0)), left=int(kv.get("left", 0)), right=int(kv.get("right", 0)),
                 val=float(kv.get("paddingVal", 0)))
    elif k == "upsample":
        st = int(kv.get("stride", 1))
        sc = float(kv.get("scale", 1))
        d.update(sx=int(kv.get("strideX", st)), sy=int(kv.get("strideY", st)), mode=kv.get("type", "nearest"),
                 scale_x=float(kv.get("scaleX", sc)), scale_y=float(kv.get("scaleY", sc)), align=int(kv.get("alignCorners", 0)))
    elif k == "deconv":
        d.update(_geom(kids))
        d.update(filters=int(kv.get("filters", 1)), groups=int(kv.get("groups", 1)), use_bias=int(kv.get("useBias", 1)))
        d["act"], d["act_p"] = _act(kv.get("activation", "none"))
        if d["groups"] != 1:
            raise ValueError("deconv groups > 1 not covered by the oracle")
    elif k == "clip":
        d.update(lo=float(kv.get("min", -3.402823466e+38)), hi=float(kv.get("max", 3.402823466e+38)))
    elif k == "permute":
        d.update(dims=[int(kv.get(f"dim{i}", i)) for i in range(3)])
    elif k == "view":
        d.update(dims=[int(kv.get(f"dim{i}", -1)) for i in range(3)])
    elif k == "pixshf":
        d.update(factor=int(kv.get("factor", 0)))
    elif k == "reduction":
        d.update(axis=int(kv.get("axis", -1)), mean=kv.get("type", "sum") == "mean")
    elif k == "route":
        d.update(layers=layers_list(kv["layers"]), groups=int(kv.get("groups", 1)), group_id=int(kv.get("groupsId", 0)),
                 add=int(kv.get("addModel", 0)))
        d["act"], d["act_p"] = _act(kv.get("activation", "none"))
    elif k == "varop":
        d.update(layers=layers_list(kv["layers"]) if "layers" in kv else [], op=kv.get("type", "add"), const=float(kv.get("constVal", 0)))
    elif k == "slice":
        d.update(start=[int(kv.get(f"start{i}", 0)) for i in range(3)], step=[int(kv.get(f"step{i}", 1)) for i in range(3)])
    elif k == "connect":
        d.update(output=int(kv["output"]), bn=int(kv.get("batchNorm", 0)), use_bias=int(kv.get("useBias", 1)), eps=float(kv.get("bnEps", 1e-5)))
        d["act"], d["act_p"] = _act(kv.get("activation", "none"))
    elif k == "softmax":
        d.update(groups=int(kv.get("groups", 1)), temperature=float(kv.get("temperature", 1)))
    elif k == "empty":
        pass
    elif k == "yolo":
        d.update(anchors=[float(p) for p in kv["anchors"].split(",")], classes=int(kv.get("classNum", 1)), ytype=kv.get("yoloType", "yolov3"))
    elif k == "yoloout":
        d.update(layers=layers_list(kv["layers"]), conf=float(kv.get("confThresh", 0)), nms=float(kv.get("nmsThresh", 0)),
                 soft=int(kv.get("useSoftNms", 0)), ytype=kv.get("yoloType", "yolov3"))
    elif k in ("resblock", "res2block", "addblock", "concatblock"):
        d["act"], d["act_p"] = _act(kv.get("activation", "none"))
        if k == "resblock":
            d["chain"] = [_layer(c, -1) for c in kids if c[0] not in ("size", "activation")]
        elif k == "res2block":
            d["branches"] = [[_layer(c, -1) for c in kk] for ck, _, kk, _ in kids if ck in ("base", "branch")]
            order = [ck for ck, _, _, _ in kids if ck in ("base", "branch")]
            if order != ["base", "branch"]:
                raise ValueError("res2block wants base then branch")
        else:
            d["branches"] = [[_layer(c, -1) for c in kk] for ck, _, kk, _ in kids if ck == "branch"]
    else:
        raise ValueError(f"layer type {k} not covered by the oracle (line {ln})")
    return d


def parse_msnhnet(text):
    roots = _tree(text)
    if not roots or roots[0][0] != "config":
        raise ValueError("first node must be config")
    cfg = {k: int(v) for k, v, _, _ in roots[0][2]}
    layers = []
    for node in roots[1:]:
        size = 1
        if node[0] in ("resblock", "res2block", "addblock", "concatblock"):
            for ck, cv, _, _ in node[2]:
                if ck == "size":
                    size = int(cv)
        for _ in range(size):
            layers.append(_layer(node, len(layers)))
    return cfg, layers


# ------------------------------------------------------------------------------------------------
# activations: scalar definitions of include/Msnhnet/layers/MsnhActivations.h:39-168
# ------------------------------------------------------------------------------------------------
def activate(x, name, params=()):
    x = x.astype(F32, copy=False)
    if name == "none":
        return x
    if name == "logistic":
        return (1.0 / (1.0 + np.exp(-x))).astype(F32)
    if name == "loggy":
        return (2.0 / (1.0 + np.exp(-x)) - 1.0).astype(F32)
    if name == "relu6":
        return np.minimum(np.maximum(x, 0), 6).astype(F32)
    if name == "hardswish":                       # x*relu6(x+3)/6 (:59-62)
        return (x * np.minimum(np.maximum(x + F32(3), 0), 6) / F32(6)).astype(F32)
    if name == "elu":
        return np.where(x >= 0, x, np.exp(x) - 1).astype(F32)
    if name == "selu":
        return np.where(x >= 0, F32(1.0507) * x, F32(1.0507) * F32(1.6732) * (np.exp(x) - 1)).astype(F32)
    if name == "relie":
        return np.where(x > 0, x, F32(0.01) * x).astype(F32)
    if name == "ramp":
        return (x * (x > 0) + F32(0.1) * x).astype(F32)
    if name == "leaky":                           # default slope 0.1 (:84)
        a = F32(params[0]) if params else F32(0.1)
        return np.where(x > 0, x, a * x).astype(F32)
    if name == "tanh":
        e = np.exp(2 * x)
        return ((e - 1) / (e + 1)).astype(F32)
    if name == "hardtan":
        return np.clip(x, -1, 1).astype(F32)
    if name == "softplus":
        t = F32(params[0]) if params else F32(20)
        return _softplus(x, t)
    if name == "plse":
        return np.where(x < -4, F32(0.01) * (x + 4), np.where(x > 4, F32(0.01) * (x - 4) + 1, F32(0.125) * x + F32(0.5))).astype(F32)
    if name == "lhtan":
        return np.where(x < 0, F32(0.001) * x, np.where(x > 1, F32(0.001) * (x - 1) + 1, x)).astype(F32)
    if name == "mish":                            # x*tanh(softplus(x, 20)) (:160-164)
        return (x * np.tanh(_softplus(x, F32(20)))).astype(F32)
    if name == "swish":
        return (x / (1.0 + np.exp(-x))).astype(F32)
    if name == "stair":
        n = np.floor(x)
        return np.where(n % 2 == 0, np.floor(x / 2), (x - n) + np.floor(x / 2)).astype(F32)
    # every unknown name means relu in the reference (src/layers/MsnhActivations.cpp:29)
    return (x * (x > 0)).astype(F32)


# VariableOpLayer's one-operand types (include/Msnhnet/io/MsnhParser.h:400-428): libm functions of the input, `pow`
# with the layer's constVal as the exponent
UNARY_VAROPS = {"abs": lambda x, c: np.abs(x), "acos": lambda x, c: np.arccos(x), "asin": lambda x, c: np.arcsin(x), "atan": lambda x, c: np.arctan(x),
                "cos": lambda x, c: np.cos(x), "cosh": lambda x, c: np.cosh(x), "sin": lambda x, c: np.sin(x), "sinh": lambda x, c: np.sinh(x),
                "tan": lambda x, c: np.tan(x), "tanh": lambda x, c: np.tanh(x), "exp": lambda x, c: np.exp(x), "pow": lambda x, c: np.power(x, c),
                "log": lambda x, c: np.log(x), "log10": lambda x, c: np.log10(x), "sqrt": lambda x, c: np.sqrt(x)}


def _softplus(x, t):
    with np.errstate(over="ignore"):
        mid = np.log(np.exp(np.minimum(x, t)) + 1)
    return np.where(x > t, x, np.where(x < -t, np.exp(x), mid)).astype(F32)


# ------------------------------------------------------------------------------------------------
# layer math
# ------------------------------------------------------------------------------------------------
def conv2d(x, w, kx, ky, sx, sy, px, py, dx, dy, groups):
    """x [C,H,W], w [Cout, C/g, ky, kx] -> [Cout, OH, OW]; im2col + GEMM per group like
    ConvolutionalLayer::forward (src/layers/MsnhConvolutionalLayer.cpp:553-911), out size :388-398."""
    C, H, W = x.shape
    cout = w.shape[0]
    oh = (H + 2 * py - (dy * (ky - 1) + 1)) // sy + 1
    ow = (W + 2 * px - (dx * (kx - 1) + 1)) // sx + 1
    xp = np.zeros((C, H + 2 * py, W + 2 * px), F32)
    xp[:, py:py + H, px:px + W] = x
    cg, og = C // groups, cout // groups
    out = np.empty((cout, oh, ow), F32)
    if groups == C and og == 1:          # depthwise: per-channel taps
        acc = np.zeros((C, oh, ow), F32)
        for r in range(ky):
            for s in range(kx):
                patch = xp[:, r * dy: r * dy + (oh - 1) * sy + 1: sy, s * dx: s * dx + (ow - 1) * sx + 1: sx]
                acc += patch * w[:, 0, r, s][:, None, None]
        return acc
    for g in range(groups):
        cols = np.empty((cg, ky, kx, oh, ow), F32)
        for r in range(ky):
            for s in range(kx):
                cols[:, r, s] = xp[g * cg:(g + 1) * cg, r * dy: r * dy + (oh - 1) * sy + 1: sy, s * dx: s * dx + (ow - 1) * sx + 1: sx]
        wm = w[g * og:(g + 1) * og].reshape(og, cg * ky * kx)
        out[g * og:(g + 1) * og] = (wm @ cols.reshape(cg * ky * kx, oh * ow)).reshape(og, oh, ow)
    return out


def batchnorm(x, scales, biases, mean, var, eps):
    """scale*(x-mean)/sqrt(var+eps)+bias per channel (CPU form scaleSqrt*x + meanSqrt + bias,
    src/layers/MsnhConvolutionalLayer.cpp:811-856; BatchNormLayer the same)."""
    s = (scales / np.sqrt(var + F32(eps))).astype(F32)
    return (x * s[:, None, None] + (biases - mean * s)[:, None, None]).astype(F32)


def pool_out(n, pad, k, s, ceil):
    """MaxPoolLayer out-size rules (src/layers/MsnhMaxPoolLayer.cpp:37-100)."""
    if ceil == 1:
        rem = (n + 2 * pad - k) % s
        return (n + 2 * pad - k) // s + (1 if rem <= pad else 2)
    if ceil == 0:
        return (n + 2 * pad - k) // s + 1
    return (n + pad - k) // s + 1


def maxpool(x, kx, ky, sx, sy, px, py, ceil):
    """Window max; taps outside the plane never win (-FLT_MAX start, src/layers/MsnhMaxPoolLayer.cpp:318,334)."""
    C, H, W = x.shape
    oh, ow = pool_out(H, py, ky, sy, ceil), pool_out(W, px, kx, sx, ceil)
    eh, ew = (oh - 1) * sy + ky, (ow - 1) * sx + kx
    xp = np.full((C, max(eh, H + 2 * py), max(ew, W + 2 * px)), -FLT_MAX, F32)
    xp[:, py:py + H, px:px + W] = x
    out = np.full((C, oh, ow), -FLT_MAX, F32)
    for r in range(ky):
        for s in range(kx):
            out = np.maximum(out, xp[:, r: r + (oh - 1) * sy + 1: sy, s: s + (ow - 1) * sx + 1: sx])
    return out


def avgpool(x, kx, ky, sx, sy, px, py, ceil):
    """Mean over the taps inside the plane (src/layers/MsnhLocalAvgPoolLayer.cpp:300-340)."""
    C, H, W = x.shape
    oh, ow = pool_out(H, py, ky, sy, ceil), pool_out(W, px, kx, sx, ceil)
    eh, ew = (oh - 1) * sy + ky, (ow - 1) * sx + kx
    xp = np.zeros((C, max(eh, H + 2 * py), max(ew, W + 2 * px)), F32)
    cnt = np.zeros((1,) + xp.shape[1:], F32)
    xp[:, py:py + H, px:px + W] = x
    cnt[:, py:py + H, px:px + W] = 1
    acc = np.zeros((C, oh, ow), F32)
    n = np.zeros((1, oh, ow), F32)
    for r in range(ky):
        for s in range(kx):
            acc += xp[:, r: r + (oh - 1) * sy + 1: sy, s: s + (ow - 1) * sx + 1: sx]
            n += cnt[:, r: r + (oh - 1) * sy + 1: sy, s: s + (ow - 1) * sx + 1: sx]
    return (acc / n).astype(F32)


def upsample(x, sx, sy):
    """Nearest: out[h][w] = in[h/s][w/s] (Blas::cpuUpSample; GPU twin src/core/cuda/MsnhBlasGPU.cu:541-578)."""
    return np.repeat(np.repeat(x, sy, axis=1), sx, axis=2)


def bilinear_resize(x, out_w, out_h, align):
    """Blas::cpuBilinearResize (src/core/MsnhBlas.cpp:2400-2464), float32 step by step as written there."""
    c, h, w = x.shape
    rh = F32(1.0) * F32(h) / F32(out_h) if align == 0 else F32(1.0) * F32(h - 1) / F32(out_h - 1)
    rw = F32(1.0) * F32(w) / F32(out_w) if align == 0 else F32(1.0) * F32(w - 1) / F32(out_w - 1)
    h2 = np.arange(out_h, dtype=F32)
    w2 = np.arange(out_w, dtype=F32)
    if align == 0:
        h1r = np.maximum((rh * (h2 + F32(0.5))).astype(F32) - F32(0.5), F32(0)).astype(F32)
        w1r = np.maximum((rw * (w2 + F32(0.5))).astype(F32) - F32(0.5), F32(0)).astype(F32)
    else:
        h1r = (rh * h2).astype(F32)
        w1r = (rw * w2).astype(F32)
    h1 = h1r.astype(np.int64)
    w1 = w1r.astype(np.int64)
    h1p = (h1 < h - 1).astype(np.int64)
    w1p = (w1 < w - 1).astype(np.int64)
    lh1 = (h1r - h1.astype(F32)).astype(F32)[None, :, None]
    lh0 = (F32(1) - lh1).astype(F32)
    lw1 = (w1r - w1.astype(F32)).astype(F32)[None, None, :]
    lw0 = (F32(1) - lw1).astype(F32)
    a = x[:, h1][:, :, w1]
    b = x[:, h1][:, :, w1 + w1p]
    cc = x[:, h1 + h1p][:, :, w1]
    dd = x[:, h1 + h1p][:, :, w1 + w1p]
    top = ((lw0 * a).astype(F32) + (lw1 * b).astype(F32)).astype(F32)
    bot = ((lw0 * cc).astype(F32) + (lw1 * dd).astype(F32)).astype(F32)
    return ((lh0 * top).astype(F32) + (lh1 * bot).astype(F32)).astype(F32)


def deconv2d(x, w, kx, ky, sx, sy, px, py):
    """DeConvolutionalLayer::forward for groups 1 (src/layers/MsnhDeConvolutionalLayer.cpp:98-127): GEMM of the
    transposed weights [Cin][Cout*ky*kx] with the input planes, then Gemm::cpuCol2Im (src/core/MsnhGemm.cpp:115-154)."""
    cin, h, wd = x.shape
    cout = w.shape[1]
    oh = (h - 1) * sy - 2 * py + ky
    ow = (wd - 1) * sx - 2 * px + kx
    col = (w.reshape(cin, cout * ky * kx).T.astype(F32) @ x.reshape(cin, h * wd)).astype(F32).reshape(cout, ky, kx, h, wd)
    y = np.zeros((cout, oh + 2 * py, ow + 2 * px), F32)      # padded canvas; the border is what col2im drops
    for a in range(ky):
        for b in range(kx):
            y[:, a:a + (h - 1) * sy + 1:sy, b:b + (wd - 1) * sx + 1:sx] += col[:, a, b]
    return np.ascontiguousarray(y[:, py:py + oh, px:px + ow])


def permute_chw(x, dims):
    """PermuteLayer::forward (src/layers/MsnhPermuteLayer.cpp:127-183): input axis dims[k] becomes output axis k."""
    return np.ascontiguousarray(np.transpose(x, dims))


def pixel_shuffle(x, f):
    """PixelShuffleLayer::forward with the reference's own source index (src/layers/MsnhPixelShuffleLayer.cpp:98-104)."""
    c, h, w = x.shape
    oc, oh, ow = c // (f * f), h * f, w * f
    ci, hi, wi = np.meshgrid(np.arange(oc), np.arange(oh), np.arange(ow), indexing="ij")
    src = ci * f * w * h + hi * w + (wi % f) * w * h + wi // f
    return x.reshape(-1)[src].astype(F32)


def reduction(x, axis, mean):
    """ReductionLayer::forward (src/layers/MsnhReductionLayer.cpp:76-160), one image."""
    if axis == -1:
        y = x.sum(dtype=np.float64).astype(F32).reshape(1, 1, 1)
        n = x.size
    else:
        y = x.sum(axis=axis, keepdims=True, dtype=np.float64).astype(F32)
        n = x.shape[axis]
    return (y / F32(n)).astype(F32) if mean else y


def softmax(x, groups, temperature):
    """Blas::softmax per (image, group) over the flattened CHW order (src/core/MsnhBlas.cpp:1970-2110)."""
    flat = x.reshape(groups, -1).astype(F32)
    m = flat.max(axis=1, keepdims=True)
    e = np.exp(flat / F32(temperature) - m / F32(temperature)).astype(F32)
    return (e / e.sum(axis=1, keepdims=True)).astype(F32).reshape(x.shape)


def yolo_decode(x, anchors, classes, ytype, net_h):
    """YoloLayer::forward (src/layers/MsnhYoloLayer.cpp:217-284 for the math, :34 for the ratio)."""
    C, H, W = x.shape
    per = 5 + classes
    ratio = F32(net_h) / F32(H)
    out = x.reshape(3, per, H, W).astype(F32).copy()
    sig = lambda t: (F32(1) / (F32(1) + np.exp(-t))).astype(F32)
    col = np.arange(W, dtype=F32)[None, :].repeat(H, 0)
    row = np.arange(H, dtype=F32)[:, None].repeat(W, 1)
    for a in range(3):
        aw, ah = F32(anchors[2 * a]), F32(anchors[2 * a + 1])
        if ytype == "yolov5":
            out[a, 0] = (F32(2) * sig(out[a, 0]) - F32(0.5) + col) * ratio
            out[a, 1] = (F32(2) * sig(out[a, 1]) - F32(0.5) + row) * ratio
            out[a, 2] = aw * np.power(F32(2) * sig(out[a, 2]), F32(2))
            out[a, 3] = ah * np.power(F32(2) * sig(out[a, 3]), F32(2))
        else:
            out[a, 0] = (sig(out[a, 0]) + col) * ratio
            out[a, 1] = (sig(out[a, 1]) + row) * ratio
            with np.errstate(over="ignore"):
                out[a, 2] = aw * np.exp(out[a, 2])
                out[a, 3] = ah * np.exp(out[a, 3])
        out[a, 4:] = sig(out[a, 4:])
    return out.reshape(C, H, W)


def iou(b1, b2):
    """Box::iou with the +1 pixel convention (include/Msnhnet/utils/MsnhTypes.h:123-140)."""
    def corners(b):
        x, y, w, h = (F32(v) for v in b[:4])
        return x - w / F32(2), y - h / F32(2), x + w / F32(2), y + h / F32(2)
    ax1, ay1, ax2, ay2 = corners(b1)
    bx1, by1, bx2, by2 = corners(b2)
    iw = F32(min(ax2, bx2) - max(ax1, bx1) + F32(1))
    ih = F32(min(ay2, by2) - max(ay1, by1) + F32(1))
    inter = F32((F32(0) if iw < 0 else iw) * (F32(0) if ih < 0 else ih))
    a = F32((ax2 - ax1 + F32(1)) * (ay2 - ay1 + F32(1)))
    b = F32((bx2 - bx1 + F32(1)) * (by2 - by1 + F32(1)))
    return F32(inter / F32(a + b - inter))


def yolo_candidates(decoded_heads, classes, conf_thresh):
    """The scan of YoloOutLayer::forward (src/layers/MsnhYoloOutLayer.cpp:93-165): heads in order, per head
    anchor-major then cell; keep cells with objectness > threshold. Rows {x,y,w,h,conf,bestClsConf,bestClsIdx,order}."""
    rows = []
    base = 0
    per = 5 + classes
    for dec in decoded_heads:
        C, H, W = dec.shape
        d = dec.reshape(3, per, H * W)
        for a in range(3):
            keep = np.nonzero(d[a, 4] > F32(conf_thresh))[0]
            if keep.size:
                cls = d[a, 5:, keep]                       # [n, classes]
                best = cls.argmax(axis=1)                  # first maximum, like std::max_element
                r = np.empty((keep.size, 8), F32)
                r[:, 0:4] = d[a, 0:4, keep]
                r[:, 4] = d[a, 4, keep]
                r[:, 5] = cls[np.arange(keep.size), best]
                r[:, 6] = best
                r[:, 7] = base + a * H * W + keep
                rows.append(r)
        base += 3 * H * W
    return np.concatenate(rows, 0) if rows else np.zeros((0, 8), F32)


def _introsort_desc(keys):
    """Order produced by std::sort(idx, [](i,j){return a[i] > a[j];}) in libstdc++ is not stable; boxes with
    equal scores are vanishingly rare with float scores, so a stable descending argsort is used here and ties
    are reported by the parity tests instead of being reproduced."""
    return np.argsort(-keys, kind="stable")


def nms(rows, nms_thresh, soft=False, sigma=0.3):
    """Score sort + per-class greedy NMS keyed on objectness (src/layers/MsnhYoloOutLayer.cpp:167-197, :381-461)."""
    if len(rows) == 0:
        return np.zeros((0, 8), F32)
    score = (rows[:, 4] * rows[:, 5]).astype(F32)
    rows = rows[_introsort_desc(score)]
    classes = []
    for c in rows[:, 6].astype(int):
        if c not in classes:
            classes.append(c)
    best = []
    for c in classes:
        cur = [r for r in rows if int(r[6]) == c]
        if len(cur) == 1:
            best.append(cur[0])
            continue
        while cur:
            bi, bc = 0, -FLT_MAX
            for j, r in enumerate(cur):
                if r[4] > bc:
                    bi, bc = j, r[4]
            top = cur.pop(bi)
            best.append(top)
            keep = []
            for r in cur:
                v = iou(r, top)
                drop = (r[4] * math.exp(-(float(v) * float(v) / sigma)) <= 0) if soft else (v > F32(nms_thresh))
                if not drop:
                    keep.append(r)
            cur = keep
    return np.stack(best, 0).astype(F32)


# ------------------------------------------------------------------------------------------------
# the net
# ------------------------------------------------------------------------------------------------
class OracleNet:
    """Layer list + weights; `forward` runs one image like NetBuilder::runYolo / runClassify
    (src/net/MsnhNetBuilder.cpp:665-817)."""

    def __init__(self, text):
        self.cfg, self.layers = parse_msnhnet(text)
        self.weights = None
        self.calibration = None       # list filled by forward(calibrate=True)

    # ---- weight blob order (src/net/MsnhNetBuilder.cpp:635-661 and each layer's loadAllWeigths) ----
    def _weight_layers(self):
        """Leaf layers that own weights, in blob order."""
        out = []
        def leaf(d):
            if d["kind"] in ("conv", "connect", "batchnorm", "deconv") or (d["kind"] == "act" and d["act"] == "prelu"):
                out.append(d)
        for d in self.layers:
            if d["kind"] == "resblock":
                for c in d["chain"]:
                    leaf(c)
            elif d["kind"] in ("res2block", "addblock", "concatblock"):
                for br in d["branches"]:
                    for c in br:
                        leaf(c)
            else:
                leaf(d)
        return out

    def _shapes_pass(self):
        """Attach input channel counts to weight layers (needed to slice the blob)."""
        img = np.zeros((self.cfg["channels"], self.cfg["height"], self.cfg["width"]), F32)
        self.forward(img, shapes_only=True)

    def weight_count(self):
        self._shapes_pass()
        return sum(sum(n for _, n in self._slots(d)) for d in self._weight_layers())

    @staticmethod
    def _slots(d):
        if d["kind"] == "conv":
            n = d["filters"]
            s = [("w", n * (d["cin"] // d["groups"]) * d["ky"] * d["kx"])]
            if d["bn"]:
                s += [("scales", n), ("biases", n), ("mean", n), ("var", n)]    # src/layers/MsnhConvolutionalLayer.cpp:1303-1308
            elif d["use_bias"]:
                s += [("biases", n)]
            if d["act"] == "prelu":
                s += [("slopes", n)]                                            # src/layers/MsnhConvolutionalLayer.cpp:1316-1320
            return s
        if d["kind"] == "act":
            return [("slopes", d["cin"])]                                       # src/layers/MsnhActivationLayer.cpp:24-27
        if d["kind"] == "deconv":                          # src/layers/MsnhDeConvolutionalLayer.cpp:171-183
            n = d["filters"]
            s = [("w", d["cin"] * n * d["ky"] * d["kx"])]
            if d["use_bias"]:
                s += [("biases", n)]
            return s
        if d["kind"] == "connect":
            n = d["output"]
            s = [("w", n * d["inputs"])]
            if d["bn"]:
                s += [("scales", n), ("mean", n), ("var", n), ("biases", n)]    # src/layers/MsnhConnectedLayer.cpp:519-522
            elif d["use_bias"]:
                s += [("biases", n)]
            return s
        n = d["cin"]
        return [("scales", n), ("biases", n), ("mean", n), ("var", n)]          # src/layers/MsnhBatchNormLayer.cpp:469-472

    def load_weights(self, blob):
        blob = np.asarray(blob, F32)
        self._shapes_pass()
        off = 0
        for d in self._weight_layers():
            for name, n in self._slots(d):
                d[name] = blob[off:off + n]
                off += n
        if off != blob.size:
            raise ValueError(f"weights load err. needed : {off} given : {blob.size}")   # src/net/MsnhNetBuilder.cpp:657-661
        self.weights = blob

    # ---- forward ----
    def _simple(self, d, x, shapes_only, hook):
        k = d["kind"]
        if k == "conv":
            d["cin"] = x.shape[0]
            if shapes_only:
                oh = (x.shape[1] + 2 * d["py"] - (d["dy"] * (d["ky"] - 1) + 1)) // d["sy"] + 1
                ow = (x.shape[2] + 2 * d["px"] - (d["dx"] * (d["kx"] - 1) + 1)) // d["sx"] + 1
                return np.zeros((d["filters"], oh, ow), F32)
            w = d["w"].reshape(d["filters"], x.shape[0] // d["groups"], d["ky"], d["kx"])
            y = conv2d(x, w, d["kx"], d["ky"], d["sx"], d["sy"], d["px"], d["py"], d["dx"], d["dy"], d["groups"])
            if d["bn"]:
                y = batchnorm(y, d["scales"], d["biases"], d["mean"], d["var"], d["eps"])
            elif d["use_bias"]:
                y = (y + d["biases"][:, None, None]).astype(F32)
            if hook:
                y = hook(d, y)
            if d["act"] == "prelu":               # Activations::activatePRelu (src/layers/MsnhActivations.cpp:411-470)
                return np.where(y > 0, y, d["slopes"][:, None, None] * y).astype(F32)
            return activate(y, d["act"], d["act_p"])
        if k == "connect":
            d["inputs"] = x.size
            if shapes_only:
                return np.zeros((d["output"], 1, 1), F32)
            y = (d["w"].reshape(d["output"], x.size) @ x.reshape(-1)).astype(F32)
            if d["bn"]:
                s = (d["scales"] / np.sqrt(d["var"] + F32(d["eps"]))).astype(F32)
                y = (y * s + (d["biases"] - d["mean"] * s)).astype(F32)
            elif d["use_bias"]:
                y = (y + d["biases"]).astype(F32)
            y = y.reshape(-1, 1, 1)
            if hook:
                y = hook(d, y)
            return activate(y, d["act"], d["act_p"])
        if k == "batchnorm":
            d["cin"] = x.shape[0]
            if shapes_only:
                return x
            y = batchnorm(x, d["scales"], d["biases"], d["mean"], d["var"], d["eps"])
            if hook:
                y = hook(d, y)
            return activate(y, d["act"], d["act_p"])
        if k == "act":
            if d["act"] == "prelu":
                d["cin"] = x.shape[0]
                return x if shapes_only else np.where(x > 0, x, d["slopes"][:, None, None] * x).astype(F32)
            return activate(x, d["act"], d["act_p"])
        if k == "maxpool":
            if d["depth"]:                        # src/layers/MsnhMaxPoolLayer.cpp:244-270
                g = d["out_channels"]
                return np.stack([x[j::g].max(axis=0) for j in range(g)]).astype(F32)
            return maxpool(x, d["kx"], d["ky"], d["sx"], d["sy"], d["px"], d["py"], d["ceil"])
        if k == "localavgpool":
            return avgpool(x, d["kx"], d["ky"], d["sx"], d["sy"], d["px"], d["py"], d["ceil"])
        if k == "globalavgpool":
            return x.mean(axis=(1, 2), keepdims=True).astype(F32)
        if k == "padding":
            return np.pad(x, ((0, 0), (d["top"], d["down"]), (d["left"], d["right"])), constant_values=F32(d["val"])).astype(F32)
        if k == "upsample":
            if d["mode"] == "bilinear":              # src/layers/MsnhUpSampleLayer.cpp:19-23, :84-87
                return bilinear_resize(x, int(x.shape[2] * F32(d["scale_x"])), int(x.shape[1] * F32(d["scale_y"])), d["align"])
            return upsample(x, d["sx"], d["sy"])
        if k == "deconv":
            d["cin"] = x.shape[0]
            if shapes_only:
                return np.zeros((d["filters"], (x.shape[1] - 1) * d["sy"] - 2 * d["py"] + d["ky"], (x.shape[2] - 1) * d["sx"] - 2 * d["px"] + d["kx"]), F32)
            y = deconv2d(x, d["w"].reshape(x.shape[0], d["filters"], d["ky"], d["kx"]), d["kx"], d["ky"], d["sx"], d["sy"], d["px"], d["py"])
            if d["use_bias"]:
                y = (y + d["biases"][:, None, None]).astype(F32)
            if hook:
                y = hook(d, y)
            return activate(y, d["act"], d["act_p"])
        if k == "clip":                               # src/layers/MsnhClipLayer.cpp
            return np.minimum(np.maximum(x, F32(d["lo"])), F32(d["hi"])).astype(F32)
        if k == "permute":
            return permute_chw(x, d["dims"])
        if k == "view":                               # dim0/1/2 = outWidth/outHeight/outChannel (src/net/MsnhNetBuilder.cpp:478-482)
            if d["dims"][0] * d["dims"][1] * d["dims"][2] != x.size:
                raise ValueError("view op params error")
            return np.ascontiguousarray(x.reshape(d["dims"][2], d["dims"][1], d["dims"][0]))
        if k == "pixshf":
            return pixel_shuffle(x, d["factor"])
        if k == "reduction":
            return reduction(x, d["axis"], d["mean"])
        if k == "slice":                # src/layers/MsnhSliceLayer.cpp:24-50
            s, t = d["start"], d["step"]
            return np.ascontiguousarray(x[s[0]::t[0], s[1]::t[1], s[2]::t[2]])
        if k == "softmax":
            return softmax(x, d["groups"], d["temperature"])
        if k == "empty":
            return x
        raise ValueError(k)

    def forward(self, img, shapes_only=False, hook=None, keep_layers=True):
        """img: [C,H,W] fp32. Returns dict(layers=[per top-level layer output or None], decoded=[yolo heads],
        candidates=rows, boxes=rows after NMS, out=last tensor)."""
        outs = []
        x = np.asarray(img, F32)
        res = {"decoded": {}, "candidates": None, "boxes": None}
        for li, d in enumerate(self.layers):
            k = d["kind"]
            if k == "route":                                  # src/layers/MsnhRouteLayer.cpp:93-190
                ins = [outs[i] for i in d["layers"]]
                if d["add"] == 1:
                    y = ins[0].copy()
                    for t in ins[1:]:
                        y = (y + t).astype(F32)
                else:
                    g = d["groups"]
                    parts = []
                    for t in ins:
                        c = t.shape[0] // g
                        parts.append(t[c * d["group_id"]: c * (d["group_id"] + 1)])
                    y = np.concatenate(parts, 0)
                y = activate(y, d["act"], d["act_p"])
            elif k == "varop":                                # src/layers/MsnhVariableOpLayer.cpp:80-190
                op = d["op"]
                if op in UNARY_VAROPS:                        # one-operand forms, src/core/MsnhBlas.cpp:425-1400 (cpuScientific)
                    y = UNARY_VAROPS[op](x.astype(F32), F32(d["const"])).astype(F32)
                elif op.endswith("Const") or op.endswith("ConstInv"):
                    a, b = x, F32(d["const"])
                    op = op.replace("Const", "")
                elif len(d["layers"]) == 2:
                    a, b = outs[d["layers"][0]], outs[d["layers"][1]]
                else:
                    a, b = x, outs[d["layers"][0]]
                if d["op"] not in UNARY_VAROPS:
                    y = {"add": lambda: a + b, "sub": lambda: a - b, "subInv": lambda: b - a, "mul": lambda: a * b,
                         "div": lambda: a / b, "divInv": lambda: b / a}[op]().astype(F32)
            elif k == "resblock":                             # src/layers/MsnhResBlockLayer.cpp:230-300
                y = x
                for c in d["chain"]:
                    y = self._simple(c, y, shapes_only, hook)
                y = activate((x + y).astype(F32), d["act"], d["act_p"])
            elif k == "res2block":                            # src/layers/MsnhRes2BlockLayer.cpp
                ys = []
                for br in d["branches"]:
                    y = x
                    for c in br:
                        y = self._simple(c, y, shapes_only, hook)
                    ys.append(y)
                y = activate((ys[0] + ys[1]).astype(F32), d["act"], d["act_p"])
            elif k in ("addblock", "concatblock"):            # src/layers/MsnhAddBlockLayer.cpp:255-358, MsnhConcatBlockLayer.cpp:255-355
                ys = []
                for br in d["branches"]:
                    y = x
                    for c in br:
                        y = self._simple(c, y, shapes_only, hook)
                    ys.append(y)
                if k == "addblock":
                    y = ys[0]
                    for t in ys[1:]:
                        y = (y + t).astype(F32)
                else:
                    y = np.concatenate(ys, 0)
                y = activate(y, d["act"], d["act_p"])
            elif k == "yolo":
                y = x if shapes_only else yolo_decode(x, d["anchors"], d["classes"], d["ytype"], self.cfg["height"])
                res["decoded"][li] = y
            elif k == "yoloout":
                if not shapes_only:
                    heads = [res["decoded"][i] for i in d["layers"]]
                    classes = self.layers[d["layers"][0]]["classes"]
                    res["candidates"] = yolo_candidates(heads, classes, d["conf"])
                    res["boxes"] = nms(res["candidates"], d["nms"], bool(d["soft"]))
                outs.append(None)
                continue
            else:
                y = self._simple(d, x, shapes_only, hook)
            outs.append(y if keep_layers or True else None)
            x = y
        res["layers"] = outs
        res["out"] = x
        return res


# ---------------------------------------------------------------------------------------------------
# Image preprocessing in front of the net (the reference's own Mat path, i.e. the C API built without OpenCV)
# ---------------------------------------------------------------------------------------------------
def resize_bilinear_u8(src, out_w, out_h):
    """MatOp::resize, RESIZE_BILINEAR on 8-bit pixels (src/cv/MsnhCVMatOp.cpp:142-160, :399-434): float32
    arithmetic in the source's operation order, result converted float -> uint16 (truncation, wrapping for
    the negative values the clamped last row/column produce) and clamped to 255. src: [h][w][c] uint8."""
    h, w = src.shape[:2]
    if (out_w, out_h) == (w, h):
        return src
    one, half = F32(1.0), F32(0.5)
    fx, fy = one * F32(w) / F32(out_w), one * F32(h) / F32(out_h)
    ih = (np.arange(out_h, dtype=F32) + half) * fy - half
    ih = np.where(ih < 0, F32(0), ih).astype(F32)
    iw = (np.arange(out_w, dtype=F32) + half) * fx - half
    iw = np.where(iw < 0, F32(0), iw).astype(F32)
    h0 = ih.astype(np.int32); h1 = np.minimum(h0 + 1, h - 1)
    w0 = iw.astype(np.int32); w1 = np.minimum(w0 + 1, w - 1)
    wh1 = (h1.astype(F32) - ih)[:, None, None]; wh0 = (ih - h0.astype(F32))[:, None, None]
    ww1 = (w1.astype(F32) - iw)[None, :, None]; ww0 = (iw - w0.astype(F32))[None, :, None]
    p = src.astype(F32)
    p00, p01 = p[h0][:, w0], p[h0][:, w1]
    p10, p11 = p[h1][:, w0], p[h1][:, w1]
    top = (wh1 * ((ww1 * p00).astype(F32) + (ww0 * p01).astype(F32)).astype(F32)).astype(F32)
    bot = (wh0 * ((ww1 * p10).astype(F32) + (ww0 * p11).astype(F32)).astype(F32)).astype(F32)
    res = (top + bot).astype(F32)
    r16 = (np.trunc(res).astype(np.int64) & 0xFFFF)           # static_cast<uint16_t>(float)
    return np.where(r16 > 255, 255, r16).astype(np.uint8)


def letterbox_127(src):
    """The pad-to-square step of getPaddingZeroF32C3 (src/utils/MsnhCVUtil.cpp:219-229): 127-gray bars of
    diff/2 and diff - diff/2 pixels on the short side."""
    h, w = src.shape[:2]
    diff = abs(w - h)
    if w > h:
        return np.pad(src, ((diff // 2, diff - diff // 2), (0, 0), (0, 0)), constant_values=127)
    if w < h:
        return np.pad(src, ((0, 0), (diff // 2, diff - diff // 2), (0, 0)), constant_values=127)
    return src


def preprocess_u8(image, out_w, out_h, mode, swap_rgb, mean=None, std=None):
    """What the reference's C API does to a raw 8-bit RGB image before the net (src/c_api/MsnhnetLib.cpp:540-600
    runClassifyList, :754-778 runYoloList): channel swap when swapRGB == 0 (sic), then one of
    src/utils/MsnhCVUtil.cpp's getters: 'yolo'/'padzero' :203-258, 'c3' :91-137, 'googlenet' :146-193,
    'transformed' :269-316, 'caffe' :326-373. image: [h][w][3] uint8 -> planar CHW float32."""
    assert image.ndim == 3 and image.shape[2] == 3 and image.dtype == np.uint8
    img = image if swap_rgb else image[:, :, ::-1]
    if mode in ("yolo", "padzero"):
        img = letterbox_127(img)
    img = resize_bilinear_u8(np.ascontiguousarray(img), out_w, out_h)
    if mode not in ("yolo", "padzero"):                  # these getters default to needShuffleRGB = true
        img = img[:, :, ::-1]
    u = img.astype(F32).transpose(2, 0, 1)
    if mode in ("yolo", "padzero", "c3"):
        return (u / F32(255.0)).astype(F32)
    if mode == "googlenet":
        a = [F32(0.229) / F32(0.5), F32(0.224) / F32(0.5), F32(0.225) / F32(0.5)]
        b = [(F32(0.485) - F32(0.5)) / F32(0.5), (F32(0.456) - F32(0.5)) / F32(0.5), (F32(0.406) - F32(0.5)) / F32(0.5)]
        return np.stack([(((u[k] / F32(255.0)).astype(F32) * a[k]).astype(F32) + b[k]).astype(F32) for k in range(3)])
    if mode == "transformed":
        return np.stack([(((u[k] / F32(255.0)).astype(F32) - F32(mean[k])).astype(F32) / F32(std[k])).astype(F32) for k in range(3)])
    if mode == "caffe":
        return np.stack([(u[k] - F32(v)).astype(F32) for k, v in enumerate((123.68, 116.779, 103.939))])
    raise ValueError(mode)
