"""Generators of `.msnhnet` topology text for the benchmark nets and two nets that cover the remaining layer kinds.

The text is written in the reference's own grammar (src/io/MsnhParser.cpp:140-682 of the Msnhnet
source tree: order-significant `key: value` nodes, block nodes with `size:` repeat counts) and uses
the same node kinds the reference's model files use for these architectures (addblock / resblock /
res2block / concatblock for residual and SPP structure, separate conv / batchnorm / act nodes for
YOLOv5m), so the parser, the block lowering and the weight-blob order are exercised the way a
user's own file would. The architectures themselves are the published ones (ResNet-18,
YOLOv3-tiny, MobileNetV2, YOLOv4 = CSPDarknet53 + SPP + PANet, YOLOv5m with Focus and
BottleneckCSP); nothing here is read from a file.
"""


class _Writer:
    def __init__(self, batch, width, height, channels=3):
        self.lines = ["config:", f"  batch: {batch}", f"  width: {width}", f"  height: {height}", f"  channels: {channels}", ""]
        self.n = 0  # top-level layers emitted so far (block size counts)

    def node(self, kind, params=(), size=1):
        self.lines.append(f"# [{self.n}]")
        self.lines.append(f"{kind}:")
        for k, v in params:
            self.lines.append(f"  {k}: {v}")
        self.lines.append("")
        idx = self.n
        self.n += size
        return idx

    def raw(self, text, size=1):
        self.lines.append(f"# [{self.n}]")
        self.lines.extend(text.rstrip("\n").split("\n"))
        self.lines.append("")
        idx = self.n
        self.n += size
        return idx

    def text(self):
        return "\n".join(self.lines) + "\n"


def _conv_params(filters, k, s=1, p=None, act="none", bn=1, groups=1, use_bias=None):
    if p is None:
        p = (k - 1) // 2
    out = [("batchNorm", bn), ("filters", filters), ("kSize", k), ("stride", s)]
    if p:
        out.append(("padding", p))
    if groups != 1:
        out.append(("groups", groups))
    if use_bias is not None:
        out.append(("useBias", use_bias))
    out.append(("activation", act))
    return out


def _indent(params, depth):
    pad = "  " * depth
    return "\n".join(f"{pad}{k}: {v}" for k, v in params)


def _branch(convs):
    """A `branch:` of conv children (or the `empty:` branch when convs is None)."""
    if convs is None:
        return "  branch:\n    empty:\n"
    s = "  branch:\n"
    for c in convs:
        s += "    conv:\n" + _indent(c, 3) + "\n"
    return s


# --------------------------------------------------------------------------------------------------
def yolov3_tiny(size=416, batch=1, conf=0.2, nms=0.2):
    w = _Writer(batch, size, size)
    for i, f in enumerate((16, 32, 64, 128, 256)):
        w.node("conv", _conv_params(f, 3, act="leaky"))
        w.node("maxpool", [("kSize", 2), ("stride", 2)])
    route_src = w.n - 2  # the 256-channel conv at 26x26 for a 416 input
    w.node("conv", _conv_params(512, 3, act="leaky"))
    w.node("padding", [("top", 0), ("down", 1), ("left", 0), ("right", 1), ("paddingVal", 0)])
    w.node("maxpool", [("kSize", 2), ("stride", 1), ("ceilMode", 1)])
    w.node("conv", _conv_params(1024, 3, act="leaky"))
    w.node("conv", _conv_params(256, 1, act="leaky"))
    w.node("conv", _conv_params(512, 3, act="leaky"))
    w.node("conv", _conv_params(255, 1, bn=0))
    y0 = w.node("yolo", [("anchors", "81,82, 135,169, 344,319"), ("classNum", 80)])
    w.node("route", [("layers", -4)])
    w.node("conv", _conv_params(128, 1, act="leaky"))
    w.node("upsample", [("stride", 2)])
    w.node("route", [("layers", f"-1,{route_src}")])
    w.node("conv", _conv_params(256, 3, act="leaky"))
    w.node("conv", _conv_params(255, 1, bn=0))
    y1 = w.node("yolo", [("anchors", "10,14, 23,27, 37,58"), ("classNum", 80)])
    w.node("yoloout", [("layers", f"{y0},{y1}"), ("confThresh", conf), ("nmsThresh", nms), ("useSoftNms", 0), ("yoloType", "yolov3")])
    return w.text()


# --------------------------------------------------------------------------------------------------
def resnet18(size=224, batch=1, softmax=False):
    w = _Writer(batch, size, size)
    plain = dict(bn=0, use_bias=0)
    w.node("conv", _conv_params(64, 7, 2, 3, **plain))
    w.node("batchnorm", [("activation", "relu")])
    w.node("maxpool", [("kSize", 3), ("stride", 2), ("padding", 1)])

    def basic(c):
        s = "resblock:\n  size: 1\n"
        s += "  conv:\n" + _indent(_conv_params(c, 3, **plain), 2) + "\n  batchnorm:\n    activation: relu\n"
        s += "  conv:\n" + _indent(_conv_params(c, 3, **plain), 2) + "\n  batchnorm:\n    activation: none\n"
        s += "  activation: relu\n"
        w.raw(s)

    def down(c):
        s = "res2block:\n  size: 1\n  base:\n"
        s += "    conv:\n" + _indent(_conv_params(c, 3, 2, **plain), 3) + "\n    batchnorm:\n      activation: relu\n"
        s += "    conv:\n" + _indent(_conv_params(c, 3, **plain), 3) + "\n    batchnorm:\n      activation: none\n"
        s += "  branch:\n    conv:\n" + _indent(_conv_params(c, 1, 2, 0, **plain) + [("padding", 0)], 3) + "\n    batchnorm:\n      activation: none\n"
        s += "  activation: relu\n"
        w.raw(s)

    basic(64); basic(64)
    for c in (128, 256, 512):
        down(c); basic(c)
    w.node("localavgpool", [("kSize", 7), ("stride", 1), ("padding", 0)])
    w.node("connect", [("output", 1000), ("activation", "none")])
    if softmax:
        w.node("softmax", [])
    return w.text()


# --------------------------------------------------------------------------------------------------
def mobilenetv2(size=224, batch=1):
    w = _Writer(batch, size, size)
    w.node("conv", _conv_params(32, 3, 2, act="relu6"))

    def inverted(cin, cout, stride, t, repeats_with_identity=0):
        hidden = cin * t
        convs = []
        if t != 1:
            convs.append(_conv_params(hidden, 1, act="relu6"))
        convs.append(_conv_params(hidden, 3, stride, 1, act="relu6", groups=hidden))
        convs.append(_conv_params(cout, 1, act="none"))
        w.raw("addblock:\n  size: 1\n" + _branch(convs), 1)
        if repeats_with_identity:
            hidden2 = cout * t
            convs2 = [_conv_params(hidden2, 1, act="relu6"), _conv_params(hidden2, 3, 1, 1, act="relu6", groups=hidden2),
                      _conv_params(cout, 1, act="none")]
            w.raw(f"addblock:\n  size: {repeats_with_identity}\n" + _branch(convs2) + _branch(None), repeats_with_identity)

    # (expansion t, channels c, repeats n, stride s) of the published architecture
    cin = 32
    for t, c, n, s in ((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)):
        inverted(cin, c, s, t, n - 1)
        cin = c
    w.node("conv", _conv_params(1280, 1, act="relu6"))
    w.node("localavgpool", [("kSize", max(1, size // 32)), ("stride", 1), ("padding", 0)])
    w.node("connect", [("output", 1000), ("activation", "none")])
    return w.text()


# --------------------------------------------------------------------------------------------------
def yolov4(size=608, batch=1, conf=0.4, nms=0.5):
    w = _Writer(batch, size, size)
    m, l = "mish", "leaky"
    C = lambda f, k, s=1, a=m: w.node("conv", _conv_params(f, k, s, act=a))

    def residuals(c_mid, c_out, n, act):
        convs = [_conv_params(c_mid, 1, act=act), _conv_params(c_out, 3, act=act)]
        w.raw(f"addblock:\n  size: {n}\n" + _branch(convs) + _branch(None), n)

    def pairs(c1, k1, c2, k2, n):
        convs = [_conv_params(c1, k1, act=l), _conv_params(c2, k2, act=l)]
        w.raw(f"addblock:\n  size: {n}\n" + _branch(convs), n)

    def csp_stage(c_down, c_half, c_res_mid, n):
        C(c_down, 3, 2)
        C(c_half, 1)
        w.node("route", [("layers", -2)])
        C(c_half, 1)
        residuals(c_res_mid, c_half, n, m)
        C(c_half, 1)
        w.node("route", [("layers", f"-1,{-(n + 4)}")])
        return C(c_down if c_half != c_down else c_half, 1)

    C(32, 3)
    # stage 1 keeps the full width in both halves
    C(64, 3, 2); C(64, 1); w.node("route", [("layers", -2)]); C(64, 1)
    residuals(32, 64, 1, m)
    C(64, 1); w.node("route", [("layers", "-1,-5")]); C(64, 1)
    csp_stage(128, 64, 64, 2)
    s8 = csp_stage(256, 128, 128, 8)      # stride 8 feature
    s16 = csp_stage(512, 256, 256, 8)     # stride 16 feature
    csp_stage(1024, 512, 512, 4)
    C(512, 1, a=l); C(1024, 3, a=l); C(512, 1, a=l)
    spp = "concatblock:\n"
    for k in (13, 9, 5):
        spp += f"  branch:\n    maxpool:\n      kSize: {k}\n      stride: 1\n      padding: {(k - 1) // 2}\n"
    spp += "  branch:\n    empty:\n"
    w.raw(spp)
    C(512, 1, a=l); C(1024, 3, a=l); p5 = C(512, 1, a=l)
    C(256, 1, a=l); w.node("upsample", [("stride", 2)])
    w.node("route", [("layers", s16)]); C(256, 1, a=l); w.node("route", [("layers", "-1,-3")])
    pairs(256, 1, 512, 3, 2)
    p4 = C(256, 1, a=l)
    C(128, 1, a=l); w.node("upsample", [("stride", 2)])
    w.node("route", [("layers", s8)]); C(128, 1, a=l); w.node("route", [("layers", "-1,-3")])
    C(128, 1, a=l)
    pairs(256, 3, 128, 1, 2)
    C(256, 3, a=l)
    w.node("conv", _conv_params(255, 1, bn=0))
    y0 = w.node("yolo", [("anchors", "12, 16, 19, 36, 40, 28"), ("classNum", 80)])
    w.node("route", [("layers", -4)])
    C(256, 3, 2, a=l)
    w.node("route", [("layers", f"-1,{p4}")])
    pairs(256, 1, 512, 3, 2)
    C(256, 1, a=l)
    C(512, 3, a=l)
    w.node("conv", _conv_params(255, 1, bn=0))
    y1 = w.node("yolo", [("anchors", "36, 75, 76, 55, 72, 146"), ("classNum", 80)])
    w.node("route", [("layers", -4)])
    C(512, 3, 2, a=l)
    w.node("route", [("layers", f"-1,{p5}")])
    pairs(512, 1, 1024, 3, 3)
    w.node("conv", _conv_params(255, 1, bn=0))
    y2 = w.node("yolo", [("anchors", "142, 110, 192, 243, 459, 401"), ("classNum", 80)])
    w.node("yoloout", [("layers", f"{y0},{y1},{y2}"), ("confThresh", conf), ("nmsThresh", nms), ("useSoftNms", 0), ("yoloType", "yolov4")])
    return w.text()


# --------------------------------------------------------------------------------------------------
def yolov5m(size=640, batch=1, conf=0.25, nms=0.5, act="hardswish"):
    """YOLOv5m with Focus, BottleneckCSP blocks, SPP and a PANet head, written with separate
    conv / batchnorm (eps 1e-3) / act nodes. `act="swish"` gives the SiLU variant."""
    w = _Writer(batch, size, size)

    def conv(f, k, s=1, bias=0):
        return w.node("conv", [("filters", f), ("kSizeX", k), ("kSizeY", k), ("paddingX", k // 2), ("paddingY", k // 2),
                               ("strideX", s), ("strideY", s), ("dilationX", 1), ("dilationY", 1), ("groups", 1), ("useBias", bias)])

    def bn():
        return w.node("batchnorm", [("activation", "none"), ("eps", 0.001)])

    def cba(f, k, s=1):
        conv(f, k, s); bn()
        return w.node("act", [("activation", act)])

    def csp(c_out, n, shortcut):
        c_ = c_out // 2
        block_in = w.n - 1
        x = cba(c_, 1)
        for _ in range(n):
            cba(c_, 1)
            y = cba(c_, 3)
            x = w.node("varop", [("layers", x), ("type", "add"), ("constVal", 0.0)]) if shortcut else y
        a = conv(c_, 1)
        w.node("route", [("layers", block_in), ("addModel", 0)])
        b = conv(c_, 1)
        w.node("route", [("layers", f"{a},{b}"), ("addModel", 0)])
        bn()
        w.node("act", [("activation", "leaky,0.1")])
        return cba(c_out, 1)

    # Focus: four pixel-parity slices of the image, concatenated along channels
    w.node("act", [("activation", "none")])
    slices = []
    for i, (h0, w0) in enumerate(((0, 0), (1, 0), (0, 1), (1, 1))):
        if i:
            w.node("route", [("layers", 0), ("addModel", 0)])
        slices.append(w.node("slice", [("start0", 0), ("step0", 1), ("start1", h0), ("step1", 2), ("start2", w0), ("step2", 2)]))
    w.node("route", [("layers", ",".join(str(s) for s in slices)), ("addModel", 0)])
    cba(48, 3)
    cba(96, 3, 2); csp(96, 2, True)
    cba(192, 3, 2); p3 = csp(192, 6, True)
    cba(384, 3, 2); p4 = csp(384, 6, True)
    cba(768, 3, 2)
    x = cba(384, 1)
    pools = [x]
    for i, k in enumerate((5, 9, 13)):
        if i:
            w.node("route", [("layers", x), ("addModel", 0)])
        pools.append(w.node("maxpool", [("kSizeX", k), ("kSizeY", k), ("paddingX", k // 2), ("paddingY", k // 2),
                                        ("strideX", 1), ("strideY", 1), ("ceilMode", 0)]))
    w.node("route", [("layers", ",".join(str(p) for p in pools)), ("addModel", 0)])
    cba(768, 1)
    csp(768, 2, False)
    h5 = cba(384, 1)
    up = w.node("upsample", [("type", "nearest"), ("strideX", 2), ("strideY", 2), ("scaleX", 1.0), ("scaleY", 1.0), ("alignCorners", 0)])
    w.node("route", [("layers", f"{up},{p4}"), ("addModel", 0)])
    csp(384, 2, False)
    h4 = cba(192, 1)
    up = w.node("upsample", [("type", "nearest"), ("strideX", 2), ("strideY", 2), ("scaleX", 1.0), ("scaleY", 1.0), ("alignCorners", 0)])
    w.node("route", [("layers", f"{up},{p3}"), ("addModel", 0)])
    o3 = csp(192, 2, False)
    d = cba(192, 3, 2)
    w.node("route", [("layers", f"{d},{h4}"), ("addModel", 0)])
    o4 = csp(384, 2, False)
    d = cba(384, 3, 2)
    w.node("route", [("layers", f"{d},{h5}"), ("addModel", 0)])
    o5 = csp(768, 2, False)
    heads = []
    for src, anchors in ((o3, "10.0,13.0,16.0,30.0,33.0,23.0"), (o4, "30.0,61.0,62.0,45.0,59.0,119.0"), (o5, "116.0,90.0,156.0,198.0,373.0,326.0")):
        w.node("route", [("layers", src), ("addModel", 0)])
        conv(255, 1, 1, bias=1)
        heads.append(w.node("yolo", [("anchors", anchors), ("classNum", 80), ("yoloType", "yolov5")]))
    w.node("yoloout", [("layers", ",".join(str(h) for h in heads)), ("confThresh", conf), ("nmsThresh", nms), ("useSoftNms", 0), ("yoloType", "yolov5")])
    return w.text()


# --------------------------------------------------------------------------------------------------
def fcns(size=320, batch=1, classes=2):
    """FCN-8s-style segmentation net: VGG-16 encoder, five stride-2 transposed convolutions each followed by a
    BatchNorm and summed with the encoder's pooled feature map of the same size, 1x1 classifier with a sigmoid
    (the structure the reference ships as models/fcns/fcns.msnhnet)."""
    w = _Writer(batch, size, size)
    plain = dict(bn=0)
    pools = []
    for c, n in ((64, 2), (128, 2), (256, 3), (512, 3), (512, 3)):
        for _ in range(n):
            w.node("conv", _conv_params(c, 3, act="relu", **plain))
        pools.append(w.node("maxpool", [("kSize", 2), ("stride", 2)]))
    for c, skip in ((512, pools[3]), (256, pools[2]), (128, pools[1]), (64, pools[0]), (32, None)):
        w.node("deconv", [("filters", c), ("kSize", 2), ("stride", 2), ("activation", "relu")])
        w.node("batchnorm", [("activation", "none")])
        if skip is not None:
            w.node("route", [("layers", f"-1, {skip}"), ("addModel", 1)])
    w.node("conv", [("batchNorm", 0), ("filters", classes), ("kSize", 1), ("stride", 1), ("activation", "logistic")])
    return w.text()


def layer_zoo(size=64, batch=1):
    """A small net that strings together the layer kinds no benchmark net uses: transposed convolutions
    (non-overlapping, overlapping, padded, without bias), bilinear upsampling with and without aligned corners,
    clip, PReLU (on a conv and as a layer), depth max-pooling, pixel shuffle, permute, view and the four reductions, with odd channel counts in places so that the
    element-by-element kernel forms run too."""
    w = _Writer(batch, size, size)
    first = w.node("conv", _conv_params(16, 3, act="relu"))
    w.node("maxpool", [("kSize", 2), ("stride", 2)])
    w.node("deconv", [("filters", 16), ("kSize", 2), ("stride", 2), ("activation", "relu")])
    w.node("batchnorm", [("activation", "none")])
    w.node("route", [("layers", f"-1, {first}"), ("addModel", 1)])
    w.node("conv", _conv_params(32, 3, 2, act="prelu"))
    w.node("deconv", [("filters", 24), ("kSize", 3), ("stride", 2), ("padding", 1), ("activation", "none")])
    w.node("deconv", [("filters", 8), ("kSizeX", 4), ("kSizeY", 4), ("stride", 2), ("padding", 1), ("useBias", 0), ("activation", "leaky")])
    w.node("conv", _conv_params(32, 3, 2, act="relu"))
    w.node("upsample", [("type", "bilinear"), ("strideX", 1), ("strideY", 1), ("scaleX", 2.0), ("scaleY", 2.0), ("alignCorners", 0)])
    w.node("clip", [("min", 0.05), ("max", 0.5)])
    w.node("conv", _conv_params(24, 1, bn=0))
    w.node("act", [("activation", "prelu")])
    w.node("maxpool", [("maxPoolDepth", 1), ("outChannels", 16)])
    w.node("pixshf", [("factor", 2)])
    w.node("conv", _conv_params(8, 3, 4, 1, act="leaky"))
    w.node("permute", [("dim0", 1), ("dim1", 0), ("dim2", 2)])
    w.node("conv", _conv_params(16, 1, bn=0, act="relu"))
    n = size - 1                                              # plane edge after the stride-4 conv
    if (8 * n) % 24:
        raise ValueError("layer_zoo wants size - 1 divisible by 3")
    # view arguments: dim0 = new width, dim1 = new height, dim2 = new channel count
    w.node("view", [("dim0", n // 3), ("dim1", 24), ("dim2", 16)])
    up = w.node("upsample", [("type", "bilinear"), ("scaleX", 1.5), ("scaleY", 2.5), ("alignCorners", 1)])
    w.node("reduction", [("axis", 1), ("type", "mean")])
    w.node("route", [("layers", up)])
    w.node("reduction", [("axis", 0), ("type", "sum")])
    w.node("route", [("layers", up)])
    w.node("reduction", [("axis", 2), ("type", "mean")])
    w.node("route", [("layers", up)])
    w.node("reduction", [("axis", -1), ("type", "mean")])
    w.node("route", [("layers", up)])
    w.node("permute", [("dim0", 2), ("dim1", 1), ("dim2", 0)])
    w.node("conv", _conv_params(10, 3, act="relu"))
    w.node("globalavgpool")
    w.node("connect", [("output", 10), ("activation", "none")])
    return w.text()


def yolov5m_silu(**kw):
    """YOLOv5m with SiLU (the reference's `activation: swish`) in place of hard-swish."""
    return yolov5m(act="swish", **kw)


NETS = {
    "resnet18": resnet18,
    "yolov3_tiny": yolov3_tiny,
    "mobilenetv2": mobilenetv2,
    "yolov4": yolov4,
    "yolov5m": yolov5m,
    "yolov5m_silu": yolov5m_silu,
    "fcns": fcns,
    "layer_zoo": layer_zoo,
}
