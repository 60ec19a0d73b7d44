#include "msnh_netbuilder.h"

#include <algorithm>
#include <cfloat>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sys/stat.h>
#include <iomanip>
#include <sstream>

#include "msnh_b200.h"

namespace Msnhnet {

bool NetBuilder::onlyUseGpu = false;
bool NetBuilder::onlyUseCpu = false;
bool NetBuilder::useFp16 = false;
bool NetBuilder::onlyUseCuda = false;
bool NetBuilder::isPreviewMode = false;

void NetBuilder::setPreviewMode(const bool &mode) { isPreviewMode = mode; }
void NetBuilder::setMemAlign(const bool &) {}
void NetBuilder::setOnlyGpu(const bool &v) { onlyUseGpu = v; }
void NetBuilder::setOnlyCpu(const bool &v) { onlyUseCpu = v; }
void NetBuilder::setUseFp16(const bool &v) { useFp16 = v; }
void NetBuilder::setForceUseCuda(const bool &v) { onlyUseCuda = v; }

// include/Msnhnet/utils/MsnhTypes.h:123-140: corner boxes, +1 pixel convention
float Box::iou(const XYWHBox &a, const XYWHBox &b) {
    const float ax1 = a.x - a.w / 2.f, ax2 = a.x + a.w / 2.f, ay1 = a.y - a.h / 2.f, ay2 = a.y + a.h / 2.f;
    const float bx1 = b.x - b.w / 2.f, bx2 = b.x + b.w / 2.f, by1 = b.y - b.h / 2.f, by2 = b.y + b.h / 2.f;
    const float ix1 = std::max(ax1, bx1), iy1 = std::max(ay1, by1), ix2 = std::min(ax2, bx2), iy2 = std::min(ay2, by2);
    const float iw = ix2 - ix1 + 1, ih = iy2 - iy1 + 1;
    const float inter = (iw < 0 ? 0 : iw) * (ih < 0 ? 0 : ih);
    const float areaA = (ax2 - ax1 + 1) * (ay2 - ay1 + 1), areaB = (bx2 - bx1 + 1) * (by2 - by1 + 1);
    return 1.f * inter / (areaA + areaB - inter);
}

NetBuilder::NetBuilder() {}
NetBuilder::~NetBuilder() {
    destroyPlan();
    if (_ctx) msnh_b200_ctx_destroy(_ctx);
}
void NetBuilder::destroyPlan() {
    if (_plan) { msnh_b200_plan_destroy(_plan); _plan = nullptr; }
}
void NetBuilder::clearLayers() {
    destroyPlan();
    _layerOp.clear(); _layerNames.clear(); _weightSlots.clear();
    _totalWeights = 0; _weightsLoaded = false; _lastOp = -1; _collectOp = -1;
}
void NetBuilder::setDevice(int device) { _device = device; }
void NetBuilder::setBatch(int batch) { _batchOverride = batch; }
void NetBuilder::setPlanFlags(unsigned flags) { _planFlags = flags; }

void NetBuilder::checkK(int rc, const char *what) {
    if (rc != MSNH_B200_OK)
        MSNH_THROW(std::string(what) + " failed (status " + std::to_string(rc) + "): " + (_ctx ? msnh_b200_last_error(_ctx) : "no context"));
}

// ------------------------------------------------------------------------------------------------
// lowering: Msnhnet layers -> primitive ops of the kernel library
// ------------------------------------------------------------------------------------------------
namespace {

struct Sh { int c = 0, h = 0, w = 0; };

int actCode(const std::string &name, int line) {
    static const struct { const char *n; int code; } table[] = {
        {"none", MSNH_ACT_NONE}, {"logistic", MSNH_ACT_LOGISTIC}, {"loggy", MSNH_ACT_LOGGY}, {"relu", MSNH_ACT_RELU},
        {"relu6", MSNH_ACT_RELU6}, {"hardswish", MSNH_ACT_HARD_SWISH}, {"elu", MSNH_ACT_ELU}, {"selu", MSNH_ACT_SELU},
        {"relie", MSNH_ACT_RELIE}, {"ramp", MSNH_ACT_RAMP}, {"leaky", MSNH_ACT_LEAKY}, {"tanh", MSNH_ACT_TANH},
        {"stair", MSNH_ACT_STAIR}, {"hardtan", MSNH_ACT_HARDTAN}, {"softplus", MSNH_ACT_SOFT_PLUS}, {"plse", MSNH_ACT_PLSE},
        {"lhtan", MSNH_ACT_LHTAN}, {"mish", MSNH_ACT_MISH}, {"swish", MSNH_ACT_SWISH}};
    for (auto &t : table) if (name == t.n) return t.code;
    if (name == "prelu") MSNH_THROW("activation 'prelu' is only supported on conv and act layers (line " + std::to_string(line) + ")");
    if (name.rfind("normalize_channels", 0) == 0)
        MSNH_THROW("activation '" + name + "' is not supported by this backend (line " + std::to_string(line) + ")");
    return MSNH_ACT_RELU;   // the reference maps every unknown name to relu (src/layers/MsnhActivations.cpp:29)
}
float actParam(const LayerDesc &d, int code) {
    if (!d.actParams.empty()) return d.actParams[0];
    if (code == MSNH_ACT_LEAKY) return 0.1f;        // include/Msnhnet/layers/MsnhActivations.h:84
    if (code == MSNH_ACT_SOFT_PLUS) return 20.f;
    return 0.f;
}

struct Lowering {
    std::vector<MsnhB200Op> ops;
    std::vector<Sh> shapes;
    struct WS { int op, slot; size_t count; int rows; };
    std::vector<WS> weights;

    static MsnhB200Op blank(int kind) {
        MsnhB200Op o;
        std::memset(&o, 0, sizeof(o));
        o.kind = kind;
        o.k_h = o.k_w = o.stride_h = o.stride_w = o.dil_h = o.dil_w = o.groups = 1;
        o.bn_eps = 1e-5f; o.scale = 1.f; o.route_groups = 1; o.softmax_groups = 1; o.softmax_temperature = 1.f;
        for (int i = 0; i < 3; ++i) o.slice_step[i] = 1;
        return o;
    }
    Sh shapeOf(int op, const Sh &input) const { return op == MSNH_B200_INPUT ? input : shapes[op]; }
    int emit(const MsnhB200Op &o, const Sh &s) { ops.push_back(o); shapes.push_back(s); return static_cast<int>(ops.size()) - 1; }
    void setAct(MsnhB200Op &o, const LayerDesc &d) { o.act = actCode(d.activation, d.line); o.act_param = actParam(d, o.act); }

    int activation(int in, const Sh &s, const LayerDesc &d) {
        const int code = actCode(d.activation, d.line);
        if (code == MSNH_ACT_NONE) return in;
        MsnhB200Op o = blank(MSNH_OP_ACTIVATION);
        o.n_in = 1; o.in[0] = in; o.act = code; o.act_param = actParam(d, code);
        return emit(o, s);
    }

    int prelu(int in, const Sh *inShape = nullptr) {
        const Sh a = inShape ? *inShape : shapes[in];
        MsnhB200Op o = blank(MSNH_OP_PRELU);
        o.n_in = 1; o.in[0] = in;
        const int id = emit(o, a);
        weights.push_back({id, MSNH_W_WEIGHTS, static_cast<size_t>(a.c), a.c});
        return id;
    }

    // one non-block layer applied to `in`; returns the op holding its output
    int simple(const LayerDesc &d, int in, const Sh &netIn) {
        const Sh a = shapeOf(in, netIn);
        switch (d.kind) {
            case LayerKind::Conv: {
                if (d.activation == "prelu") {
                    // per-channel slopes follow the conv's own tensors in the blob (src/layers/MsnhConvolutionalLayer.cpp:1316-1320)
                    LayerDesc plain = d; plain.activation = "none"; plain.actParams.clear();
                    return prelu(simple(plain, in, netIn));
                }
                MsnhB200Op o = blank(MSNH_OP_CONV);
                o.n_in = 1; o.in[0] = in; o.filters = d.filters;
                o.k_h = d.kSizeY; o.k_w = d.kSizeX; o.stride_h = d.strideY; o.stride_w = d.strideX;
                o.pad_h = d.paddingY; o.pad_w = d.paddingX; o.dil_h = d.dilationY; o.dil_w = d.dilationX; o.groups = d.groups;
                o.has_bn = d.batchNorm ? 1 : 0; o.has_bias = (!d.batchNorm && d.useBias) ? 1 : 0; o.bn_eps = d.eps;
                setAct(o, d);
                if (d.groups < 1 || a.c % d.groups || d.filters % d.groups) MSNH_THROW("[conv] groups must divide channels (line " + std::to_string(d.line) + ")");
                Sh s; s.c = d.filters;
                s.h = (a.h + 2 * o.pad_h - (o.dil_h * (o.k_h - 1) + 1)) / o.stride_h + 1;   // src/layers/MsnhConvolutionalLayer.cpp:388-398
                s.w = (a.w + 2 * o.pad_w - (o.dil_w * (o.k_w - 1) + 1)) / o.stride_w + 1;
                if (s.h < 1 || s.w < 1) MSNH_THROW("[conv] kernel larger than padded input (line " + std::to_string(d.line) + ")");
                const int id = emit(o, s);
                weights.push_back({id, MSNH_W_WEIGHTS, static_cast<size_t>(d.filters) * (a.c / d.groups) * o.k_h * o.k_w, d.filters});
                if (d.batchNorm) for (int sl : {MSNH_W_BN_SCALE, MSNH_W_BN_BIAS, MSNH_W_BN_MEAN, MSNH_W_BN_VAR}) weights.push_back({id, sl, static_cast<size_t>(d.filters), 0});
                else if (d.useBias) weights.push_back({id, MSNH_W_BIAS, static_cast<size_t>(d.filters), 0});
                return id;
            }
            case LayerKind::Connect: {
                MsnhB200Op o = blank(MSNH_OP_CONNECTED);
                o.n_in = 1; o.in[0] = in; o.filters = d.output;
                o.has_bn = d.batchNorm ? 1 : 0; o.has_bias = (!d.batchNorm && d.useBias) ? 1 : 0; o.bn_eps = d.eps;
                setAct(o, d);
                if (d.output < 1) MSNH_THROW("[connect] output must be positive (line " + std::to_string(d.line) + ")");
                Sh s; s.c = d.output; s.h = 1; s.w = 1;
                const int id = emit(o, s);
                weights.push_back({id, MSNH_W_WEIGHTS, static_cast<size_t>(d.output) * a.c * a.h * a.w, d.output});
                // blob order of the connected layer: scales, rollMean, rollVariance, biases (src/layers/MsnhConnectedLayer.cpp:519-522)
                if (d.batchNorm) for (int sl : {MSNH_W_BN_SCALE, MSNH_W_BN_MEAN, MSNH_W_BN_VAR, MSNH_W_BN_BIAS}) weights.push_back({id, sl, static_cast<size_t>(d.output), 0});
                else if (d.useBias) weights.push_back({id, MSNH_W_BIAS, static_cast<size_t>(d.output), 0});
                return id;
            }
            case LayerKind::BatchNorm: {
                MsnhB200Op o = blank(MSNH_OP_BATCHNORM);
                o.n_in = 1; o.in[0] = in; o.bn_eps = d.eps; setAct(o, d);
                const int id = emit(o, a);
                for (int sl : {MSNH_W_BN_SCALE, MSNH_W_BN_BIAS, MSNH_W_BN_MEAN, MSNH_W_BN_VAR}) weights.push_back({id, sl, static_cast<size_t>(a.c), 0});
                return id;
            }
            case LayerKind::Act: {
                if (d.activation == "prelu") return prelu(in, &a);      // src/layers/MsnhActivationLayer.cpp:24-27, :132-136
                MsnhB200Op o = blank(MSNH_OP_ACTIVATION);
                o.n_in = 1; o.in[0] = in; setAct(o, d);
                return emit(o, a);
            }
            case LayerKind::MaxPool: case LayerKind::LocalAvgPool: {
                MsnhB200Op o = blank(d.kind == LayerKind::MaxPool ? MSNH_OP_MAXPOOL : MSNH_OP_AVGPOOL);
                o.n_in = 1; o.in[0] = in;
                o.k_h = d.kSizeY; o.k_w = d.kSizeX; o.stride_h = d.strideY; o.stride_w = d.strideX; o.pad_h = d.paddingY; o.pad_w = d.paddingX;
                if (d.kind == LayerKind::MaxPool && d.maxPoolDepth) {       // src/layers/MsnhMaxPoolLayer.cpp:37-42
                    if (d.outChannels < 1 || d.outChannels > a.c) MSNH_THROW("[maxpool] outChannels must be 1..channels with maxPoolDepth (line " + std::to_string(d.line) + ")");
                    o.filters = d.outChannels;
                    Sh s = a; s.c = d.outChannels;
                    return emit(o, s);
                }
                Sh s; s.c = a.c;
                // output plane rules of the reference (src/layers/MsnhMaxPoolLayer.cpp:37-100)
                auto dim = [&](int len, int pad, int k, int st) {
                    if (d.ceilMode == 1) {
                        const int rem = (len + 2 * pad - k) % st;
                        if (rem >= k) MSNH_THROW("pool padding error (line " + std::to_string(d.line) + ")");
                        return (len + 2 * pad - k) / st + (rem <= pad ? 1 : 2);
                    }
                    if (d.ceilMode == 0) return (len + 2 * pad - k) / st + 1;
                    return (len + pad - k) / st + 1;
                };
                s.w = dim(a.w, o.pad_w, o.k_w, o.stride_w); s.h = dim(a.h, o.pad_h, o.k_h, o.stride_h);
                if (s.h < 1 || s.w < 1) MSNH_THROW("pool window larger than input (line " + std::to_string(d.line) + ")");
                o.out_h = s.h; o.out_w = s.w;
                return emit(o, s);
            }
            case LayerKind::GlobalAvgPool: {
                MsnhB200Op o = blank(MSNH_OP_AVGPOOL);
                o.n_in = 1; o.in[0] = in; o.k_h = a.h; o.k_w = a.w; o.out_h = 1; o.out_w = 1;
                Sh s; s.c = a.c; s.h = 1; s.w = 1;
                return emit(o, s);
            }
            case LayerKind::Padding: {
                MsnhB200Op o = blank(MSNH_OP_PAD);
                o.n_in = 1; o.in[0] = in; o.pad_top = d.top; o.pad_down = d.down; o.pad_left = d.left; o.pad_right = d.right; o.const_val = d.paddingVal;
                Sh s; s.c = a.c; s.h = a.h + d.top + d.down; s.w = a.w + d.left + d.right;
                return emit(o, s);
            }
            case LayerKind::UpSample: {
                MsnhB200Op o = blank(MSNH_OP_UPSAMPLE);
                o.n_in = 1; o.in[0] = in; o.stride_h = d.strideY; o.stride_w = d.strideX; o.scale = 1.f;
                Sh s; s.c = a.c; s.h = a.h * d.strideY; s.w = a.w * d.strideX;
                if (d.upsampleType == "bilinear") {                 // src/layers/MsnhUpSampleLayer.cpp:19-23
                    s.w = static_cast<int>(a.w * d.scaleX); s.h = static_cast<int>(a.h * d.scaleY);
                    if (s.h < 1 || s.w < 1) MSNH_THROW("w*x and outw*outx must > 1 (line " + std::to_string(d.line) + ")");
                    if (d.alignCorners && (s.h < 2 || s.w < 2)) MSNH_THROW("[upsample] alignCorners needs an output plane of at least 2x2 (line " + std::to_string(d.line) + ")");
                    o.upsample_mode = MSNH_UPSAMPLE_BILINEAR; o.align_corners = d.alignCorners ? 1 : 0; o.out_h = s.h; o.out_w = s.w;
                }
                return emit(o, s);
            }
            case LayerKind::DeConv: {
                if (d.groups > 1) MSNH_THROW("[deconv] groups > 1 is not supported by this backend (line " + std::to_string(d.line) + ")");
                MsnhB200Op o = blank(MSNH_OP_DECONV);
                o.n_in = 1; o.in[0] = in; o.filters = d.filters;
                o.k_h = d.kSizeY; o.k_w = d.kSizeX; o.stride_h = d.strideY; o.stride_w = d.strideX; o.pad_h = d.paddingY; o.pad_w = d.paddingX;
                o.has_bias = d.useBias ? 1 : 0;
                setAct(o, d);
                Sh s; s.c = d.filters;
                s.h = (a.h - 1) * o.stride_h - 2 * o.pad_h + o.k_h;      // src/layers/MsnhDeConvolutionalLayer.cpp:229-237
                s.w = (a.w - 1) * o.stride_w - 2 * o.pad_w + o.k_w;
                if (d.filters < 1 || s.h < 1 || s.w < 1) MSNH_THROW("[deconv] empty output (line " + std::to_string(d.line) + ")");
                const int id = emit(o, s);
                weights.push_back({id, MSNH_W_WEIGHTS, static_cast<size_t>(a.c) * d.filters * o.k_h * o.k_w, a.c});
                if (d.useBias) weights.push_back({id, MSNH_W_BIAS, static_cast<size_t>(d.filters), 0});
                return id;
            }
            case LayerKind::Clip: {
                MsnhB200Op o = blank(MSNH_OP_CLIP);
                o.n_in = 1; o.in[0] = in; o.const_val = d.clipMin; o.scale = d.clipMax;
                return emit(o, a);
            }
            case LayerKind::Permute: {
                // src/layers/MsnhPermuteLayer.cpp:15-26 (its range check only fires when all three are out of range; a
                // value outside 0..2 would index nothing there, so it is refused here)
                for (int k = 0; k < 3; ++k) if (d.dim[k] < 0 || d.dim[k] > 2) MSNH_THROW("dim value must be 0/1/2 --> c/h/w (line " + std::to_string(d.line) + ")");
                if (d.dim[0] == d.dim[1] || d.dim[1] == d.dim[2] || d.dim[2] == d.dim[0]) MSNH_THROW("dims can't equal (line " + std::to_string(d.line) + ")");
                MsnhB200Op o = blank(MSNH_OP_REMAP);
                o.n_in = 1; o.in[0] = in; o.remap_kind = MSNH_REMAP_PERMUTE;
                const int dims[3] = {a.c, a.h, a.w};
                for (int k = 0; k < 3; ++k) o.remap_dims[k] = d.dim[k];
                Sh s; s.c = dims[d.dim[0]]; s.h = dims[d.dim[1]]; s.w = dims[d.dim[2]];
                return emit(o, s);
            }
            case LayerKind::PixShuffle: {
                if (d.factor <= 0) MSNH_THROW("factor must > 0 (line " + std::to_string(d.line) + ")");
                if (a.c % (d.factor * d.factor)) MSNH_THROW("channel is not divisible by factor^2 (line " + std::to_string(d.line) + ")");
                MsnhB200Op o = blank(MSNH_OP_REMAP);
                o.n_in = 1; o.in[0] = in; o.remap_kind = MSNH_REMAP_PIXSHF; o.remap_dims[0] = d.factor;
                Sh s; s.c = a.c / (d.factor * d.factor); s.h = a.h * d.factor; s.w = a.w * d.factor;
                return emit(o, s);
            }
            case LayerKind::View: {
                // dim0 / dim1 / dim2 land in ViewLayer's outWidth / outHeight / outChannel (src/net/MsnhNetBuilder.cpp:478-482)
                Sh s; s.w = d.dim[0]; s.h = d.dim[1]; s.c = d.dim[2];
                if (s.w < 1 || s.h < 1 || s.c < 1 || static_cast<long long>(s.w) * s.h * s.c != static_cast<long long>(a.w) * a.h * a.c)
                    MSNH_THROW("view op params error (line " + std::to_string(d.line) + ")");
                MsnhB200Op o = blank(MSNH_OP_REMAP);
                o.n_in = 1; o.in[0] = in; o.remap_kind = MSNH_REMAP_VIEW; o.out_c = s.c; o.out_h = s.h; o.out_w = s.w;
                return emit(o, s);
            }
            case LayerKind::Reduction: {
                MsnhB200Op o = blank(MSNH_OP_REDUCE);
                o.n_in = 1; o.in[0] = in; o.binary_kind = d.axis; o.binary_const = d.reduceMean ? 1 : 0;
                Sh s = a;
                if (d.axis == -1) { s.c = 1; s.h = 1; s.w = 1; } else if (d.axis == 0) s.c = 1; else if (d.axis == 1) s.h = 1; else s.w = 1;
                return emit(o, s);
            }
            case LayerKind::Slice: {
                MsnhB200Op o = blank(MSNH_OP_SLICE);
                o.n_in = 1; o.in[0] = in;
                const int dims[3] = {a.c, a.h, a.w};
                int out[3];
                for (int k = 0; k < 3; ++k) {
                    if (d.step[k] < 1 || d.start[k] < 0 || d.start[k] >= dims[k]) MSNH_THROW("[slice] start/step out of range (line " + std::to_string(d.line) + ")");
                    o.slice_start[k] = d.start[k]; o.slice_step[k] = d.step[k];
                    out[k] = (dims[k] - d.start[k] + d.step[k] - 1) / d.step[k];
                }
                Sh s; s.c = out[0]; s.h = out[1]; s.w = out[2];
                return emit(o, s);
            }
            case LayerKind::SoftMax: {
                MsnhB200Op o = blank(MSNH_OP_SOFTMAX);
                o.n_in = 1; o.in[0] = in; o.softmax_groups = d.softmaxGroups; o.softmax_temperature = d.temperature;
                return emit(o, a);
            }
            case LayerKind::Empty: {
                MsnhB200Op o = blank(MSNH_OP_IDENTITY);
                o.n_in = 1; o.in[0] = in;
                return emit(o, a);
            }
            default: MSNH_THROW("layer kind not allowed here (line " + std::to_string(d.line) + ")");
        }
    }

    int chain(const std::vector<LayerDesc> &seq, int in, const Sh &netIn) {
        int cur = in;
        for (const LayerDesc &d : seq) cur = simple(d, cur, netIn);
        return cur;
    }

    int add(const std::vector<int> &ins, const LayerDesc &blockAct, const Sh &netIn) {
        const Sh a = shapeOf(ins[0], netIn);
        for (int i : ins) { const Sh s = shapeOf(i, netIn); if (s.c != a.c || s.h != a.h || s.w != a.w) MSNH_THROW("branches to be added differ in shape (line " + std::to_string(blockAct.line) + ")"); }
        if (ins.size() > MSNH_B200_MAX_IN) MSNH_THROW("too many inputs to one add");
        MsnhB200Op o = blank(MSNH_OP_ADD);
        o.n_in = static_cast<int>(ins.size());
        for (size_t k = 0; k < ins.size(); ++k) o.in[k] = ins[k];
        setAct(o, blockAct);
        return emit(o, a);
    }
    int concat(const std::vector<int> &ins, int groups, int groupId, const LayerDesc &d, const Sh &netIn) {
        if (ins.size() > MSNH_B200_MAX_IN) MSNH_THROW("too many inputs to one route");
        const Sh a = shapeOf(ins[0], netIn);
        MsnhB200Op o = blank(MSNH_OP_CONCAT);
        o.n_in = static_cast<int>(ins.size()); o.route_groups = groups; o.route_group_id = groupId;
        Sh s; s.h = a.h; s.w = a.w; s.c = 0;
        for (size_t k = 0; k < ins.size(); ++k) {
            o.in[k] = ins[k];
            const Sh t = shapeOf(ins[k], netIn);
            if (t.h != a.h || t.w != a.w) MSNH_THROW("[route] inputs differ in plane size (line " + std::to_string(d.line) + ")");
            if (t.c % groups) MSNH_THROW("[route] groups must divide channels (line " + std::to_string(d.line) + ")");
            s.c += t.c / groups;
        }
        return emit(o, s);
    }
};

int varopKind(const std::string &t, bool &isConst, int line) {
    static const struct { const char *n; int k; bool c; } table[] = {
        {"add", MSNH_BIN_ADD, false}, {"sub", MSNH_BIN_SUB, false}, {"subInv", MSNH_BIN_SUB_INV, false}, {"mul", MSNH_BIN_MUL, false},
        {"div", MSNH_BIN_DIV, false}, {"divInv", MSNH_BIN_DIV_INV, false}, {"addConst", MSNH_BIN_ADD, true}, {"subConst", MSNH_BIN_SUB, true},
        {"subConstInv", MSNH_BIN_SUB_INV, true}, {"mulConst", MSNH_BIN_MUL, true}, {"divConst", MSNH_BIN_DIV, true}, {"divConstInv", MSNH_BIN_DIV_INV, true},
        // one-operand types: the previous layer through a library function (pow: to the power constVal)
        {"abs", MSNH_UN_ABS, true}, {"acos", MSNH_UN_ACOS, true}, {"asin", MSNH_UN_ASIN, true}, {"atan", MSNH_UN_ATAN, true}, {"cos", MSNH_UN_COS, true},
        {"cosh", MSNH_UN_COSH, true}, {"sin", MSNH_UN_SIN, true}, {"sinh", MSNH_UN_SINH, true}, {"tan", MSNH_UN_TAN, true}, {"tanh", MSNH_UN_TANH, true},
        {"exp", MSNH_UN_EXP, true}, {"pow", MSNH_UN_POW, true}, {"log", MSNH_UN_LOG, true}, {"log10", MSNH_UN_LOG10, true}, {"sqrt", MSNH_UN_SQRT, true}};
    for (auto &e : table) if (t == e.n) { isConst = e.c; return e.k; }
    MSNH_THROW("[varop] type '" + t + "' is not supported by this backend (line " + std::to_string(line) + ")");
}

}  // namespace

void NetBuilder::lower(const NetDesc &net) {
    Lowering L;
    Sh netIn; netIn.c = net.channels; netIn.h = net.height; netIn.w = net.width;
    _layerOp.clear(); _layerNames.clear();
    std::ostringstream detail;
    int prev = MSNH_B200_INPUT;
    auto layerRef = [&](int idx, const LayerDesc &d) {
        if (idx < 0 || idx >= static_cast<int>(_layerOp.size()) || _layerOp[idx] < 0)
            MSNH_THROW("layer index " + std::to_string(idx) + " does not name an earlier layer (line " + std::to_string(d.line) + ")");
        return _layerOp[idx];
    };
    for (size_t li = 0; li < net.layers.size(); ++li) {
        const LayerDesc &d = net.layers[li];
        int out = -1;
        const char *name = "";
        if (_collectOp >= 0) MSNH_THROW("yoloout must be the last layer");
        switch (d.kind) {
            case LayerKind::Route: {
                name = "Route";
                std::vector<int> ins;
                for (int idx : d.layers) ins.push_back(layerRef(idx, d));
                if (d.addModel == 1) out = L.add(ins, d, netIn);
                else { out = L.concat(ins, d.routeGroups, d.routeGroupsId, d, netIn); out = L.activation(out, L.shapes[out], d); }
                break;
            }
            case LayerKind::VarOp: {
                name = "VarOp";
                bool isConst = false;
                const int kind = varopKind(d.varOpType, isConst, d.line);
                // operands as in VariableOpLayer::forward (src/layers/MsnhVariableOpLayer.cpp:80-150):
                // two indices: A = layers[0], B = layers[1]; one index: A = previous layer, B = layers[0];
                // constant forms: A = previous layer
                int a = prev, b = -1;
                if (!isConst) {
                    if (d.layers.size() == 2) { a = layerRef(d.layers[0], d); b = layerRef(d.layers[1], d); }
                    else if (d.layers.size() == 1) b = layerRef(d.layers[0], d);
                    else MSNH_THROW("[varop] needs one or two layers (line " + std::to_string(d.line) + ")");
                }
                if (!isConst && kind == MSNH_BIN_ADD) {
                    LayerDesc none; none.line = d.line;
                    out = L.add({a, b}, none, netIn);
                } else {
                    MsnhB200Op o = Lowering::blank(MSNH_OP_BINARY);
                    o.binary_kind = kind; o.binary_const = isConst ? 1 : 0; o.const_val = d.constVal;
                    o.n_in = isConst ? 1 : 2; o.in[0] = a;
                    if (!isConst) o.in[1] = b;
                    out = L.emit(o, L.shapeOf(a, netIn));
                }
                break;
            }
            case LayerKind::ResBlock: {
                name = "ResBlock";
                const int f = L.chain(d.chain, prev, netIn);
                out = L.add({prev, f}, d, netIn);
                break;
            }
            case LayerKind::Res2Block: {
                name = "Res2Block";
                const int base = L.chain(d.branches[0], prev, netIn);
                const int br = L.chain(d.branches[1], prev, netIn);
                out = L.add({base, br}, d, netIn);
                break;
            }
            case LayerKind::AddBlock: case LayerKind::ConcatBlock: {
                name = d.kind == LayerKind::AddBlock ? "AddBlock" : "ConcatBlock";
                std::vector<int> outs;
                for (const auto &br : d.branches) {
                    // an `empty:` branch is the block input itself
                    bool allEmpty = true;
                    for (const LayerDesc &c : br) if (c.kind != LayerKind::Empty) allEmpty = false;
                    outs.push_back(allEmpty ? prev : L.chain(br, prev, netIn));
                }
                if (d.kind == LayerKind::AddBlock) {
                    if (outs.size() == 1) out = L.activation(outs[0], L.shapeOf(outs[0], netIn), d);
                    else out = L.add(outs, d, netIn);
                } else {
                    out = L.concat(outs, 1, 0, d, netIn);
                    out = L.activation(out, L.shapes[out], d);
                }
                if (out == prev) {   // single empty branch: still its own layer
                    MsnhB200Op o = Lowering::blank(MSNH_OP_IDENTITY); o.n_in = 1; o.in[0] = prev; out = L.emit(o, L.shapeOf(prev, netIn));
                }
                break;
            }
            case LayerKind::Yolo: {
                name = "Yolo";
                const Sh a = L.shapeOf(prev, netIn);
                // src/layers/MsnhYoloLayer.cpp:36-39
                if (a.c != 3 * (d.classNum + 5)) MSNH_THROW("class num error! (line " + std::to_string(d.line) + ")");
                MsnhB200Op o = Lowering::blank(MSNH_OP_YOLO);
                o.n_in = 1; o.in[0] = prev; o.yolo_classes = d.classNum;
                o.yolo_type = d.yoloType == "yolov5" ? MSNH_YOLO_V5 : (d.yoloType == "yolov4" ? MSNH_YOLO_V4 : MSNH_YOLO_V3);
                if (d.yoloType != "yolov3" && d.yoloType != "yolov4" && d.yoloType != "yolov5") MSNH_THROW("[yolo] yoloType '" + d.yoloType + "' is not supported by this backend");
                for (int k = 0; k < 6; ++k) o.yolo_anchors[k] = d.anchors[k];
                // not marked as a plan output: a head that only feeds the candidate collection is decoded inside it
                out = L.emit(o, a);
                break;
            }
            case LayerKind::YoloOut: {
                name = "YoloOut";
                MsnhB200Op o = Lowering::blank(MSNH_OP_YOLO_COLLECT);
                if (d.layers.empty() || d.layers.size() > MSNH_B200_MAX_IN) MSNH_THROW("[yoloout] needs 1..8 layers");
                int cells = 0;
                for (size_t k = 0; k < d.layers.size(); ++k) {
                    const int src = layerRef(d.layers[k], d);
                    if (L.ops[src].kind != MSNH_OP_YOLO) MSNH_THROW("[yoloout] layer " + std::to_string(d.layers[k]) + " is not a yolo layer");
                    o.in[k] = src; cells += 3 * L.shapes[src].h * L.shapes[src].w;
                }
                o.n_in = static_cast<int>(d.layers.size()); o.const_val = d.confThresh; o.is_output = 1;
                Sh s; s.c = 8; s.h = 1; s.w = cells;
                _collectOp = L.emit(o, s);
                _confThresh = d.confThresh; _nmsThresh = d.nmsThresh; _useSoftNms = d.useSoftNms != 0;
                _maxRows = cells;
                out = -1;
                break;
            }
            default: {
                static const char *names[] = {"Config", "Conv", "BatchNorm", "Activate", "MaxPool", "LocalAvgPool", "GlobalAvgPool", "Padding", "UpSample",
                                              "Route", "VarOp", "Slice", "Connected", "SoftMax", "", "", "", "", "", "", "Empty",
                                              "DeConv", "Clip", "Permute", "PixelShuffle", "View", "Reduction"};
                name = names[static_cast<int>(d.kind)];
                out = L.simple(d, prev, netIn);
                break;
            }
        }
        _layerOp.push_back(out);
        _layerNames.push_back(name);
        if (out >= 0) {
            const Sh s = L.shapes[out];
            detail << li << " " << name << " -> " << s.c << " x " << s.h << " x " << s.w << "\n";
            prev = out;
        } else detail << li << " " << name << "\n";
    }
    _detail = detail.str();
    _lastOp = prev;
    if (_lastOp >= 0) {
        if (_collectOp < 0) L.ops[_lastOp].is_output = 1;   // detection nets read the collected candidates instead
        const Sh s = L.shapes[_lastOp];
        _lastC = s.c; _lastH = s.h; _lastW = s.w; _lastNum = static_cast<size_t>(s.c) * s.h * s.w;
    }
    if (_saveLayerOutput) _planFlags |= MSNH_PLAN_KEEP_ALL;

    _batch = _batchOverride > 0 ? _batchOverride : net.batch;
    _inC = net.channels; _inH = net.height; _inW = net.width;
    _weightSlots.clear(); _totalWeights = 0;
    for (auto &w : L.weights) { _weightSlots.push_back({w.op, w.slot, w.count, w.rows}); _totalWeights += w.count; }
    _ops = L.ops;

    if (isPreviewMode) return;   // shapes only, no device work (include/Msnhnet/layers/MsnhBaseLayer.h:25)
    if (!_ctx) {
        int rc = msnh_b200_ctx_create(_device, &_ctx);
        if (rc != MSNH_B200_OK) MSNH_THROW("no usable B200 device " + std::to_string(_device) + " (status " + std::to_string(rc) + "); this backend has no CPU fallback");
    }
    checkK(msnh_b200_plan_create(_ctx, L.ops.data(), static_cast<int>(L.ops.size()), _inC, _inH, _inW, _batch,
                                 useFp16 ? MSNH_B200_F16 : MSNH_B200_F32, _planFlags, &_plan), "plan_create");
    for (auto &w : _weightSlots) {
        size_t n = 0;
        checkK(msnh_b200_plan_weight_count(_plan, w.op, w.slot, &n), "plan_weight_count");
        if (n != w.count) MSNH_THROW("internal: weight count mismatch for op " + std::to_string(w.op));
    }
}

void NetBuilder::buildNetFromMsnhNetText(const std::string &text) {
    clearLayers();
    lower(parseMsnhNet(text));
}
void NetBuilder::buildNetFromMsnhNet(const std::string &path) {
    clearLayers();
    lower(readMsnhNet(path));
}

void NetBuilder::loadWeightsFromMemory(const float *data, size_t count) {
    if (_layerOp.empty()) MSNH_THROW("build the net before loading weights");
    // exact-length check of the reference (src/net/MsnhNetBuilder.cpp:657-661)
    if (count != _totalWeights) MSNH_THROW("weights load err. needed : " + std::to_string(_totalWeights) + " given : " + std::to_string(count));
    if (isPreviewMode) return;
    if (_weightsLoaded) MSNH_THROW("weights already loaded; rebuild the net to load another blob");
    const bool trace = std::getenv("MSNH_B200_BUILD_TRACE") != nullptr;     // stage times on stderr
    auto t0 = std::chrono::steady_clock::now();
    auto stage = [&](const char *what) {
        if (!trace) return;
        const auto now = std::chrono::steady_clock::now();
        std::fprintf(stderr, "[msnh_b200 build] %-28s %8.2f ms\n", what, std::chrono::duration<double, std::milli>(now - t0).count());
        t0 = now;
    };
    size_t off = 0;
    for (auto &w : _weightSlots) {
        checkK(msnh_b200_plan_set_weights(_plan, w.op, w.slot, data + off, w.count), "plan_set_weights");
        off += w.count;
    }
    stage("hand slices to the plan");
    checkK(msnh_b200_plan_finalize(_plan), "plan_finalize");
    stage("plan_finalize (total)");
    _weightsLoaded = true;
}
void NetBuilder::loadWeightsFromMsnhBin(const std::string &path) {
    _usedPack = false;
    if (_packCache && !isPreviewMode && !_layerOp.empty() && !_weightsLoaded) {
        struct stat st;
        if (::stat(path.c_str(), &st) != 0) MSNH_THROW("can not open " + path);
        if (static_cast<size_t>(st.st_size) != _totalWeights * sizeof(float))      // the reference's exact-length check, on the file size
            MSNH_THROW("weights load err. needed : " + std::to_string(_totalWeights) + " given : " + std::to_string(st.st_size / sizeof(float)));
        const uint64_t tag = static_cast<uint64_t>(st.st_size) * 1000003ull ^ (static_cast<uint64_t>(st.st_mtim.tv_sec) * 1000000000ull + static_cast<uint64_t>(st.st_mtim.tv_nsec));
        int usable = 0;
        checkK(msnh_b200_plan_use_pack(_plan, (path + ".b200pack").c_str(), tag, &usable), "plan_use_pack");
        if (usable) {
            const auto t0 = std::chrono::steady_clock::now();
            checkK(msnh_b200_plan_finalize(_plan), "plan_finalize");
            if (std::getenv("MSNH_B200_BUILD_TRACE"))
                std::fprintf(stderr, "[msnh_b200 build] %-28s %8.2f ms\n", "plan_finalize from pack", std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count());
            _weightsLoaded = true; _usedPack = true;
            return;
        }
    }
    const auto t0 = std::chrono::steady_clock::now();
    std::vector<float> blob = readMsnhBin(path);
    if (std::getenv("MSNH_B200_BUILD_TRACE"))
        std::fprintf(stderr, "[msnh_b200 build] %-28s %8.2f ms\n", "read .msnhbin", std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count());
    loadWeightsFromMemory(blob.data(), blob.size());
}

// ------------------------------------------------------------------------------------------------
// running
// ------------------------------------------------------------------------------------------------
std::vector<float> NetBuilder::runClassify(std::vector<float>) { MSNH_THROW("Gpu mode , can not run with cpu: the CPU path is not part of this backend"); }
std::vector<std::vector<YoloBox>> NetBuilder::runYolo(std::vector<float>) { MSNH_THROW("Gpu mode , can not run with cpu: the CPU path is not part of this backend"); }

void NetBuilder::forwardGPU(const float *images, int nImages) {
    if (isPreviewMode) MSNH_THROW("Can not infer in preview mode !");
    if (!_plan || !_weightsLoaded) MSNH_THROW("net not built or weights not loaded");
    if (nImages < 1 || nImages > _batch) MSNH_THROW("image count " + std::to_string(nImages) + " outside 1.." + std::to_string(_batch));
    checkK(msnh_b200_plan_run(_plan, images, nImages), "plan_run");
}
void NetBuilder::forwardGPUDeviceResident(int nImages, bool sync) {
    if (!_plan || !_weightsLoaded) MSNH_THROW("net not built or weights not loaded");
    checkK(msnh_b200_plan_run_device(_plan, nullptr, nImages, sync ? 1 : 0), "plan_run_device");
}

std::vector<float> NetBuilder::runClassifyGPUBatch(const float *images, int nImages) {
    auto t0 = std::chrono::steady_clock::now();
    if (_lastOp < 0) MSNH_THROW("net has no output layer");
    if (_collectOp >= 0) MSNH_THROW("detection net: its result is read with runYoloGPU");
    forwardGPU(images, nImages);
    std::vector<float> out(static_cast<size_t>(nImages) * _lastNum);
    checkK(msnh_b200_plan_read_output(_plan, _lastOp, out.data(), out.size()), "plan_read_output");
    _gpuInferenceTime = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return out;
}

std::vector<float> NetBuilder::runClassifyGPU(std::vector<float> img) {
    // size check of the reference (src/net/MsnhNetBuilder.cpp:837-841)
    const size_t need = static_cast<size_t>(_inC) * _inH * _inW;
    if (img.size() != need) MSNH_THROW("input image size err. Needed :" + std::to_string(need) + " given :" + std::to_string(img.size()));
    return runClassifyGPUBatch(img.data(), 1);
}

std::vector<float> NetBuilder::getCandidates(int nImages, std::vector<int> &counts) {
    if (_collectOp < 0) MSNH_THROW("not a yolo net");
    _candRows.resize(static_cast<size_t>(nImages) * _maxRows * 8);
    counts.assign(nImages, 0);
    checkK(msnh_b200_plan_read_candidates(_plan, _collectOp, nImages, _candRows.data(), _maxRows, counts.data()), "plan_read_candidates");
    return _candRows;
}

std::vector<YoloBox> NetBuilder::boxesFromRows(const float *rows, int count) {
    std::vector<YoloBox> out(static_cast<size_t>(count));
    for (int i = 0; i < count; ++i) {
        const float *r = rows + static_cast<size_t>(i) * 8;
        out[i].xywhBox = Box::XYWHBox(r[0], r[1], r[2], r[3]);
        out[i].conf = r[4]; out[i].bestClsConf = r[5]; out[i].bestClsIdx = static_cast<int>(r[6]);
    }
    return out;
}

std::vector<YoloBox> NetBuilder::postProcess(const float *rows, int count, float nmsThresh, bool useSoftNms) {
    std::vector<YoloBox> tmpBox(static_cast<size_t>(count));
    for (int i = 0; i < count; ++i) {
        const float *r = rows + static_cast<size_t>(i) * 8;
        YoloBox &b = tmpBox[i];
        b.xywhBox = Box::XYWHBox(r[0], r[1], r[2], r[3]);
        b.conf = r[4]; b.bestClsConf = r[5]; b.bestClsIdx = static_cast<int>(r[6]);
    }
    if (count > 0) {
        // score sort exactly as the reference: argsort over conf*bestClsConf, descending, std::sort
        // on the index vector (include/Msnhnet/utils/MsnhExVector.h:58-74)
        std::vector<float> confs(tmpBox.size());
        for (size_t i = 0; i < tmpBox.size(); ++i) confs[i] = tmpBox[i].conf * tmpBox[i].bestClsConf;
        std::vector<int> idx(tmpBox.size());
        for (size_t i = 0; i < idx.size(); ++i) idx[i] = static_cast<int>(i);
        std::sort(idx.begin(), idx.end(), [&confs](int i1, int i2) { return confs[i1] > confs[i2]; });
        std::vector<YoloBox> sorted(tmpBox.size());
        for (size_t i = 0; i < idx.size(); ++i) sorted[i] = tmpBox[static_cast<size_t>(idx[i])];
        tmpBox.swap(sorted);
    }
    return nms(tmpBox, nmsThresh, useSoftNms);
}

// Per-class greedy NMS keyed on objectness, the reference's algorithm and tie rules
// (src/layers/MsnhYoloOutLayer.cpp:381-461): classes in first-seen order of the score-sorted list,
// a class with a single box keeps it, otherwise repeatedly take the highest-conf box (first on
// ties) and drop every remaining box whose IoU with it exceeds the threshold.
std::vector<YoloBox> NetBuilder::nms(const std::vector<YoloBox> &bboxes, const float &nmsThresh, const bool &useSoftNms, const float &sigma) {
    std::vector<YoloBox> best;
    std::vector<int> classes;
    for (const YoloBox &b : bboxes)
        if (std::find(classes.begin(), classes.end(), b.bestClsIdx) == classes.end()) classes.push_back(b.bestClsIdx);
    for (int cls : classes) {
        std::vector<YoloBox> cur;
        for (const YoloBox &b : bboxes) if (b.bestClsIdx == cls) cur.push_back(b);
        if (cur.size() == 1) { best.push_back(cur[0]); continue; }
        while (!cur.empty()) {
            size_t bi = 0; float bc = -FLT_MAX;
            for (size_t j = 0; j < cur.size(); ++j) if (cur[j].conf > bc) { bi = j; bc = cur[j].conf; }
            const YoloBox top = cur[bi];
            best.push_back(top);
            cur.erase(cur.begin() + static_cast<long>(bi));
            std::vector<YoloBox> keep;
            keep.reserve(cur.size());
            for (const YoloBox &b : cur) {
                const float iou = Box::iou(b.xywhBox, top.xywhBox);
                bool drop;
                if (useSoftNms) drop = b.conf * expf(-(1.f * iou * iou / sigma)) <= 0;
                else drop = iou > nmsThresh;
                if (!drop) keep.push_back(b);
            }
            cur.swap(keep);
        }
    }
    return best;
}

std::vector<std::vector<YoloBox>> NetBuilder::runYoloGPUBatch(const float *images, int nImages) {
    auto t0 = std::chrono::steady_clock::now();
    if (_collectOp < 0) MSNH_THROW("not a yolo net");
    forwardGPU(images, nImages);
    std::vector<std::vector<YoloBox>> out = yoloResults(nImages);
    _gpuInferenceTime = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return out;
}

// 8-bit image in, boxes out: the preprocessing of the reference's runYoloList (src/c_api/MsnhnetLib.cpp:754-778,
// CVUtil::getPaddingZeroF32C3) runs on the device, straight into the plan's input buffer.
std::vector<std::vector<YoloBox>> NetBuilder::runYoloGPUImage(const unsigned char *image, int width, int height, bool swapRGB) {
    auto t0 = std::chrono::steady_clock::now();
    if (_collectOp < 0) MSNH_THROW("not a yolo net");
    if (!_plan || !_weightsLoaded) MSNH_THROW("net not built or weights not loaded");
    checkK(msnh_b200_plan_preprocess_u8(_plan, image, width, height, 0, MSNH_PREP_PAD_SQUARE, swapRGB ? 1 : 0, nullptr, nullptr), "plan_preprocess_u8");
    forwardGPUDeviceResident(1, true);
    std::vector<std::vector<YoloBox>> out = yoloResults(1);
    _gpuInferenceTime = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return out;
}

std::vector<float> NetBuilder::runClassifyGPUImage(const unsigned char *image, int width, int height, int prepMode, bool swapRGB,
                                                   const float *mean, const float *std) {
    auto t0 = std::chrono::steady_clock::now();
    if (_lastOp < 0) MSNH_THROW("net has no output layer");
    if (_collectOp >= 0) MSNH_THROW("detection net: its result is read with runYoloGPU");
    if (!_plan || !_weightsLoaded) MSNH_THROW("net not built or weights not loaded");
    checkK(msnh_b200_plan_preprocess_u8(_plan, image, width, height, 0, prepMode, swapRGB ? 1 : 0, mean, std), "plan_preprocess_u8");
    forwardGPUDeviceResident(1, true);
    std::vector<float> out(_lastNum);
    checkK(msnh_b200_plan_read_output(_plan, _lastOp, out.data(), out.size()), "plan_read_output");
    _gpuInferenceTime = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return out;
}

// boxes of the last forward: device or host NMS over the collected candidates
std::vector<std::vector<YoloBox>> NetBuilder::yoloResults(int nImages) {
    std::vector<std::vector<YoloBox>> out(static_cast<size_t>(nImages));
    std::vector<int> kept(static_cast<size_t>(nImages), -1);
    if (_deviceNms) {
        const int cap = 4096;
        std::vector<float> boxes(static_cast<size_t>(nImages) * cap * 8);
        checkK(msnh_b200_plan_nms(_plan, _collectOp, nImages, _nmsThresh, _useSoftNms ? 1 : 0, 0.3f, boxes.data(), cap, kept.data()), "plan_nms");
        for (int i = 0; i < nImages; ++i)
            if (kept[i] >= 0) out[i] = boxesFromRows(boxes.data() + static_cast<size_t>(i) * cap * 8, kept[i]);
    }
    bool hostNeeded = false;
    for (int k : kept) hostNeeded = hostNeeded || k < 0;
    if (hostNeeded) {
        std::vector<int> counts;
        getCandidates(nImages, counts);
        for (int i = 0; i < nImages; ++i)
            if (kept[i] < 0) out[i] = postProcess(_candRows.data() + static_cast<size_t>(i) * _maxRows * 8, counts[i], _nmsThresh, _useSoftNms);
    }
    return out;
}

// The streaming loop of the yolo calls: push(b) queues batch b, again(i) runs image i alone through the path that keeps
// every candidate.
template <typename Push, typename Again>
std::vector<std::vector<YoloBox>> NetBuilder::yoloStream(int nBatches, Push &&push, Again &&again) {
    auto t0 = std::chrono::steady_clock::now();
    const int cap = std::min(_maxRows, 4096);
    std::vector<float> rows(static_cast<size_t>(_batch) * cap * 8);
    std::vector<int> counts(static_cast<size_t>(_batch));
    std::vector<std::vector<YoloBox>> out;
    out.reserve(static_cast<size_t>(nBatches) * _batch);
    checkK(msnh_b200_plan_stream_nms(_plan, _deviceNms ? 1 : 0, _nmsThresh, _useSoftNms ? 1 : 0, 0.3f), "plan_stream_nms");
    std::vector<size_t> flagged;      // images the streaming slots could not deliver whole (see plan_stream_pop)
    auto pop = [&]() {
        int n = 0;
        checkK(msnh_b200_plan_stream_pop(_plan, rows.data(), rows.size(), cap, counts.data(), &n), "plan_stream_pop");
        for (int i = 0; i < n; ++i) {
            if (counts[i] < 0) { flagged.push_back(out.size()); out.emplace_back(); continue; }
            out.push_back(_deviceNms ? boxesFromRows(rows.data() + static_cast<size_t>(i) * cap * 8, counts[i])
                                     : postProcess(rows.data() + static_cast<size_t>(i) * cap * 8, counts[i], _nmsThresh, _useSoftNms));
        }
    };
    try {
        push(0);
        for (int b = 1; b < nBatches; ++b) {
            push(b);
            pop();      // batch b-1: waits for its result only; batch b is already queued behind it
        }
        pop();
    } catch (...) {
        msnh_b200_plan_stream_reset(_plan);      // nothing stays in flight behind an error
        throw;
    }
    // images with more candidates than a slot holds (or than the device NMS takes): one synchronous forward each,
    // then the path that keeps every candidate
    for (size_t idx : flagged) out[idx] = again(idx);
    _gpuInferenceTime = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return out;
}

std::vector<std::vector<YoloBox>> NetBuilder::runYoloGPUStream(const float *images, int nBatches) {
    if (_collectOp < 0) MSNH_THROW("not a yolo net");
    if (!_plan || !_weightsLoaded) MSNH_THROW("net not built or weights not loaded");
    if (!images || nBatches < 1) MSNH_THROW("runYoloGPUStream: no images");
    const size_t perBatch = static_cast<size_t>(_batch) * _inC * _inH * _inW, perImage = perBatch / static_cast<size_t>(_batch);
    return yoloStream(nBatches,
                      [&](int b) { checkK(msnh_b200_plan_stream_push(_plan, _collectOp, images + perBatch * b, _batch), "plan_stream_push"); },
                      [&](size_t i) { forwardGPU(images + perImage * i, 1); return yoloResults(1)[0]; });
}

std::vector<std::vector<YoloBox>> NetBuilder::runYoloGPUStreamU8(const unsigned char *images, int width, int height, bool swapRGB, int nBatches) {
    if (_collectOp < 0) MSNH_THROW("not a yolo net");
    if (!_plan || !_weightsLoaded) MSNH_THROW("net not built or weights not loaded");
    if (!images || nBatches < 1 || width < 1 || height < 1) MSNH_THROW("runYoloGPUStreamU8: no images");
    const size_t perImage = static_cast<size_t>(width) * height * 3, perBatch = perImage * static_cast<size_t>(_batch);
    return yoloStream(nBatches,
                      [&](int b) { checkK(msnh_b200_plan_stream_push_u8(_plan, _collectOp, images + perBatch * b, width, height, _batch, MSNH_PREP_PAD_SQUARE, swapRGB ? 1 : 0, nullptr, nullptr), "plan_stream_push_u8"); },
                      [&](size_t i) { return runYoloGPUImage(images + perImage * i, width, height, swapRGB)[0]; });
}

std::vector<float> NetBuilder::runClassifyGPUStream(const float *images, int nBatches) {
    if (_lastOp < 0 || _collectOp >= 0) MSNH_THROW("not a classification net");
    if (nBatches < 1) MSNH_THROW("runClassifyGPUStream: no images");
    std::vector<float> out(static_cast<size_t>(_batch) * _lastNum * nBatches);
    runClassifyGPUStreamInto(images, nBatches, out.data(), out.size());
    return out;
}

// The same, results written straight into the caller's buffer (segmentation-sized outputs: no second copy).
void NetBuilder::runClassifyGPUStreamInto(const float *images, int nBatches, float *out, size_t capacity) {
    if (!images) MSNH_THROW("runClassifyGPUStream: no images");
    const size_t perBatch = static_cast<size_t>(_batch) * _inC * _inH * _inW;
    classifyStream(nBatches, out, capacity, [&](int b) { checkK(msnh_b200_plan_stream_push(_plan, _lastOp, images + perBatch * b, _batch), "plan_stream_push"); });
}

void NetBuilder::runClassifyGPUStreamU8Into(const unsigned char *images, int width, int height, int prepMode, bool swapRGB,
                                            const float *mean, const float *std, int nBatches, float *out, size_t capacity) {
    if (!images || width < 1 || height < 1) MSNH_THROW("runClassifyGPUStreamU8: no images");
    const size_t perBatch = static_cast<size_t>(width) * height * 3 * static_cast<size_t>(_batch);
    classifyStream(nBatches, out, capacity, [&](int b) {
        checkK(msnh_b200_plan_stream_push_u8(_plan, _lastOp, images + perBatch * b, width, height, _batch, prepMode, swapRGB ? 1 : 0, mean, std), "plan_stream_push_u8");
    });
}

template <typename Push>
void NetBuilder::classifyStream(int nBatches, float *out, size_t capacity, Push &&push) {
    auto t0 = std::chrono::steady_clock::now();
    if (_lastOp < 0 || _collectOp >= 0) MSNH_THROW("not a classification net");
    if (!_plan || !_weightsLoaded) MSNH_THROW("net not built or weights not loaded");
    if (!out || nBatches < 1) MSNH_THROW("runClassifyGPUStream: no images");
    const size_t outPer = static_cast<size_t>(_batch) * _lastNum;
    if (outPer * nBatches > capacity) MSNH_THROW("output buffer too small: need " + std::to_string(outPer * nBatches));
    int n = 0;
    try {
        push(0);
        for (int b = 1; b < nBatches; ++b) {
            push(b);
            checkK(msnh_b200_plan_stream_pop(_plan, out + outPer * (b - 1), outPer, 0, nullptr, &n), "plan_stream_pop");
        }
        checkK(msnh_b200_plan_stream_pop(_plan, out + outPer * (nBatches - 1), outPer, 0, nullptr, &n), "plan_stream_pop");
    } catch (...) {
        msnh_b200_plan_stream_reset(_plan);      // nothing stays in flight behind an error
        throw;
    }
    _gpuInferenceTime = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
}

std::vector<std::vector<YoloBox>> NetBuilder::runYoloGPU(std::vector<float> img) {
    const size_t need = static_cast<size_t>(_inC) * _inH * _inW;
    if (img.size() != need) MSNH_THROW("input image size err. Needed :" + std::to_string(need) + " given :" + std::to_string(img.size()));
    return runYoloGPUBatch(img.data(), 1);
}

std::vector<float> NetBuilder::getLayerOutput(int layer, int nImages, int *c, int *h, int *w) {
    if (layer < 0 || layer >= static_cast<int>(_layerOp.size()) || _layerOp[layer] < 0) MSNH_THROW("layer " + std::to_string(layer) + " has no tensor output");
    int cc = 0, hh = 0, ww = 0;
    checkK(msnh_b200_plan_op_shape(_plan, _layerOp[layer], &cc, &hh, &ww), "plan_op_shape");
    std::vector<float> out(static_cast<size_t>(nImages) * cc * hh * ww);
    checkK(msnh_b200_plan_read_output(_plan, _layerOp[layer], out.data(), out.size()), "plan_read_output");
    if (c) *c = cc;
    if (h) *h = hh;
    if (w) *w = ww;
    return out;
}

Point2I NetBuilder::getInputSize() {
    if (_layerOp.empty()) MSNH_THROW("net not built");
    return Point2I(_inW, _inH);
}
int NetBuilder::getInputChannel() {
    if (_layerOp.empty()) MSNH_THROW("net not built");
    return _inC;
}
float NetBuilder::getInferenceTime() { return 0.f; }
float NetBuilder::getGpuInferenceTime() const { return _gpuInferenceTime; }
float NetBuilder::getGpuKernelTime() const {
    float ms = 0.f;
    if (_plan) msnh_b200_plan_last_ms(_plan, &ms);
    return ms;
}
std::string NetBuilder::getLayerDetail() { return _detail; }

// The op list handed to msnh_b200_plan_create, one line per op with every field of MsnhB200Op in declaration order.
std::string NetBuilder::getOpList() const {
    std::ostringstream out;
    out << std::setprecision(9);
    for (const MsnhB200Op &o : _ops) {
        out << "op " << o.kind << " " << o.n_in;
        for (int k = 0; k < MSNH_B200_MAX_IN; ++k) out << " " << (k < o.n_in ? o.in[k] : 0);
        out << " " << o.filters << " " << o.k_h << " " << o.k_w << " " << o.stride_h << " " << o.stride_w << " " << o.pad_h << " " << o.pad_w << " " << o.dil_h << " "
            << o.dil_w << " " << o.groups << " " << o.out_h << " " << o.out_w << " " << o.pad_top << " " << o.pad_down << " " << o.pad_left << " " << o.pad_right;
        for (int k = 0; k < 3; ++k) out << " " << o.slice_start[k] << " " << o.slice_step[k];
        out << " " << o.route_groups << " " << o.route_group_id << " " << o.has_bn << " " << o.has_bias << " " << o.bn_eps << " " << o.act << " " << o.act_param << " "
            << o.scale << " " << o.const_val << " " << o.binary_kind << " " << o.binary_const << " " << o.softmax_groups << " " << o.softmax_temperature << " "
            << o.yolo_type << " " << o.yolo_classes;
        for (int k = 0; k < 6; ++k) out << " " << o.yolo_anchors[k];
        out << " " << o.is_output << " " << o.upsample_mode << " " << o.align_corners << " " << o.remap_kind << " " << o.remap_dims[0] << " " << o.remap_dims[1] << " "
            << o.remap_dims[2] << " " << o.out_c << "\n";
    }
    return out.str();
}

std::string NetBuilder::getWeightLayout() const {
    std::ostringstream out;
    for (const WeightSlot &w : _weightSlots) out << w.op << " " << w.slot << " " << w.count << " " << w.rows << "\n";
    return out.str();
}

// Per-launch device times (the reference's per-layer table is CPU-only; its GPU timers are
// stubbed out, src/layers/MsnhBaseLayer.cpp:300-319).
std::string NetBuilder::getTimeDetail() {
    if (!_plan || !_weightsLoaded) return "";
    int n = 0; size_t arena = 0;
    msnh_b200_plan_stats(_plan, &n, &arena);
    std::vector<float> ms(static_cast<size_t>(n));
    if (msnh_b200_plan_profile(_plan, 3, ms.data(), n) != MSNH_B200_OK) return "";
    std::istringstream desc(msnh_b200_plan_describe(_plan));
    std::ostringstream out;
    float total = 0.f;
    for (float v : ms) total += v;
    std::string line;
    for (int i = 0; i < n && std::getline(desc, line); ++i)
        out << line << " ms=" << ms[i] << " (" << (total > 0 ? 100.f * ms[i] / total : 0.f) << "%)\n";
    out << "total " << total << " ms, arena " << arena << " bytes\n";
    return out.str();
}

}  // namespace Msnhnet
