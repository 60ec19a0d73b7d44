// Test infrastructure, not product code: the seam between the reference's own host classes and the kernel library,
// compiled against the UNMODIFIED reference (oracle/Makefile builds it from the sources where they lie).
//
// lowerLayers() walks real Msnhnet::BaseLayer objects - the vector a Msnhnet::NetBuilder holds after
// buildNetFromMsnhNet (include/Msnhnet/net/MsnhNetwork.h:17, include/Msnhnet/layers/MsnhBaseLayer.h:47-59; block
// layers through their public baseLayers / branchLayers members) - and emits the MsnhB200Op list and the weight-slot
// order of include/msnh_b200.h, i.e. what a maintainer's replacement of the per-layer forwardGPU calls would hand to
// msnh_b200_plan_create / plan_set_weights. tests/test_format_cpu.py checks that this list equals, op for op and slot for
// slot, what the product's own NetBuilder::lower derives from the same topology text.
//
//   seam_adapter <net.msnhnet>    prints "op <all fields>" lines, then "w <op> <slot> <count>" lines
//
// Standard headers first: the access override below must not reach them.
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>
#include <map>
#include <memory>
#include <sstream>
#include <fstream>
#include <iostream>
#include <algorithm>
#include <stdexcept>
#include <cmath>
#include <cfloat>
#include <climits>
#include <limits>
#include <iomanip>
#include <functional>
#include <numeric>
#include <list>
#include <set>
#include <unordered_map>
#include <thread>
#include <mutex>
#include <chrono>
#include <cassert>
#include <immintrin.h>
// BatchNorm's eps and the activation parameters have no public getter in the reference; an in-tree adapter would be a
// member or a friend of the layer classes. Test infrastructure only.
#define private public
#define protected public
#include "Msnhnet/net/MsnhNetBuilder.h"
#undef private
#undef protected
#include "../include/msnh_b200.h"

using namespace Msnhnet;

namespace {

struct Shape { int c = 0, h = 0, w = 0; };
struct WeightSlot { int op, slot; size_t count; };

int actCode(ActivationType a) {
    switch (a) {
        case LOGISTIC: return MSNH_ACT_LOGISTIC; case RELU: return MSNH_ACT_RELU; case RELU6: return MSNH_ACT_RELU6;
        case RELIE: return MSNH_ACT_RELIE; case RAMP: return MSNH_ACT_RAMP; case TANH: return MSNH_ACT_TANH;
        case PLSE: return MSNH_ACT_PLSE; case LEAKY: return MSNH_ACT_LEAKY; case ELU: return MSNH_ACT_ELU;
        case LOGGY: return MSNH_ACT_LOGGY; case STAIR: return MSNH_ACT_STAIR; case HARDTAN: return MSNH_ACT_HARDTAN;
        case LHTAN: return MSNH_ACT_LHTAN; case SOFT_PLUS: return MSNH_ACT_SOFT_PLUS; case SELU: return MSNH_ACT_SELU;
        case SWISH: return MSNH_ACT_SWISH; case HARD_SWISH: return MSNH_ACT_HARD_SWISH; case MISH: return MSNH_ACT_MISH;
        case NONE: return MSNH_ACT_NONE;
        default: throw std::runtime_error("activation not supported by the kernel library");
    }
}

struct Lowering {
    std::vector<MsnhB200Op> ops;
    std::vector<Shape> shapes;
    std::vector<WeightSlot> weights;

    static MsnhB200Op blank(int kind) {
        MsnhB200Op o;
        std::memset(&o, 0, sizeof(o));
        o.kind = kind;
        o.k_h = o.k_w = o.stride_h = o.stride_w = o.dil_h = o.dil_w = o.groups = 1;
        o.bn_eps = 1e-5f; o.scale = 1.f; o.route_groups = 1; o.softmax_groups = 1; o.softmax_temperature = 1.f;
        for (int i = 0; i < 3; ++i) o.slice_step[i] = 1;
        return o;
    }
    int emit(const MsnhB200Op &o, const Shape &s) { ops.push_back(o); shapes.push_back(s); return static_cast<int>(ops.size()) - 1; }
    static Shape outShape(const BaseLayer *l) { Shape s; s.c = l->getOutChannel(); s.h = l->getOutHeight(); s.w = l->getOutWidth(); return s; }
    void setAct(MsnhB200Op &o, const BaseLayer *l) {
        o.act = actCode(l->getActivation());
        o.act_param = !l->_actParams.empty() ? l->_actParams[0] : (o.act == MSNH_ACT_LEAKY ? 0.1f : (o.act == MSNH_ACT_SOFT_PLUS ? 20.f : 0.f));
    }
    int activation(int in, const BaseLayer *l, const Shape &s) {
        if (l->getActivation() == NONE) return in;
        MsnhB200Op o = blank(MSNH_OP_ACTIVATION);
        o.n_in = 1; o.in[0] = in; setAct(o, l);
        return emit(o, s);
    }

    // one non-block layer applied to op `in`
    int simple(BaseLayer *l, int in) {
        const Shape s = outShape(l);
        switch (l->type()) {
            case CONVOLUTIONAL: {
                auto *c = static_cast<ConvolutionalLayer *>(l);
                MsnhB200Op o = blank(MSNH_OP_CONV);
                o.n_in = 1; o.in[0] = in; o.filters = c->getOutChannel();
                o.k_h = c->getKSizeY(); o.k_w = c->getKSizeX(); o.stride_h = c->getStrideY(); o.stride_w = c->getStrideX();
                o.pad_h = c->getPaddingY(); o.pad_w = c->getPaddingX(); o.dil_h = c->getDilationY(); o.dil_w = c->getDilationX(); o.groups = c->getGroups();
                o.has_bn = c->getBatchNorm() ? 1 : 0; o.has_bias = (!c->getBatchNorm() && c->getUseBias()) ? 1 : 0; o.bn_eps = c->_bnEps;
                setAct(o, l);
                const int id = emit(o, s);
                // blob order of the layer's tensors: ConvolutionalLayer::loadAllWeigths (src/layers/MsnhConvolutionalLayer.cpp:1255-1329)
                weights.push_back({id, MSNH_W_WEIGHTS, static_cast<size_t>(c->getNWeights())});
                if (c->getBatchNorm()) for (int sl : {MSNH_W_BN_SCALE, MSNH_W_BN_BIAS, MSNH_W_BN_MEAN, MSNH_W_BN_VAR}) weights.push_back({id, sl, static_cast<size_t>(c->getOutChannel())});
                else if (c->getUseBias()) weights.push_back({id, MSNH_W_BIAS, static_cast<size_t>(c->getNBiases())});
                return id;
            }
            case CONNECTED: {
                auto *c = static_cast<ConnectedLayer *>(l);
                MsnhB200Op o = blank(MSNH_OP_CONNECTED);
                o.n_in = 1; o.in[0] = in; o.filters = c->getOutputNum();
                o.has_bn = c->getBatchNorm() ? 1 : 0; o.has_bias = (!c->getBatchNorm() && c->_useBias) ? 1 : 0; o.bn_eps = c->_bnEps;
                setAct(o, l);
                Shape fs; fs.c = c->getOutputNum(); fs.h = 1; fs.w = 1;
                const int id = emit(o, fs);
                weights.push_back({id, MSNH_W_WEIGHTS, static_cast<size_t>(c->getNWeights())});
                if (c->getBatchNorm()) for (int sl : {MSNH_W_BN_SCALE, MSNH_W_BN_MEAN, MSNH_W_BN_VAR, MSNH_W_BN_BIAS}) weights.push_back({id, sl, static_cast<size_t>(c->getOutputNum())});
                else if (c->_useBias) weights.push_back({id, MSNH_W_BIAS, static_cast<size_t>(c->getNBiases())});
                return id;
            }
            case BATCHNORM: {
                auto *b = static_cast<BatchNormLayer *>(l);
                MsnhB200Op o = blank(MSNH_OP_BATCHNORM);
                o.n_in = 1; o.in[0] = in; o.bn_eps = b->_eps; setAct(o, l);
                const int id = emit(o, s);
                for (int sl : {MSNH_W_BN_SCALE, MSNH_W_BN_BIAS, MSNH_W_BN_MEAN, MSNH_W_BN_VAR}) weights.push_back({id, sl, static_cast<size_t>(s.c)});
                return id;
            }
            case ACTIVE: {
                MsnhB200Op o = blank(MSNH_OP_ACTIVATION);
                o.n_in = 1; o.in[0] = in; setAct(o, l);
                return emit(o, s);
            }
            case MAXPOOL: {
                auto *p = static_cast<MaxPoolLayer *>(l);
                MsnhB200Op o = blank(MSNH_OP_MAXPOOL);
                o.n_in = 1; o.in[0] = in;
                o.k_h = p->getKSizeY(); o.k_w = p->getKSizeX(); o.stride_h = p->getStrideY(); o.stride_w = p->getStrideX(); o.pad_h = p->getPaddingY(); o.pad_w = p->getPaddingX();
                o.out_h = s.h; o.out_w = s.w;
                return emit(o, s);
            }
            case LOCAL_AVGPOOL: {
                auto *p = static_cast<LocalAvgPoolLayer *>(l);
                MsnhB200Op o = blank(MSNH_OP_AVGPOOL);
                o.n_in = 1; o.in[0] = in;
                o.k_h = p->getKSizeY(); o.k_w = p->getKSizeX(); o.stride_h = p->getStrideY(); o.stride_w = p->getStrideX(); o.pad_h = p->getPaddingY(); o.pad_w = p->getPaddingX();
                o.out_h = s.h; o.out_w = s.w;
                return emit(o, s);
            }
            case PADDING: {
                auto *p = static_cast<PaddingLayer *>(l);
                MsnhB200Op o = blank(MSNH_OP_PAD);
                o.n_in = 1; o.in[0] = in; o.pad_top = p->getTop(); o.pad_down = p->getDown(); o.pad_left = p->getLeft(); o.pad_right = p->getRight(); o.const_val = p->getPaddingVal();
                return emit(o, s);
            }
            case UPSAMPLE: {
                auto *u = static_cast<UpSampleLayer *>(l);
                MsnhB200Op o = blank(MSNH_OP_UPSAMPLE);
                o.n_in = 1; o.in[0] = in; o.stride_h = u->getStrideY(); o.stride_w = u->getStrideX(); o.scale = 1.f;
                return emit(o, s);
            }
            case SLICE: {
                auto *c = static_cast<SliceLayer *>(l);
                MsnhB200Op o = blank(MSNH_OP_SLICE);
                o.n_in = 1; o.in[0] = in;
                o.slice_start[0] = c->getStart0(); o.slice_step[0] = c->getStep0(); o.slice_start[1] = c->getStart1(); o.slice_step[1] = c->getStep1();
                o.slice_start[2] = c->getStart2(); o.slice_step[2] = c->getStep2();
                return emit(o, s);
            }
            case SOFTMAX: {
                auto *c = static_cast<SoftMaxLayer *>(l);
                MsnhB200Op o = blank(MSNH_OP_SOFTMAX);
                o.n_in = 1; o.in[0] = in; o.softmax_groups = c->getGroups(); o.softmax_temperature = c->getTemperature();
                return emit(o, s);
            }
            case EMPTY: {
                MsnhB200Op o = blank(MSNH_OP_IDENTITY);
                o.n_in = 1; o.in[0] = in;
                return emit(o, s);
            }
            default: throw std::runtime_error("layer type " + l->getLayerName() + " is not part of this adapter");
        }
    }
    int chain(const std::vector<BaseLayer *> &seq, int in) { for (BaseLayer *l : seq) in = simple(l, in); return in; }
    int add(const std::vector<int> &ins, const BaseLayer *block, const Shape &s) {
        MsnhB200Op o = blank(MSNH_OP_ADD);
        o.n_in = static_cast<int>(ins.size());
        for (size_t k = 0; k < ins.size(); ++k) o.in[k] = ins[k];
        if (block) setAct(o, block);
        return emit(o, s);
    }
    int concat(const std::vector<int> &ins, int groups, int groupId, const Shape &s) {
        MsnhB200Op o = blank(MSNH_OP_CONCAT);
        o.n_in = static_cast<int>(ins.size()); o.route_groups = groups; o.route_group_id = groupId;
        for (size_t k = 0; k < ins.size(); ++k) o.in[k] = ins[k];
        return emit(o, s);
    }
};

// The layers of a built net -> ops + weight slots; layerOp[i] = op holding layer i's output (-1: none).
void lowerLayers(const std::vector<BaseLayer *> &layers, Lowering &L, std::vector<int> &layerOp) {
    int prev = MSNH_B200_INPUT;
    for (size_t li = 0; li < layers.size(); ++li) {
        BaseLayer *l = layers[li];
        const Shape s = Lowering::outShape(l);
        int out = -1;
        switch (l->type()) {
            case ROUTE: {
                auto *r = static_cast<RouteLayer *>(l);
                std::vector<int> ins;
                for (int idx : r->getInputLayerIndexes()) ins.push_back(layerOp.at(static_cast<size_t>(idx)));
                if (r->getAddModel() == 1) out = L.add(ins, l, s);
                else { out = L.concat(ins, r->getGroups(), r->getGroupIndex(), s); out = L.activation(out, l, s); }
                break;
            }
            case VARIABLE_OP: {
                auto *v = static_cast<VariableOpLayer *>(l);
                if (v->getVarOpType() != VariableOpParams::VAR_OP_ADD) throw std::runtime_error("varop types other than add are not part of this adapter");
                const std::vector<int> idx = v->getInputLayerIndexes();
                const int a = idx.size() == 2 ? layerOp.at(static_cast<size_t>(idx[0])) : prev;
                const int b = layerOp.at(static_cast<size_t>(idx.size() == 2 ? idx[1] : idx[0]));
                out = L.add({a, b}, nullptr, s);
                break;
            }
            case RES_BLOCK: {
                auto *b = static_cast<ResBlockLayer *>(l);
                out = L.add({prev, L.chain(b->baseLayers, prev)}, l, s);
                break;
            }
            case RES_2_BLOCK: {
                auto *b = static_cast<Res2BlockLayer *>(l);
                const int base = L.chain(b->baseLayers, prev);
                const int br = L.chain(b->branchLayers, prev);
                out = L.add({base, br}, l, s);
                break;
            }
            case ADD_BLOCK: case CONCAT_BLOCK: {
                const std::vector<std::vector<BaseLayer *>> &branches = l->type() == ADD_BLOCK ? static_cast<AddBlockLayer *>(l)->branchLayers
                                                                                                  : static_cast<ConcatBlockLayer *>(l)->branchLayers;
                std::vector<int> outs;
                for (const auto &br : branches) {
                    bool allEmpty = true;                       // an `empty` branch is the block input itself
                    for (BaseLayer *c : br) if (c->type() != EMPTY) allEmpty = false;
                    outs.push_back(allEmpty ? prev : L.chain(br, prev));
                }
                if (l->type() == ADD_BLOCK) out = outs.size() == 1 ? L.activation(outs[0], l, s) : L.add(outs, l, s);
                else { out = L.concat(outs, 1, 0, s); out = L.activation(out, l, s); }
                if (out == prev) { MsnhB200Op o = Lowering::blank(MSNH_OP_IDENTITY); o.n_in = 1; o.in[0] = prev; out = L.emit(o, s); }
                break;
            }
            case YOLO: {
                auto *y = static_cast<YoloLayer *>(l);
                MsnhB200Op o = Lowering::blank(MSNH_OP_YOLO);
                o.n_in = 1; o.in[0] = prev; o.yolo_classes = y->getClassNum();
                o.yolo_type = y->getYoloType() == YoloType::YoloV5 ? MSNH_YOLO_V5 : (y->getYoloType() == YoloType::YoloV4 ? MSNH_YOLO_V4 : MSNH_YOLO_V3);
                for (int k = 0; k < 6; ++k) o.yolo_anchors[k] = y->anchors[static_cast<size_t>(k)];
                out = L.emit(o, s);
                break;
            }
            case YOLO_OUT: {
                auto *y = static_cast<YoloOutLayer *>(l);
                MsnhB200Op o = Lowering::blank(MSNH_OP_YOLO_COLLECT);
                int cells = 0, k = 0;
                for (int idx : y->getYoloIndexes()) {
                    const int src = layerOp.at(static_cast<size_t>(idx));
                    o.in[k++] = src; cells += 3 * L.shapes[src].h * L.shapes[src].w;
                }
                o.n_in = k; o.const_val = y->getConfThresh(); o.is_output = 1;
                Shape cs; cs.c = 8; cs.h = 1; cs.w = cells;
                L.emit(o, cs);
                out = -1;
                break;
            }
            default: out = L.simple(l, prev);
        }
        layerOp.push_back(out);
        if (out >= 0) prev = out;
    }
    bool yolo = !layers.empty() && layers.back()->type() == YOLO_OUT;
    if (!yolo && prev >= 0) L.ops[static_cast<size_t>(prev)].is_output = 1;
}

void printOp(const MsnhB200Op &o) {
    std::printf("op %d %d", o.kind, o.n_in);
    for (int k = 0; k < MSNH_B200_MAX_IN; ++k) std::printf(" %d", k < o.n_in ? o.in[k] : 0);
    std::printf(" %d %d %d %d %d %d %d %d %d %d %d %d", o.filters, o.k_h, o.k_w, o.stride_h, o.stride_w, o.pad_h, o.pad_w, o.dil_h, o.dil_w, o.groups, o.out_h, o.out_w);
    std::printf(" %d %d %d %d", o.pad_top, o.pad_down, o.pad_left, o.pad_right);
    for (int k = 0; k < 3; ++k) std::printf(" %d %d", o.slice_start[k], o.slice_step[k]);
    std::printf(" %d %d %d %d %.9g %d %.9g %.9g %.9g %d %d %d %.9g %d %d", o.route_groups, o.route_group_id, o.has_bn, o.has_bias, o.bn_eps, o.act, o.act_param,
                o.scale, o.const_val, o.binary_kind, o.binary_const, o.softmax_groups, o.softmax_temperature, o.yolo_type, o.yolo_classes);
    for (int k = 0; k < 6; ++k) std::printf(" %.9g", o.yolo_anchors[k]);
    std::printf(" %d %d %d %d %d %d %d %d\n", o.is_output, o.upsample_mode, o.align_corners, o.remap_kind, o.remap_dims[0], o.remap_dims[1], o.remap_dims[2], o.out_c);
}

}  // namespace

int main(int argc, char **argv) {
    if (argc < 2) { std::fprintf(stderr, "usage: seam_adapter <net.msnhnet>\n"); return 1; }
    try {
        NetBuilder::setPreviewMode(true);         // shapes and layer objects only: no buffers, no weights
        NetBuilder nb;
        nb.buildNetFromMsnhNet(argv[1]);
        Lowering L;
        std::vector<int> layerOp;
        lowerLayers(nb.getNet()->layers, L, layerOp);
        for (const MsnhB200Op &o : L.ops) printOp(o);
        for (const WeightSlot &w : L.weights) std::printf("w %d %d %zu\n", w.op, w.slot, w.count);
    } catch (Exception &e) {
        std::fprintf(stderr, "reference exception: %s\n", e.what());
        return 4;
    } catch (std::exception &e) {
        std::fprintf(stderr, "adapter: %s\n", e.what());
        return 5;
    }
    return 0;
}
