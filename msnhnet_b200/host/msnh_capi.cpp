// The reference's C entry points (src/c_api/MsnhnetLib.cpp) over the NetBuilder mirror, plus the
// batched additions declared in include/msnhnet_capi.h.
#include "msnhnet_capi.h"

#include <algorithm>
#include <cstring>
#include <memory>
#include <string>

#include "msnh_b200.h"
#include "msnh_netbuilder.h"

namespace {

std::unique_ptr<Msnhnet::NetBuilder> net;      // one net per process, as in the reference
int optDevice = 0, optBatch = 0;
unsigned optFlags = 0;
thread_local std::string lastMsg;

int setMsg(char **msg, const std::string &text) {
    lastMsg = text;
    if (msg) *msg = const_cast<char *>(lastMsg.c_str());
    return -1;
}
#define NEED_NET(msg) do { if (!net) return setMsg(msg, "call initMsnhnet first"); } while (0)

void fill(BBox &o, const Msnhnet::YoloBox &b) {
    o.x = b.xywhBox.x; o.y = b.xywhBox.y; o.w = b.xywhBox.w; o.h = b.xywhBox.h;
    o.conf = b.conf; o.bestClsConf = b.bestClsConf; o.bestClsIdx = static_cast<uint32_t>(b.bestClsIdx); o.angle = b.angle;
}

}  // namespace

extern "C" {

int initMsnhnet(void) {
    try { net.reset(new Msnhnet::NetBuilder()); } catch (...) { return -1; }
    return 1;
}

int msnhB200SetOptions(int device, int batch, unsigned planFlags) {
    optDevice = device; optBatch = batch; optFlags = planFlags;
    return 1;
}

int msnhB200SetPackCache(int enable) {
    if (!net) return -1;
    net->setWeightPackCache(enable != 0);
    return 1;
}

int msnhB200LastLoadUsedPack(void) { return net ? (net->lastLoadUsedPack() ? 1 : 0) : -1; }

int msnhB200SetDeviceNms(int enable) {
    if (!net) return -1;
    net->setDeviceNms(enable != 0);
    return 1;
}

int buildMsnhnet(char **msg, const char *msnhnet, const char *msnhbin, int useFp16, int useCudaOnly) {
    NEED_NET(msg);
    try {
        Msnhnet::NetBuilder::setUseFp16(useFp16 != 0);
        Msnhnet::NetBuilder::setForceUseCuda(useCudaOnly != 0);
        net->setDevice(optDevice); net->setBatch(optBatch); net->setPlanFlags(optFlags);
        net->buildNetFromMsnhNet(msnhnet);
        net->loadWeightsFromMsnhBin(msnhbin);
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200BuildFromMemory(char **msg, const char *text, const float *weights, size_t weightCount, int useFp16) {
    NEED_NET(msg);
    if (!text || !weights) return setMsg(msg, "null argument");
    try {
        Msnhnet::NetBuilder::setUseFp16(useFp16 != 0);
        net->setDevice(optDevice); net->setBatch(optBatch); net->setPlanFlags(optFlags);
        net->buildNetFromMsnhNetText(text);
        net->loadWeightsFromMemory(weights, weightCount);
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200Inspect(char **msg, const char *text, int *layers, size_t *weightCount, int *isYolo) {
    if (!text) return setMsg(msg, "null argument");
    const bool before = Msnhnet::NetBuilder::isPreviewMode;
    try {
        Msnhnet::NetBuilder::setPreviewMode(true);
        Msnhnet::NetBuilder probe;
        probe.buildNetFromMsnhNetText(text);
        if (layers) *layers = static_cast<int>(probe.getLayerCount());
        if (weightCount) *weightCount = probe.getWeightCount();
        if (isYolo) *isYolo = probe.isYoloNet() ? 1 : 0;
        lastMsg = probe.getLayerDetail();
        if (msg) *msg = const_cast<char *>(lastMsg.c_str());
    } catch (const std::exception &e) { Msnhnet::NetBuilder::setPreviewMode(before); return setMsg(msg, e.what()); }
    Msnhnet::NetBuilder::setPreviewMode(before);
    return 1;
}

// Image decoding and the resize/letterbox preprocessing of src/utils/MsnhCVUtil.cpp are outside this
// backend: callers pass planar CHW floats (runClassifyNoPred, msnhB200Run*Batch).
int msnhB200WeightLayout(char **msg, const char *text) {
    if (!text || !msg) return -1;
    const bool before = Msnhnet::NetBuilder::isPreviewMode;
    try {
        Msnhnet::NetBuilder::setPreviewMode(true);
        Msnhnet::NetBuilder probe;
        probe.buildNetFromMsnhNetText(text);
        lastMsg = probe.getWeightLayout();
        *msg = const_cast<char *>(lastMsg.c_str());
    } catch (const std::exception &e) { Msnhnet::NetBuilder::setPreviewMode(before); return setMsg(msg, e.what()); }
    Msnhnet::NetBuilder::setPreviewMode(before);
    return 1;
}

int msnhB200OpList(char **msg, const char *text) {
    if (!text || !msg) return -1;
    const bool before = Msnhnet::NetBuilder::isPreviewMode;
    try {
        Msnhnet::NetBuilder::setPreviewMode(true);
        Msnhnet::NetBuilder probe;
        probe.buildNetFromMsnhNetText(text);
        lastMsg = probe.getOpList();
        *msg = const_cast<char *>(lastMsg.c_str());
    } catch (const std::exception &e) { Msnhnet::NetBuilder::setPreviewMode(before); return setMsg(msg, e.what()); }
    Msnhnet::NetBuilder::setPreviewMode(before);
    return 1;
}

int runClassifyFile(char **msg, const char *, int *, PredDataType, int, const float *, const float *) {
    return setMsg(msg, "runClassifyFile: image decoding is not part of this backend; pass CHW floats to runClassifyNoPred");
}
// src/c_api/MsnhnetLib.cpp:540-626 (the variant on the reference's own Mat): same argument checks and the same
// preprocessing per PredDataType, run on the device. PRE_DATA_FC32_C1 (gray nets) is not part of this backend.
int runClassifyList(char **msg, unsigned char *imageData, const int width, const int height, const int channel, int *bestIndex,
                    PredDataType preDataType, const int swapRGB, int runGPU, const float *mean, const float *std) {
    NEED_NET(msg);
    if (!imageData || !bestIndex) return setMsg(msg, "null argument");
    if (!runGPU) return setMsg(msg, "this backend has no CPU path: call with runGPU = 1");
    if (channel != 1 && channel != 3) return setMsg(msg, "channel must be 1 or 3");
    if (channel == 1 && preDataType != PRE_DATA_FC32_C1) return setMsg(msg, "channel 1 must preprocess with F32_C1");
    if (channel == 3 && preDataType == PRE_DATA_FC32_C1) return setMsg(msg, "channel 1 can't preprocess with F32_C1");
    int mode;
    switch (preDataType) {
        case PRE_DATA_NONE: return setMsg(msg, "preDataType can't be none");
        case PRE_DATA_FC32_C1: return setMsg(msg, "PRE_DATA_FC32_C1 (gray input) is not supported by this backend; pass CHW floats to runClassifyNoPred");
        case PRE_DATA_FC32_C3: mode = MSNH_PREP_UNIT; break;
        case PRE_DATA_GOOGLENET_FC3: mode = MSNH_PREP_GOOGLENET; break;
        case PRE_DATA_PADDING_ZERO_FC3: mode = MSNH_PREP_PAD_SQUARE; break;
        case PRE_DATA_CAFFE_FC3: mode = MSNH_PREP_CAFFE; break;
        case PRE_DATA_TRANSFORMED_FC3:
            if (!mean || !std) return setMsg(msg, "mean or std can't be null");
            mode = MSNH_PREP_TRANSFORMED; break;
        default: return setMsg(msg, "unknown preDataType");
    }
    try {
        std::vector<float> out = net->runClassifyGPUImage(imageData, width, height, mode, swapRGB != 0, mean, std);
        *bestIndex = static_cast<int>(std::max_element(out.begin(), out.end()) - out.begin());
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}
int runYoloFile(char **msg, const char *, BBoxContainer *, int *, const int) {
    return setMsg(msg, "runYoloFile: image decoding is not part of this backend; pass CHW floats to msnhB200RunYoloBatch");
}
// src/c_api/MsnhnetLib.cpp:754-826: pad to a square with 127, resize to the net input, /255 (on the device), forward,
// boxes in net-input coordinates as there.
int runYoloList(char **msg, unsigned char *imageData, const int width, const int height, const int channel, BBoxContainer *bboxContainer,
                int *detectedNum, const int swapRGB, const int runGPU) {
    NEED_NET(msg);
    if (!imageData || !bboxContainer || !detectedNum) return setMsg(msg, "null argument");
    if (!runGPU) return setMsg(msg, "this backend has no CPU path: call with runGPU = 1");
    if (channel != 1 && channel != 3) return setMsg(msg, "channel must be 1 or 3");
    if (channel == 1) return setMsg(msg, "gray input is not supported by this backend (the reference's own path yields a 1-plane image the net rejects)");
    try {
        auto r = net->runYoloGPUImage(imageData, width, height, swapRGB != 0);
        if (r[0].size() > MSNH_MAX_BBOX_NUM) return setMsg(msg, "BBox buffer is not enough, please change MaxBBoxNum and rebuild");
        *detectedNum = static_cast<int>(r[0].size());
        for (size_t k = 0; k < r[0].size(); ++k) fill(bboxContainer->boxes[k], r[0][k]);
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int runClassifyNoPred(char **msg, const float *data, const int len, int *bestIndex, int runGPU) {
    NEED_NET(msg);
    if (!data || !bestIndex || len <= 0) return setMsg(msg, "null argument");
    if (!runGPU) return setMsg(msg, "this backend has no CPU path: call with runGPU = 1");
    try {
        std::vector<float> img(data, data + len);
        std::vector<float> out = net->runClassifyGPU(img);
        *bestIndex = static_cast<int>(std::max_element(out.begin(), out.end()) - out.begin());
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int dispose(void) { net.reset(); return 1; }
int withGPU(int *GPU) { if (GPU) *GPU = 1; return 1; }
int withCUDNN(int *CUDNN) { if (CUDNN) *CUDNN = 0; return 0; }
int getCpuForwardTime(float *time) { if (!net || !time) return -1; *time = net->getInferenceTime(); return 1; }
int getGpuForwardTime(float *time) { if (!net || !time) return -1; *time = net->getGpuInferenceTime(); return 1; }
int getInputDim(int *width, int *heigth, int *channel) {
    if (!net) return -1;
    try {
        Msnhnet::Point2I wh = net->getInputSize();
        if (width) *width = wh.x;
        if (heigth) *heigth = wh.y;
        if (channel) *channel = net->getInputChannel();
    } catch (...) { return -1; }
    return 1;
}

int msnhB200RunClassifyBatch(char **msg, const float *images, int nImages, float *out, size_t outCapacity) {
    NEED_NET(msg);
    if (!images || !out) return setMsg(msg, "null argument");
    try {
        std::vector<float> r = net->runClassifyGPUBatch(images, nImages);
        if (r.size() > outCapacity) return setMsg(msg, "output buffer too small: need " + std::to_string(r.size()));
        std::memcpy(out, r.data(), r.size() * sizeof(float));
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200RunYoloBatch(char **msg, const float *images, int nImages, BBox *boxes, int maxBoxes, int *counts) {
    NEED_NET(msg);
    if (!images || !boxes || !counts || maxBoxes < 1) return setMsg(msg, "null argument");
    try {
        auto r = net->runYoloGPUBatch(images, nImages);
        for (int i = 0; i < nImages; ++i) {
            const int n = std::min<int>(static_cast<int>(r[i].size()), maxBoxes);
            counts[i] = n;
            for (int k = 0; k < n; ++k) fill(boxes[static_cast<size_t>(i) * maxBoxes + k], r[i][k]);
        }
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200RunYoloStream(char **msg, const float *images, int nBatches, BBox *boxes, int maxBoxes, int *counts) {
    NEED_NET(msg);
    if (!images || !boxes || !counts || maxBoxes < 1) return setMsg(msg, "null argument");
    try {
        auto r = net->runYoloGPUStream(images, nBatches);
        for (size_t i = 0; i < r.size(); ++i) {
            const int n = std::min<int>(static_cast<int>(r[i].size()), maxBoxes);
            counts[i] = n;
            for (int k = 0; k < n; ++k) fill(boxes[i * maxBoxes + k], r[i][k]);
        }
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200RunClassifyStream(char **msg, const float *images, int nBatches, float *out, size_t outCapacity) {
    NEED_NET(msg);
    if (!images || !out) return setMsg(msg, "null argument");
    try {
        net->runClassifyGPUStreamInto(images, nBatches, out, outCapacity);
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200RunYoloStreamU8(char **msg, const unsigned char *images, int width, int height, int swapRGB, int nBatches,
                            BBox *boxes, int maxBoxes, int *counts) {
    NEED_NET(msg);
    if (!images || !boxes || !counts || maxBoxes < 1) return setMsg(msg, "null argument");
    try {
        auto r = net->runYoloGPUStreamU8(images, width, height, swapRGB != 0, nBatches);
        for (size_t i = 0; i < r.size(); ++i) {
            const int n = std::min<int>(static_cast<int>(r[i].size()), maxBoxes);
            counts[i] = n;
            for (int k = 0; k < n; ++k) fill(boxes[i * maxBoxes + k], r[i][k]);
        }
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200RunClassifyStreamU8(char **msg, const unsigned char *images, int width, int height, int prepMode, int swapRGB,
                                const float *mean, const float *std, int nBatches, float *out, size_t outCapacity) {
    NEED_NET(msg);
    if (!images || !out) return setMsg(msg, "null argument");
    try {
        net->runClassifyGPUStreamU8Into(images, width, height, prepMode, swapRGB != 0, mean, std, nBatches, out, outCapacity);
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200Forward(char **msg, const float *images, int nImages) {
    NEED_NET(msg);
    if (!images) return setMsg(msg, "null argument");
    try { net->forwardGPU(images, nImages); } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}
int msnhB200ForwardResident(char **msg, int nImages, int sync) {
    NEED_NET(msg);
    try { net->forwardGPUDeviceResident(nImages, sync != 0); } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200GetLayerOutput(char **msg, int layer, int nImages, float *out, size_t capacity, int *c, int *h, int *w) {
    NEED_NET(msg);
    try {
        std::vector<float> r = net->getLayerOutput(layer, nImages, c, h, w);
        if (!out || r.size() > capacity) return setMsg(msg, "output buffer too small: need " + std::to_string(r.size()));
        std::memcpy(out, r.data(), r.size() * sizeof(float));
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200GetCandidates(char **msg, int nImages, float *rows, int maxRows, int *counts) {
    NEED_NET(msg);
    if (!rows || !counts) return setMsg(msg, "null argument");
    try {
        int layers, isYolo, batch, c, h, w; size_t wc; float ct, nt;
        (void)layers; (void)isYolo; (void)batch; (void)c; (void)h; (void)w; (void)wc; (void)ct; (void)nt;
        std::vector<int> cnt;
        std::vector<float> all = net->getCandidates(nImages, cnt);
        const size_t stride = all.size() / static_cast<size_t>(nImages) / 8;
        for (int i = 0; i < nImages; ++i) {
            const int n = std::min(cnt[i], maxRows);
            counts[i] = n;
            std::memcpy(rows + static_cast<size_t>(i) * maxRows * 8, all.data() + static_cast<size_t>(i) * stride * 8, sizeof(float) * 8 * n);
        }
    } catch (const std::exception &e) { return setMsg(msg, e.what()); }
    return 1;
}

int msnhB200PostProcess(const float *rows, int count, float nmsThresh, int useSoftNms, BBox *out, int maxOut, int *n) {
    if (!rows || !out || !n || count < 0) return -1;
    std::vector<Msnhnet::YoloBox> r = Msnhnet::NetBuilder::postProcess(rows, count, nmsThresh, useSoftNms != 0);
    *n = std::min<int>(static_cast<int>(r.size()), maxOut);
    for (int k = 0; k < *n; ++k) fill(out[k], r[k]);
    return 1;
}

int msnhB200GetInfo(int *layers, size_t *weightCount, int *isYolo, int *batch, int *lastC, int *lastH, int *lastW, float *confThresh, float *nmsThresh) {
    if (!net) return -1;
    if (layers) *layers = static_cast<int>(net->getLayerCount());
    if (weightCount) *weightCount = net->getWeightCount();
    if (isYolo) *isYolo = net->isYoloNet() ? 1 : 0;
    if (batch) *batch = net->getBatch();
    if (lastC) *lastC = net->getLastLayerOutChannel();
    if (lastH) *lastH = net->getLastLayerOutHeight();
    if (lastW) *lastW = net->getLastLayerOutWidth();
    if (confThresh) *confThresh = net->confThresh();
    if (nmsThresh) *nmsThresh = net->nmsThresh();
    return 1;
}

int msnhB200KernelTimeMs(float *ms) { if (!net || !ms) return -1; *ms = net->getGpuKernelTime(); return 1; }
void *msnhB200PlanHandle(void) { return net ? net->plan() : nullptr; }
void *msnhB200CtxHandle(void) { return net ? net->context() : nullptr; }

}  // extern "C"
