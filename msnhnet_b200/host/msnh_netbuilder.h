// Host-side mirror of the reference's net builder for the GPU forward path: same class and method
// names, argument meaning and error behaviour as Msnhnet::NetBuilder
// (include/Msnhnet/net/MsnhNetBuilder.h:48-117, src/net/MsnhNetBuilder.cpp), with the per-layer
// forwardGPU loop replaced by one plan of the B200 kernel library (include/msnh_b200.h).
// The CPU entry points (runClassify / runYolo) are not part of this backend and throw.
#pragma once
#include <string>
#include <vector>

#include "msnh_format.h"

#include "msnh_b200.h"      // MsnhB200Op (the context and plan types stay opaque)

namespace Msnhnet {

struct Point2I { Point2I(int x, int y) : x(x), y(y) {} int x = 0, y = 0; };

// include/Msnhnet/utils/MsnhTypes.h:72-140
class Box {
public:
    struct XYWHBox {
        XYWHBox() {}
        XYWHBox(float x, float y, float w, float h) : x(x), y(y), w(w), h(h) {}
        float x = 0, y = 0, w = 0, h = 0;
    };
    static float iou(const XYWHBox &a, const XYWHBox &b);
};

// include/Msnhnet/layers/MsnhYoloDef.h:21-33 (the fields this path fills)
struct YoloBox {
    Box::XYWHBox xywhBox;
    float conf = 0, bestClsConf = 0;
    int   bestClsIdx = 0;
    float angle = 0, regAngle = 0;
};

class NetBuilder {
public:
    NetBuilder();
    ~NetBuilder();
    NetBuilder(const NetBuilder &) = delete;
    NetBuilder &operator=(const NetBuilder &) = delete;

    // process-wide switches of the reference (src/net/MsnhNetBuilder.cpp:28-66)
    static void setPreviewMode(const bool &mode);
    static void setMemAlign(const bool &memAlign);
    static void setOnlyGpu(const bool &onlyGpu);
    static void setOnlyCpu(const bool &onlyCpu);
    static void setUseFp16(const bool &useFp16);       // fp16 storage + fp16 tensor cores for the whole net
    static void setForceUseCuda(const bool &onlyUseCuda);

    // additions of this backend (set before buildNetFromMsnhNet)
    void setDevice(int device);        // CUDA device ordinal, default 0
    void setBatch(int batch);          // overrides the file's `batch:` (images per forward)
    void setPlanFlags(unsigned flags); // MSNH_PLAN_* debug flags
    // score sort + NMS on the device instead of on the host (YoloOutLayer's host half, src/layers/MsnhYoloOutLayer.cpp:167-197,
    // :381-461); images with more than 4096 candidates still take the host path. May be switched at any time.
    // Weight pack cache: loadWeightsFromMsnhBin(path) keeps the packed device form of the weights in
    // path + ".b200pack" and, when that file matches the net, the build options and the blob's size and
    // modification time, loads it instead of reading and repacking the float blob. Off by default.
    void setWeightPackCache(bool on) { _packCache = on; }
    bool lastLoadUsedPack() const { return _usedPack; }
    void setDeviceNms(bool on) { _deviceNms = on; }
    bool getDeviceNms() const { return _deviceNms; }

    void buildNetFromMsnhNet(const std::string &path);
    void buildNetFromMsnhNetText(const std::string &text);
    void loadWeightsFromMsnhBin(const std::string &path);
    void loadWeightsFromMemory(const float *data, size_t count);

    std::vector<float> runClassify(std::vector<float> img);                 // throws: CPU path not in this backend
    std::vector<std::vector<YoloBox>> runYolo(std::vector<float> img);      // throws
    std::vector<float> runClassifyGPU(std::vector<float> img);
    std::vector<std::vector<YoloBox>> runYoloGPU(std::vector<float> img);
    // batched forms: `images` holds nImages planar CHW float images back to back (host memory)
    std::vector<float> runClassifyGPUBatch(const float *images, int nImages);
    std::vector<std::vector<YoloBox>> runYoloGPUBatch(const float *images, int nImages);
    // raw 8-bit RGB image (HWC) in: the reference's host preprocessing (src/utils/MsnhCVUtil.cpp:91-373, what
    // runYoloList / runClassifyList of its C API do first) runs on the device; prepMode = MSNH_PREP_* of msnh_b200.h
    std::vector<std::vector<YoloBox>> runYoloGPUImage(const unsigned char *image, int width, int height, bool swapRGB);
    std::vector<float> runClassifyGPUImage(const unsigned char *image, int width, int height, int prepMode, bool swapRGB,
                                           const float *mean, const float *std);
    // streaming forms: nBatches batches of getBatch() images back to back in host (ideally pinned)
    // memory; the copy-in of batch i+1, the forward of batch i and the host post-processing of
    // batch i-1 overlap. Results in image order.
    std::vector<std::vector<YoloBox>> runYoloGPUStream(const float *images, int nBatches);
    std::vector<float> runClassifyGPUStream(const float *images, int nBatches);
    void runClassifyGPUStreamInto(const float *images, int nBatches, float *out, size_t capacity);
    // the same for raw 8-bit HWC images of width x height pixels (preprocessing on the device, as in run*GPUImage)
    std::vector<std::vector<YoloBox>> runYoloGPUStreamU8(const unsigned char *images, int width, int height, bool swapRGB, int nBatches);
    void runClassifyGPUStreamU8Into(const unsigned char *images, int width, int height, int prepMode, bool swapRGB,
                                    const float *mean, const float *std, int nBatches, float *out, size_t capacity);
    // forward only (no read-back of the result, no NMS): used for throughput timing
    void forwardGPU(const float *images, int nImages);
    void forwardGPUDeviceResident(int nImages, bool sync);   // input already in the plan's staging buffer

    Point2I getInputSize();
    int     getInputChannel();
    int     getBatch() const { return _batch; }
    void    clearLayers();
    float   getInferenceTime();          // CPU path: always 0 here
    float   getGpuInferenceTime() const; // ms of the last run*GPU call (host wall clock, like the reference)
    float   getGpuKernelTime() const;    // ms between the first and last kernel of the last forward (CUDA events)
    std::string getLayerDetail();
    std::string getTimeDetail();
    int     getLastLayerOutWidth() const { return _lastW; }
    int     getLastLayerOutHeight() const { return _lastH; }
    int     getLastLayerOutChannel() const { return _lastC; }
    size_t  getLastLayerOutNum() const { return _lastNum; }
    void    setSaveLayerOutput(bool v) { _saveLayerOutput = v; }
    void    setSaveLayerWeights(bool v) { _saveLayerWeights = v; }
    bool    getSaveLayerWeights() const { return _saveLayerWeights; }

    // parity / test access
    size_t  getLayerCount() const { return _layerOp.size(); }
    size_t  getWeightCount() const { return _totalWeights; }
    bool    isYoloNet() const { return _collectOp >= 0; }
    // one line per tensor of the .msnhbin blob, in blob order: "op slot count rows" (slot = MSNH_W_*;
    // rows = output channels of a weight tensor, so fan-in = count / rows)
    std::string getWeightLayout() const;
    std::string getOpList() const;          // the lowered op list, one text line per op (every field of MsnhB200Op)
    // output of top-level layer `layer` of the last forward as planar CHW floats per image
    // (needs MSNH_PLAN_KEEP_ALL); C,H,W returned through the pointers
    std::vector<float> getLayerOutput(int layer, int nImages, int *c, int *h, int *w);
    // detection candidates before NMS for image i of the last forward, rows {x,y,w,h,conf,bestClsConf,bestClsIdx,order}
    std::vector<float> getCandidates(int nImages, std::vector<int> &counts);
    MsnhB200Plan *plan() const { return _plan; }
    MsnhB200Ctx  *context() const { return _ctx; }
    float confThresh() const { return _confThresh; }
    float nmsThresh() const { return _nmsThresh; }

    // the reference's host-side NMS (src/layers/MsnhYoloOutLayer.cpp:381-461), exposed for tests
    static std::vector<YoloBox> nms(const std::vector<YoloBox> &bboxes, const float &nmsThresh, const bool &useSoftNms,
                                    const float &sigma = 0.3f);
    // candidate rows -> score-sorted boxes -> nms, as YoloOutLayer::forward does (src/layers/MsnhYoloOutLayer.cpp:119-197)
    static std::vector<YoloBox> postProcess(const float *rows, int count, float nmsThresh, bool useSoftNms);
    // rows {x,y,w,h,conf,bestClsConf,bestClsIdx,_} that are already final boxes (device NMS output) -> YoloBox
    static std::vector<YoloBox> boxesFromRows(const float *rows, int count);

    static bool onlyUseGpu, onlyUseCpu, useFp16, onlyUseCuda, isPreviewMode;

private:
    struct WeightSlot { int op, slot; size_t count; int rows; };
    void lower(const NetDesc &net);
    std::vector<std::vector<YoloBox>> yoloResults(int nImages);
    template <typename Push, typename Again> std::vector<std::vector<YoloBox>> yoloStream(int nBatches, Push &&push, Again &&again);
    template <typename Push> void classifyStream(int nBatches, float *out, size_t capacity, Push &&push);
    void destroyPlan();
    void checkK(int rc, const char *what);

    MsnhB200Ctx  *_ctx = nullptr;
    MsnhB200Plan *_plan = nullptr;
    int _device = 0, _batchOverride = 0, _batch = 1;
    unsigned _planFlags = 0;
    int _inW = 0, _inH = 0, _inC = 0;
    std::vector<int> _layerOp;            // top-level layer index -> op that holds its output (-1: yoloout)
    std::vector<std::string> _layerNames; // for getLayerDetail
    std::vector<WeightSlot> _weightSlots; // in .msnhbin order
    std::vector<MsnhB200Op> _ops;         // what lower() handed to the kernel library
    size_t _totalWeights = 0;
    bool _weightsLoaded = false;
    int _lastOp = -1, _collectOp = -1;
    float _confThresh = 0.f, _nmsThresh = 0.f; bool _useSoftNms = false;
    int _lastW = 0, _lastH = 0, _lastC = 0; size_t _lastNum = 0;
    float _gpuInferenceTime = 0.f;
    bool _saveLayerOutput = false, _saveLayerWeights = false;
    bool _deviceNms = false;
    bool _packCache = false, _usedPack = false;
    std::string _detail;
    std::vector<float> _candRows; std::vector<int> _candCounts; int _maxRows = 0;
};

}  // namespace Msnhnet
