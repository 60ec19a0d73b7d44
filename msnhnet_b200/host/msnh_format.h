// The two file formats of the boundary, read exactly as the reference reads them:
//   .msnhnet  order-significant YAML-style topology (duplicate keys are distinct nodes); grammar and
//             defaults follow Parser::readCfg and the *Params structs
//             (src/io/MsnhParser.cpp:140-682, include/Msnhnet/io/MsnhParser.h:16-565)
//   .msnhbin  headerless little-endian float32 blob (src/io/MsnhParser.cpp:684-726)
#pragma once
#include <stdexcept>
#include <string>
#include <vector>

namespace Msnhnet {

// Same role as Msnhnet::Exception (include/Msnhnet/utils/MsnhException.h): config / shape / size errors.
class Exception : public std::runtime_error {
public:
    Exception(int code, const std::string &msg, const char *file, int line, const char *func)
        : std::runtime_error(msg + " [" + file + ":" + std::to_string(line) + " " + func + "]"), errCode(code) {}
    int errCode;
};
#define MSNH_THROW(msg) throw ::Msnhnet::Exception(1, (msg), __FILE__, __LINE__, __FUNCTION__)

enum class LayerKind {
    Config, Conv, BatchNorm, Act, MaxPool, LocalAvgPool, GlobalAvgPool, Padding, UpSample, Route, VarOp, Slice,
    Connect, SoftMax, ResBlock, Res2Block, AddBlock, ConcatBlock, Yolo, YoloOut, Empty,
    DeConv, Clip, Permute, PixShuffle, View, Reduction
};

struct LayerDesc {
    LayerKind kind = LayerKind::Empty;
    int line = 0;                       // line of the node in the file (error messages)
    // conv / pools / connect
    int batchNorm = 0, filters = 1, groups = 1, useBias = 1;
    int kSizeX = 1, kSizeY = 1, strideX = 1, strideY = 1, paddingX = 0, paddingY = 0, dilationX = 1, dilationY = 1;
    int ceilMode = 0, maxPoolDepth = 0, outChannels = 1;   // MaxPoolParams (include/Msnhnet/io/MsnhParser.h)
    int output = 0;                     // connect
    float eps = 1e-5f;
    std::string activation = "none";    // name as written; unknown names mean relu (src/layers/MsnhActivations.cpp:29)
    std::vector<float> actParams;
    // padding
    int top = 0, down = 0, left = 0, right = 0; float paddingVal = 0.f;
    // upsample
    std::string upsampleType = "nearest"; float scaleX = 1.f, scaleY = 1.f; int alignCorners = 0;
    // route / varop / yoloout
    std::vector<int> layers;            // absolute indices (negative ones already resolved)
    int routeGroups = 1, routeGroupsId = 0, addModel = 0;
    std::string varOpType = "add"; float constVal = 0.f;
    // slice
    int start[3] = {0, 0, 0}, step[3] = {1, 1, 1};
    // clip (defaults of ClipParams, include/Msnhnet/io/MsnhParser.h:83-84)
    float clipMin = -3.402823466e+38f, clipMax = 3.402823466e+38f;
    // permute: dim[k] = input axis (0 C, 1 H, 2 W) that becomes output axis k; view: dim0/1/2 = the reference's
    // outWidth / outHeight / outChannel arguments (src/net/MsnhNetBuilder.cpp:478-482); pixshf: factor
    int dim[3] = {0, 1, 2}; int factor = 0;
    // reduction
    int axis = -1; bool reduceMean = false;
    // softmax
    int softmaxGroups = 1; float temperature = 1.f;
    // yolo / yoloout
    std::vector<float> anchors; int classNum = 1; std::string yoloType = "yolov3";
    float confThresh = 0.f, nmsThresh = 0.f; int useSoftNms = 0;
    // blocks
    std::vector<LayerDesc> chain;                   // resblock
    std::vector<std::vector<LayerDesc>> branches;   // res2block: {base, branch}; addblock / concatblock
};

struct NetDesc {
    int batch = 1, width = 0, height = 0, channels = 0;
    std::vector<LayerDesc> layers;      // block nodes with size: n already expanded to n entries
};

// Throws Msnhnet::Exception on unknown keys / bad values, like the reference parser.
NetDesc parseMsnhNet(const std::string &text);
NetDesc readMsnhNet(const std::string &path);
std::vector<float> readMsnhBin(const std::string &path);

}  // namespace Msnhnet
