#include "msnh_format.h"

#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

namespace Msnhnet {
namespace {

struct Node {
    std::string key, value;
    int line = 0;
    std::vector<Node> children;
};

std::string trim(const std::string &s) {
    size_t b = s.find_first_not_of(" \t\r\n");
    if (b == std::string::npos) return "";
    size_t e = s.find_last_not_of(" \t\r\n");
    return s.substr(b, e - b + 1);
}

// Indentation tree of "key: value" lines. Comments (#...) and blank lines are dropped; a UTF-8 BOM
// at the start of the file is skipped.
std::vector<Node> parseTree(const std::string &text) {
    struct Item { int indent; Node node; };
    std::vector<Item> flat;
    std::istringstream in(text);
    std::string raw;
    int lineNo = 0;
    while (std::getline(in, raw)) {
        ++lineNo;
        if (lineNo == 1 && raw.size() >= 3 && static_cast<unsigned char>(raw[0]) == 0xEF) raw = raw.substr(3);
        size_t hash = raw.find('#');
        if (hash != std::string::npos) raw = raw.substr(0, hash);
        if (trim(raw).empty()) continue;
        int indent = 0;
        while (indent < static_cast<int>(raw.size()) && (raw[indent] == ' ' || raw[indent] == '\t')) ++indent;
        std::string body = trim(raw);
        size_t colon = body.find(':');
        if (colon == std::string::npos) MSNH_THROW("line " + std::to_string(lineNo) + ": expected 'key: value'");
        Item it;
        it.indent = indent;
        it.node.key = trim(body.substr(0, colon));
        it.node.value = trim(body.substr(colon + 1));
        it.node.line = lineNo;
        flat.push_back(it);
    }
    // fold by indentation
    std::vector<Node> roots;
    size_t pos = 0;
    struct Builder {
        const std::vector<Item> &flat;
        void build(size_t &pos, int indent, std::vector<Node> &out) {
            while (pos < flat.size() && flat[pos].indent == indent) {
                Node n = flat[pos].node;
                ++pos;
                if (pos < flat.size() && flat[pos].indent > indent) build(pos, flat[pos].indent, n.children);
                out.push_back(std::move(n));
            }
            if (pos < flat.size() && flat[pos].indent > indent)
                MSNH_THROW("line " + std::to_string(flat[pos].node.line) + ": inconsistent indentation");
        }
    } b{flat};
    if (!flat.empty()) {
        if (flat[0].indent != 0) MSNH_THROW("first node must not be indented");
        b.build(pos, 0, roots);
        if (pos != flat.size()) MSNH_THROW("line " + std::to_string(flat[pos].node.line) + ": inconsistent indentation");
    }
    return roots;
}

int toInt(const Node &n, const char *ctx) {
    char *end = nullptr;
    long v = std::strtol(n.value.c_str(), &end, 10);
    if (n.value.empty() || *end != '\0') MSNH_THROW(std::string("[") + ctx + "] " + n.key + " can't convert to int (line " + std::to_string(n.line) + ")");
    return static_cast<int>(v);
}
float toFloat(const std::string &s, const Node &n, const char *ctx) {
    char *end = nullptr;
    std::string t = trim(s);
    float v = std::strtof(t.c_str(), &end);
    if (t.empty() || *end != '\0') MSNH_THROW(std::string("[") + ctx + "] " + n.key + " can't convert to float (line " + std::to_string(n.line) + ")");
    return v;
}
std::vector<std::string> splitComma(const std::string &s) {
    std::vector<std::string> out;
    std::string cur;
    for (char c : s) { if (c == ',') { out.push_back(trim(cur)); cur.clear(); } else cur += c; }
    if (!trim(cur).empty() || !out.empty()) out.push_back(trim(cur));
    return out;
}
void parseActivation(const Node &n, LayerDesc &d, const char *ctx) {
    std::vector<std::string> parts = splitComma(n.value);
    if (parts.empty()) MSNH_THROW(std::string("[") + ctx + "] activation is empty (line " + std::to_string(n.line) + ")");
    d.activation = parts[0];
    d.actParams.clear();
    for (size_t i = 1; i < parts.size(); ++i) d.actParams.push_back(toFloat(parts[i], n, ctx));
}
void parseLayerList(const Node &n, LayerDesc &d, int selfIndex, const char *ctx) {
    for (const std::string &p : splitComma(n.value)) {
        Node t = n; t.value = p;
        int idx = toInt(t, ctx);
        if (idx < 0) idx += selfIndex;   // relative to this layer (src/io/MsnhParser.cpp:2162-2165)
        d.layers.push_back(idx);
    }
}

LayerDesc parseLayer(const Node &n, int selfIndex);

void parseSeq(const std::vector<Node> &nodes, std::vector<LayerDesc> &out, const char *ctx, bool allowEmpty) {
    for (const Node &c : nodes) {
        static const char *ok[] = {"conv", "batchnorm", "maxpool", "localavgpool", "globalavgpool", "connect", "padding", "act", "empty"};
        bool found = false;
        for (const char *k : ok) if (c.key == k) found = true;
        if (!found || (c.key == "empty" && !allowEmpty))
            MSNH_THROW(std::string("[") + ctx + "] unsupported child '" + c.key + "' (line " + std::to_string(c.line) + ")");
        out.push_back(parseLayer(c, -1));
    }
}

LayerDesc parseLayer(const Node &n, int selfIndex) {
    LayerDesc d;
    d.line = n.line;
    const std::string &k = n.key;
    auto bad = [&](const Node &c) { MSNH_THROW("[" + k + "] unknown key '" + c.key + "' (line " + std::to_string(c.line) + ")"); };
    int kSize = -1, stride = -1, padding = -1, dilation = -1;
    int kx = -1, ky = -1, sx = -1, sy = -1, px = -1, py = -1, dx = -1, dy = -1;
    float scale = -1.f;
    auto geometry = [&](const Node &c) -> bool {
        const char *ctx = k.c_str();
        if (c.key == "kSize") kSize = toInt(c, ctx); else if (c.key == "kSizeX") kx = toInt(c, ctx); else if (c.key == "kSizeY") ky = toInt(c, ctx);
        else if (c.key == "stride") stride = toInt(c, ctx); else if (c.key == "strideX") sx = toInt(c, ctx); else if (c.key == "strideY") sy = toInt(c, ctx);
        else if (c.key == "padding") padding = toInt(c, ctx); else if (c.key == "paddingX") px = toInt(c, ctx); else if (c.key == "paddingY") py = toInt(c, ctx);
        else if (c.key == "dilation") dilation = toInt(c, ctx); else if (c.key == "dilationX") dx = toInt(c, ctx); else if (c.key == "dilationY") dy = toInt(c, ctx);
        else return false;
        return true;
    };
    auto finishGeometry = [&]() {
        // X/Y variants win over the square value; square defaults: kSize 1, stride 1, padding 0, dilation 1
        d.kSizeX = kx > 0 ? kx : (kSize > 0 ? kSize : 1);      d.kSizeY = ky > 0 ? ky : (kSize > 0 ? kSize : 1);
        d.strideX = sx > 0 ? sx : (stride > 0 ? stride : 1);   d.strideY = sy > 0 ? sy : (stride > 0 ? stride : 1);
        d.paddingX = px >= 0 ? px : (padding >= 0 ? padding : 0); d.paddingY = py >= 0 ? py : (padding >= 0 ? padding : 0);
        d.dilationX = dx > 0 ? dx : (dilation > 0 ? dilation : 1); d.dilationY = dy > 0 ? dy : (dilation > 0 ? dilation : 1);
    };

    if (k == "conv") {
        d.kind = LayerKind::Conv;
        for (const Node &c : n.children) {
            if (geometry(c)) continue;
            if (c.key == "batchNorm") d.batchNorm = toInt(c, "conv"); else if (c.key == "filters") d.filters = toInt(c, "conv");
            else if (c.key == "groups") d.groups = toInt(c, "conv"); else if (c.key == "useBias") d.useBias = toInt(c, "conv");
            else if (c.key == "eps") d.eps = toFloat(c.value, c, "conv"); else if (c.key == "antialiasing") { if (toInt(c, "conv") != 0) MSNH_THROW("[conv] antialiasing is not supported"); }
            else if (c.key == "activation") parseActivation(c, d, "conv"); else bad(c);
        }
        finishGeometry();
    } else if (k == "batchnorm") {
        d.kind = LayerKind::BatchNorm;
        for (const Node &c : n.children) {
            if (c.key == "activation") parseActivation(c, d, "batchnorm"); else if (c.key == "eps") d.eps = toFloat(c.value, c, "batchnorm"); else bad(c);
        }
    } else if (k == "act") {
        d.kind = LayerKind::Act;
        for (const Node &c : n.children) { if (c.key == "activation") parseActivation(c, d, "act"); else bad(c); }
    } else if (k == "maxpool" || k == "localavgpool") {
        d.kind = k == "maxpool" ? LayerKind::MaxPool : LayerKind::LocalAvgPool;
        for (const Node &c : n.children) {
            if (geometry(c)) continue;
            if (c.key == "ceilMode") d.ceilMode = toInt(c, k.c_str());
            else if (c.key == "maxPoolDepth") d.maxPoolDepth = toInt(c, k.c_str());
            else if (c.key == "outChannels") d.outChannels = toInt(c, k.c_str());
            else bad(c);
        }
        finishGeometry();
    } else if (k == "globalavgpool") {
        d.kind = LayerKind::GlobalAvgPool;
        if (!n.children.empty()) bad(n.children[0]);
    } else if (k == "padding") {
        d.kind = LayerKind::Padding;
        for (const Node &c : n.children) {
            if (c.key == "top") d.top = toInt(c, "padding"); else if (c.key == "down") d.down = toInt(c, "padding");
            else if (c.key == "left") d.left = toInt(c, "padding"); else if (c.key == "right") d.right = toInt(c, "padding");
            else if (c.key == "paddingVal") d.paddingVal = toFloat(c.value, c, "padding"); else bad(c);
        }
    } else if (k == "upsample") {
        d.kind = LayerKind::UpSample;
        float scx = -1.f, scy = -1.f;
        for (const Node &c : n.children) {
            if (c.key == "stride") stride = toInt(c, "upsample"); else if (c.key == "strideX") sx = toInt(c, "upsample"); else if (c.key == "strideY") sy = toInt(c, "upsample");
            else if (c.key == "scale") scale = toFloat(c.value, c, "upsample"); else if (c.key == "scaleX") scx = toFloat(c.value, c, "upsample");
            else if (c.key == "scaleY") scy = toFloat(c.value, c, "upsample"); else if (c.key == "type") d.upsampleType = c.value;
            else if (c.key == "alignCorners") d.alignCorners = toInt(c, "upsample"); else bad(c);
        }
        d.strideX = sx > 0 ? sx : (stride > 0 ? stride : 1); d.strideY = sy > 0 ? sy : (stride > 0 ? stride : 1);
        d.scaleX = scx > 0 ? scx : (scale > 0 ? scale : 1.f); d.scaleY = scy > 0 ? scy : (scale > 0 ? scale : 1.f);
        // UpSampleParams::getUnsampleTypeFromStr (src/io/MsnhParser.cpp): nearest | bilinear
        if (d.upsampleType != "nearest" && d.upsampleType != "bilinear") MSNH_THROW("[upsample] type '" + d.upsampleType + "' is not supported (line " + std::to_string(n.line) + ")");
    } else if (k == "deconv") {
        // keys of Parser::parseDeConvParams (src/io/MsnhParser.cpp:1299-1395)
        d.kind = LayerKind::DeConv;
        for (const Node &c : n.children) {
            if (c.key == "dilation" || c.key == "dilationX" || c.key == "dilationY") bad(c);
            if (geometry(c)) continue;
            if (c.key == "filters") d.filters = toInt(c, "deconv"); else if (c.key == "groups") d.groups = toInt(c, "deconv");
            else if (c.key == "useBias") d.useBias = toInt(c, "deconv"); else if (c.key == "activation") parseActivation(c, d, "deconv"); else bad(c);
        }
        finishGeometry();
    } else if (k == "clip") {
        d.kind = LayerKind::Clip;
        for (const Node &c : n.children) {
            if (c.key == "min") d.clipMin = toFloat(c.value, c, "clip"); else if (c.key == "max") d.clipMax = toFloat(c.value, c, "clip"); else bad(c);
        }
        if (d.clipMin > d.clipMax) MSNH_THROW("[clip] min should > max [min:max]=[" + std::to_string(d.clipMin) + ":" + std::to_string(d.clipMax) + "]");
    } else if (k == "permute" || k == "view") {
        d.kind = k == "permute" ? LayerKind::Permute : LayerKind::View;
        if (k == "view") d.dim[0] = d.dim[1] = d.dim[2] = -1;    // ViewParams defaults (include/Msnhnet/io/MsnhParser.h:59-61)
        for (const Node &c : n.children) {
            if (c.key == "dim0") d.dim[0] = toInt(c, k.c_str()); else if (c.key == "dim1") d.dim[1] = toInt(c, k.c_str());
            else if (c.key == "dim2") d.dim[2] = toInt(c, k.c_str()); else bad(c);
        }
    } else if (k == "pixshf") {
        d.kind = LayerKind::PixShuffle;
        for (const Node &c : n.children) { if (c.key == "factor") d.factor = toInt(c, "pixshf"); else bad(c); }
    } else if (k == "reduction") {
        d.kind = LayerKind::Reduction;
        for (const Node &c : n.children) {
            if (c.key == "axis") {
                d.axis = toInt(c, "reduction");
                if (d.axis < -1 || d.axis > 2) MSNH_THROW("[reduction] axis must be 0/1/2 : " + std::to_string(d.axis) + " is error");
            } else if (c.key == "type") {
                if (c.value == "sum") d.reduceMean = false; else if (c.value == "mean") d.reduceMean = true;
                else MSNH_THROW("[reduction] " + c.value + " is not supported");
            } else bad(c);
        }
    } else if (k == "route") {
        d.kind = LayerKind::Route;
        for (const Node &c : n.children) {
            if (c.key == "layers") parseLayerList(c, d, selfIndex, "route"); else if (c.key == "groups") d.routeGroups = toInt(c, "route");
            else if (c.key == "groupsId") d.routeGroupsId = toInt(c, "route"); else if (c.key == "addModel") d.addModel = toInt(c, "route");
            else if (c.key == "activation") parseActivation(c, d, "route"); else bad(c);
        }
        if (d.layers.empty()) MSNH_THROW("[route] needs layers (line " + std::to_string(n.line) + ")");
    } else if (k == "varop") {
        d.kind = LayerKind::VarOp;
        for (const Node &c : n.children) {
            if (c.key == "layers") parseLayerList(c, d, selfIndex, "varop"); else if (c.key == "type") d.varOpType = c.value;
            else if (c.key == "constVal") d.constVal = toFloat(c.value, c, "varop"); else bad(c);
        }
    } else if (k == "slice") {
        d.kind = LayerKind::Slice;
        for (const Node &c : n.children) {
            bool hit = false;
            for (int a = 0; a < 3; ++a) {
                if (c.key == "start" + std::to_string(a)) { d.start[a] = toInt(c, "slice"); hit = true; }
                if (c.key == "step" + std::to_string(a)) { d.step[a] = toInt(c, "slice"); hit = true; }
            }
            if (!hit) bad(c);
        }
    } else if (k == "connect") {
        d.kind = LayerKind::Connect;
        for (const Node &c : n.children) {
            if (c.key == "output") d.output = toInt(c, "connect"); else if (c.key == "batchNorm") d.batchNorm = toInt(c, "connect");
            else if (c.key == "useBias") d.useBias = toInt(c, "connect"); else if (c.key == "bnEps") d.eps = toFloat(c.value, c, "connect");
            else if (c.key == "activation") parseActivation(c, d, "connect"); else bad(c);
        }
    } else if (k == "softmax") {
        d.kind = LayerKind::SoftMax;
        for (const Node &c : n.children) {
            if (c.key == "groups") d.softmaxGroups = toInt(c, "softmax"); else if (c.key == "temperature") d.temperature = toFloat(c.value, c, "softmax"); else bad(c);
        }
    } else if (k == "empty") {
        d.kind = LayerKind::Empty;
    } else if (k == "yolo") {
        d.kind = LayerKind::Yolo;
        for (const Node &c : n.children) {
            if (c.key == "anchors") { for (const std::string &p : splitComma(c.value)) d.anchors.push_back(toFloat(p, c, "yolo")); }
            else if (c.key == "classNum") d.classNum = toInt(c, "yolo"); else if (c.key == "yoloType") d.yoloType = c.value; else bad(c);
        }
        if (d.anchors.size() != 6) MSNH_THROW("[yolo] anchors must hold 3 w,h pairs (line " + std::to_string(n.line) + ")");
    } else if (k == "yoloout") {
        d.kind = LayerKind::YoloOut;
        for (const Node &c : n.children) {
            if (c.key == "layers") parseLayerList(c, d, selfIndex, "yoloout"); else if (c.key == "confThresh") d.confThresh = toFloat(c.value, c, "yoloout");
            else if (c.key == "nmsThresh") d.nmsThresh = toFloat(c.value, c, "yoloout"); else if (c.key == "useSoftNms") d.useSoftNms = toInt(c, "yoloout");
            else if (c.key == "yoloType") d.yoloType = c.value; else bad(c);
        }
    } else if (k == "resblock") {
        d.kind = LayerKind::ResBlock;
        std::vector<Node> seq;
        for (const Node &c : n.children) {
            if (c.key == "size") continue;
            if (c.key == "activation") { parseActivation(c, d, "resblock"); continue; }
            seq.push_back(c);
        }
        parseSeq(seq, d.chain, "resblock", false);
    } else if (k == "res2block") {
        d.kind = LayerKind::Res2Block;
        d.branches.resize(2);
        for (const Node &c : n.children) {
            if (c.key == "size") continue;
            if (c.key == "activation") { parseActivation(c, d, "res2block"); continue; }
            if (c.key == "base") parseSeq(c.children, d.branches[0], "res2block", false);
            else if (c.key == "branch") parseSeq(c.children, d.branches[1], "res2block", false);
            else bad(c);
        }
    } else if (k == "addblock" || k == "concatblock") {
        d.kind = k == "addblock" ? LayerKind::AddBlock : LayerKind::ConcatBlock;
        for (const Node &c : n.children) {
            if (c.key == "size") continue;
            if (c.key == "activation") { parseActivation(c, d, k.c_str()); continue; }
            if (c.key == "branch") { d.branches.emplace_back(); parseSeq(c.children, d.branches.back(), k.c_str(), true); }
            else bad(c);
        }
        if (d.branches.empty()) MSNH_THROW("[" + k + "] needs at least one branch (line " + std::to_string(n.line) + ")");
    } else {
        MSNH_THROW("layer type '" + k + "' is not supported by this backend (line " + std::to_string(n.line) + ")");
    }
    return d;
}

}  // namespace

NetDesc parseMsnhNet(const std::string &text) {
    std::vector<Node> roots = parseTree(text);
    if (roots.empty() || roots[0].key != "config") MSNH_THROW("first node must be config");
    NetDesc net;
    for (const Node &c : roots[0].children) {
        if (c.key == "batch") net.batch = toInt(c, "config"); else if (c.key == "width") net.width = toInt(c, "config");
        else if (c.key == "height") net.height = toInt(c, "config"); else if (c.key == "channels") net.channels = toInt(c, "config");
        else MSNH_THROW("[config] unknown key '" + c.key + "'");
    }
    if (net.batch < 1 || net.width < 1 || net.height < 1 || net.channels < 1) MSNH_THROW("[config] batch/width/height/channels must be positive");
    for (size_t i = 1; i < roots.size(); ++i) {
        const Node &n = roots[i];
        int size = 1;
        if (n.key == "resblock" || n.key == "res2block" || n.key == "addblock" || n.key == "concatblock")
            for (const Node &c : n.children) if (c.key == "size") size = toInt(c, n.key.c_str());
        if (size < 1) MSNH_THROW("[" + n.key + "] size must be >= 1");
        for (int r = 0; r < size; ++r) net.layers.push_back(parseLayer(n, static_cast<int>(net.layers.size())));
    }
    if (net.layers.empty()) MSNH_THROW("net has no layers");
    return net;
}

NetDesc readMsnhNet(const std::string &path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) MSNH_THROW("can not open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    return parseMsnhNet(ss.str());
}

std::vector<float> readMsnhBin(const std::string &path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) MSNH_THROW("can not open " + path);
    const std::streamoff bytes = f.tellg();
    if (bytes % 4 != 0) MSNH_THROW("msnhbin file size is not a multiple of 4: " + path);
    std::vector<float> v(static_cast<size_t>(bytes / 4));
    f.seekg(0);
    f.read(reinterpret_cast<char *>(v.data()), bytes);
    if (!f) MSNH_THROW("short read on " + path);
    return v;
}

}  // namespace Msnhnet
