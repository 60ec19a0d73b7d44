// Test infrastructure, not product code: a small command-line driver around the UNMODIFIED
// reference CPU path (Msnhnet::NetBuilder, include/Msnhnet/net/MsnhNetBuilder.h:48-117), built by
// oracle/Makefile from the reference sources where they lie. It is the checker and the timed CPU
// baseline; nothing in the product links or executes it.
//
//   ref_driver run    <net.msnhnet> <weights.msnhbin> <input.f32> <outdir> [avx=0|1] [dump=0|1]
//       One CPU forward of a batch-1 CHW float image. Writes <outdir>/final.f32 (classifier
//       logits) or <outdir>/boxes.f32 (rows x,y,w,h,conf,bestClsConf,bestClsIdx) and, with
//       dump=1, <outdir>/layer_<i>.f32 for every top-level layer (NCHW, as the reference's
//       setSaveLayerOutput does in src/net/MsnhNetBuilder.cpp:704-720, but binary).
//   ref_driver time   <net.msnhnet> <weights.msnhbin> <input.f32> <warmup> <iters> [avx=1]
//       Prints "ms_per_image <mean> threads <n> iters <k>" for runYolo / runClassify, then
//       "conv_share <fraction> layer_ms_total <ms>" from the per-layer timers of the last image.
//   ref_driver layout <net.msnhnet>
//       Prints one line per top-level layer: index, type name, weight count, output C H W.
// Standard headers first: the access override below must not reach them.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>
#include <algorithm>
#include <map>
#include <memory>
#include <sstream>
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
#include <cassert>
#include <immintrin.h>
#define private public   // the per-layer loop needs NetBuilder::_netState (test infra only)
#include "Msnhnet/net/MsnhNetBuilder.h"
#undef private
#ifdef _OPENMP
#include <omp.h>
#endif

using namespace Msnhnet;

static std::vector<float> readF32(const std::string &path)
{
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) { std::fprintf(stderr, "cannot open %s\n", path.c_str()); std::exit(2); }
    size_t n = static_cast<size_t>(f.tellg());
    f.seekg(0);
    std::vector<float> v(n / 4);
    f.read(reinterpret_cast<char *>(v.data()), static_cast<std::streamsize>(n));
    return v;
}

static void writeF32(const std::string &path, const float *p, size_t n)
{
    std::ofstream f(path, std::ios::binary);
    f.write(reinterpret_cast<const char *>(p), static_cast<std::streamsize>(n * 4));
}

static bool isYolo(NetBuilder &nb)
{
    Network *net = nb.getNet();
    return net->layers.back()->type() == LayerType::YOLO_OUT;
}

static int cmdRun(int argc, char **argv)
{
    if (argc < 6) return 1;
    bool avx  = argc > 6 ? std::atoi(argv[6]) != 0 : false;
    bool dump = argc > 7 ? std::atoi(argv[7]) != 0 : false;
    std::string outdir = argv[5];
    NetBuilder nb;
    nb.buildNetFromMsnhNet(argv[2]);
    nb.loadWeightsFromMsnhBin(argv[3]);
    BaseLayer::supportAvx = avx;
    std::vector<float> img = readF32(argv[4]);
    Network *net = nb.getNet();
    NetworkState *st = nb._netState;
    if (net->layers[0]->getInputNum() != static_cast<int>(img.size()))
    {
        std::fprintf(stderr, "input size %zu, net wants %d\n", img.size(), net->layers[0]->getInputNum());
        return 3;
    }
    // Same loop as NetBuilder::runYolo / runClassify (src/net/MsnhNetBuilder.cpp:665-817).
    st->input    = img.data();
    st->inputNum = static_cast<int>(img.size());
    for (size_t i = 0; i < net->layers.size(); ++i)
    {
        net->layers[i]->forward(*st);
        if (net->layers[i]->getMemReUse() == 0) st->input = net->layers[i]->getOutput();
        st->inputNum = net->layers[i]->getOutputNum();
        if (dump && net->layers[i]->type() != LayerType::YOLO_OUT)
        {
            const float *p = net->layers[i]->getMemReUse() == 1 ? st->getInput() : st->input;
            writeF32(outdir + "/layer_" + std::to_string(i) + ".f32", p, static_cast<size_t>(st->inputNum));
        }
    }
    if (isYolo(nb))
    {
        auto &boxes = reinterpret_cast<YoloOutLayer *>(net->layers.back())->finalOut;
        std::vector<float> rows;
        for (auto &b : boxes[0])
        {
            rows.push_back(b.xywhBox.x); rows.push_back(b.xywhBox.y);
            rows.push_back(b.xywhBox.w); rows.push_back(b.xywhBox.h);
            rows.push_back(b.conf);      rows.push_back(b.bestClsConf);
            rows.push_back(static_cast<float>(b.bestClsIdx));
        }
        writeF32(outdir + "/boxes.f32", rows.data(), rows.size());
        std::printf("boxes %zu\n", boxes[0].size());
    }
    else
    {
        const float *p = net->layers.back()->getMemReUse() == 1 ? st->getInput() : st->input;
        writeF32(outdir + "/final.f32", p, static_cast<size_t>(st->inputNum));
        std::printf("final %d\n", st->inputNum);
    }
    return 0;
}

static int cmdTime(int argc, char **argv)
{
    if (argc < 7) return 1;
    int warm = std::atoi(argv[5]), iters = std::atoi(argv[6]);
    bool avx = argc > 7 ? std::atoi(argv[7]) != 0 : true;
    NetBuilder nb;
    nb.buildNetFromMsnhNet(argv[2]);
    nb.loadWeightsFromMsnhBin(argv[3]);
    BaseLayer::supportAvx = avx;
    std::vector<float> img = readF32(argv[4]);
    bool yolo = isYolo(nb);
    for (int i = 0; i < warm; ++i) { if (yolo) nb.runYolo(img); else nb.runClassify(img); }
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; ++i) { if (yolo) nb.runYolo(img); else nb.runClassify(img); }
    auto t1 = std::chrono::steady_clock::now();
    double ms = std::chrono::duration<double, std::milli>(t1 - t0).count() / (iters > 0 ? iters : 1);
    int threads = 1;
#ifdef _OPENMP
    threads = omp_get_max_threads();
#endif
    std::printf("ms_per_image %.4f threads %d iters %d\n", ms, threads, iters);
    // Where the time of the last image went, from the reference's own per-layer timers (what getTimeDetail() prints,
    // src/net/MsnhNetBuilder.cpp:1184-1201): the share of the conv layers and of the block layers, which are conv chains.
    Network *net = nb.getNet();
    float total = 0.f, conv = 0.f;
    for (size_t i = 0; i < net->layers.size(); ++i)
    {
        const float t = net->layers[i]->getForwardTime();
        const std::string name = net->layers[i]->getLayerName();
        total += t;
        if (name.find("Conv") != std::string::npos || name.find("Block") != std::string::npos) conv += t;
    }
    if (total > 0.f) std::printf("conv_share %.3f layer_ms_total %.2f\n", conv / total, total);
    return 0;
}

static int cmdLayout(int argc, char **argv)
{
    if (argc < 3) return 1;
    NetBuilder::setPreviewMode(true);
    NetBuilder nb;
    nb.buildNetFromMsnhNet(argv[2]);
    Network *net = nb.getNet();
    for (size_t i = 0; i < net->layers.size(); ++i)
    {
        BaseLayer *l = net->layers[i];
        std::printf("%zu %s %zu %d %d %d\n", i, l->getLayerName().c_str(), static_cast<size_t>(l->getNumWeights()),
                    l->getOutChannel(), l->getOutHeight(), l->getOutWidth());
    }
    return 0;
}

int main(int argc, char **argv)
{
    try
    {
        if (argc >= 2 && !std::strcmp(argv[1], "run"))    return cmdRun(argc, argv);
        if (argc >= 2 && !std::strcmp(argv[1], "time"))   return cmdTime(argc, argv);
        if (argc >= 2 && !std::strcmp(argv[1], "layout")) return cmdLayout(argc, argv);
    }
    catch (Exception &e)
    {
        std::fprintf(stderr, "reference exception: %s\n", e.what());
        return 4;
    }
    std::fprintf(stderr, "usage: ref_driver run|time|layout ...\n");
    return 1;
}
