// Test infrastructure: drives the reference's own image preprocessing (src/utils/MsnhCVUtil.cpp on the
// reference's Mat, src/cv/MsnhCVMat*.cpp) exactly as its C API does for a raw 8-bit image
// (src/c_api/MsnhnetLib.cpp:540-620 runClassifyList, :754-778 runYoloList, the variant without OpenCV).
// Usage: ref_prep <mode> <in.u8> <w> <h> <c> <outW> <outH> <swapRGB> <out.f32> [mean0 mean1 mean2 std0 std1 std2]
//   mode: yolo | c1 | c3 | googlenet | padzero | caffe | transformed
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include "Msnhnet/cv/MsnhCVMat.h"
#include "Msnhnet/cv/MsnhCVMatOp.h"
#include "Msnhnet/utils/MsnhCVUtil.h"

// The Mat source refers to this callback of the video writer (src/cv/MsnhCVVideo.cpp:646, a file that needs a
// camera stack); it only serves JPEG/PNG encoding, which this driver never reaches.
namespace Msnhnet { void bufferFromCallback(void *, void *, int) {} }

int main(int argc, char **argv) {
    if (argc < 10) { std::fprintf(stderr, "usage: see source header\n"); return 2; }
    const std::string mode = argv[1];
    const int w = std::atoi(argv[3]), h = std::atoi(argv[4]), c = std::atoi(argv[5]);
    const int ow = std::atoi(argv[6]), oh = std::atoi(argv[7]), swapRGB = std::atoi(argv[8]);
    std::vector<unsigned char> in(static_cast<size_t>(w) * h * c);
    FILE *f = std::fopen(argv[2], "rb");
    if (!f || std::fread(in.data(), 1, in.size(), f) != in.size()) { std::fprintf(stderr, "cannot read %s\n", argv[2]); return 2; }
    std::fclose(f);
    try {
        Msnhnet::Mat inMat(w, h, c == 1 ? Msnhnet::MAT_GRAY_U8 : Msnhnet::MAT_RGB_U8, in.data());
        if (!swapRGB) Msnhnet::MatOp::cvtColor(inMat, inMat, Msnhnet::CvtColorType::CVT_RGB2BGR);
        std::vector<float> img;
        if (mode == "yolo" || mode == "padzero") img = Msnhnet::CVUtil::getPaddingZeroF32C3(inMat, {ow, oh});
        else if (mode == "c1") img = Msnhnet::CVUtil::getImgDataF32C1(inMat, {ow, oh});
        else if (mode == "c3") img = Msnhnet::CVUtil::getImgDataF32C3(inMat, {ow, oh});
        else if (mode == "googlenet") img = Msnhnet::CVUtil::getGoogLenetF32C3(inMat, {ow, oh});
        else if (mode == "caffe") img = Msnhnet::CVUtil::getCaffeModeF32C3(inMat, {ow, oh});
        else if (mode == "transformed") {
            if (argc < 16) { std::fprintf(stderr, "transformed needs mean and std\n"); return 2; }
            img = Msnhnet::CVUtil::getTransformedF32C3(inMat, {ow, oh}, {(float)std::atof(argv[10]), (float)std::atof(argv[11]), (float)std::atof(argv[12])},
                                                       {(float)std::atof(argv[13]), (float)std::atof(argv[14]), (float)std::atof(argv[15])});
        } else { std::fprintf(stderr, "unknown mode\n"); return 2; }
        f = std::fopen(argv[9], "wb");
        std::fwrite(img.data(), sizeof(float), img.size(), f);
        std::fclose(f);
        std::printf("%zu\n", img.size());
    } catch (Msnhnet::Exception &ex) {
        std::printf("EXCEPTION %s\n", ex.what());
        return 1;
    }
    return 0;
}
