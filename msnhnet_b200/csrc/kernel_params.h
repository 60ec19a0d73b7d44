// Launch parameters of the kernels in this folder: the structs a kernel takes by value and the constants that size its
// launch. Plain host-compilable declarations (no device code), so that the plan compiler's translation units can fill
// them in without compiling the kernels; the kernel headers include this file for the same definitions.
#pragma once
#include <cstddef>
#include <stdint.h>
#include "../../include/msnh_b200.h"

#ifdef __CUDACC__
#define MSNH_HOST_DEVICE __host__ __device__
#else
#define MSNH_HOST_DEVICE
#endif

namespace msnh {

// ---- tensors ----------------------------------------------------------------------------------------------------------
// A channels-last tensor (or a channel slice of one): element (n,h,w,c) lives at
// ptr[((n*H + h)*W + w)*ldc + c]. `ptr` already includes the slice's channel offset.
struct TView {
    void *ptr;
    int   N, H, W, C;
    int   ldc;
    int   tf32;   // fp32 tensors only: round values to tf32 (nearest) when storing, because a
                  // tensor-core conv reads this tensor and the hardware would otherwise truncate
};

// Device error flag codes written by kernels whose bounded waits ran out.
enum { DEV_ERR_NONE = 0, DEV_ERR_WAIT_FULL = 1, DEV_ERR_WAIT_EMPTY = 2, DEV_ERR_WAIT_ACC_FULL = 3,
       DEV_ERR_WAIT_ACC_EMPTY = 4, DEV_ERR_TMEM_ALLOC = 5 };


// ---- tensor-core convolution (conv_umma.cuh) --------------------------------------------------------------------------
constexpr int kUmmaM          = 128;  // output pixels per tile (TMEM lanes)
constexpr int kUmmaThreads    = 576;  // warp 0: TMA producer, warp 1: MMA issuer, warps 2-17: epilogue (two teams of 8)
constexpr int kUmmaMaxStages  = 8;
constexpr int kUmmaMaxAccStages = 8; // accumulator ring in TMEM: 2, 4 or 8 stages, as many as fit in 512 columns
constexpr uint32_t kStageCBytes = 128 * 128;   // one output staging slab: 128 rows x up to 128 bytes

enum { A_MODE_LINEAR = 0,   // 2-D map (C, pixels), 1x1 stride-1 pad-0 convs and connected layers
       A_MODE_IM2COL = 1 }; // 4-D im2col map (C, W, H, N)

struct ConvUmmaParams {
    // tiling
    int m_total;          // N * OH * OW
    int cout;
    int tiles_m, tiles_n;
    int m_mult;           // a tile covers m_mult (1, 2 or 4) sub-tiles of 128 pixels: one A load, m_mult MMAs sharing B
    int pair;             // 1: CTA-pair kernel, tiles of 256 pixels (tiles_m counts those), m_mult = 1
    int stream_k;         // 1: stream-K kernel (grid = number of SMs, equal shares of tiles x k-blocks)
    int bn;               // output channels per sub-tile (16..128, multiple of 16); m_mult * bn <= 256
    int bk_bytes;         // bytes of one A/B row per k-block: 128, 64 or 32 (= the swizzle span)
    int bk_elems;         // bk_bytes / sizeof(element)
    int num_stages;
    int a_mode;
    // k loop
    int taps, kh, kw;     // taps = kh*kw
    int chunks_per_tap;   // ceil(Cin / bk_elems)
    int cin_pad;          // k extent of one tap in the packed weights
    int dil_h, dil_w;
    // im2col start coordinates
    int oh, ow, stride_h, stride_w, pad_h, pad_w;
    // epilogue
    int out_chunk_bytes;  // width of one output store slab: 128, 64 or 32 bytes (= swizzle of map_c)
    const void *res;      int ldc_res;     // residual added after act1 (nullptr = none)
    const float *scale;   // y = acc * scale[c] + bias[c]: the folded BatchNorm (ones / conv bias without one),
    const float *bias;    // both padded past the last channel tile
    int act1; float act1_param;
    int act2; float act2_param;            // applied after the residual add
    int *err_flag;
    // stream-K (kStreamK kernels): CTA c takes units [c*U/G, (c+1)*U/G) of the U = tiles * k-blocks sequence
    float *sk_ws;         // one fp32 slot of tile_rows x bn per CTA for the partial sums it hands over
    int *sk_flags;        // one flag per CTA: its slot is filled (reset by the reader)
    uint32_t idesc;       // tcgen05 instruction descriptor
    int acc_shift;        // log2 of the number of accumulator stages (1..3)
    uint32_t tmem_cols;   // power of two >= acc stages * m_mult * bn
    int round_tf32;       // fp32 output feeds another tensor-core conv: store tf32-rounded values
    int sb_channels;      // channels of scale / bias staged in shared memory at kernel start (0: read through L1 instead)
    int split_n;          // two convs over the same input run as one launch: output channels from split_n on (a multiple
                          // of the store slab) are the second conv's and go to map_c2, as its channels 0, 1, ... (INT_MAX: one conv)
    long long *trace;     // per-CTA clock64 stamps (kTraceSlots per CTA), written by the kTrace instantiations only
    int trace_tile;       // which of the CTA's tiles (0 = its first) the producer / MMA stamps describe
};
constexpr int kSbMaxChannels = 1024;   // capacity of the staged scale / bias tables
// Activation handled by a dedicated epilogue instantiation (no switch inside the loops); every other activation takes
// the generic instantiation, which switches per 16 values.
constexpr int kActGeneric = -1;
constexpr int kTraceSlots = 64;

// ---- other layers (layer_kernels.cuh) ---------------------------------------------------------------------------------
// inputs of an n-ary sum
struct AddInputs { const void *ptr[MSNH_B200_MAX_IN]; int ldc[MSNH_B200_MAX_IN]; int n; };
// the pools of one maxpool_plane_kernel launch: up to three stride-1 windows over the same staged plane
struct PoolSet { TView out[3]; int kh[3], kw[3], ph[3], pw[3]; int n; };
// merged stride-2 slices of an image (focus_kernel)
struct FocusParams { int n; int o1[4], o2[4]; };   // slice k (in channel order of the output) picks pixel (2y + o1[k], 2x + o2[k])
// YOLO heads: anchors of one head, and the heads one decode + collect launch walks
struct YoloAnchors { float w[3], h[3]; };
struct YoloHead { TView in; YoloAnchors an; float ratio; int classes, yolo_type, order_base, end; };  // end: one past the head's last item
struct YoloHeadSet { YoloHead h[4]; int n; };
// image preprocessing (preprocess_u8_kernel)
struct PrepParams {
    int w, h;             // source image (HWC, 3 channels)
    int out_w, out_h;
    int letterbox;        // pad to a square with 127 before the resize
    int rev_in, rev_out;  // reverse the channel order before / after the resize
    int mode;             // MSNH_PREP_*
    float mean[3], std[3];
};
// what follows a transposed convolution's gather (col2im_kernel)
struct Col2ImTail {
    const float *scale2, *bias2; int act_mid; float act_mid_p;     // BatchNorm after the layer (scale2 == nullptr: none)
    const void *res; int ldc_res; int act2; float act2_p;          // residual added last (res == nullptr: none)
};

// ---- score sort + NMS (nms_kernel.cuh) --------------------------------------------------------------------------------
constexpr int kNmsMaxCandidates = 4096;   // candidates per image this kernel takes
constexpr int kNmsMaxClasses = 1024;      // class ids this kernel takes (scratch tables in shared memory)
constexpr size_t kNmsSmemBytes = static_cast<size_t>(kNmsMaxCandidates) * (8 + 6 * 4 + 2 + 2 + 1 + 1) +
                                 static_cast<size_t>(kNmsMaxClasses) * (8 + 3 * 4);   // dynamic shared memory per CTA
constexpr int kNmsThreads = 256;


// ---- CUDA-core tiled convolution (conv_tiled.cuh) ---------------------------------------------------------------------
constexpr int kCtBM = 128, kCtBN = 64, kCtThreads = 256;

struct ConvTiledParams {
    int kh, kw, sh, sw, ph, pw, dh, dw;
    int cin_pad;                 // k extent of one tap in the packed weights
    const float *scale, *bias;   // folded BatchNorm / bias per output channel (nullptr: 1 / 0)
    const void *res; int ldc_res;
    int act1; float act1_param; int act2; float act2_param;
};


// ---- depthwise 3x3 on shared-memory tiles (dwconv_tile.cuh) -----------------------------------------------------------
struct DwTileParams {
    int tiles_w, tiles_h, tiles_c;   // tiles per plane and channel groups per pixel
    int th;                          // output rows per tile (a multiple of the rows per thread); columns and channels are fixed
    int ih;                          // input rows per tile: (th - 1) * S + 3
    int stages;                      // shared-memory stages of the load ring (2 or 3)
    int ph, pw;
    int act; float act_param;
    int *err_flag;
};

constexpr int kDwThreads = 128;
constexpr int kDwMaxStages = 3;
constexpr int kDwTileW = 16;         // output columns per tile
constexpr int kDwChannels = 32;      // channels per tile
// output rows per thread (R) and input columns of a tile, by stride
MSNH_HOST_DEVICE constexpr int dw_rows(int S) { return S == 1 ? 4 : 2; }
MSNH_HOST_DEVICE constexpr int dw_in_w(int S) { return (kDwTileW - 1) * S + 3; }


}  // namespace msnh
