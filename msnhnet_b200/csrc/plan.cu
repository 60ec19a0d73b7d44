// Plan compiler and executor behind the C ABI of include/msnh_b200.h.
//
// A plan is built once per (net, batch, dtype): shape inference -> fusion of conv + BatchNorm +
// activation + residual add into one tensor-core launch -> zero-copy placement of route/concat
// inputs as channel slices of the concat buffer -> liveness-based static arena -> weight folding
// and packing -> one list of kernel launches with resolved pointers and TMA tensor maps, captured
// as a CUDA graph. Running a plan is one H2D copy, one graph launch and (optionally) one sync.
// It stands in for NetBuilder's GPU loop and memory pools (src/net/MsnhNetBuilder.cpp:565-620,
// :820-1007 in the reference) and for the per-layer forwardGPU bodies.
#include <cuda.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <thread>
#include <array>
#include <map>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/msnh_b200.h"
#include "common.cuh"
#include "conv_umma.cuh"
#include "nms_kernel.cuh"
#include "layer_kernels.cuh"
#include "dwconv_tile.cuh"
#include "conv_tiled.cuh"

using namespace msnh;

// ------------------------------------------------------------------------------------------------
// context
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct MsnhB200Ctx {
    int device = 0;
    int sm_count = 148;
    int driver_version = 0;
    cudaStream_t stream = nullptr;
    EncodeTiledFn encode_tiled = nullptr;
    EncodeIm2colFn encode_im2col = nullptr;
    int *dev_err_flag = nullptr;
    bool pdl = true;                // programmatic dependent launch between consecutive kernels (MSNH_B200_NO_PDL=1 turns it off)
    float *flush_buf = nullptr;     // > L2 size, for per-launch profiling
    size_t flush_elems = 0;
    std::string last_error;
};

static int fail(MsnhB200Ctx *ctx, int code, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    return code;
}
#define CUDA_TRY(ctx, expr)                                                                          \
    do {                                                                                             \
        cudaError_t e_ = (expr);                                                                     \
        if (e_ != cudaSuccess)                                                                       \
            return fail(ctx, MSNH_B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                        __FILE__, __LINE__);                                                         \
    } while (0)

// ------------------------------------------------------------------------------------------------
// plan data model
// ------------------------------------------------------------------------------------------------
namespace {

struct Shape { int C = 0, H = 0, W = 0; };

// Where a tensor lives: a root buffer of the arena plus a channel offset (concat slices).
struct Tensor {
    Shape s;
    int   dtype = MSNH_B200_F16;
    int   buffer = -1;     // root buffer id
    int   c_off = 0;
    int   ldc = 0;
    bool  placed = false;  // already a slice of some concat buffer
};

struct Buffer {
    int    ldc = 0, dtype = 0;
    size_t pixels = 0;     // batch*H*W
    size_t bytes = 0, offset = 0;
    int    first = 1 << 30, last = -1;
    bool   persistent = false;
    int    alias_of = -1;  // buffer merged into another one (nested concat): root id
    int    alias_c_off = 0;
};

enum LaunchKind { L_INPUT = 0, L_CONV_UMMA, L_CONV_DIRECT, L_DWCONV, L_SBA, L_ADD, L_BINARY, L_MAXPOOL, L_AVGPOOL,
                  L_UPSAMPLE, L_SLICE, L_PAD, L_SOFTMAX, L_YOLO, L_COLLECT_ZERO, L_COLLECT, L_INPUT_PATCH, L_COLLECT_RAW, L_FOCUS,
                  L_BILINEAR, L_COL2IM, L_CLIP, L_REMAP, L_REDUCE, L_PRELU, L_MAXPOOL_DEPTH };
static const char *kLaunchNames[] = {"input_nchw_to_nhwc", "conv_umma", "conv_direct", "dwconv", "scale_bias_act",
                                     "add_n", "binary", "maxpool", "avgpool", "upsample", "slice", "pad", "softmax",
                                     "yolo_decode", "collect_zero", "yolo_collect", "input_nchw_to_patches",
                                     "yolo_decode_collect", "focus_slices", "bilinear", "deconv_col2im", "clip", "remap", "reduce", "prelu", "maxpool_depth"};

struct Launch {
    int kind = 0;
    int op = -1;               // primary op (for describe / parity)
    int dtype = 0;
    TView in{}, out{};
    bool vec = false;
    // generic params
    int kh = 1, kw = 1, sh = 1, sw = 1, ph = 0, pw = 0, dh = 1, dw = 1, groups = 1;
    int act1 = 0, act2 = 0; float act1_p = 0.f, act2_p = 0.f;
    const float *scale = nullptr, *bias = nullptr;
    const float *bias2 = nullptr; int act_mid = 0; float act_mid_p = 0.f;   // deconv gather: BatchNorm behind the layer (scale, bias2)
    const void *weights = nullptr; int cin_pad = 0;
    const void *res = nullptr; int ldc_res = 0;
    AddInputs add{};
    float fval = 0.f; int ival = 0, ival2 = 0;
    int slice_o[3] = {0, 0, 0}, slice_s[3] = {1, 1, 1};
    float anchors[6] = {0, 0, 0, 0, 0, 0};
    int yolo_type = 0; float yolo_ratio = 1.f;   // decode parameters of a fused decode + collect launch
    FocusParams focus{};                         // merged stride-2 slices
    PoolSet pools{};                             // L_MAXPOOL: the pools this launch computes (n == 0: the one in kh.. / out)
    YoloHeadSet heads{};                         // L_COLLECT_RAW: the heads this launch decodes and scans
    // yolo collect
    float *rows = nullptr; int *counts = nullptr; int max_rows = 0;
    // umma
    CUtensorMap map_a, map_b, map_c, map_c2;
    TView out2{};              // second output of two 1x1 convs over the same input merged into this launch (ptr == nullptr: none)
    int split_n = 0;           // its first channel in the merged channel range
    ConvUmmaParams up{};
    int no_split = 0;          // 128-pixel tiles with several store slabs: the epilogue teams take whole tiles in turn instead of sharing each
    int grid = 0; size_t smem = 0;
    // depthwise 3x3 on shared-memory tiles (map_a = the input's 4-D tensor map; grid / smem above)
    bool dw_tile = false; DwTileParams dwp{};
    bool tiled = false;        // L_CONV_DIRECT: dense conv on aligned views -> the shared-memory-tiled CUDA-core kernel
    // accounting
    double flops = 0, bytes = 0;
    std::string note;
};

struct OpState {
    MsnhB200Op d{};
    Shape out;
    int out_dtype = 0;
    std::vector<float> w[MSNH_W_SLOTS];
    size_t wcount[MSNH_W_SLOTS] = {0, 0, 0, 0, 0, 0};
    // fusion results
    int absorbed_into = -1;     // op index of the launch that computes this op's value
    int tensor = -1;            // tensor id holding this op's value
    bool decode_in_collect = false;   // YOLO head whose decode runs inside the collect launch (its tensor is never written)
    std::vector<int> consumers;
};

}  // namespace

struct MsnhB200Plan {
    MsnhB200Ctx *ctx = nullptr;
    int in_c = 0, in_h = 0, in_w = 0, batch = 0, dtype = 0;
    uint32_t flags = 0;
    std::vector<OpState> ops;
    std::vector<Tensor> tensors;
    std::vector<Buffer> buffers;
    std::vector<Launch> launches;
    int input_tensor = -1;
    bool finalized = false;
    bool finalize_failed = false;                   // build_launches failed part-way: the plan can only be destroyed
    // device memory
    uint8_t *arena = nullptr; size_t arena_bytes = 0;
    float *sk_ws = nullptr; int *sk_flags = nullptr;   // stream-K hand-over slots and flags (freed with dev_allocs)
    unsigned char *d_u8 = nullptr; size_t d_u8_bytes = 0;        // raw image staging of plan_preprocess_u8
    float *d_nms_boxes = nullptr; int *d_nms_counts = nullptr;   // device NMS output: [batch][kNmsMaxCandidates][8], [batch]
    bool stream_nms = false; float nms_thresh = 0.f, nms_sigma = 0.3f; int nms_soft = 0;   // streaming: NMS on the device
    float *d_input = nullptr;                       // fp32 NCHW staging
    float *d_readback = nullptr; size_t readback_elems = 0;
    std::vector<void *> dev_allocs;                 // weight arena, workspaces
    // Weight arena: every packed tensor of the plan (conv weights, scale / bias tables, slopes) sits in ONE device
    // allocation filled by one copy. While the launches are being planned the tensors are laid out in `pack_host`
    // and launches hold offsets (tagged pointers); the offsets become device pointers once the size is known.
    // With a pack file (plan_use_pack) the laid-out bytes come from the file and the repacking is skipped.
    std::vector<uint8_t> pack_host;
    size_t pack_cursor = 0;
    bool   pack_loaded = false;                     // arena bytes come from the pack file
    std::string pack_path; uint64_t pack_tag = 0;   // set by plan_use_pack
    std::vector<std::array<int32_t, 3>> pack_picks; // conv tile shapes (sub-tiles, channels, form) in launch order: stored in / taken from the pack
    uint8_t *d_pack = nullptr;
    float *h_pinned = nullptr; size_t h_pinned_bytes = 0;   // staging for pageable callers
    int *h_counts = nullptr;                        // pinned
    cudaGraph_t graph = nullptr; cudaGraphExec_t graph_exec = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.f;
    std::string description;
    // pipelined streaming (plan_stream_push / pop): two slots, a copy stream next to the compute stream
    struct StreamSlot {
        float *d_stage = nullptr;        // this slot's fp32 NCHW input staging on the device
        float *h_result = nullptr;       // pinned: candidate rows or output floats of the batch
        int   *h_counts = nullptr;       // pinned: candidate counts per image
        float *d_result = nullptr;       // device: this slot's copy of the result (candidate rows or output floats)
        int   *d_counts = nullptr;       // device: this slot's copy of the candidate counts + the error flag
        cudaEvent_t h2d_done = nullptr, consumed = nullptr, fwd_done = nullptr, done = nullptr;
        int n_images = 0; bool busy = false;
    } slots[2];
    cudaStream_t copy_stream = nullptr, d2h_stream = nullptr;   // host->device of the next batch / device->host of the last
    int stream_op = -1, stream_cap = 0; size_t stream_result_floats = 0;
    int push_count = 0, pop_count = 0;
};

namespace {

inline int esize(int dtype) { return dtype == MSNH_B200_F16 ? 2 : 4; }
inline int vec_of(int dtype) { return dtype == MSNH_B200_F16 ? 8 : 4; }
inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

int grid_for(const MsnhB200Ctx *ctx, size_t work_items, int block) {
    size_t blocks = (work_items + block - 1) / block;
    size_t cap = static_cast<size_t>(ctx->sm_count) * 8;   // multiple of the SM count, grid-stride beyond
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

// ---- shape inference ---------------------------------------------------------------------------
int infer_shape(MsnhB200Plan *pl, int i, std::string &err) {
    OpState &o = pl->ops[i];
    const MsnhB200Op &d = o.d;
    auto in_shape = [&](int k) -> Shape {
        int src = d.in[k];
        if (src == MSNH_B200_INPUT) { Shape s; s.C = pl->in_c; s.H = pl->in_h; s.W = pl->in_w; return s; }
        return pl->ops[src].out;
    };
    if (d.n_in < 1 || d.n_in > MSNH_B200_MAX_IN) { err = "bad n_in"; return MSNH_B200_ERR_ARG; }
    for (int k = 0; k < d.n_in; ++k)
        if (d.in[k] != MSNH_B200_INPUT && (d.in[k] < 0 || d.in[k] >= i)) { err = "op input must name an earlier op"; return MSNH_B200_ERR_ARG; }
    Shape a = in_shape(0);
    o.out_dtype = pl->dtype;
    switch (d.kind) {
        case MSNH_OP_CONV: {
            if (d.groups < 1 || a.C % d.groups || d.filters % d.groups) { err = "conv groups do not divide channels"; return MSNH_B200_ERR_ARG; }
            if (d.k_h < 1 || d.k_w < 1 || d.stride_h < 1 || d.stride_w < 1 || d.dil_h < 1 || d.dil_w < 1 || d.pad_h < 0 || d.pad_w < 0 || d.filters < 1) { err = "bad conv geometry (kernel, stride, dilation below 1 or negative padding)"; return MSNH_B200_ERR_ARG; }
            o.out.C = d.filters;
            o.out.H = (a.H + 2 * d.pad_h - (d.dil_h * (d.k_h - 1) + 1)) / d.stride_h + 1;
            o.out.W = (a.W + 2 * d.pad_w - (d.dil_w * (d.k_w - 1) + 1)) / d.stride_w + 1;
            o.wcount[MSNH_W_WEIGHTS] = static_cast<size_t>(d.filters) * (a.C / d.groups) * d.k_h * d.k_w;
            if (d.has_bn) for (int s = MSNH_W_BN_SCALE; s <= MSNH_W_BN_VAR; ++s) o.wcount[s] = d.filters;
            else if (d.has_bias) o.wcount[MSNH_W_BIAS] = d.filters;
            break;
        }
        case MSNH_OP_CONNECTED: {
            o.out.C = d.filters; o.out.H = 1; o.out.W = 1;
            o.wcount[MSNH_W_WEIGHTS] = static_cast<size_t>(d.filters) * a.C * a.H * a.W;
            if (d.has_bn) for (int s = MSNH_W_BN_SCALE; s <= MSNH_W_BN_VAR; ++s) o.wcount[s] = d.filters;
            else if (d.has_bias) o.wcount[MSNH_W_BIAS] = d.filters;
            break;
        }
        case MSNH_OP_BATCHNORM:
            o.out = a;
            for (int s = MSNH_W_BN_SCALE; s <= MSNH_W_BN_VAR; ++s) o.wcount[s] = a.C;
            break;
        case MSNH_OP_ACTIVATION: case MSNH_OP_IDENTITY: case MSNH_OP_SOFTMAX:
            o.out = a; break;
        case MSNH_OP_PRELU:
            o.out = a; o.wcount[MSNH_W_WEIGHTS] = a.C; break;
        case MSNH_OP_MAXPOOL: case MSNH_OP_AVGPOOL:
            if (d.kind == MSNH_OP_MAXPOOL && d.filters > 0) {   // depth pooling
                if (d.filters > a.C) { err = "depth pooling to more channels than the input has"; return MSNH_B200_ERR_ARG; }
                o.out = a; o.out.C = d.filters; break;
            }
            if (d.k_h < 1 || d.k_w < 1 || d.stride_h < 1 || d.stride_w < 1 || d.pad_h < 0 || d.pad_w < 0) { err = "bad pool geometry (kernel or stride below 1, negative padding)"; return MSNH_B200_ERR_ARG; }
            o.out.C = a.C;
            o.out.H = d.out_h > 0 ? d.out_h : (a.H + 2 * d.pad_h - d.k_h) / d.stride_h + 1;
            o.out.W = d.out_w > 0 ? d.out_w : (a.W + 2 * d.pad_w - d.k_w) / d.stride_w + 1;
            break;
        case MSNH_OP_UPSAMPLE:
            if (d.upsample_mode == MSNH_UPSAMPLE_BILINEAR) {
                if (d.out_h < 1 || d.out_w < 1) { err = "bilinear upsample needs out_h / out_w"; return MSNH_B200_ERR_ARG; }
                if (d.align_corners && (d.out_h < 2 || d.out_w < 2)) { err = "align_corners needs an output plane of at least 2x2"; return MSNH_B200_ERR_ARG; }
                o.out.C = a.C; o.out.H = d.out_h; o.out.W = d.out_w; break;
            }
            if (d.stride_h < 1 || d.stride_w < 1) { err = "upsample stride below 1"; return MSNH_B200_ERR_ARG; }
            o.out.C = a.C; o.out.H = a.H * d.stride_h; o.out.W = a.W * d.stride_w; break;
        case MSNH_OP_DECONV:
            if (d.groups != 1) { err = "deconv groups != 1 is not supported"; return MSNH_B200_ERR_UNSUPPORTED; }
            if (d.has_bn) { err = "deconv has no BatchNorm form"; return MSNH_B200_ERR_ARG; }
            if (d.k_h < 1 || d.k_w < 1 || d.stride_h < 1 || d.stride_w < 1 || d.pad_h < 0 || d.pad_w < 0) { err = "bad deconv geometry"; return MSNH_B200_ERR_ARG; }
            o.out.C = d.filters;
            o.out.H = (a.H - 1) * d.stride_h - 2 * d.pad_h + d.k_h;   // src/layers/MsnhDeConvolutionalLayer.cpp:229-237
            o.out.W = (a.W - 1) * d.stride_w - 2 * d.pad_w + d.k_w;
            o.wcount[MSNH_W_WEIGHTS] = static_cast<size_t>(a.C) * d.filters * d.k_h * d.k_w;
            if (d.has_bias) o.wcount[MSNH_W_BIAS] = d.filters;
            break;
        case MSNH_OP_CLIP:
            if (d.const_val > d.scale) { err = "clip min above max"; return MSNH_B200_ERR_ARG; }
            o.out = a; break;
        case MSNH_OP_REMAP:
            if (d.remap_kind == MSNH_REMAP_VIEW) {
                o.out.C = d.out_c; o.out.H = d.out_h; o.out.W = d.out_w;
                if (d.out_c < 1 || d.out_h < 1 || d.out_w < 1 ||
                    static_cast<long long>(o.out.C) * o.out.H * o.out.W != static_cast<long long>(a.C) * a.H * a.W) { err = "view op params error"; return MSNH_B200_ERR_ARG; }
            } else if (d.remap_kind == MSNH_REMAP_PERMUTE) {
                const int dims[3] = {a.C, a.H, a.W};
                bool seen[3] = {false, false, false};
                for (int k = 0; k < 3; ++k) {
                    if (d.remap_dims[k] < 0 || d.remap_dims[k] > 2 || seen[d.remap_dims[k]]) { err = "permute dims must be a permutation of 0/1/2"; return MSNH_B200_ERR_ARG; }
                    seen[d.remap_dims[k]] = true;
                }
                o.out.C = dims[d.remap_dims[0]]; o.out.H = dims[d.remap_dims[1]]; o.out.W = dims[d.remap_dims[2]];
            } else if (d.remap_kind == MSNH_REMAP_PIXSHF) {
                const int f = d.remap_dims[0];
                if (f < 1) { err = "factor must > 0"; return MSNH_B200_ERR_ARG; }
                if (a.C % (f * f)) { err = "channel is not divisible by factor^2"; return MSNH_B200_ERR_ARG; }
                o.out.C = a.C / (f * f); o.out.H = a.H * f; o.out.W = a.W * f;
            } else { err = "unknown remap kind"; return MSNH_B200_ERR_ARG; }
            break;
        case MSNH_OP_REDUCE:
            o.out = a;
            if (d.binary_kind == -1) { o.out.C = 1; o.out.H = 1; o.out.W = 1; }
            else if (d.binary_kind == 0) o.out.C = 1;
            else if (d.binary_kind == 1) o.out.H = 1;
            else if (d.binary_kind == 2) o.out.W = 1;
            else { err = "reduce axis must be -1, 0, 1 or 2"; return MSNH_B200_ERR_ARG; }
            break;
        case MSNH_OP_CONCAT: {
            int c = 0;
            for (int k = 0; k < d.n_in; ++k) {
                Shape s = in_shape(k);
                if (s.H != a.H || s.W != a.W) { err = "concat inputs differ in plane size"; return MSNH_B200_ERR_ARG; }
                int g = d.route_groups > 0 ? d.route_groups : 1;
                if (s.C % g) { err = "route groups do not divide channels"; return MSNH_B200_ERR_ARG; }
                c += s.C / g;
            }
            o.out.C = c; o.out.H = a.H; o.out.W = a.W;
            break;
        }
        case MSNH_OP_ADD:
            for (int k = 1; k < d.n_in; ++k) {
                Shape s = in_shape(k);
                if (s.C != a.C || s.H != a.H || s.W != a.W) { err = "add inputs differ in shape"; return MSNH_B200_ERR_ARG; }
            }
            o.out = a; break;
        case MSNH_OP_BINARY:
            if (d.binary_kind < 0 || d.binary_kind >= MSNH_BIN_COUNT) { err = "unknown binary kind"; return MSNH_B200_ERR_ARG; }
            if (d.binary_kind > MSNH_BIN_DIV_INV && !d.binary_const) { err = "one-operand kinds take binary_const = 1"; return MSNH_B200_ERR_ARG; }
            if (!d.binary_const) {
                if (d.n_in != 2) { err = "binary needs two inputs"; return MSNH_B200_ERR_ARG; }
                Shape s = in_shape(1);
                if (s.C != a.C || s.H != a.H || s.W != a.W) { err = "binary inputs differ in shape"; return MSNH_B200_ERR_ARG; }
            }
            o.out = a; break;
        case MSNH_OP_SLICE:
            // out = ceil((dim - start) / step), the reference's rule (src/layers/MsnhSliceLayer.cpp:24-50)
            for (int k = 0; k < 3; ++k) {
                const int dim = k == 0 ? a.C : (k == 1 ? a.H : a.W);
                if (d.slice_step[k] < 1 || d.slice_start[k] < 0 || d.slice_start[k] >= dim) { err = "slice start outside the tensor or step below 1"; return MSNH_B200_ERR_ARG; }
            }
            o.out.C = (a.C - d.slice_start[0] + d.slice_step[0] - 1) / d.slice_step[0];
            o.out.H = (a.H - d.slice_start[1] + d.slice_step[1] - 1) / d.slice_step[1];
            o.out.W = (a.W - d.slice_start[2] + d.slice_step[2] - 1) / d.slice_step[2];
            break;
        case MSNH_OP_PAD:
            if (d.pad_top < 0 || d.pad_down < 0 || d.pad_left < 0 || d.pad_right < 0) { err = "negative padding"; return MSNH_B200_ERR_ARG; }
            o.out.C = a.C; o.out.H = a.H + d.pad_top + d.pad_down; o.out.W = a.W + d.pad_left + d.pad_right; break;
        case MSNH_OP_YOLO:
            if (a.C != 3 * (5 + d.yolo_classes)) { err = "yolo head channels != 3*(classes+5)"; return MSNH_B200_ERR_ARG; }
            o.out = a; o.out_dtype = MSNH_B200_F32; break;
        case MSNH_OP_YOLO_COLLECT: {
            int cells = 0;
            for (int k = 0; k < d.n_in; ++k) {
                if (d.in[k] < 0 || pl->ops[d.in[k]].d.kind != MSNH_OP_YOLO) { err = "yolo collect inputs must be yolo ops"; return MSNH_B200_ERR_ARG; }
                Shape s = in_shape(k); cells += 3 * s.H * s.W;
            }
            o.out.C = 8; o.out.H = 1; o.out.W = cells; o.out_dtype = MSNH_B200_F32;
            break;
        }
        default: err = "unknown op kind"; return MSNH_B200_ERR_UNSUPPORTED;
    }
    if (o.out.C <= 0 || o.out.H <= 0 || o.out.W <= 0) { err = "op produces an empty tensor"; return MSNH_B200_ERR_ARG; }
    // the element-wise kernels index vectors with 32 bits
    if (static_cast<double>(pl->batch) * o.out.C * o.out.H * o.out.W >= 2147483648.0) { err = "tensor of 2^31 or more elements"; return MSNH_B200_ERR_UNSUPPORTED; }
    return MSNH_B200_OK;
}

// ---- tensors / buffers -------------------------------------------------------------------------
int new_tensor(MsnhB200Plan *pl, Shape s, int dtype) {
    Tensor t; t.s = s; t.dtype = dtype; t.ldc = round_up(s.C, vec_of(dtype));
    pl->tensors.push_back(t);
    return static_cast<int>(pl->tensors.size()) - 1;
}
int new_buffer(MsnhB200Plan *pl, int tensor) {
    Tensor &t = pl->tensors[tensor];
    Buffer b; b.ldc = t.ldc; b.dtype = t.dtype;
    b.pixels = static_cast<size_t>(pl->batch) * t.s.H * t.s.W;
    pl->buffers.push_back(b);
    t.buffer = static_cast<int>(pl->buffers.size()) - 1; t.c_off = 0;
    return t.buffer;
}
int root_of(MsnhB200Plan *pl, int buf, int *c_off) {
    int off = 0;
    while (pl->buffers[buf].alias_of >= 0) { off += pl->buffers[buf].alias_c_off; buf = pl->buffers[buf].alias_of; }
    if (c_off) *c_off = off;
    return buf;
}
TView view_of(MsnhB200Plan *pl, int tensor) {
    const Tensor &t = pl->tensors[tensor];
    int extra = 0;
    int root = root_of(pl, t.buffer, &extra);
    const Buffer &b = pl->buffers[root];
    TView v;
    v.ptr = pl->arena + b.offset + static_cast<size_t>(t.c_off + extra) * esize(t.dtype);
    v.N = pl->batch; v.H = t.s.H; v.W = t.s.W; v.C = t.s.C; v.ldc = b.ldc; v.tf32 = 0;
    return v;
}
void touch(MsnhB200Plan *pl, int tensor, int step) {
    int root = root_of(pl, pl->tensors[tensor].buffer, nullptr);
    Buffer &b = pl->buffers[root];
    b.first = std::min(b.first, step); b.last = std::max(b.last, step);
}

// ---- tensor maps -------------------------------------------------------------------------------
CUtensorMapSwizzle swizzle_of(int bk_bytes) {
    return bk_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bk_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}
CUtensorMapDataType tm_type(int dtype) { return dtype == MSNH_B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32; }

int make_map_2d(MsnhB200Ctx *ctx, CUtensorMap *m, int dtype, const void *base, uint64_t inner, uint64_t outer,
                uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int bk_bytes) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ctx->encode_tiled(m, tm_type(dtype), 2, const_cast<void *>(base), dims, strides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_of(bk_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ctx, MSNH_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d): dims %llu x %llu stride %llu box %u x %u", (int)r,
                    (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_stride_bytes, box_inner, box_outer);
    return MSNH_B200_OK;
}

int make_map_im2col(MsnhB200Ctx *ctx, CUtensorMap *m, int dtype, const TView &in, int kh, int kw, int sh, int sw,
                    int ph, int pw, int dh, int dw, int bk_elems, int bk_bytes, int pixels) {
    const uint64_t es = esize(dtype);
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(in.C), static_cast<cuuint64_t>(in.W), static_cast<cuuint64_t>(in.H),
                          static_cast<cuuint64_t>(in.N)};
    cuuint64_t strides[3] = {in.ldc * es, static_cast<cuuint64_t>(in.W) * in.ldc * es,
                             static_cast<cuuint64_t>(in.H) * in.W * in.ldc * es};
    // The filter's top-left tap may sit anywhere in [-pad, dim + pad - dilation*(k-1) - 1].
    int lower[2] = {-pw, -ph};
    int upper[2] = {pw - dw * (kw - 1), ph - dh * (kh - 1)};
    cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(sw), static_cast<cuuint32_t>(sh), 1};
    CUresult r = ctx->encode_im2col(m, tm_type(dtype), 4, in.ptr, dims, strides, lower, upper,
                                    static_cast<cuuint32_t>(bk_elems), static_cast<cuuint32_t>(pixels), estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                    swizzle_of(bk_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ctx, MSNH_B200_ERR_CUDA, "cuTensorMapEncodeIm2col failed (%d): C%d W%d H%d N%d ldc%d k%dx%d s%d p%d", (int)r,
                    in.C, in.W, in.H, in.N, in.ldc, kh, kw, sh, ph);
    // Drivers up to 13.1 mis-encode im2col maps of tensors smaller than 128 KiB; clearing bit 21 of
    // the second descriptor word is the published workaround (CUTLASS applies the same patch).
    const uint64_t span = static_cast<uint64_t>(in.N) * in.H * in.W * in.ldc * es;
    if (ctx->driver_version <= 13010 && span < 131072) reinterpret_cast<uint64_t *>(m)[1] &= ~(1ull << 21);
    return MSNH_B200_OK;
}

// pick the k-block width (bytes per row per stage) for `cin` input channels of `es` bytes
int pick_bk_bytes(int cin, int es) {
    const int row = cin * es;
    int best = 128; long best_cost = -1;
    for (int bk : {128, 64, 32}) {
        long chunks = (row + bk - 1) / bk;
        long cost = chunks * (bk + 32);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bk; }
    }
    return best;
}

// The instantiation of the tensor-core conv kernel a launch runs: tile form (sub-tiles per tile, epilogue teams sharing
// or alternating tiles, CTA pair, stream-K), the activation compiled into the epilogue (mish and leaky with a slope in
// [0, 1] have their own fp16 instantiations; everything else switches at run time) and, for plans made with
// MSNH_PLAN_TRACE, the form that records clock stamps.
template <typename T> const void *umma_kernel(const Launch &L) {
    const ConvUmmaParams &u = L.up;
    if (u.stream_k) return u.m_mult == 2 ? reinterpret_cast<const void *>(conv_umma_kernel<T, 2, true, false, true>)
                                         : reinterpret_cast<const void *>(conv_umma_kernel<T, 1, true, false, true>);
    if (u.pair) return reinterpret_cast<const void *>(conv_umma_kernel<T, 1, true, true, false>);
    // both epilogue teams share every tile once a tile has at least two store slabs
    const bool split = u.m_mult > 1 || (u.bn * static_cast<int>(sizeof(T)) > u.out_chunk_bytes && !L.no_split);
    const bool trace = u.trace != nullptr;
    int act = kActGeneric;
    if (sizeof(T) == 2 && !trace) {
        if (u.act1 == MSNH_ACT_MISH) act = MSNH_ACT_MISH;
        else if (u.act1 == MSNH_ACT_LEAKY && u.act1_param >= 0.f && u.act1_param <= 1.f) act = MSNH_ACT_LEAKY;
    }
#define MSNH_UMMA_FORM(MM, SP)                                                                                                   \
    do {                                                                                                                         \
        if (trace) return reinterpret_cast<const void *>(conv_umma_kernel<T, MM, SP, false, false, kActGeneric, true>);          \
        if constexpr (sizeof(T) == 2) {                                                                                          \
            if (act == MSNH_ACT_MISH) return reinterpret_cast<const void *>(conv_umma_kernel<T, MM, SP, false, false, MSNH_ACT_MISH>);   \
            if (act == MSNH_ACT_LEAKY) return reinterpret_cast<const void *>(conv_umma_kernel<T, MM, SP, false, false, MSNH_ACT_LEAKY>); \
        }                                                                                                                        \
        return reinterpret_cast<const void *>(conv_umma_kernel<T, MM, SP, false, false>);                                        \
    } while (0)
    if (u.m_mult == 4) MSNH_UMMA_FORM(4, true);
    if (u.m_mult == 3) MSNH_UMMA_FORM(3, true);
    if (u.m_mult == 2) MSNH_UMMA_FORM(2, true);
    if (split) MSNH_UMMA_FORM(1, true);
    MSNH_UMMA_FORM(1, false);
#undef MSNH_UMMA_FORM
}
const void *umma_kernel_of(const Launch &L) { return L.dtype == MSNH_B200_F16 ? umma_kernel<__half>(L) : umma_kernel<float>(L); }

// dynamic shared memory opt-in of the kernel a launch runs (raised as needed, once per size and kernel)
void set_smem_attr(const Launch &L) {
    static std::mutex m;
    static std::map<const void *, size_t> current;
    const void *k = umma_kernel_of(L);
    std::lock_guard<std::mutex> g(m);
    size_t &cur = current[k];
    if (L.smem > cur) { cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(L.smem)); cur = L.smem; }
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// launching
// ------------------------------------------------------------------------------------------------
namespace {

// Launch with the programmatic-dependent-launch attribute: the grid may be scheduled while its
// predecessor in the stream drains; every kernel of this library calls griddepcontrol.wait before it
// touches memory, so only launch latency and per-CTA set-up overlap, never data.
template <typename... KArgs, typename... Args>
void launch_k(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
template <typename T>
void launch_typed(MsnhB200Ctx *ctx, const Launch &L, cudaStream_t st) {
    constexpr int V = Elem<T>::kVec;
    const int block = 256;
    const size_t out_items = static_cast<size_t>(L.out.N) * L.out.H * L.out.W * (L.vec ? L.out.C / V : L.out.C);
    const int grid = grid_for(ctx, out_items, block);
    switch (L.kind) {
        case L_INPUT:
            launch_k(ctx->pdl, nchw_f32_to_nhwc_kernel<T>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W, block), block, 0, st, 
                static_cast<const float *>(L.in.ptr), L.out);
            break;
        case L_INPUT_PATCH:
            if (L.ival == 3 && L.kh == 3 && L.kw == 3 && L.out.ldc == 32)
                launch_k(ctx->pdl, nchw_f32_to_patches_fixed_kernel<T, 3, 3, 3>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W, 128), 128, 0, st, 
                    static_cast<const float *>(L.in.ptr), L.out, L.ival2, L.max_rows, L.sh, L.sw, L.ph, L.pw, L.dh, L.dw);
            else
            launch_k(ctx->pdl, nchw_f32_to_patches_kernel<T>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W, block), block, 0, st, 
                static_cast<const float *>(L.in.ptr), L.out, L.ival, L.ival2, L.max_rows, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, L.dh, L.dw);
            break;
        case L_CONV_UMMA: {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(L.grid); cfg.blockDim = dim3(kUmmaThreads); cfg.dynamicSmemBytes = L.smem; cfg.stream = st;
            cudaLaunchAttribute attr[2];
            int na = 0;
            if (L.up.pair) { attr[na].id = cudaLaunchAttributeClusterDimension; attr[na].val.clusterDim.x = 2; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1; ++na; }
            if (ctx->pdl) { attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[na].val.programmaticStreamSerializationAllowed = 1; ++na; }
            cfg.attrs = attr; cfg.numAttrs = na;
            void *args[5] = {const_cast<CUtensorMap *>(&L.map_a), const_cast<CUtensorMap *>(&L.map_b), const_cast<CUtensorMap *>(&L.map_c),
                             const_cast<CUtensorMap *>(L.out2.ptr ? &L.map_c2 : &L.map_c), const_cast<ConvUmmaParams *>(&L.up)};
            cudaLaunchKernelExC(&cfg, umma_kernel<T>(L), args);
            break;
        }
        case L_CONV_DIRECT:
            if (L.tiled) {
                const ConvTiledParams cp{L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, L.dh, L.dw, L.cin_pad, L.scale, L.bias, L.res, L.ldc_res, L.act1, L.act1_p, L.act2, L.act2_p};
                const int m_total = L.out.N * L.out.H * L.out.W;
                launch_k(ctx->pdl, conv_tiled_kernel<T>, dim3((m_total + kCtBM - 1) / kCtBM, (L.out.C + kCtBN - 1) / kCtBN), kCtThreads, 0, st, L.in, L.out, static_cast<const T *>(L.weights), cp);
                break;
            }
            launch_k(ctx->pdl, conv_direct_kernel<T>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W * L.out.C, block), block, 0, st, L.in, L.out, static_cast<const T *>(L.weights), L.cin_pad, L.scale, L.bias,
                                                          L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, L.dh, L.dw, L.groups,
                                                          static_cast<const T *>(L.res), L.ldc_res, L.act1, L.act1_p, L.act2, L.act2_p);
            break;
        case L_DWCONV:
            if (L.dw_tile) {
                auto go = [&](auto kernel) {
                    launch_k(ctx->pdl, kernel, L.grid, kDwThreads, L.smem, st, L.map_a, L.out, static_cast<const T *>(L.weights), L.scale, L.bias, L.dwp);
                };
                const bool relu6 = L.act1 == MSNH_ACT_RELU6;
                if (L.sh == 1) { if (relu6) go(dwconv3x3_tile_kernel<T, 1, true>); else go(dwconv3x3_tile_kernel<T, 1, false>); }
                else           { if (relu6) go(dwconv3x3_tile_kernel<T, 2, true>); else go(dwconv3x3_tile_kernel<T, 2, false>); }
                break;
            }
            if (L.vec && L.kh == 3 && L.kw == 3 && L.dh == 1 && L.dw == 1 && L.sh == L.sw && (L.sh == 1 || L.sh == 2)) {
                // strips of four output pixels per thread
                const size_t items = static_cast<size_t>(L.out.N) * L.out.H * ((L.out.W + 3) / 4) * (L.out.C / V);
                const int g = grid_for(ctx, items, 128);
                if (L.sh == 1) launch_k(ctx->pdl, dwconv3x3_kernel<T, V, 1>, g, 128, 0, st, L.in, L.out, static_cast<const T *>(L.weights), L.scale, L.bias, L.ph, L.pw, L.act1, L.act1_p);
                else           launch_k(ctx->pdl, dwconv3x3_kernel<T, V, 2>, g, 128, 0, st, L.in, L.out, static_cast<const T *>(L.weights), L.scale, L.bias, L.ph, L.pw, L.act1, L.act1_p);
                break;
            }
            if (L.vec) launch_k(ctx->pdl, dwconv_kernel<T, V>, grid, block, 0, st, L.in, L.out, static_cast<const T *>(L.weights), L.scale, L.bias, L.kh, L.kw,
                                                                   L.sh, L.sw, L.ph, L.pw, L.dh, L.dw, L.act1, L.act1_p);
            else       launch_k(ctx->pdl, dwconv_kernel<T, 1>, grid, block, 0, st, L.in, L.out, static_cast<const T *>(L.weights), L.scale, L.bias, L.kh, L.kw,
                                                                   L.sh, L.sw, L.ph, L.pw, L.dh, L.dw, L.act1, L.act1_p);
            break;
        case L_SBA:
            if (L.vec) launch_k(ctx->pdl, scale_bias_act_kernel<T, V>, grid, block, 0, st, L.in, L.out, L.scale, L.bias, L.act1, L.act1_p);
            else       launch_k(ctx->pdl, scale_bias_act_kernel<T, 1>, grid, block, 0, st, L.in, L.out, L.scale, L.bias, L.act1, L.act1_p);
            break;
        case L_ADD:
            if (L.vec) launch_k(ctx->pdl, add_n_kernel<T, V>, grid, block, 0, st, L.add, L.out, L.act1, L.act1_p);
            else       launch_k(ctx->pdl, add_n_kernel<T, 1>, grid, block, 0, st, L.add, L.out, L.act1, L.act1_p);
            break;
        case L_BINARY:
            if (L.vec) launch_k(ctx->pdl, binary_kernel<T, V>, grid, block, 0, st, L.in, L.res, L.ldc_res, L.fval, L.ival, L.out);
            else       launch_k(ctx->pdl, binary_kernel<T, 1>, grid, block, 0, st, L.in, L.res, L.ldc_res, L.fval, L.ival, L.out);
            break;
        case L_MAXPOOL: {
            // plane-in-shared-memory form for stride-1 pools that keep the plane size and window wider than 3
            const int hw = L.in.H * L.in.W;
            const bool same = L.sh == 1 && L.sw == 1 && L.out.H == L.in.H && L.out.W == L.in.W && L.kh * L.kw > 9 &&
                              L.kh <= 2 * L.ph + 1 && L.kw <= 2 * L.pw + 1;
            if (L.vec && same && hw * 32 <= 48 * 1024) {
                int G = std::min(4, 48 * 1024 / (hw * 32));
                const int cv = L.in.C / V;
                while (G > 1 && L.in.N * ((cv + G - 1) / G) < ctx->sm_count) --G;
                launch_k(ctx->pdl, maxpool_plane_kernel<T>, std::min(L.in.N * ((cv + G - 1) / G), 4 * ctx->sm_count), 256,
                         static_cast<size_t>(hw) * G * 32, st, L.in, L.pools, G);
                break;
            }
            if (L.pools.n > 1) break;    // (cannot happen: pools are merged only where the plane form applies; plan_finalize checks)
            if (L.vec) launch_k(ctx->pdl, maxpool_kernel<T, V>, grid, block, 0, st, L.in, L.out, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw);
            else       launch_k(ctx->pdl, maxpool_kernel<T, 1>, grid, block, 0, st, L.in, L.out, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw);
            break;
        }
        case L_AVGPOOL:
            if (L.vec) launch_k(ctx->pdl, avgpool_kernel<T, V>, grid, block, 0, st, L.in, L.out, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw);
            else       launch_k(ctx->pdl, avgpool_kernel<T, 1>, grid, block, 0, st, L.in, L.out, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw);
            break;
        case L_UPSAMPLE:
            if (L.vec) launch_k(ctx->pdl, upsample_kernel<T, V>, grid, block, 0, st, L.in, L.out, L.sh, L.sw, L.fval);
            else       launch_k(ctx->pdl, upsample_kernel<T, 1>, grid, block, 0, st, L.in, L.out, L.sh, L.sw, L.fval);
            break;
        case L_BILINEAR:
            if (L.vec) launch_k(ctx->pdl, bilinear_kernel<T, V>, grid, block, 0, st, L.in, L.out, L.fval, L.act1_p, L.ival);
            else       launch_k(ctx->pdl, bilinear_kernel<T, 1>, grid, block, 0, st, L.in, L.out, L.fval, L.act1_p, L.ival);
            break;
        case L_COL2IM:
        {
            const Col2ImTail tail{L.scale, L.bias2, L.act_mid, L.act_mid_p, L.res, L.ldc_res, L.act2, L.act2_p};
            const int grid = std::min(L.out.N * L.out.H, 16 * ctx->sm_count);    // CTAs walk output rows
            const int cvn = L.vec ? L.out.C / V : L.out.C;
            int lc = 0; while (lc < 8 && (2 << lc) <= cvn) ++lc;                  // threads along channels: largest power of two <= channel vectors (<= 256)
            if (L.vec) launch_k(ctx->pdl, col2im_kernel<T, V>, grid, block, 0, st, L.in, L.out, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, L.bias, L.act1, L.act1_p, tail, lc);
            else       launch_k(ctx->pdl, col2im_kernel<T, 1>, grid, block, 0, st, L.in, L.out, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, L.bias, L.act1, L.act1_p, tail, lc);
        }
            break;
        case L_PRELU:
            if (L.vec) launch_k(ctx->pdl, prelu_kernel<T, V>, grid, block, 0, st, L.in, L.out, L.scale);
            else       launch_k(ctx->pdl, prelu_kernel<T, 1>, grid, block, 0, st, L.in, L.out, L.scale);
            break;
        case L_MAXPOOL_DEPTH:
            launch_k(ctx->pdl, maxpool_depth_kernel<T>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W * L.out.C, block), block, 0, st, L.in, L.out);
            break;
        case L_CLIP:
            if (L.vec) launch_k(ctx->pdl, clip_kernel<T, V>, grid, block, 0, st, L.in, L.out, L.fval, L.act1_p);
            else       launch_k(ctx->pdl, clip_kernel<T, 1>, grid, block, 0, st, L.in, L.out, L.fval, L.act1_p);
            break;
        case L_REMAP:
            launch_k(ctx->pdl, remap_kernel<T>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W * L.out.C, block), block, 0, st,
                L.in, L.out, L.ival, L.slice_o[0], L.slice_o[1], L.slice_o[2]);
            break;
        case L_REDUCE:
            launch_k(ctx->pdl, reduce_kernel<T>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W * L.out.C * 32, block), block, 0, st,
                L.in, L.out, L.ival, L.ival2);
            break;
        case L_SLICE:
            launch_k(ctx->pdl, slice_kernel<T>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W, block), block, 0, st, L.in, L.out, L.slice_o[0], L.slice_s[0], L.slice_o[1], L.slice_s[1], L.slice_o[2], L.slice_s[2]);
            break;
        case L_PAD:
            if (L.vec) launch_k(ctx->pdl, pad_kernel<T, V>, grid, block, 0, st, L.in, L.out, L.ph, L.pw, L.fval);
            else       launch_k(ctx->pdl, pad_kernel<T, 1>, grid, block, 0, st, L.in, L.out, L.ph, L.pw, L.fval);
            break;
        case L_SOFTMAX: {
            const size_t rows = static_cast<size_t>(L.in.N) * L.ival;
            launch_k(ctx->pdl, softmax_kernel<T>, grid_for(ctx, rows * 32, block), block, 0, st, L.in, L.out, L.ival, L.fval);
            break;
        }
        case L_YOLO:
            launch_k(ctx->pdl, yolo_decode_kernel<T>, grid_for(ctx, static_cast<size_t>(L.in.N) * L.in.H * L.in.W * L.in.C, block), block, 0, st,
                L.in, L.out, L.ival, L.ival2, L.fval, YoloAnchors{{L.anchors[0], L.anchors[2], L.anchors[4]}, {L.anchors[1], L.anchors[3], L.anchors[5]}});
            break;
        case L_FOCUS:
            launch_k(ctx->pdl, focus_kernel<T, 3>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W, block), block, 0, st, L.in, L.out, L.focus);
            break;
        case L_COLLECT_RAW:
            launch_k(ctx->pdl, yolo_decode_collect_kernel<T>, grid_for(ctx, static_cast<size_t>(L.heads.h[L.heads.n - 1].end), 256), 256, 0, st,
                L.heads, L.fval, L.rows, L.max_rows, L.counts);
            break;
        default: break;
    }
}

void launch_one(MsnhB200Ctx *ctx, const Launch &L, cudaStream_t st) {
    if (L.kind == L_COLLECT_ZERO) {
        cudaMemsetAsync(L.counts, 0, sizeof(int) * L.out.N, st);
        return;
    }
    if (L.kind == L_COLLECT) {
        const size_t items = static_cast<size_t>(L.in.N) * L.in.H * L.in.W * 3;
        launch_k(ctx->pdl, yolo_collect_kernel, grid_for(ctx, items, 256), 256, 0, st, L.in, L.ival, L.fval, L.ival2, L.rows, L.max_rows, L.counts);
        return;
    }
    if (L.dtype == MSNH_B200_F16) launch_typed<__half>(ctx, L, st);
    else                          launch_typed<float>(ctx, L, st);
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// finalize: fusion, placement, arena, weights, launches, graph
// ------------------------------------------------------------------------------------------------
namespace {

struct Fused {          // one conv-like or elementwise producer with what it absorbed
    int bn_op = -1;     // absorbed standalone BatchNorm
    int act_op = -1;    // absorbed activation (before the add)
    int add_op = -1;    // absorbed residual add
    int act2_op = -1;   // absorbed activation after the add
    // BatchNorm (+ activation) that follows a concat of plain convs: every producer applies its channel slice
    int cat_bn_op = -1, cat_act_op = -1, cat_c_off = 0;
    int last_op = -1;   // op whose value the launch produces
    int res_op = MSNH_B200_INPUT - 1;  // residual source op
};

bool sole_consumer(MsnhB200Plan *pl, int op, int *consumer) {
    const OpState &o = pl->ops[op];
    if (o.d.is_output || (pl->flags & (MSNH_PLAN_KEEP_ALL | MSNH_PLAN_NO_FUSION))) return false;
    if (o.consumers.size() != 1) return false;
    *consumer = o.consumers[0];
    return true;
}

// rows 0..n-1 of a weight repack, spread over host threads when the tensor is large enough to pay for them
template <typename F> void parallel_rows(int n, size_t work_per_row, F &&fn) {
    const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
    const int threads = static_cast<int>(std::min<size_t>(std::min<unsigned>(hw, 16), static_cast<size_t>(n) * work_per_row / 262144 + 1));
    if (threads <= 1) { for (int i = 0; i < n; ++i) fn(i); return; }
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
        pool.emplace_back([&, t]() { for (int i = t; i < n; i += threads) fn(i); });
    for (auto &th : pool) th.join();
}

// fp32 -> nearest tf32 (10-bit mantissa, ties away from zero like cvt.rna), still stored as fp32
float host_round_tf32(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return x;
    u += 0x1000u;
    u &= 0xFFFFE000u;
    std::memcpy(&x, &u, 4);
    return x;
}

// A slot of n elements in the weight arena: `dev` is the slot's offset as a tagged pointer (resolved by
// resolve_pack), `host` its zero-filled staging bytes to fill right away — valid until the next reserve — or nullptr
// when the arena is loaded from a pack file.
constexpr uintptr_t kPackTag = static_cast<uintptr_t>(1) << 44;
template <typename T> struct PackSlot { T *host; void *dev; };
template <typename T> PackSlot<T> reserve_pack(MsnhB200Plan *pl, size_t n) {
    const size_t off = pl->pack_cursor;
    pl->pack_cursor = (off + std::max<size_t>(n * sizeof(T), 16) + 255) / 256 * 256;
    PackSlot<T> s;
    s.dev = reinterpret_cast<void *>(kPackTag | off);
    s.host = nullptr;
    if (!pl->pack_loaded) {
        if (pl->pack_host.size() < pl->pack_cursor) pl->pack_host.resize(pl->pack_cursor, 0);
        s.host = reinterpret_cast<T *>(pl->pack_host.data() + off);
    }
    return s;
}
template <typename T> void *upload(MsnhB200Plan *pl, const std::vector<T> &host) {
    PackSlot<T> s = reserve_pack<T>(pl, host.size());
    if (s.host && !host.empty()) std::memcpy(s.host, host.data(), host.size() * sizeof(T));
    return s.dev;
}
template <typename P> void resolve_pack(const MsnhB200Plan *pl, P *&p) {
    const uintptr_t v = reinterpret_cast<uintptr_t>(p);
    if (v & kPackTag) p = reinterpret_cast<P *>(pl->d_pack + (v & (kPackTag - 1)));
}

// ---- pack file: header + the arena bytes -----------------------------------------------------------
// header, `bytes` of arena, then `picks` conv tile shapes (3 x int32 each: sub-tiles, channels, form) in launch order
struct PackHeader { char magic[8]; uint64_t key; uint64_t tag; uint64_t bytes; uint64_t picks; };
constexpr char kPackMagic[8] = {'M', 'S', 'N', 'H', 'P', 'K', '0', '2'};
uint64_t fnv1a(uint64_t h, const void *data, size_t n) {
    const uint8_t *p = static_cast<const uint8_t *>(data);
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}
// Everything the arena's layout and contents depend on besides the weight values themselves.
uint64_t pack_key(const MsnhB200Plan *pl) {
    uint64_t h = 1469598103934665603ull;
    for (const OpState &o : pl->ops) h = fnv1a(h, &o.d, sizeof(o.d));
    const int32_t v[9] = {pl->in_c, pl->in_h, pl->in_w, pl->batch, pl->dtype, static_cast<int32_t>(pl->flags & (MSNH_PLAN_NO_FUSION | MSNH_PLAN_NO_TENSOR_CORE | MSNH_PLAN_KEEP_ALL)), 6 /* layout version */,
                          pl->ctx->sm_count /* the stored tile shapes were timed on this many SMs */, std::getenv("MSNH_B200_NO_MERGE") ? 1 : 0};
    return fnv1a(h, v, sizeof(v));
}
bool read_pack_header(const MsnhB200Plan *pl, PackHeader *hd) {
    FILE *f = std::fopen(pl->pack_path.c_str(), "rb");
    if (!f) return false;
    bool ok = std::fread(hd, sizeof(*hd), 1, f) == 1 && std::memcmp(hd->magic, kPackMagic, 8) == 0 &&
              hd->key == pack_key(pl) && hd->tag == pl->pack_tag;
    // a file cut short (a writer that died, a full disk) is no pack
    ok = ok && std::fseek(f, 0, SEEK_END) == 0 && static_cast<uint64_t>(std::ftell(f)) == sizeof(*hd) + hd->bytes + hd->picks * 12;
    std::fclose(f);
    return ok;
}

// BatchNorm folded to y = x*scale + bias (scale = gamma/sqrt(var+eps), bias = beta - mean*scale),
// the same algebra as the reference's convBn kernel (src/layers/cuda/MsnhConvolutionalLayerGPU.cu:6-35).
void fold_bn(const OpState &o, int channels, std::vector<float> &scale, std::vector<float> &bias) {
    scale.resize(channels); bias.resize(channels);
    for (int c = 0; c < channels; ++c) {
        const float s = o.w[MSNH_W_BN_SCALE][c] / std::sqrt(o.w[MSNH_W_BN_VAR][c] + o.d.bn_eps);
        scale[c] = s;
        bias[c] = o.w[MSNH_W_BN_BIAS][c] - o.w[MSNH_W_BN_MEAN][c] * s;
    }
}

}  // namespace

// measured tile shapes, one entry per distinct conv layer signature (process-wide)
using TuneKey = std::array<int, 22>;
static std::mutex &tune_mutex() { static std::mutex m; return m; }
static std::map<TuneKey, std::array<int, 3>> &tune_cache() { static std::map<TuneKey, std::array<int, 3>> c; return c; }

static int build_launches(MsnhB200Plan *pl) {
    MsnhB200Ctx *ctx = pl->ctx;
    const int n_ops = static_cast<int>(pl->ops.size());
    const bool no_fusion = (pl->flags & MSNH_PLAN_NO_FUSION) != 0;
    const bool keep_all = (pl->flags & MSNH_PLAN_KEEP_ALL) != 0;
    // MSNH_B200_BUILD_TRACE=1: wall-clock of each stage of the build on stderr
    const bool build_trace = std::getenv("MSNH_B200_BUILD_TRACE") != nullptr;
    auto t_stage = std::chrono::steady_clock::now();
    auto stage = [&](const char *what) {
        if (!build_trace) return;
        const auto now = std::chrono::steady_clock::now();
        std::fprintf(stderr, "[msnh_b200 build] %-28s %8.2f ms\n", what, std::chrono::duration<double, std::milli>(now - t_stage).count());
        t_stage = now;
    };

    // A usable pack file stands in for the weights: the per-channel tensors are given zeros so that the folding
    // code below runs as usual (its results are discarded), the large repacking loops are skipped.
    PackHeader pack_hd{};
    pl->pack_cursor = 0; pl->pack_host.clear();
    pl->pack_loaded = !pl->pack_path.empty() && read_pack_header(pl, &pack_hd);
    const bool fresh = !pl->pack_loaded;
    if (fresh) {
        size_t guess = 0;
        for (const OpState &o : pl->ops) guess += o.wcount[MSNH_W_WEIGHTS] * static_cast<size_t>(esize(pl->dtype));
        pl->pack_host.reserve(guess + guess / 4 + (1u << 20));
    }
    for (int i = 0; i < n_ops; ++i) {
        OpState &o = pl->ops[i];
        if (!fresh) {
            for (int s = 0; s < MSNH_W_SLOTS; ++s)
                if (o.wcount[s] && (s != MSNH_W_WEIGHTS || o.d.kind == MSNH_OP_PRELU)) o.w[s].assign(o.wcount[s], 0.f);
            continue;
        }
        for (int s = 0; s < MSNH_W_SLOTS; ++s)
            if (o.wcount[s] && o.w[s].size() != o.wcount[s])
                return fail(ctx, MSNH_B200_ERR_STATE, "op %d: weight slot %d not set (%zu of %zu floats)", i, s, o.w[s].size(), o.wcount[s]);
        for (int k = 0; k < o.d.n_in; ++k)
            if (o.d.in[k] >= 0) pl->ops[o.d.in[k]].consumers.push_back(i);
    }

    // ---- 1. fusion: decide which ops are absorbed into an earlier launch ----
    std::vector<Fused> fused(n_ops);
    // 1a. concat of plain convs -> BatchNorm (-> activation), the CSP pattern of YOLOv5 (cv2 | cv3 -> cat -> bn -> act):
    //     each conv applies its channel slice of the BatchNorm and the activation in its own epilogue, and
    //     the BatchNorm / activation outputs become the concat buffer itself.
    std::vector<int> alias_to_op(n_ops, -1);       // absorbed op whose tensor is another op's tensor
    if (!no_fusion && !keep_all)
        for (int b = 0; b < n_ops; ++b) {
            OpState &bn = pl->ops[b];
            if (bn.d.kind != MSNH_OP_BATCHNORM || bn.absorbed_into >= 0 || bn.d.in[0] < 0) continue;
            const int cat = bn.d.in[0];
            OpState &co = pl->ops[cat];
            int only;
            if (co.d.kind != MSNH_OP_CONCAT || co.d.n_in < 2 || co.d.route_groups > 1 || !sole_consumer(pl, cat, &only) || only != b) continue;
            bool ok = true;
            for (int k = 0; k < co.d.n_in && ok; ++k) {
                const int src = co.d.in[k];
                if (src < 0) { ok = false; break; }
                const OpState &po = pl->ops[src];
                int cons;
                ok = po.d.kind == MSNH_OP_CONV && !po.d.has_bn && po.d.act == MSNH_ACT_NONE && po.absorbed_into < 0 &&
                     fused[src].cat_bn_op < 0 && sole_consumer(pl, src, &cons) && cons == cat;
                for (int j = 0; j < k; ++j) ok = ok && co.d.in[j] != src;
            }
            if (!ok) continue;
            int act_op = -1, a;
            if (bn.d.act == MSNH_ACT_NONE && !bn.d.is_output && sole_consumer(pl, b, &a) && pl->ops[a].d.kind == MSNH_OP_ACTIVATION) act_op = a;
            int off = 0;
            for (int k = 0; k < co.d.n_in; ++k) {
                const int src = co.d.in[k];
                fused[src].cat_bn_op = b; fused[src].cat_act_op = act_op; fused[src].cat_c_off = off;
                off += pl->ops[src].out.C;
            }
            bn.absorbed_into = co.d.in[0]; alias_to_op[b] = cat;
            if (act_op >= 0) { pl->ops[act_op].absorbed_into = co.d.in[0]; alias_to_op[act_op] = cat; }
        }
    for (int i = 0; i < n_ops; ++i) {
        OpState &o = pl->ops[i];
        if (o.absorbed_into >= 0) continue;
        Fused &f = fused[i];
        f.last_op = i;
        const int kind = o.d.kind;
        const bool conv_like = kind == MSNH_OP_CONV || kind == MSNH_OP_CONNECTED;
        const bool depthwise = kind == MSNH_OP_CONV && o.d.groups > 1;
        const bool deconv = kind == MSNH_OP_DECONV;   // its gather kernel applies act, then a following BatchNorm, then a route's add
        if (!(conv_like || deconv || kind == MSNH_OP_BATCHNORM || kind == MSNH_OP_ADD)) continue;
        if (f.cat_bn_op >= 0) continue;            // its BatchNorm and activation come through the concat (1a)
        int cur_act = o.d.act;
        int c;
        if ((deconv || (conv_like && !o.d.has_bn && cur_act == MSNH_ACT_NONE)) && sole_consumer(pl, f.last_op, &c) &&
            pl->ops[c].d.kind == MSNH_OP_BATCHNORM && pl->ops[c].absorbed_into < 0) {
            f.bn_op = c; f.last_op = c; pl->ops[c].absorbed_into = i; cur_act = pl->ops[c].d.act;
        }
        if (cur_act == MSNH_ACT_NONE && sole_consumer(pl, f.last_op, &c) && pl->ops[c].d.kind == MSNH_OP_ACTIVATION) {
            f.act_op = c; f.last_op = c; pl->ops[c].absorbed_into = i; cur_act = pl->ops[c].d.act;
        }
        if (((conv_like && !depthwise) || deconv) && sole_consumer(pl, f.last_op, &c) && pl->ops[c].d.kind == MSNH_OP_ADD &&
            pl->ops[c].d.n_in == 2 && pl->ops[c].absorbed_into < 0) {
            const MsnhB200Op &ad = pl->ops[c].d;
            const int other = ad.in[0] == f.last_op ? ad.in[1] : ad.in[0];
            // the residual must exist before this launch runs: an op computed earlier whose own
            // launch (if it is absorbed, its host launch) precedes op i
            int other_launch = other;
            if (other >= 0 && pl->ops[other].absorbed_into >= 0) other_launch = pl->ops[other].absorbed_into;
            if (other != f.last_op && other_launch < i) {
                f.add_op = c; f.res_op = other; f.last_op = c; pl->ops[c].absorbed_into = i;
                int c2;
                if (ad.act == MSNH_ACT_NONE && sole_consumer(pl, c, &c2) && pl->ops[c2].d.kind == MSNH_OP_ACTIVATION) {
                    f.act2_op = c2; f.last_op = c2; pl->ops[c2].absorbed_into = i;
                }
            }
        }
    }

    // YOLO heads whose only reader is the candidate collection are decoded inside it
    if (!no_fusion && !keep_all)
        for (int i = 0; i < n_ops; ++i) {
            OpState &o = pl->ops[i];
            int c;
            if (o.d.kind == MSNH_OP_YOLO && !o.d.is_output && sole_consumer(pl, i, &c) && pl->ops[c].d.kind == MSNH_OP_YOLO_COLLECT &&
                o.d.in[0] >= 0)
                o.decode_in_collect = true;
        }

    // ---- 2. tensors: one per launch-producing op; absorbed ops and identities alias ----
    pl->tensors.clear(); pl->buffers.clear(); pl->launches.clear();
    Shape in_s; in_s.C = pl->in_c; in_s.H = pl->in_h; in_s.W = pl->in_w;
    // First-layer patch mode: when the image feeds exactly one dense conv whose whole receptive
    // field (Cin*kh*kw values) fits one k-block, the input layout kernel writes the conv's patch
    // matrix [pixel][tap*Cin + c] directly and the conv runs as a 1x1 GEMM over it. An image has so
    // few channels that per-tap im2col loads would move 6 useful bytes per 32-byte row.
    int patch_op = -1, patch_k = 0;
    if (!no_fusion && !(pl->flags & MSNH_PLAN_NO_TENSOR_CORE)) {
        int users = 0, user = -1;
        for (int i = 0; i < n_ops; ++i) for (int k = 0; k < pl->ops[i].d.n_in; ++k) if (pl->ops[i].d.in[k] == MSNH_B200_INPUT) { ++users; user = i; }
        if (users == 1 && pl->ops[user].d.kind == MSNH_OP_CONV && pl->ops[user].d.groups == 1 && pl->ops[user].absorbed_into < 0 &&
            pl->in_c * pl->ops[user].d.k_h * pl->ops[user].d.k_w <= 64 && pl->ops[user].d.k_h * pl->ops[user].d.k_w > 1) {
            patch_op = user;
            patch_k = round_up(pl->in_c * pl->ops[user].d.k_h * pl->ops[user].d.k_w, 16);
            in_s.C = patch_k; in_s.H = pl->ops[user].out.H; in_s.W = pl->ops[user].out.W;
        }
    }
    pl->input_tensor = new_tensor(pl, in_s, pl->dtype);
    new_buffer(pl, pl->input_tensor);
    auto tensor_of = [&](int op) { return op == MSNH_B200_INPUT ? pl->input_tensor : pl->ops[op].tensor; };

    for (int i = 0; i < n_ops; ++i) {
        OpState &o = pl->ops[i];
        if (o.absorbed_into >= 0) continue;
        const bool single_alias = (o.d.kind == MSNH_OP_IDENTITY) ||
                                  (o.d.kind == MSNH_OP_ACTIVATION && o.d.act == MSNH_ACT_NONE && !o.d.is_output && !keep_all && !no_fusion) ||
                                  (o.d.kind == MSNH_OP_CONCAT && o.d.n_in == 1 && !no_fusion);
        if (single_alias && !no_fusion) {
            // identity / single-input route: a view of the input (one channel group of it for
            // grouped routes), no launch
            const int src = tensor_of(o.d.in[0]);
            Tensor t = pl->tensors[src];
            const int g = (o.d.kind == MSNH_OP_CONCAT && o.d.route_groups > 1) ? o.d.route_groups : 1;
            if (g > 1) { t.s.C = t.s.C / g; t.c_off += t.s.C * o.d.route_group_id; }
            pl->tensors.push_back(t);
            o.tensor = static_cast<int>(pl->tensors.size()) - 1;
            continue;
        }
        const int last = fused[i].last_op >= 0 ? fused[i].last_op : i;
        const int t = new_tensor(pl, pl->ops[last].out, pl->ops[last].out_dtype);
        new_buffer(pl, t);
        o.tensor = t;
        const Fused &f = fused[i];
        for (int a : {f.bn_op, f.act_op, f.add_op, f.act2_op}) if (a >= 0) pl->ops[a].tensor = t;
    }

    for (int i = 0; i < n_ops; ++i)
        if (alias_to_op[i] >= 0) pl->ops[i].tensor = pl->ops[alias_to_op[i]].tensor;

    // ---- 3. zero-copy concat: later concats first so nested concats resolve to one root ----
    std::vector<std::vector<int>> concat_copy(n_ops);   // inputs that still need a copy launch
    for (int i = n_ops - 1; i >= 0; --i) {
        OpState &o = pl->ops[i];
        if (o.d.kind != MSNH_OP_CONCAT || o.absorbed_into >= 0) continue;
        if (o.d.n_in == 1 && !no_fusion) continue;
        const int g = o.d.route_groups > 1 ? o.d.route_groups : 1;
        Tensor &dst = pl->tensors[o.tensor];
        int c_cursor = 0;
        for (int k = 0; k < o.d.n_in; ++k) {
            const int src_op = o.d.in[k];
            const int src_t = tensor_of(src_op);
            Tensor &st = pl->tensors[src_t];
            const int c_take = st.s.C / g;
            // a channel offset that is not a multiple of a 16-byte vector is only taken for producers
            // that write element by element (slice: the Focus layer's 3-channel pieces)
            const bool scalar_producer = src_op >= 0 && pl->ops[src_op].d.kind == MSNH_OP_SLICE;
            bool zero_copy = !no_fusion && g == 1 && src_op != MSNH_B200_INPUT && !st.placed && st.c_off == 0 &&
                             st.dtype == dst.dtype && ((c_cursor % vec_of(dst.dtype)) == 0 || scalar_producer) &&
                             pl->buffers[st.buffer].alias_of < 0 && st.buffer != dst.buffer;
            // every tensor sharing st's buffer (aliases made by identities) moves with it
            if (zero_copy) {
                // a tensor that is a strict channel-slice alias of another buffer cannot move
                for (const Tensor &other : pl->tensors)
                    if (&other != &st && other.buffer == st.buffer && (other.c_off != 0 || other.s.C != st.s.C)) zero_copy = false;
                // the same tensor twice in one concat: only the first occurrence is zero-copy
                for (int kk = 0; kk < k; ++kk) if (tensor_of(o.d.in[kk]) == src_t) zero_copy = false;
            }
            if (zero_copy) {
                Buffer &sb = pl->buffers[st.buffer];
                sb.alias_of = dst.buffer; sb.alias_c_off = dst.c_off + c_cursor;
                for (Tensor &other : pl->tensors) if (other.buffer == st.buffer) other.placed = true;
            } else {
                concat_copy[i].push_back(k);
            }
            c_cursor += c_take;
        }
    }

    // ---- 4. launches (arena pointers are patched in after allocation) ----
    struct Pending { Launch L; int in_t = -1, out_t = -1, res_t = -1; std::vector<int> add_t; int c_off_out = 0; int c_sub = -1; int c_in_off = 0; int c_in_sub = -1;
                     int out2_t = -1;      // second output tensor of a merged pair of 1x1 convs
                     std::vector<int> more_in_t, more_out_t; };   // further heads of a collect launch / further pools over one input
    std::vector<Pending> pend;
    auto push = [&](Pending p) { pend.push_back(std::move(p)); return static_cast<int>(pend.size()) - 1; };
    {
        Pending p; p.L.kind = L_INPUT; p.L.op = -1; p.L.dtype = pl->dtype; p.out_t = pl->input_tensor;
        if (patch_op >= 0) {
            const MsnhB200Op &c = pl->ops[patch_op].d;
            p.L.kind = L_INPUT_PATCH; p.L.op = patch_op;
            p.L.kh = c.k_h; p.L.kw = c.k_w; p.L.sh = c.stride_h; p.L.sw = c.stride_w; p.L.ph = c.pad_h; p.L.pw = c.pad_w; p.L.dh = c.dil_h; p.L.dw = c.dil_w;
            p.L.ival = pl->in_c; p.L.ival2 = pl->in_h; p.L.max_rows = pl->in_w;
            p.L.bytes = static_cast<double>(pl->in_c) * pl->in_h * pl->in_w * pl->batch * 4.0 +
                        static_cast<double>(patch_k) * pl->ops[patch_op].out.H * pl->ops[patch_op].out.W * pl->batch * esize(pl->dtype);
        }
        push(p);
    }
    const int es = esize(pl->dtype), V = vec_of(pl->dtype);
    for (int i = 0; i < n_ops; ++i) {
        OpState &o = pl->ops[i];
        if (o.absorbed_into >= 0) continue;
        const MsnhB200Op &d = o.d;
        const int in0 = tensor_of(d.in[0]);
        Shape a = pl->tensors[in0].s;
        Pending p; p.L.op = i; p.L.dtype = pl->dtype; p.in_t = in0; p.out_t = o.tensor;
        switch (d.kind) {
            case MSNH_OP_IDENTITY:
                if (!no_fusion) continue;
                p.L.kind = L_SBA; push(p); break;
            case MSNH_OP_CONV: case MSNH_OP_CONNECTED: {
                const Fused &f = fused[i];
                const bool fc = d.kind == MSNH_OP_CONNECTED;
                const bool patched = i == patch_op;
                if (patched) { a.C = pl->in_c; a.H = pl->in_h; a.W = pl->in_w; }   // the conv's real input, not the patch matrix
                const int kh = fc ? a.H : d.k_h, kw = fc ? a.W : d.k_w;
                const int groups = fc ? 1 : d.groups;
                const int cin_g = a.C / groups;
                const int cout = d.filters;
                // scale / bias
                std::vector<float> scale, bias;
                bool has_scale = false;
                if (d.has_bn) { fold_bn(o, cout, scale, bias); has_scale = true; }
                else { bias.assign(cout, 0.f); if (d.has_bias) bias = o.w[MSNH_W_BIAS]; }
                int act1 = d.act; float act1_p = d.act_param;
                if (f.bn_op >= 0) {
                    std::vector<float> s2, b2; fold_bn(pl->ops[f.bn_op], cout, s2, b2);
                    scale.resize(cout);
                    for (int c = 0; c < cout; ++c) { scale[c] = s2[c]; bias[c] = bias[c] * s2[c] + b2[c]; }
                    has_scale = true; act1 = pl->ops[f.bn_op].d.act; act1_p = pl->ops[f.bn_op].d.act_param;
                }
                if (f.act_op >= 0) { act1 = pl->ops[f.act_op].d.act; act1_p = pl->ops[f.act_op].d.act_param; }
                if (f.cat_bn_op >= 0) {   // this conv's channel slice of the BatchNorm behind the concat
                    std::vector<float> s2, b2; fold_bn(pl->ops[f.cat_bn_op], pl->ops[f.cat_bn_op].out.C, s2, b2);
                    scale.resize(cout);
                    for (int c = 0; c < cout; ++c) { scale[c] = s2[f.cat_c_off + c]; bias[c] = bias[c] * s2[f.cat_c_off + c] + b2[f.cat_c_off + c]; }
                    has_scale = true; act1 = pl->ops[f.cat_bn_op].d.act; act1_p = pl->ops[f.cat_bn_op].d.act_param;
                    if (f.cat_act_op >= 0) { act1 = pl->ops[f.cat_act_op].d.act; act1_p = pl->ops[f.cat_act_op].d.act_param; }
                }
                p.L.act1 = act1; p.L.act1_p = act1_p;
                if (f.add_op >= 0) {
                    p.res_t = tensor_of(f.res_op);
                    p.L.act2 = pl->ops[f.add_op].d.act; p.L.act2_p = pl->ops[f.add_op].d.act_param;
                    if (f.act2_op >= 0) { p.L.act2 = pl->ops[f.act2_op].d.act; p.L.act2_p = pl->ops[f.act2_op].d.act_param; }
                }
                // padded (scale with ones, bias with zeros): the tensor-core epilogue reads whole channel groups of
                // a tile. The scale stays out of the packed weights: a BatchNorm scale far from 1 would push
                // fp16 weights into the subnormal range.
                if (!has_scale) scale.assign(cout, 1.f);
                const bool dense = groups == 1;
                scale.resize(round_up(cout, 256) + 64, 1.f); bias.resize(round_up(cout, 256) + 64, 0.f);
                p.L.scale = (has_scale || dense) ? static_cast<const float *>(upload(pl, scale)) : nullptr;
                p.L.bias = static_cast<const float *>(upload(pl, bias));
                p.L.kh = kh; p.L.kw = kw; p.L.sh = fc ? 1 : d.stride_h; p.L.sw = fc ? 1 : d.stride_w;
                p.L.ph = fc ? 0 : d.pad_h; p.L.pw = fc ? 0 : d.pad_w; p.L.dh = fc ? 1 : d.dil_h; p.L.dw = fc ? 1 : d.dil_w;
                p.L.groups = groups;
                const int taps = kh * kw;
                const Shape os = pl->ops[i].out;
                p.L.flops = 2.0 * cin_g * taps * cout * os.H * os.W * pl->batch;
                p.L.bytes = (static_cast<double>(a.C) * a.H * a.W + static_cast<double>(cout) * os.H * os.W) * pl->batch * es +
                            static_cast<double>(o.wcount[MSNH_W_WEIGHTS]) * es;
                const bool depthwise = groups > 1 && groups == a.C && cout == a.C;
                const std::vector<float> &w = o.w[MSNH_W_WEIGHTS];
                if (depthwise) {
                    // [C][1][kh][kw] -> [tap][C]
                    p.L.kind = L_DWCONV;
                    if (pl->dtype == MSNH_B200_F16) {
                        PackSlot<__half> ps = reserve_pack<__half>(pl, static_cast<size_t>(taps) * cout);
                        __half *pk = ps.host;
                        if (pk) for (int c = 0; c < cout; ++c) for (int t = 0; t < taps; ++t) pk[static_cast<size_t>(t) * cout + c] = __float2half_rn(w[static_cast<size_t>(c) * taps + t]);
                        p.L.weights = ps.dev;
                    } else {
                        PackSlot<float> ps = reserve_pack<float>(pl, static_cast<size_t>(taps) * cout);
                        float *pk = ps.host;
                        if (pk) for (int c = 0; c < cout; ++c) for (int t = 0; t < taps; ++t) pk[static_cast<size_t>(t) * cout + c] = w[static_cast<size_t>(c) * taps + t];
                        p.L.weights = ps.dev;
                    }
                } else {
                    // [Cout][Cin/g][kh][kw] -> [Cout][tap][cin_pad], zero in the pad channels
                    // (patch mode: one "tap" of patch_k values ordered tap-major, like the patch matrix)
                    const int cin_pad = patched ? patch_k : round_up(cin_g, V);
                    const int tap_stride = patched ? cin_g : cin_pad;        // distance between taps inside a row
                    const size_t row_len = patched ? static_cast<size_t>(patch_k) : static_cast<size_t>(taps) * cin_pad;
                    p.L.cin_pad = cin_pad;
                    const size_t n = static_cast<size_t>(cout) * row_len;
                    // packed straight into the arena's staging bytes (zero-filled, so the pad channels stay zero)
                    if (pl->dtype == MSNH_B200_F16) {
                        PackSlot<__half> ps = reserve_pack<__half>(pl, n);
                        __half *pk = ps.host;
                        if (pk) parallel_rows(cout, static_cast<size_t>(cin_g) * taps, [&](int co) {
                            for (int ci = 0; ci < cin_g; ++ci) for (int t = 0; t < taps; ++t)
                                pk[static_cast<size_t>(co) * row_len + static_cast<size_t>(t) * tap_stride + ci] = __float2half_rn(w[(static_cast<size_t>(co) * cin_g + ci) * taps + t]);
                        });
                        p.L.weights = ps.dev;
                    } else {
                        PackSlot<float> ps = reserve_pack<float>(pl, n);
                        float *pk = ps.host;
                        const bool tc = groups == 1 && !(pl->flags & MSNH_PLAN_NO_TENSOR_CORE);
                        if (pk) parallel_rows(cout, static_cast<size_t>(cin_g) * taps, [&](int co) {
                            for (int ci = 0; ci < cin_g; ++ci) for (int t = 0; t < taps; ++t) {
                                const float v = w[(static_cast<size_t>(co) * cin_g + ci) * taps + t];
                                pk[static_cast<size_t>(co) * row_len + static_cast<size_t>(t) * tap_stride + ci] = tc ? host_round_tf32(v) : v;
                            }
                        });
                        p.L.weights = ps.dev;
                    }
                    const bool tensor_core = groups == 1 && !(pl->flags & MSNH_PLAN_NO_TENSOR_CORE) && p.L.sh <= 8 && p.L.sw <= 8 &&
                                             p.L.ph < 128 && p.L.pw < 128 && kh * p.L.dh < 256 && kw * p.L.dw < 256;
                    p.L.kind = tensor_core ? L_CONV_UMMA : L_CONV_DIRECT;
                    if (patched) { p.L.kh = p.L.kw = 1; p.L.sh = p.L.sw = 1; p.L.ph = p.L.pw = 0; p.L.dh = p.L.dw = 1; p.L.note = "patch-matrix input"; }
                }
                if (!p.L.weights || !p.L.bias) return fail(ctx, MSNH_B200_ERR_NOMEM, "weight upload failed for op %d", i);
                push(p);
                break;
            }
            case MSNH_OP_BATCHNORM: {
                std::vector<float> scale, bias; fold_bn(o, a.C, scale, bias);
                p.L.kind = L_SBA; p.L.scale = static_cast<const float *>(upload(pl, scale)); p.L.bias = static_cast<const float *>(upload(pl, bias));
                p.L.act1 = d.act; p.L.act1_p = d.act_param;
                if (fused[i].act_op >= 0) { p.L.act1 = pl->ops[fused[i].act_op].d.act; p.L.act1_p = pl->ops[fused[i].act_op].d.act_param; }
                p.L.bytes = 2.0 * a.C * a.H * a.W * pl->batch * es;
                push(p); break;
            }
            case MSNH_OP_ACTIVATION:
                if (d.act == MSNH_ACT_NONE && !d.is_output && !keep_all && !no_fusion) continue;   // aliased to its input above
                p.L.kind = L_SBA; p.L.act1 = d.act; p.L.act1_p = d.act_param; p.L.bytes = 2.0 * a.C * a.H * a.W * pl->batch * es; push(p); break;
            case MSNH_OP_PRELU: {
                std::vector<float> slope = o.w[MSNH_W_WEIGHTS];
                slope.resize(round_up(a.C, 8), 0.f);
                p.L.kind = L_PRELU; p.L.scale = static_cast<const float *>(upload(pl, slope));
                if (!p.L.scale) return fail(ctx, MSNH_B200_ERR_NOMEM, "slope upload failed for op %d", i);
                p.L.bytes = 2.0 * a.C * a.H * a.W * pl->batch * es;
                push(p); break;
            }
            case MSNH_OP_MAXPOOL: case MSNH_OP_AVGPOOL:
                if (d.kind == MSNH_OP_MAXPOOL && d.filters > 0) {
                    p.L.kind = L_MAXPOOL_DEPTH;
                    p.L.bytes = (static_cast<double>(a.C) + o.out.C) * a.H * a.W * pl->batch * es;
                    push(p); break;
                }
                p.L.kind = d.kind == MSNH_OP_MAXPOOL ? L_MAXPOOL : L_AVGPOOL;
                p.L.kh = d.k_h; p.L.kw = d.k_w; p.L.sh = d.stride_h; p.L.sw = d.stride_w; p.L.ph = d.pad_h; p.L.pw = d.pad_w;
                p.L.bytes = (static_cast<double>(a.C) * a.H * a.W + static_cast<double>(o.out.C) * o.out.H * o.out.W) * pl->batch * es;
                push(p); break;
            case MSNH_OP_DECONV: {
                // transposed conv = GEMM over the input pixels (a 1x1 conv producing kh*kw*Cout channels,
                // one group of Cout per tap) + a gather of the taps that land on each output pixel
                const int cout = d.filters, taps = d.k_h * d.k_w, cin = a.C;
                const std::vector<float> &w = o.w[MSNH_W_WEIGHTS];     // [Cin][Cout][kh][kw]
                Shape cs; cs.C = taps * cout; cs.H = a.H; cs.W = a.W;
                const int col_t = new_tensor(pl, cs, pl->dtype);
                new_buffer(pl, col_t);
                Pending g; g.L.op = i; g.L.dtype = pl->dtype; g.in_t = in0; g.out_t = col_t;
                const int cin_pad = round_up(cin, V);
                g.L.cin_pad = cin_pad; g.L.groups = 1;
                const bool tc = !(pl->flags & MSNH_PLAN_NO_TENSOR_CORE);
                const size_t rows = static_cast<size_t>(taps) * cout;
                if (pl->dtype == MSNH_B200_F16) {
                    PackSlot<__half> ps = reserve_pack<__half>(pl, rows * cin_pad);
                    __half *pk = ps.host;
                    if (pk) parallel_rows(static_cast<int>(rows), static_cast<size_t>(cin), [&](int r) {
                        const int t = r / cout, co = r % cout;
                        for (int ci = 0; ci < cin; ++ci) pk[static_cast<size_t>(r) * cin_pad + ci] = __float2half_rn(w[(static_cast<size_t>(ci) * cout + co) * taps + t]);
                    });
                    g.L.weights = ps.dev;
                } else {
                    PackSlot<float> ps = reserve_pack<float>(pl, rows * cin_pad);
                    float *pk = ps.host;
                    if (pk) parallel_rows(static_cast<int>(rows), static_cast<size_t>(cin), [&](int r) {
                        const int t = r / cout, co = r % cout;
                        for (int ci = 0; ci < cin; ++ci) {
                            const float v = w[(static_cast<size_t>(ci) * cout + co) * taps + t];
                            pk[static_cast<size_t>(r) * cin_pad + ci] = tc ? host_round_tf32(v) : v;
                        }
                    });
                    g.L.weights = ps.dev;
                }
                std::vector<float> ones(round_up(static_cast<int>(rows), 256) + 64, 1.f), zeros(round_up(static_cast<int>(rows), 256) + 64, 0.f);
                g.L.scale = static_cast<const float *>(upload(pl, ones));
                g.L.bias = static_cast<const float *>(upload(pl, zeros));
                g.L.kind = tc ? L_CONV_UMMA : L_CONV_DIRECT;
                g.L.flops = 2.0 * cin * static_cast<double>(rows) * a.H * a.W * pl->batch;
                g.L.bytes = (static_cast<double>(cin) + static_cast<double>(rows)) * a.H * a.W * pl->batch * es + static_cast<double>(rows) * cin * es;
                g.L.note = "deconv GEMM";
                if (!g.L.weights || !g.L.scale || !g.L.bias) return fail(ctx, MSNH_B200_ERR_NOMEM, "weight upload failed for op %d", i);
                push(g);
                p.in_t = col_t;
                p.L.kind = L_COL2IM; p.L.kh = d.k_h; p.L.kw = d.k_w; p.L.sh = d.stride_h; p.L.sw = d.stride_w; p.L.ph = d.pad_h; p.L.pw = d.pad_w;
                p.L.act1 = d.act; p.L.act1_p = d.act_param;
                {   // what the gather absorbed: BatchNorm (+ activation) behind the layer, then a residual add (+ activation)
                    const Fused &f = fused[i];
                    if (f.bn_op >= 0) {
                        std::vector<float> s2, b2; fold_bn(pl->ops[f.bn_op], cout, s2, b2);
                        s2.resize(round_up(cout, 8), 1.f); b2.resize(round_up(cout, 8), 0.f);
                        p.L.scale = static_cast<const float *>(upload(pl, s2)); p.L.bias2 = static_cast<const float *>(upload(pl, b2));
                        p.L.act_mid = pl->ops[f.bn_op].d.act; p.L.act_mid_p = pl->ops[f.bn_op].d.act_param;
                        if (f.act_op >= 0) { p.L.act_mid = pl->ops[f.act_op].d.act; p.L.act_mid_p = pl->ops[f.act_op].d.act_param; }
                    } else if (f.act_op >= 0) { p.L.act1 = pl->ops[f.act_op].d.act; p.L.act1_p = pl->ops[f.act_op].d.act_param; }
                    if (f.add_op >= 0) {
                        p.res_t = tensor_of(f.res_op);
                        p.L.act2 = pl->ops[f.add_op].d.act; p.L.act2_p = pl->ops[f.add_op].d.act_param;
                        if (f.act2_op >= 0) { p.L.act2 = pl->ops[f.act2_op].d.act; p.L.act2_p = pl->ops[f.act2_op].d.act_param; }
                    }
                }
                if (d.has_bias) {
                    std::vector<float> bias = o.w[MSNH_W_BIAS];
                    bias.resize(round_up(cout, 8), 0.f);
                    p.L.bias = static_cast<const float *>(upload(pl, bias));
                    if (!p.L.bias) return fail(ctx, MSNH_B200_ERR_NOMEM, "bias upload failed for op %d", i);
                }
                p.L.bytes = (static_cast<double>(rows) * a.H * a.W + static_cast<double>(cout) * o.out.H * o.out.W * (p.res_t >= 0 ? 2.0 : 1.0)) * pl->batch * es;
                push(p); break;
            }
            case MSNH_OP_CLIP:
                p.L.kind = L_CLIP; p.L.fval = d.const_val; p.L.act1_p = d.scale;
                p.L.bytes = 2.0 * a.C * a.H * a.W * pl->batch * es;
                push(p); break;
            case MSNH_OP_REMAP:
                p.L.kind = L_REMAP; p.L.ival = d.remap_kind;
                for (int k = 0; k < 3; ++k) p.L.slice_o[k] = d.remap_dims[k];
                p.L.bytes = 2.0 * a.C * a.H * a.W * pl->batch * es;
                push(p); break;
            case MSNH_OP_REDUCE:
                p.L.kind = L_REDUCE; p.L.ival = d.binary_kind; p.L.ival2 = d.binary_const ? 1 : 0;
                p.L.bytes = (static_cast<double>(a.C) * a.H * a.W + static_cast<double>(o.out.C) * o.out.H * o.out.W) * pl->batch * es;
                push(p); break;
            case MSNH_OP_UPSAMPLE:
                if (d.upsample_mode == MSNH_UPSAMPLE_BILINEAR) {
                    p.L.kind = L_BILINEAR; p.L.ival = d.align_corners ? 1 : 0;
                    // the reference's source steps, in float as it computes them (src/core/MsnhBlas.cpp:2409-2410)
                    p.L.fval   = d.align_corners ? (1.0f * (a.H - 1) / (o.out.H - 1)) : (1.0f * a.H / o.out.H);
                    p.L.act1_p = d.align_corners ? (1.0f * (a.W - 1) / (o.out.W - 1)) : (1.0f * a.W / o.out.W);
                    p.L.bytes = (static_cast<double>(a.C) * a.H * a.W + static_cast<double>(o.out.C) * o.out.H * o.out.W) * pl->batch * es;
                    push(p); break;
                }
                p.L.kind = L_UPSAMPLE; p.L.sh = d.stride_h; p.L.sw = d.stride_w; p.L.fval = d.scale == 0.f ? 1.f : d.scale;
                p.L.bytes = (static_cast<double>(a.C) * a.H * a.W + static_cast<double>(o.out.C) * o.out.H * o.out.W) * pl->batch * es;
                push(p); break;
            case MSNH_OP_CONCAT: {
                const int g = d.route_groups > 1 ? d.route_groups : 1;
                int c_cursor = 0;
                for (int k = 0; k < d.n_in; ++k) {
                    const int src_t = tensor_of(d.in[k]);
                    const int c_take = pl->tensors[src_t].s.C / g;
                    if (std::find(concat_copy[i].begin(), concat_copy[i].end(), k) != concat_copy[i].end()) {
                        Pending q; q.L.kind = L_SBA; q.L.op = i; q.L.dtype = pl->dtype; q.in_t = src_t; q.out_t = o.tensor;
                        q.c_off_out = c_cursor; q.c_sub = c_take; q.c_in_off = c_take * (g > 1 ? d.route_group_id : 0); q.c_in_sub = c_take;
                        q.L.bytes = 2.0 * c_take * a.H * a.W * pl->batch * es;
                        q.L.note = "concat copy";
                        push(q);
                    }
                    c_cursor += c_take;
                }
                break;
            }
            case MSNH_OP_ADD: {
                p.L.kind = L_ADD; p.L.act1 = d.act; p.L.act1_p = d.act_param;
                if (fused[i].act_op >= 0) { p.L.act1 = pl->ops[fused[i].act_op].d.act; p.L.act1_p = pl->ops[fused[i].act_op].d.act_param; }
                for (int k = 0; k < d.n_in; ++k) p.add_t.push_back(tensor_of(d.in[k]));
                p.L.bytes = (d.n_in + 1.0) * a.C * a.H * a.W * pl->batch * es;
                push(p); break;
            }
            case MSNH_OP_BINARY:
                p.L.kind = L_BINARY; p.L.ival = d.binary_kind; p.L.fval = d.const_val;
                if (!d.binary_const) p.res_t = tensor_of(d.in[1]);
                p.L.bytes = (d.binary_const ? 2.0 : 3.0) * a.C * a.H * a.W * pl->batch * es;
                push(p); break;
            case MSNH_OP_SLICE:
                p.L.kind = L_SLICE;
                for (int k = 0; k < 3; ++k) { p.L.slice_o[k] = d.slice_start[k]; p.L.slice_s[k] = d.slice_step[k]; }
                p.L.bytes = 2.0 * o.out.C * o.out.H * o.out.W * pl->batch * es;
                push(p); break;
            case MSNH_OP_PAD:
                p.L.kind = L_PAD; p.L.ph = d.pad_top; p.L.pw = d.pad_left; p.L.fval = d.const_val;
                p.L.bytes = (static_cast<double>(a.C) * a.H * a.W + static_cast<double>(o.out.C) * o.out.H * o.out.W) * pl->batch * es;
                push(p); break;
            case MSNH_OP_SOFTMAX:
                p.L.kind = L_SOFTMAX; p.L.ival = d.softmax_groups > 0 ? d.softmax_groups : 1;
                p.L.fval = d.softmax_temperature == 0.f ? 1.f : d.softmax_temperature;
                p.L.bytes = 2.0 * a.C * a.H * a.W * pl->batch * es;
                push(p); break;
            case MSNH_OP_YOLO:
                if (o.decode_in_collect) break;
                p.L.kind = L_YOLO; p.L.ival = d.yolo_classes; p.L.ival2 = d.yolo_type;
                p.L.fval = static_cast<float>(pl->in_h) / static_cast<float>(a.H);   // reference: orgHeight / outHeight
                for (int k = 0; k < 6; ++k) p.L.anchors[k] = d.yolo_anchors[k];
                p.L.bytes = static_cast<double>(a.C) * a.H * a.W * pl->batch * (es + 4.0);
                push(p); break;
            case MSNH_OP_YOLO_COLLECT: {
                Pending z; z.L.kind = L_COLLECT_ZERO; z.L.op = i; z.out_t = o.tensor; push(z);
                int order_base = 0;
                Pending raw; raw.L.kind = L_COLLECT_RAW; raw.L.op = i; raw.L.dtype = pl->dtype; raw.out_t = o.tensor; raw.L.fval = d.const_val;
                auto flush_raw = [&]() {
                    if (raw.L.heads.n) push(raw);
                    raw.L.heads.n = 0; raw.L.bytes = 0; raw.in_t = -1; raw.more_in_t.clear();
                };
                for (int k = 0; k < d.n_in; ++k) {
                    const OpState &head = pl->ops[d.in[k]];
                    const Shape hs = pl->tensors[tensor_of(d.in[k])].s;
                    if (head.decode_in_collect) {
                        // read the raw logits the head would have decoded; objectness of every cell, the rest for few.
                        // All such heads share one launch (up to four per launch).
                        if (raw.L.heads.n == 4) flush_raw();
                        YoloHead &yh = raw.L.heads.h[raw.L.heads.n++];
                        yh = YoloHead{};
                        yh.classes = head.d.yolo_classes; yh.yolo_type = head.d.yolo_type; yh.order_base = order_base;
                        yh.ratio = static_cast<float>(pl->in_h) / static_cast<float>(hs.H);
                        for (int e = 0; e < 3; ++e) { yh.an.w[e] = head.d.yolo_anchors[2 * e]; yh.an.h[e] = head.d.yolo_anchors[2 * e + 1]; }
                        const int t = tensor_of(head.d.in[0]);
                        if (raw.in_t < 0) raw.in_t = t; else raw.more_in_t.push_back(t);
                        raw.L.bytes += 3.0 * hs.H * hs.W * pl->batch * 32.0;
                    } else {
                        flush_raw();
                        Pending q; q.L.kind = L_COLLECT; q.L.op = i; q.in_t = tensor_of(d.in[k]); q.out_t = o.tensor;
                        q.L.ival = head.d.yolo_classes; q.L.fval = d.const_val; q.L.ival2 = order_base;
                        q.L.bytes = static_cast<double>(hs.C) * hs.H * hs.W * pl->batch * 4.0;
                        push(q);
                    }
                    order_base += 3 * hs.H * hs.W;
                }
                flush_raw();
                break;
            }
            default: return fail(ctx, MSNH_B200_ERR_UNSUPPORTED, "op %d: kind %d not supported", i, d.kind);
        }
    }

    // ---- 4a. two plain 1x1 convs that read the same tensor (the two branches a CSP stage opens with) run as one launch
    //          over the concatenated output channels: the input is read once and the MMAs are twice as wide. Each conv
    //          keeps its own output tensor; the kernel sends store slabs from channel `split_n` on to the second one.
    if (!no_fusion && !keep_all && !std::getenv("MSNH_B200_NO_MERGE")) {
        const int slab_cols = 128 / es;
        auto off_of = [](const void *tagged) { return static_cast<size_t>(reinterpret_cast<uintptr_t>(tagged) & (kPackTag - 1)); };
        auto plain_1x1 = [&](const Pending &q) {
            return q.L.kind == L_CONV_UMMA && q.L.op != patch_op && q.L.op >= 0 && pl->ops[q.L.op].d.kind == MSNH_OP_CONV && q.L.note.empty() && q.L.kh == 1 && q.L.kw == 1 &&
                   q.L.sh == 1 && q.L.sw == 1 && q.L.ph == 0 && q.L.pw == 0 && q.L.groups == 1 && q.res_t < 0 && q.out2_t < 0 && q.c_sub < 0 && q.L.act2 == MSNH_ACT_NONE;
        };
        auto same_data = [&](int t0, int t1) {
            const Tensor &x = pl->tensors[t0], &y = pl->tensors[t1];
            int ox = 0, oy = 0;
            return root_of(pl, x.buffer, &ox) == root_of(pl, y.buffer, &oy) && x.c_off + ox == y.c_off + oy && x.s.C == y.s.C && x.dtype == y.dtype;
        };
        for (size_t i = 0; i < pend.size(); ++i) {
            if (!plain_1x1(pend[i])) continue;
            const int ca = pl->tensors[pend[i].out_t].s.C;
            if (ca % slab_cols) continue;                     // the second conv's channels start on a store slab
            for (size_t j = i + 1; j < pend.size(); ++j) {
                const Pending &b = pend[j];
                Pending &a = pend[i];
                if (!plain_1x1(b) || !same_data(a.in_t, b.in_t) || b.out_t == a.out_t || b.L.act1 != a.L.act1 || b.L.act1_p != a.L.act1_p ||
                    b.L.cin_pad != a.L.cin_pad) continue;
                const int cb = pl->tensors[b.out_t].s.C;
                const size_t row_bytes = static_cast<size_t>(a.L.cin_pad) * es;
                const size_t wa = off_of(a.L.weights), wb = off_of(b.L.weights), sa = off_of(a.L.scale), sb = off_of(b.L.scale), ba = off_of(a.L.bias), bb = off_of(b.L.bias);
                PackSlot<uint8_t> ws = reserve_pack<uint8_t>(pl, (static_cast<size_t>(ca) + cb) * row_bytes);
                if (ws.host) {       // (nullptr: the arena comes from a pack file, which holds the merged copy at this offset)
                    std::memcpy(ws.host, pl->pack_host.data() + wa, ca * row_bytes);
                    std::memcpy(ws.host + ca * row_bytes, pl->pack_host.data() + wb, cb * row_bytes);
                }
                std::vector<float> sc(round_up(ca + cb, 256) + 64, 1.f), bi(round_up(ca + cb, 256) + 64, 0.f);
                if (!pl->pack_loaded) {
                    const uint8_t *base = pl->pack_host.data();
                    std::memcpy(sc.data(), base + sa, sizeof(float) * ca); std::memcpy(sc.data() + ca, base + sb, sizeof(float) * cb);
                    std::memcpy(bi.data(), base + ba, sizeof(float) * ca); std::memcpy(bi.data() + ca, base + bb, sizeof(float) * cb);
                }
                a.L.weights = ws.dev;
                a.L.scale = static_cast<const float *>(upload(pl, sc));
                a.L.bias = static_cast<const float *>(upload(pl, bi));
                a.out2_t = b.out_t; a.L.split_n = ca;
                const Shape is = pl->tensors[a.in_t].s;
                a.L.flops += b.L.flops;
                a.L.bytes += b.L.bytes - static_cast<double>(is.C) * is.H * is.W * pl->batch * es;
                a.L.note = "with the 1x1 conv of op " + std::to_string(b.L.op) + " (+" + std::to_string(cb) + " channels)";
                pend.erase(pend.begin() + static_cast<long>(j));
                break;                                        // one partner per launch
            }
        }
    }
    // ---- 4a'. stride-1 max pools that keep the plane size and read the same tensor one after the other (an SPP block) run as
    //           one launch: the plane is staged in shared memory once (maxpool_plane_kernel).
    if (!no_fusion && !keep_all && !std::getenv("MSNH_B200_NO_MERGE")) {
        auto same_pool = [&](const Pending &q) {
            if (q.L.kind != L_MAXPOOL || q.in_t < 0 || q.out_t < 0 || q.c_sub >= 0) return false;
            const Shape a = pl->tensors[q.in_t].s, b = pl->tensors[q.out_t].s;
            for (int t : {q.in_t, q.out_t}) {             // whole 16-byte channel vectors at vector-aligned channel offsets
                int off = 0;
                root_of(pl, pl->tensors[t].buffer, &off);
                if ((pl->tensors[t].c_off + off) % V || pl->tensors[t].s.C % V) return false;
            }
            return q.L.sh == 1 && q.L.sw == 1 && a.H == b.H && a.W == b.W && q.L.kh * q.L.kw > 9 && q.L.kh <= 2 * q.L.ph + 1 && q.L.kw <= 2 * q.L.pw + 1 &&
                   a.H * a.W * 32 <= 48 * 1024;
        };
        for (size_t i = 0; i + 1 < pend.size(); ++i) {
            if (!same_pool(pend[i])) continue;
            while (i + 1 < pend.size() && pend[i].more_out_t.size() < 2 && same_pool(pend[i + 1]) && pend[i + 1].in_t == pend[i].in_t) {
                Pending &a = pend[i]; const Pending &b = pend[i + 1];
                PoolSet &ps = a.L.pools;
                if (ps.n == 0) { ps.kh[0] = a.L.kh; ps.kw[0] = a.L.kw; ps.ph[0] = a.L.ph; ps.pw[0] = a.L.pw; ps.n = 1; }
                ps.kh[ps.n] = b.L.kh; ps.kw[ps.n] = b.L.kw; ps.ph[ps.n] = b.L.ph; ps.pw[ps.n] = b.L.pw; ++ps.n;
                a.more_out_t.push_back(b.out_t);
                const Shape is = pl->tensors[a.in_t].s;
                a.L.bytes += b.L.bytes - static_cast<double>(is.C) * is.H * is.W * pl->batch * es;
                a.L.note = (a.L.note.empty() ? "with the pool of op " : a.L.note + ", ") + std::to_string(b.L.op);
                pend.erase(pend.begin() + static_cast<long>(i) + 1);
            }
        }
    }
    stage("fold, repack");
    // ---- 4b. the weight arena: one allocation, one copy (from the staging bytes or from the pack file) ----
    {
        const size_t total = std::max<size_t>(pl->pack_cursor, 256);
        if (pl->pack_loaded && pack_hd.bytes != pl->pack_cursor)
            return fail(ctx, MSNH_B200_ERR_STATE, "pack file %s holds %llu bytes, this plan lays out %zu", pl->pack_path.c_str(),
                        static_cast<unsigned long long>(pack_hd.bytes), pl->pack_cursor);
        CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->d_pack), total));
        pl->dev_allocs.push_back(pl->d_pack);
        if (pl->pack_loaded) {
            FILE *f = std::fopen(pl->pack_path.c_str(), "rb");
            std::unique_ptr<uint8_t[]> buf(new (std::nothrow) uint8_t[pl->pack_cursor + 1]);
            bool ok = f && buf && std::fseek(f, sizeof(PackHeader), SEEK_SET) == 0 &&
                      std::fread(buf.get(), 1, pl->pack_cursor, f) == pl->pack_cursor;
            pl->pack_picks.assign(static_cast<size_t>(pack_hd.picks), std::array<int32_t, 3>{0, 0, 0});
            if (ok && pack_hd.picks) ok = std::fread(pl->pack_picks.data(), 12, pl->pack_picks.size(), f) == pl->pack_picks.size();
            if (f) std::fclose(f);
            if (!ok) return fail(ctx, MSNH_B200_ERR_STATE, "pack file %s is truncated or unreadable", pl->pack_path.c_str());
            CUDA_TRY(ctx, cudaMemcpy(pl->d_pack, buf.get(), pl->pack_cursor, cudaMemcpyHostToDevice));
        } else {
            if (pl->pack_cursor) CUDA_TRY(ctx, cudaMemcpy(pl->d_pack, pl->pack_host.data(), pl->pack_cursor, cudaMemcpyHostToDevice));
            pl->pack_picks.clear();
        }
        // (a pack file to write keeps the staging bytes until the conv tile shapes are known: end of step 6)
        if (pl->pack_loaded || pl->pack_path.empty()) std::vector<uint8_t>().swap(pl->pack_host);
        for (Pending &q : pend) { resolve_pack(pl, q.L.weights); resolve_pack(pl, q.L.scale); resolve_pack(pl, q.L.bias); resolve_pack(pl, q.L.bias2); }
    }
    stage("weight arena copy");
    // ---- 5. liveness + arena ----
    for (size_t s = 0; s < pend.size(); ++s) {
        const Pending &p = pend[s];
        if (p.in_t >= 0) touch(pl, p.in_t, static_cast<int>(s));
        if (p.out_t >= 0) touch(pl, p.out_t, static_cast<int>(s));
        if (p.out2_t >= 0) touch(pl, p.out2_t, static_cast<int>(s));
        for (int t : p.more_in_t) touch(pl, t, static_cast<int>(s));
        for (int t : p.more_out_t) touch(pl, t, static_cast<int>(s));
        if (p.res_t >= 0) touch(pl, p.res_t, static_cast<int>(s));
        for (int t : p.add_t) touch(pl, t, static_cast<int>(s));
    }
    for (int i = 0; i < n_ops; ++i) {
        const OpState &o = pl->ops[i];
        if ((o.d.is_output || keep_all) && o.tensor >= 0) pl->buffers[root_of(pl, pl->tensors[o.tensor].buffer, nullptr)].persistent = true;
    }
    // widen concat roots: a root's pitch is the concat's pitch already (children alias into it)
    std::vector<int> order;
    for (size_t b = 0; b < pl->buffers.size(); ++b) {
        Buffer &bf = pl->buffers[b];
        if (bf.alias_of >= 0 || bf.last < 0) continue;
        if (bf.persistent) bf.last = 1 << 30;
        bf.bytes = (bf.pixels * bf.ldc * esize(bf.dtype) + 1023) / 1024 * 1024;
        order.push_back(static_cast<int>(b));
    }
    std::sort(order.begin(), order.end(), [&](int x, int y) {
        if (pl->buffers[x].first != pl->buffers[y].first) return pl->buffers[x].first < pl->buffers[y].first;
        return x < y;
    });
    std::vector<int> placed;
    size_t arena = 0;
    for (int b : order) {
        Buffer &bf = pl->buffers[b];
        // candidate offsets: 0 and the end of every conflicting buffer; take the lowest that fits
        std::vector<std::pair<size_t, size_t>> busy;
        for (int q : placed) {
            const Buffer &o = pl->buffers[q];
            if (o.last < bf.first || o.first > bf.last) continue;
            busy.push_back({o.offset, o.offset + o.bytes});
        }
        std::sort(busy.begin(), busy.end());
        size_t off = 0;
        for (auto &iv : busy) {
            if (off + bf.bytes <= iv.first) break;
            off = std::max(off, iv.second);
        }
        bf.offset = off;
        arena = std::max(arena, off + bf.bytes);
        placed.push_back(b);
    }
    pl->arena_bytes = arena + 1024;
    CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->arena), pl->arena_bytes));
    CUDA_TRY(ctx, cudaMemset(pl->arena, 0, pl->arena_bytes));
    const size_t in_elems = static_cast<size_t>(pl->batch) * pl->in_c * pl->in_h * pl->in_w;
    CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->d_input), in_elems * sizeof(float)));
    CUDA_TRY(ctx, cudaMemset(pl->d_input, 0, in_elems * sizeof(float)));

    stage("arena");
    // ---- 6. resolve views, build tensor maps ----
    // MSNH_B200_AUTOTUNE=0 keeps the modelled tile shapes; plans made for debugging (no graph, no fusion, every output
    // kept, traced) keep them too
    bool autotune = !(pl->flags & (MSNH_PLAN_NO_GRAPH | MSNH_PLAN_NO_FUSION | MSNH_PLAN_KEEP_ALL | (std::getenv("MSNH_B200_TRACE_TUNE") ? 0u : static_cast<uint32_t>(MSNH_PLAN_TRACE))));
    if (const char *e = getenv("MSNH_B200_AUTOTUNE")) autotune = autotune && atoi(e) != 0;
    std::vector<std::array<int, 3>> tune_cands;
    size_t umma_seen = 0;                       // tensor-core conv launches configured so far (index into the pack's shapes)
    cudaEvent_t tune_ev0 = nullptr, tune_ev1 = nullptr;
    if (autotune) { CUDA_TRY(ctx, cudaEventCreate(&tune_ev0)); CUDA_TRY(ctx, cudaEventCreate(&tune_ev1)); }
    for (Pending &p : pend) {
        Launch &L = p.L;
        if (p.in_t >= 0) L.in = view_of(pl, p.in_t);
        if (p.out_t >= 0) L.out = view_of(pl, p.out_t);
        if (p.out2_t >= 0) L.out2 = view_of(pl, p.out2_t);
        if (L.kind == L_INPUT || L.kind == L_INPUT_PATCH) { L.in.ptr = pl->d_input; }
        if (p.c_sub >= 0) {   // concat copy: a channel window of the destination / source
            L.out.ptr = static_cast<uint8_t *>(L.out.ptr) + static_cast<size_t>(p.c_off_out) * es; L.out.C = p.c_sub;
            L.in.ptr = static_cast<uint8_t *>(L.in.ptr) + static_cast<size_t>(p.c_in_off) * es; L.in.C = p.c_in_sub;
        }
        if (p.res_t >= 0) { TView r = view_of(pl, p.res_t); L.res = r.ptr; L.ldc_res = r.ldc; }
        if (!p.add_t.empty()) {
            L.add.n = static_cast<int>(p.add_t.size());
            for (int k = 0; k < L.add.n; ++k) { TView r = view_of(pl, p.add_t[k]); L.add.ptr[k] = r.ptr; L.add.ldc[k] = r.ldc; }
        }
        // 16-byte vector path: channel count, pitches and base addresses all multiples of a vector
        auto aligned = [&](const TView &v) { return v.ptr == nullptr || ((reinterpret_cast<uintptr_t>(v.ptr) % 16 == 0) && (v.ldc % V == 0)); };
        L.vec = (L.out.C % V == 0) && aligned(L.in) && aligned(L.out) && (L.res == nullptr || (reinterpret_cast<uintptr_t>(L.res) % 16 == 0 && L.ldc_res % V == 0));
        for (int k = 0; k < L.add.n; ++k) if (reinterpret_cast<uintptr_t>(L.add.ptr[k]) % 16 || L.add.ldc[k] % V) L.vec = false;
        if (L.kind == L_AVGPOOL || L.kind == L_MAXPOOL || L.kind == L_UPSAMPLE || L.kind == L_PAD || L.kind == L_DWCONV || L.kind == L_BILINEAR || L.kind == L_CLIP || L.kind == L_PRELU) L.vec = L.vec && (L.in.C % V == 0);

        if (L.kind == L_MAXPOOL) {
            if (L.pools.n == 0) { L.pools.kh[0] = L.kh; L.pools.kw[0] = L.kw; L.pools.ph[0] = L.ph; L.pools.pw[0] = L.pw; L.pools.n = 1; }
            L.pools.out[0] = L.out;
            for (size_t k = 0; k < p.more_out_t.size(); ++k) {
                L.pools.out[k + 1] = view_of(pl, p.more_out_t[k]);
                L.vec = L.vec && aligned(L.pools.out[k + 1]) && L.pools.out[k + 1].C % V == 0;
            }
            if (!p.more_out_t.empty() && !L.vec) return fail(ctx, MSNH_B200_ERR_STATE, "merged pools of op %d landed on an unaligned view", L.op);
        }
        if (L.kind == L_COLLECT_RAW) {
            int end = 0;
            for (int k = 0; k < L.heads.n; ++k) {
                YoloHead &yh = L.heads.h[k];
                yh.in = k == 0 ? L.in : view_of(pl, p.more_in_t[k - 1]);
                end += yh.in.N * yh.in.H * yh.in.W * 3;
                yh.end = end;
            }
        }
        if (L.kind == L_COLLECT_ZERO || L.kind == L_COLLECT || L.kind == L_COLLECT_RAW) {
            // the collect op's tensor is [N][1][cells][8] fp32 rows; the counters sit behind them
            TView rows = view_of(pl, p.out_t);
            L.rows = static_cast<float *>(rows.ptr); L.max_rows = rows.W;
            L.counts = nullptr;   // patched below
            L.out.N = pl->batch;
        }
        if (L.kind == L_DWCONV && L.vec && L.kh == 3 && L.kw == 3 && L.dh == 1 && L.dw == 1 && L.sh == L.sw && (L.sh == 1 || L.sh == 2) &&
            !std::getenv("MSNH_B200_DW_SIMPLE")) {
            // Output tiles of th x 16 pixels x 32 channels; th (a multiple of the rows a thread computes) is the candidate that
            // loads and computes the fewest rows over the plane among those whose input tile fits a 24 KB stage.
            const int S = L.sh, R = dw_rows(S), iw = dw_in_w(S);
            DwTileParams &d = L.dwp;
            long best_cost = -1;
            for (int th = R; th <= 16; th += R) {
                const int ih = (th - 1) * S + 3;
                if (static_cast<size_t>(ih) * iw * kDwChannels * es > 24 * 1024) break;
                const int tiles = (L.out.H + th - 1) / th;
                const long cost = static_cast<long>(tiles) * (ih + th * S);
                if (best_cost < 0 || cost <= best_cost) { best_cost = cost; d.th = th; d.ih = ih; }
            }
            d.tiles_w = (L.out.W + kDwTileW - 1) / kDwTileW; d.tiles_h = (L.out.H + d.th - 1) / d.th;
            d.tiles_c = (L.in.C + kDwChannels - 1) / kDwChannels;
            d.ph = L.ph; d.pw = L.pw; d.act = L.act1; d.act_param = L.act1_p; d.err_flag = ctx->dev_err_flag;
            const size_t stage = (static_cast<size_t>(d.ih) * iw * kDwChannels * es + 127) / 128 * 128;
            L.smem = kDwStages * stage + 128;
            const int total = L.out.N * d.tiles_h * d.tiles_w * d.tiles_c;
            const int per_sm = std::max(1, std::min(4, static_cast<int>((200 * 1024) / (L.smem + 1024))));
            int grid = std::min(total, per_sm * ctx->sm_count);
            if (grid > d.tiles_c) grid -= grid % d.tiles_c;          // a CTA keeps its channel group from tile to tile
            L.grid = grid;
            // 4-D map of the input: channels, W, H, images; the box is one input tile
            cuuint64_t dims[4] = {static_cast<cuuint64_t>(L.in.C), static_cast<cuuint64_t>(L.in.W), static_cast<cuuint64_t>(L.in.H), static_cast<cuuint64_t>(L.in.N)};
            cuuint64_t strides[3] = {static_cast<cuuint64_t>(L.in.ldc) * es, static_cast<cuuint64_t>(L.in.W) * L.in.ldc * es, static_cast<cuuint64_t>(L.in.H) * L.in.W * L.in.ldc * es};
            cuuint32_t box[4] = {static_cast<cuuint32_t>(kDwChannels), static_cast<cuuint32_t>(iw), static_cast<cuuint32_t>(d.ih), 1};
            cuuint32_t estr[4] = {1, 1, 1, 1};
            const CUresult r = best_cost < 0 ? CUDA_ERROR_INVALID_VALUE :
                               ctx->encode_tiled(&L.map_a, tm_type(pl->dtype), 4, L.in.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                 CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r == CUDA_SUCCESS && L.smem <= 100 * 1024 && L.in.C % 4 == 0 && grid % d.tiles_c == 0) {
                L.dw_tile = true;
                auto opt_in = [](auto kernel) { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); };
                if (pl->dtype == MSNH_B200_F16) {
                    opt_in(dwconv3x3_tile_kernel<__half, 1, true>); opt_in(dwconv3x3_tile_kernel<__half, 1, false>);
                    opt_in(dwconv3x3_tile_kernel<__half, 2, true>); opt_in(dwconv3x3_tile_kernel<__half, 2, false>);
                } else {
                    opt_in(dwconv3x3_tile_kernel<float, 1, true>); opt_in(dwconv3x3_tile_kernel<float, 1, false>);
                    opt_in(dwconv3x3_tile_kernel<float, 2, true>); opt_in(dwconv3x3_tile_kernel<float, 2, false>);
                }
                char note[96];
                snprintf(note, sizeof(note), "tiles %dx%dx%d ch, grid %d, smem %zu", d.th, kDwTileW, kDwChannels, L.grid, L.smem);
                L.note = note;
            }
        }
        if (L.kind == L_CONV_UMMA) {
            // alignment the tensor-core path needs; otherwise fall back to the CUDA-core kernel
            const bool ok = aligned(L.in) && aligned(L.out) && (L.res == nullptr || (reinterpret_cast<uintptr_t>(L.res) % 16 == 0 && L.ldc_res % V == 0));
            if (!ok && p.out2_t >= 0) return fail(ctx, MSNH_B200_ERR_STATE, "merged 1x1 convs of op %d landed on an unaligned view", L.op);
            if (p.out2_t >= 0 && !aligned(L.out2)) return fail(ctx, MSNH_B200_ERR_STATE, "merged 1x1 convs of op %d: second output unaligned", L.op);
            if (!ok) { L.kind = L_CONV_DIRECT; L.note = "unaligned view: CUDA-core fallback"; }
        }
        if (L.kind == L_CONV_UMMA) {
            ConvUmmaParams &u = L.up;
            const int cin = L.in.C, cout = L.out.C + (L.out2.ptr ? L.out2.C : 0);   // (two merged convs: both channel ranges)
            u.split_n = L.out2.ptr ? L.split_n : 0x7fffffff;
            u.m_total = L.out.N * L.out.H * L.out.W;
            u.cout = cout;
            // Output channels per sub-tile (bn): a multiple of the 128-byte store slab once Cout exceeds one slab
            // (a slab must not spill into the next channel tile), otherwise Cout rounded up to 16. Chosen
            // together with the pixels per tile further down.
            const int slab_cols = 128 / es;
            u.bk_bytes = pick_bk_bytes(cin, es);
            u.bk_elems = u.bk_bytes / es;
            u.taps = L.kh * L.kw; u.kh = L.kh; u.kw = L.kw;
            u.chunks_per_tap = (cin + u.bk_elems - 1) / u.bk_elems;
            u.cin_pad = L.cin_pad;
            u.dil_h = L.dh; u.dil_w = L.dw;
            u.oh = L.out.H; u.ow = L.out.W; u.stride_h = L.sh; u.stride_w = L.sw; u.pad_h = L.ph; u.pad_w = L.pw;
            u.res = L.res; u.ldc_res = L.ldc_res;
            u.scale = L.scale; u.bias = L.bias;
            u.act1 = L.act1; u.act1_param = L.act1_p; u.act2 = L.act2; u.act2_param = L.act2_p;
            u.err_flag = ctx->dev_err_flag;
            u.round_tf32 = 0;
            u.trace = nullptr; u.trace_tile = 0;
            if (pl->flags & MSNH_PLAN_TRACE) {
                if (const char *e = getenv("MSNH_B200_TRACE_TILE")) u.trace_tile = atoi(e);
                void *tr = nullptr;
                CUDA_TRY(ctx, cudaMalloc(&tr, sizeof(long long) * kTraceSlots * ctx->sm_count));
                CUDA_TRY(ctx, cudaMemset(tr, 0, sizeof(long long) * kTraceSlots * ctx->sm_count));
                pl->dev_allocs.push_back(tr);
                u.trace = static_cast<long long *>(tr);
            }
            const uint32_t fmt = pl->dtype == MSNH_B200_F16 ? 0u : 2u;   // f16 / tf32 operands, f32 accumulate
            // the epilogue reads TMEM 32 columns at a time, so the last accumulator needs 32 columns of room
            const bool linear = L.kh == 1 && L.kw == 1 && L.sh == 1 && L.sw == 1 && L.ph == 0 && L.pw == 0;
            u.a_mode = linear ? A_MODE_LINEAR : A_MODE_IM2COL;
            const size_t fixed = 4 * kStageCBytes + 2 * 1024 + 512 + 2 * 4 * kSbMaxChannels;   // output staging slabs (2 per epilogue team), alignment slack, barriers, scale/bias tables
            const size_t budget = 227 * 1024 - fixed;
            // Tile shape: 128 * m_mult pixels x bn channels (m_mult MMAs of 128 x bn per 32 bytes of K, sharing
            // the weight tile). Measured on B200 (SM cycles): an MMA issues about every 156 cycles whatever its
            // width up to 224 columns (165 at 256) when its neighbours use other weight slices; consecutive MMAs
            // that share the weight slice (the sub-tiles of one k-step) issue every 48 + 108 / sub-tiles cycles
            // (102 for two, 75 for four); an im2col load costs about 600 cycles whatever its pixel count. So the main loop of a k-block takes
            // max(load issue, MMAs x issue interval, bytes / TMA rate), wide tiles are cheapest per FLOP, and
            // the choice below trades that against the number of tiles left to spread over the SMs.
            // Modelled cost: waves x k-blocks x k-block time + drain of the last tile + start-up.
            {
                const int k_iters = u.taps * u.chunks_per_tap;
                int forced_mm = 0, forced_bn = 0;
                if (const char *e = getenv("MSNH_B200_M_MULT")) forced_mm = atoi(e);
                if (const char *e = getenv("MSNH_B200_BN")) forced_bn = atoi(e);
                std::vector<int> bns;
                if (cout <= slab_cols) bns.push_back(round_up(cout, 16));
                else for (int bn = slab_cols; bn <= 256; bn += slab_cols) { bns.push_back(bn); if (bn >= cout) break; }
                double best = 1e30; int best_mm = 1, best_bn = bns[0], best_pair = 0, best_sk = 0;
                struct Cand { double cost; int mm, bn, sk; };
                std::vector<Cand> cands;                         // every plain (no pair, no stream-K) shape the layer allows
                // Stream-K (equal shares of tiles x k-blocks per SM, partial tiles handed over through global
                // memory): built and parity-tested; on YOLOv4-608 the hand-over (~6k cycles to write a 128 KB
                // partial tile, ~3-4k per slot to add it, serial on the critical path) eats what the balanced
                // shares save (2.646 vs 2.623 ms per step with the model below choosing), so it is off unless
                // MSNH_B200_STREAM_K asks for it: -1 by cost, 0 never (default), 1 whenever possible.
                int sk_mode = 0;
                if (const char *e = getenv("MSNH_B200_STREAM_K")) sk_mode = atoi(e);
                // CTA pairs (cta_group::2, tiles of 256 pixels x bn): measured no faster than single CTAs with
                // the same bn, because the MMA issue interval and not shared-memory traffic bounds the main
                // loop; kept selectable (MSNH_B200_PAIR=1) and covered by the GPU tests.
                int pair_mode = 0;
                if (const char *e = getenv("MSNH_B200_PAIR")) pair_mode = atoi(e);
                const int n_mma = u.bk_bytes / 32;
                auto kblock_cycles = [&](int mm, int bn, size_t stage_bytes, bool pair) {
                    // measured per-MMA interval: 48 + 108 / (sub-tiles sharing the weight tile) cycles, 165 for one sub-tile of 256 channels
                    const double interval = std::max(mm >= 2 ? 48.0 + 108.0 / mm : (bn > 224 ? 165.0 : 156.0), bn * 0.5);
                    const double issue = linear ? 150.0 * mm : 600.0;
                    (void)pair;
                    return std::max(std::max(issue, mm * n_mma * interval), static_cast<double>(stage_bytes) / 75.0);
                };
                for (int bn : bns) {
                    if (pair_mode != 1 || bn * es <= 128 || (forced_bn && bn != std::min(forced_bn, bns.back()))) continue;
                    const int tiles_n = (cout + bn - 1) / bn;
                    const size_t stage = static_cast<size_t>(kUmmaM + bn / 2) * u.bk_bytes;
                    const int pairs = ((u.m_total + 2 * kUmmaM - 1) / (2 * kUmmaM)) * tiles_n;
                    const double waves = std::ceil(static_cast<double>(pairs) / (ctx->sm_count / 2));
                    const double drain = 900.0 * ((((bn + slab_cols - 1) / slab_cols) + 1) / 2);
                    const double cost = (waves * k_iters * kblock_cycles(1, bn, stage, true) + drain + 3000.0) * 1e-3;
                    if (cost < best * 0.97) { best = cost; best_mm = 1; best_bn = bn; best_pair = 1; }
                }
                for (int bn : bns) {
                    if (forced_bn && bn != std::min(forced_bn, bns.back())) continue;
                    const int tiles_n = (cout + bn - 1) / bn;
                    for (int mm = 1; mm <= 4; ++mm) {
                        // 384 columns (3 x 128): one accumulator stage. 256 x 256 tiles (512 columns) were tried and lost
                        // to 128 x 192 on the layers they fit (46 vs 42 us on 3x3 256->512 at 38x38).
                        // Shapes that fill more than half of TMEM (a single accumulator stage, so the epilogue of a tile does
                        // not run under the next tile's main loop) are only offered to the measured choice, except 384 x 128.
                        if (mm * bn > 512) continue;
                        const bool measured_only = mm * bn > 256 && !(mm == 3 && bn == 128);
                        if (forced_mm && mm != forced_mm && !(mm == 1 && forced_mm * bn > 256)) continue;
                        const size_t stage = static_cast<size_t>(kUmmaM * mm + bn) * u.bk_bytes;
                        // stages to keep the loads ahead: two suffice when a k-block's MMAs outlast a load's latency
                        const size_t min_stages = (k_iters <= 2 || kblock_cycles(mm, bn, stage, false) >= 1000.0) ? 2 : 3;
                        if (budget / stage < min_stages && !(mm == 1 && bn == bns[0])) continue;
                        const int tiles = ((u.m_total + kUmmaM * mm - 1) / (kUmmaM * mm)) * tiles_n;
                        const double waves = std::ceil(static_cast<double>(tiles) / ctx->sm_count);
                        const double drain = 900.0 * ((mm * ((bn + slab_cols - 1) / slab_cols) + 1) / 2);
                        const double cost = waves * k_iters * kblock_cycles(mm, bn, stage, false) + drain + 2500.0;
                        cands.push_back({cost, mm, bn, 0});
                        // (sk = 2: the same 128-pixel tiles with the epilogue teams alternating over whole tiles)
                        if (mm == 1 && bn * es > 128 && tiles > ctx->sm_count) cands.push_back({cost * 1.02, mm, bn, 2});
                        if (measured_only && !(forced_mm && forced_bn)) continue;    // (forcing both picks such a shape: parity tests)
                        if (cost < best * 0.97 && sk_mode != 1) { best = cost; best_mm = mm; best_bn = bn; best_pair = 0; best_sk = 0; }
                        // stream-K: every SM takes units / SMs k-blocks; hand-over and completion of split tiles
                        // cost about one extra drain. Needs two store slabs per tile (both epilogue teams meet).
                        const long long units = static_cast<long long>(tiles) * k_iters;
                        const bool sk_fits = mm <= 2 && mm * ((bn + slab_cols - 1) / slab_cols) >= 2 && bn * es > 128 / (mm > 1 ? 2 : 1) &&
                                             units >= 2LL * ctx->sm_count && tiles % ctx->sm_count != 0;
                        if (sk_mode != 0 && sk_fits) {
                            const double share = std::ceil(static_cast<double>(units) / ctx->sm_count);
                            // measured: handing a 128 KB partial tile over costs ~6k cycles on the writer and ~3k per
                            // slot on the reader, one after the other on the critical path
                            const double parts = std::ceil(static_cast<double>(k_iters) / share);
                            double cost_sk = share * kblock_cycles(mm, bn, stage, false) + drain + 2500.0 +
                                             (6000.0 + 4000.0 * parts) * (mm * bn / 256.0);
                            if (sk_mode == 1) cost_sk *= 1e-3;
                            if (cost_sk < best * 0.95) { best = cost_sk; best_mm = mm; best_bn = bn; best_pair = 0; best_sk = 1; }
                        }
                    }
                }
                u.m_mult = best_mm; u.bn = best_bn; u.pair = best_pair; u.stream_k = best_sk;
                if (const char *e = getenv("MSNH_B200_NO_SPLIT")) L.no_split = atoi(e) != 0;   // parity tests of that epilogue form
                tune_cands.clear();
                // a pack file carries the shapes its plan ended up with: no need to time them again
                const bool stored = pl->pack_loaded && umma_seen < pl->pack_picks.size() && !forced_mm && !forced_bn && pair_mode != 1 && sk_mode == 0 &&
                                    !getenv("MSNH_B200_NO_SPLIT");
                if (stored) {
                    const std::array<int32_t, 3> &pk = pl->pack_picks[umma_seen];
                    bool valid = false;
                    for (const Cand &c : cands) valid = valid || (c.mm == pk[0] && c.bn == pk[1]);
                    if (valid) { u.m_mult = pk[0]; u.bn = pk[1]; u.pair = 0; u.stream_k = 0; L.no_split = (pk[2] & 0xff) == 2; if (pk[2] >= 0x100) L.note += L.note.empty() ? "measured shape" : ", measured shape"; }
                }
                if (!stored && autotune && !best_pair && !best_sk && !forced_mm && !forced_bn) {
                    std::sort(cands.begin(), cands.end(), [](const Cand &x, const Cand &y) { return x.cost < y.cost; });
                    // (stream-K forms were measured too and never won a layer; more than six runners-up changed nothing)
                    int tune_max = 6;
                    if (const char *e = getenv("MSNH_B200_AUTOTUNE")) tune_max = std::max(1, atoi(e));
                    for (const Cand &c : cands)
                        if (static_cast<int>(tune_cands.size()) < tune_max && !(c.mm == best_mm && c.bn == best_bn && c.sk == 0)) tune_cands.push_back({c.mm, c.bn, c.sk});
                }
            }
            // everything that follows from the tile shape in L.up: ring sizes, shared memory, grid, tensor maps
            auto configure = [&](Launch &L) -> int {
            ConvUmmaParams &u = L.up;
            u.tiles_n = (cout + u.bn - 1) / u.bn;
            u.out_chunk_bytes = u.bn * es >= 128 ? 128 : (u.bn * es >= 64 ? 64 : 32);
            const int tile_rows = u.pair ? 2 * kUmmaM : kUmmaM * u.m_mult;   // the pair's MMA spans 256 rows
            u.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(u.bn >> 3) << 17) |
                      (static_cast<uint32_t>((u.pair ? 2 * kUmmaM : kUmmaM) >> 4) << 24);
            u.tiles_m = (u.m_total + tile_rows - 1) / tile_rows;
            const int acc_cols = u.m_mult * u.bn;
            // accumulator ring: as many stages (2, 4, 8) as fit in the 512 TMEM columns; the epilogue reads 32
            // columns at a time, so the last accumulator needs up to 32 columns of room
            u.acc_shift = 2 * acc_cols - u.bn + round_up(u.bn, 32) <= 512 ? 1 : 0;   // (384-column tiles: a single stage)
            while (u.acc_shift >= 1 && u.acc_shift < 3 && (2 << u.acc_shift) * acc_cols - u.bn + round_up(u.bn, 32) <= 512) ++u.acc_shift;
            uint32_t cols = 32; while (cols < static_cast<uint32_t>((1 << u.acc_shift) * acc_cols - u.bn + round_up(u.bn, 32))) cols <<= 1;
            u.tmem_cols = cols;
            const int b_rows = u.pair ? u.bn / 2 : u.bn;                     // weight rows one CTA stages
            const size_t stage = static_cast<size_t>(kUmmaM * u.m_mult + b_rows) * u.bk_bytes;
            u.num_stages = static_cast<int>(std::min<size_t>(kUmmaMaxStages, budget / stage));
            L.smem = u.num_stages * stage + fixed;
            L.grid = u.pair ? 2 * std::min(u.tiles_m * u.tiles_n, ctx->sm_count / 2) : std::min(u.tiles_m * u.tiles_n, ctx->sm_count);
            u.sk_ws = nullptr; u.sk_flags = nullptr;
            if (u.stream_k) {
                // one hand-over slot (largest tile: 256 x 128 or 128 x 256 fp32) and one flag per CTA, shared by
                // all stream-K launches of the plan: a launch fills its slots only after its predecessor is complete
                L.grid = ctx->sm_count;
                if (!pl->sk_ws) {
                    CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->sk_ws), static_cast<size_t>(ctx->sm_count) * 256 * 256 * sizeof(float)));
                    CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->sk_flags), sizeof(int) * ctx->sm_count));
                    CUDA_TRY(ctx, cudaMemset(pl->sk_flags, 0, sizeof(int) * ctx->sm_count));
                    pl->dev_allocs.push_back(pl->sk_ws); pl->dev_allocs.push_back(pl->sk_flags);
                }
                u.sk_ws = pl->sk_ws; u.sk_flags = pl->sk_flags;
            }
            int rc;
            if (linear)
                rc = make_map_2d(ctx, &L.map_a, pl->dtype, L.in.ptr, static_cast<uint64_t>(cin), static_cast<uint64_t>(L.in.N) * L.in.H * L.in.W,
                                 static_cast<uint64_t>(L.in.ldc) * es, static_cast<uint32_t>(u.bk_elems), kUmmaM, u.bk_bytes);
            else
                rc = make_map_im2col(ctx, &L.map_a, pl->dtype, L.in, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, L.dh, L.dw, u.bk_elems, u.bk_bytes, kUmmaM * u.m_mult);
            if (rc) return rc;
            const uint64_t ktot = static_cast<uint64_t>(u.taps) * u.cin_pad;
            rc = make_map_2d(ctx, &L.map_b, pl->dtype, L.weights, ktot, static_cast<uint64_t>(cout), ktot * es,
                             static_cast<uint32_t>(u.bk_elems), static_cast<uint32_t>(b_rows), u.bk_bytes);
            if (rc) return rc;
            // store boxes: 32 rows (one warp's rows; plain kernels) or 128 (the team epilogue of the pair / stream-K kernels)
            const uint32_t store_rows = (u.pair || u.stream_k) ? kUmmaM : 32;
            rc = make_map_2d(ctx, &L.map_c, pl->dtype, L.out.ptr, static_cast<uint64_t>(L.out.C), static_cast<uint64_t>(u.m_total),
                             static_cast<uint64_t>(L.out.ldc) * es, static_cast<uint32_t>(u.out_chunk_bytes / es), store_rows, u.out_chunk_bytes);
            if (rc) return rc;
            if (L.out2.ptr) {
                rc = make_map_2d(ctx, &L.map_c2, pl->dtype, L.out2.ptr, static_cast<uint64_t>(L.out2.C), static_cast<uint64_t>(u.m_total),
                                 static_cast<uint64_t>(L.out2.ldc) * es, static_cast<uint32_t>(u.out_chunk_bytes / es), store_rows, u.out_chunk_bytes);
                if (rc) return rc;
            }
            u.sb_channels = round_up(cout, 64) <= kSbMaxChannels ? round_up(cout, 64) : 0;
            set_smem_attr(L);
            return MSNH_B200_OK;
            };
            // Measured choice: the modelled costs are within some ten percent of the truth, which is the margin
            // between neighbouring shapes, so the model's best shape and its runners-up are each run on the layer's
            // real buffers (contents do not matter) and the fastest wins. One measurement per distinct layer
            // signature and process; a shape has to beat the model's choice by 3 % to replace it.
            if (!tune_cands.empty()) {
                const TuneKey key{pl->dtype, pl->batch, cin, cout, L.in.H, L.in.W, L.out.H, L.out.W, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, L.dh, L.dw,
                                  L.act1, L.act2, L.res ? 1 : 0, L.in.ldc, L.out.ldc, ctx->sm_count};
                std::array<int, 3> pick{u.m_mult, u.bn, 0};
                bool known = false;
                { std::lock_guard<std::mutex> g(tune_mutex()); auto it = tune_cache().find(key); if (it != tune_cache().end()) { pick = it->second; known = true; } }
                if (!known) {
                    auto time_shape = [&](int mm, int bn, int sk, float *ms) -> int {
                        Launch t = L; t.up.m_mult = mm; t.up.bn = bn; t.up.pair = 0; t.up.stream_k = sk == 1; t.no_split = sk == 2;
                        const int rc = configure(t);
                        if (rc) return rc;
                        launch_one(ctx, t, ctx->stream);
                        *ms = 1e30f;
                        for (int rep = 0; rep < 2; ++rep) {          // the better of two short bursts
                            float burst = 0.f;
                            CUDA_TRY(ctx, cudaEventRecord(tune_ev0, ctx->stream));
                            for (int r = 0; r < 3; ++r) launch_one(ctx, t, ctx->stream);
                            CUDA_TRY(ctx, cudaEventRecord(tune_ev1, ctx->stream));
                            CUDA_TRY(ctx, cudaEventSynchronize(tune_ev1));
                            CUDA_TRY(ctx, cudaEventElapsedTime(&burst, tune_ev0, tune_ev1));
                            *ms = std::min(*ms, burst);
                        }
                        // a shape whose bounded waits ran out is no candidate (and must not leave the flag set)
                        int flag = 0;
                        CUDA_TRY(ctx, cudaMemcpy(&flag, ctx->dev_err_flag, sizeof(int), cudaMemcpyDeviceToHost));
                        if (flag != 0) { CUDA_TRY(ctx, cudaMemset(ctx->dev_err_flag, 0, sizeof(int))); *ms = 1e30f; }
                        return MSNH_B200_OK;
                    };
                    float best_ms = 0.f;
                    int rc = time_shape(u.m_mult, u.bn, 0, &best_ms);
                    if (rc) return rc;
                    if (best_ms > 1e29f) return fail(ctx, MSNH_B200_ERR_DEVICE_TIMEOUT, "a bounded wait ran out while timing the conv of op %d", L.op);
                    const float model_ms = best_ms;
                    for (const auto &c : tune_cands) {
                        float ms = 0.f;
                        rc = time_shape(c[0], c[1], c[2], &ms);
                        if (rc) return rc;
                        if (ms < best_ms && ms < model_ms * 0.97f) { best_ms = ms; pick = c; }
                    }
                    std::lock_guard<std::mutex> g(tune_mutex());
                    tune_cache()[key] = pick;
                }
                if (pick[0] != u.m_mult || pick[1] != u.bn || pick[2] != 0) { u.m_mult = pick[0]; u.bn = pick[1]; u.stream_k = pick[2] == 1; L.no_split = pick[2] == 2; L.note += L.note.empty() ? "measured shape" : ", measured shape"; }
            }
            { const int rc = configure(L); if (rc) return rc; }
            // form: 0 plain, 1 stream-K, 2 whole-tile epilogue teams, 4 CTA pair; + 0x100 when the shape was a measured choice
            if (!pl->pack_loaded) pl->pack_picks.push_back({u.m_mult, u.bn, (u.stream_k ? 1 : (u.pair ? 4 : (L.no_split ? 2 : 0))) | (L.note.find("measured shape") != std::string::npos ? 0x100 : 0)});
            ++umma_seen;
        }
        if (L.kind == L_CONV_DIRECT)
            L.tiled = L.groups == 1 && aligned(L.in) && (L.out.N * static_cast<long long>(L.out.H) * L.out.W + kCtBM - 1) / kCtBM < 2147483647LL &&
                      (L.out.C + kCtBN - 1) / kCtBN <= 65535 && !std::getenv("MSNH_B200_CONV_SIMPLE");
        if (L.kind == L_CONV_DIRECT && L.tiled) L.note += L.note.empty() ? "fp32 arithmetic, shared-memory tiles" : ", fp32 arithmetic, shared-memory tiles";
        pl->launches.push_back(L);
    }
    if (tune_ev0) { cudaEventDestroy(tune_ev0); cudaEventDestroy(tune_ev1); CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream)); }
    // fp32 plans: every launch that writes a tensor some tensor-core conv reads rounds to tf32
    if (pl->dtype == MSNH_B200_F32) {
        std::vector<std::pair<const uint8_t *, const uint8_t *>> reads;   // [begin, end) of root buffers read by UMMA convs
        for (size_t k = 0; k < pend.size(); ++k) {
            if (pl->launches[k].kind != L_CONV_UMMA) continue;
            const Buffer &b = pl->buffers[root_of(pl, pl->tensors[pend[k].in_t].buffer, nullptr)];
            reads.push_back({pl->arena + b.offset, pl->arena + b.offset + b.bytes});
        }
        for (size_t k = 0; k < pend.size(); ++k) {
            Launch &L = pl->launches[k];
            if (pend[k].out_t < 0) continue;
            bool hit = false;
            for (int t : {pend[k].out_t, pend[k].out2_t}) {
                if (t < 0) continue;
                const Buffer &b = pl->buffers[root_of(pl, pl->tensors[t].buffer, nullptr)];
                const uint8_t *lo = pl->arena + b.offset;
                for (auto &r : reads) if (lo >= r.first && lo < r.second) hit = true;
            }
            // buffers are reused over time, so this may round a little more than needed, never less
            if (hit) { L.out.tf32 = 1; if (L.kind == L_CONV_UMMA) L.up.round_tf32 = 1; }
        }
    }
    // candidate counters: one int per image per collect op
    {
        int n_collect = 0;
        for (const OpState &o : pl->ops) if (o.d.kind == MSNH_OP_YOLO_COLLECT) ++n_collect;
        if (n_collect) {
            int *d_counts = nullptr;
            CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&d_counts), sizeof(int) * pl->batch * n_collect));
            CUDA_TRY(ctx, cudaMemset(d_counts, 0, sizeof(int) * pl->batch * n_collect));
            pl->dev_allocs.push_back(d_counts);
            int idx = -1, cur_op = -1;
            for (Launch &L : pl->launches)
                if (L.kind == L_COLLECT_ZERO || L.kind == L_COLLECT || L.kind == L_COLLECT_RAW) {
                    if (L.op != cur_op) { cur_op = L.op; ++idx; }
                    L.counts = d_counts + static_cast<size_t>(idx) * pl->batch;
                }
            CUDA_TRY(ctx, cudaMallocHost(reinterpret_cast<void **>(&pl->h_counts), sizeof(int) * pl->batch));
        }
    }

    // ---- 6b. consecutive stride-2 slices of the image that fill one concat buffer side by side (YOLOv5's Focus)
    //          become one launch
    if (!no_fusion && !keep_all) {
        const int V = vec_of(pl->dtype);
        for (size_t k = 0; k + 1 < pl->launches.size(); ++k) {
            Launch &a = pl->launches[k];
            auto focus_like = [&](const Launch &L) {
                return L.kind == L_SLICE && L.in.C == 3 && L.in.ldc == V && L.slice_o[0] == 0 && L.slice_s[0] == 1 && L.slice_s[1] == 2 && L.slice_s[2] == 2 &&
                       L.slice_o[1] >= 0 && L.slice_o[1] < 2 && L.slice_o[2] >= 0 && L.slice_o[2] < 2 && L.out.C == 3 &&
                       reinterpret_cast<uintptr_t>(L.in.ptr) % 16 == 0;
            };
            if (!focus_like(a)) continue;
            size_t end = k + 1;
            while (end < pl->launches.size() && end - k < 4 && focus_like(pl->launches[end]) && pl->launches[end].in.ptr == a.in.ptr &&
                   pl->launches[end].out.ldc == a.out.ldc && pl->launches[end].out.H == a.out.H && pl->launches[end].out.W == a.out.W) ++end;
            const int n = static_cast<int>(end - k);
            const int outv = (4 * 3 + V - 1) / V * V;          // channels the fused kernel writes per pixel
            if (n < 2 || a.out.ldc != outv || reinterpret_cast<uintptr_t>(a.out.ptr) % 16 != 0) continue;
            // the slices must sit at channels 0, 3, 6, ... of the same pixel rows, in launch order
            bool ok = true;
            for (int j = 0; j < n; ++j)
                ok = ok && static_cast<const uint8_t *>(pl->launches[k + j].out.ptr) == static_cast<const uint8_t *>(a.out.ptr) + static_cast<size_t>(3 * j) * es;
            if (!ok || n != 4) continue;                        // (fewer slices would leave channels of other tensors to overwrite)
            Launch f = a;
            f.kind = L_FOCUS; f.focus.n = n; f.out.C = 3 * n; f.bytes = 0; f.note = "4 slices";
            for (int j = 0; j < n; ++j) { f.focus.o1[j] = pl->launches[k + j].slice_o[1]; f.focus.o2[j] = pl->launches[k + j].slice_o[2]; f.bytes += pl->launches[k + j].bytes; }
            pl->launches[k] = f;
            pl->launches.erase(pl->launches.begin() + static_cast<long>(k) + 1, pl->launches.begin() + static_cast<long>(end));
        }
    }

    if (!pl->pack_loaded && !pl->pack_path.empty()) {
        // written under a temporary name and renamed, so that a reader never sees half a file
        const std::string tmp = pl->pack_path + ".tmp";
        PackHeader hd{}; std::memcpy(hd.magic, kPackMagic, 8); hd.key = pack_key(pl); hd.tag = pl->pack_tag; hd.bytes = pl->pack_cursor; hd.picks = pl->pack_picks.size();
        FILE *f = std::fopen(tmp.c_str(), "wb");
        bool ok = f && std::fwrite(&hd, sizeof(hd), 1, f) == 1 && std::fwrite(pl->pack_host.data(), 1, pl->pack_cursor, f) == pl->pack_cursor &&
                  (pl->pack_picks.empty() || std::fwrite(pl->pack_picks.data(), 12, pl->pack_picks.size(), f) == pl->pack_picks.size());
        if (f) ok = (std::fclose(f) == 0) && ok;
        if (!ok || std::rename(tmp.c_str(), pl->pack_path.c_str()) != 0) std::remove(tmp.c_str());   // the cache is best effort
        std::vector<uint8_t>().swap(pl->pack_host);
    }
    stage("tile choice, tensor maps");
    // ---- 7. description ----
    {
        std::string s;
        char line[512];
        for (size_t k = 0; k < pl->launches.size(); ++k) {
            const Launch &L = pl->launches[k];
            snprintf(line, sizeof(line), "%zu %s op=%d in=%dx%dx%d(ld%d) out=%dx%dx%d(ld%d) k=%dx%d s=%d vec=%d flops=%.4g bytes=%.4g", k,
                     kLaunchNames[L.kind], L.op, L.in.C, L.in.H, L.in.W, L.in.ldc, L.out.C, L.out.H, L.out.W, L.out.ldc, L.kh, L.kw, L.sh,
                     L.vec ? 1 : 0, L.flops, L.bytes);
            s += line;
            if (L.kind == L_CONV_UMMA) {
                snprintf(line, sizeof(line), " tiles=%dx%d mm=%d%s%s%s bn=%d bk=%dB stages=%d mode=%s grid=%d smem=%zu", L.up.tiles_m, L.up.tiles_n, L.up.m_mult, L.up.pair ? " pair" : "", L.up.stream_k ? " streamk" : "", (L.no_split && L.up.m_mult == 1) ? " nosplit" : "", L.up.bn,
                         L.up.bk_bytes, L.up.num_stages, L.up.a_mode == A_MODE_LINEAR ? "linear" : "im2col", L.grid, L.smem);
                s += line;
            }
            if (!L.note.empty()) { s += " ["; s += L.note; s += "]"; }
            s += "\n";
        }
        pl->description = s;
    }
    return MSNH_B200_OK;
}

static int check_device_flag(MsnhB200Plan *pl) {
    int flag = 0;
    CUDA_TRY(pl->ctx, cudaMemcpy(&flag, pl->ctx->dev_err_flag, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag != 0) {
        cudaMemset(pl->ctx->dev_err_flag, 0, sizeof(int));
        return fail(pl->ctx, MSNH_B200_ERR_DEVICE_TIMEOUT, "a bounded wait inside the conv kernel ran out (code %d)", flag);
    }
    return MSNH_B200_OK;
}

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------
extern "C" {

int msnh_b200_device_count(int *count) {
    if (!count) return MSNH_B200_ERR_ARG;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { *count = 0; cudaGetLastError(); return MSNH_B200_ERR_CUDA; }
    *count = n;
    return MSNH_B200_OK;
}

int msnh_b200_ctx_create(int device, MsnhB200Ctx **out) {
    if (!out) return MSNH_B200_ERR_ARG;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) { cudaGetLastError(); return MSNH_B200_ERR_CUDA; }
    MsnhB200Ctx *ctx = new MsnhB200Ctx();
    ctx->device = device;
    cudaDeviceProp prop;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete ctx; return MSNH_B200_ERR_CUDA; }
    if (prop.major != 10) { delete ctx; return MSNH_B200_ERR_UNSUPPORTED; }   // sm_100a code only
    ctx->sm_count = prop.multiProcessorCount;
    { const char *e = getenv("MSNH_B200_NO_PDL"); ctx->pdl = !(e && e[0] == '1'); }
    cudaDriverGetVersion(&ctx->driver_version);
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) { delete ctx; return MSNH_B200_ERR_CUDA; }
    cudaDriverEntryPointQueryResult q;
    void *fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) { delete ctx; return MSNH_B200_ERR_CUDA; }
    ctx->encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) { delete ctx; return MSNH_B200_ERR_CUDA; }
    ctx->encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
    if (cudaMalloc(reinterpret_cast<void **>(&ctx->dev_err_flag), sizeof(int)) != cudaSuccess) { delete ctx; return MSNH_B200_ERR_NOMEM; }
    cudaMemset(ctx->dev_err_flag, 0, sizeof(int));
    *out = ctx;
    return MSNH_B200_OK;
}

int msnh_b200_ctx_destroy(MsnhB200Ctx *ctx) {
    if (!ctx) return MSNH_B200_ERR_ARG;
    cudaSetDevice(ctx->device);
    if (ctx->flush_buf) cudaFree(ctx->flush_buf);
    if (ctx->dev_err_flag) cudaFree(ctx->dev_err_flag);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return MSNH_B200_OK;
}

const char *msnh_b200_last_error(MsnhB200Ctx *ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int msnh_b200_host_alloc(MsnhB200Ctx *ctx, size_t bytes, void **ptr) {
    if (!ctx || !ptr) return MSNH_B200_ERR_ARG;
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    CUDA_TRY(ctx, cudaMallocHost(ptr, bytes));
    return MSNH_B200_OK;
}
int msnh_b200_host_free(MsnhB200Ctx *ctx, void *ptr) {
    if (!ctx) return MSNH_B200_ERR_ARG;
    CUDA_TRY(ctx, cudaFreeHost(ptr));
    return MSNH_B200_OK;
}

int msnh_b200_plan_create(MsnhB200Ctx *ctx, const MsnhB200Op *ops, int n_ops, int in_c, int in_h, int in_w, int batch,
                          int dtype, uint32_t flags, MsnhB200Plan **out) {
    if (!ctx || !ops || !out || n_ops <= 0) return fail(ctx, MSNH_B200_ERR_ARG, "plan_create: null or empty argument");
    *out = nullptr;
    if (in_c <= 0 || in_h <= 0 || in_w <= 0 || batch <= 0) return fail(ctx, MSNH_B200_ERR_ARG, "plan_create: bad input shape %dx%dx%d batch %d", in_c, in_h, in_w, batch);
    if (dtype != MSNH_B200_F32 && dtype != MSNH_B200_F16) return fail(ctx, MSNH_B200_ERR_ARG, "plan_create: dtype %d", dtype);
    MsnhB200Plan *pl = new MsnhB200Plan();
    pl->ctx = ctx; pl->in_c = in_c; pl->in_h = in_h; pl->in_w = in_w; pl->batch = batch; pl->dtype = dtype; pl->flags = flags;
    pl->ops.resize(n_ops);
    for (int i = 0; i < n_ops; ++i) {
        pl->ops[i].d = ops[i];
        std::string err;
        int rc = infer_shape(pl, i, err);
        if (rc) { int r = fail(ctx, rc, "op %d (kind %d): %s", i, ops[i].kind, err.c_str()); delete pl; return r; }
        if (ops[i].act < 0 || ops[i].act >= MSNH_ACT_COUNT) { int r = fail(ctx, MSNH_B200_ERR_UNSUPPORTED, "op %d: activation %d not supported", i, ops[i].act); delete pl; return r; }
    }
    // fp32 detection nets: fp32 arithmetic throughout unless tf32 is asked for (see MSNH_PLAN_TF32_DETECT)
    if (dtype == MSNH_B200_F32 && !(flags & MSNH_PLAN_TF32_DETECT))
        for (int i = 0; i < n_ops; ++i) if (ops[i].kind == MSNH_OP_YOLO) { pl->flags |= MSNH_PLAN_NO_TENSOR_CORE; break; }
    *out = pl;
    return MSNH_B200_OK;
}

int msnh_b200_plan_op_shape(MsnhB200Plan *pl, int op, int *c, int *h, int *w) {
    if (!pl || op < 0 || op >= static_cast<int>(pl->ops.size())) return MSNH_B200_ERR_ARG;
    if (c) *c = pl->ops[op].out.C; if (h) *h = pl->ops[op].out.H; if (w) *w = pl->ops[op].out.W;
    return MSNH_B200_OK;
}

int msnh_b200_plan_weight_count(MsnhB200Plan *pl, int op, int slot, size_t *count) {
    if (!pl || !count || op < 0 || op >= static_cast<int>(pl->ops.size()) || slot < 0 || slot >= MSNH_W_SLOTS) return MSNH_B200_ERR_ARG;
    *count = pl->ops[op].wcount[slot];
    return MSNH_B200_OK;
}

int msnh_b200_plan_set_weights(MsnhB200Plan *pl, int op, int slot, const float *data, size_t count) {
    if (!pl) return MSNH_B200_ERR_ARG;
    if (pl->finalized) return fail(pl->ctx, MSNH_B200_ERR_STATE, "set_weights after finalize");
    if (!data || op < 0 || op >= static_cast<int>(pl->ops.size()) || slot < 0 || slot >= MSNH_W_SLOTS) return fail(pl->ctx, MSNH_B200_ERR_ARG, "set_weights: bad argument");
    if (count != pl->ops[op].wcount[slot]) return fail(pl->ctx, MSNH_B200_ERR_ARG, "set_weights: op %d slot %d expects %zu floats, got %zu", op, slot, pl->ops[op].wcount[slot], count);
    pl->ops[op].w[slot].assign(data, data + count);
    return MSNH_B200_OK;
}

int msnh_b200_plan_use_pack(MsnhB200Plan *pl, const char *path, uint64_t weights_tag, int *usable) {
    if (!pl || !path || !*path) return MSNH_B200_ERR_ARG;
    if (pl->finalized) return fail(pl->ctx, MSNH_B200_ERR_STATE, "use_pack after finalize");
    pl->pack_path = path; pl->pack_tag = weights_tag;
    PackHeader hd{};
    if (usable) *usable = read_pack_header(pl, &hd) ? 1 : 0;
    return MSNH_B200_OK;
}

int msnh_b200_plan_finalize(MsnhB200Plan *pl) {
    if (!pl) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "finalize called twice");
    if (pl->finalize_failed) return fail(ctx, MSNH_B200_ERR_STATE, "an earlier finalize of this plan failed: destroy it and build a new one");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    int rc = build_launches(pl);
    if (rc) {
        // weights that were merely missing can still be set; anything later leaves half-built state behind
        bool missing_weights = rc == MSNH_B200_ERR_STATE && pl->launches.empty() && pl->tensors.empty();
        if (!missing_weights) pl->finalize_failed = true;
        for (OpState &o : pl->ops) o.consumers.clear();
        return rc;
    }
    CUDA_TRY(ctx, cudaEventCreate(&pl->ev0));
    CUDA_TRY(ctx, cudaEventCreate(&pl->ev1));
    for (OpState &o : pl->ops) for (int s = 0; s < MSNH_W_SLOTS; ++s) { std::vector<float>().swap(o.w[s]); }
    if (!(pl->flags & MSNH_PLAN_NO_GRAPH)) {
        CUDA_TRY(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        for (const Launch &L : pl->launches) launch_one(ctx, L, ctx->stream);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &pl->graph);
        if (e != cudaSuccess) return fail(ctx, MSNH_B200_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        CUDA_TRY(ctx, cudaGraphInstantiate(&pl->graph_exec, pl->graph, 0));
    }
    CUDA_TRY(ctx, cudaGetLastError());
    pl->finalized = true;
    return MSNH_B200_OK;
}

int msnh_b200_plan_input_buffer(MsnhB200Plan *pl, float **dev_ptr) {
    if (!pl || !dev_ptr) return MSNH_B200_ERR_ARG;
    if (!pl->finalized) return fail(pl->ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    *dev_ptr = pl->d_input;
    return MSNH_B200_OK;
}

static int run_common(MsnhB200Plan *pl, int sync) {
    MsnhB200Ctx *ctx = pl->ctx;
    CUDA_TRY(ctx, cudaEventRecord(pl->ev0, ctx->stream));
    if (pl->graph_exec) CUDA_TRY(ctx, cudaGraphLaunch(pl->graph_exec, ctx->stream));
    else for (const Launch &L : pl->launches) launch_one(ctx, L, ctx->stream);
    CUDA_TRY(ctx, cudaEventRecord(pl->ev1, ctx->stream));
    if (sync) {
        CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        CUDA_TRY(ctx, cudaEventElapsedTime(&pl->last_ms, pl->ev0, pl->ev1));
        return check_device_flag(pl);
    }
    return MSNH_B200_OK;
}

int msnh_b200_plan_run(MsnhB200Plan *pl, const float *host_nchw, int n_images) {
    if (!pl || !host_nchw) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    if (n_images < 1 || n_images > pl->batch) return fail(ctx, MSNH_B200_ERR_ARG, "n_images %d outside 1..%d", n_images, pl->batch);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const size_t bytes = static_cast<size_t>(n_images) * pl->in_c * pl->in_h * pl->in_w * sizeof(float);
    CUDA_TRY(ctx, cudaMemcpyAsync(pl->d_input, host_nchw, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return run_common(pl, 1);
}

int msnh_b200_plan_run_device(MsnhB200Plan *pl, const float *dev_nchw, int n_images, int sync) {
    if (!pl) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    if (n_images < 1 || n_images > pl->batch) return fail(ctx, MSNH_B200_ERR_ARG, "n_images %d outside 1..%d", n_images, pl->batch);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (dev_nchw && dev_nchw != pl->d_input) {
        const size_t bytes = static_cast<size_t>(n_images) * pl->in_c * pl->in_h * pl->in_w * sizeof(float);
        CUDA_TRY(ctx, cudaMemcpyAsync(pl->d_input, dev_nchw, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    }
    return run_common(pl, sync);
}

int msnh_b200_plan_run_timed(MsnhB200Plan *pl, int n_images, int steps, float *total_ms) {
    if (!pl || !total_ms || steps < 1) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    if (n_images < 1 || n_images > pl->batch) return fail(ctx, MSNH_B200_ERR_ARG, "n_images %d outside 1..%d", n_images, pl->batch);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(ctx, cudaEventRecord(pl->ev0, ctx->stream));
    for (int s = 0; s < steps; ++s) {
        if (pl->graph_exec) CUDA_TRY(ctx, cudaGraphLaunch(pl->graph_exec, ctx->stream));
        else for (const Launch &L : pl->launches) launch_one(ctx, L, ctx->stream);
    }
    CUDA_TRY(ctx, cudaEventRecord(pl->ev1, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(ctx, cudaEventElapsedTime(total_ms, pl->ev0, pl->ev1));
    pl->last_ms = *total_ms / steps;
    return check_device_flag(pl);
}

int msnh_b200_plan_run_instrumented(MsnhB200Plan *pl, int n_images, int steps, float *ms, int capacity) {
    if (!pl || !ms || steps < 1) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    const int n = static_cast<int>(pl->launches.size());
    if (capacity < n) return fail(ctx, MSNH_B200_ERR_ARG, "run_instrumented: capacity %d < %d launches", capacity, n);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    std::vector<cudaEvent_t> ev(static_cast<size_t>(n) + 1);
    for (auto &e : ev) CUDA_TRY(ctx, cudaEventCreate(&e));
    for (int k = 0; k < n; ++k) ms[k] = 0.f;
    for (int s = 0; s < steps; ++s) {
        CUDA_TRY(ctx, cudaEventRecord(ev[0], ctx->stream));
        for (int k = 0; k < n; ++k) {
            launch_one(ctx, pl->launches[k], ctx->stream);
            CUDA_TRY(ctx, cudaEventRecord(ev[k + 1], ctx->stream));
        }
        CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        for (int k = 0; k < n; ++k) {
            float t = 0.f;
            CUDA_TRY(ctx, cudaEventElapsedTime(&t, ev[k], ev[k + 1]));
            ms[k] += t;
        }
    }
    for (int k = 0; k < n; ++k) ms[k] /= steps;
    for (auto &e : ev) cudaEventDestroy(e);
    (void)n_images;
    return check_device_flag(pl);
}

int msnh_b200_plan_read_output(MsnhB200Plan *pl, int op, float *host, size_t count) {
    if (!pl || !host) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    if (op < 0 || op >= static_cast<int>(pl->ops.size())) return fail(ctx, MSNH_B200_ERR_ARG, "read_output: op %d", op);
    const OpState &o = pl->ops[op];
    if (!(o.d.is_output || (pl->flags & MSNH_PLAN_KEEP_ALL))) return fail(ctx, MSNH_B200_ERR_STATE, "op %d is not an output of this plan", op);
    if (o.d.kind == MSNH_OP_YOLO_COLLECT) return fail(ctx, MSNH_B200_ERR_ARG, "use plan_read_candidates for op %d", op);
    const size_t per = static_cast<size_t>(o.out.C) * o.out.H * o.out.W;
    if (count == 0 || count % per || count / per > static_cast<size_t>(pl->batch)) return fail(ctx, MSNH_B200_ERR_ARG, "read_output: count %zu is not 1..%d images of %zu", count, pl->batch, per);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (pl->readback_elems < count) {
        if (pl->d_readback) cudaFree(pl->d_readback);
        pl->d_readback = nullptr; pl->readback_elems = 0;
        CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->d_readback), count * sizeof(float)));
        pl->readback_elems = count;
    }
    TView v = view_of(pl, o.tensor);
    v.N = static_cast<int>(count / per);
    const int dt = pl->tensors[o.tensor].dtype;
    const int grid = grid_for(ctx, count, 256);
    if (dt == MSNH_B200_F16) nhwc_to_nchw_f32_kernel<__half><<<grid, 256, 0, ctx->stream>>>(v, pl->d_readback);
    else                     nhwc_to_nchw_f32_kernel<float><<<grid, 256, 0, ctx->stream>>>(v, pl->d_readback);
    CUDA_TRY(ctx, cudaMemcpyAsync(host, pl->d_readback, count * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return MSNH_B200_OK;
}

int msnh_b200_plan_read_candidates(MsnhB200Plan *pl, int op, int n_images, float *rows, int max_rows, int *counts) {
    if (!pl || !rows || !counts) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    if (op < 0 || op >= static_cast<int>(pl->ops.size()) || pl->ops[op].d.kind != MSNH_OP_YOLO_COLLECT) return fail(ctx, MSNH_B200_ERR_ARG, "op %d is not a yolo collect op", op);
    if (n_images < 1 || n_images > pl->batch || max_rows < 1) return fail(ctx, MSNH_B200_ERR_ARG, "read_candidates: bad n_images / max_rows");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const Launch *zl = nullptr;
    for (const Launch &L : pl->launches) if (L.kind == L_COLLECT_ZERO && L.op == op) zl = &L;
    if (!zl) return fail(ctx, MSNH_B200_ERR_STATE, "collect launch missing");
    CUDA_TRY(ctx, cudaMemcpyAsync(pl->h_counts, zl->counts, sizeof(int) * n_images, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    for (int i = 0; i < n_images; ++i) {
        int c = std::min(pl->h_counts[i], std::min(zl->max_rows, max_rows));
        counts[i] = c;
        if (c > 0)
            CUDA_TRY(ctx, cudaMemcpyAsync(rows + static_cast<size_t>(i) * max_rows * 8, zl->rows + static_cast<size_t>(i) * zl->max_rows * 8,
                                          sizeof(float) * 8 * c, cudaMemcpyDeviceToHost, ctx->stream));
    }
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    // restore the reference's scan order (the device appends in arbitrary order)
    struct Row { float v[8]; };
    for (int i = 0; i < n_images; ++i) {
        Row *r = reinterpret_cast<Row *>(rows + static_cast<size_t>(i) * max_rows * 8);
        std::sort(r, r + counts[i], [](const Row &a, const Row &b) { return a.v[7] < b.v[7]; });
    }
    return MSNH_B200_OK;
}

static int prep_params(MsnhB200Plan *pl, int width, int height, int mode, int swap_rgb, const float *mean, const float *std, PrepParams *p);

int msnh_b200_plan_preprocess_u8(MsnhB200Plan *pl, const unsigned char *host_hwc, int width, int height, int image, int mode,
                                 int swap_rgb, const float *mean, const float *std) {
    if (!pl || !host_hwc) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    if (image < 0 || image >= pl->batch) return fail(ctx, MSNH_B200_ERR_ARG, "preprocess_u8: image slot %d", image);
    PrepParams p{};
    { const int rc = prep_params(pl, width, height, mode, swap_rgb, mean, std, &p); if (rc) return rc; }
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const size_t bytes = static_cast<size_t>(width) * height * 3;
    if (bytes > pl->d_u8_bytes) {
        CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        if (pl->d_u8) cudaFree(pl->d_u8);
        pl->d_u8 = nullptr; pl->d_u8_bytes = 0;
        CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->d_u8), bytes));
        pl->d_u8_bytes = bytes;
    }
    CUDA_TRY(ctx, cudaMemcpyAsync(pl->d_u8, host_hwc, bytes, cudaMemcpyHostToDevice, ctx->stream));
    const dim3 grid((pl->in_w + 127) / 128, pl->in_h);
    preprocess_u8_kernel<<<grid, 128, 0, ctx->stream>>>(pl->d_u8, pl->d_input + static_cast<size_t>(image) * 3 * pl->in_h * pl->in_w, p);
    CUDA_TRY(ctx, cudaGetLastError());
    // the staging image may be overwritten by the next call: finish this one first
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return MSNH_B200_OK;
}

static int nms_buffers(MsnhB200Plan *pl) {
    MsnhB200Ctx *ctx = pl->ctx;
    if (pl->d_nms_boxes) return MSNH_B200_OK;
    CUDA_TRY(ctx, cudaFuncSetAttribute(yolo_nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kNmsSmemBytes)));
    CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->d_nms_boxes), sizeof(float) * 8 * kNmsMaxCandidates * pl->batch));
    CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->d_nms_counts), sizeof(int) * pl->batch));
    pl->dev_allocs.push_back(pl->d_nms_boxes); pl->dev_allocs.push_back(pl->d_nms_counts);
    return MSNH_B200_OK;
}

int msnh_b200_plan_nms(MsnhB200Plan *pl, int op, int n_images, float nms_thresh, int use_soft_nms, float sigma, float *boxes, int max_boxes, int *counts) {
    if (!pl || !boxes || !counts) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    if (op < 0 || op >= static_cast<int>(pl->ops.size()) || pl->ops[op].d.kind != MSNH_OP_YOLO_COLLECT) return fail(ctx, MSNH_B200_ERR_ARG, "op %d is not a yolo collect op", op);
    if (n_images < 1 || n_images > pl->batch || max_boxes < 1) return fail(ctx, MSNH_B200_ERR_ARG, "plan_nms: bad n_images / max_boxes");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const Launch *zl = nullptr;
    for (const Launch &L : pl->launches) if (L.kind == L_COLLECT_ZERO && L.op == op) zl = &L;
    if (!zl) return fail(ctx, MSNH_B200_ERR_STATE, "collect launch missing");
    int rc = nms_buffers(pl);
    if (rc) return rc;
    const int cap = std::min(max_boxes, kNmsMaxCandidates);
    yolo_nms_kernel<<<n_images, kNmsThreads, kNmsSmemBytes, ctx->stream>>>(zl->rows, zl->counts, zl->max_rows, nms_thresh, use_soft_nms, sigma,
                                                                pl->d_nms_boxes, kNmsMaxCandidates, pl->d_nms_counts);
    CUDA_TRY(ctx, cudaGetLastError());
    CUDA_TRY(ctx, cudaMemcpyAsync(pl->h_counts, pl->d_nms_counts, sizeof(int) * n_images, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    for (int i = 0; i < n_images; ++i) {
        counts[i] = pl->h_counts[i] < 0 ? -1 : std::min(pl->h_counts[i], cap);
        if (counts[i] > 0)
            CUDA_TRY(ctx, cudaMemcpyAsync(boxes + static_cast<size_t>(i) * max_boxes * 8, pl->d_nms_boxes + static_cast<size_t>(i) * kNmsMaxCandidates * 8,
                                          sizeof(float) * 8 * counts[i], cudaMemcpyDeviceToHost, ctx->stream));
    }
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return check_device_flag(pl);
}

int msnh_b200_plan_stream_nms(MsnhB200Plan *pl, int enable, float nms_thresh, int use_soft_nms, float sigma) {
    if (!pl) return MSNH_B200_ERR_ARG;
    if (pl->push_count != pl->pop_count) return fail(pl->ctx, MSNH_B200_ERR_STATE, "stream_nms: batches in flight");
    pl->stream_nms = enable != 0; pl->nms_thresh = nms_thresh; pl->nms_soft = use_soft_nms; pl->nms_sigma = sigma;
    return enable ? nms_buffers(pl) : MSNH_B200_OK;
}

// ---- pipelined streaming -------------------------------------------------------------------------
// Batch i+1 is copied host->device on the copy stream while batch i computes; the (small) result of
// batch i is copied back right behind its graph so the host can post-process it while batch i+1 runs.
static int stream_setup(MsnhB200Plan *pl, int op) {
    MsnhB200Ctx *ctx = pl->ctx;
    if (pl->copy_stream && pl->stream_op == op) return MSNH_B200_OK;
    if (pl->copy_stream) return fail(ctx, MSNH_B200_ERR_STATE, "streaming was set up for op %d; one result op per plan", pl->stream_op);
    if (op < 0 || op >= static_cast<int>(pl->ops.size())) return fail(ctx, MSNH_B200_ERR_ARG, "stream: op %d", op);
    const OpState &o = pl->ops[op];
    if (!(o.d.is_output || (pl->flags & MSNH_PLAN_KEEP_ALL))) return fail(ctx, MSNH_B200_ERR_STATE, "op %d is not an output of this plan", op);
    const size_t in_elems = static_cast<size_t>(pl->batch) * pl->in_c * pl->in_h * pl->in_w;
    if (o.d.kind == MSNH_OP_YOLO_COLLECT) {
        pl->stream_cap = std::min(o.out.W, 4096);                    // candidate rows kept per image
        pl->stream_result_floats = static_cast<size_t>(pl->batch) * pl->stream_cap * 8;
    } else {
        pl->stream_cap = 0;
        pl->stream_result_floats = static_cast<size_t>(pl->batch) * o.out.C * o.out.H * o.out.W;
    }
    CUDA_TRY(ctx, cudaStreamCreateWithFlags(&pl->copy_stream, cudaStreamNonBlocking));
    CUDA_TRY(ctx, cudaStreamCreateWithFlags(&pl->d2h_stream, cudaStreamNonBlocking));
    for (auto &s : pl->slots) {
        CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&s.d_stage), in_elems * sizeof(float)));
        CUDA_TRY(ctx, cudaMallocHost(reinterpret_cast<void **>(&s.h_result), pl->stream_result_floats * sizeof(float)));
        CUDA_TRY(ctx, cudaMallocHost(reinterpret_cast<void **>(&s.h_counts), sizeof(int) * (pl->batch + 1)));   // + the device error flag
        CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&s.d_result), pl->stream_result_floats * sizeof(float)));
        CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&s.d_counts), sizeof(int) * (pl->batch + 1)));
        CUDA_TRY(ctx, cudaEventCreateWithFlags(&s.fwd_done, cudaEventDisableTiming));
        CUDA_TRY(ctx, cudaEventCreateWithFlags(&s.h2d_done, cudaEventDisableTiming));
        CUDA_TRY(ctx, cudaEventCreateWithFlags(&s.consumed, cudaEventDisableTiming));
        CUDA_TRY(ctx, cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming));
    }
    pl->stream_op = op;
    return MSNH_B200_OK;
}

// One batch into the pipeline. `prep` == nullptr: host_images holds fp32 planar CHW images (what the reference's run* calls
// take); otherwise n_images 8-bit HWC images of prep->w x prep->h pixels, a quarter of the bytes over PCIe, which the
// preprocessing kernel turns into the plan's input on the compute stream (what the reference's runYoloList / runClassifyList
// do on the host before the forward, src/c_api/MsnhnetLib.cpp:508-560, 754-778).
static int stream_push_common(MsnhB200Plan *pl, int op, const void *host_images, int n_images, const PrepParams *prep) {
    if (!pl || !host_images) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    if (n_images < 1 || n_images > pl->batch) return fail(ctx, MSNH_B200_ERR_ARG, "n_images %d outside 1..%d", n_images, pl->batch);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    int rc = stream_setup(pl, op);
    if (rc) return rc;
    if (pl->push_count - pl->pop_count >= 2) return fail(ctx, MSNH_B200_ERR_STATE, "stream_push: both slots in flight, pop first");
    auto &s = pl->slots[pl->push_count & 1];
    const size_t image_floats = static_cast<size_t>(pl->in_c) * pl->in_h * pl->in_w;
    const size_t u8_per_image = prep ? static_cast<size_t>(prep->w) * prep->h * 3 : 0;
    const size_t bytes = prep ? static_cast<size_t>(n_images) * u8_per_image : static_cast<size_t>(n_images) * image_floats * sizeof(float);
    if (prep && bytes > static_cast<size_t>(pl->batch) * image_floats * sizeof(float))
        return fail(ctx, MSNH_B200_ERR_ARG, "stream_push_u8: %d images of %dx%d do not fit the staging buffer of a batch", n_images, prep->w, prep->h);
    // the slot's staging buffer was last read by the device copy of the batch two pushes ago
    if (pl->push_count >= 2) CUDA_TRY(ctx, cudaStreamWaitEvent(pl->copy_stream, s.consumed, 0));
    CUDA_TRY(ctx, cudaMemcpyAsync(s.d_stage, host_images, bytes, cudaMemcpyHostToDevice, pl->copy_stream));
    CUDA_TRY(ctx, cudaEventRecord(s.h2d_done, pl->copy_stream));
    CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, s.h2d_done, 0));
    if (prep) {
        const dim3 grid((pl->in_w + 127) / 128, pl->in_h);
        for (int i = 0; i < n_images; ++i)
            preprocess_u8_kernel<<<grid, 128, 0, ctx->stream>>>(reinterpret_cast<const unsigned char *>(s.d_stage) + static_cast<size_t>(i) * u8_per_image,
                                                                pl->d_input + static_cast<size_t>(i) * image_floats, *prep);
        CUDA_TRY(ctx, cudaGetLastError());
    } else {
        CUDA_TRY(ctx, cudaMemcpyAsync(pl->d_input, s.d_stage, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    }
    CUDA_TRY(ctx, cudaEventRecord(s.consumed, ctx->stream));
    if (pl->graph_exec) CUDA_TRY(ctx, cudaGraphLaunch(pl->graph_exec, ctx->stream));
    else for (const Launch &L : pl->launches) launch_one(ctx, L, ctx->stream);
    const OpState &o = pl->ops[op];
    // The result goes to the slot's own device buffer on the compute stream (a short device copy), and
    // from there to pinned host memory on a third stream, so the next forward does not wait for PCIe.
    // The conv kernels' error flag rides along.
    size_t result_bytes;
    if (pl->stream_cap) {
        const Launch *zl = nullptr;
        for (const Launch &L : pl->launches) if (L.kind == L_COLLECT_ZERO && L.op == op) zl = &L;
        if (!zl) return fail(ctx, MSNH_B200_ERR_STATE, "collect launch missing");
        if (pl->stream_nms) {
            // sort + NMS on the device, straight into the slot: only the kept boxes cross PCIe
            const int cap = std::min(pl->stream_cap, kNmsMaxCandidates);
            yolo_nms_kernel<<<n_images, kNmsThreads, kNmsSmemBytes, ctx->stream>>>(zl->rows, zl->counts, zl->max_rows, pl->nms_thresh, pl->nms_soft, pl->nms_sigma,
                                                                        s.d_result, pl->stream_cap, s.d_counts);
            (void)cap; result_bytes = 0;   // copied as a 2-D block below
        } else {
            CUDA_TRY(ctx, cudaMemcpyAsync(s.d_counts, zl->counts, sizeof(int) * n_images, cudaMemcpyDeviceToDevice, ctx->stream));
            CUDA_TRY(ctx, cudaMemcpy2DAsync(s.d_result, static_cast<size_t>(pl->stream_cap) * 32, zl->rows, static_cast<size_t>(zl->max_rows) * 32,
                                            static_cast<size_t>(pl->stream_cap) * 32, n_images, cudaMemcpyDeviceToDevice, ctx->stream));
            result_bytes = static_cast<size_t>(pl->stream_cap) * 32 * n_images;
        }
    } else {
        const size_t per = static_cast<size_t>(o.out.C) * o.out.H * o.out.W;
        TView v = view_of(pl, o.tensor);
        v.N = n_images;
        const int grid = grid_for(ctx, per * n_images, 256);
        if (pl->tensors[o.tensor].dtype == MSNH_B200_F16) nhwc_to_nchw_f32_kernel<__half><<<grid, 256, 0, ctx->stream>>>(v, s.d_result);
        else                                              nhwc_to_nchw_f32_kernel<float><<<grid, 256, 0, ctx->stream>>>(v, s.d_result);
        result_bytes = per * n_images * sizeof(float);
    }
    CUDA_TRY(ctx, cudaMemcpyAsync(s.d_counts + pl->batch, ctx->dev_err_flag, sizeof(int), cudaMemcpyDeviceToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaEventRecord(s.fwd_done, ctx->stream));
    CUDA_TRY(ctx, cudaStreamWaitEvent(pl->d2h_stream, s.fwd_done, 0));
    CUDA_TRY(ctx, cudaMemcpyAsync(s.h_counts, s.d_counts, sizeof(int) * (pl->batch + 1), cudaMemcpyDeviceToHost, pl->d2h_stream));
    if (pl->stream_cap && pl->stream_nms)
        CUDA_TRY(ctx, cudaMemcpy2DAsync(s.h_result, static_cast<size_t>(pl->stream_cap) * 32, s.d_result, static_cast<size_t>(pl->stream_cap) * 32,
                                        static_cast<size_t>(std::min(pl->stream_cap, kNmsMaxCandidates)) * 32, n_images, cudaMemcpyDeviceToHost, pl->d2h_stream));
    else
        CUDA_TRY(ctx, cudaMemcpyAsync(s.h_result, s.d_result, result_bytes, cudaMemcpyDeviceToHost, pl->d2h_stream));
    CUDA_TRY(ctx, cudaEventRecord(s.done, pl->d2h_stream));
    s.n_images = n_images; s.busy = true;
    ++pl->push_count;
    return MSNH_B200_OK;
}

int msnh_b200_plan_stream_push(MsnhB200Plan *pl, int op, const float *host_nchw, int n_images) {
    return stream_push_common(pl, op, host_nchw, n_images, nullptr);
}

static int prep_params(MsnhB200Plan *pl, int width, int height, int mode, int swap_rgb, const float *mean, const float *std, PrepParams *p) {
    MsnhB200Ctx *ctx = pl->ctx;
    if (pl->in_c != 3) return fail(ctx, MSNH_B200_ERR_UNSUPPORTED, "preprocess_u8: the net takes %d channels, 8-bit preprocessing is for 3", pl->in_c);
    if (width < 1 || height < 1) return fail(ctx, MSNH_B200_ERR_ARG, "preprocess_u8: bad size %dx%d", width, height);
    if (mode < MSNH_PREP_UNIT || mode > MSNH_PREP_CAFFE) return fail(ctx, MSNH_B200_ERR_ARG, "preprocess_u8: mode %d", mode);
    if (mode == MSNH_PREP_TRANSFORMED && (!mean || !std)) return fail(ctx, MSNH_B200_ERR_ARG, "preprocess_u8: mean or std can't be null");
    *p = PrepParams{};
    p->w = width; p->h = height; p->out_w = pl->in_w; p->out_h = pl->in_h;
    p->letterbox = mode == MSNH_PREP_PAD_SQUARE; p->rev_in = swap_rgb ? 0 : 1; p->rev_out = mode == MSNH_PREP_PAD_SQUARE ? 0 : 1;
    p->mode = mode;
    for (int k = 0; k < 3; ++k) { p->mean[k] = mean ? mean[k] : 0.f; p->std[k] = std ? std[k] : 1.f; }
    return MSNH_B200_OK;
}

int msnh_b200_plan_stream_push_u8(MsnhB200Plan *pl, int op, const unsigned char *host_hwc, int width, int height, int n_images, int mode,
                                  int swap_rgb, const float *mean, const float *std) {
    if (!pl || !host_hwc) return MSNH_B200_ERR_ARG;
    PrepParams p{};
    const int rc = prep_params(pl, width, height, mode, swap_rgb, mean, std, &p);
    if (rc) return rc;
    return stream_push_common(pl, op, host_hwc, n_images, &p);
}

int msnh_b200_plan_stream_pop(MsnhB200Plan *pl, float *result, size_t capacity_floats, int max_rows, int *counts, int *n_images) {
    if (!pl || !result) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (pl->pop_count >= pl->push_count) return fail(ctx, MSNH_B200_ERR_STATE, "stream_pop: nothing in flight");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    auto &s = pl->slots[pl->pop_count & 1];
    CUDA_TRY(ctx, cudaEventSynchronize(s.done));
    if (n_images) *n_images = s.n_images;
    if (pl->stream_cap) {
        if (!counts || max_rows < 1 || capacity_floats < static_cast<size_t>(s.n_images) * max_rows * 8)
            return fail(ctx, MSNH_B200_ERR_ARG, "stream_pop: rows buffer too small or counts missing");
        struct Row { float v[8]; };
        for (int i = 0; i < s.n_images; ++i) {
            // An image the streaming path cannot deliver whole is flagged with -1 and the slot is consumed all the same
            // (the caller runs that image again through plan_run + read_candidates / plan_nms, which keep every
            // candidate): the device NMS refused it (too many candidates, a class id beyond its table), or more
            // candidates passed the threshold than a slot holds - which of them arrived first is a matter of timing.
            if ((pl->stream_nms && s.h_counts[i] < 0) || (!pl->stream_nms && s.h_counts[i] > pl->stream_cap)) { counts[i] = -1; continue; }
            const int c = std::min(s.h_counts[i], std::min(pl->stream_cap, max_rows));
            counts[i] = c;
            Row *dst = reinterpret_cast<Row *>(result + static_cast<size_t>(i) * max_rows * 8);
            std::memcpy(dst, s.h_result + static_cast<size_t>(i) * pl->stream_cap * 8, sizeof(Row) * c);
            // candidates: restore the reference's scan order; device-NMS boxes already are in output order
            if (!pl->stream_nms) std::sort(dst, dst + c, [](const Row &a, const Row &b) { return a.v[7] < b.v[7]; });
        }
    } else {
        const OpState &o = pl->ops[pl->stream_op];
        const size_t n = static_cast<size_t>(s.n_images) * o.out.C * o.out.H * o.out.W;
        if (capacity_floats < n) return fail(ctx, MSNH_B200_ERR_ARG, "stream_pop: output buffer too small (%zu floats needed)", n);
        std::memcpy(result, s.h_result, n * sizeof(float));
    }
    s.busy = false;
    ++pl->pop_count;
    if (s.h_counts[pl->batch] != 0) return check_device_flag(pl);
    return MSNH_B200_OK;
}

int msnh_b200_plan_stream_reset(MsnhB200Plan *pl) {
    if (!pl) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (pl->copy_stream) CUDA_TRY(ctx, cudaStreamSynchronize(pl->copy_stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    if (pl->d2h_stream) CUDA_TRY(ctx, cudaStreamSynchronize(pl->d2h_stream));
    for (auto &s : pl->slots) s.busy = false;
    pl->pop_count = pl->push_count;
    return MSNH_B200_OK;
}

int msnh_b200_plan_last_ms(MsnhB200Plan *pl, float *ms) {
    if (!pl || !ms) return MSNH_B200_ERR_ARG;
    *ms = pl->last_ms;
    return MSNH_B200_OK;
}

int msnh_b200_plan_stats(MsnhB200Plan *pl, int *launches, size_t *arena_bytes) {
    if (!pl) return MSNH_B200_ERR_ARG;
    if (launches) *launches = static_cast<int>(pl->launches.size());
    if (arena_bytes) *arena_bytes = pl->arena_bytes;
    return MSNH_B200_OK;
}

const char *msnh_b200_plan_describe(MsnhB200Plan *pl) { return pl ? pl->description.c_str() : ""; }

int msnh_b200_plan_profile(MsnhB200Plan *pl, int iters, float *ms, int capacity) {
    if (!pl || !ms || iters < 1) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (!pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "plan not finalized");
    const int n = static_cast<int>(pl->launches.size());
    if (capacity < n) return fail(ctx, MSNH_B200_ERR_ARG, "profile: capacity %d < %d launches", capacity, n);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (!ctx->flush_buf) {
        ctx->flush_elems = static_cast<size_t>(256) * 1024 * 1024 / sizeof(float);   // 256 MiB > 126 MB L2
        CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&ctx->flush_buf), ctx->flush_elems * sizeof(float)));
    }
    // one full forward first so every launch sees real inputs
    for (const Launch &L : pl->launches) launch_one(ctx, L, ctx->stream);
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    for (int k = 0; k < n; ++k) {
        float total = 0.f;
        for (int it = 0; it < iters; ++it) {
            fill_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(ctx->flush_buf, ctx->flush_elems, 0.f);
            CUDA_TRY(ctx, cudaEventRecord(pl->ev0, ctx->stream));
            launch_one(ctx, pl->launches[k], ctx->stream);
            CUDA_TRY(ctx, cudaEventRecord(pl->ev1, ctx->stream));
            CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            float t = 0.f;
            CUDA_TRY(ctx, cudaEventElapsedTime(&t, pl->ev0, pl->ev1));
            total += t;
        }
        ms[k] = total / iters;
    }
    return check_device_flag(pl);
}

int msnh_b200_plan_read_trace(MsnhB200Plan *pl, int launch, long long *stamps, int capacity, int *ctas) {
    if (!pl || !stamps || !ctas) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (launch < 0 || launch >= static_cast<int>(pl->launches.size())) return fail(ctx, MSNH_B200_ERR_ARG, "read_trace: launch %d", launch);
    const Launch &L = pl->launches[launch];
    if (L.kind != L_CONV_UMMA || !L.up.trace) return fail(ctx, MSNH_B200_ERR_STATE, "launch %d has no trace (plan needs MSNH_PLAN_TRACE)", launch);
    const int n = L.grid * kTraceSlots;
    if (capacity < n) return fail(ctx, MSNH_B200_ERR_ARG, "read_trace: capacity %d < %d", capacity, n);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(ctx, cudaMemcpy(stamps, L.up.trace, sizeof(long long) * n, cudaMemcpyDeviceToHost));
    CUDA_TRY(ctx, cudaMemset(L.up.trace, 0, sizeof(long long) * n));
    *ctas = L.grid;
    return MSNH_B200_OK;
}

int msnh_b200_plan_destroy(MsnhB200Plan *pl) {
    if (!pl) return MSNH_B200_ERR_ARG;
    cudaSetDevice(pl->ctx->device);
    if (pl->graph_exec) cudaGraphExecDestroy(pl->graph_exec);
    if (pl->graph) cudaGraphDestroy(pl->graph);
    if (pl->ev0) cudaEventDestroy(pl->ev0);
    if (pl->ev1) cudaEventDestroy(pl->ev1);
    for (void *d : pl->dev_allocs) cudaFree(d);
    if (pl->arena) cudaFree(pl->arena);
    if (pl->d_input) cudaFree(pl->d_input);
    if (pl->d_readback) cudaFree(pl->d_readback);
    if (pl->d_u8) cudaFree(pl->d_u8);
    if (pl->h_counts) cudaFreeHost(pl->h_counts);
    for (auto &sl : pl->slots) {
        if (sl.d_stage) cudaFree(sl.d_stage);
        if (sl.d_result) cudaFree(sl.d_result);
        if (sl.h_result) cudaFreeHost(sl.h_result);
        if (sl.h_counts) cudaFreeHost(sl.h_counts);
        if (sl.h2d_done) cudaEventDestroy(sl.h2d_done);
        if (sl.consumed) cudaEventDestroy(sl.consumed);
        if (sl.done) cudaEventDestroy(sl.done);
        if (sl.d_counts) cudaFree(sl.d_counts);
        if (sl.fwd_done) cudaEventDestroy(sl.fwd_done);
    }
    if (pl->copy_stream) cudaStreamDestroy(pl->copy_stream);
    if (pl->d2h_stream) cudaStreamDestroy(pl->d2h_stream);
    delete pl;
    return MSNH_B200_OK;
}

}  // extern "C"
