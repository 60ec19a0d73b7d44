// Shared declarations of the plan compiler and executor behind include/msnh_b200.h: the context, the plan's data model
// (ops, tensors, buffers, launches), the debug switches, and the functions its translation units call across files:
//   plan.cu          context, plan lifetime, run / read-back entry points
//   plan_shapes.cu   shape inference and validation of the op list
//   plan_build.cu    lowering: fusion, tensors, zero-copy concat, launches, liveness arena, description
//   plan_tiles.cu    tensor maps; tile-shape model and measured choice of the tensor-core conv; depthwise tiles
//   plan_pack.cu     weight arena staging and the pack cache file
//   plan_launch.cu   the only file that compiles the kernels: one launch per Launch record, small launch wrappers
//   plan_stream.cu   preprocessing, device NMS and the pipelined streaming calls
#pragma once
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
#include "kernel_params.h"

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

namespace msnh {

// records the message on the context (when there is one) and returns `code`
int fail(MsnhB200Ctx *ctx, int code, const char *fmt, ...);
#define CUDA_TRY(ctx, expr)                                                                          \
    do {                                                                                             \
        cudaError_t e_ = (expr);                                                                     \
        if (e_ != cudaSuccess)                                                                       \
            return fail(ctx, MSNH_B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                        __FILE__, __LINE__);                                                         \
    } while (0)

// Debug switches, read from the environment once per plan_finalize (and context creation). They change how a plan is
// built, never what it computes.
struct PlanDebugOptions {
    bool no_pdl = false;        // MSNH_B200_NO_PDL=1: plain stream order between kernels
    bool no_merge = false;      // MSNH_B200_NO_MERGE: no sibling 1x1 / SPP pool merging
    bool build_trace = false;   // MSNH_B200_BUILD_TRACE: wall-clock of each build stage on stderr
    bool trace_tune = false;    // MSNH_B200_TRACE_TUNE: traced plans take the measured tile shapes too
    bool dw_simple = false;     // MSNH_B200_DW_SIMPLE: depthwise 3x3 without the shared-memory tile kernel
    int dw_th = 0, dw_stages = 0;   // MSNH_B200_DW_TH, MSNH_B200_DW_STAGES: force the depthwise tile height / ring depth
    bool conv_simple = false;   // MSNH_B200_CONV_SIMPLE: CUDA-core convs without the shared-memory tiled kernel
    int autotune = -1;          // MSNH_B200_AUTOTUNE: -1 unset (time six runners-up), 0 off, n runners-up
    int trace_tile = 0;         // MSNH_B200_TRACE_TILE: which tile of a CTA the producer / MMA stamps describe
    int forced_mm = 0, forced_bn = 0;   // MSNH_B200_M_MULT, MSNH_B200_BN: force the conv tile shape
    int stream_k = 0;           // MSNH_B200_STREAM_K: -1 by cost, 0 never, 1 wherever possible
    int pair = 0;               // MSNH_B200_PAIR: 1 = CTA pairs wherever possible
    int no_split = -1;          // MSNH_B200_NO_SPLIT: -1 unset, else the epilogue teams alternate over whole tiles (1) or not (0)
    static PlanDebugOptions from_env();
    // any switch that forces tile shapes: such plans neither take shapes from a pack file nor write one
    bool forces_tiles() const { return forced_mm || forced_bn || pair == 1 || stream_k != 0 || no_split >= 0; }
};

// ------------------------------------------------------------------------------------------------
// plan data model
// ------------------------------------------------------------------------------------------------
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
extern const char *const kLaunchNames[];

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
    bool focus_planar = false;                   // ... read straight from the planar fp32 image (in.ptr = the input staging)
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

// A launch while it is being planned: tensors by id, arena pointers patched in after allocation.
struct Pending { Launch L; int in_t = -1, out_t = -1, res_t = -1; std::vector<int> add_t; int c_off_out = 0; int c_sub = -1; int c_in_off = 0; int c_in_sub = -1;
                 int out2_t = -1;      // second output tensor of a merged pair of 1x1 convs
                 std::vector<int> more_in_t, more_out_t; };   // further heads of a collect launch / further pools over one input

}  // namespace msnh

struct MsnhB200Plan {
    MsnhB200Ctx *ctx = nullptr;
    int in_c = 0, in_h = 0, in_w = 0, batch = 0, dtype = 0;
    uint32_t flags = 0;
    msnh::PlanDebugOptions dbg;                     // the debug switches as they stood when plan_finalize began
    std::vector<msnh::OpState> ops;
    std::vector<msnh::Tensor> tensors;
    std::vector<msnh::Buffer> buffers;
    std::vector<msnh::Launch> launches;
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
    std::vector<uint8_t> pack_blob; uint64_t pack_blob_bytes = 0, pack_blob_key = 0, pack_blob_tag = 0;   // a probed pack file: its arena bytes until they are copied
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
        cudaGraphExec_t graph_exec = nullptr;   // the plan's graph with this slot's staging buffer as the image (float pushes: no device copy)
    } slots[2];
    cudaStream_t copy_stream = nullptr, d2h_stream = nullptr;   // host->device of the next batch / device->host of the last
    int stream_op = -1, stream_cap = 0; size_t stream_result_floats = 0;
    int push_count = 0, pop_count = 0;
};

namespace msnh {

inline int esize(int dtype) { return dtype == MSNH_B200_F16 ? 2 : 4; }
inline int vec_of(int dtype) { return dtype == MSNH_B200_F16 ? 8 : 4; }
inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

inline int grid_for(const MsnhB200Ctx *ctx, size_t work_items, int block) {
    size_t blocks = (work_items + block - 1) / block;
    size_t cap = static_cast<size_t>(ctx->sm_count) * 8;   // multiple of the SM count, grid-stride beyond
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

// ---- plan_shapes.cu ----
int infer_shape(MsnhB200Plan *pl, int i, std::string &err);

// ---- plan_build.cu ----
int new_tensor(MsnhB200Plan *pl, Shape s, int dtype);
int new_buffer(MsnhB200Plan *pl, int tensor);
int root_of(MsnhB200Plan *pl, int buf, int *c_off);
TView view_of(MsnhB200Plan *pl, int tensor);
void touch(MsnhB200Plan *pl, int tensor, int step);
int build_launches(MsnhB200Plan *pl);

// ---- plan_tiles.cu ----
CUtensorMapDataType tm_type(int dtype);
// state of the measured tile-shape choice that lives across the launches of one build
struct TileTuning { bool autotune = false; cudaEvent_t ev0 = nullptr, ev1 = nullptr; size_t umma_seen = 0; };
int tile_tuning_begin(MsnhB200Plan *pl, TileTuning &tt);
int tile_tuning_end(MsnhB200Plan *pl, TileTuning &tt);
// tile shape, ring sizes, grid, shared memory and tensor maps of a tensor-core conv launch whose views are resolved
int configure_conv_umma(MsnhB200Plan *pl, TileTuning &tt, Launch &L);
// the shared-memory tile form of a 3x3 depthwise launch, where it applies (sets L.dw_tile)
void configure_dw_tile(MsnhB200Plan *pl, Launch &L);

// ---- plan_pack.cu ----
// A slot of n elements in the weight arena: `dev` is the slot's offset as a tagged pointer (resolved by
// resolve_pack), `host` its zero-filled staging bytes to fill right away -- valid until the next reserve -- or nullptr
// when the arena is loaded from a pack file.
constexpr uintptr_t kPackTag = static_cast<uintptr_t>(1) << 44;
template <typename T> struct PackSlot { T *host; void *dev; };
uint8_t *reserve_pack_bytes(MsnhB200Plan *pl, size_t bytes, void **dev);
template <typename T> PackSlot<T> reserve_pack(MsnhB200Plan *pl, size_t n) {
    void *dev = nullptr;
    uint8_t *host = reserve_pack_bytes(pl, n * sizeof(T), &dev);
    return {reinterpret_cast<T *>(host), dev};
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
// A pack file that matches this plan (op list, shapes, flags, blob tag) and whose checksum holds: its arena bytes and
// stored tile shapes are kept in the plan for pack_load_arena. False: there is none, or it does not fit.
bool pack_probe(MsnhB200Plan *pl);
int pack_load_arena(MsnhB200Plan *pl);        // cudaMalloc + copy of the probed bytes (pl->d_pack)
void pack_write(MsnhB200Plan *pl);            // best effort: temporary file unique to this process, then rename

// ---- plan_launch.cu ----
void launch_one(MsnhB200Ctx *ctx, const Launch &L, cudaStream_t st);
void prepare_conv_umma_launch(const Launch &L);   // dynamic shared memory opt-in of the kernel instantiation L runs
void launch_readback(MsnhB200Ctx *ctx, int dtype, const TView &v, float *dst_nchw, size_t count, cudaStream_t st);
void launch_preprocess_u8(const unsigned char *src, float *dst, const PrepParams &p, int n_images, cudaStream_t st);
int prepare_yolo_nms(MsnhB200Ctx *ctx);           // shared memory opt-in of the NMS kernel
void launch_yolo_nms(const float *rows, const int *counts, int max_rows, float nms_thresh, int use_soft_nms, float sigma,
                     float *boxes, int box_pitch, int *box_counts, int n_images, cudaStream_t st);
void prepare_dw_tile_launch(int dtype);
void launch_fill(MsnhB200Ctx *ctx, float *dst, size_t n, float value, cudaStream_t st);

// ---- plan.cu ----
int check_device_flag(MsnhB200Plan *pl);

}  // namespace msnh
