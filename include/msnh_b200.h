/*
 * msnh_b200.h — C ABI of the B200 (sm_100a) forward backend for Msnhnet nets.
 *
 * This is the whole boundary between the host side (the NetBuilder mirror, any other language
 * over FFI) and the device code. Plain pointers and sizes only; every call returns an int status
 * (MSNH_B200_OK == 0), never throws and never calls exit(). Handles are opaque. Host buffers are
 * caller-owned; all device memory belongs to the library. One context per device; a context and
 * the plans made from it may be driven by one host thread at a time.
 *
 * What each group replaces in the reference (paths inside the Msnhnet source tree):
 *   - context      : the global stream/handle wrapper, src/config/MsnhnetCuda.cpp:148-262
 *   - plan         : the per-layer GPU loop and its memory pools,
 *                    src/net/MsnhNetBuilder.cpp:565-620 (pools), :820-1007 (runClassifyGPU /
 *                    runYoloGPU), and every BaseLayer::forwardGPU it calls
 *                    (include/Msnhnet/layers/MsnhBaseLayer.h:47-59)
 *   - kernel calls : the .cu files under src/layers/cuda and src/core/cuda (MsnhBlasGPU.cu, MsnhGemmGPU.cu)
 */
#ifndef MSNH_B200_H
#define MSNH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------- */
enum {
    MSNH_B200_OK            = 0,
    MSNH_B200_ERR_ARG       = 1,  /* bad pointer / size / index                                 */
    MSNH_B200_ERR_UNSUPPORTED = 2,/* op or parameter combination this backend does not cover     */
    MSNH_B200_ERR_CUDA      = 3,  /* a CUDA runtime / driver call failed (text in last_error)    */
    MSNH_B200_ERR_STATE     = 4,  /* call order (e.g. run before finalize)                       */
    MSNH_B200_ERR_DEVICE_TIMEOUT = 5, /* a bounded wait inside a kernel ran out (flag from device)*/
    MSNH_B200_ERR_NOMEM     = 6
};

/* ---- element types of activations ---------------------------------------------------------- */
enum { MSNH_B200_F32 = 0,  /* fp32 storage, tf32 tensor-core contraction, fp32 accumulate       */
       MSNH_B200_F16 = 1 };/* fp16 storage, fp16 tensor-core contraction, fp32 accumulate       */

/* ---- activations: same set and formulas as include/Msnhnet/layers/MsnhActivations.h:39-168 -- */
enum {
    MSNH_ACT_NONE = 0, MSNH_ACT_LOGISTIC, MSNH_ACT_LOGGY, MSNH_ACT_RELU, MSNH_ACT_RELU6,
    MSNH_ACT_HARD_SWISH, MSNH_ACT_ELU, MSNH_ACT_SELU, MSNH_ACT_RELIE, MSNH_ACT_RAMP,
    MSNH_ACT_LEAKY, MSNH_ACT_TANH, MSNH_ACT_STAIR, MSNH_ACT_HARDTAN, MSNH_ACT_SOFT_PLUS,
    MSNH_ACT_PLSE, MSNH_ACT_LHTAN, MSNH_ACT_MISH, MSNH_ACT_SWISH, MSNH_ACT_COUNT
};

/* ---- primitive ops of a plan ----------------------------------------------------------------
 * The host flattens Msnhnet layers (block layers included) into these. Each op has ONE output
 * tensor, identified by the op's index; inputs name earlier ops (or MSNH_B200_INPUT = the image).
 * Tensors are 4-D (batch, H, W, C); the library stores them channels-last.
 */
#define MSNH_B200_INPUT (-1)
#define MSNH_B200_MAX_IN 8

enum {
    MSNH_OP_CONV = 1,     /* a1/a3/a4: conv (+folded BatchNorm or bias) (+activation)              */
    MSNH_OP_BATCHNORM,    /* a6 : standalone inference BatchNorm (+activation)                     */
    MSNH_OP_ACTIVATION,   /* a4 : standalone activation                                           */
    MSNH_OP_MAXPOOL,      /* a7; filters > 0 = depth pooling: out channel g = max over input channels
                             g, g+filters, ... at the same pixel (src/layers/MsnhMaxPoolLayer.cpp:244-270) */
    MSNH_OP_AVGPOOL,      /* a16: local average pool (global = kernel covering the plane)         */
    MSNH_OP_UPSAMPLE,     /* a9 : nearest-neighbour                                               */
    MSNH_OP_CONCAT,       /* a10: route addModel 0 (optionally one channel group of each input)    */
    MSNH_OP_ADD,          /* a10 addModel 1, a11 block sums, a12 varop add (+activation)           */
    MSNH_OP_SLICE,        /* a13                                                                  */
    MSNH_OP_PAD,          /* a16: constant padding                                                */
    MSNH_OP_CONNECTED,    /* a16: fully connected (+BN or bias) (+activation)                     */
    MSNH_OP_SOFTMAX,      /* a16                                                                  */
    MSNH_OP_YOLO,         /* a14: head decode                                                     */
    MSNH_OP_IDENTITY,     /* empty layer / single-input route                                     */
    MSNH_OP_BINARY,       /* a12: varop sub/mul/div of two tensors, or tensor (op) constant        */
    MSNH_OP_YOLO_COLLECT, /* a15: device half of YoloOut: objectness threshold + best class over the
                             MSNH_OP_YOLO heads in `in`, threshold in const_val; the result is a
                             per-image candidate list read with plan_read_candidates              */
    MSNH_OP_DECONV,       /* transposed conv (+bias) (+activation), groups == 1
                             (src/layers/MsnhDeConvolutionalLayer.cpp:98-170); weights [Cin][Cout][kh][kw] */
    MSNH_OP_CLIP,         /* clamp to [clip_min, clip_max] (src/layers/MsnhClipLayer.cpp)               */
    MSNH_OP_REMAP,        /* view / permute / pixel shuffle: out[flat CHW i] = in[flat CHW g(i)], g chosen by
                             remap_kind (src/layers/MsnhViewLayer.cpp, MsnhPermuteLayer.cpp:127-183,
                             MsnhPixelShuffleLayer.cpp:87-108)                                          */
    MSNH_OP_REDUCE,       /* sum or mean over one axis or the whole image (src/layers/MsnhReductionLayer.cpp) */
    MSNH_OP_PRELU         /* x > 0 ? x : slope[c] * x, slopes (one per channel) in MSNH_W_WEIGHTS
                             (Activations::activatePRelu, src/layers/MsnhActivations.cpp:411-470)        */
};

/* MSNH_OP_UPSAMPLE modes (src/layers/MsnhUpSampleLayer.cpp:14-24) */
enum { MSNH_UPSAMPLE_NEAREST = 0, MSNH_UPSAMPLE_BILINEAR = 1 };
/* MSNH_OP_REMAP kinds. VIEW: out_c/out_h/out_w give the new shape (same element count). PERMUTE: remap_dims[k]
 * names the input axis (0 C, 1 H, 2 W) that becomes output axis k. PIXSHF: remap_dims[0] = factor. */
enum { MSNH_REMAP_VIEW = 0, MSNH_REMAP_PERMUTE = 1, MSNH_REMAP_PIXSHF = 2 };

/* binary kinds for MSNH_OP_BINARY (src/layers/MsnhVariableOpLayer.cpp) */
enum { MSNH_BIN_ADD = 0, MSNH_BIN_SUB, MSNH_BIN_SUB_INV, MSNH_BIN_MUL, MSNH_BIN_DIV, MSNH_BIN_DIV_INV,
       /* VariableOpLayer's one-operand types (include/Msnhnet/io/MsnhParser.h:400-428, Blas::cpuScientific,
        * src/core/cuda/MsnhBlasGPU.cu:142-202): MSNH_OP_BINARY with binary_const = 1; const_val is pow's exponent */
       MSNH_UN_ABS, MSNH_UN_ACOS, MSNH_UN_ASIN, MSNH_UN_ATAN, MSNH_UN_COS, MSNH_UN_COSH, MSNH_UN_SIN, MSNH_UN_SINH,
       MSNH_UN_TAN, MSNH_UN_TANH, MSNH_UN_EXP, MSNH_UN_POW, MSNH_UN_LOG, MSNH_UN_LOG10, MSNH_UN_SQRT, MSNH_BIN_COUNT };

/* yolo head flavours (include/Msnhnet/layers/MsnhYoloDef.h) */
enum { MSNH_YOLO_V3 = 30, MSNH_YOLO_V4 = 40, MSNH_YOLO_V5 = 50 };

typedef struct MsnhB200Op {
    int32_t kind;                      /* MSNH_OP_*                                               */
    int32_t n_in;
    int32_t in[MSNH_B200_MAX_IN];      /* producer op index or MSNH_B200_INPUT                    */
    /* geometry (conv / pools / pad / upsample / slice) */
    int32_t filters;                   /* conv: Cout; connected: outputs                          */
    int32_t k_h, k_w, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w, groups;
    int32_t out_h, out_w;              /* pools: output plane computed by the host (ceilMode etc.);
                                          0 = derive with floor rule                              */
    int32_t pad_top, pad_down, pad_left, pad_right; /* MSNH_OP_PAD                                */
    int32_t slice_start[3], slice_step[3]; /* C,H,W                                               */
    int32_t route_groups, route_group_id;  /* concat: take channel group id of `groups` per input */
    /* numerics */
    int32_t has_bn, has_bias;
    float   bn_eps;
    int32_t act;  float act_param;     /* MSNH_ACT_*                                              */
    float   scale;                     /* upsample: multiplier (reference default 1)              */
    float   const_val;                 /* pad value; binary const; clip: lower bound               */
    /* (clip's upper bound travels in `scale`; reduce: axis in binary_kind (-1 all, 0 C, 1 H, 2 W), mean flag in
     *  binary_const) */
    int32_t binary_kind, binary_const; /* MSNH_OP_BINARY: kind; 1 = second operand is const_val    */
    /* softmax */
    int32_t softmax_groups; float softmax_temperature;
    /* yolo */
    int32_t yolo_type, yolo_classes;   float yolo_anchors[6];
    /* bookkeeping */
    int32_t is_output;                 /* keep the tensor alive after the run and allow read-back  */
    /* upsample: MSNH_UPSAMPLE_*; bilinear takes its output plane from out_h/out_w and align_corners */
    int32_t upsample_mode, align_corners;
    /* remap: MSNH_REMAP_*, its dims (see the enum), VIEW's output channel count (plane in out_h/out_w) */
    int32_t remap_kind, remap_dims[3], out_c;
} MsnhB200Op;

/* weight slots of plan_set_weights, in the order the .msnhbin blob stores them
 * (src/layers/MsnhConvolutionalLayer.cpp:1255-1329, MsnhBatchNormLayer.cpp:469-472)          */
enum { MSNH_W_WEIGHTS = 0, MSNH_W_BIAS = 1, MSNH_W_BN_SCALE = 2, MSNH_W_BN_BIAS = 3,
       MSNH_W_BN_MEAN = 4, MSNH_W_BN_VAR = 5, MSNH_W_SLOTS = 6 };

/* plan flags */
enum { MSNH_PLAN_NO_GRAPH   = 1u,   /* launch kernels directly instead of replaying a CUDA graph  */
       MSNH_PLAN_NO_FUSION  = 2u,   /* one kernel per op, no zero-copy concat (debug / parity)    */
       MSNH_PLAN_KEEP_ALL   = 4u,   /* every op output stays readable (per-layer parity dumps)     */
       MSNH_PLAN_NO_TENSOR_CORE = 8u,/* run convs on the CUDA-core kernel (device cross-check)     */
       MSNH_PLAN_TRACE      = 16u,  /* tensor-core convs record per-CTA clock stamps (read_trace)  */
       /* fp32 plans of detection nets (plans with a MSNH_OP_YOLO op) run their convs in fp32 arithmetic on the CUDA
        * cores by default: the reference's GPU path is fp32 Sgemm (src/layers/MsnhConvolutionalLayer.cpp:1026-1160)
        * and exp()-decoded box sizes do not hold 1e-3 through tf32's 10-bit mantissa. This flag asks for the tf32
        * tensor-core convs all the same (about 6e-3 on decoded boxes). fp32 classifiers use tf32 either way. */
       MSNH_PLAN_TF32_DETECT = 32u };

typedef struct MsnhB200Ctx  MsnhB200Ctx;
typedef struct MsnhB200Plan MsnhB200Plan;

/* ---- context ------------------------------------------------------------------------------ */
int  msnh_b200_device_count(int *count);
int  msnh_b200_ctx_create(int device, MsnhB200Ctx **ctx);
int  msnh_b200_ctx_destroy(MsnhB200Ctx *ctx);
/* Text of the last failure on this context (valid until the next call on it). Never NULL. */
const char *msnh_b200_last_error(MsnhB200Ctx *ctx);
/* Pinned host memory for inputs/outputs of plan_run (plain malloc'ed buffers work too, slower). */
int  msnh_b200_host_alloc(MsnhB200Ctx *ctx, size_t bytes, void **ptr);
int  msnh_b200_host_free(MsnhB200Ctx *ctx, void *ptr);

/* ---- plan: replaces NetBuilder's GPU loop --------------------------------------------------- */
int  msnh_b200_plan_create(MsnhB200Ctx *ctx, const MsnhB200Op *ops, int n_ops,
                           int in_c, int in_h, int in_w, int batch, int dtype, uint32_t flags,
                           MsnhB200Plan **plan);
/* Shape of op's output as (C,H,W); valid right after plan_create. */
int  msnh_b200_plan_op_shape(MsnhB200Plan *plan, int op, int *c, int *h, int *w);
/* Number of floats slot `slot` of op `op` expects (0 if the op has no such tensor). */
int  msnh_b200_plan_weight_count(MsnhB200Plan *plan, int op, int slot, size_t *count);
/* fp32 host data in the reference's own order (conv: [Cout][Cin/g][kh][kw]). Copied. */
int  msnh_b200_plan_set_weights(MsnhB200Plan *plan, int op, int slot, const float *data, size_t count);
/* Folds BN, packs weights, lays out the arena, builds tensor maps and captures the CUDA graph. */
int  msnh_b200_plan_finalize(MsnhB200Plan *plan);
/* Weight pack cache, in place of the reference's loader that pushes the blob float by float into a vector and
 * copies it per layer (src/io/MsnhParser.cpp:684-726, src/net/MsnhNetBuilder.cpp:624-663). Call before
 * plan_finalize. All packed weights of a plan (fp16 / tf32-rounded, channels-last, BatchNorm folded) live in one
 * device allocation filled by one copy; with a pack file registered, finalize writes those bytes to `path` after
 * building them, or — when `path` already holds a pack made for the same ops, shapes, batch, dtype, flags and
 * `weights_tag` — reads them from it and skips the repacking, in which case plan_set_weights need not have been
 * called at all. *usable (may be NULL) tells which of the two will happen. `weights_tag` identifies the float
 * blob (the host side uses size and modification time of the .msnhbin file); a pack whose header does not match
 * is ignored and rewritten. The .msnhbin format itself is unchanged. */
int  msnh_b200_plan_use_pack(MsnhB200Plan *plan, const char *path, uint64_t weights_tag, int *usable);
/* One forward of n_images (<= batch) planar CHW fp32 images held in HOST memory: H2D copy,
 * layout change, all kernels, then the stream is synchronised. */
int  msnh_b200_plan_run(MsnhB200Plan *plan, const float *host_nchw, int n_images);
/* Same, input already on the device (fp32 NCHW, n_images * C*H*W floats). No host sync unless
 * `sync` is non-zero. Used for device-resident throughput timing. */
int  msnh_b200_plan_run_device(MsnhB200Plan *plan, const float *dev_nchw, int n_images, int sync);
/* Throughput timing with the input resident in the staging buffer: `steps` forwards back to back on
 * the plan's stream between two CUDA events; *total_ms is the device time of all of them. */
int  msnh_b200_plan_run_timed(MsnhB200Plan *plan, int n_images, int steps, float *total_ms);
/* The same forward launched kernel by kernel (no graph) with a CUDA event between consecutive
 * launches: ms[k] = mean device time of launch k over `steps` forwards, warm caches, real data flow. */
int  msnh_b200_plan_run_instrumented(MsnhB200Plan *plan, int n_images, int steps, float *ms, int capacity);
/* Pipelined streaming over many batches in host (ideally pinned) memory. push is asynchronous: the
 * batch is copied in on a second stream while the previous batch computes, then runs, then its result
 * (candidate rows of MSNH_OP_YOLO_COLLECT op `op`, or the fp32 NCHW output of any other output op) is
 * copied to a pinned slot. At most two batches may be in flight; pop waits for the oldest one and
 * hands out its result: for a collect op rows/counts as plan_read_candidates does, otherwise
 * n_images*C*H*W floats. One result op per plan. A slot holds at most 4096 candidate rows per image: an
 * image with more candidates than that (which ones reached the slot first is a matter of timing), or one the
 * device NMS does not take (plan_stream_nms), comes back with counts[i] = -1 and no rows; pop still succeeds
 * and frees the slot, and the caller runs that image again through plan_run and plan_read_candidates /
 * plan_nms, which keep every candidate. stream_reset waits for everything in flight and drops it (for a
 * caller that gives up in the middle of a stream, e.g. on an error). */
int  msnh_b200_plan_stream_push(MsnhB200Plan *plan, int op, const float *host_nchw, int n_images);
int  msnh_b200_plan_stream_pop(MsnhB200Plan *plan, float *result, size_t capacity_floats, int max_rows_per_image,
                               int *counts, int *n_images);
int  msnh_b200_plan_stream_reset(MsnhB200Plan *plan);
/* stream_push for 8-bit images: n_images raw HWC RGB images of width x height pixels back to back (a quarter of the
 * bytes of the float images over PCIe); the preprocessing of plan_preprocess_u8 (same mode / swap_rgb / mean / std)
 * runs on the device between the copy and the forward. The images of one batch must fit the staging buffer of a
 * float batch (n_images * width * height * 3 <= batch * C * H * W * 4). */
int  msnh_b200_plan_stream_push_u8(MsnhB200Plan *plan, int op, const unsigned char *host_hwc, int width, int height, int n_images,
                                   int mode, int swap_rgb, const float *mean, const float *std);
/* Copies op's output of the last run to the host as fp32 NCHW (n_images*C*H*W floats).
 * The op must be an output (is_output) or the plan made with MSNH_PLAN_KEEP_ALL. */
int  msnh_b200_plan_read_output(MsnhB200Plan *plan, int op, float *host_nchw, size_t count);
/* Detection candidates of the last run, from MSNH_OP_YOLO_COLLECT op `op`: rows of 8 floats
 * {x, y, w, h, conf, bestClsConf, bestClsIdx, order} for every cell of every head whose
 * objectness exceeds the op's threshold, grouped per image; `order` is the cell's position in the
 * reference's candidate scan (src/layers/MsnhYoloOutLayer.cpp:119-165) and rows come sorted by
 * it. counts[i] receives image i's row count; rows of image i start at
 * rows + i*max_rows_per_image*8. Rows beyond max_rows_per_image are dropped and counts[i] is
 * clamped to it. Only the surviving rows cross PCIe. */
int  msnh_b200_plan_read_candidates(MsnhB200Plan *plan, int op, int n_images, float *rows,
                                    int max_rows_per_image, int *counts);

/* Raw 8-bit RGB image (HWC, 3 channels) -> image slot `image` of the plan's fp32 input staging buffer, on the
 * device: what the reference's C API does on the host before the forward (src/c_api/MsnhnetLib.cpp:540-600
 * runClassifyList, :754-778 runYoloList; src/utils/MsnhCVUtil.cpp:91-373; MatOp::resize,
 * src/cv/MsnhCVMatOp.cpp:142-160, :399-434). mode: MSNH_PREP_UNIT resize, /255 (getImgDataF32C3) |
 * MSNH_PREP_PAD_SQUARE 127-gray bars to a square, resize, /255 (getPaddingZeroF32C3, what runYoloList uses) |
 * MSNH_PREP_GOOGLENET | MSNH_PREP_TRANSFORMED (mean, std required) | MSNH_PREP_CAFFE. swap_rgb as in the C API
 * (0 reverses the channel order first, as the reference does). Bit-identical to the reference's code
 * compiled without FMA contraction. Follow with msnh_b200_plan_run_device(plan, NULL, n_images, sync). */
#define MSNH_PREP_UNIT        0
#define MSNH_PREP_PAD_SQUARE  1
#define MSNH_PREP_GOOGLENET   2
#define MSNH_PREP_TRANSFORMED 3
#define MSNH_PREP_CAFFE       4
int  msnh_b200_plan_preprocess_u8(MsnhB200Plan *plan, const unsigned char *host_hwc, int width, int height, int image,
                                  int mode, int swap_rgb, const float *mean, const float *std);

/* Device-side score sort + per-class greedy NMS of the candidates the last forward collected: the host half of
 * YoloOutLayer::forward (src/layers/MsnhYoloOutLayer.cpp:167-197 sort by conf*bestClsConf, :381-461 nms), run as one
 * CTA per image. boxes: n_images * max_boxes rows of 8 floats {x, y, w, h, conf, bestClsConf, bestClsIdx, rank} in
 * the reference's output order. counts[i] = boxes kept, or -1 when image i had more than 4096 candidates (read
 * them with msnh_b200_plan_read_candidates and run the host NMS). Candidates whose scores are bit-identical keep
 * scan order (the reference's unstable sort leaves their order unspecified); everything else is exact. */
int  msnh_b200_plan_nms(MsnhB200Plan *plan, int op, int n_images, float nms_thresh, int use_soft_nms, float sigma,
                        float *boxes, int max_boxes, int *counts);
/* Streaming (plan_stream_push / _pop) with the NMS on the device: pop then returns kept boxes (rows as above)
 * instead of candidates. Call with no batch in flight. */
int  msnh_b200_plan_stream_nms(MsnhB200Plan *plan, int enable, float nms_thresh, int use_soft_nms, float sigma);
/* Device address of the plan's fp32 NCHW input staging buffer (batch*C*H*W floats). A caller that
 * fills it itself passes dev_nchw = NULL to plan_run_device. */
int  msnh_b200_plan_input_buffer(MsnhB200Plan *plan, float **dev_ptr);
/* Device time of the last plan_run / plan_run_device between its first and last kernel, ms. */
int  msnh_b200_plan_last_ms(MsnhB200Plan *plan, float *ms);
/* Kernel launches per forward (graph nodes); arena bytes. */
int  msnh_b200_plan_stats(MsnhB200Plan *plan, int *launches, size_t *arena_bytes);
/* Text table: one line per launch "idx kernel op_kind shape flops bytes". Caller frees nothing:
 * the pointer stays valid until the plan is destroyed. */
const char *msnh_b200_plan_describe(MsnhB200Plan *plan);
/* Times every launch of the plan separately (CUDA events, `iters` repetitions, L2 flushed between
 * repetitions) and writes per-launch mean ms into ms[0..launches). Not for use during capture. */
int  msnh_b200_plan_profile(MsnhB200Plan *plan, int iters, float *ms, int capacity);
/* Tracing (the reference's per-layer GPU timers are stubbed out, src/layers/MsnhBaseLayer.cpp:300-319):
 * for a plan made with MSNH_PLAN_TRACE, the SM clock stamps the tensor-core conv of launch `launch`
 * recorded in its last execution: 64 int64 per CTA (slot meaning in csrc/conv_umma.cuh). */
int  msnh_b200_plan_read_trace(MsnhB200Plan *plan, int launch, long long *stamps, int capacity, int *ctas);
int  msnh_b200_plan_destroy(MsnhB200Plan *plan);

/* Effective SM clock under load (no counterpart in the reference, whose GPU timers are stubbed out,
 * src/layers/MsnhBaseLayer.cpp:300-319): start launches one warp on a stream of its own that samples the device's
 * nanosecond timer and its SM's cycle counter about once a millisecond for at most max_ms milliseconds (1..60000);
 * stop ends it and reports the cycle counter's rate over the sampled intervals in MHz. The management library's SM
 * clock is the clock the GPU is asked to run at; this is the rate at which cycle counts of kernels that ran meanwhile
 * convert to time. Measurement aid of bench.py; allocates a few KB on the device between start and stop. */
int  msnh_b200_clock_probe_start(int device, int max_ms, void **handle);
int  msnh_b200_clock_probe_stop(void *handle, double *mhz_median, double *mhz_min, double *mhz_max, int *samples);

/* ---- candidate collection without any allocation ------------------------------------------------
 * No counterpart in the reference (its YoloOut copies every cell to the host and thresholds there).
 * For callers that cannot allocate device memory where they need detections - real-time loops and
 * stream callbacks that must not enter the allocator, plugins with a fixed memory grant, processes
 * whose device memory a framework has already carved up. The caller owns every buffer it passes;
 * the kernel's only scratch (one append counter per image) is a static __device__ array of
 * MSNH_B200_STATIC_MAX_IMAGES ints that each GPU loading the library holds until exit. The call
 * makes no cudaMalloc / cudaFree and needs no context.
 *   dev_decoded : decoded head, fp32 channels-last [n_images][grid_h][grid_w][channel_pitch],
 *                 channel a*(5+classes)+k as written by MSNH_OP_YOLO
 *   dev_rows    : [n_images][max_rows_per_image][8] floats {x,y,w,h,conf,bestClsConf,bestClsIdx,order}
 *                 in arbitrary order within an image (sort by `order` for the reference's scan order)
 *   dev_counts  : [n_images] ints, rows written per image (clamped to max_rows_per_image)
 * n_images above MSNH_B200_STATIC_MAX_IMAGES is rejected with MSNH_B200_ERR_ARG. The first call on
 * a device looks up the array's device address (cudaGetSymbolAddress) and should therefore come
 * before any stream capture. The address is looked up once per device and kept for the life of the
 * process: it does not survive a cudaDeviceReset by the caller (after one, this entry point must not be
 * used again in that process). All calls on a device share the array: it still holds the previous
 * call's counts (this call clears what it uses), and two calls that overlap on the GPU race. */
#define MSNH_B200_STATIC_MAX_IMAGES 1024
int  msnh_b200_yolo_collect_static(const float *dev_decoded, int n_images, int grid_h, int grid_w, int channel_pitch,
                                   int classes, float conf_thresh, int order_base, float *dev_rows,
                                   int max_rows_per_image, int *dev_counts, void *stream);
/* Text of the last failure of msnh_b200_yolo_collect_static on this thread (static buffer). */
const char *msnh_b200_static_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* MSNH_B200_H */
