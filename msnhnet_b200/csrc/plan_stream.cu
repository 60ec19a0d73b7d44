// Image preprocessing on the device, score sort + NMS on the device, and the pipelined streaming calls.
#include "plan_internal.h"

using namespace msnh;

extern "C" {

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
    launch_preprocess_u8(pl->d_u8, pl->d_input + static_cast<size_t>(image) * 3 * pl->in_h * pl->in_w, p, 1, ctx->stream);
    CUDA_TRY(ctx, cudaGetLastError());
    // the staging image may be overwritten by the next call: finish this one first
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return MSNH_B200_OK;
}

static int nms_buffers(MsnhB200Plan *pl) {
    MsnhB200Ctx *ctx = pl->ctx;
    if (pl->d_nms_boxes) return MSNH_B200_OK;
    { const int rc = prepare_yolo_nms(ctx); if (rc) return rc; }
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
    launch_yolo_nms(zl->rows, zl->counts, zl->max_rows, nms_thresh, use_soft_nms, sigma, pl->d_nms_boxes, kNmsMaxCandidates, pl->d_nms_counts, n_images, ctx->stream);
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
        // Float images go from the slot's staging buffer straight into the forward: a copy of the plan's graph whose
        // input kernel reads this slot's buffer instead of the plan's own input buffer.
        if (pl->graph_exec) {
            std::vector<Launch> mine = pl->launches;
            bool found = false;
            for (Launch &L : mine) if (L.in.ptr == pl->d_input) { L.in.ptr = s.d_stage; found = true; }
            if (found) {
                cudaGraph_t g = nullptr;
                CUDA_TRY(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
                for (const Launch &L : mine) launch_one(ctx, L, ctx->stream);
                const cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
                if (e != cudaSuccess) return fail(ctx, MSNH_B200_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
                const cudaError_t ei = cudaGraphInstantiate(&s.graph_exec, g, 0);
                cudaGraphDestroy(g);
                if (ei != cudaSuccess) return fail(ctx, MSNH_B200_ERR_CUDA, "graph instantiation failed: %s", cudaGetErrorString(ei));
            }
        }
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
        launch_preprocess_u8(reinterpret_cast<const unsigned char *>(s.d_stage), pl->d_input, *prep, n_images, ctx->stream);
        CUDA_TRY(ctx, cudaGetLastError());
    } else if (!s.graph_exec) {
        CUDA_TRY(ctx, cudaMemcpyAsync(pl->d_input, s.d_stage, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    }
    if (!prep && s.graph_exec) {
        // the forward reads the staging buffer itself: it is free for the next copy-in when the forward is done
        CUDA_TRY(ctx, cudaGraphLaunch(s.graph_exec, ctx->stream));
        CUDA_TRY(ctx, cudaEventRecord(s.consumed, ctx->stream));
    } else {
        CUDA_TRY(ctx, cudaEventRecord(s.consumed, ctx->stream));
        if (pl->graph_exec) CUDA_TRY(ctx, cudaGraphLaunch(pl->graph_exec, ctx->stream));
        else for (const Launch &L : pl->launches) launch_one(ctx, L, ctx->stream);
    }
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
            launch_yolo_nms(zl->rows, zl->counts, zl->max_rows, pl->nms_thresh, pl->nms_soft, pl->nms_sigma, s.d_result, pl->stream_cap, s.d_counts, n_images, ctx->stream);
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
        launch_readback(ctx, pl->tensors[o.tensor].dtype, v, s.d_result, per * n_images, ctx->stream);
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

}  // extern "C"
