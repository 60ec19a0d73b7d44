// Plan compiler and executor behind the C ABI of include/msnh_b200.h.
//
// A plan is built once per (net, batch, dtype): shape inference -> fusion of conv + BatchNorm +
// activation + residual add into one tensor-core launch -> zero-copy placement of route/concat
// inputs as channel slices of the concat buffer -> liveness-based static arena -> weight folding
// and packing -> one list of kernel launches with resolved pointers and TMA tensor maps, captured
// as a CUDA graph. Running a plan is one H2D copy, one graph launch and (optionally) one sync.
// It stands in for NetBuilder's GPU loop and memory pools (src/net/MsnhNetBuilder.cpp:565-620,
// :820-1007 in the reference) and for the per-layer forwardGPU bodies.
#include "plan_internal.h"

using namespace msnh;

namespace msnh {

const char *const kLaunchNames[] = {"input_nchw_to_nhwc", "conv_umma", "conv_direct", "dwconv", "scale_bias_act",
                                    "add_n", "binary", "maxpool", "avgpool", "upsample", "slice", "pad", "softmax",
                                    "yolo_decode", "collect_zero", "yolo_collect", "input_nchw_to_patches",
                                    "yolo_decode_collect", "focus_slices", "bilinear", "deconv_col2im", "clip", "remap", "reduce", "prelu", "maxpool_depth"};

int fail(MsnhB200Ctx *ctx, int code, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    return code;
}

PlanDebugOptions PlanDebugOptions::from_env() {
    auto flag = [](const char *name) { const char *e = std::getenv(name); return e != nullptr; };
    auto num = [](const char *name, int unset) { const char *e = std::getenv(name); return e ? atoi(e) : unset; };
    PlanDebugOptions o;
    { const char *e = std::getenv("MSNH_B200_NO_PDL"); o.no_pdl = e && e[0] == '1'; }
    o.no_merge = flag("MSNH_B200_NO_MERGE");
    o.build_trace = flag("MSNH_B200_BUILD_TRACE");
    o.trace_tune = flag("MSNH_B200_TRACE_TUNE");
    o.dw_simple = flag("MSNH_B200_DW_SIMPLE");
    o.conv_simple = flag("MSNH_B200_CONV_SIMPLE");
    o.dw_th = num("MSNH_B200_DW_TH", 0);
    o.dw_stages = num("MSNH_B200_DW_STAGES", 0);
    o.autotune = num("MSNH_B200_AUTOTUNE", -1);
    o.trace_tile = num("MSNH_B200_TRACE_TILE", 0);
    o.forced_mm = num("MSNH_B200_M_MULT", 0);
    o.forced_bn = num("MSNH_B200_BN", 0);
    o.stream_k = num("MSNH_B200_STREAM_K", 0);
    o.pair = num("MSNH_B200_PAIR", 0);
    o.no_split = num("MSNH_B200_NO_SPLIT", -1);
    return o;
}
int check_device_flag(MsnhB200Plan *pl) {
    int flag = 0;
    CUDA_TRY(pl->ctx, cudaMemcpy(&flag, pl->ctx->dev_err_flag, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag != 0) {
        cudaMemset(pl->ctx->dev_err_flag, 0, sizeof(int));
        return fail(pl->ctx, MSNH_B200_ERR_DEVICE_TIMEOUT, "a bounded wait inside the conv kernel ran out (code %d)", flag);
    }
    return MSNH_B200_OK;
}

}  // namespace msnh

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
    ctx->pdl = !PlanDebugOptions::from_env().no_pdl;
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
    pl->dbg = PlanDebugOptions::from_env();
    if (usable) *usable = pack_probe(pl) ? 1 : 0;
    return MSNH_B200_OK;
}

int msnh_b200_plan_finalize(MsnhB200Plan *pl) {
    if (!pl) return MSNH_B200_ERR_ARG;
    MsnhB200Ctx *ctx = pl->ctx;
    if (pl->finalized) return fail(ctx, MSNH_B200_ERR_STATE, "finalize called twice");
    if (pl->finalize_failed) return fail(ctx, MSNH_B200_ERR_STATE, "an earlier finalize of this plan failed: destroy it and build a new one");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    pl->dbg = PlanDebugOptions::from_env();
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
    launch_readback(ctx, dt, v, pl->d_readback, count, ctx->stream);
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
            launch_fill(ctx, ctx->flush_buf, ctx->flush_elems, 0.f, ctx->stream);
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
        if (sl.graph_exec) cudaGraphExecDestroy(sl.graph_exec);
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
