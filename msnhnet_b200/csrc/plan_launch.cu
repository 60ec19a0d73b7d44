// The one translation unit that compiles the kernels: turns a Launch record into a kernel launch, and wraps the few
// launches the entry points make directly (read-back layout change, image preprocessing, device NMS, cache flush).
#include "plan_internal.h"

using namespace msnh;
#include "common.cuh"
#include "conv_umma.cuh"
#include "nms_kernel.cuh"
#include "layer_kernels.cuh"
#include "dwconv_tile.cuh"
#include "conv_tiled.cuh"

namespace msnh {
namespace {

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

void prepare_conv_umma_launch(const Launch &L) { set_smem_attr(L); }

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
            if (L.focus_planar) {
                launch_k(ctx->pdl, focus_planar_kernel<T, 3>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W, block), block, 0, st,
                         static_cast<const float *>(L.in.ptr), L.in.H, L.in.W, L.out, L.focus);
                break;
            }
            launch_k(ctx->pdl, focus_kernel<T, 3>, grid_for(ctx, static_cast<size_t>(L.out.N) * L.out.H * L.out.W, block), block, 0, st, L.in, L.out, L.focus);
            break;
        case L_COLLECT_RAW:
            launch_k(ctx->pdl, yolo_decode_collect_kernel<T>, grid_for(ctx, static_cast<size_t>(L.heads.h[L.heads.n - 1].end), 256), 256, 0, st,
                L.heads, L.fval, L.rows, L.max_rows, L.counts);
            break;
        default: break;
    }
}

}  // namespace

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

// ---- launches the entry points make directly ----
// channels-last tensor of `dtype` -> planar fp32 (what the read-back calls hand to the caller)
void launch_readback(MsnhB200Ctx *ctx, int dtype, const TView &v, float *dst_nchw, size_t count, cudaStream_t st) {
    const int grid = grid_for(ctx, count, 256);
    if (dtype == MSNH_B200_F16) nhwc_to_nchw_f32_kernel<__half><<<grid, 256, 0, st>>>(v, dst_nchw);
    else                        nhwc_to_nchw_f32_kernel<float><<<grid, 256, 0, st>>>(v, dst_nchw);
}
void launch_preprocess_u8(const unsigned char *src, float *dst, const PrepParams &p, int n_images, cudaStream_t st) {
    // n_images raw images of p.w x p.h back to back -> n_images planar float images back to back, one launch
    const dim3 grid((p.out_w + 127) / 128, p.out_h, n_images);
    preprocess_u8_kernel<<<grid, 128, 0, st>>>(src, dst, p, static_cast<size_t>(p.w) * p.h * 3, static_cast<size_t>(p.out_w) * p.out_h * 3);
}
int prepare_yolo_nms(MsnhB200Ctx *ctx) {
    CUDA_TRY(ctx, cudaFuncSetAttribute(yolo_nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kNmsSmemBytes)));
    return MSNH_B200_OK;
}
void launch_yolo_nms(const float *rows, const int *counts, int max_rows, float nms_thresh, int use_soft_nms, float sigma,
                     float *boxes, int box_pitch, int *box_counts, int n_images, cudaStream_t st) {
    yolo_nms_kernel<<<n_images, kNmsThreads, kNmsSmemBytes, st>>>(rows, counts, max_rows, nms_thresh, use_soft_nms, sigma, boxes, box_pitch, box_counts);
}
void launch_fill(MsnhB200Ctx *ctx, float *dst, size_t n, float value, cudaStream_t st) {
    fill_kernel<<<ctx->sm_count * 8, 256, 0, st>>>(dst, n, value);
}
// dynamic shared memory opt-in of the depthwise tile kernels of one dtype
void prepare_dw_tile_launch(int dtype) {
    auto opt_in = [](auto kernel) { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); };
    if (dtype == MSNH_B200_F16) {
        opt_in(dwconv3x3_tile_kernel<__half, 1, true>); opt_in(dwconv3x3_tile_kernel<__half, 1, false>);
        opt_in(dwconv3x3_tile_kernel<__half, 2, true>); opt_in(dwconv3x3_tile_kernel<__half, 2, false>);
    } else {
        opt_in(dwconv3x3_tile_kernel<float, 1, true>); opt_in(dwconv3x3_tile_kernel<float, 1, false>);
        opt_in(dwconv3x3_tile_kernel<float, 2, true>); opt_in(dwconv3x3_tile_kernel<float, 2, false>);
    }
}
}  // namespace msnh
