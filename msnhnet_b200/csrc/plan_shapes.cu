// Shape inference and validation of the op list a caller hands to msnh_b200_plan_create.
#include "plan_internal.h"

using namespace msnh;

namespace msnh {

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

}  // namespace msnh
