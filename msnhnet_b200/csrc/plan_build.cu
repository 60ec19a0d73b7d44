// Lowering of the op list to launches: fusion, tensors, zero-copy concat, launch records, merges of sibling launches,
// the weight arena, the liveness-based activation arena, resolved views and the plan's description.
#include <cuda_fp16.h>
#include "plan_internal.h"

using namespace msnh;

namespace msnh {

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

int build_launches(MsnhB200Plan *pl) {
    MsnhB200Ctx *ctx = pl->ctx;
    const int n_ops = static_cast<int>(pl->ops.size());
    const bool no_fusion = (pl->flags & MSNH_PLAN_NO_FUSION) != 0;
    const bool keep_all = (pl->flags & MSNH_PLAN_KEEP_ALL) != 0;
    // MSNH_B200_BUILD_TRACE=1: wall-clock of each stage of the build on stderr
    const PlanDebugOptions &dbg = pl->dbg;
    const bool build_trace = dbg.build_trace;
    auto t_stage = std::chrono::steady_clock::now();
    auto stage = [&](const char *what) {
        if (!build_trace) return;
        const auto now = std::chrono::steady_clock::now();
        std::fprintf(stderr, "[msnh_b200 build] %-28s %8.2f ms\n", what, std::chrono::duration<double, std::milli>(now - t_stage).count());
        t_stage = now;
    };

    // A usable pack file stands in for the weights: the per-channel tensors are given zeros so that the folding
    // code below runs as usual (its results are discarded), the large repacking loops are skipped.
    pl->pack_cursor = 0; pl->pack_host.clear();
    pl->pack_loaded = pack_probe(pl);
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
    if (!no_fusion && !keep_all && !dbg.no_merge) {
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
    if (!no_fusion && !keep_all && !dbg.no_merge) {
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
            auto same_input = [&](int t0, int t1) {          // the same tensor, or an alias of it (a single-input route)
                const Tensor &x = pl->tensors[t0], &y = pl->tensors[t1];
                int ox = 0, oy = 0;
                return root_of(pl, x.buffer, &ox) == root_of(pl, y.buffer, &oy) && x.c_off + ox == y.c_off + oy && x.s.C == y.s.C &&
                       x.s.H == y.s.H && x.s.W == y.s.W && x.dtype == y.dtype;
            };
            while (i + 1 < pend.size() && pend[i].more_out_t.size() < 2 && same_pool(pend[i + 1]) && same_input(pend[i + 1].in_t, pend[i].in_t)) {
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
        CUDA_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->d_pack), total));
        pl->dev_allocs.push_back(pl->d_pack);
        if (pl->pack_loaded) {
            const int rc = pack_load_arena(pl);
            if (rc) return rc;
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
    TileTuning tt;
    { const int rc = tile_tuning_begin(pl, tt); if (rc) return rc; }
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
        configure_dw_tile(pl, L);
        if (L.kind == L_CONV_UMMA) {
            // alignment the tensor-core path needs; otherwise fall back to the CUDA-core kernel
            const bool ok = aligned(L.in) && aligned(L.out) && (L.res == nullptr || (reinterpret_cast<uintptr_t>(L.res) % 16 == 0 && L.ldc_res % V == 0));
            if (!ok && p.out2_t >= 0) return fail(ctx, MSNH_B200_ERR_STATE, "merged 1x1 convs of op %d landed on an unaligned view", L.op);
            if (p.out2_t >= 0 && !aligned(L.out2)) return fail(ctx, MSNH_B200_ERR_STATE, "merged 1x1 convs of op %d: second output unaligned", L.op);
            if (!ok) { L.kind = L_CONV_DIRECT; L.note = "unaligned view: CUDA-core fallback"; }
        }
        if (L.kind == L_CONV_UMMA) { const int rc = configure_conv_umma(pl, tt, L); if (rc) return rc; }
        if (L.kind == L_CONV_DIRECT)
            L.tiled = L.groups == 1 && aligned(L.in) && (L.out.N * static_cast<long long>(L.out.H) * L.out.W + kCtBM - 1) / kCtBM < 2147483647LL &&
                      (L.out.C + kCtBN - 1) / kCtBN <= 65535 && !dbg.conv_simple;
        if (L.kind == L_CONV_DIRECT && L.tiled) L.note += L.note.empty() ? "fp32 arithmetic, shared-memory tiles" : ", fp32 arithmetic, shared-memory tiles";
        pl->launches.push_back(L);
    }
    { const int rc = tile_tuning_end(pl, tt); if (rc) return rc; }
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
        bool launches_shifted = false;
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
            // Where the image feeds nothing but these slices, the fused kernel reads the caller's planar fp32 image itself
            // and the channels-last copy of the image (the input layout launch) is dropped.
            size_t input_launch = pl->launches.size();
            for (size_t j = 0; j < k; ++j) if (pl->launches[j].kind == L_INPUT && pl->launches[j].out.ptr == a.in.ptr) input_launch = j;
            // (launch indices still equal the liveness steps as long as nothing was erased: the image's buffer is last
            //  touched by the last of these slices, so nothing else reads it)
            const Buffer &ibuf = pl->buffers[root_of(pl, pl->tensors[pl->input_tensor].buffer, nullptr)];
            const bool sliced_only = !launches_shifted && input_launch < k && pl->in_c == 3 && ibuf.last == static_cast<int>(end) - 1 &&
                                     !ibuf.persistent;
            if (sliced_only) {
                f.focus_planar = true; f.in.ptr = pl->d_input; f.note += ", from the planar image";
                f.bytes = (static_cast<double>(pl->in_c) * pl->in_h * pl->in_w * 4.0 + static_cast<double>(f.out.ldc) * f.out.H * f.out.W * es) * pl->batch;
            }
            pl->launches[k] = f;
            pl->launches.erase(pl->launches.begin() + static_cast<long>(k) + 1, pl->launches.begin() + static_cast<long>(end));
            launches_shifted = true;
            if (sliced_only) { pl->launches.erase(pl->launches.begin() + static_cast<long>(input_launch)); --k; }
        }
    }

    if (!pl->pack_loaded && !pl->pack_path.empty()) {
        pack_write(pl);
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

}  // namespace msnh
