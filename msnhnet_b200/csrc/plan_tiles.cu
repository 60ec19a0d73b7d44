// Tensor maps, the tile-shape model and measured choice of the tensor-core convolution, and the depthwise tile form.
#include "plan_internal.h"

using namespace msnh;

namespace msnh {

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

// measured tile shapes, one entry per distinct conv layer signature (process-wide)
using TuneKey = std::array<int, 22>;
static std::mutex &tune_mutex() { static std::mutex m; return m; }
static std::map<TuneKey, std::array<int, 3>> &tune_cache() { static std::map<TuneKey, std::array<int, 3>> c; return c; }

// The shared-memory tile form of a 3x3 depthwise launch (dwconv_tile.cuh) where it applies: stride 1 or 2, no dilation,
// whole 16-byte channel vectors. Fills L.dwp, L.map_a, L.grid, L.smem and sets L.dw_tile; leaves L untouched otherwise.
void configure_dw_tile(MsnhB200Plan *pl, Launch &L) {
    MsnhB200Ctx *ctx = pl->ctx;
    const int es = esize(pl->dtype);
    if (!(L.kind == L_DWCONV && L.vec && L.kh == 3 && L.kw == 3 && L.dh == 1 && L.dw == 1 && L.sh == L.sw && (L.sh == 1 || L.sh == 2)) || pl->dbg.dw_simple) return;
    // Output tiles of th x 16 pixels x 32 channels; th (a multiple of the rows a thread computes) is the candidate that
    // loads and computes the fewest rows over the plane among those whose input tile fits a 24 KB stage.
    const int S = L.sh, R = dw_rows(S), iw = dw_in_w(S);
    DwTileParams &d = L.dwp;
    long best_cost = -1;
    for (int th = R; th <= 16; th += R) {
        if (pl->dbg.dw_th > 0 && th != pl->dbg.dw_th / R * R) continue;
        const int ih = (th - 1) * S + 3;
        if (static_cast<size_t>(ih) * iw * kDwChannels * es > 24 * 1024) break;
        const int tiles = (L.out.H + th - 1) / th;
        const long cost = static_cast<long>(tiles) * (ih + th * S);
        if (best_cost < 0 || cost <= best_cost) { best_cost = cost; d.th = th; d.ih = ih; }
    }
    if (best_cost < 0) return;                   // (no tile height fits a stage: the strip kernel takes the layer)
    d.tiles_w = (L.out.W + kDwTileW - 1) / kDwTileW; d.tiles_h = (L.out.H + d.th - 1) / d.th;
    d.tiles_c = (L.in.C + kDwChannels - 1) / kDwChannels;
    d.ph = L.ph; d.pw = L.pw; d.act = L.act1; d.act_param = L.act1_p; d.err_flag = ctx->dev_err_flag;
    const size_t stage = (static_cast<size_t>(d.ih) * iw * kDwChannels * es + 127) / 128 * 128;
    // two stages when that lets a fourth CTA share the SM (four warps each: the arithmetic hides latency through the
    // number of resident warps), three otherwise
    d.stages = (2 * stage + 128 + 1024) * 4 <= 200 * 1024 && (3 * stage + 128 + 1024) * 4 > 200 * 1024 ? 2 : 3;
    if (pl->dbg.dw_stages >= 2 && pl->dbg.dw_stages <= kDwMaxStages) d.stages = pl->dbg.dw_stages;
    L.smem = d.stages * stage + 128;
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
    const CUresult r = ctx->encode_tiled(&L.map_a, tm_type(pl->dtype), 4, L.in.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS && L.smem <= 100 * 1024 && L.in.C % 4 == 0 && grid % d.tiles_c == 0) {
        L.dw_tile = true;
        prepare_dw_tile_launch(pl->dtype);
        char note[96];
        snprintf(note, sizeof(note), "tiles %dx%dx%d ch, grid %d, smem %zu", d.th, kDwTileW, kDwChannels, L.grid, L.smem);
        L.note = note;
    }
}

int tile_tuning_begin(MsnhB200Plan *pl, TileTuning &tt) {
    // MSNH_B200_AUTOTUNE=0 keeps the modelled tile shapes; plans made for debugging (no graph, no fusion, every output
    // kept, traced) keep them too
    tt.autotune = !(pl->flags & (MSNH_PLAN_NO_GRAPH | MSNH_PLAN_NO_FUSION | MSNH_PLAN_KEEP_ALL | (pl->dbg.trace_tune ? 0u : static_cast<uint32_t>(MSNH_PLAN_TRACE))));
    if (pl->dbg.autotune >= 0) tt.autotune = tt.autotune && pl->dbg.autotune != 0;
    tt.umma_seen = 0;
    if (tt.autotune) { CUDA_TRY(pl->ctx, cudaEventCreate(&tt.ev0)); CUDA_TRY(pl->ctx, cudaEventCreate(&tt.ev1)); }
    return MSNH_B200_OK;
}
int tile_tuning_end(MsnhB200Plan *pl, TileTuning &tt) {
    if (tt.ev0) { cudaEventDestroy(tt.ev0); cudaEventDestroy(tt.ev1); tt.ev0 = tt.ev1 = nullptr; CUDA_TRY(pl->ctx, cudaStreamSynchronize(pl->ctx->stream)); }
    return MSNH_B200_OK;
}

int configure_conv_umma(MsnhB200Plan *pl, TileTuning &tt, Launch &L) {
    MsnhB200Ctx *ctx = pl->ctx;
    const int es = esize(pl->dtype);
    const PlanDebugOptions &dbg = pl->dbg;
    std::vector<std::array<int, 3>> tune_cands;
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
        u.trace_tile = dbg.trace_tile;
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
        const int forced_mm = dbg.forced_mm, forced_bn = dbg.forced_bn;
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
        const int sk_mode = dbg.stream_k;
        // CTA pairs (cta_group::2, tiles of 256 pixels x bn): measured no faster than single CTAs with
        // the same bn, because the MMA issue interval and not shared-memory traffic bounds the main
        // loop; kept selectable (MSNH_B200_PAIR=1) and covered by the GPU tests.
        const int pair_mode = dbg.pair;
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
        if (dbg.no_split >= 0) L.no_split = dbg.no_split != 0;   // parity tests of that epilogue form
        tune_cands.clear();
        // a pack file carries the shapes its plan ended up with: no need to time them again
        const bool stored = pl->pack_loaded && tt.umma_seen < pl->pack_picks.size() && !forced_mm && !forced_bn && pair_mode != 1 && sk_mode == 0 &&
                            dbg.no_split < 0;
        if (stored) {
            const std::array<int32_t, 3> &pk = pl->pack_picks[tt.umma_seen];
            bool valid = false;
            for (const Cand &c : cands) valid = valid || (c.mm == pk[0] && c.bn == pk[1]);
            if (valid) { u.m_mult = pk[0]; u.bn = pk[1]; u.pair = 0; u.stream_k = 0; L.no_split = (pk[2] & 0xff) == 2; if (pk[2] >= 0x100) L.note += L.note.empty() ? "measured shape" : ", measured shape"; }
        }
        if (!stored && tt.autotune && !best_pair && !best_sk && !forced_mm && !forced_bn) {
            std::sort(cands.begin(), cands.end(), [](const Cand &x, const Cand &y) { return x.cost < y.cost; });
            // (stream-K forms were measured too and never won a layer; more than six runners-up changed nothing)
            const int tune_max = dbg.autotune > 0 ? dbg.autotune : 6;
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
    prepare_conv_umma_launch(L);
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
                    CUDA_TRY(ctx, cudaEventRecord(tt.ev0, ctx->stream));
                    for (int r = 0; r < 3; ++r) launch_one(ctx, t, ctx->stream);
                    CUDA_TRY(ctx, cudaEventRecord(tt.ev1, ctx->stream));
                    CUDA_TRY(ctx, cudaEventSynchronize(tt.ev1));
                    CUDA_TRY(ctx, cudaEventElapsedTime(&burst, tt.ev0, tt.ev1));
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
    ++tt.umma_seen;
    return MSNH_B200_OK;
}

}  // namespace msnh
