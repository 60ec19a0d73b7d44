// 3x3 depthwise convolution (groups == Cin == Cout, dilation 1, stride 1 or 2) with the folded BatchNorm / bias and the
// activation, on channels-last tensors. The reference runs one im2col + Sgemm per channel and image
// (src/layers/MsnhConvolutionalLayer.cpp:1028-1066). Here a CTA walks output tiles of th x tw pixels x a group of channels:
// the input tile with its one-pixel halo is brought into shared memory by ONE TMA load (4-D box over channels, W, H, image;
// pixels outside the plane arrive as zeros, which is the conv's padding), double-buffered so the load of the next tile
// runs under the arithmetic of this one, and every input value is read from HBM once. A thread computes a column of R
// output pixels for four channels: each input value it reads from shared memory is converted once and feeds up to three
// output rows; the nine weight vectors of its channels sit in registers.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "conv_umma.cuh"     // mbarrier / TMA wrappers

namespace msnh {

struct DwTileParams {
    int tiles_w, tiles_h, tiles_c;   // tiles per plane and channel groups per pixel
    int th, tw;                      // output pixels per tile
    int ih, iw;                      // input pixels per tile: (th - 1) * S + 3, (tw - 1) * S + 3
    int cg;                          // channels per tile (a multiple of the 16-byte vector, at most 256)
    int ph, pw;
    int act; float act_param;
    int *err_flag;
};

constexpr int kDwThreads = 256;
constexpr int kDwRows = 4;           // output rows per thread (R)

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c, int w, int h, int n) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n) : "memory");
}

// four consecutive channels of one pixel from shared memory, as fp32
template <typename T> __device__ __forceinline__ void lds4(uint32_t addr, float (&v)[4]);
template <> __device__ __forceinline__ void lds4<__half>(uint32_t addr, float (&v)[4]) {
    uint32_t a, b;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&a)), hi = __half22float2(*reinterpret_cast<const __half2 *>(&b));
    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
}
template <> __device__ __forceinline__ void lds4<float>(uint32_t addr, float (&v)[4]) {
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(addr));
}

// Dynamic shared memory: [2 stages x input tile (128-byte aligned)] [weights 9 x cg fp32] [scale cg] [bias cg].
template <typename T, int S>
__global__ void __launch_bounds__(kDwThreads)
dwconv3x3_tile_kernel(const __grid_constant__ CUtensorMap map_in, TView out, const T *__restrict__ w, const float *__restrict__ scale,
                      const float *__restrict__ bias, const DwTileParams p) {
    constexpr int R = kDwRows;
    constexpr int IR = (R - 1) * S + 3;                       // input rows a thread's column of outputs reads
    extern __shared__ uint8_t dw_smem_raw[];
    __shared__ uint64_t bars[2];
    __shared__ int abort_slot;
    volatile int *cta_abort = &abort_slot;
    const uint32_t smem_base = (smem_u32(dw_smem_raw) + 127u) & ~127u;
    const uint32_t stage_bytes = (static_cast<uint32_t>(p.ih * p.iw * p.cg) * sizeof(T) + 127u) & ~127u;
    const uint32_t wts_base = smem_base + 2u * stage_bytes;                    // fp32 [9][cg], then scale [cg], bias [cg]
    float *wts = reinterpret_cast<float *>(dw_smem_raw + (wts_base - smem_u32(dw_smem_raw)));
    const uint32_t bar0 = smem_u32(&bars[0]);
    const int total = out.N * p.tiles_h * p.tiles_w * p.tiles_c;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_in) : "memory");
        abort_slot = 0;
        mbar_init(bar0, 1); mbar_init(bar0 + 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // tile index -> coordinates; channel groups innermost so that CTAs running together share input rows in L2
    auto coords = [&](int t, int &n, int &ty, int &tx, int &tc) {
        tc = t % p.tiles_c; t /= p.tiles_c;
        tx = t % p.tiles_w; t /= p.tiles_w;
        ty = t % p.tiles_h; n = t / p.tiles_h;
    };
    auto issue = [&](int t, int stage) {       // one thread: the whole input tile of tile t, zeros outside the plane
        int n, ty, tx, tc; coords(t, n, ty, tx, tc);
        const uint32_t bar = bar0 + 8u * stage;
        mbar_expect_tx(bar, static_cast<uint32_t>(p.ih * p.iw * p.cg) * sizeof(T));
        tma_load_4d(smem_base + stage * stage_bytes, &map_in, bar, tc * p.cg, tx * p.tw * S - p.pw, ty * p.th * S - p.ph, n);
    };
    pdl_wait();
    if (threadIdx.x == 0 && static_cast<int>(blockIdx.x) < total) issue(blockIdx.x, 0);

    const int cq = p.cg / 4;                         // groups of four channels per tile
    const int rgs = (p.th + R - 1) / R;              // row groups per tile
    const int items = cq * p.tw * rgs;
    int last_tc = -1;
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++it) {
        const int stage = it & 1;
        int n, ty, tx, tc; coords(t, n, ty, tx, tc);
        // the other stage was last read one iteration ago (barrier at the end of that iteration): prefetch the next tile
        if (threadIdx.x == 0 && t + static_cast<int>(gridDim.x) < total) issue(t + gridDim.x, stage ^ 1);
        if (tc != last_tc) {                         // weights, scale, bias of this channel group -> shared memory as fp32
            if (last_tc >= 0) __syncthreads();       // (everybody is past its reads of the previous group's tables)
            for (int i = threadIdx.x; i < 11 * p.cg; i += blockDim.x) {
                const int row = i / p.cg, c = i - row * p.cg, ch = tc * p.cg + c;
                float v = 0.f;
                if (ch < out.C) v = row < 9 ? Elem<T>::ld(w + static_cast<size_t>(row) * out.C + ch) : (row == 9 ? (scale ? scale[ch] : 1.f) : (bias ? bias[ch] : 0.f));
                wts[i] = v;
            }
            last_tc = tc;
            __syncthreads();
        }
        ok = mbar_wait(bar0 + 8u * stage, static_cast<uint32_t>(it >> 1) & 1u, cta_abort, p.err_flag, DEV_ERR_WAIT_FULL);
        if (!ok) break;
        const uint32_t tile = smem_base + stage * stage_bytes;
        const int oy0 = ty * p.th, ox0 = tx * p.tw;
        for (int i = threadIdx.x; i < items; i += blockDim.x) {
            const int q = i % cq; int rest = i / cq;
            const int ox = rest % p.tw; const int rg = rest / p.tw;
            const int c = q * 4, ch = tc * p.cg + c;
            if (ch >= out.C || ox0 + ox >= out.W) continue;
            float wr[9][4];
#pragma unroll
            for (int k = 0; k < 9; ++k) {
                const float4 f = *reinterpret_cast<const float4 *>(wts + k * p.cg + c);
                wr[k][0] = f.x; wr[k][1] = f.y; wr[k][2] = f.z; wr[k][3] = f.w;
            }
            float acc[R][4];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[r][e] = 0.f;
            const int iy0 = rg * R * S, ix0 = ox * S;
            const uint32_t col = tile + static_cast<uint32_t>((iy0 * p.iw + ix0) * p.cg + c) * sizeof(T);
            const uint32_t row_pitch = static_cast<uint32_t>(p.iw * p.cg) * sizeof(T), px_pitch = static_cast<uint32_t>(p.cg) * sizeof(T);
#pragma unroll
            for (int iy = 0; iy < IR; ++iy) {
                if (iy0 + iy >= p.ih) break;                               // (last row group of a tile whose height is no multiple of R)
                float x[3][4];
#pragma unroll
                for (int s = 0; s < 3; ++s) lds4<T>(col + iy * row_pitch + s * px_pitch, x[s]);
#pragma unroll
                for (int kh = 0; kh < 3; ++kh) {
                    if ((iy - kh) % S != 0 || iy - kh < 0) continue;       // (resolved at compile time: the loops are unrolled)
                    const int r = (iy - kh) / S;
                    if (r >= R) continue;
#pragma unroll
                    for (int s = 0; s < 3; ++s)
#pragma unroll
                        for (int e = 0; e < 4; ++e) acc[r][e] = fmaf(x[s][e], wr[kh * 3 + s][e], acc[r][e]);
                }
            }
            const float4 sc = *reinterpret_cast<const float4 *>(wts + 9 * p.cg + c), bi = *reinterpret_cast<const float4 *>(wts + 10 * p.cg + c);
            const float scv[4] = {sc.x, sc.y, sc.z, sc.w}, biv[4] = {bi.x, bi.y, bi.z, bi.w};
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int oy = oy0 + rg * R + r;
                if (rg * R + r >= p.th || oy >= out.H) break;
                float y[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) y[e] = fmaf(acc[r][e], scv[e], biv[e]);
                switch (p.act) {
                    case MSNH_ACT_NONE: break;
                    case MSNH_ACT_RELU6:
#pragma unroll
                        for (int e = 0; e < 4; ++e) y[e] = fminf(fmaxf(y[e], 0.f), 6.f);
                        break;
                    case MSNH_ACT_RELU:
#pragma unroll
                        for (int e = 0; e < 4; ++e) y[e] = y[e] > 0.f ? y[e] : 0.f;
                        break;
                    default:
#pragma unroll
                        for (int e = 0; e < 4; ++e) y[e] = activate(y[e], p.act, p.act_param);
                        break;
                }
                T *dst = static_cast<T *>(out.ptr) + pix_off(out, n, oy, ox0 + ox) + ch;
                if constexpr (sizeof(T) == 2) {
                    const __half2 a = __floats2half2_rn(y[0], y[1]), b = __floats2half2_rn(y[2], y[3]);
                    *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
                } else {
                    if (out.tf32) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) y[e] = round_tf32(y[e]);
                    }
                    *reinterpret_cast<float4 *>(dst) = make_float4(y[0], y[1], y[2], y[3]);
                }
            }
        }
        __syncthreads();          // every thread is done with this stage before the next iteration's prefetch overwrites it
    }
}

}  // namespace msnh
