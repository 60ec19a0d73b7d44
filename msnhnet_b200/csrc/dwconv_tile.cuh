// 3x3 depthwise convolution (groups == Cin == Cout, dilation 1, stride 1 or 2) with the folded BatchNorm / bias and the
// activation, on channels-last tensors. The reference runs one im2col + Sgemm per channel and image
// (src/layers/MsnhConvolutionalLayer.cpp:1028-1066). Here a CTA walks output tiles of th x tw pixels x a group of channels:
// the input tile with its one-pixel halo is brought into shared memory by ONE TMA load (4-D box over channels, W, H, image;
// pixels outside the plane arrive as zeros, which is the conv's padding), double-buffered so the load of the next tile
// runs under the arithmetic of this one, and every input value is read from HBM once. A thread computes R rows x 2 columns
// of output pixels for four channels in packed fp32 pairs: each input value it reads from shared memory is converted once
// and feeds up to six outputs; the nine weight vectors of its channels stay in registers for the whole kernel.
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

// four consecutive channels of one pixel from shared memory, as two packed fp32 pairs
template <typename T> __device__ __forceinline__ void lds4(uint32_t addr, F2 &lo, F2 &hi);
template <> __device__ __forceinline__ void lds4<__half>(uint32_t addr, F2 &lo, F2 &hi) {
    uint32_t a, b;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
    const float2 x = __half22float2(*reinterpret_cast<const __half2 *>(&a)), y = __half22float2(*reinterpret_cast<const __half2 *>(&b));
    lo = f2_pack(x.x, x.y); hi = f2_pack(y.x, y.y);
}
template <> __device__ __forceinline__ void lds4<float>(uint32_t addr, F2 &lo, F2 &hi) {
    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(lo.v), "=l"(hi.v) : "r"(addr));
}

// Dynamic shared memory: [2 stages x input tile (128-byte aligned)].
// Threads: blockDim.x = nq * cq, cq = channel quads per tile; thread t owns quad t % cq for the whole kernel (its nine
// weight vectors, scale and bias stay in registers) and takes the tile's work items (pair of output columns, group of R
// output rows) t / cq, t / cq + nq, ... A work item reads (R - 1) * S + 3 input rows of (S + 3) pixels, each value once.
template <typename T, int S>
__global__ void __launch_bounds__(kDwThreads)
dwconv3x3_tile_kernel(const __grid_constant__ CUtensorMap map_in, TView out, const T *__restrict__ w, const float *__restrict__ scale,
                      const float *__restrict__ bias, const DwTileParams p) {
    constexpr int R = kDwRows;
    constexpr int IR = (R - 1) * S + 3;                       // input rows of a work item
    constexpr int IC = S + 3;                                 // input columns of a work item (two output columns)
    extern __shared__ uint8_t dw_smem_raw[];
    __shared__ uint64_t bars[2];
    __shared__ int abort_slot;
    volatile int *cta_abort = &abort_slot;
    const uint32_t smem_base = (smem_u32(dw_smem_raw) + 127u) & ~127u;
    const uint32_t stage_bytes = (static_cast<uint32_t>(p.ih * p.iw * p.cg) * sizeof(T) + 127u) & ~127u;
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
    // tile index -> coordinates; channel groups innermost, and the grid is a multiple of their number, so a CTA keeps its group
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
    // constants of this thread's four channels (not produced by the previous kernel: read before waiting for it)
    const int cq = p.cg / 4;
    const int q = threadIdx.x % cq, j0 = threadIdx.x / cq, nq = blockDim.x / cq;
    const int ch = (static_cast<int>(blockIdx.x) % p.tiles_c) * p.cg + q * 4;
    const bool ch_ok = ch < out.C;                   // (out.C is a multiple of four here: whole quads)
    F2 wr[9][2], sc[2], bi[2];
#pragma unroll
    for (int k = 0; k < 9; ++k)
#pragma unroll
        for (int h = 0; h < 2; ++h)
            wr[k][h] = ch_ok ? f2_pack(Elem<T>::ld(w + static_cast<size_t>(k) * out.C + ch + 2 * h), Elem<T>::ld(w + static_cast<size_t>(k) * out.C + ch + 2 * h + 1)) : f2_pack(0.f, 0.f);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        sc[h] = (ch_ok && scale) ? f2_pack(scale[ch + 2 * h], scale[ch + 2 * h + 1]) : f2_pack(1.f, 1.f);
        bi[h] = (ch_ok && bias) ? f2_pack(bias[ch + 2 * h], bias[ch + 2 * h + 1]) : f2_pack(0.f, 0.f);
    }
    pdl_wait();
    if (threadIdx.x == 0 && static_cast<int>(blockIdx.x) < total) issue(blockIdx.x, 0);

    const int rgs = (p.th + R - 1) / R;              // row groups per tile
    const int cps = (p.tw + 1) / 2;                  // column pairs per tile
    const int items = cps * rgs;
    const uint32_t row_pitch = static_cast<uint32_t>(p.iw * p.cg) * sizeof(T), px_pitch = static_cast<uint32_t>(p.cg) * sizeof(T);
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++it) {
        const int stage = it & 1;
        int n, ty, tx, tc; coords(t, n, ty, tx, tc);
        // the other stage was last read one iteration ago (barrier at the end of that iteration): prefetch the next tile
        if (threadIdx.x == 0 && t + static_cast<int>(gridDim.x) < total) issue(t + gridDim.x, stage ^ 1);
        ok = mbar_wait(bar0 + 8u * stage, static_cast<uint32_t>(it >> 1) & 1u, cta_abort, p.err_flag, DEV_ERR_WAIT_FULL);
        if (!ok) break;
        const uint32_t tile = smem_base + stage * stage_bytes + static_cast<uint32_t>(q * 4) * sizeof(T);
        const int oy0 = ty * p.th, ox0 = tx * p.tw;
        for (int i = j0; ch_ok && i < items; i += nq) {
            const int cp = i % cps, rg = i / cps;
            const int ox = 2 * cp;                                          // first of the two output columns, within the tile
            const bool second = ox + 1 < p.tw && ox0 + ox + 1 < out.W;
            if (ox0 + ox >= out.W) continue;
            F2 acc[R][2][2];                                                // [row][column][channel pair]
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c) { acc[r][c][0] = f2_pack(0.f, 0.f); acc[r][c][1] = f2_pack(0.f, 0.f); }
            const int iy0 = rg * R * S;
            const uint32_t col = tile + static_cast<uint32_t>(iy0 * p.iw + ox * S) * px_pitch;
            // (an input column past the tile's box exists only for a second output column that does not: its products are discarded)
            const int cols_in = min(IC, p.iw - ox * S);
#pragma unroll
            for (int iy = 0; iy < IR; ++iy) {
                if (iy0 + iy >= p.ih) break;                               // (last row group of a tile whose height is no multiple of R)
                F2 x[IC][2];
#pragma unroll
                for (int s = 0; s < IC; ++s) {
                    if (s < cols_in) lds4<T>(col + iy * row_pitch + s * px_pitch, x[s][0], x[s][1]);
                    else { x[s][0] = f2_pack(0.f, 0.f); x[s][1] = x[s][0]; }
                }
#pragma unroll
                for (int kh = 0; kh < 3; ++kh) {
                    if ((iy - kh) % S != 0 || iy - kh < 0) continue;       // (resolved at compile time: the loops are unrolled)
                    const int r = (iy - kh) / S;
                    if (r >= R) continue;
#pragma unroll
                    for (int c = 0; c < 2; ++c)
#pragma unroll
                        for (int s = 0; s < 3; ++s) {
                            acc[r][c][0] = f2_fma(x[c * S + s][0], wr[kh * 3 + s][0], acc[r][c][0]);
                            acc[r][c][1] = f2_fma(x[c * S + s][1], wr[kh * 3 + s][1], acc[r][c][1]);
                        }
                }
            }
            T *dst0 = static_cast<T *>(out.ptr) + pix_off(out, n, oy0 + rg * R, ox0 + ox) + ch;
            const size_t out_row = static_cast<size_t>(out.W) * out.ldc;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (rg * R + r >= p.th || oy0 + rg * R + r >= out.H) break;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    if (c == 1 && !second) break;
                    float y[4];
                    f2_unpack(f2_fma(acc[r][c][0], sc[0], bi[0]), y[0], y[1]);
                    f2_unpack(f2_fma(acc[r][c][1], sc[1], bi[1]), y[2], y[3]);
                    switch (p.act) {
                        case MSNH_ACT_NONE: break;
                        case MSNH_ACT_RELU6:
#pragma unroll
                            for (int e = 0; e < 4; ++e) y[e] = fminf(fmaxf(y[e], 0.f), 6.f);
                            break;
                        case MSNH_ACT_RELU:
#pragma unroll
                            for (int e = 0; e < 4; ++e) y[e] = fmaxf(y[e], 0.f);
                            break;
                        default:
#pragma unroll
                            for (int e = 0; e < 4; ++e) y[e] = activate(y[e], p.act, p.act_param);
                            break;
                    }
                    T *dst = dst0 + r * out_row + c * out.ldc;
                    if constexpr (sizeof(T) == 2) {
                        uint32_t a, b;
                        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(a) : "f"(y[1]), "f"(y[0]));
                        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(b) : "f"(y[3]), "f"(y[2]));
                        *reinterpret_cast<uint2 *>(dst) = make_uint2(a, b);
                    } else {
                        if (out.tf32) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) y[e] = round_tf32(y[e]);
                        }
                        *reinterpret_cast<float4 *>(dst) = make_float4(y[0], y[1], y[2], y[3]);
                    }
                }
            }
        }
        __syncthreads();          // every thread is done with this stage before the next iteration's prefetch overwrites it
    }
}

}  // namespace msnh
