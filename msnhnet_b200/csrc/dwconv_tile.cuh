// 3x3 depthwise convolution (groups == Cin == Cout, dilation 1, stride 1 or 2) with the folded BatchNorm / bias and the
// activation, on channels-last tensors. The reference runs one im2col + Sgemm per channel and image
// (src/layers/MsnhConvolutionalLayer.cpp:1028-1066). Here a CTA of four warps walks output tiles of th x 16 pixels x 32
// channels: the input tile with its one-pixel halo is brought into shared memory by ONE TMA load (4-D box over channels, W,
// H, image; pixels outside the plane arrive as zeros, which is the conv's padding) into a ring of two or three stages, so
// that loads are in flight under the arithmetic of a tile and every input value is read from HBM once. There is no
// block-wide barrier: a stage is handed over through a "full" mbarrier (the load's byte count) and an "empty" one (one
// arrival per warp). A thread computes R rows x 2 columns of output pixels for four channels in packed fp32 pairs: each
// input value it reads from shared memory (at an offset that is an immediate of the load) is converted once and feeds up
// to six outputs; the nine weight vectors of its channels stay in registers for the whole kernel.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "conv_umma.cuh"     // mbarrier / TMA wrappers

namespace msnh {

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

// Dynamic shared memory: [p.stages x input tile (128-byte aligned)].
// Thread t owns channel quad t % 8 of its CTA's channel group for the whole kernel and takes the tile's work items
// (pair of output columns, group of R output rows) t / 8, t / 8 + 16, ... kRelu6: the activation is min(max(y, 0), 6),
// applied to the rounded 16-bit pair (the same value as rounding the clamped fp32: 0 and 6 are exact and rounding is
// monotonic); otherwise p.act is dispatched per value.
template <typename T, int S, bool kRelu6>
__global__ void __launch_bounds__(kDwThreads, 4)
dwconv3x3_tile_kernel(const __grid_constant__ CUtensorMap map_in, TView out, const T *__restrict__ w, const float *__restrict__ scale,
                      const float *__restrict__ bias, const DwTileParams p) {
    constexpr int R = dw_rows(S);
    constexpr int IW = dw_in_w(S);
    constexpr int IR = (R - 1) * S + 3;                       // input rows of a work item
    constexpr int IC = S + 3;                                 // input columns of a work item (two output columns)
    constexpr int CG = kDwChannels, QUADS = CG / 4, ROUND = kDwThreads / QUADS, CPS = kDwTileW / 2;
    constexpr uint32_t PX = CG * sizeof(T), ROW = IW * PX;    // byte pitches of the tile in shared memory
    extern __shared__ uint8_t dw_smem_raw[];
    __shared__ uint64_t bars[2 * kDwMaxStages];
    __shared__ int abort_slot;
    volatile int *cta_abort = &abort_slot;
    const uint32_t smem_base = (smem_u32(dw_smem_raw) + 127u) & ~127u;
    const uint32_t tile_bytes = static_cast<uint32_t>(p.ih) * ROW;
    const uint32_t stage_bytes = (tile_bytes + 127u) & ~127u;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kDwMaxStages]);
    const int NS = p.stages;
    const int total = out.N * p.tiles_h * p.tiles_w * p.tiles_c;
    const int lane = threadIdx.x & 31;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_in) : "memory");
        abort_slot = 0;
        for (int s = 0; s < NS; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, kDwThreads / 32); }
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
        const uint32_t bar = full0 + 8u * stage;
        mbar_expect_tx(bar, tile_bytes);
        tma_load_4d(smem_base + stage * stage_bytes, &map_in, bar, tc * CG, tx * kDwTileW * S - p.pw, ty * p.th * S - p.ph, n);
    };
    // constants of this thread's four channels (not produced by the previous kernel: read before waiting for it)
    const int q = threadIdx.x % QUADS, j0 = threadIdx.x / QUADS;
    const int ch = (static_cast<int>(blockIdx.x) % p.tiles_c) * CG + q * 4;
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
    if (threadIdx.x == 0) {
        for (int s = 0; s < NS - 1; ++s) {
            const int t = static_cast<int>(blockIdx.x) + s * static_cast<int>(gridDim.x);
            if (t < total) issue(t, s);
        }
    }

    const int items = CPS * (p.th / R);
    const size_t out_row = static_cast<size_t>(out.W) * out.ldc;
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++it) {
        const int stage = it % NS;
        // refill the stage that tile it - 1 used (every warp has arrived on its "empty" barrier when done with it)
        if (threadIdx.x == 0) {
            const int tn = t + (NS - 1) * static_cast<int>(gridDim.x);
            if (tn < total) {
                const int sn = (it + NS - 1) % NS;
                if (it >= 1) ok = mbar_wait(empty0 + 8u * sn, static_cast<uint32_t>((it - 1) / NS) & 1u, cta_abort, p.err_flag, DEV_ERR_WAIT_EMPTY);
                if (ok) issue(tn, sn);
            }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0) && mbar_wait(full0 + 8u * stage, static_cast<uint32_t>(it / NS) & 1u, cta_abort, p.err_flag, DEV_ERR_WAIT_FULL);
        if (!ok) break;
        int n, ty, tx, tc; coords(t, n, ty, tx, tc);
        const uint32_t tile = smem_base + stage * stage_bytes + static_cast<uint32_t>(q * 4) * sizeof(T);
        const int oy0 = ty * p.th, ox0 = tx * kDwTileW;
        for (int i = j0; i < items; i += ROUND) {
            const int cp = i % CPS, rg = i / CPS;
            const int ox = ox0 + 2 * cp, oy = oy0 + rg * R;                  // first output pixel of the item
            if (!ch_ok || ox >= out.W || oy >= out.H) continue;
            F2 acc[R][2][2];                                                // [row][column][channel pair]
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c) { acc[r][c][0] = f2_pack(0.f, 0.f); acc[r][c][1] = f2_pack(0.f, 0.f); }
            const uint32_t a0 = tile + static_cast<uint32_t>(rg * R * S) * ROW + static_cast<uint32_t>(2 * cp * S) * PX;
#pragma unroll
            for (int iy = 0; iy < IR; ++iy) {
                F2 x[IC][2];
#pragma unroll
                for (int s = 0; s < IC; ++s) lds4<T>(a0 + iy * ROW + s * PX, x[s][0], x[s][1]);
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
            T *dst0 = static_cast<T *>(out.ptr) + pix_off(out, n, oy, ox) + ch;
            const bool second = ox + 1 < out.W;
            const int rows = min(R, out.H - oy);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (r >= rows) break;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    if (c == 1 && !second) break;
                    const F2 y01 = f2_fma(acc[r][c][0], sc[0], bi[0]), y23 = f2_fma(acc[r][c][1], sc[1], bi[1]);
                    float y[4];
                    f2_unpack(y01, y[0], y[1]);
                    f2_unpack(y23, y[2], y[3]);
                    T *dst = dst0 + r * out_row + c * out.ldc;
                    if constexpr (sizeof(T) == 2 && kRelu6) {
                        uint32_t a, b;
                        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(a) : "f"(y[1]), "f"(y[0]));
                        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(b) : "f"(y[3]), "f"(y[2]));
                        const __half2 zero = __float2half2_rn(0.f), six = __float2half2_rn(6.f);
                        __half2 ha = __hmin2(__hmax2(*reinterpret_cast<__half2 *>(&a), zero), six);
                        __half2 hb = __hmin2(__hmax2(*reinterpret_cast<__half2 *>(&b), zero), six);
                        *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<uint32_t *>(&ha), *reinterpret_cast<uint32_t *>(&hb));
                    } else {
                        if constexpr (kRelu6) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) y[e] = fminf(fmaxf(y[e], 0.f), 6.f);
                        } else if (p.act != MSNH_ACT_NONE) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) y[e] = activate(y[e], p.act, p.act_param);
                        }
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
        }
        // this warp is done reading the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8u * stage);
    }
}

}  // namespace msnh
