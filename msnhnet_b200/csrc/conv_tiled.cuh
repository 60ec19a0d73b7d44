// Dense convolution on the CUDA cores in fp32 arithmetic: an implicit GEMM with shared-memory tiles, for the plans that must
// reproduce the reference's fp32 results (its GPU path is fp32 Sgemm throughout, src/layers/MsnhConvolutionalLayer.cpp:1026-1160):
// fp32 detection nets, whose exp()-decoded boxes do not survive tf32's 10-bit mantissa, and plans built without tensor cores.
// D[m][n] = sum_k A[m][k] * B[n][k]: m = output pixel (linear over image, row, column), n = output channel, k = (filter
// tap, input channel) tap-major like the packed weights [Cout][tap][cin_pad]. A CTA of 256 threads computes 128 pixels x
// 64 channels; a k-step stages 128 x BK input values (gathered with the conv's stride / padding / dilation, zero outside the
// plane) and 64 x BK weights in shared memory as fp32, k-major, so that the inner loop reads them without bank conflicts;
// the next k-step's global loads are in flight while this one's products are summed. A thread owns 8 pixels x 4 channels.
#pragma once
#include "common.cuh"
#include "layer_kernels.cuh"

namespace msnh {

template <typename T>
__global__ void __launch_bounds__(kCtThreads)
conv_tiled_kernel(TView in, TView out, const T *__restrict__ w, const ConvTiledParams p) {
    constexpr int V = Elem<T>::kVec;           // elements per 16-byte vector
    constexpr int BK = 4 * V;                  // k elements per step: four vectors per pixel / per output channel
    __shared__ float As[BK][kCtBM + 4];
    __shared__ float Bs[BK][kCtBN + 4];
    pdl_prologue();
    const int tid = threadIdx.x;
    const int m_total = out.N * out.H * out.W;
    const int m0 = blockIdx.x * kCtBM, n0 = blockIdx.y * kCtBN;
    const int cin = in.C, cout = out.C;
    // this thread's global loads: two pixels (64 apart) x one vector of A, one output channel x one vector of B
    const int kq = tid & 3;                    // which of the four vectors of the k-step
    const int lrow = tid >> 2;                 // 0..63
    int pn[2], py[2], px[2]; bool pvalid[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int m = m0 + lrow + 64 * j;
        pvalid[j] = m < m_total;
        const int mm = pvalid[j] ? m : 0;
        pn[j] = mm / (out.H * out.W);
        const int rem = mm - pn[j] * out.H * out.W;
        py[j] = rem / out.W; px[j] = rem - py[j] * out.W;
    }
    const int co_ld = n0 + lrow;               // (lrow < 64: every thread loads one vector of B)
    const T *wrow = w + static_cast<size_t>(co_ld < cout ? co_ld : 0) * p.kh * p.kw * p.cin_pad;
    // compute mapping: pixels tm + 16 i (i < 8), channels 4 tn .. 4 tn + 3
    const int tm = tid & 15, tn = tid >> 4;
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

    const int chunks = (cin + BK - 1) / BK;
    const int steps = p.kh * p.kw * chunks;
    float ra[2][V], rb[V];
    auto load_step = [&](int step) {
        const int tap = step / chunks, c = (step - tap * chunks) * BK + kq * V;
        const int r = tap / p.kw, s = tap - r * p.kw;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int iy = py[j] * p.sh - p.ph + r * p.dh, ix = px[j] * p.sw - p.pw + s * p.dw;
            const bool inside = pvalid[j] && iy >= 0 && iy < in.H && ix >= 0 && ix < in.W && c < cin;
            if (inside) {
                const T *src = static_cast<const T *>(in.ptr) + pix_off(in, pn[j], iy, ix) + c;
                if (c + V <= in.ldc) VecIO<T, V>::ld(src, ra[j]);
                else {
#pragma unroll
                    for (int e = 0; e < V; ++e) ra[j][e] = c + e < cin ? Elem<T>::ld(src + e) : 0.f;
                }
#pragma unroll
                for (int e = 0; e < V; ++e) if (c + e >= cin) ra[j][e] = 0.f;     // pad channels of the pitch hold no data
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) ra[j][e] = 0.f;
            }
        }
        if (co_ld < cout && c < p.cin_pad) VecIO<T, V>::ld(wrow + static_cast<size_t>(tap) * p.cin_pad + c, rb);
        else {
#pragma unroll
            for (int e = 0; e < V; ++e) rb[e] = 0.f;
        }
    };
    load_step(0);
    for (int step = 0; step < steps; ++step) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
            As[kq * V + e][lrow] = ra[0][e];
            As[kq * V + e][lrow + 64] = ra[1][e];
            Bs[kq * V + e][lrow] = rb[e];
        }
        __syncthreads();
        if (step + 1 < steps) load_step(step + 1);          // in flight under the arithmetic below
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = As[k][tm + 16 * i];
            const float4 b = *reinterpret_cast<const float4 *>(&Bs[k][4 * tn]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                acc[i][0] = fmaf(a[i], b.x, acc[i][0]); acc[i][1] = fmaf(a[i], b.y, acc[i][1]);
                acc[i][2] = fmaf(a[i], b.z, acc[i][2]); acc[i][3] = fmaf(a[i], b.w, acc[i][3]);
            }
        }
        __syncthreads();
    }
    // epilogue: scale / bias, activation, residual (+ second activation), store
    const int c0 = n0 + 4 * tn;
    if (c0 >= cout) return;
    float sc[4], bi[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        sc[e] = (p.scale && c0 + e < cout) ? p.scale[c0 + e] : 1.f;
        bi[e] = (p.bias && c0 + e < cout) ? p.bias[c0 + e] : 0.f;
    }
    const T *res = static_cast<const T *>(p.res);
    const bool vec_ok = c0 + 4 <= cout && (out.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(out.ptr) & 15) == 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + tm + 16 * i;
        if (m >= m_total) continue;
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            y[e] = activate(fmaf(acc[i][e], sc[e], bi[e]), p.act1, p.act1_param);
            if (res && c0 + e < cout) y[e] = activate(y[e] + Elem<T>::ld(res + static_cast<size_t>(m) * p.ldc_res + c0 + e), p.act2, p.act2_param);
            if (sizeof(T) == 4 && out.tf32) y[e] = round_tf32(y[e]);
        }
        T *dst = static_cast<T *>(out.ptr) + static_cast<size_t>(m) * out.ldc + c0;
        if (vec_ok) {
            if constexpr (sizeof(T) == 4) *reinterpret_cast<float4 *>(dst) = make_float4(y[0], y[1], y[2], y[3]);
            else {
                const __half2 lo = __floats2half2_rn(y[0], y[1]), hi = __floats2half2_rn(y[2], y[3]);
                *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
            }
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) if (c0 + e < cout) Elem<T>::st(dst + e, y[e]);
        }
    }
}

}  // namespace msnh
