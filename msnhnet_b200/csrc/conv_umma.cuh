// Implicit-GEMM convolution on the Blackwell tensor cores (tcgen05.mma, accumulators in TMEM,
// operands staged in shared memory by TMA), with the folded BatchNorm scale/bias, the activation
// and an optional residual add applied in the epilogue. Replaces, for one conv layer, the
// reference's fill + im2col + cublasSgemm + convBn + activation sequence
// (src/layers/MsnhConvolutionalLayer.cpp:1026-1160, src/core/cuda/MsnhGemmGPU.cu:57-145).
//
// GEMM view:  D[m][n] = sum_k A[m][k] * B[n][k]
//   m : output pixel, linear over (image, oh, ow)            -> TMEM lane
//   n : output channel                                       -> TMEM column
//   k : (filter tap r,s) x (input channel), tap-major        -> one k-block = one tap x BK channels
// A is never materialised: each k-block of A is one TMA load of the channels-last activation
// tensor, either an im2col-mode load (any kernel / stride / padding / dilation; the hardware walks
// 128 consecutive output pixels across row and image boundaries and zero-fills the padding) or,
// for 1x1 stride-1 layers, a plain 2-D tile of the [pixels][channels] matrix.
// B is the weight tensor packed as [Cout][tap][Cin] (K-major), one 2-D TMA tile per k-block.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace msnh {

// trace slots per CTA: 0 kernel start, 1 setup done, 2 end; 8+k: producer issued k-block k of its
// first tile; 24+k: MMA thread saw k-block k full; 40: accumulator of the first tile complete
// (epilogue side); 41: first tile's epilogue done; 42: tiles processed by this CTA; 43+4q..46+4q
// (q < 5): output slab q: start, store issued, values staged, all warps staged.

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One poll of a barrier phase.
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// The same with a suspend-time hint: the hardware parks the thread until the phase completes or the hint
// (nanoseconds) runs out, so a waiting warp neither takes issue slots from the warps that work nor polls shared
// memory. Measured on B200: with the sixteen epilogue warps parked like this while they wait for their first
// accumulator, the MMA thread's k-block period over a CTA's first tile drops from 622 to 554 cycles (one sub-tile) and
// from 814 to 749 (two); over a whole YOLOv4 step, where the epilogue warps mostly work instead of waiting, the gain is
// within the noise. A parked thread wakes later than a polling one, so the two latency-critical waits (the producer's
// for a free stage, the MMA thread's for a full one) keep polling.
#ifndef MSNH_WAIT_HINT_NS
#define MSNH_WAIT_HINT_NS 2000
#endif
__device__ __forceinline__ uint32_t mbar_try_wait_parked(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(static_cast<uint32_t>(MSNH_WAIT_HINT_NS)) : "memory");
    return ok;
}
// Bounded wait: gives up after ~kWaitCycles SM cycles (or as soon as another role of this CTA gave
// up), records `code` in the global error flag and returns false. The kernel then drains and exits.
constexpr long long kWaitCycles = 1500000000LL;
template <bool kParked = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *cta_abort,
                                          int *err_flag, int code) {
    auto poll = [&]() { return (kParked && MSNH_WAIT_HINT_NS > 0) ? mbar_try_wait_parked(bar, parity) : mbar_try_wait(bar, parity); };
    if (poll()) return true;
    const long long t0 = clock64();
    while (true) {
        for (int i = 0; i < 64; ++i)
            if (poll()) return true;
        if (*cta_abort) return false;
        if (clock64() - t0 > kWaitCycles) {
            *cta_abort = 1;
            atomicCAS(err_flag, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                                   int c, int w, int h, int n, uint16_t off_w, uint16_t off_h) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h) : "memory");
}
// ---- CTA-pair forms (cta_group::2): both CTAs of a 2-CTA cluster feed one MMA of 256 rows ----
// Loads land in the executing CTA's shared memory but may signal the barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                                        int c, int w, int h, int n, uint16_t off_w, uint16_t off_h) {
    asm volatile(
        "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h) : "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far retire
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}
template <bool kTf32>
__device__ __forceinline__ void tcgen05_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if (kTf32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    }
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <bool kTf32>
__device__ __forceinline__ void tcgen05_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if (kTf32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    }
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile whose rows are exactly one swizzle
// span wide (bk_bytes = 128/64/32 -> SWIZZLE_128B/64B/32B). Rows are packed back to back, so a
// group of 8 rows (one swizzle atom) is 8*bk_bytes apart from the next: that is the stride byte
// offset. The leading byte offset is unused for this layout (encoded 1). Bits 46-47 = 1 mark the
// sm_100 descriptor version.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, int bk_bytes) {
    const uint64_t layout = bk_bytes == 128 ? 2ull : (bk_bytes == 64 ? 4ull : 6ull);
    const uint64_t sbo    = static_cast<uint64_t>((8 * bk_bytes) >> 4);
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
    d |= 1ull << 16;
    d |= sbo << 32;
    d |= 1ull << 46;
    d |= layout << 61;
    return d;
}

// Activation of 16 accumulator values held in registers. The switch sits outside the loop so each
// case is a short unrolled loop; the rarely used activations share one out-of-line call.
// single SFU instructions (flush-to-zero forms: no range fix-up code around them)
__device__ __forceinline__ float fast_ex2(float x) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ float fast_rcp(float x) { float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __noinline__ float activate_slow(float x, int act, float param) { return activate(x, act, param); }
// Packed fp32 pairs (sm_100 fma/mul/add .f32x2): two lanes of arithmetic per issued instruction.
struct F2 { unsigned long long v; };
__device__ __forceinline__ F2 f2_pack(float a, float b) { F2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void f2_unpack(F2 x, float &a, float &b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(x.v)); }
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) { F2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v)); return r; }
__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) { F2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) { F2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }
__device__ __forceinline__ void activate16(float (&y)[16], int act, float param) {
    switch (act) {
        case MSNH_ACT_NONE: break;
        case MSNH_ACT_LEAKY:
            if (param >= 0.f && param <= 1.f) {      // max(x, a*x) equals the select for slopes in [0, 1]
                const F2 a2 = f2_pack(param, param);
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    float m0, m1; f2_unpack(f2_mul(f2_pack(y[j], y[j + 1]), a2), m0, m1);
                    y[j] = fmaxf(y[j], m0); y[j + 1] = fmaxf(y[j + 1], m1);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) y[j] = y[j] > 0.f ? y[j] : param * y[j];
            }
            break;
        case MSNH_ACT_RELU:
#pragma unroll
            for (int j = 0; j < 16; ++j) y[j] = fmaxf(y[j], 0.f);
            break;
        case MSNH_ACT_RELU6:
#pragma unroll
            for (int j = 0; j < 16; ++j) y[j] = fminf(fmaxf(y[j], 0.f), 6.f);
            break;
        case MSNH_ACT_MISH: {
            // x * tanh(log(1 + e^x)) = x * n / (n + 2), n = e^x (e^x + 2). Only e^x uses the SFU pipe; 1 / (n + 2)
            // is computed on the FMA pipe: a bit-pattern first guess (12 % off), one Newton step and one cubic
            // step, relative error ~1e-7. The arithmetic runs on packed fp32 pairs (half the instructions). The
            // exponent is clamped at 20, where n / (n + 2) rounds to 1.
            const F2 two = f2_pack(2.f, 2.f), one = f2_pack(1.f, 1.f), l2e = f2_pack(1.4426950408889634f, 1.4426950408889634f);
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                const F2 t = f2_mul(f2_pack(fminf(y[j], 20.f), fminf(y[j + 1], 20.f)), l2e);
                float t0, t1; f2_unpack(t, t0, t1);
                const F2 e = f2_pack(fast_ex2(t0), fast_ex2(t1));
                const F2 n = f2_mul(e, f2_add(e, two));
                const F2 d = f2_add(n, two);
                float d0, d1; f2_unpack(d, d0, d1);
                F2 g = f2_pack(__uint_as_float(0x7EF311C7u - __float_as_uint(d0)), __uint_as_float(0x7EF311C7u - __float_as_uint(d1)));
                const F2 nd = f2_pack(-d0, -d1);
                g = f2_mul(g, f2_fma(nd, g, two));                       // Newton: error e -> e^2
                const F2 h = f2_fma(nd, g, one);                          // cubic: g (1 + h + h^2), error e -> e^3
                const F2 r = f2_mul(n, f2_fma(g, f2_fma(h, h, h), g));
                const F2 out = f2_mul(f2_pack(y[j], y[j + 1]), r);
                f2_unpack(out, y[j], y[j + 1]);
            }
            break;
        }
        case MSNH_ACT_HARD_SWISH: {
            const F2 three = f2_pack(3.f, 3.f), sixth = f2_pack(0.16666667f, 0.16666667f);
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                const F2 x = f2_pack(y[j], y[j + 1]);
                float c0, c1; f2_unpack(f2_add(x, three), c0, c1);
                const F2 c = f2_pack(fminf(fmaxf(c0, 0.f), 6.f), fminf(fmaxf(c1, 0.f), 6.f));
                f2_unpack(f2_mul(f2_mul(x, c), sixth), y[j], y[j + 1]);     // (x * clamp) * (1/6), the order of the scalar form
            }
            break;
        }
        case MSNH_ACT_SWISH: {
            float d[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) d[j] = 1.f + fast_ex2(-y[j] * 1.4426950408889634f);
#pragma unroll
            for (int j = 0; j < 16; ++j) d[j] = fast_rcp(d[j]);
#pragma unroll
            for (int j = 0; j < 16; ++j) y[j] *= d[j];
            break;
        }
        case MSNH_ACT_LOGISTIC: {
            float d[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) d[j] = 1.f + fast_ex2(-y[j] * 1.4426950408889634f);
#pragma unroll
            for (int j = 0; j < 16; ++j) y[j] = fast_rcp(d[j]);
            break;
        }
        default:
#pragma unroll
            for (int j = 0; j < 16; ++j) y[j] = activate_slow(y[j], act, param);
            break;
    }
}

// The same on eight packed pairs, for the epilogue instantiations dedicated to one activation. The values never leave
// their register pairs except for the two scalar steps (ex2 and the reciprocal).
__device__ __forceinline__ void mish_pairs(F2 (&y)[8]) {
    // x * tanh(softplus(x)) = x * n / (n + 2) with n = e^x (e^x + 2), written as x - 2 x / d, d = n + 2 = e^x (e^x + 2) + 2:
    // one packed add and one packed FMA give d, and the form needs no guard against overflow (e^x = inf gives d = inf,
    // 1 / d = 0 and the result x, where n / (n + 2) would be inf * 0), so per pair: five packed operations and four SFU
    // ones (ex2 and the reciprocal of each value). The difference 1 - 2 / d cancels for x << 0, where the result itself
    // vanishes: the absolute error stays below 1e-7 |x|. The reciprocal stays on the SFU pipe: the epilogue is short of
    // registers and of instructions in flight rather than of SFU throughput (measured on the 1x1 64->64 layer at
    // 304x304: 47.7 us against 51.1 with the reciprocal refined on the FMA pipe).
    const F2 two = f2_pack(2.f, 2.f), minus2 = f2_pack(-2.f, -2.f), l2e = f2_pack(1.4426950408889634f, 1.4426950408889634f);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        float t0, t1; f2_unpack(f2_mul(y[q], l2e), t0, t1);
        const F2 e = f2_pack(fast_ex2(t0), fast_ex2(t1));
        float d0, d1; f2_unpack(f2_fma(e, f2_add(e, two), two), d0, d1);
        y[q] = f2_fma(f2_mul(y[q], f2_pack(fast_rcp(d0), fast_rcp(d1))), minus2, y[q]);
    }
}
__device__ __forceinline__ void leaky_pairs(F2 (&y)[8], float slope) {   // slope in [0, 1]: max(x, slope * x)
    const F2 a2 = f2_pack(slope, slope);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        float x0, x1, m0, m1;
        f2_unpack(y[q], x0, x1); f2_unpack(f2_mul(y[q], a2), m0, m1);
        y[q] = f2_pack(fmaxf(x0, m0), fmaxf(x1, m1));
    }
}
template <int kAct>
__device__ __forceinline__ void activate_pairs(F2 (&y)[8], int act, float param) {
    if constexpr (kAct == MSNH_ACT_MISH) mish_pairs(y);
    else if constexpr (kAct == MSNH_ACT_LEAKY) leaky_pairs(y, param);
    else {
        if (act == MSNH_ACT_NONE) return;
        float f[16];
#pragma unroll
        for (int q = 0; q < 8; ++q) f2_unpack(y[q], f[2 * q], f[2 * q + 1]);
        activate16(f, act, param);
#pragma unroll
        for (int q = 0; q < 8; ++q) y[q] = f2_pack(f[2 * q], f[2 * q + 1]);
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel. Persistent: CTA b processes tiles b, b+grid, b+2*grid, ... (tile = m_tile * tiles_n
// + n_tile, so CTAs running together share weight tiles and neighbouring pixel tiles in L2).
// Dynamic shared memory: [stages x A tile][stages x B tile][2 output staging slabs] (1024-byte
// aligned), then barriers.
// The accumulators form a ring of 2-8 TMEM stages, so the MMA warp runs several tiles ahead of the
// drain. The two epilogue groups (4 warps each) either split the store slabs of every tile between
// them (kSplit: a tile has at least two slabs, so its drain latency halves) or take alternate tiles.
// ---------------------------------------------------------------------------------------------
// kPair: the kernel runs as clusters of two CTAs that share tiles of 256 pixels x bn channels through
// cta_group::2 MMAs: each CTA stages its own 128 pixels of A and its half of the weight tile (so the
// shared-memory traffic per FLOP halves), the even CTA issues the MMAs for both, and each CTA drains the
// 128 accumulator rows that live in its own TMEM.
// kStreamK: instead of whole tiles, every CTA takes an equal share of the (tile, k-block) sequence, so no SM
// idles in a last partial wave. A CTA whose share ends inside a tile writes that tile's partial sums (raw
// fp32 accumulators) to its slot in global memory and raises its flag; the CTA that owns the tile's last
// k-block adds the slots of its predecessors before the usual epilogue. Each CTA handles the segment it
// hands over first and the segment it has to complete last, so nobody waits on a CTA that is itself waiting.
// kAct: MSNH_ACT_MISH / MSNH_ACT_LEAKY (slope in [0, 1]) compile the first activation into the epilogue loops, kActGeneric
// switches at run time. kTrace: the instantiation that records clock stamps (plans made with MSNH_PLAN_TRACE); the
// production instantiations carry none of that code.
template <typename T, int kMult, bool kSplit, bool kPair, bool kStreamK, int kAct = kActGeneric, bool kTrace = false>   // kMult: 128-pixel sub-tiles per tile (1, 2, 3, 4)
__global__ void __launch_bounds__(kUmmaThreads, 1)
conv_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_c2, const ConvUmmaParams p) {
    constexpr bool kTf32 = sizeof(T) == 4;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment of the operand stages (required by the 128-byte swizzle atoms).
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    constexpr int m_mult = kMult;
    const uint32_t sub_bytes = kUmmaM * p.bk_bytes;          // one 128-pixel sub-tile of A
    const uint32_t a_bytes = m_mult * sub_bytes;
    uint32_t rank = 0;                                     // CTA rank in the pair
    if constexpr (kPair) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const bool lead = rank == 0;
    const int b_rows = kPair ? p.bn / 2 : p.bn;            // weight rows this CTA stages
    const uint32_t b_bytes = b_rows * p.bk_bytes;
    const int first_tile  = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_stride = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const int tile_rows   = kPair ? 2 * kUmmaM : kUmmaM * kMult;
    const uint32_t a_base = smem_base;
    const uint32_t b_base = a_base + p.num_stages * a_bytes;
    const uint32_t stage_c_base = (b_base + p.num_stages * b_bytes + 1023u) & ~1023u;   // two output staging slabs
    const uint32_t bar_base = stage_c_base + 4 * kStageCBytes;
    auto full_bar      = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar     = [&](int s) { return bar_base + 8u * (kUmmaMaxStages + s); };
    auto acc_full_bar  = [&](int s) { return bar_base + 8u * (2 * kUmmaMaxStages + s); };
    auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * kUmmaMaxStages + kUmmaMaxAccStages + s); };
    const int acc_mask = (1 << p.acc_shift) - 1;
    // per-channel scale and bias of the whole layer, staged once (layers of up to kSbMaxChannels channels)
    const uint32_t sb_base = bar_base + 512;                 // [2][kSbMaxChannels] floats
    const bool sb_staged = p.sb_channels > 0;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int cta_abort_slot;
    volatile int *cta_abort = &cta_abort_slot;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    long long *trace = nullptr;
    if constexpr (kTrace) {
        trace = p.trace ? p.trace + static_cast<size_t>(blockIdx.x) * kTraceSlots : nullptr;
        if (trace && threadIdx.x == 0) { trace[0] = clock64(); long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); trace[3] = g; }
    }
    const int num_tiles   = p.tiles_m * p.tiles_n;
    const int num_k_iters = p.taps * p.chunks_per_tap;
    // This CTA's work: segments (tile, k-blocks [k0, k1)). Regular kernels: whole tiles first_tile, +stride, ...
    long long sk_u0 = 0, sk_u1 = 0;
    int sk_tile_first = 0, sk_tile_last = 0, nseg;
    if constexpr (kStreamK) {
        const long long units = static_cast<long long>(num_tiles) * num_k_iters;
        sk_u0 = units * blockIdx.x / gridDim.x; sk_u1 = units * (blockIdx.x + 1) / gridDim.x;
        sk_tile_first = static_cast<int>(sk_u0 / num_k_iters); sk_tile_last = static_cast<int>((sk_u1 - 1) / num_k_iters);
        nseg = sk_u1 > sk_u0 ? sk_tile_last - sk_tile_first + 1 : 0;
    } else {
        nseg = first_tile < num_tiles ? (num_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    }
    // order of a stream-K CTA: the segment of its last tile (possibly handed over) first, the segment of
    // its first tile (possibly completing someone else's) last
    auto segment = [&](int i, int &tile, int &k0, int &k1) {
        if constexpr (kStreamK) {
            tile = i == 0 ? sk_tile_last : (i == nseg - 1 ? sk_tile_first : sk_tile_first + i);
            const long long base = static_cast<long long>(tile) * num_k_iters;
            k0 = static_cast<int>(max(sk_u0, base) - base);
            k1 = static_cast<int>(min(sk_u1, base + num_k_iters) - base);
        } else {
            tile = first_tile + i * tile_stride; k0 = 0; k1 = num_k_iters;
        }
    };

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
        if (p.split_n != 0x7fffffff) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c2) : "memory");
        cta_abort_slot = 0;
        for (int s = 0; s < p.num_stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        // arrivals that free an accumulator: the team epilogue's warps (pair / stream-K kernels), or one per warp and
        // store unit of a tile (plain kernels: four warps x sub-tiles x slabs)
        const int units = kMult * ((p.bn * static_cast<int>(sizeof(T)) + p.out_chunk_bytes - 1) / p.out_chunk_bytes);
        const uint32_t acc_arrivals = (kPair || kStreamK) ? (kSplit ? 16u : 8u) * (kPair ? 2u : 1u) : 4u * static_cast<uint32_t>(units);
        for (int s = 0; s <= acc_mask; ++s) { mbar_init(acc_full_bar(s), 1); mbar_init(acc_empty_bar(s), acc_arrivals); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (sb_staged && threadIdx.x >= 64) {   // constants: no need to wait for the previous kernel
        const int t = threadIdx.x - 64;      // 256 float4 of scale, then 256 of bias
        const float *src = (t < 256 ? p.scale : p.bias) + 4 * (t & 255);
        if (4 * (t & 255) < p.sb_channels) {
            const float4 q = __ldg(reinterpret_cast<const float4 *>(src));
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(sb_base + 16u * t), "f"(q.x), "f"(q.y), "f"(q.z), "f"(q.w) : "memory");
        }
    }
    if (warp == 1) {  // TMEM allocation (whole warp), address lands in shared memory
        if constexpr (kPair) {   // the same warp of both CTAs allocates the same columns in both TMEMs
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(&tmem_base_slot)), "r"(p.tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(&tmem_base_slot)), "r"(p.tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();   // the peer's barriers exist before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // Programmatic dependent launch: everything up to here overlapped the previous kernel's tail. Only the
    // producer thread waits for that kernel (just before its first activation load); every other role
    // starts from data the producer's loads deliver, so it is ordered behind that wait.

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            // Weights do not depend on the previous kernel: the weight tiles of the first k-blocks are
            // requested before waiting for it, which also takes the tensor-map fetches off the critical path.
            // pair: both CTAs' loads complete on the even CTA's full barrier, which expects the bytes of both
            const uint32_t full0 = kPair ? map_to_cta(full_bar(0), 0) : full_bar(0);
            const uint32_t stage_tx = (a_bytes + b_bytes) * (kPair ? 2u : 1u);
            int pre_b = 0;
            if (nseg > 0) {
                int tile, k0, k1; segment(0, tile, k0, k1);
                pre_b = min(p.num_stages, k1 - k0);
                const int n0 = (tile % p.tiles_n) * p.bn + static_cast<int>(rank) * b_rows;
                int tap = k0 / p.chunks_per_tap, chunk = k0 - tap * p.chunks_per_tap;
                for (int kt = 0; kt < pre_b; ++kt) {
                    if (lead) mbar_expect_tx(full_bar(kt), stage_tx);
                    if constexpr (kPair) tma_load_2d_pair(b_base + kt * b_bytes, &map_b, full0 + 8u * kt, tap * p.cin_pad + chunk * p.bk_elems, n0);
                    else                 tma_load_2d(b_base + kt * b_bytes, &map_b, full_bar(kt), tap * p.cin_pad + chunk * p.bk_elems, n0);
                    if (++chunk == p.chunks_per_tap) { chunk = 0; ++tap; }
                }
            }
            bool waited = false;
            for (int i = 0; i < nseg && ok; ++i) {
                int tile, k0, k1; segment(i, tile, k0, k1);
                const int tm = tile / p.tiles_n, tn = tile % p.tiles_n;
                const int m0 = tm * tile_rows + static_cast<int>(rank) * kUmmaM, n0 = tn * p.bn + static_cast<int>(rank) * b_rows;
                int img = 0, y0 = 0, x0 = 0;
                if (p.a_mode == A_MODE_IM2COL) {
                    img = m0 / (p.oh * p.ow);
                    const int rem = m0 - img * p.oh * p.ow;
                    y0 = rem / p.ow; x0 = rem - y0 * p.ow;
                }
                const int cx = x0 * p.stride_w - p.pad_w, cy = y0 * p.stride_h - p.pad_h;
                // k-blocks in tap-major order; plain counters instead of divisions keep this
                // single-thread issue loop short
                int chunk = 0, r = 0, s = 0;
                if (k0 > 0) {
                    const int tap = k0 / p.chunks_per_tap;
                    chunk = k0 - tap * p.chunks_per_tap; r = tap / p.kw; s = tap - r * p.kw;
                }
                for (int kt = k0; kt < k1; ++kt) {
                    const int kb = (r * p.kw + s) * p.cin_pad;
                    const int c0 = chunk * p.bk_elems;
                    if (pre_b > 0) {
                        --pre_b;                       // stage is fresh, its weight tile is already on the way
                        if (!waited) {
                            waited = true;
                            pdl_wait();
                            if constexpr (kTrace) { if (trace) trace[1] = clock64(); }
                        }
                    } else {
                        ok = mbar_wait(empty_bar(stage), phase ^ 1u, cta_abort, p.err_flag, DEV_ERR_WAIT_EMPTY);
                        if (!ok) break;
                        if (lead) mbar_expect_tx(full_bar(stage), stage_tx);
                        if constexpr (kPair) tma_load_2d_pair(b_base + stage * b_bytes, &map_b, full0 + 8u * stage, kb + c0, n0);
                        else                 tma_load_2d(b_base + stage * b_bytes, &map_b, full_bar(stage), kb + c0, n0);
                    }
                    if constexpr (kPair) {
                        if (p.a_mode == A_MODE_IM2COL)
                            tma_load_im2col_4d_pair(a_base + stage * a_bytes, &map_a, full0 + 8u * stage, c0, cx, cy, img,
                                                    static_cast<uint16_t>(s * p.dil_w), static_cast<uint16_t>(r * p.dil_h));
                        else
                            tma_load_2d_pair(a_base + stage * a_bytes, &map_a, full0 + 8u * stage, c0, m0);
                    } else if (p.a_mode == A_MODE_IM2COL)
                        tma_load_im2col_4d(a_base + stage * a_bytes, &map_a, full_bar(stage), c0, cx, cy, img,
                                           static_cast<uint16_t>(s * p.dil_w), static_cast<uint16_t>(r * p.dil_h));
                    else
                        for (int j = 0; j < m_mult; ++j)
                            tma_load_2d(a_base + stage * a_bytes + j * sub_bytes, &map_a, full_bar(stage), c0, m0 + j * kUmmaM);
                    if constexpr (kTrace) { if (trace && i == p.trace_tile && kt - k0 < 16) trace[8 + kt - k0] = clock64(); }
                    if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
                    if (++chunk == p.chunks_per_tap) { chunk = 0; if (++s == p.kw) { s = 0; ++r; } }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0 && lead) {   // pair: the even CTA issues for both
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            const int mmas_per_block = p.bk_bytes / 32;   // each MMA consumes 32 bytes of K per row
            for (int tl = 0; tl < nseg && ok; ++tl) {     // tl: segments this CTA has started
                int tile, k0, k1; segment(tl, tile, k0, k1);
                const int seg_k = k1 - k0;
                const int acc = tl & acc_mask;
                const uint32_t acc_phase = static_cast<uint32_t>(tl >> p.acc_shift) & 1u;
                ok = mbar_wait<true>(acc_empty_bar(acc), acc_phase ^ 1u, cta_abort, p.err_flag, DEV_ERR_WAIT_ACC_EMPTY);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * m_mult * p.bn);
                for (int kt = 0; kt < seg_k; ++kt) {
                    ok = mbar_wait(full_bar(stage), phase, cta_abort, p.err_flag, DEV_ERR_WAIT_FULL);
                    if (!ok) break;
                    if constexpr (kTrace) { if (trace && tl == p.trace_tile && kt < 16) trace[24 + kt] = clock64(); }
                    tcgen05_fence_after();
                    const uint64_t db = make_smem_desc(b_base + stage * b_bytes, p.bk_bytes);
                    const uint64_t da0 = make_smem_desc(a_base + stage * a_bytes, p.bk_bytes);
                    const uint64_t da_step = static_cast<uint64_t>(sub_bytes >> 4);   // next sub-tile of A, in descriptor units
                    // consecutive MMAs go to different accumulators (the sub-tiles share the weight tile), so an
                    // MMA never waits for the one before it to write the accumulator back
                    for (int k = 0; k < mmas_per_block; ++k) {
                        for (int j = 0; j < m_mult; ++j) {
                            // advancing K inside the swizzle span = advancing the start address
                            if constexpr (kPair)
                                tcgen05_mma_pair<kTf32>(tmem_d, da0 + static_cast<uint64_t>(2 * k), db + static_cast<uint64_t>(2 * k),
                                                        p.idesc, (kt | k) != 0 ? 1u : 0u);
                            else
                                tcgen05_mma<kTf32>(tmem_d + static_cast<uint32_t>(j * p.bn), da0 + j * da_step + static_cast<uint64_t>(2 * k),
                                                   db + static_cast<uint64_t>(2 * k), p.idesc, (kt | k) != 0 ? 1u : 0u);
                        }
                    }
                    if constexpr (kPair) tcgen05_commit_pair(empty_bar(stage));   // frees the stage in both CTAs
                    else                 tcgen05_commit(empty_bar(stage));        // frees the stage when these MMAs retire
                    if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if constexpr (kPair) tcgen05_commit_pair(acc_full_bar(acc));   // accumulator complete, in both CTAs
                else                 tcgen05_commit(acc_full_bar(acc));
            }
        }
    } else if constexpr (!kPair && !kStreamK) {
        // ------------------------------ epilogue (16 warps), plain kernels ------------------------
        // Warp w may read TMEM lanes [32*(w%4), 32*(w%4)+32): one output pixel (row) per thread. The warps form four
        // groups of four (one warp per lane quarter). The store units of the CTA's tiles - (tile, 128-pixel sub-tile,
        // slab of up to 128 bytes of channels), in that order - go round the groups; a warp handles its 32 rows of a
        // unit alone: TMEM -> registers -> scale/bias/activation(/residual) -> its own swizzled staging tile (32 rows)
        // -> its own TMA store (which also clips rows past the last pixel and channels past Cout). No barrier between
        // warps: a warp that waits (for the accumulator, for an SFU result, for its staging tile) holds nobody else up.
        const int e = warp - 2;
        const int grp = e >> 2;
        const int lane_base = (warp & 3) * 32;
        const T *res = static_cast<const T *>(p.res);
        constexpr int kVec = Elem<T>::kVec;
        const int cols_per_store = p.out_chunk_bytes / static_cast<int>(sizeof(T));
        const int cols_shift = 31 - __clz(cols_per_store);                 // a power of two
        const int swz_shift = p.out_chunk_bytes == 128 ? 0 : (p.out_chunk_bytes == 64 ? 1 : 2);
        const int swz_mask  = p.out_chunk_bytes == 128 ? 7 : (p.out_chunk_bytes == 64 ? 3 : 1);
        const uint32_t row_swz = static_cast<uint32_t>((lane >> swz_shift) & swz_mask);
        const uint32_t buf = stage_c_base + static_cast<uint32_t>(e) * 4096u;      // this warp's staging tile: 32 rows x up to 128 bytes
        const uint32_t row_addr = buf + static_cast<uint32_t>(lane * p.out_chunk_bytes);
        const int slabs_max = (p.bn + cols_per_store - 1) >> cols_shift;
        const int units_per_tile = kMult * slabs_max;
        const int total_units = nseg * units_per_tile;
        bool ok = true, store_pending = false;
        int tl = 0, item = grp;                      // unit u = tl * units_per_tile + item; this group takes u = grp, grp + 4, ...
        while (item >= units_per_tile && tl < nseg) { item -= units_per_tile; ++tl; }
        int tl_ready = -1;
        for (int u = grp; ok && u < total_units; u += 4) {
            const int tile = first_tile + tl * tile_stride;
            int tm = tile, tn = 0;
            if (p.tiles_n > 1) { tm = tile / p.tiles_n; tn = tile - tm * p.tiles_n; }
            const int n0 = tn * p.bn;
            const int acc = tl & acc_mask;
            if (tl != tl_ready) {                    // first unit of this tile for this warp: its accumulator has to be complete
                const uint32_t acc_phase = static_cast<uint32_t>(tl >> p.acc_shift) & 1u;
                ok = mbar_wait<true>(acc_full_bar(acc), acc_phase, cta_abort, p.err_flag, DEV_ERR_WAIT_ACC_FULL);
                if (!ok) break;
                tcgen05_fence_after();
                tl_ready = tl;
                if constexpr (kTrace) { if (trace && e == 0 && lane == 0 && tl == 0) trace[40] = clock64(); }
            }
            int sub = 0, slab = item;
            if (kMult > 1) { while (slab >= slabs_max) { slab -= slabs_max; ++sub; } }
            const int slabs = (min(p.bn, p.cout - n0) + cols_per_store - 1) >> cols_shift;   // slabs this tile really has
            const int c0 = slab << cols_shift;
            const int mw = tm * tile_rows + sub * kUmmaM + lane_base;      // this warp's first pixel of the unit
            if (slab < slabs && mw < p.m_total) {                          // (otherwise nothing to compute, only the release below)
                const int m = mw + lane;
                const bool row_ok = m < p.m_total;
                const uint32_t acc_col = static_cast<uint32_t>((acc * kMult + sub) * p.bn);
                // the staging tile is free once the previous store of this warp has read it
                if (store_pending) {
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    __syncwarp();
                }
                for (int l0 = 0; l0 < cols_per_store; l0 += 16) {
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(tmem_base + (static_cast<uint32_t>(lane_base) << 16) + acc_col + static_cast<uint32_t>(c0 + l0), v);
                    tmem_ld_wait();
                    const int cbase = n0 + c0 + l0;          // the scale / bias arrays are padded past the last channel tile
                    F2 y[8];
                    if (sb_staged) {
                        const uint32_t sa = sb_base + 4u * static_cast<uint32_t>(cbase);
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            F2 s01, s23, b01, b23;
                            asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(s01.v), "=l"(s23.v) : "r"(sa + 4u * j));
                            asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(b01.v), "=l"(b23.v) : "r"(sa + 4u * kSbMaxChannels + 4u * j));
                            y[j / 2]     = f2_fma(f2_pack(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), s01, b01);
                            y[j / 2 + 1] = f2_fma(f2_pack(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])), s23, b23);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            const float4 sc = __ldg(reinterpret_cast<const float4 *>(p.scale + cbase + j));
                            const float4 bi = __ldg(reinterpret_cast<const float4 *>(p.bias + cbase + j));
                            y[j / 2]     = f2_fma(f2_pack(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), f2_pack(sc.x, sc.y), f2_pack(bi.x, bi.y));
                            y[j / 2 + 1] = f2_fma(f2_pack(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])), f2_pack(sc.z, sc.w), f2_pack(bi.z, bi.w));
                        }
                    }
                    activate_pairs<kAct>(y, p.act1, p.act1_param);
                    if (res && row_ok) {
                        const T *rrow = res + static_cast<size_t>(m) * p.ldc_res + cbase;
#pragma unroll
                        for (int j = 0; j < 16; j += kVec) {
                            if (cbase + j < p.cout) {
                                float rr[kVec];
                                ld_vec(rrow + j, rr);
#pragma unroll
                                for (int q = 0; q < kVec; q += 2)
                                    y[(j + q) / 2] = f2_add(y[(j + q) / 2], f2_pack(rr[q], rr[q + 1]));
                            }
                        }
                        activate_pairs<kActGeneric>(y, p.act2, p.act2_param);
                    }
                    if (kTf32 && p.round_tf32) {
#pragma unroll
                        for (int q = 0; q < 8; ++q) { float a, b; f2_unpack(y[q], a, b); y[q] = f2_pack(round_tf32(a), round_tf32(b)); }
                    }
                    // this thread's 16 columns of the slab, 16 bytes at a time, XOR-swizzled like the TMA map
                    const uint32_t piece0 = static_cast<uint32_t>(l0 / kVec);
#pragma unroll
                    for (int q = 0; q < 16 / kVec; ++q) {
                        const uint32_t addr = row_addr + (((piece0 + q) ^ row_swz) << 4);
                        if constexpr (sizeof(T) == 2) {
                            uint32_t h[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                float a, b; f2_unpack(y[4 * q + k], a, b);
                                asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(h[k]) : "f"(b), "f"(a));
                            }
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
                        } else {
                            asm volatile("st.shared.v2.b64 [%0], {%1, %2};" ::"r"(addr), "l"(y[2 * q].v), "l"(y[2 * q + 1].v) : "memory");
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // staging writes -> visible to the TMA engine
                __syncwarp();
                if (lane == 0) {
                    const bool second = n0 + c0 >= p.split_n;          // slab of the second of two merged convs
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                 ::"l"(second ? &map_c2 : &map_c), "r"(buf), "r"(second ? n0 + c0 - p.split_n : n0 + c0), "r"(mw) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                store_pending = true;
            }
            // this warp's TMEM reads of the unit are done: one of the arrivals that hand the accumulator back to the MMA warp
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
            if constexpr (kTrace) { if (trace && e == 0 && lane == 0) { if (u == 0) trace[41] = clock64(); trace[42] += 1; } }
            item += 4;
            while (item >= units_per_tile) { item -= units_per_tile; ++tl; }
        }
        // the staging tile must outlive the store's reads of it; the writes themselves are complete when the grid is
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    } else {
        // ------------------------------ epilogue (16 warps), CTA-pair and stream-K kernels ------------------------
        // Warp w may read TMEM lanes [32*(w%4), 32*(w%4)+32): one output pixel (row) per thread.
        // Two teams of 8 warps; a team drains one store slab (a 128/64/32-byte wide column slab of a
        // 128-pixel sub-tile) at a time: its two halves of 4 warps take alternate 16-column chunks,
        // TMEM -> registers -> scale/bias/activation(/residual) -> swizzled staging tile in shared memory,
        // then one TMA store, which also clips rows past the last pixel and channels past Cout. Two
        // staging buffers per team alternate so the store of one slab overlaps the math of the next.
        const int e = warp - 2;
        const int lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int team = (e >> 2) & 1;
        const int half = e >> 3;
        const bool leader = e == team * 4 && lane == 0;
        const uint32_t team_stage_c = stage_c_base + static_cast<uint32_t>(team) * 2u * kStageCBytes;
        bool ok = true;
        const T *res = static_cast<const T *>(p.res);
        constexpr int kVec = Elem<T>::kVec;
        const int cols_per_store = p.out_chunk_bytes / static_cast<int>(sizeof(T));
        const int cols_shift = 31 - __clz(cols_per_store);                 // a power of two
        const int swz_shift = p.out_chunk_bytes == 128 ? 0 : (p.out_chunk_bytes == 64 ? 1 : 2);
        const int swz_mask  = p.out_chunk_bytes == 128 ? 7 : (p.out_chunk_bytes == 64 ? 3 : 1);
        const uint32_t row_smem = static_cast<uint32_t>(row * p.out_chunk_bytes);
        const uint32_t row_swz = static_cast<uint32_t>((row >> swz_shift) & swz_mask);
        uint32_t store_count = 0;
        if constexpr (kTrace) { if (team == 1) trace = nullptr; }
        // kSplit: every tile, items (sub-tile, slab) team, team+2, ...; otherwise tiles team, team+2, ... whole
        const int tl_step = kSplit ? 1 : 2;
        for (int tl = kSplit ? 0 : team; ok && tl < nseg; tl += tl_step) {
            int tile, seg_k0, seg_k1; segment(tl, tile, seg_k0, seg_k1);
            // stream-K: a segment that stops short of the tile's last k-block hands its partial sums over
            // (sk_export); one that starts after the first k-block completes its predecessors' (CTAs
            // sk_first .. this - 1)
            const bool sk_export = kStreamK && seg_k1 < num_k_iters;
            const bool sk_import = kStreamK && !sk_export && seg_k0 > 0;
            int sk_first = 0;
            if constexpr (kStreamK) {
                if (sk_import) {
                    const long long units = static_cast<long long>(num_tiles) * num_k_iters;
                    const long long u = static_cast<long long>(tile) * num_k_iters;          // the tile's first unit
                    sk_first = static_cast<int>(u * gridDim.x / units);
                    while (units * (sk_first + 1) / gridDim.x <= u) ++sk_first;              // owner: bound(j) <= u < bound(j+1)
                    while (units * sk_first / gridDim.x > u) --sk_first;
                    // wait (bounded) until every predecessor has filled its slot
                    if (lane == 0) {
                        for (int j = sk_first; j < static_cast<int>(blockIdx.x) && ok; ++j) {
                            const long long t0 = clock64();
                            while (*reinterpret_cast<volatile int *>(p.sk_flags + j) == 0) {
                                if (*cta_abort || clock64() - t0 > kWaitCycles) { *cta_abort = 1; atomicCAS(p.err_flag, 0, DEV_ERR_WAIT_ACC_FULL); ok = false; break; }
                            }
                        }
                        __threadfence();
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                }
            }
            // (all 512 threads run this bookkeeping, so it avoids integer divisions)
            int tm = tile, tn = 0;
            if (p.tiles_n > 1) { tm = tile / p.tiles_n; tn = tile - tm * p.tiles_n; }
            const int n0 = tn * p.bn;
            const int acc = tl & acc_mask;
            const uint32_t acc_phase = static_cast<uint32_t>(tl >> p.acc_shift) & 1u;
            { const bool got = mbar_wait<true>(acc_full_bar(acc), acc_phase, cta_abort, p.err_flag, DEV_ERR_WAIT_ACC_FULL); ok = ok && got; }
            {   // one decision for the eight warps of this team (they meet at the team's named barrier below);
                // stream-K kernels decide for both teams at once, because those also meet at barrier 3
                uint32_t all_ok;
                if constexpr (kStreamK)
                    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 3, 512, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(all_ok) : "r"(static_cast<uint32_t>(ok)) : "memory");
                else
                    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, %2, 256, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(all_ok) : "r"(static_cast<uint32_t>(ok)), "r"(1 + team) : "memory");
                ok = all_ok != 0;
            }
            if (!ok) break;
            if constexpr (kTrace) { if (trace && tl == 0 && leader) trace[40] = clock64(); }
            tcgen05_fence_after();
            const int slabs = (min(p.bn, p.cout - n0) + cols_per_store - 1) >> cols_shift;   // store slabs per sub-tile
            for (int item = kSplit ? team : 0; item < kMult * slabs; item += kSplit ? 2 : 1) {
                int sub = 0;
                if (kMult > 1) { while (item >= (sub + 1) * slabs) ++sub; }
                const int c0 = (item - sub * slabs) << cols_shift;
                const int m0 = tm * tile_rows + (kPair ? static_cast<int>(rank) : sub) * kUmmaM, m = m0 + row;
                if (m0 >= p.m_total) break;                        // sub-tile entirely past the last pixel
                const bool row_ok = m < p.m_total;
                const uint32_t acc_col = static_cast<uint32_t>((acc * kMult + sub) * p.bn);
                // stream-K slot layout: [16-column chunk][4-column group][row][4 floats], so that the 32 rows of a
                // warp make one contiguous 512-byte access per instruction
                constexpr int sk_rows = kMult * kUmmaM;
                const int sk_row = sub * kUmmaM + row;
                if constexpr (kStreamK) {
                    if (sk_export) {   // raw accumulators -> this CTA's slot; no activation, no output store
                        float *slot = p.sk_ws + static_cast<size_t>(blockIdx.x) * (static_cast<size_t>(sk_rows) * p.bn);
                        for (int l0 = half * 16; l0 < cols_per_store; l0 += 32) {
                            uint32_t v[16];
                            tmem_ld_32x32b_x16(tmem_base + (static_cast<uint32_t>(lane_base) << 16) + acc_col + static_cast<uint32_t>(c0 + l0), v);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 16; j += 4)
                                *reinterpret_cast<uint4 *>(slot + (static_cast<size_t>(((c0 + l0) >> 2) + (j >> 2)) * sk_rows + sk_row) * 4) =
                                    make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        }
                        continue;
                    }
                }
                // Staging buffers alternate. The buffer written now was last read by the store issued two
                // slabs ago, and the leader confirmed that store's reads before the previous barrier.
                const uint32_t buf = team_stage_c + (store_count & 1u) * kStageCBytes;
                if constexpr (kTrace) { if (trace && leader && store_count < 5) trace[43 + 4 * store_count] = clock64(); }
                // one 16-column chunk of this thread's row: scale / bias, activation, residual, conversion, staging store
                auto finish_chunk = [&](const int l0, const uint32_t (&v)[16]) {
                    const int cbase = n0 + c0 + l0;          // the scale / bias arrays are padded past the last channel tile
                    // y = acc * scale + bias on packed pairs; the tables come from shared memory (one 16-byte load per
                    // four channels, the same address for the whole warp) or, for very wide layers, through L1
                    F2 y[8];
                    if (sb_staged) {
                        const uint32_t sa = sb_base + 4u * static_cast<uint32_t>(cbase);
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            F2 s01, s23, b01, b23;
                            asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(s01.v), "=l"(s23.v) : "r"(sa + 4u * j));
                            asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(b01.v), "=l"(b23.v) : "r"(sa + 4u * kSbMaxChannels + 4u * j));
                            y[j / 2]     = f2_fma(f2_pack(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), s01, b01);
                            y[j / 2 + 1] = f2_fma(f2_pack(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])), s23, b23);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            const float4 sc = __ldg(reinterpret_cast<const float4 *>(p.scale + cbase + j));
                            const float4 bi = __ldg(reinterpret_cast<const float4 *>(p.bias + cbase + j));
                            y[j / 2]     = f2_fma(f2_pack(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), f2_pack(sc.x, sc.y), f2_pack(bi.x, bi.y));
                            y[j / 2 + 1] = f2_fma(f2_pack(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])), f2_pack(sc.z, sc.w), f2_pack(bi.z, bi.w));
                        }
                    }
                    activate_pairs<kAct>(y, p.act1, p.act1_param);
                    if (res && row_ok) {
                        const T *rrow = res + static_cast<size_t>(m) * p.ldc_res + cbase;
#pragma unroll
                        for (int j = 0; j < 16; j += kVec) {
                            if (cbase + j < p.cout) {
                                float rr[kVec];
                                ld_vec(rrow + j, rr);
#pragma unroll
                                for (int q = 0; q < kVec; q += 2)
                                    y[(j + q) / 2] = f2_add(y[(j + q) / 2], f2_pack(rr[q], rr[q + 1]));
                            }
                        }
                        activate_pairs<kActGeneric>(y, p.act2, p.act2_param);
                    }
                    if (kTf32 && p.round_tf32) {
#pragma unroll
                        for (int q = 0; q < 8; ++q) { float a, b; f2_unpack(y[q], a, b); y[q] = f2_pack(round_tf32(a), round_tf32(b)); }
                    }
                    // this thread's 16 columns of the slab, 16 bytes at a time, XOR-swizzled like the TMA map
                    const uint32_t row_addr = buf + row_smem;
                    const uint32_t piece0 = static_cast<uint32_t>(l0 / kVec);
#pragma unroll
                    for (int q = 0; q < 16 / kVec; ++q) {
                        const uint32_t addr = row_addr + (((piece0 + q) ^ row_swz) << 4);
                        if constexpr (sizeof(T) == 2) {
                            uint32_t h[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                float a, b; f2_unpack(y[4 * q + k], a, b);
                                asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(h[k]) : "f"(b), "f"(a));
                            }
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
                        } else {
                            asm volatile("st.shared.v2.b64 [%0], {%1, %2};" ::"r"(addr), "l"(y[2 * q].v), "l"(y[2 * q + 1].v) : "memory");
                        }
                    }
                };
                for (int l0 = half * 16; l0 < cols_per_store; l0 += 32) {
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(tmem_base + (static_cast<uint32_t>(lane_base) << 16) +
                                       acc_col + static_cast<uint32_t>(c0 + l0), v);
                    tmem_ld_wait();
                    if constexpr (kStreamK) {
                        if (sk_import) {   // add the predecessors' partial sums, in CTA order (deterministic)
                            for (int c = sk_first; c < static_cast<int>(blockIdx.x); ++c) {
                                const float *slot = p.sk_ws + static_cast<size_t>(c) * (static_cast<size_t>(sk_rows) * p.bn);
#pragma unroll
                                for (int j = 0; j < 16; j += 4) {
                                    // L2 read: the slot was written by another SM
                                    const float4 q = __ldcg(reinterpret_cast<const float4 *>(slot + (static_cast<size_t>(((c0 + l0) >> 2) + (j >> 2)) * sk_rows + sk_row) * 4));
                                    v[j]     = __float_as_uint(__uint_as_float(v[j]) + q.x);     v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + q.y);
                                    v[j + 2] = __float_as_uint(__uint_as_float(v[j + 2]) + q.z); v[j + 3] = __float_as_uint(__uint_as_float(v[j + 3]) + q.w);
                                }
                            }
                        }
                    }
                    finish_chunk(l0, v);
                }
                if constexpr (kTrace) { if (trace && leader && store_count < 5) trace[45 + 4 * store_count] = clock64(); }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // staging writes -> visible to the TMA engine
                // every earlier store of this team has finished reading shared memory (the newest one was
                // issued a whole slab ago), so after this barrier the other buffer may be overwritten
                if (leader) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                asm volatile("bar.sync %0, 256;" ::"r"(1 + team) : "memory");
                if constexpr (kTrace) { if (trace && leader && store_count < 5) trace[46 + 4 * store_count] = clock64(); }
                if (leader) {
                    const bool second = n0 + c0 >= p.split_n;          // slab of the second of two merged convs
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                 ::"l"(second ? &map_c2 : &map_c), "r"(buf), "r"(second ? n0 + c0 - p.split_n : n0 + c0), "r"(m0) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    if constexpr (kTrace) { if (trace && store_count < 5) trace[44 + 4 * store_count] = clock64(); }
                }
                ++store_count;
            }
            if constexpr (kStreamK) {
                if (sk_export || sk_import) {
                    // every epilogue thread's slot writes are visible / slot reads are done before the flag moves
                    __threadfence();
                    asm volatile("bar.sync 3, 512;" ::: "memory");
                    if (e == 0 && lane == 0) {
                        if (sk_export) *reinterpret_cast<volatile int *>(p.sk_flags + blockIdx.x) = 1;
                        else for (int c = sk_first; c < static_cast<int>(blockIdx.x); ++c) *reinterpret_cast<volatile int *>(p.sk_flags + c) = 0;
                    }
                }
            }
            // all TMEM reads of this accumulator are done: hand it back to the MMA warp
            tcgen05_fence_before();
            __syncwarp();
            if constexpr (kTrace) { if (trace && leader) { if (tl == 0) trace[41] = clock64(); trace[42] += 1; } }
            if (lane == 0) {
                if constexpr (kPair) mbar_arrive_cluster(map_to_cta(acc_empty_bar(acc), 0));   // the even CTA's MMA thread waits on it
                else                 mbar_arrive(acc_empty_bar(acc));
            }
        }
        // the staging slabs must outlive the stores' reads of them; the writes themselves are complete when the grid is
        if (leader) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }

    // teardown: everybody is past its last TMEM access (or gave up) before the columns are freed
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();   // nothing of the peer targets this CTA's barriers or TMEM any more
    if constexpr (kTrace) { if (trace && threadIdx.x == 0) { trace[2] = clock64(); long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); trace[4] = g; } }
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after();
        if constexpr (kPair) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
        else                 asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
}

}  // namespace msnh
