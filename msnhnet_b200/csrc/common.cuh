// Shared device/host helpers of the sm_100a kernels: tensor views, activation math, vector types.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/msnh_b200.h"
#include "kernel_params.h"

namespace msnh {

// Round-to-nearest to the 10-bit tf32 mantissa. The tf32 MMA ignores the low 13 mantissa bits of
// its fp32 operands, i.e. truncates; truncation is biased toward zero and the bias compounds layer
// after layer, so producers round instead.
__device__ __forceinline__ float round_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// Programmatic dependent launch: let the next grid in the stream be scheduled early, then wait until
// every grid this one depends on has completed and its writes are visible. Both are no-ops for a
// grid launched without the attribute. Called first thing by every kernel that reads tensors.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() { pdl_launch_dependents(); pdl_wait(); }

template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int kVec = 4;  // elements per 16-byte vector
    __device__ __forceinline__ static float ld(const float *p) { return *p; }
    __device__ __forceinline__ static void  st(float *p, float v) { *p = v; }
};
template <> struct Elem<__half> {
    static constexpr int kVec = 8;
    __device__ __forceinline__ static float ld(const __half *p) { return __half2float(*p); }
    __device__ __forceinline__ static void  st(__half *p, float v) { *p = __float2half_rn(v); }
};

// 16-byte vector load/store of kVec elements to/from fp32 registers.
__device__ __forceinline__ void ld_vec(const float *p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void st_vec(float *p, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void ld_vec(const __half *p, float (&v)[8]) {
    uint4 t = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void st_vec(__half *p, const float (&v)[8]) {
    uint4 t;
    __half2 *h = reinterpret_cast<__half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = t;
}

// Activation set of the reference (include/Msnhnet/layers/MsnhActivations.h:39-168). The branch is
// uniform across a launch. mish uses tanh(log(1+e^x)) = (e^2x + 2e^x) / (e^2x + 2e^x + 2), which
// is the same function as the reference's x*tanh(softplus(x, 20)) to fp32 rounding.
__device__ __forceinline__ float activate(float x, int act, float param) {
    switch (act) {
        case MSNH_ACT_NONE:     return x;
        case MSNH_ACT_LOGISTIC: return 1.f / (1.f + __expf(-x));
        case MSNH_ACT_LOGGY:    return 2.f / (1.f + __expf(-x)) - 1.f;
        case MSNH_ACT_RELU:     return x > 0.f ? x : 0.f;
        case MSNH_ACT_RELU6:    return fminf(fmaxf(x, 0.f), 6.f);
        case MSNH_ACT_HARD_SWISH: return x * fminf(fmaxf(x + 3.f, 0.f), 6.f) / 6.f;
        case MSNH_ACT_ELU:      return x >= 0.f ? x : (__expf(x) - 1.f);
        case MSNH_ACT_SELU:     return x >= 0.f ? 1.0507f * x : 1.0507f * 1.6732f * (__expf(x) - 1.f);
        case MSNH_ACT_RELIE:    return x > 0.f ? x : 0.01f * x;
        case MSNH_ACT_RAMP:     return (x > 0.f ? x : 0.f) + 0.1f * x;
        case MSNH_ACT_LEAKY:    return x > 0.f ? x : param * x;
        case MSNH_ACT_TANH:     { float e = __expf(2.f * x); return (e - 1.f) / (e + 1.f); }
        case MSNH_ACT_STAIR: {
            int n = static_cast<int>(floorf(x));
            return (n % 2 == 0) ? floorf(x * 0.5f) : (x - n) + floorf(x * 0.5f);
        }
        case MSNH_ACT_HARDTAN:  return fminf(fmaxf(x, -1.f), 1.f);
        case MSNH_ACT_SOFT_PLUS:
            return x > param ? x : (x < -param ? __expf(x) : __logf(__expf(x) + 1.f));
        case MSNH_ACT_PLSE:     return x < -4.f ? 0.01f * (x + 4.f) : (x > 4.f ? 0.01f * (x - 4.f) + 1.f : 0.125f * x + 0.5f);
        case MSNH_ACT_LHTAN:    return x < 0.f ? 0.001f * x : (x > 1.f ? 0.001f * (x - 1.f) + 1.f : x);
        case MSNH_ACT_MISH: {
            if (x > 20.f) return x;                      // softplus(x) = x and tanh(x) = 1 in fp32
            float e = __expf(x);
            float n = e * (e + 2.f);
            return x * (n / (n + 2.f));
        }
        case MSNH_ACT_SWISH:    return x / (1.f + __expf(-x));
        default:                return x;
    }
}

}  // namespace msnh
