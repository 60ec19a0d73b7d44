// Effective SM clock while other kernels run: one warp on its own stream reads the nanosecond timer and its SM's
// cycle counter about once a millisecond. The management library reports the clock the GPU is asked to run at; under
// load the SMs' cycle counters advance more slowly than that, and this is the rate a kernel's cycle counts convert
// with. Measurement aid of the benchmark (the reference's per-layer GPU timers are stubbed out,
// src/layers/MsnhBaseLayer.cpp:300-319); not on the inference path.
#include <cuda_runtime.h>
#include <algorithm>
#include <new>
#include <vector>

#include "../../include/msnh_b200.h"

namespace {

struct ClockProbe {
    int device = 0;
    cudaStream_t stream = nullptr;
    long long *d_samples = nullptr;       // [max_samples][2]: nanosecond timer, SM cycle counter
    int *d_count = nullptr;               // samples written
    volatile int *h_stop = nullptr;       // mapped host flag, read by the kernel between samples
    int *d_stop = nullptr;
    int max_samples = 0;
};

// The loop is bounded by max_samples (about a millisecond each), whatever the flag does.
__global__ void clock_probe_kernel(long long *samples, int *count, const volatile int *stop, int max_samples) {
    if (threadIdx.x != 0) return;
    int n = 0;
    while (n < max_samples) {
        long long g;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
        samples[2 * n] = g;
        samples[2 * n + 1] = clock64();
        ++n;
        *count = n;
        if (*stop) break;
        __nanosleep(1000000u);
    }
}

}  // namespace

extern "C" {

int msnh_b200_clock_probe_start(int device, int max_ms, void **handle) {
    if (!handle || max_ms < 1 || max_ms > 60000) return MSNH_B200_ERR_ARG;
    *handle = nullptr;
    ClockProbe *p = new (std::nothrow) ClockProbe();
    if (!p) return MSNH_B200_ERR_NOMEM;
    p->device = device; p->max_samples = max_ms;
    int prev = 0;
    cudaGetDevice(&prev);
    bool ok = cudaSetDevice(device) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void **>(&p->d_samples), sizeof(long long) * 2 * max_ms) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void **>(&p->d_count), sizeof(int)) == cudaSuccess &&
              cudaMemset(p->d_count, 0, sizeof(int)) == cudaSuccess &&
              cudaHostAlloc(reinterpret_cast<void **>(const_cast<int **>(&p->h_stop)), sizeof(int), cudaHostAllocMapped) == cudaSuccess;
    if (ok) {
        *p->h_stop = 0;
        ok = cudaHostGetDevicePointer(reinterpret_cast<void **>(&p->d_stop), const_cast<int *>(p->h_stop), 0) == cudaSuccess;
    }
    if (ok) {
        clock_probe_kernel<<<1, 32, 0, p->stream>>>(p->d_samples, p->d_count, p->d_stop, p->max_samples);
        ok = cudaGetLastError() == cudaSuccess;
    }
    cudaSetDevice(prev);
    if (!ok) {
        if (p->stream) cudaStreamDestroy(p->stream);
        cudaFree(p->d_samples); cudaFree(p->d_count);
        if (p->h_stop) cudaFreeHost(const_cast<int *>(p->h_stop));
        delete p;
        return MSNH_B200_ERR_CUDA;
    }
    *handle = p;
    return MSNH_B200_OK;
}

int msnh_b200_clock_probe_stop(void *handle, double *mhz_median, double *mhz_min, double *mhz_max, int *samples) {
    ClockProbe *p = static_cast<ClockProbe *>(handle);
    if (!p) return MSNH_B200_ERR_ARG;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(p->device);
    *p->h_stop = 1;
    int rc = cudaStreamSynchronize(p->stream) == cudaSuccess ? MSNH_B200_OK : MSNH_B200_ERR_CUDA;
    int n = 0;
    std::vector<long long> s;
    if (rc == MSNH_B200_OK && cudaMemcpy(&n, p->d_count, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess && n > 1) {
        s.resize(2 * static_cast<size_t>(n));
        if (cudaMemcpy(s.data(), p->d_samples, sizeof(long long) * s.size(), cudaMemcpyDeviceToHost) != cudaSuccess) n = 0;
    }
    std::vector<double> mhz;
    for (int i = 1; i < n; ++i) {
        const double ns = static_cast<double>(s[2 * i] - s[2 * i - 2]);
        if (ns > 0) mhz.push_back(static_cast<double>(s[2 * i + 1] - s[2 * i - 1]) / ns * 1000.0);
    }
    std::sort(mhz.begin(), mhz.end());
    if (mhz_median) *mhz_median = mhz.empty() ? 0.0 : mhz[mhz.size() / 2];
    if (mhz_min) *mhz_min = mhz.empty() ? 0.0 : mhz.front();
    if (mhz_max) *mhz_max = mhz.empty() ? 0.0 : mhz.back();
    if (samples) *samples = static_cast<int>(mhz.size());
    cudaStreamDestroy(p->stream);
    cudaFree(p->d_samples); cudaFree(p->d_count);
    cudaFreeHost(const_cast<int *>(p->h_stop));
    cudaSetDevice(prev);
    delete p;
    return rc;
}

}  // extern "C"
