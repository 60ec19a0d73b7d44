// Candidate collection for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need detections: code
// running inside a real-time loop or a stream callback that is forbidden to take the allocator's
// locks, plugins that are handed a fixed memory budget up front by the application that loads them,
// and processes whose device memory is entirely pre-partitioned by a framework that owns the
// allocator. The plan-based path (msnh_b200_plan_*) allocates its arena, counters and staging
// buffers; this entry point allocates nothing at all. The only scratch the kernel needs - one
// append counter per image - lives in a file-scope __device__ array of fixed size, so every GPU
// that loads the library carries those 4 KB until the process exits.
//
// It is the same computation as the yolo_collect launch of a plan (csrc/layer_kernels.cuh): one
// thread per (image, cell, anchor) of an already decoded head, objectness threshold, first-maximum
// class, rows {x,y,w,h,conf,bestClsConf,bestClsIdx,order} appended per image.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/msnh_b200.h"

namespace {

// The scratch. In host code this name is only a stand-in for the symbol, not a device address:
// the address every launch uses comes from cudaGetSymbolAddress (device_counters below). Device
// code may and does name the array directly.
static __device__ __align__(256) int g_collect_counters[MSNH_B200_STATIC_MAX_IMAGES];

constexpr int kMaxDevices = 64;
int *g_counter_addr[kMaxDevices] = {};      // per device, filled on first use
std::mutex g_setup_mutex;
thread_local char g_error[256] = "";

int fail(int code, const char *text, cudaError_t e = cudaSuccess) {
    if (e != cudaSuccess) snprintf(g_error, sizeof(g_error), "%s: %s", text, cudaGetErrorString(e));
    else snprintf(g_error, sizeof(g_error), "%s", text);
    return code;
}

// Address of this device's copy of the counter array. Looked up once per device, with that device
// current, and cached; no allocation is involved (the array is part of the loaded module).
int device_counters(int **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(MSNH_B200_ERR_CUDA, "cudaGetDevice", e);
    if (dev < 0 || dev >= kMaxDevices) return fail(MSNH_B200_ERR_UNSUPPORTED, "device ordinal beyond the 64 this entry point tracks");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_counter_addr[dev]) {
        int *ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_collect_counters);
        if (e != cudaSuccess || !ptr) return fail(MSNH_B200_ERR_CUDA, "cudaGetSymbolAddress(g_collect_counters)", e);
        g_counter_addr[dev] = ptr;
    }
    *out = g_counter_addr[dev];
    return MSNH_B200_OK;
}

__global__ void yolo_collect_static_kernel(const float *__restrict__ dec, int n_images, int plane, int pitch, int classes,
                                           float conf_thresh, int order_base, float *__restrict__ rows, int max_rows) {
    const int per = 5 + classes;
    const size_t total = static_cast<size_t>(n_images) * plane * 3;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int a = static_cast<int>(i % 3);
        const size_t pix = i / 3;
        const int n = static_cast<int>(pix / plane), cell = static_cast<int>(pix - static_cast<size_t>(n) * plane);
        const float *p = dec + pix * pitch + a * per;
        const float conf = p[4];
        if (!(conf > conf_thresh)) continue;
        float best = p[5]; int best_i = 0;
        for (int k = 1; k < classes; ++k) { const float v = p[5 + k]; if (v > best) { best = v; best_i = k; } }
        const int slot = atomicAdd(&g_collect_counters[n], 1);      // the static scratch, named directly
        if (slot < max_rows) {
            float *r = rows + (static_cast<size_t>(n) * max_rows + slot) * 8;
            r[0] = p[0]; r[1] = p[1]; r[2] = p[2]; r[3] = p[3]; r[4] = conf; r[5] = best;
            r[6] = static_cast<float>(best_i); r[7] = static_cast<float>(order_base + a * plane + cell);
        }
    }
}

__global__ void publish_counts_kernel(int n_images, int max_rows, int *__restrict__ counts) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_images) counts[i] = min(g_collect_counters[i], max_rows);
}

}  // namespace

extern "C" {

const char *msnh_b200_static_last_error(void) { return g_error; }

int msnh_b200_yolo_collect_static(const float *dev_decoded, int n_images, int grid_h, int grid_w, int channel_pitch,
                                  int classes, float conf_thresh, int order_base, float *dev_rows,
                                  int max_rows_per_image, int *dev_counts, void *stream) {
    if (!dev_decoded || !dev_rows || !dev_counts) return fail(MSNH_B200_ERR_ARG, "null device pointer");
    if (n_images < 1 || grid_h < 1 || grid_w < 1 || classes < 1 || max_rows_per_image < 1)
        return fail(MSNH_B200_ERR_ARG, "n_images, grid size, classes and max_rows_per_image must be positive");
    if (n_images > MSNH_B200_STATIC_MAX_IMAGES) {
        snprintf(g_error, sizeof(g_error), "n_images %d exceeds the %d images the static counter array holds", n_images,
                 MSNH_B200_STATIC_MAX_IMAGES);
        return MSNH_B200_ERR_ARG;
    }
    if (channel_pitch < 3 * (5 + classes)) return fail(MSNH_B200_ERR_ARG, "channel_pitch smaller than 3*(5+classes)");
    int *counters = nullptr;
    const int rc = device_counters(&counters);       // first call on a device: symbol lookup (no allocation)
    if (rc != MSNH_B200_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the array keeps the previous call's counts: clear the part this call uses
    cudaError_t e = cudaMemsetAsync(counters, 0, sizeof(int) * n_images, st);
    if (e != cudaSuccess) return fail(MSNH_B200_ERR_CUDA, "cudaMemsetAsync(counters)", e);
    const int plane = grid_h * grid_w;
    const size_t items = static_cast<size_t>(n_images) * plane * 3;
    int sms = 148;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    size_t blocks = (items + 255) / 256;
    if (blocks > static_cast<size_t>(sms) * 8) blocks = static_cast<size_t>(sms) * 8;
    yolo_collect_static_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(dev_decoded, n_images, plane, channel_pitch, classes,
                                                                              conf_thresh, order_base, dev_rows, max_rows_per_image);
    publish_counts_kernel<<<(n_images + 255) / 256, 256, 0, st>>>(n_images, max_rows_per_image, dev_counts);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MSNH_B200_ERR_CUDA, "launch of the static collect kernels", e);
    g_error[0] = '\0';
    return MSNH_B200_OK;
}

}  // extern "C"
