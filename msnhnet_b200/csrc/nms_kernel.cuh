// Score sort + per-class greedy NMS of one image's detection candidates on the device: what
// YoloOutLayer does on the host after the candidate scan (src/layers/MsnhYoloOutLayer.cpp:167-197 sort by
// conf * bestClsConf, :381-461 nms; IoU with the reference's +1 convention, include/Msnhnet/utils/MsnhTypes.h:123-140).
// One CTA per image. Candidate rows are {x, y, w, h, conf, bestClsConf, bestClsIdx, order} in arbitrary slot
// order (appended through an atomic counter); `order` is the candidate's position in the reference's scan.
//  1. bitonic sort of (score descending, order ascending) keys in shared memory. The reference sorts with an
//     unstable std::sort, so two candidates with bit-identical scores may come out in either order there;
//     here they keep scan order. Everything else is order-exact.
//  2. per class, repeatedly take the box with the highest objectness (first in list order on ties) and drop
//     every remaining box of the class whose IoU with it exceeds the threshold (soft-NMS: whose decayed
//     objectness is <= 0); a class with one box keeps it. All classes advance together, one pick per round.
//     Output: classes in first-seen order of the sorted list, picks in order within a class.
// All arithmetic uses round-to-nearest intrinsics in the host code's order (no FMA contraction), so the
// kept set equals the host result bit for bit.
#pragma once
#include <cfloat>
#include "common.cuh"

namespace msnh {

__device__ __forceinline__ float nms_iou(float ax, float ay, float aw, float ah, float bx, float by, float bw, float bh) {
    const float ax1 = __fsub_rn(ax, __fmul_rn(aw, 0.5f)), ax2 = __fadd_rn(ax, __fmul_rn(aw, 0.5f));
    const float ay1 = __fsub_rn(ay, __fmul_rn(ah, 0.5f)), ay2 = __fadd_rn(ay, __fmul_rn(ah, 0.5f));
    const float bx1 = __fsub_rn(bx, __fmul_rn(bw, 0.5f)), bx2 = __fadd_rn(bx, __fmul_rn(bw, 0.5f));
    const float by1 = __fsub_rn(by, __fmul_rn(bh, 0.5f)), by2 = __fadd_rn(by, __fmul_rn(bh, 0.5f));
    const float ix1 = fmaxf(ax1, bx1), iy1 = fmaxf(ay1, by1), ix2 = fminf(ax2, bx2), iy2 = fminf(ay2, by2);
    const float iw = __fadd_rn(__fsub_rn(ix2, ix1), 1.f), ih = __fadd_rn(__fsub_rn(iy2, iy1), 1.f);
    const float inter = __fmul_rn(iw < 0.f ? 0.f : iw, ih < 0.f ? 0.f : ih);
    const float area_a = __fmul_rn(__fadd_rn(__fsub_rn(ax2, ax1), 1.f), __fadd_rn(__fsub_rn(ay2, ay1), 1.f));
    const float area_b = __fmul_rn(__fadd_rn(__fsub_rn(bx2, bx1), 1.f), __fadd_rn(__fsub_rn(by2, by1), 1.f));
    return __fdiv_rn(inter, __fsub_rn(__fadd_rn(area_a, area_b), inter));
}

// rows: [images][max_rows][8]; counts: candidates per image; out: [images][max_out][8] kept boxes in the
// reference's output order {x, y, w, h, conf, bestClsConf, bestClsIdx, rank in the score-sorted list};
// out_counts[i] = kept boxes, or -1 when the image has more than kNmsMaxCandidates candidates.
__global__ void __launch_bounds__(kNmsThreads)
yolo_nms_kernel(const float *__restrict__ rows, const int *__restrict__ counts, int max_rows, float nms_thresh, int use_soft,
                float sigma, float *__restrict__ out, int max_out, int *__restrict__ out_counts) {
    pdl_prologue();
    extern __shared__ unsigned long long nms_smem[];
    unsigned long long *key = nms_smem;
    float *bx = reinterpret_cast<float *>(key + kNmsMaxCandidates), *by = bx + kNmsMaxCandidates, *bw = by + kNmsMaxCandidates,
          *bh = bw + kNmsMaxCandidates, *conf = bh + kNmsMaxCandidates, *cls_conf = conf + kNmsMaxCandidates;
    short *cls = reinterpret_cast<short *>(cls_conf + kNmsMaxCandidates);
    unsigned char *alive = reinterpret_cast<unsigned char *>(cls + kNmsMaxCandidates);   // 1: of the current class, not yet taken or dropped
    unsigned char *done_cls = alive + kNmsMaxCandidates;                                  // state of a box: taken or not (see below)
    unsigned short *kept_round = reinterpret_cast<unsigned short *>(done_cls + kNmsMaxCandidates);
    unsigned long long *s_best = reinterpret_cast<unsigned long long *>(kept_round + kNmsMaxCandidates);   // [kNmsMaxClasses], 8-byte aligned
    int *s_class_i = reinterpret_cast<int *>(s_best + kNmsMaxClasses);                  // 3 x [kNmsMaxClasses]
    __shared__ int s_kept, s_alive, s_bad;
    const int img = blockIdx.x, tid = threadIdx.x;
    const int n = min(counts[img], max_rows);
    if (n > kNmsMaxCandidates) { if (tid == 0) out_counts[img] = -1; return; }
    const float *r = rows + static_cast<size_t>(img) * max_rows * 8;
    int np2 = 1; while (np2 < n) np2 <<= 1;
    // 1. keys: high word = ~bits(score) (scores are positive, so ascending keys = descending scores), low = order
    for (int i = tid; i < np2; i += kNmsThreads) {
        unsigned long long k = ~0ull;
        if (i < n) {
            const float score = __fmul_rn(r[i * 8 + 4], r[i * 8 + 5]);
            k = (static_cast<unsigned long long>(~__float_as_uint(score)) << 32) | static_cast<unsigned>(__float2int_rz(r[i * 8 + 7]));
        }
        key[i] = k;
    }
    __syncthreads();
    // (orders are unique per image, so after the sort every slot finds its rank by a binary search of its key)
    for (int size = 2; size <= np2; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < np2; i += kNmsThreads) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool up = (i & size) == 0;
                    const unsigned long long a = key[i], b = key[j];
                    if ((a > b) == up) { key[i] = b; key[j] = a; }
                }
            }
            __syncthreads();
        }
    // rank of every slot: binary search of its key in the sorted array, then scatter its data to that rank
    for (int i = tid; i < n; i += kNmsThreads) {
        const float score = __fmul_rn(r[i * 8 + 4], r[i * 8 + 5]);
        const unsigned long long k = (static_cast<unsigned long long>(~__float_as_uint(score)) << 32) | static_cast<unsigned>(__float2int_rz(r[i * 8 + 7]));
        int lo = 0, hi = n - 1;
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (key[mid] < k) lo = mid + 1; else hi = mid; }
        bx[lo] = r[i * 8 + 0]; by[lo] = r[i * 8 + 1]; bw[lo] = r[i * 8 + 2]; bh[lo] = r[i * 8 + 3];
        conf[lo] = r[i * 8 + 4]; cls_conf[lo] = r[i * 8 + 5]; cls[lo] = static_cast<short>(__float2int_rz(r[i * 8 + 6]));
        done_cls[lo] = 0;
    }
    if (tid == 0) s_kept = 0;
    __syncthreads();
    float *o = out + static_cast<size_t>(img) * max_out * 8;
    // 2. All classes at once, one greedy step per round: every class takes its alive box with the highest
    //    objectness (first in list order on ties) and drops the remaining boxes of the class that overlap it.
    //    Classes are independent, so this keeps what the per-class loops of the reference keep; a box's place
    //    in the output is (rank of its class in first-seen order, round in which it was taken).
    //    Scratch per class id: first sorted position, best key of the round, boxes kept, output offset.
    int *first_pos = s_class_i;                                  // [kNmsMaxClasses]
    int *kept_cnt = s_class_i + kNmsMaxClasses;                  // [kNmsMaxClasses]
    int *cls_off = s_class_i + 2 * kNmsMaxClasses;               // [kNmsMaxClasses]
    for (int c = tid; c < kNmsMaxClasses; c += kNmsThreads) { first_pos[c] = 0x7fffffff; kept_cnt[c] = 0; s_best[c] = 0ull; }
    if (tid == 0) { s_bad = 0; s_alive = 0; }
    __syncthreads();
    for (int i = tid; i < n; i += kNmsThreads) {
        const int c = cls[i];
        if (c < 0 || c >= kNmsMaxClasses) s_bad = 1; else atomicMin(&first_pos[c], i);
        alive[i] = 1; done_cls[i] = 0xff;                        // done_cls: round in which the box was taken (0xff: not taken)
    }
    __syncthreads();
    if (s_bad) { if (tid == 0) out_counts[img] = -1; return; }   // class ids beyond the scratch tables: host path
    int remaining = n;
    for (int round = 0; remaining > 0; ++round) {
        // a. best alive box per class: key = objectness bits (positive floats order like their bits), then lowest position
        for (int i = tid; i < n; i += kNmsThreads)
            if (alive[i]) atomicMax(&s_best[cls[i]], (static_cast<unsigned long long>(__float_as_uint(fmaxf(conf[i], 0.f))) << 32) | static_cast<unsigned>(0x7fffffff - i));
        __syncthreads();
        // b. take it; drop what overlaps it
        for (int i = tid; i < n; i += kNmsThreads)
            if (alive[i]) {
                const int top = 0x7fffffff - static_cast<int>(s_best[cls[i]] & 0xffffffffu);
                if (top == i) { alive[i] = 0; kept_round[i] = static_cast<unsigned short>(round); done_cls[i] = 1; atomicAdd(&kept_cnt[cls[i]], 1); }
                else {
                    const float iou = nms_iou(bx[i], by[i], bw[i], bh[i], bx[top], by[top], bw[top], bh[top]);
                    const bool drop = use_soft ? (__fmul_rn(conf[i], expf(-__fdiv_rn(__fmul_rn(iou, iou), sigma))) <= 0.f) : (iou > nms_thresh);
                    if (drop) alive[i] = 0;
                }
            }
        if (tid == 0) s_alive = 0;
        __syncthreads();
        // c. reset the round's keys, count what is left
        int left = 0;
        for (int i = tid; i < n; i += kNmsThreads) if (alive[i]) { ++left; s_best[cls[i]] = 0ull; }
        for (int i = tid; i < n; i += kNmsThreads) if (done_cls[i] == 1) { s_best[cls[i]] = 0ull; done_cls[i] = 2; }
        if (left) atomicAdd(&s_alive, left);
        __syncthreads();
        remaining = s_alive;
        if (round >= 65534) break;
    }
    // 3. output offsets: classes in first-seen order. A class's rank = number of first occurrences before its own.
    //    (serial over the sorted list by one thread: n <= 4096, a few microseconds)
    if (tid == 0) {
        int off = 0;
        for (int i = 0; i < n; ++i) {
            const int c = cls[i];
            if (first_pos[c] == i) { cls_off[c] = off; off += kept_cnt[c]; }
        }
        s_kept = off;
    }
    __syncthreads();
    for (int i = tid; i < n; i += kNmsThreads)
        if (done_cls[i] == 2) {
            const int slot = cls_off[cls[i]] + kept_round[i];
            if (slot < max_out) {
                float *q = o + static_cast<size_t>(slot) * 8;
                q[0] = bx[i]; q[1] = by[i]; q[2] = bw[i]; q[3] = bh[i]; q[4] = conf[i]; q[5] = cls_conf[i];
                q[6] = static_cast<float>(cls[i]); q[7] = static_cast<float>(i);
            }
        }
    if (tid == 0) out_counts[img] = s_kept;
}

}  // namespace msnh
