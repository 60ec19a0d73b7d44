/*
 * msnhnet_capi.h — the reference's own C ABI for this path, kept symbol for symbol
 * (src/c_api/MsnhnetLib.h:39-61 in the Msnhnet source tree), plus batched entry points.
 *
 * One process-global net, as in the reference (src/c_api/MsnhnetLib.cpp:3). Return values as there:
 * 1 = ok, -1 = error with *msg pointing at a NUL-terminated text (a thread-local buffer that stays
 * valid until the next call on the same thread; the reference's pointer dangled,
 * src/c_api/MsnhnetLib.cpp:25-32). runGPU must be non-zero: this backend has no CPU path.
 * runClassifyList / runYoloList take a raw 8-bit RGB image and run the reference's preprocessing on the device;
 * runClassifyFile / runYoloFile (image decoding) return -1.
 */
#ifndef MSNHNET_CAPI_H
#define MSNHNET_CAPI_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define MSNH_MAX_BBOX_NUM 1024

typedef enum PredDataType {
    PRE_DATA_NONE = 0, PRE_DATA_FC32_C1, PRE_DATA_FC32_C3, PRE_DATA_GOOGLENET_FC3, PRE_DATA_PADDING_ZERO_FC3,
    PRE_DATA_TRANSFORMED_FC3, PRE_DATA_CAFFE_FC3
} PredDataType;

typedef struct BBox {
    float x, y, w, h, conf, bestClsConf;
    uint32_t bestClsIdx;
    float angle;
} BBox;
typedef struct BBoxContainer { BBox boxes[MSNH_MAX_BBOX_NUM]; } BBoxContainer;

/* ---- the reference's 13 entry points (src/c_api/MsnhnetLib.h:39-61) ---- */
int initMsnhnet(void);
int buildMsnhnet(char **msg, const char *msnhnet, const char *msnhbin, int useFp16, int useCudaOnly);
int runClassifyFile(char **msg, const char *imagePath, int *bestIndex, PredDataType preDataType, int runGPU,
                    const float *mean, const float *std);
int runClassifyList(char **msg, unsigned char *imageData, const int width, const int height, const int channel,
                    int *bestIndex, PredDataType preDataType, const int swapRGB, int runGPU, const float *mean,
                    const float *std);
int runClassifyNoPred(char **msg, const float *data, const int len, int *bestIndex, int runGPU);
int runYoloFile(char **msg, const char *imagePath, BBoxContainer *bboxContainer, int *detectedNum, const int runGPU);
int runYoloList(char **msg, unsigned char *imageData, const int width, const int height, const int channel,
                BBoxContainer *bboxContainer, int *detectedNum, const int swapRGB, const int runGPU);
int dispose(void);
int withGPU(int *GPU);
int withCUDNN(int *CUDNN);
int getCpuForwardTime(float *time);
int getGpuForwardTime(float *time);
int getInputDim(int *width, int *heigth, int *channel);

/* ---- additions: batched inference on planar CHW float images in host memory ---- */
/* Before buildMsnhnet: CUDA device, images per forward (0 = the file's batch), MSNH_PLAN_* flags. */
int msnhB200SetOptions(int device, int batch, unsigned planFlags);
/* After initMsnhnet: run the score sort + NMS of runYolo* on the device (1) or on the host as the reference does
 * (0, default). Images with more than 4096 candidates take the host path either way. Returns -1 without a net. */
int msnhB200SetDeviceNms(int enable);
/* After initMsnhnet, before buildMsnhnet: keep the packed device form of the weights in "<msnhbin>.b200pack" and
 * load it on later builds of the same net, options and blob (size + modification time) instead of reading and
 * repacking the float blob. Off by default. msnhB200LastLoadUsedPack: 1 if the last buildMsnhnet loaded a pack. */
int msnhB200SetPackCache(int enable);
int msnhB200LastLoadUsedPack(void);
/* Build from memory instead of files (topology text + float blob). */
int msnhB200BuildFromMemory(char **msg, const char *msnhnetText, const float *weights, size_t weightCount, int useFp16);
/* Parse + shape-check only (no GPU needed): layer count and blob length the topology implies. */
int msnhB200Inspect(char **msg, const char *msnhnetText, int *layers, size_t *weightCount, int *isYolo);
/* On success *msg holds one line per tensor of the .msnhbin blob, in blob order: "op slot count rows"
 * (slot = MSNH_W_* of include/msnh_b200.h; rows = output channels of a weight tensor). No GPU needed. */
int msnhB200WeightLayout(char **msg, const char *msnhnetText);
/* On success *msg holds the op list the topology lowers to, what is handed to msnh_b200_plan_create: one line per op,
 * "op" followed by every field of MsnhB200Op in declaration order. No GPU needed. */
int msnhB200OpList(char **msg, const char *msnhnetText);
int msnhB200RunClassifyBatch(char **msg, const float *images, int nImages, float *out, size_t outCapacity);
/* boxes: nImages * maxBoxesPerImage entries; counts[i] boxes of image i start at i*maxBoxesPerImage. */
int msnhB200RunYoloBatch(char **msg, const float *images, int nImages, BBox *boxes, int maxBoxesPerImage, int *counts);
/* Streaming forms: nBatches batches (of the net's batch size each) back to back in host memory,
 * pinned for full overlap. Copy-in of batch i+1, forward of batch i and host NMS of batch i-1 run
 * concurrently. Results for all nBatches*batch images in image order, laid out as above. */
int msnhB200RunYoloStream(char **msg, const float *images, int nBatches, BBox *boxes, int maxBoxesPerImage, int *counts);
int msnhB200RunClassifyStream(char **msg, const float *images, int nBatches, float *out, size_t outCapacity);
/* The streaming forms for raw 8-bit images, the input runYoloList / runClassifyList take (src/c_api/MsnhnetLib.cpp:508,
 * 754): nBatches * batch HWC RGB images of width x height pixels back to back; resize / letterbox / scaling run on the
 * device, so a quarter of the bytes cross PCIe. swapRGB as in runYoloList; prepMode = MSNH_PREP_* of msnh_b200.h with
 * mean / std for the transformed mode (NULL otherwise). */
int msnhB200RunYoloStreamU8(char **msg, const unsigned char *images, int width, int height, int swapRGB, int nBatches,
                            BBox *boxes, int maxBoxesPerImage, int *counts);
int msnhB200RunClassifyStreamU8(char **msg, const unsigned char *images, int width, int height, int prepMode, int swapRGB,
                                const float *mean, const float *std, int nBatches, float *out, size_t outCapacity);
/* Forward only: H2D copy + kernels + sync, no result read-back. */
int msnhB200Forward(char **msg, const float *images, int nImages);
/* Forward with the input already in the plan's device staging buffer; sync = 0 returns at once. */
int msnhB200ForwardResident(char **msg, int nImages, int sync);
/* Output of top-level layer `layer` of the last forward (plan must keep all outputs). */
int msnhB200GetLayerOutput(char **msg, int layer, int nImages, float *out, size_t capacity, int *c, int *h, int *w);
/* Candidate rows {x,y,w,h,conf,bestClsConf,bestClsIdx,order} of the last forward, before NMS. */
int msnhB200GetCandidates(char **msg, int nImages, float *rows, int maxRowsPerImage, int *counts);
/* The host half of YoloOut on caller-supplied candidate rows: score sort + NMS. */
int msnhB200PostProcess(const float *rows, int count, float nmsThresh, int useSoftNms, BBox *out, int maxOut, int *n);
int msnhB200GetInfo(int *layers, size_t *weightCount, int *isYolo, int *batch, int *lastC, int *lastH, int *lastW,
                    float *confThresh, float *nmsThresh);
int msnhB200KernelTimeMs(float *ms);
/* Opaque MsnhB200Plan* / MsnhB200Ctx* of the global net (include/msnh_b200.h), for profiling. */
void *msnhB200PlanHandle(void);
void *msnhB200CtxHandle(void);

#ifdef __cplusplus
}
#endif
#endif
