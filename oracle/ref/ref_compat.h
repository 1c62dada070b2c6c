// Compatibility shim that lets the reference's layer.cu compile unmodified against cuDNN 9.
// TEST INFRASTRUCTURE ONLY (force-included with `nvcc -include` by oracle/build_ref.py).
//
// The reference picks its convolution algorithms with cudnnGetConvolution{Forward,BackwardData,
// BackwardFilter}Algorithm and the *_NO_WORKSPACE / *_PREFER_FASTEST preferences (layer.cu:1013-1089),
// an interface cuDNN removed in version 8.  The three functions and their preference enums are
// re-created here on top of the heuristic queries that remain (cudnnGet...Algorithm_v7):
//   NO_WORKSPACE    -> the best-ranked algorithm that reports zero workspace
//   PREFER_FASTEST  -> the best-ranked algorithm
#ifndef VDNN_ORACLE_REF_COMPAT_H_
#define VDNN_ORACLE_REF_COMPAT_H_

#include <cudnn.h>

typedef enum {
    CUDNN_CONVOLUTION_FWD_NO_WORKSPACE = 0,
    CUDNN_CONVOLUTION_FWD_PREFER_FASTEST = 1,
    CUDNN_CONVOLUTION_FWD_SPECIFY_WORKSPACE_LIMIT = 2
} cudnnConvolutionFwdPreference_t;
typedef enum {
    CUDNN_CONVOLUTION_BWD_DATA_NO_WORKSPACE = 0,
    CUDNN_CONVOLUTION_BWD_DATA_PREFER_FASTEST = 1,
    CUDNN_CONVOLUTION_BWD_DATA_SPECIFY_WORKSPACE_LIMIT = 2
} cudnnConvolutionBwdDataPreference_t;
typedef enum {
    CUDNN_CONVOLUTION_BWD_FILTER_NO_WORKSPACE = 0,
    CUDNN_CONVOLUTION_BWD_FILTER_PREFER_FASTEST = 1,
    CUDNN_CONVOLUTION_BWD_FILTER_SPECIFY_WORKSPACE_LIMIT = 2
} cudnnConvolutionBwdFilterPreference_t;

template <class Perf, class Algo>
static inline cudnnStatus_t vdnn_ref_pick(const Perf* perf, int count, int preference, size_t limit, Algo* out) {
    for (int i = 0; i < count; ++i) {
        if (perf[i].status != CUDNN_STATUS_SUCCESS) continue;
        if (preference == 0 && perf[i].memory != 0) continue;
        if (preference == 2 && perf[i].memory > limit) continue;
        *out = perf[i].algo;
        return CUDNN_STATUS_SUCCESS;
    }
    return CUDNN_STATUS_NOT_SUPPORTED;
}

static inline cudnnStatus_t cudnnGetConvolutionForwardAlgorithm(
    cudnnHandle_t handle, const cudnnTensorDescriptor_t x, const cudnnFilterDescriptor_t w,
    const cudnnConvolutionDescriptor_t conv, const cudnnTensorDescriptor_t y,
    cudnnConvolutionFwdPreference_t preference, size_t limit, cudnnConvolutionFwdAlgo_t* algo) {
    cudnnConvolutionFwdAlgoPerf_t perf[16];
    int n = 0;
    cudnnStatus_t st = cudnnGetConvolutionForwardAlgorithm_v7(handle, x, w, conv, y, 16, &n, perf);
    return st != CUDNN_STATUS_SUCCESS ? st : vdnn_ref_pick(perf, n, preference, limit, algo);
}

static inline cudnnStatus_t cudnnGetConvolutionBackwardDataAlgorithm(
    cudnnHandle_t handle, const cudnnFilterDescriptor_t w, const cudnnTensorDescriptor_t dy,
    const cudnnConvolutionDescriptor_t conv, const cudnnTensorDescriptor_t dx,
    cudnnConvolutionBwdDataPreference_t preference, size_t limit, cudnnConvolutionBwdDataAlgo_t* algo) {
    cudnnConvolutionBwdDataAlgoPerf_t perf[16];
    int n = 0;
    cudnnStatus_t st = cudnnGetConvolutionBackwardDataAlgorithm_v7(handle, w, dy, conv, dx, 16, &n, perf);
    return st != CUDNN_STATUS_SUCCESS ? st : vdnn_ref_pick(perf, n, preference, limit, algo);
}

static inline cudnnStatus_t cudnnGetConvolutionBackwardFilterAlgorithm(
    cudnnHandle_t handle, const cudnnTensorDescriptor_t x, const cudnnTensorDescriptor_t dy,
    const cudnnConvolutionDescriptor_t conv, const cudnnFilterDescriptor_t dw,
    cudnnConvolutionBwdFilterPreference_t preference, size_t limit, cudnnConvolutionBwdFilterAlgo_t* algo) {
    cudnnConvolutionBwdFilterAlgoPerf_t perf[16];
    int n = 0;
    cudnnStatus_t st = cudnnGetConvolutionBackwardFilterAlgorithm_v7(handle, x, dy, conv, dw, 16, &n, perf);
    return st != CUDNN_STATUS_SUCCESS ? st : vdnn_ref_pick(perf, n, preference, limit, algo);
}

#endif
