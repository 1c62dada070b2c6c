// Force-include header (nvcc -include) that lets the reference's own driver sources -- network.cu and vdnn.cu,
// unmodified -- compile against this library's Layer class instead of the reference's cuDNN / cuBLAS one:
//
//   nvcc -include <this file> -I <csrc> -I <include> <reference>/vdnn.cu <reference>/network.cu -lvdnn_b200
//
// The reference's network.h pulls in "layer.h" and "vdnn.h" from its own directory; their include guards are claimed
// here, so those two files contribute nothing and this library's layer.h / vdnn.h (same class name, method names,
// argument lists and enumerators: layer.h:130-251, vdnn.h:5-61) take their place.  What the driver sources use beyond
// the Layer class is supplied below:
//   * the two handle types and the six handle calls of network.cu:39-40, 56-57, 96-97, mapped onto vdnnHandle_t;
//   * the checking macros and helpers of the reference's layer.h:60-128 (same names and behaviour: print and abort,
//     or -1 for a soft out-of-memory in dynamic mode).
#ifndef VDNN_B200_REF_DROPIN_H_
#define VDNN_B200_REF_DROPIN_H_

#define _LAYER_H_
#define _VDNN_H_

#include <assert.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <chrono>
#include <fstream>
#include <iostream>
#include <random>
#include <sstream>
#include <string>
#include <vector>

#include "layer.h"

typedef vdnnHandle_t cudnnHandle_t;
typedef vdnnHandle_t cublasHandle_t;
enum { CUDNN_STATUS_SUCCESS = 0, CUBLAS_STATUS_SUCCESS = 0 };
static inline int cudnnCreate(cudnnHandle_t* h) { return vdnnCreate(h); }
static inline int cublasCreate(cublasHandle_t* h) { return vdnnCreate(h); }
static inline int cudnnSetStream(cudnnHandle_t h, cudaStream_t s) { return vdnnSetStream(h, s); }
static inline int cublasSetStream(cublasHandle_t h, cudaStream_t s) { return vdnnSetStream(h, s); }
static inline int cudnnDestroy(cudnnHandle_t) { return 0; }
static inline int cublasDestroy(cublasHandle_t h) { return vdnnDestroy(h); }

#define M_ASSERT(EXPR, MESSAGE) { assert(((void)(MESSAGE), (EXPR))); }

#define FatalError(s) {                                                                   \
    std::cerr << std::string(s) << "\n" << __FILE__ << ':' << __LINE__ << "\nAborting...\n"; \
    cudaDeviceReset();                                                                    \
    exit(EXIT_FAILURE);                                                                   \
}
#define checkCUDNN(status) { if ((status) != 0) { std::stringstream _e; _e << "vdnn_b200 failure: " << (status); FatalError(_e.str()); } }
#define checkCUBLAS(status) checkCUDNN(status)
#define checkCudaErrors(status) { if ((status) != 0) { std::stringstream _e; _e << "Cuda failure: " << (status); FatalError(_e.str()); } }

static inline cudaError_t checkCuda(cudaError_t result) {
    if (result != cudaSuccess) {
        fprintf(stderr, "CUDA Runtime Error: %s\n", cudaGetErrorString(result));
        assert(result == cudaSuccess);
    }
    return result;
}

// 0 on success; in dynamic mode an exhausted pool is reported as -1 instead of aborting (layer.h:112-128)
static inline int ASSERT_EQ(cnmemStatus_t result, bool isDynamicMode = false) {
    if (result == CNMEM_STATUS_SUCCESS) return 0;
    if (isDynamicMode) return result == CNMEM_STATUS_OUT_OF_MEMORY ? -1 : -2;
    printf("\n[CNMEM FAILED with error %s]\n", cnmemGetErrorString(result));
    assert(0);
    return 0;
}

#endif
