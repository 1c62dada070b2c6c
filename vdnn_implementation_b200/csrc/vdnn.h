// Enumerations and constants of the vDNN driver.  The enumerator names and values are the ones
// the reference exposes in vdnn.h:5-61, so code written against it keeps compiling; LRN and
// ALEXNET_LRN are additions.
#ifndef VDNN_B200_VDNN_H_
#define VDNN_B200_VDNN_H_

#define DEFAULT_DEVICE 0
#define DEFAULT_NUM_LAYER 40
#define DEFAULT_BATCH_SIZE 128
#define LEARNING_RATE 1e-5
#define BLOCK_SIZE 256
#define RANDOM_VALUE_LIMIT 1e-2
#define DATATYPE float

typedef enum { BASELINE = 0, VDNN_NONE = 1, VDNN_ALL = 2, VDNN_CONV = 3 } vdnn_t;

typedef enum { VDNN_MEMORY_OPT_ALGO = 0, VDNN_PERF_OPT_ALGO = 1, VDNN_DYNAMIC_ALGO = 2 } vdnnAlgoMode_t;

typedef enum {
    FC_GEMM = 0, CONV = 1, FC_CONV = 2, RELU = 3, TANH = 4, SIGMOID = 5, SOFTMAX = 6, POOL = 7,
    CONCATENATE = 8, LRN = 9, NUM_LAYER_TYPES = 10
} Layer_t;

typedef enum {
    ALEXNET = 0, OVERFEAT = 1, GOOGLENET = 2, VGG16_64 = 3, VGG16_128 = 4, VGG16_256 = 5,
    CUSTOM_CNN = 6, ALEXNET_LRN = 7
} CNN_t;

#endif
