// Command-line driver:  vdnn {CNN_MODEL} {VDNN_TYPE} {ALGO_MODE} [iterations]
// The three positional arguments, their spellings and the banner are those of the reference's
// vdnn.cu:8-54; an optional fourth argument repeats the forward + backward iteration.
#include <chrono>
#include <cstring>
#include <iostream>

#include "network.h"

static bool pick(const char* arg, const char* const* names, const int* values, int count, int* out) {
    for (int i = 0; i < count; ++i)
        if (strcmp(arg, names[i]) == 0) { *out = values[i]; return true; }
    return false;
}

static bool parseVdnnInputs(char** argv, CNN_t* cnnType, vdnn_t* vdnnType, vdnnAlgoMode_t* algoMode) {
    static const char* const cnn_names[] = {"ALEXNET", "OVERFEAT", "GOOGLENET", "VGG16_64", "VGG16_128", "VGG16_256", "CUSTOM_CNN", "ALEXNET_LRN"};
    static const int cnn_values[] = {ALEXNET, OVERFEAT, GOOGLENET, VGG16_64, VGG16_128, VGG16_256, CUSTOM_CNN, ALEXNET_LRN};
    static const char* const vdnn_names[] = {"BASELINE", "VDNN_NONE", "VDNN_ALL", "VDNN_CONV"};
    static const int vdnn_values[] = {BASELINE, VDNN_NONE, VDNN_ALL, VDNN_CONV};
    static const char* const algo_names[] = {"VDNN_MEMORY_OPT_ALGO", "VDNN_PERF_OPT_ALGO", "VDNN_DYNAMIC_ALGO"};
    static const int algo_values[] = {VDNN_MEMORY_OPT_ALGO, VDNN_PERF_OPT_ALGO, VDNN_DYNAMIC_ALGO};
    int a, b, c;
    if (!pick(argv[1], cnn_names, cnn_values, 8, &a)) {
        fprintf(stderr, "CNN type must be one of ALEXNET, OVERFEAT, GOOGLENET, VGG16_64, VGG16_128, VGG16_256, CUSTOM_CNN\n");
        return false;
    }
    if (!pick(argv[2], vdnn_names, vdnn_values, 4, &b)) {
        fprintf(stderr, "VDNN type must be one of BASELINE, VDNN_NONE, VDNN_ALL, VDNN_CONV\n");
        return false;
    }
    if (!pick(argv[3], algo_names, algo_values, 3, &c)) {
        fprintf(stderr, "Algorithm type must be one of VDNN_MEMORY_OPT_ALGO, VDNN_PERF_OPT_ALGO, VDNN_DYNAMIC_ALGO\n");
        return false;
    }
    *cnnType = static_cast<CNN_t>(a); *vdnnType = static_cast<vdnn_t>(b); *algoMode = static_cast<vdnnAlgoMode_t>(c);
    printf("################# VDNN Configurations #################\n");
    printf("CNN Model Type: %s\n", argv[1]);
    printf("VDNN Mode: %s\n", argv[2]);
    printf("Convolution Algorithm: %s\n", argv[3]);
    printf("#######################################################\n\n");
    return true;
}

int main(int argc, char** argv) {
    if (argc != 4 && argc != 5) {
        fprintf(stderr, "Need to specify CNN model, VDNN mode, and Algorithm choice\n");
        return 2;
    }
    CNN_t cnnType; vdnn_t vdnnType; vdnnAlgoMode_t algoMode;
    if (!parseVdnnInputs(argv, &cnnType, &vdnnType, &algoMode)) return 2;
    const int iterations = argc == 5 ? atoi(argv[4]) : 1;

    Network network(cnnType, vdnnType, algoMode);
    if (network.status() != VDNN_OK) {
        fprintf(stderr, "network construction failed: %s\n", vdnn_status_string(network.status()));
        return 1;
    }
    for (int it = 0; it < (iterations > 0 ? iterations : 1); ++it) {
        auto t1 = std::chrono::high_resolution_clock::now();
        int st = network.forwardPropagation();
        if (st == 0) st = network.backwardPropagation();
        if (st == 0) st = network.synchronize();
        auto t2 = std::chrono::high_resolution_clock::now();
        if (st != 0) { fprintf(stderr, "iteration failed: %s\n", vdnn_status_string(st)); return 1; }
        // the reference labels microseconds "ms" (vdnn.cu:78-79); both units are printed here
        const long long us = std::chrono::duration_cast<std::chrono::microseconds>(t2 - t1).count();
        std::cout << "Elapsed Time: " << us << "us (" << us / 1000.0 << " ms)" << std::endl << std::endl;
    }
    return 0;
}
