// Times the reference's own training iteration WARM: one process, one Network object of the reference (its
// network.cu / layer.cu compiled unmodified, on cuDNN / cuBLAS), its own forwardPropagation() + backwardPropagation()
// called again and again through its public interface.  TEST / MEASUREMENT INFRASTRUCTURE ONLY; built by
// oracle/build_ref.py, runs on a machine with a GPU.
//
//   ref_warm <MODEL> <POLICY> <ALGO> <iterations> <warm-up iterations> <result file>
//
// The reference program itself (vdnn.cu:72-79) times a single, cold iteration per process with a wall clock that
// also covers host-side input generation: forwardPropagation() fills the input from a std::mt19937 on the host and
// copies it synchronously (network.cu:819-829, 1059/1078), backwardPropagation() does the same for the labels
// (network.cu:1045).  Here every iteration is bracketed by cudaDeviceSynchronize() and a wall clock, so the host
// generation runs while the GPU is idle and its time adds to the iteration exactly; that time is measured on its own
// (the same public randomInitializeData() on a scratch buffer of the same sizes) and subtracted:
//     net_ms = wall_ms - rng_ms
// The reference's per-layer printf lines go to stdout; redirect it.  Environment: VDNN_POOL_BYTES caps the pool
// (the reference asks for the whole device, network.cu:49); NVIDIA_TF32_OVERRIDE=0 makes cuDNN use FMA arithmetic.
#include "network.h"

#include <chrono>
#include <string>
#include <vector>

static int lookup(const char* s, const char* const* names, int count) {
    for (int i = 0; i < count; ++i) if (strcmp(s, names[i]) == 0) return i;
    fprintf(stderr, "ref_warm: unknown argument %s\n", s);
    exit(2);
}

static double now_ms() {
    using namespace std::chrono;
    return duration_cast<duration<double, std::milli>>(steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
    if (argc != 7) { fprintf(stderr, "usage: ref_warm MODEL POLICY ALGO iterations warmup result.json\n"); return 2; }
    static const char* const models[] = {"ALEXNET", "OVERFEAT", "GOOGLENET", "VGG16_64", "VGG16_128", "VGG16_256"};     // vdnn.h:52-61
    static const char* const policies[] = {"BASELINE", "VDNN_NONE", "VDNN_ALL", "VDNN_CONV"};                           // vdnn.h:23-29
    static const char* const algos[] = {"VDNN_MEMORY_OPT_ALGO", "VDNN_PERF_OPT_ALGO"};                                  // vdnn.h:31-36
    const CNN_t cnn = static_cast<CNN_t>(lookup(argv[1], models, 6));
    const vdnn_t policy = static_cast<vdnn_t>(lookup(argv[2], policies, 4));
    const vdnnAlgoMode_t algo = static_cast<vdnnAlgoMode_t>(lookup(argv[3], algos, 2));
    const int iters = atoi(argv[4]), warm = atoi(argv[5]);
    if (iters < 1 || warm < 0) return 2;
    checkCuda(cudaSetDevice(DEFAULT_DEVICE));

    Network net(cnn, policy, algo);
    const int in_size = net.getInputSize(), out_size = net.getOutputSize();
    const int batch = net.layerArray()[0]->InputN();

    std::vector<double> wall;
    for (int i = 0; i < warm + iters; ++i) {
        checkCuda(cudaDeviceSynchronize());
        const double t0 = now_ms();
        if (net.forwardPropagation() < 0 || net.backwardPropagation() < 0) { fprintf(stderr, "ref_warm: iteration failed\n"); return 1; }
        checkCuda(cudaDeviceSynchronize());
        const double t1 = now_ms();
        if (i >= warm) wall.push_back(t1 - t0);
    }

    // host-side generation + synchronous upload of one input and one label tensor, as each iteration did
    void* scratch = NULL;
    checkCuda(cudaMalloc(&scratch, sizeof(DATATYPE) * (size_t)in_size));
    std::vector<double> rng;
    for (int i = 0; i < 3; ++i) {
        checkCuda(cudaDeviceSynchronize());
        const double t0 = now_ms();
        net.randomInitializeData(scratch, in_size);
        net.randomInitializeData(scratch, out_size);
        checkCuda(cudaDeviceSynchronize());
        rng.push_back(now_ms() - t0);
    }
    checkCuda(cudaFree(scratch));

    double wall_mean = 0, rng_mean = 0, wall_min = wall[0];
    for (double v : wall) { wall_mean += v; if (v < wall_min) wall_min = v; }
    for (double v : rng) rng_mean += v;
    wall_mean /= wall.size(); rng_mean /= rng.size();
    FILE* f = fopen(argv[6], "w");
    if (!f) return 1;
    fprintf(f, "{\"model\": \"%s\", \"policy\": \"%s\", \"algo\": \"%s\", \"batch\": %d, \"iterations\": %d, \"warmup\": %d, "
               "\"wall_ms_mean\": %.3f, \"wall_ms_min\": %.3f, \"rng_ms_mean\": %.3f, \"net_ms_mean\": %.3f, \"images_per_s\": %.2f, "
               "\"cudnn_version\": %zu, \"tf32_override\": \"%s\", \"per_iteration_ms\": [",
            argv[1], argv[2], argv[3], batch, iters, warm, wall_mean, wall_min, rng_mean, wall_mean - rng_mean,
            batch / ((wall_mean - rng_mean) / 1e3), cudnnGetVersion(), getenv("NVIDIA_TF32_OVERRIDE") ? getenv("NVIDIA_TF32_OVERRIDE") : "");
    for (size_t i = 0; i < wall.size(); ++i) fprintf(f, "%s%.3f", i ? ", " : "", wall[i]);
    fprintf(f, "]}\n");
    fclose(f);
    return 0;
}
