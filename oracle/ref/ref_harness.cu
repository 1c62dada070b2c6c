// Drives the reference's own Layer class (compiled unmodified from its sources, on cuDNN / cuBLAS)
// on seeded inputs and dumps what it computes.  TEST INFRASTRUCTURE ONLY: the dumps become the golden
// fixtures under tests/golden/ that pin the CPU oracle (and through it the CUDA kernels) to the
// reference's arithmetic.  Built by oracle/build_ref.py; runs on a machine with a GPU.
//
//   ref_harness <output directory> [big]
//
// Inputs are not stored: they come from the counter-based generator (seed = 100 * case + role), which
// the oracle reproduces bit for bit.  Outputs are raw little-endian float32 files plus manifest.json.
// With `big` the cases are convolutions and an FC layer at or near the sizes the benchmarked networks run them at
// (every tile shape, split plan and special-case kernel of the CUDA library is reached); their tensors are too large
// to keep, so each is reduced to SAMPLE_COUNT evenly strided elements plus sum, sum of squares (both in double) and
// largest magnitude over the whole tensor.
#define private public          // the Layer class keeps filterData / biasData / convDesc private
#include "layer.h"
#undef private

#include <string>
#include <vector>

#include "vdnn_b200.h"          // host generators only (vdnn_host_fill_*)

static cudnnHandle_t g_cudnn;
static cublasHandle_t g_cublas;
static cudaStream_t g_compute, g_memory;
static std::string g_dir;
static FILE* g_manifest;
static bool g_first = true;
static bool g_big = false;
static const size_t SAMPLE_COUNT = 4096;
static std::string g_stats;          // big mode: one JSON object per dumped tensor

static void* dev_from(const std::vector<float>& h) {
    void* p = NULL;
    ASSERT_EQ(cnmemMalloc(&p, h.size() * sizeof(float), NULL));
    checkCudaErrors(cudaMemcpy(p, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice));
    return p;
}
static void dump(const std::string& name, const void* dev, size_t count) {
    std::vector<float> h(count);
    checkCudaErrors(cudaDeviceSynchronize());
    checkCudaErrors(cudaMemcpy(h.data(), dev, count * sizeof(float), cudaMemcpyDeviceToHost));
    FILE* f = fopen((g_dir + "/" + name + ".bin").c_str(), "wb");
    if (!g_big) {
        fwrite(h.data(), sizeof(float), count, f);
        fclose(f);
        return;
    }
    const size_t stride = count > SAMPLE_COUNT ? count / SAMPLE_COUNT : 1;
    size_t samples = 0;
    double sum = 0.0, sumsq = 0.0, maxabs = 0.0;
    for (size_t i = 0; i < count; ++i) {
        const double v = h[i];
        sum += v; sumsq += v * v;
        if (fabs(v) > maxabs) maxabs = fabs(v);
        if (i % stride == 0 && samples < SAMPLE_COUNT) { fwrite(&h[i], sizeof(float), 1, f); ++samples; }
    }
    fclose(f);
    char buf[512];
    snprintf(buf, sizeof buf, "%s\n  {\"name\": \"%s\", \"count\": %zu, \"stride\": %zu, \"samples\": %zu, \"sum\": %.17g, \"sumsq\": %.17g, \"maxabs\": %.9g}",
             g_stats.empty() ? "" : ",", name.c_str(), count, stride, samples, sum, sumsq, maxabs);
    g_stats += buf;
}
static std::vector<float> normal(size_t n, uint64_t seed, float std) {
    std::vector<float> v(n);
    vdnn_host_fill_normal(v.data(), n, seed, 0.0f, std);
    return v;
}
static void entry(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    fprintf(g_manifest, g_first ? "\n  " : ",\n  ");
    vfprintf(g_manifest, fmt, ap);
    va_end(ap);
    g_first = false;
}

// CONV / FC_CONV layer: forward, then backward twice -- once with the real weights (data gradient uses
// the pre-update weights, layer.cu:616-625) and once from zero weights so that the stored filter / bias
// equal (-LEARNING_RATE) * gradient exactly (layer.cu:631-660 fold the SGD step into the call).
static void conv_case(int id, int n, int c, int h, int w, int k, int r, int pad, int stride, float wstd = 0.2f) {
    bool off[DEFAULT_NUM_LAYER] = {false};
    Layer L(VDNN_NONE, VDNN_MEMORY_OPT_ALGO, FC_CONV, &g_cudnn, &g_compute, &g_memory, 0, n, c, h, w, pad, pad, stride, stride, k, r, r);
    const size_t xs = (size_t)n * c * h * w, ws = (size_t)k * c * r * r, ys = (size_t)L.DstDataSize();
    std::vector<float> x = normal(xs, 100 * id + 1, 1.0f), wt = normal(ws, 100 * id + 2, wstd), b = normal(k, 100 * id + 3, 1.0f),
                       dy = normal(ys, 100 * id + 4, 1.0f), zero_w(ws, 0.0f), zero_b(k, 0.0f);
    checkCudaErrors(cudaMemcpy(L.filterData, wt.data(), ws * sizeof(float), cudaMemcpyHostToDevice));
    checkCudaErrors(cudaMemcpy(L.biasData, b.data(), k * sizeof(float), cudaMemcpyHostToDevice));
    L.copySrcData(dev_from(x));
    L.forward(off, NULL, NULL, false);
    std::string tag = "conv" + std::to_string(id);
    dump(tag + "_y", L.DstData(), ys);
    L.copyDiffData(dev_from(dy));
    L.backward(-1, NULL, NULL, 0, NULL, false);
    dump(tag + "_dx", L.GradData(), xs);
    checkCudaErrors(cudaMemcpy(L.filterData, zero_w.data(), ws * sizeof(float), cudaMemcpyHostToDevice));
    checkCudaErrors(cudaMemcpy(L.biasData, zero_b.data(), k * sizeof(float), cudaMemcpyHostToDevice));
    L.backward(-1, NULL, NULL, 0, NULL, false);
    dump(tag + "_wstep", L.filterData, ws);
    dump(tag + "_bstep", L.biasData, k);
    entry("{\"kind\": \"conv\", \"id\": %d, \"n\": %d, \"c\": %d, \"h\": %d, \"w\": %d, \"k\": %d, \"r\": %d, \"pad\": %d, \"stride\": %d, "
          "\"p\": %d, \"q\": %d, \"fwd_algo\": %d, \"bwd_data_algo\": %d, \"bwd_filter_algo\": %d, \"lr\": %.9g, \"wstd\": %.9g}",
          id, n, c, h, w, k, r, pad, stride, L.OutputH(), L.OutputW(), (int)L.fwdAlgo, (int)L.bwdDataAlgo, (int)L.bwdFilterAlgo,
          (double)(float)(LEARNING_RATE), (double)wstd);
}

// FC_GEMM layer (cuBLAS): layer.cu:667-764.
static void fc_case(int id, int n, int cin, int cout, float wstd = 0.1f) {
    bool off[DEFAULT_NUM_LAYER] = {false};
    Layer L(VDNN_NONE, VDNN_MEMORY_OPT_ALGO, FC_GEMM, &g_cublas, &g_compute, &g_memory, 0, n, cin, 1, 1, 0, 0, 0, 0, cout, 1, 1);
    const size_t xs = (size_t)n * cin, ws = (size_t)cin * cout, ys = (size_t)n * cout;
    std::vector<float> x = normal(xs, 100 * id + 1, 1.0f), wt = normal(ws, 100 * id + 2, wstd), b = normal(cout, 100 * id + 3, 1.0f),
                       dy = normal(ys, 100 * id + 4, 1.0f), zero_w(ws, 0.0f), zero_b(cout, 0.0f);
    checkCudaErrors(cudaMemcpy(L.filterData, wt.data(), ws * sizeof(float), cudaMemcpyHostToDevice));
    checkCudaErrors(cudaMemcpy(L.biasData, b.data(), cout * sizeof(float), cudaMemcpyHostToDevice));
    L.copySrcData(dev_from(x));
    L.forward(off, NULL, NULL, false);
    std::string tag = "fc" + std::to_string(id);
    dump(tag + "_y", L.DstData(), ys);
    L.copyDiffData(dev_from(dy));
    L.backward(-1, NULL, NULL, 0, NULL, false);
    dump(tag + "_dx", L.GradData(), xs);
    checkCudaErrors(cudaMemcpy(L.filterData, zero_w.data(), ws * sizeof(float), cudaMemcpyHostToDevice));
    checkCudaErrors(cudaMemcpy(L.biasData, zero_b.data(), cout * sizeof(float), cudaMemcpyHostToDevice));
    L.backward(-1, NULL, NULL, 0, NULL, false);
    dump(tag + "_wstep", L.filterData, ws);
    dump(tag + "_bstep", L.biasData, cout);
    entry("{\"kind\": \"fc\", \"id\": %d, \"n\": %d, \"cin\": %d, \"cout\": %d, \"lr\": %.9g, \"wstd\": %.9g}", id, n, cin, cout,
          (double)(float)(LEARNING_RATE), (double)wstd);
}

// RELU / POOL / SOFTMAX layers.  mode: 0 = N(0,1) input, 1 = input clamped at zero with the upper half
// of every image set to zero (what a pool sees after ReLU: windows of equal values), 2 = all equal.
static void simple_case(const char* kind, Layer_t type, int id, int n, int c, int h, int w, int win, int stride, int mode) {
    bool off[DEFAULT_NUM_LAYER] = {false};
    Layer L(VDNN_NONE, VDNN_MEMORY_OPT_ALGO, type, &g_cudnn, &g_compute, &g_memory, 0, n, c, h, w, 0, 0, stride, stride, 0, win, win);
    const size_t xs = (size_t)n * c * h * w, ys = (size_t)L.DstDataSize();
    std::vector<float> x = normal(xs, 100 * id + 1, type == SOFTMAX ? 4.0f : 1.0f), dy = normal(ys, 100 * id + 4, 1.0f);
    if (mode >= 1)
        for (size_t i = 0; i < xs; ++i) {
            const size_t row = (i / w) % h;
            x[i] = (mode == 2) ? 1.0f : ((x[i] > 0.0f && row >= (size_t)h / 2) ? x[i] : 0.0f);
        }
    L.copySrcData(dev_from(x));
    L.forward(off, NULL, NULL, false);
    std::string tag = std::string(kind) + std::to_string(id);
    dump(tag + "_y", L.DstData(), ys);
    L.copyDiffData(dev_from(dy));
    L.backward(-1, NULL, NULL, 0, NULL, false);
    dump(tag + "_dx", L.GradData(), xs);
    entry("{\"kind\": \"%s\", \"id\": %d, \"n\": %d, \"c\": %d, \"h\": %d, \"w\": %d, \"win\": %d, \"stride\": %d, \"mode\": %d, \"p\": %d, \"q\": %d}",
          kind, id, n, c, h, w, win, stride, mode, L.OutputH(), L.OutputW());
}

int main(int argc, char** argv) {
    if (argc != 2 && !(argc == 3 && strcmp(argv[2], "big") == 0)) { fprintf(stderr, "usage: ref_harness <output directory> [big]\n"); return 2; }
    g_dir = argv[1];
    g_big = argc == 3;
    checkCudaErrors(cudaSetDevice(0));
    checkCUDNN(cudnnCreate(&g_cudnn));
    checkCUBLAS(cublasCreate(&g_cublas));
    checkCudaErrors(cudaStreamCreate(&g_compute));
    checkCudaErrors(cudaStreamCreate(&g_memory));
    cudaStream_t streams[2] = {g_compute, g_memory};
    size_t sizes[2] = {0, 0};
    cnmemDevice_t dev;
    dev.device = 0; dev.size = g_big ? (size_t)12 << 30 : (size_t)2 << 30; dev.numStreams = 2; dev.streams = streams; dev.streamSizes = sizes;
    ASSERT_EQ(cnmemInit(1, &dev, 0));
    cudnnSetStream(g_cudnn, g_compute);
    cublasSetStream(g_cublas, g_compute);
    g_manifest = fopen((g_dir + "/manifest.json").c_str(), "w");
    fprintf(g_manifest, "{\"cudnn_version\": %zu, \"cases\": [", cudnnGetVersion());

    if (g_big) {
        // He-style weight scale sqrt(2 / fan-in) keeps outputs near the inputs' magnitude at these reduction lengths
        conv_case(20, 2, 64, 224, 224, 64, 3, 1, 1, sqrtf(2.0f / (64 * 9)));       // VGG16 conv1_2: 64-column tiles, two CTAs per SM
        conv_case(21, 4, 256, 56, 56, 256, 3, 1, 1, sqrtf(2.0f / (256 * 9)));      // VGG16 conv3_2: 256-column tiles
        conv_case(22, 8, 512, 14, 14, 512, 3, 1, 1, sqrtf(2.0f / (512 * 9)));      // VGG16 conv5_x: few tiles, reduction split, packed dy
        conv_case(23, 8, 3, 227, 227, 96, 11, 0, 4, sqrtf(2.0f / (3 * 121)));      // AlexNet conv1: phase-class data gradient
        conv_case(24, 4, 128, 112, 112, 128, 3, 1, 1, sqrtf(2.0f / (128 * 9)));    // VGG16 conv2_2: 128-column tiles
        conv_case(25, 8, 96, 27, 27, 256, 5, 2, 1, sqrtf(2.0f / (96 * 25)));       // AlexNet conv2: 5x5, pad 2, ragged 27x27 rows
        conv_case(26, 8, 1024, 6, 6, 3072, 6, 0, 1, sqrtf(2.0f / (1024 * 36)));    // OverFeat classifier: filter covers the input
        fc_case(27, 128, 25088, 4096, sqrtf(2.0f / 25088));                          // VGG16 fc1 at batch 128
        fprintf(g_manifest, "\n], \"tensors\": [%s\n]}\n", g_stats.c_str());
        fclose(g_manifest);
        printf("ref_harness: wrote reduced fixtures of the large cases to %s\n", g_dir.c_str());
        return 0;
    }
    // every filter / stride / pad combination of AlexNet, OverFeat and VGG16 at small extents
    conv_case(1, 2, 3, 27, 27, 6, 11, 0, 4);
    conv_case(2, 2, 5, 9, 9, 7, 5, 2, 1);
    conv_case(3, 2, 4, 12, 12, 6, 5, 0, 1);
    conv_case(4, 2, 6, 13, 13, 5, 3, 1, 1);
    conv_case(5, 3, 6, 6, 6, 8, 6, 0, 1);
    conv_case(6, 2, 8, 1, 1, 4, 1, 0, 1);
    conv_case(7, 2, 16, 14, 14, 24, 3, 1, 1);
    fc_case(8, 4, 96, 40);
    fc_case(9, 3, 50, 10);
    simple_case("relu", RELU, 10, 2, 3, 7, 7, 0, 0, 0);
    simple_case("pool", POOL, 11, 2, 3, 13, 13, 3, 2, 0);
    simple_case("pool", POOL, 12, 2, 3, 12, 12, 2, 2, 0);
    simple_case("pool", POOL, 13, 2, 3, 13, 13, 3, 2, 1);      // ties after ReLU, overlapping windows
    simple_case("pool", POOL, 14, 2, 3, 12, 12, 2, 2, 1);      // ties after ReLU, disjoint windows
    simple_case("pool", POOL, 15, 1, 1, 7, 7, 3, 2, 2);        // every window all-equal
    simple_case("pool", POOL, 16, 1, 1, 6, 6, 2, 2, 2);
    simple_case("softmax", SOFTMAX, 17, 4, 1000, 1, 1, 0, 0, 0);
    simple_case("softmax", SOFTMAX, 18, 3, 10, 1, 1, 0, 0, 0);

    fprintf(g_manifest, "\n]}\n");
    fclose(g_manifest);
    printf("ref_harness: wrote fixtures to %s\n", g_dir.c_str());
    return 0;
}
