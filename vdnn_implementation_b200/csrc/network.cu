// Network: topology tables, vDNN policy, forward / backward loops.
//
// What is kept from the reference (network.cu): the three topologies, the four policies
// (setVdnnType, 875-940), the prefetch choice (findPrefetchLayer, 1198-1207) and the host-side
// order of every pool allocation and release in the two loops (1056-1191), so that the placement
// and the pool's byte counts are the same.  What differs: the loops do not synchronise the host
// after every layer; offload (D2H) and prefetch (H2D) run on two dedicated streams ordered against
// the compute stream with events, and a released block carries the events that must complete
// before its bytes are reused.
#include "network.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "dp_nccl.h"
#include "dp_peer.h"

namespace vdnn { extern unsigned long long g_kernel_launches; }

#define NET_CU(call)                                                                      \
    do {                                                                                  \
        if (!ctx.dry_run && (call) != cudaSuccess) {                                      \
            fprintf(stderr, "CUDA failure at %s:%d: %s\n", __FILE__, __LINE__,            \
                    cudaGetErrorString(cudaGetLastError()));                              \
            return VDNN_ERR_CUDA;                                                         \
        }                                                                                 \
    } while (0)
#define NET_TRY(call) do { const int _s = (call); if (_s != 0) return _s; } while (0)

static const char* env_or(const char* name, const char* fallback) {
    const char* v = getenv(name);
    return (v && *v) ? v : fallback;
}

static int g_lean_offload_default = -1;      // -1: follow VDNN_LEAN_OFFLOAD in the environment
void Network::setLeanOffloadDefault(int on) { g_lean_offload_default = on < 0 ? -1 : (on != 0); }

/* ------------------------------------------------------------------ construction (network.cu:10-92) */

Network::Network(CNN_t _cnnType, vdnn_t _vdnnType, vdnnAlgoMode_t _algoMode, int _batchSize) {
    // The reference fixes these in vdnn.h:5-10 and network.cu:49; the environment may override them.
    vdnn_network_config cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.cnn_type = _cnnType; cfg.vdnn_type = _vdnnType; cfg.algo_mode = _algoMode;
    cfg.batch_size = (_batchSize == DEFAULT_BATCH_SIZE) ? 0 : _batchSize;
    cfg.device = atoi(env_or("VDNN_DEVICE", "0"));
    cfg.pool_bytes = strtoull(env_or("VDNN_POOL_BYTES", "0"), NULL, 10);
    cfg.learning_rate = static_cast<float>(atof(env_or("VDNN_LR", "0")));
    cfg.init_mode = atoi(env_or("VDNN_INIT_MODE", "1"));
    cfg.weight_seed_base = strtoull(env_or("VDNN_SEED", "3000"), NULL, 10);
    cfg.fix_input_leak = atoi(env_or("VDNN_FIX_INPUT_LEAK", "1"));
    cfg.host_sync_per_layer = atoi(env_or("VDNN_HOST_SYNC", "0"));
    cfg.verbose = atoi(env_or("VDNN_VERBOSE", "1"));
    init(cfg, false);
}

Network::Network(const vdnn_network_config& cfg, bool dry_run) { init(cfg, dry_run); }

Network::Network(const vdnn_network_config& cfg, bool dry_run, const std::vector<unsigned char>& ops) {
    layerOps = ops;
    ctx.quiet = true;
    init(cfg, dry_run);
}

/* ------------------------------------------------------------------ VDNN_DYNAMIC_ALGO (network.cu:946-1008) */

// The reference finds out whether a (policy, algorithm mode) pair fits by running a training iteration
// with soft allocation failures and rebuilding the whole network for the next candidate.  What decides is
// the pool's bookkeeping in host order, so the same question is answered here by replaying two iterations of
// the candidate against a bookkeeping-only pool of the same capacity: no kernel runs and nothing is allocated.
bool Network::trainable(const vdnn_network_config& cfg, vdnn_t type, vdnnAlgoMode_t algo,
                        const std::vector<unsigned char>* ops, size_t* peak) {
    vdnn_network_config c = cfg;
    c.vdnn_type = type; c.algo_mode = algo; c.device = -1; c.verbose = 0; c.capture = 0;
    static const std::vector<unsigned char> none;
    Network trial(c, true, ops ? *ops : none);
    if (trial.status() != VDNN_OK) return false;
    trial.context().trace_enabled = false;
    for (int it = 0; it < 2; ++it)
        if (trial.forwardPropagation(true) != 0 || trial.backwardPropagation(true) != 0) return false;
    if (peak) vdnnPoolHighWater(peak, 0);
    return true;
}

int Network::vdnnDynamicAlgo(const vdnn_network_config& cfg) {
    const bool say = cfg.verbose != 0;
    if (say) printf("\n1. Test VDNN_ALL and VDNN_MEMORY_OPT_ALGO\n");
    if (!trainable(cfg, VDNN_ALL, VDNN_MEMORY_OPT_ALGO, NULL)) {
        fprintf(stderr, "This CNN model cannot be trained\n");
        return VDNN_ERR_OUT_OF_MEMORY;
    }
    static const struct { vdnn_t type; const char* name; } order[3] = {
        {VDNN_NONE, "VDNN_NONE"}, {VDNN_CONV, "VDNN_CONV"}, {VDNN_ALL, "VDNN_ALL"}};
    for (int i = 0; i < 3; ++i) {
        if (say) printf("\n%d. Test %s and VDNN_PERF_OPT_ALGO\n", i + 2, order[i].name);
        if (trainable(cfg, order[i].type, VDNN_PERF_OPT_ALGO, NULL)) {
            if (say) printf("%s and VDNN_PERF_OPT_ALGO Passed!\n", order[i].name);
            vdnnType = order[i].type;
            algoMode = VDNN_PERF_OPT_ALGO;
            return VDNN_OK;
        }
    }
    // Per layer and operation under VDNN_ALL (layer.cu:1091-1147 tries each layer's algorithms from the fastest
    // down until the workspace can be had): starting from zero workspace everywhere, which step 1 showed to
    // fit, an operation moves to its workspace-using algorithm when the whole iteration still fits with it.
    if (say) printf("\n5. Dynamic Algorithm with VDNN_ALL\n");
    vdnn_network_config c = cfg;
    c.vdnn_type = VDNN_ALL; c.algo_mode = VDNN_MEMORY_OPT_ALGO; c.device = -1; c.verbose = 0; c.capture = 0;
    std::vector<unsigned char> ops;
    {
        Network shape(c, true, ops);
        if (shape.status() != VDNN_OK) return shape.status();
        ops.assign(shape.numLayers_(), 0);
        for (int l = 0; l < shape.numLayers_(); ++l) {
            const Layer_t t = shape.layerArray()[l]->LayerType();
            if (t != CONV && t != FC_CONV) ops[l] = 0x80;            // not a convolution: nothing to choose
        }
    }
    for (size_t l = 0; l < ops.size(); ++l) {
        if (ops[l] & 0x80) { ops[l] = 0; continue; }
        for (int op = 0; op < 3; ++op) {
            ops[l] |= static_cast<unsigned char>(1u << op);
            if (!trainable(cfg, VDNN_ALL, VDNN_MEMORY_OPT_ALGO, &ops)) ops[l] &= static_cast<unsigned char>(~(1u << op));
        }
    }
    vdnnType = VDNN_ALL;
    algoMode = VDNN_MEMORY_OPT_ALGO;
    dynamicPerLayer = true;
    layerOps = ops;
    return VDNN_OK;
}

void Network::selected(int* vdnn_type, int* algo) const {
    if (vdnn_type) *vdnn_type = vdnnType;
    if (algo) *algo = dynamicPerLayer ? VDNN_DYNAMIC_ALGO : algoMode;
}

int Network::layerAlgos(int layerId, int out3[3]) const {
    if (layerId < 0 || layerId >= numLayers || !out3) return VDNN_ERR_BAD_ARG;
    layer[layerId]->opAlgos(out3);
    return VDNN_OK;
}

void Network::init(const vdnn_network_config& cfg, bool dry_run) {
    cnnType = static_cast<CNN_t>(cfg.cnn_type);
    vdnnType = static_cast<vdnn_t>(cfg.vdnn_type);
    algoMode = static_cast<vdnnAlgoMode_t>(cfg.algo_mode);
    batchSize = cfg.batch_size;
    numLayers = 0; state = VDNN_OK; device = cfg.device; poolOwner = false;
    inputData = labelData = networkDiffData = networkGradData = workSpace = NULL;
    workSpaceBytes = dxdyBytes = 0;
    stream_compute = stream_memory = NULL;
    customLayers = cfg.custom_layers; numCustomLayers = cfg.num_custom_layers;
    externalInput = false; forwardDone = false; stepCounter = 0;
    stage_h = NULL; loss_h = NULL; ev_loss = NULL; ev_step_end = NULL;
    ev_fwd_t0 = ev_fwd_t1 = NULL; fwdTimed = false; fwdMsBest = 0.0f;
    launchesAtStepStart = launchesLastStep = 0;
    n_in = c_in = h_in = w_in = n_out = c_out = h_out = w_out = 0;
    for (int i = 0; i < DEFAULT_NUM_LAYER; i++) {
        layer[i] = NULL; isOffload[i] = false; isPrefetched[i] = false; offloadedSrcData_h[i] = NULL; leanDrop[i] = false;
    }
    lean = g_lean_offload_default >= 0 ? g_lean_offload_default != 0 : atoi(env_or("VDNN_LEAN_OFFLOAD", "0")) != 0;
    handle = &ctx;
    ctx.dry_run = dry_run;
    ctx.learning_rate = cfg.learning_rate > 0.0f ? cfg.learning_rate : static_cast<float>(LEARNING_RATE);
    ctx.init_mode = cfg.init_mode;
    ctx.weight_seed_base = cfg.weight_seed_base;
    ctx.verbose = cfg.verbose != 0;
    ctx.host_sync_per_layer = cfg.host_sync_per_layer != 0;
    ctx.capture = cfg.capture != 0;
    ctx.fix_input_leak = cfg.fix_input_leak != 0;

    if (vdnnPoolIsInitialized()) {
        fprintf(stderr, "a Network already owns the device pool of this process\n");
        state = VDNN_ERR_STATE;
        return;
    }

    dynamicPerLayer = false;
    packedPool = false;
    if (algoMode == VDNN_DYNAMIC_ALGO) {          // the given policy is ignored, as network.cu:60-78 does
        const int st = vdnnDynamicAlgo(cfg);
        if (st != VDNN_OK) { state = st; return; }
    }

    const size_t pool = cfg.pool_bytes ? cfg.pool_bytes : static_cast<size_t>(24e9);
    // How much room is there?  Placement by pending events, and offload copies held back until the end of
    // forward, buy overlap with bytes: they need a pool well above the schedule's peak.  The peak comes from a
    // replay on a bookkeeping-only pool; below 1.4 x peak (or when the replay does not fit) the pool is packed
    // tightest-fit and the copies go out in layer order, which is the placement the replay was made with.
    bool packed = false;
    if (!dry_run && vdnnType != BASELINE) {
        size_t peak = 0;
        const std::vector<unsigned char>* ops = layerOps.empty() ? NULL : &layerOps;
        const bool fits = trainable(cfg, vdnnType, algoMode, ops, &peak);
        packed = !fits || static_cast<double>(pool) < 1.4 * static_cast<double>(peak);
        if (getenv("VDNN_DEBUG_POOL"))
            fprintf(stderr, "[pool] capacity %zu, replayed peak %zu, replay fits %d -> %s placement\n", pool, peak, fits ? 1 : 0,
                    packed ? "packed" : "event-ranked");
    }
    if (dry_run) {
        if (vdnnPoolInitVirtual(pool) != CNMEM_STATUS_SUCCESS) { state = VDNN_ERR_OUT_OF_MEMORY; return; }
    } else {
        if (cudaSetDevice(device) != cudaSuccess || cudaFree(0) != cudaSuccess) {
            fprintf(stderr, "no usable CUDA device %d: %s\n", device, cudaGetErrorString(cudaGetLastError()));
            state = VDNN_ERR_CUDA;
            return;
        }
        // two streams as in network.cu:41-42, plus one for the H2D direction and one for collectives
        bool ok = cudaStreamCreateWithFlags(&stream_compute, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&stream_memory, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&ctx.stream_h2d, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&ctx.stream_comm, cudaStreamNonBlocking) == cudaSuccess;
        if (!ok) { state = VDNN_ERR_CUDA; return; }
        cudaStream_t streamArray[2] = {stream_compute, stream_memory};
        size_t streamSizes[2] = {0, 0};
        cnmemDevice_t cnmemDevice;
        cnmemDevice.device = device;
        cnmemDevice.size = pool;
        cnmemDevice.numStreams = 2;
        cnmemDevice.streams = streamArray;
        cnmemDevice.streamSizes = streamSizes;
        const cnmemStatus_t st = cnmemInit(1, &cnmemDevice, 0);
        if (st != CNMEM_STATUS_SUCCESS) {
            fprintf(stderr, "\n[pool reservation of %zu bytes failed with %s]\n", pool, cnmemGetErrorString(st));
            state = VDNN_ERR_OUT_OF_MEMORY;
            return;
        }
    }
    poolOwner = true;
    ctx.stream_compute = stream_compute;
    ctx.stream_d2h = stream_memory;

    // per-layer events; created before the layers because BASELINE layers allocate in their constructor
    if (!dry_run) {
        auto make = [&](std::vector<cudaEvent_t>& v, unsigned flags) {
            v.assign(DEFAULT_NUM_LAYER, NULL);
            for (auto& e : v) if (cudaEventCreateWithFlags(&e, flags) != cudaSuccess) state = VDNN_ERR_CUDA;
        };
        make(ctx.ev_fwd_done, cudaEventDisableTiming); make(ctx.ev_bwd_done, cudaEventDisableTiming);
        make(ctx.ev_offload_done, cudaEventDisableTiming); make(ctx.ev_prefetch_done, cudaEventDisableTiming);
        make(ctx.ev_weights_ready, cudaEventDisableTiming);
        if (cudaEventCreateWithFlags(&ctx.ev_input_ready, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&ev_loss, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&ev_step_end, cudaEventDisableTiming) != cudaSuccess)
            state = VDNN_ERR_CUDA;
        if (state != VDNN_OK) return;
        // Offload copies go out in the order backward needs them unless the reference's per-layer
        // synchronisation is asked for (then each copy is enqueued, and waited for, in its own layer).
        const char* order = getenv("VDNN_OFFLOAD_ORDER");
        ctx.defer_offloads = !packed && !ctx.host_sync_per_layer && !(order && strcmp(order, "forward") == 0);
        vdnnPoolSetPacked(packed ? 1 : 0);
        packedPool = packed;
        // How many bytes of the first layers leave in their own layer (under the forward kernels): a fixed figure from the
        // environment, else measured -- the forward pass's duration on the compute stream times the copy engine's rate.
        if (const char* eager = getenv("VDNN_EAGER_OFFLOAD_BYTES")) ctx.eager_offload_budget = strtoll(eager, NULL, 10);
        else if (ctx.defer_offloads) {
            ctx.eager_offload_auto = true;
            if (cudaEventCreate(&ev_fwd_t0) != cudaSuccess || cudaEventCreate(&ev_fwd_t1) != cudaSuccess) state = VDNN_ERR_CUDA;
        }
        vdnnPoolSetResolver([](void* user, unsigned long long token) {
            static_cast<vdnnContext*>(user)->flushOffloads(static_cast<int>(token) - 1);
        }, &ctx);
    }
    ctx.weights_pending.assign(DEFAULT_NUM_LAYER, 0);

    setLayers(cnnType);
    if (state != VDNN_OK) return;
    for (size_t l = 0; l < layerOps.size() && static_cast<int>(l) < numLayers; ++l) {
        const Layer_t t = layer[l]->LayerType();
        if (t != CONV && t != FC_CONV) continue;
        const bool use[3] = {(layerOps[l] & 1) != 0, (layerOps[l] & 2) != 0, (layerOps[l] & 4) != 0};
        layer[l]->setOpAlgos(use);
    }
    setVdnnType(vdnnType);
    // placement by pending events spreads the tensors over a roomy pool; the largest workspace keeps a range of its own
    if (!dry_run && !packedPool && vdnnType != BASELINE) vdnnPoolSetTransientReserve(static_cast<size_t>(ctx.workspace_bytes_max));
    if (state != VDNN_OK) return;

    /* input and label (network.cu:87-90) */
    if (ctx.alloc(&inputData, sizeof(DATATYPE) * getInputSize(), -1, TAG_INPUT, false, {}) != 0 ||
        ctx.alloc(&labelData, sizeof(DATATYPE) * getOutputSize(), -1, TAG_LABEL, false, {}) != 0) {
        state = VDNN_ERR_OUT_OF_MEMORY;
        return;
    }
    if (!dry_run) {
        const size_t stage = sizeof(float) * (static_cast<size_t>(getInputSize()) + getOutputSize());
        if (cudaMallocHost(reinterpret_cast<void**>(&stage_h), stage) != cudaSuccess ||
            cudaMallocHost(reinterpret_cast<void**>(&loss_h), 4 * sizeof(double)) != cudaSuccess)
            state = VDNN_ERR_CUDA;
        else
            memset(loss_h, 0, 4 * sizeof(double));      // [0..1] loss, [2] the engine's status word as published after backward
    }
    if (ctx.capture) { capDst.resize(numLayers); capGrad.resize(numLayers); }
}

Network::~Network() {
    if (!ctx.dry_run) cudaDeviceSynchronize();
    vdnn::dp_shutdown(&ctx);
    if (ctx.dp_arena) cudaFree(ctx.dp_arena);
    for (int i = 0; i < DEFAULT_NUM_LAYER; i++) {
        if (layer[i]) {
            delete layer[i];
        }
        if (offloadedSrcData_h[i]) cudaFreeHost(offloadedSrcData_h[i]);
    }
    if (poolOwner) cnmemFinalize();
    if (ctx.dry_run) return;
    auto drop = [](std::vector<cudaEvent_t>& v) { for (auto e : v) if (e) cudaEventDestroy(e); v.clear(); };
    drop(ctx.ev_fwd_done); drop(ctx.ev_bwd_done); drop(ctx.ev_offload_done); drop(ctx.ev_prefetch_done);
    drop(ctx.ev_weights_ready); drop(ctx.pf_fwd_beg); drop(ctx.pf_fwd_end); drop(ctx.pf_bwd_beg); drop(ctx.pf_bwd_end);
    drop(ctx.pf_off_beg); drop(ctx.pf_off_end); drop(ctx.pf_pre_beg); drop(ctx.pf_pre_end);
    if (ctx.ev_input_ready) cudaEventDestroy(ctx.ev_input_ready);
    for (auto& v : ctx.ev_offload_chunk) drop(v);
    if (ctx.pf_step_beg) cudaEventDestroy(ctx.pf_step_beg);
    if (ctx.pf_step_end) cudaEventDestroy(ctx.pf_step_end);
    if (ev_fwd_t0) cudaEventDestroy(ev_fwd_t0);
    if (ev_fwd_t1) cudaEventDestroy(ev_fwd_t1);
    if (ev_loss) cudaEventDestroy(ev_loss);
    if (ev_step_end) cudaEventDestroy(ev_step_end);
    if (stage_h) cudaFreeHost(stage_h);
    if (loss_h) cudaFreeHost(loss_h);
    if (stream_compute) cudaStreamDestroy(stream_compute);
    if (stream_memory) cudaStreamDestroy(stream_memory);
    if (ctx.stream_h2d) cudaStreamDestroy(ctx.stream_h2d);
    if (ctx.stream_comm) cudaStreamDestroy(ctx.stream_comm);
}

/* ------------------------------------------------------------------ topologies (network.cu:134-817) */

void Network::addLayer(Layer_t type, vdnnAlgoMode_t algo, int n, int c, int h, int w, int pad, int stride, int k, int r) {
    if (state != VDNN_OK) return;
    if (numLayers >= DEFAULT_NUM_LAYER) { state = VDNN_ERR_BAD_ARG; return; }
    const int id = numLayers;
    layer[id] = new Layer(vdnnType, algo, type, &handle, &stream_compute, &stream_memory, id,
                          n, c, h, w, pad, pad, stride, stride, k, r, r);
    if (!layer[id]->ok()) { state = VDNN_ERR_OUT_OF_MEMORY; return; }
    cur_n = layer[id]->OutputN(); cur_c = layer[id]->OutputC(); cur_h = layer[id]->OutputH(); cur_w = layer[id]->OutputW();
    numLayers++;
}

// The reference tags every convolution FC_CONV (e.g. network.cu:171-178), which is what VDNN_CONV
// and findPrefetchLayer test for.
void Network::convRelu(int pad, int stride, int k, int r, bool forceMemOpt) {
    addLayer(FC_CONV, forceMemOpt ? VDNN_MEMORY_OPT_ALGO : algoMode, cur_n, cur_c, cur_h, cur_w, pad, stride, k, r);
    addLayer(RELU, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 0, 0, 0);
}

void Network::fcRelu(int k) {
    addLayer(FC_GEMM, algoMode, cur_n, cur_c * cur_h * cur_w, 1, 1, 0, 0, k, 1);
    addLayer(RELU, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 0, 0, 0);
}

void Network::setLayers(CNN_t _cnnType) {
    cnnType = _cnnType;
    switch (_cnnType) {
    case ALEXNET: case ALEXNET_LRN: setLayersAlexnet(); break;
    case OVERFEAT: setLayersOverfeat(); break;
    case GOOGLENET: setLayersGooglenet(); break;
    case VGG16_64: setLayersVgg16(64); break;
    case VGG16_128: setLayersVgg16(128); break;
    case VGG16_256: setLayersVgg16(256); break;
    case CUSTOM_CNN: setLayersCustomCNN(); break;
    default: fprintf(stderr, "Invalid CNN Type!\n"); state = VDNN_ERR_BAD_ARG; return;
    }
    if (state != VDNN_OK) return;
    if (ctx.verbose) printf("-------------------------------------------------------\n\n");
    sanityCheck();
}

void Network::setLayersAlexnet() {          // network.cu:156-323; LRN layers only for ALEXNET_LRN
    if (batchSize <= 0) batchSize = DEFAULT_BATCH_SIZE;
    n_in = batchSize; c_in = 3; h_in = w_in = 227;
    n_out = batchSize; c_out = 1000; h_out = w_out = 1;
    cur_n = n_in; cur_c = c_in; cur_h = h_in; cur_w = w_in;
    const bool lrn = cnnType == ALEXNET_LRN;
    convRelu(0, 4, 96, 11);
    if (lrn) addLayer(LRN, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 0, 0, 5);
    addLayer(POOL, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 2, 0, 3);
    convRelu(2, 1, 256, 5);
    if (lrn) addLayer(LRN, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 0, 0, 5);
    addLayer(POOL, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 2, 0, 3);
    convRelu(1, 1, 384, 3);
    convRelu(1, 1, 384, 3);
    convRelu(1, 1, 256, 3);
    addLayer(POOL, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 2, 0, 3);
    fcRelu(4096);
    fcRelu(4096);
    addLayer(FC_GEMM, algoMode, cur_n, cur_c, 1, 1, 0, 0, 1000, 1);
    addLayer(SOFTMAX, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 0, 0, 0);
}

void Network::setLayersOverfeat() {         // network.cu:325-495
    if (batchSize <= 0) batchSize = DEFAULT_BATCH_SIZE;
    n_in = batchSize; c_in = 3; h_in = w_in = 231;
    n_out = batchSize; c_out = 1000; h_out = w_out = 1;
    cur_n = n_in; cur_c = c_in; cur_h = h_in; cur_w = w_in;
    convRelu(0, 4, 96, 11);
    addLayer(POOL, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 2, 0, 2);
    convRelu(0, 1, 256, 5);
    addLayer(POOL, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 2, 0, 2);
    convRelu(1, 1, 512, 3);
    convRelu(1, 1, 1024, 3);
    convRelu(1, 1, 1024, 3);
    addLayer(POOL, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 2, 0, 2);
    // the classifier is three convolutions pinned to the zero-workspace algorithm (network.cu:447-486)
    convRelu(0, 1, 3072, 6, true);
    convRelu(0, 1, 4096, 1, true);
    addLayer(FC_CONV, VDNN_MEMORY_OPT_ALGO, cur_n, cur_c, cur_h, cur_w, 0, 1, 1000, 1);
    addLayer(SOFTMAX, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 0, 0, 0);
}

void Network::setLayersGooglenet() {        // network.cu:497-499 is an empty stub
    fprintf(stderr, "GOOGLENET has no topology in this build (nor in the reference)\n");
    state = VDNN_ERR_UNSUPPORTED;
}

void Network::setLayersVgg16(int givenBatch) {      // network.cu:501-813
    if (batchSize <= 0) batchSize = givenBatch;
    n_in = batchSize; c_in = 3; h_in = w_in = 224;
    n_out = batchSize; c_out = 1000; h_out = w_out = 1;
    cur_n = n_in; cur_c = c_in; cur_h = h_in; cur_w = w_in;
    static const int width[5] = {64, 128, 256, 512, 512};
    static const int depth[5] = {2, 2, 3, 3, 3};
    for (int b = 0; b < 5; ++b) {
        for (int i = 0; i < depth[b]; ++i) convRelu(1, 1, width[b], 3);
        addLayer(POOL, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 2, 0, 2);
    }
    fcRelu(4096);
    fcRelu(4096);
    addLayer(FC_GEMM, algoMode, cur_n, cur_c, 1, 1, 0, 0, 1000, 1);
    addLayer(SOFTMAX, algoMode, cur_n, cur_c, cur_h, cur_w, 0, 0, 0, 0);
}

// network.cu:815-817 is empty; here the topology comes from the configuration's layer list.
void Network::setLayersCustomCNN() {
    if (!customLayers || numCustomLayers <= 0 || numCustomLayers > DEFAULT_NUM_LAYER) {
        fprintf(stderr, "CUSTOM_CNN needs a layer list\n");
        state = VDNN_ERR_BAD_ARG;
        return;
    }
    for (int i = 0; i < numCustomLayers && state == VDNN_OK; ++i) {
        const vdnn_layer_spec& s = customLayers[i];
        if (numLayers >= DEFAULT_NUM_LAYER) { state = VDNN_ERR_BAD_ARG; return; }
        layer[i] = new Layer(vdnnType, algoMode, static_cast<Layer_t>(s.type), &handle, &stream_compute, &stream_memory, i,
                             s.n, s.c, s.h, s.w, s.pad_h, s.pad_w, s.stride_h, s.stride_w, s.k, s.r, s.s);
        if (!layer[i]->ok()) { state = VDNN_ERR_BAD_ARG; return; }
        numLayers++;
    }
    if (state != VDNN_OK) return;
    n_in = layer[0]->InputN(); c_in = layer[0]->InputC(); h_in = layer[0]->InputH(); w_in = layer[0]->InputW();
    Layer* last = layer[numLayers - 1];
    n_out = last->OutputN(); c_out = last->OutputC(); h_out = last->OutputH(); w_out = last->OutputW();
    batchSize = n_in;
}

void Network::sanityCheck() {               // network.cu:831-873
    for (int i = 0; i < numLayers - 1 && state == VDNN_OK; i++) {
        bool check;
        if (layer[i + 1]->LayerType() == FC_GEMM)
            check = layer[i]->DstDataSize() == layer[i + 1]->SrcDataSize();
        else
            check = layer[i]->OutputN() == layer[i + 1]->InputN() && layer[i]->OutputC() == layer[i + 1]->InputC() &&
                    layer[i]->OutputH() == layer[i + 1]->InputH() && layer[i]->OutputW() == layer[i + 1]->InputW();
        if (!check) {
            fprintf(stderr, "Sanity check error at layer %d and %d!\n", i, i + 1);
            state = VDNN_ERR_BAD_ARG;
        }
    }
}

/* ------------------------------------------------------------------ policy (network.cu:875-940) */

void Network::setVdnnType(vdnn_t newVdnnType) {
    vdnnType = newVdnnType;
    for (int i = 0; i < DEFAULT_NUM_LAYER; i++) {
        isOffload[i] = false;
        isPrefetched[i] = false;
        leanDrop[i] = false;
        if (offloadedSrcData_h[i] != NULL) cudaFreeHost(offloadedSrcData_h[i]);
        offloadedSrcData_h[i] = NULL;
        if (layer[i] != NULL) layer[i]->setVdnnMode(newVdnnType);
    }
    ctx.pinned_bytes = 0;
    auto pin = [&](int l) {
        isOffload[l] = true;
        const size_t bytes = layer[l]->SrcDataSize() * sizeof(DATATYPE);
        ctx.pinned_bytes += static_cast<int64_t>(bytes);
        if (!ctx.dry_run && cudaMallocHost(reinterpret_cast<void**>(&offloadedSrcData_h[l]), bytes) != cudaSuccess) {
            fprintf(stderr, "pinning %zu bytes of host memory for layer %d failed\n", bytes, l);
            state = VDNN_ERR_OUT_OF_MEMORY;
        }
    };
    switch (newVdnnType) {
    case BASELINE: {
        dxdyBytes = findMaxDxDySize();
        if (ctx.alloc(&networkDiffData, dxdyBytes, -1, TAG_DXDY, false, {}) != 0 ||
            ctx.alloc(&networkGradData, dxdyBytes, -1, TAG_DXDY, false, {}) != 0) { state = VDNN_ERR_OUT_OF_MEMORY; return; }
        workSpaceBytes = findMaxWorkSpaceSize();
        ctx.shared_workspace_bytes = workSpaceBytes;
        if (workSpaceBytes > 0 && ctx.alloc(&workSpace, workSpaceBytes, -1, TAG_WS, false, {}) != 0) state = VDNN_ERR_OUT_OF_MEMORY;
    } break;
    case VDNN_NONE: break;
    case VDNN_ALL:
        for (int l = 0; l < numLayers - 1 && state == VDNN_OK; l++) {
            const Layer_t below = l > 0 ? layer[l - 1]->LayerType() : RELU;
            if (lean && layer[l]->LayerType() == RELU && (below == CONV || below == FC_CONV || below == FC_GEMM)) leanDrop[l] = true;
            else pin(l);
        }
        break;
    case VDNN_CONV:
        for (int l = 0; l < numLayers - 1 && state == VDNN_OK; l++)
            if (layer[l]->LayerType() == FC_CONV || layer[l]->LayerType() == CONV) pin(l);
        break;
    }
    for (int l = 0; l < numLayers; l++) {
        const size_t m = std::max(layer[l]->FwdWorkSpaceSize(), std::max(layer[l]->BwdDataWorkSpaceSize(), layer[l]->BwdFilterWorkSpaceSize()));
        if (static_cast<int64_t>(m) > ctx.workspace_bytes_max) ctx.workspace_bytes_max = static_cast<int64_t>(m);
    }
}

// network.cu:1010-1023 (bytes).  The reference returns an int, which wraps for VGG16_256 (822 M elements
// x 4 bytes) and makes its BASELINE allocation fail; the byte count is kept in 64 bits here.
size_t Network::findMaxDxDySize() {
    int ret = 0;
    for (int i = 0; i < numLayers; i++) ret = std::max(ret, layer[i]->SrcDataSize());
    ret = std::max(ret, layer[numLayers - 1]->DstDataSize());
    return static_cast<size_t>(ret) * sizeof(DATATYPE);
}

// network.cu:1025-1040 keeps this maximum in an int.  cuDNN's workspaces of a few GB then wrap and the shared block
// comes out too small; this library's own workspaces (operand images of the large layers) pass 2^31 bytes as well,
// and a kernel writing them into a wrapped-size block would overrun it.  The maximum is therefore kept in 64 bits,
// and BASELINE hands the shared block's true size to every call so that the size check of the C ABI is real.
size_t Network::findMaxWorkSpaceSize() {
    size_t ret = 0;
    for (int i = 0; i < numLayers; i++)
        if (layer[i]->LayerType() == FC_CONV || layer[i]->LayerType() == CONV)
            ret = std::max(ret, std::max(layer[i]->FwdWorkSpaceSize(),
                                         std::max(layer[i]->BwdDataWorkSpaceSize(), layer[i]->BwdFilterWorkSpaceSize())));
    return ret;
}

void Network::resetIsPrefetchedArray() {
    for (int i = 0; i < DEFAULT_NUM_LAYER; i++) isPrefetched[i] = false;
}

int Network::findPrefetchLayer(int currLayerId) {       // network.cu:1198-1207
    for (int id = currLayerId - 1; id >= 0; id--) {
        if (isOffload[id] && !isPrefetched[id]) { isPrefetched[id] = true; return id; }
        if (layer[id]->LayerType() == FC_CONV || layer[id]->LayerType() == CONV) return -1;
    }
    return -1;
}

/* ------------------------------------------------------------------ data in */

int Network::setInput(const float* input_h, const float* label_h) {
    if (state != VDNN_OK) return state;
    if (!input_h || !label_h) return VDNN_ERR_BAD_ARG;
    externalInput = true;
    if (ctx.dry_run) return VDNN_OK;
    NET_CU(cudaMemcpyAsync(inputData, input_h, sizeof(float) * getInputSize(), cudaMemcpyHostToDevice, stream_compute));
    NET_CU(cudaMemcpyAsync(labelData, label_h, sizeof(float) * getOutputSize(), cudaMemcpyHostToDevice, stream_compute));
    NET_CU(cudaEventRecord(ctx.ev_input_ready, stream_compute));
    return VDNN_OK;
}

int Network::seedInput(uint64_t input_seed, uint64_t label_seed) {
    if (state != VDNN_OK) return state;
    if (ctx.dry_run) { externalInput = true; return VDNN_OK; }
    NET_CU(cudaStreamSynchronize(stream_compute));          // stage_h may still be in flight
    float* in = stage_h;
    float* lab = stage_h + getInputSize();
    vdnn_host_fill_normal(in, getInputSize(), input_seed, 0.0f, 1.0f);
    vdnn_host_fill_onehot(lab, n_out, c_out * h_out * w_out, label_seed);
    return setInput(in, lab);
}

// network.cu:819-829 fills a device buffer with U(-0.01, 0.01) from an unseeded generator; the
// seeded equivalent is used when the caller supplied no batch.
void Network::randomInitializeData(void* data, int size) {
    if (ctx.dry_run) return;
    cudaStreamSynchronize(stream_compute);
    vdnn_host_fill_uniform(stage_h, size, 1000 + stepCounter * 2 + (data == labelData ? 1 : 0),
                           -(float)RANDOM_VALUE_LIMIT, (float)RANDOM_VALUE_LIMIT);
    cudaMemcpyAsync(data, stage_h, sizeof(float) * size, cudaMemcpyHostToDevice, stream_compute);
    cudaStreamSynchronize(stream_compute);
}

void Network::calculateFirstDiffData(void* result, void* first, void* second) {     // network.cu:1042-1054
    if (!externalInput) randomInitializeData(labelData, getOutputSize());
    if (!ctx.dry_run) vdnn_sub(getOutputSize(), (const float*)first, (const float*)second, (float*)result, stream_compute);
}

int Network::captureTensor(std::vector<float>& dst, const void* src, size_t count) {
    if (ctx.dry_run) return VDNN_OK;
    dst.resize(count);
    NET_CU(cudaStreamSynchronize(stream_compute));
    NET_CU(cudaMemcpy(dst.data(), src, count * sizeof(float), cudaMemcpyDeviceToHost));
    return VDNN_OK;
}

void Network::memoryLine(const char* phase, int l, size_t extra) {
    if (!ctx.verbose) return;
    size_t free_b = 0, total_b = 0;
    cnmemMemGetInfo(&free_b, &total_b, NULL);
    printf("[%s] Layer %d, Free Memory: %lu, Total Memory: %lu, Memory Usage: %lu\n", phase, l,
           (unsigned long)free_b, (unsigned long)total_b, (unsigned long)(total_b - free_b + extra));
}

/* ------------------------------------------------------------------ forward (network.cu:1056-1110) */

int Network::forwardPropagation(bool isDynamic) {
    if (state != VDNN_OK) return state;
    launchesAtStepStart = vdnn::g_kernel_launches;
    ctx.offload_bytes = 0;
    if (!externalInput) {
        randomInitializeData(inputData, getInputSize());
        if (!ctx.dry_run) NET_CU(cudaEventRecord(ctx.ev_input_ready, stream_compute));
    }
    if (ctx.profiling) NET_CU(cudaEventRecord(ctx.pf_step_beg, stream_compute));
    ctx.eager_offload_used = 0;
    ctx.forced_offloads = 0;
    if (ctx.eager_offload_auto && !ctx.dry_run) {
        // the last measured forward pass (if its events have completed) sets this pass's budget; the shortest one counts,
        // since a pass that waited for copies says nothing about the time the kernels give the copy engine
        float ms = 0.0f;
        if (fwdTimed && cudaEventElapsedTime(&ms, ev_fwd_t0, ev_fwd_t1) == cudaSuccess && ms > 0.0f) {
            if (fwdMsBest <= 0.0f || ms < fwdMsBest) fwdMsBest = ms;
            ctx.eager_offload_budget = static_cast<int64_t>(fwdMsBest * 1e-3 * EAGER_OFFLOAD_RATE);
        }
        (void)cudaGetLastError();
        NET_CU(cudaEventRecord(ev_fwd_t0, stream_compute));
    }

    for (int l = 0; l < numLayers; l++) {
        layer[l]->copySrcData(l == 0 ? inputData : layer[l - 1]->DstData());
        if (ctx.weights_pending[l]) {           // data parallel: last step's update of this layer
            NET_CU(cudaStreamWaitEvent(stream_compute, ctx.ev_weights_ready[l], 0));
            ctx.weights_pending[l] = 0;
        }
        NET_TRY(layer[l]->forward(isOffload, offloadedSrcData_h, workSpace, isDynamic));
        if (ctx.profiling) NET_CU(cudaEventRecord(ctx.pf_fwd_end[l], stream_compute));

        if (vdnnType != BASELINE) {
            if (ctx.host_sync_per_layer) {       // the reference's schedule (network.cu:1090-1091)
                NET_CU(cudaStreamSynchronize(stream_compute));
                NET_CU(cudaStreamSynchronize(stream_memory));
            }
            /* Release srcData of this layer (network.cu:1094-1095); the block stays fenced until the
               copy and the kernels that read it have finished */
            if (l != 0 && isOffload[l]) {
                if (ctx.offloadPending(l))
                    NET_TRY(ctx.releaseHeld(layer[l]->SrcData(), sizeof(DATATYPE) * layer[l]->SrcDataSize(), l, TAG_SRC,
                                            {stream_compute}));
                else
                    NET_TRY(ctx.release(layer[l]->SrcData(), sizeof(DATATYPE) * layer[l]->SrcDataSize(), l, TAG_SRC,
                                        {stream_memory, stream_compute}));
            } else if (leanDrop[l]) {            // lean VDNN_ALL: nobody reads this tensor again
                NET_TRY(ctx.release(layer[l]->SrcData(), sizeof(DATATYPE) * layer[l]->SrcDataSize(), l, TAG_SRC, {stream_compute}));
            }
        }
        if (ctx.capture) NET_TRY(captureTensor(capDst[l], layer[l]->DstData(), layer[l]->DstDataSize()));
        ctx.record(4, l, TAG_NONE, 0);
        memoryLine("Fwd", l, layer[l]->FwdWorkSpaceSize());
    }
    if (ctx.eager_offload_auto && !ctx.dry_run) { NET_CU(cudaEventRecord(ev_fwd_t1, stream_compute)); fwdTimed = true; }
    if (!ctx.dry_run) NET_TRY(ctx.flushOffloads(-1));
    if (!ctx.dry_run && externalInput) {
        NET_TRY(vdnn_loss(n_out, c_out * h_out * w_out, (const float*)layer[numLayers - 1]->DstData(),
                          (const float*)labelData, loss_h, stream_compute));
        NET_CU(cudaEventRecord(ev_loss, stream_compute));
    }
    forwardDone = true;
    return 0;
}

/* ------------------------------------------------------------------ backward (network.cu:1112-1191) */

int Network::reduceAndApply(int l) {
    if (ctx.dp_world <= 1 || !layer[l]->GradFilter()) return VDNN_OK;
    Layer* L = layer[l];
    const size_t wn = L->FilterDataSize(), bn = L->OutputC();
    NET_CU(cudaStreamWaitEvent(ctx.stream_comm, ctx.ev_bwd_done[l], 0));
    const float lr = ctx.learning_rate * -1.0f;
    if (ctx.dp_fused) {
        // reduce-scatter by peer loads, all-gather by peer stores and the SGD step in one kernel (csrc/dp_peer.cu);
        // its status word sits beside the engine's (read by synchronize())
        NET_TRY(vdnn::dp_peer_allreduce_sgd(ctx.dp_peer, ctx.dp_world, ctx.dp_rank, dpOffset[l], wn + bn, l,
                                            static_cast<unsigned>(stepCounter + 1), lr, (float*)L->FilterData(), wn,
                                            (float*)L->BiasData(), reinterpret_cast<int*>(loss_h + 3), ctx.stream_comm));
        NET_CU(cudaEventRecord(ctx.ev_weights_ready[l], ctx.stream_comm));
        ctx.weights_pending[l] = 1;
        return VDNN_OK;
    }
    NET_TRY(vdnn::dp_allreduce_sum(&ctx, L->GradFilter(), wn + bn, ctx.stream_comm));
    NET_TRY(vdnn_axpy(wn, lr, L->GradFilter(), (float*)L->FilterData(), ctx.stream_comm));
    NET_TRY(vdnn_axpy(bn, lr, L->GradBias(), (float*)L->BiasData(), ctx.stream_comm));
    NET_CU(cudaEventRecord(ctx.ev_weights_ready[l], ctx.stream_comm));
    ctx.weights_pending[l] = 1;
    return VDNN_OK;
}

int Network::backwardPropagation(bool isDynamic) {
    if (state != VDNN_OK) return state;
    if (!forwardDone) return VDNN_ERR_STATE;
    ctx.prefetch_bytes = 0;
    const int last = numLayers - 1;

    if (vdnnType == BASELINE) {
        calculateFirstDiffData(networkDiffData, layer[last]->DstData(), labelData);
        for (int l = last; l >= 0; l--) {
            if (l == last) { layer[l]->copyDiffData(networkDiffData); layer[l]->copyGradData(networkGradData); }
            else { layer[l]->copyDiffData(layer[l + 1]->GradData()); layer[l]->copyGradData(layer[l + 1]->DiffData()); }
            NET_TRY(layer[l]->backward(-1, NULL, NULL, 0, workSpace, isDynamic));
            if (ctx.profiling) NET_CU(cudaEventRecord(ctx.pf_bwd_end[l], stream_compute));
            NET_TRY(reduceAndApply(l));
            if (ctx.capture) NET_TRY(captureTensor(capGrad[l], layer[l]->GradData(), layer[l]->SrcDataSize()));
            ctx.record(5, l, TAG_NONE, 0);
            memoryLine("Bwd", l, layer[l]->BwdDataWorkSpaceSize() + layer[l]->BwdFilterWorkSpaceSize());
        }
    } else {
        resetIsPrefetchedArray();
        NET_TRY(layer[last]->cnmemMallocDiffData(isDynamic));
        calculateFirstDiffData(layer[last]->DiffData(), layer[last]->DstData(), labelData);
        void* supersededInput = NULL;

        for (int l = last; l >= 0; l--) {
            if (l != last) {
                layer[l]->copyDiffData(layer[l + 1]->GradData());
                layer[l]->copyDstData(layer[l + 1]->SrcData());
            }
            if (leanDrop[l]) layer[l]->copySrcData(layer[l]->DstData());       // ReLU mask from y: y > 0 exactly where x > 0
            // this layer reads its own srcData: if that came back from the host, wait for the copy
            if (isOffload[l] && isPrefetched[l] && !ctx.dry_run)
                NET_CU(cudaStreamWaitEvent(stream_compute, ctx.ev_prefetch_done[l], 0));

            const int prefId = l > 0 ? findPrefetchLayer(l) : -1;
            if (prefId >= 0) {
                if (prefId == 0) supersededInput = layer[0]->SrcData();
                NET_TRY(layer[prefId]->cnmemMallocSrcData(isDynamic));
                NET_TRY(layer[l]->backward(prefId, offloadedSrcData_h[prefId], layer[prefId]->SrcData(),
                                           sizeof(DATATYPE) * layer[prefId]->SrcDataSize(), workSpace, isDynamic));
            } else {
                NET_TRY(layer[l]->backward(-1, NULL, NULL, 0, workSpace, isDynamic));
            }
            if (ctx.profiling) NET_CU(cudaEventRecord(ctx.pf_bwd_end[l], stream_compute));
            NET_TRY(reduceAndApply(l));

            if (ctx.host_sync_per_layer) {       // network.cu:1168-1169
                NET_CU(cudaStreamSynchronize(stream_compute));
                NET_CU(cudaStreamSynchronize(stream_memory));
                NET_CU(cudaStreamSynchronize(ctx.stream_h2d));
            }
            if (ctx.capture) NET_TRY(captureTensor(capGrad[l], layer[l]->GradData(), layer[l]->SrcDataSize()));

            /* Release dstData and diffData (network.cu:1172-1173) */
            if (l == last || !leanDrop[l + 1])      // a dropped tensor went back to the pool in forward
                NET_TRY(ctx.release(layer[l]->DstData(), sizeof(DATATYPE) * layer[l]->DstDataSize(), l, TAG_DST, {stream_compute}));
            NET_TRY(ctx.release(layer[l]->DiffData(), sizeof(DATATYPE) * layer[l]->DstDataSize(), l, TAG_DIFF, {stream_compute}));
            ctx.record(5, l, TAG_NONE, 0);
            memoryLine("Bwd", l, layer[l]->BwdDataWorkSpaceSize() + layer[l]->BwdFilterWorkSpaceSize());
        }
        NET_TRY(ctx.release(layer[0]->GradData(), sizeof(DATATYPE) * layer[0]->SrcDataSize(), 0, TAG_GRAD, {stream_compute}));
        // network.cu:1185 adopts the prefetched copy of layer 0 as the new input and forgets the old
        // buffer; unless that leak is asked for, the old buffer goes back to the pool here.
        if (supersededInput && ctx.fix_input_leak)
            NET_TRY(ctx.release(supersededInput, sizeof(DATATYPE) * getInputSize(), -1, TAG_INPUT,
                                {stream_compute, stream_memory}));
        inputData = layer[0]->SrcData();
        // The adopted buffer was filled by the prefetch stream; backward of layer 0 waited for that copy on
        // the compute stream, so "input ready" is now: the next forward's offload of layer 0 must not read it earlier.
        if (!ctx.dry_run) NET_CU(cudaEventRecord(ctx.ev_input_ready, stream_compute));
    }
    if (ctx.profiling) NET_CU(cudaEventRecord(ctx.pf_step_end, stream_compute));
    // the tensor-core engine's status word, as it stands behind this step's kernels, goes to pinned host memory
    if (!ctx.dry_run) NET_TRY(vdnn_engine_status_publish(reinterpret_cast<int*>(loss_h + 2), stream_compute));
    if (!ctx.dry_run) NET_CU(cudaEventRecord(ev_step_end, stream_compute));
    launchesLastStep = vdnn::g_kernel_launches - launchesAtStepStart;
    forwardDone = false;
    stepCounter++;
    return 0;
}

/* ------------------------------------------------------------------ results and statistics */

int Network::synchronize() {
    if (ctx.dry_run) return VDNN_OK;
    NET_CU(cudaStreamSynchronize(stream_compute));
    NET_CU(cudaStreamSynchronize(stream_memory));
    NET_CU(cudaStreamSynchronize(ctx.stream_h2d));
    NET_CU(cudaStreamSynchronize(ctx.stream_comm));
    // a bounded wait that ran out inside a contraction kernel left output tiles unwritten: the steps since are void
    if (loss_h && (*reinterpret_cast<volatile int*>(loss_h + 2) != 0 || *reinterpret_cast<volatile int*>(loss_h + 3) != 0))
        return VDNN_ERR_TIMEOUT;
    return VDNN_OK;
}

// Device-side join: the compute stream waits for the tails of the copy and collective streams.
int Network::join() {
    if (ctx.dry_run) return VDNN_OK;
    cudaStream_t others[3] = {stream_memory, ctx.stream_h2d, ctx.stream_comm};
    for (cudaStream_t s : others) {
        NET_CU(cudaEventRecord(ev_step_end, s));
        NET_CU(cudaStreamWaitEvent(stream_compute, ev_step_end, 0));
    }
    return VDNN_OK;
}

int Network::loss(double* out2) {
    if (!out2) return VDNN_ERR_BAD_ARG;
    if (ctx.dry_run) { out2[0] = out2[1] = 0.0; return VDNN_OK; }
    NET_CU(cudaEventSynchronize(ev_loss));
    out2[0] = loss_h[0]; out2[1] = loss_h[1];
    return VDNN_OK;
}

size_t Network::tensorSize(int l, int kind) {
    if (l < 0 || l >= numLayers) return 0;
    Layer* L = layer[l];
    switch (kind) {
    case VDNN_TENSOR_DST: return L->DstDataSize();
    case VDNN_TENSOR_GRAD: return L->SrcDataSize();
    case VDNN_TENSOR_WEIGHT: return L->HasWeights() ? L->FilterDataSize() : 0;
    case VDNN_TENSOR_BIAS: return L->HasWeights() ? L->OutputC() : 0;
    default: return 0;
    }
}

int Network::readTensor(int l, int kind, float* dst_h, size_t count) {
    if (!dst_h || count != tensorSize(l, kind) || count == 0) return VDNN_ERR_BAD_ARG;
    if (ctx.dry_run) return VDNN_ERR_STATE;
    if (kind == VDNN_TENSOR_DST || kind == VDNN_TENSOR_GRAD) {
        if (!ctx.capture) return VDNN_ERR_STATE;
        const std::vector<float>& v = kind == VDNN_TENSOR_DST ? capDst[l] : capGrad[l];
        if (v.size() != count) return VDNN_ERR_STATE;
        memcpy(dst_h, v.data(), count * sizeof(float));
        return VDNN_OK;
    }
    NET_TRY(synchronize());
    const void* src = kind == VDNN_TENSOR_WEIGHT ? layer[l]->FilterData() : layer[l]->BiasData();
    NET_CU(cudaMemcpy(dst_h, src, count * sizeof(float), cudaMemcpyDeviceToHost));
    return VDNN_OK;
}

int Network::writeTensor(int l, int kind, const float* src_h, size_t count) {
    if (!src_h || count != tensorSize(l, kind) || count == 0) return VDNN_ERR_BAD_ARG;
    if (kind != VDNN_TENSOR_WEIGHT && kind != VDNN_TENSOR_BIAS) return VDNN_ERR_BAD_ARG;
    if (ctx.dry_run) return VDNN_ERR_STATE;
    NET_TRY(synchronize());
    void* dst = kind == VDNN_TENSOR_WEIGHT ? layer[l]->FilterData() : layer[l]->BiasData();
    NET_CU(cudaMemcpy(dst, src_h, count * sizeof(float), cudaMemcpyHostToDevice));
    return VDNN_OK;
}

int Network::setOffloadOrder(bool forwardOrder) {
    if (state != VDNN_OK) return state;
    ctx.defer_offloads = !forwardOrder && !ctx.host_sync_per_layer && !ctx.dry_run && !packedPool;
    if (!ctx.defer_offloads) { ctx.eager_offload_auto = false; ctx.eager_offload_budget = 0; }
    return VDNN_OK;
}

int Network::setProfiling(bool enabled) {
    if (ctx.dry_run) return VDNN_OK;
    if (enabled && ctx.pf_fwd_beg.empty()) {
        auto make = [&](std::vector<cudaEvent_t>& v) {
            v.assign(DEFAULT_NUM_LAYER, NULL);
            for (auto& e : v) if (cudaEventCreate(&e) != cudaSuccess) return false;
            return true;
        };
        if (!make(ctx.pf_fwd_beg) || !make(ctx.pf_fwd_end) || !make(ctx.pf_bwd_beg) || !make(ctx.pf_bwd_end) ||
            !make(ctx.pf_off_beg) || !make(ctx.pf_off_end) || !make(ctx.pf_pre_beg) || !make(ctx.pf_pre_end) ||
            cudaEventCreate(&ctx.pf_step_beg) != cudaSuccess || cudaEventCreate(&ctx.pf_step_end) != cudaSuccess)
            return VDNN_ERR_CUDA;
    }
    ctx.profiling = enabled;
    return VDNN_OK;
}

int Network::getStats(vdnn_network_stats* out) {
    if (!out) return VDNN_ERR_BAD_ARG;
    memset(out, 0, sizeof *out);
    size_t free_b = 0, total_b = 0, peak = 0;
    cnmemMemGetInfo(&free_b, &total_b, NULL);
    vdnnPoolHighWater(&peak, 0);
    out->pool_peak_bytes = static_cast<int64_t>(peak);
    out->pool_used_bytes = static_cast<int64_t>(total_b - free_b);
    out->pool_capacity_bytes = static_cast<int64_t>(total_b);
    out->pinned_bytes = ctx.pinned_bytes;
    out->offload_bytes = ctx.offload_bytes;
    out->prefetch_bytes = ctx.prefetch_bytes;
    out->workspace_bytes_max = ctx.workspace_bytes_max;
    out->kernel_launches = static_cast<int>(launchesLastStep);
    out->forced_offloads = ctx.forced_offloads;
    for (int l = 0; l < numLayers; ++l)
        if (layer[l]->GradFilter()) out->grad_buffer_bytes += static_cast<int64_t>(sizeof(float)) * (tensorSize(l, VDNN_TENSOR_WEIGHT) + tensorSize(l, VDNN_TENSOR_BIAS));
    for (int l = 0; l < numLayers; ++l) {
        Layer* L = layer[l];
        const double src = L->SrcDataSize(), dst = L->DstDataSize();
        switch (L->LayerType()) {
        case FC_GEMM: case CONV: case FC_CONV:
            // forward, data gradient and filter gradient are each one M x N x K contraction
            out->contraction_flops += 3.0 * 2.0 * dst * (static_cast<double>(L->FilterDataSize()) / L->OutputC());
            break;
        case RELU: case TANH: case SIGMOID: out->elementwise_bytes += 4.0 * (2.0 * src + 3.0 * src); break;   // fwd r+w, bwd x (or y),dy -> dx
        case POOL: out->elementwise_bytes += 4.0 * ((src + dst) + (2.0 * src + dst)); break;
        case LRN: out->elementwise_bytes += 4.0 * (2.0 * src + 4.0 * src); break;
        case SOFTMAX: out->elementwise_bytes += 4.0 * (2.0 * src + 3.0 * src); break;
        default: break;
        }
    }
    if (!ctx.profiling || ctx.dry_run || stepCounter == 0) return VDNN_OK;
    NET_TRY(synchronize());
    // interval lists relative to the step's first event
    struct Iv { float a, b; };
    std::vector<Iv> compute, copies;
    auto at = [&](cudaEvent_t e, float* ms) { return cudaEventElapsedTime(ms, ctx.pf_step_beg, e) == cudaSuccess; };
    float t_end = 0.0f;
    if (at(ctx.pf_step_end, &t_end)) out->step_ms = t_end;
    for (int l = 0; l < numLayers; ++l) {
        Iv f, b;
        float* bucket = layer[l]->HasWeights() ? &out->contraction_ms : &out->elementwise_ms;
        if (at(ctx.pf_fwd_beg[l], &f.a) && at(ctx.pf_fwd_end[l], &f.b)) { compute.push_back(f); *bucket += f.b - f.a; }
        if (at(ctx.pf_bwd_beg[l], &b.a) && at(ctx.pf_bwd_end[l], &b.b)) { compute.push_back(b); *bucket += b.b - b.a; }
        if (isOffload[l]) {
            Iv o, p;
            if (at(ctx.pf_off_beg[l], &o.a) && at(ctx.pf_off_end[l], &o.b)) { copies.push_back(o); out->offload_ms += o.b - o.a; }
            if (at(ctx.pf_pre_beg[l], &p.a) && at(ctx.pf_pre_end[l], &p.b)) { copies.push_back(p); out->prefetch_ms += p.b - p.a; }
        }
    }
    (void)cudaGetLastError();
    for (const Iv& c : copies)
        for (const Iv& k : compute) {
            const float lo = std::max(c.a, k.a), hi = std::min(c.b, k.b);
            if (hi > lo) out->copy_overlap_ms += hi - lo;
        }
    return VDNN_OK;
}

int Network::timeline(float* out) {
    if (!out) return VDNN_ERR_BAD_ARG;
    for (int i = 0; i < 8 * numLayers; ++i) out[i] = -1.0f;
    if (!ctx.profiling || ctx.dry_run || stepCounter == 0) return VDNN_ERR_STATE;
    NET_TRY(synchronize());
    for (int l = 0; l < numLayers; ++l) {
        cudaEvent_t ev[8] = {ctx.pf_fwd_beg[l], ctx.pf_fwd_end[l], isOffload[l] ? ctx.pf_off_beg[l] : NULL,
                             isOffload[l] ? ctx.pf_off_end[l] : NULL, ctx.pf_bwd_beg[l], ctx.pf_bwd_end[l],
                             isOffload[l] ? ctx.pf_pre_beg[l] : NULL, isOffload[l] ? ctx.pf_pre_end[l] : NULL};
        for (int j = 0; j < 8; ++j) {
            float ms = 0.0f;
            if (ev[j] && cudaEventElapsedTime(&ms, ctx.pf_step_beg, ev[j]) == cudaSuccess) out[8 * l + j] = ms;
        }
    }
    (void)cudaGetLastError();
    return VDNN_OK;
}

int Network::enableDataParallel(int rank, int world, const char* unique_id128) {
    if (state != VDNN_OK) return state;
    if (world < 1 || rank < 0 || rank >= world) return VDNN_ERR_BAD_ARG;
    if (world == 1) return VDNN_OK;
    if (ctx.dry_run) { ctx.dp_rank = rank; ctx.dp_world = world; return VDNN_OK; }
    NET_TRY(vdnn::dp_init(&ctx, rank, world, unique_id128));
    // one arena: the flag words of the fused all-reduce, then every layer's staging buffer (filter gradient followed by
    // bias gradient, so that one collective covers both), each starting on a 128-byte boundary
    size_t floats = vdnn::DP_FLAG_WORDS;
    dpOffset.assign(numLayers, 0);
    for (int l = 0; l < numLayers; ++l) {
        if (!layer[l]->HasWeights()) continue;
        dpOffset[l] = floats;
        floats += (static_cast<size_t>(layer[l]->FilterDataSize()) + layer[l]->OutputC() + 31) / 32 * 32;
    }
    NET_CU(cudaMalloc(reinterpret_cast<void**>(&ctx.dp_arena), floats * sizeof(float)));
    NET_CU(cudaMemset(ctx.dp_arena, 0, floats * sizeof(float)));
    ctx.dp_arena_floats = floats;
    for (int l = 0; l < numLayers; ++l)
        if (layer[l]->HasWeights()) layer[l]->setGradientStaging(ctx.dp_arena + dpOffset[l]);
    // VDNN_DP_FUSED=1: all-reduce and SGD step in one kernel over peer-mapped arenas instead of NCCL + axpy.  Needs every
    // rank's arena mapped here; when that fails on any rank the NCCL path stays in charge on this rank, so the ranks
    // must agree: the outcome is reduced (a 1-float NCCL all-reduce of "I can") before the mode is switched.
    const char* fused = getenv("VDNN_DP_FUSED");
    if (fused && *fused && *fused != '0' && world <= vdnn::DP_MAX_RANKS && numLayers <= vdnn::DP_MAX_LAYERS) {
        const int mapped = vdnn::dp_map_peers(&ctx, ctx.stream_comm);
        float* vote = ctx.dp_arena + vdnn::DP_FLAG_WORDS - 1;           // last flag word is unused by the kernels
        const float mine = mapped == VDNN_OK ? 1.0f : 0.0f;
        NET_CU(cudaMemcpyAsync(vote, &mine, sizeof(float), cudaMemcpyHostToDevice, ctx.stream_comm));
        NET_TRY(vdnn::dp_allreduce_sum(&ctx, vote, 1, ctx.stream_comm));
        float sum = 0.0f;
        NET_CU(cudaMemcpyAsync(&sum, vote, sizeof(float), cudaMemcpyDeviceToHost, ctx.stream_comm));
        NET_CU(cudaStreamSynchronize(ctx.stream_comm));
        NET_CU(cudaMemsetAsync(vote, 0, sizeof(float), ctx.stream_comm));
        ctx.dp_fused = sum > world - 0.5f;
        if (!ctx.dp_fused && ctx.verbose) fprintf(stderr, "fused peer all-reduce unavailable (%g of %d ranks could map their peers): using NCCL\n", sum, world);
    }
    return VDNN_OK;
}

int Network::dpMode() const { return ctx.dp_world <= 1 ? 0 : (ctx.dp_fused ? 2 : 1); }

int Network::weightChecksum(uint64_t* out) {
    if (!out) return VDNN_ERR_BAD_ARG;
    if (ctx.dry_run) return VDNN_ERR_STATE;
    NET_TRY(synchronize());
    uint64_t h = 1469598103934665603ull;
    std::vector<uint32_t> buf;
    for (int l = 0; l < numLayers; ++l) {
        if (!layer[l]->HasWeights()) continue;
        for (int kind = VDNN_TENSOR_WEIGHT; kind <= VDNN_TENSOR_BIAS; ++kind) {
            const size_t n = tensorSize(l, kind);
            buf.resize(n);
            const void* src = kind == VDNN_TENSOR_WEIGHT ? layer[l]->FilterData() : layer[l]->BiasData();
            NET_CU(cudaMemcpy(buf.data(), src, n * sizeof(float), cudaMemcpyDeviceToHost));
            for (size_t i = 0; i < n; ++i) { h ^= buf[i]; h *= 1099511628211ull; }
        }
    }
    *out = h;
    return VDNN_OK;
}
