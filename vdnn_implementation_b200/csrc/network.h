// class Network: topology tables, vDNN policy and the two training loops, with the public
// interface of the reference's Network (network.h:15-95).  Additions are grouped at the end of
// the public section.
#ifndef VDNN_B200_NETWORK_H_
#define VDNN_B200_NETWORK_H_

#include <string>
#include <vector>

#include "layer.h"

class Network {
public:
    Network(CNN_t _cnnType, vdnn_t _vdnnType, vdnnAlgoMode_t _algoMode, int _batchSize = DEFAULT_BATCH_SIZE);
    explicit Network(const vdnn_network_config& cfg, bool dry_run = false);
    // trial networks of the dynamic mode: per layer, bit `op` set = workspace-using algorithm for that operation
    Network(const vdnn_network_config& cfg, bool dry_run, const std::vector<unsigned char>& layerOps);
    ~Network();

    /* Setup */
    void            setLayers(CNN_t _cnnType);
    void            setLayersAlexnet();
    void            setLayersOverfeat();
    void            setLayersGooglenet();
    void            setLayersVgg16(int givenBatch);
    void            setLayersCustomCNN();
    void            randomInitializeData(void* data, int size);
    void            sanityCheck();
    void            setVdnnType(vdnn_t newVdnnType);

    /* Find max dx, dy, workspace size */
    size_t          findMaxDxDySize();
    size_t          findMaxWorkSpaceSize();

    /* Computation for training network */
    void            calculateFirstDiffData(void* result, void* first, void* second);
    int             forwardPropagation(bool isDynamic = false);
    int             backwardPropagation(bool isDynamic = false);

    /* Find prefetch layer */
    void            resetIsPrefetchedArray();
    int             findPrefetchLayer(int currLayerId);

    /* Get functions */
    Layer**         layerArray()            { return layer;                         }
    DATATYPE**      offloadedSrcDataArray() { return offloadedSrcData_h;            }
    int             getInputSize()          { return n_in * c_in * h_in * w_in;     }
    int             getOutputSize()         { return n_out * c_out * h_out * w_out; }

    /* ---- additions ---- */
    int             status() const          { return state;     }   // VDNN_OK or the error that stopped construction
    int             numLayers_() const      { return numLayers; }
    vdnnContext&    context()               { return ctx;       }
    int             setInput(const float* input_h, const float* label_h);
    int             seedInput(uint64_t input_seed, uint64_t label_seed);
    int             synchronize();
    int             join();
    int             loss(double* out2);
    size_t          tensorSize(int layerId, int kind);
    int             readTensor(int layerId, int kind, float* dst_h, size_t count);
    int             writeTensor(int layerId, int kind, const float* src_h, size_t count);
    int             getStats(vdnn_network_stats* out);
    /* VDNN_DYNAMIC_ALGO (network.cu:946-1008): what the constructor settled on.  algo is VDNN_DYNAMIC_ALGO when
       the algorithms were chosen per layer and operation (see layerAlgos), else the mode all layers share. */
    void            selected(int* vdnn_type, int* algo) const;
    int             layerAlgos(int layerId, int out3[3]) const;
    int             setProfiling(bool enabled);
    int             setOffloadOrder(bool forwardOrder);
    int             timeline(float* out);
    int             enableDataParallel(int rank, int world, const char* unique_id128);
    int             weightChecksum(uint64_t* out);
    int             dpMode() const;            // 0 single device, 1 NCCL all-reduce + axpy, 2 fused peer all-reduce + SGD
    /* Lean variant of VDNN_ALL (not in the reference; it moves fewer bytes, so it is never the default): the srcData of
       a ReLU layer that follows a CONV / FC layer is neither offloaded nor kept -- it is released after the ReLU's
       forward, and the ReLU's backward takes its mask from dstData (y > 0 exactly where x > 0), which the next layer's
       prefetch brings back anyway.  CONV / FC backward never read their own output.  Networks constructed while the
       switch is on (or with VDNN_LEAN_OFFLOAD=1 in the environment) follow it. */
    static void     setLeanOffloadDefault(int on);
    bool            leanOffload() const { return lean; }

private:
    void            init(const vdnn_network_config& cfg, bool dry_run);
    int             vdnnDynamicAlgo(const vdnn_network_config& cfg);
    // peak: the replay's pool high-water mark (bytes), when asked for
    static bool     trainable(const vdnn_network_config& cfg, vdnn_t type, vdnnAlgoMode_t algo,
                              const std::vector<unsigned char>* layerOps, size_t* peak = NULL);
    void            addLayer(Layer_t type, vdnnAlgoMode_t algo, int n, int c, int h, int w, int pad, int stride, int k, int r);
    void            convRelu(int pad, int stride, int k, int r, bool forceMemOpt = false);
    void            fcRelu(int k);
    int             captureTensor(std::vector<float>& dst, const void* src, size_t count);
    int             reduceAndApply(int layerId);
    void            memoryLine(const char* phase, int l, size_t extra);

    CNN_t               cnnType;
    vdnn_t              vdnnType;
    vdnnAlgoMode_t      algoMode;
    bool                dynamicPerLayer;
    bool                packedPool;            // pool below 1.4 x the schedule's peak: tightest fit, copies in layer order
    std::vector<unsigned char> layerOps;       // set by the dynamic mode (empty: every layer follows algoMode)
    vdnnContext         ctx;
    vdnnHandle_t        handle;
    cudaStream_t        stream_compute;
    cudaStream_t        stream_memory;
    int                 batchSize;
    int                 numLayers;
    int                 state;
    int                 device;
    bool                poolOwner;

    int n_in, c_in, h_in, w_in;
    int n_out, c_out, h_out, w_out;
    int cur_n, cur_c, cur_h, cur_w;           // running shape while the table is built

    void*               inputData;
    void*               labelData;
    void*               networkDiffData;
    void*               networkGradData;
    void*               workSpace;
    size_t              workSpaceBytes, dxdyBytes;

    Layer*              layer[DEFAULT_NUM_LAYER];
    bool                isOffload[DEFAULT_NUM_LAYER];
    bool                isPrefetched[DEFAULT_NUM_LAYER];
    bool                lean;                              // lean VDNN_ALL (see setLeanOffloadDefault)
    bool                leanDrop[DEFAULT_NUM_LAYER];       // this layer's srcData is released after its forward, not offloaded
    DATATYPE*           offloadedSrcData_h[DEFAULT_NUM_LAYER];

    const vdnn_layer_spec* customLayers;
    int                 numCustomLayers;
    bool                externalInput;
    bool                forwardDone;
    uint64_t            stepCounter;
    float*              stage_h;               // pinned staging for generated input / labels
    double*             loss_h;
    cudaEvent_t         ev_fwd_t0, ev_fwd_t1;  // timing events around the forward pass (eager offload budget)
    bool                fwdTimed;
    float               fwdMsBest;
    cudaEvent_t         ev_loss;
    cudaEvent_t         ev_step_end;
    std::vector<std::vector<float>> capDst, capGrad;
    std::vector<size_t> dpOffset;              // data parallel: each layer's staging buffer inside ctx.dp_arena (floats)
    unsigned long long  launchesAtStepStart, launchesLastStep;
};

#endif
