// class Layer: one operator of the network, with the public interface of the reference's Layer
// (layer.h:130-251): same constructor arguments, same forward / backward / cnmemMalloc*Data /
// copy*Data / accessor names.  Where the reference holds cuDNN descriptors and a cuDNN or cuBLAS
// handle, this class holds plain shapes and a vdnnHandle_t; the arithmetic goes through the C ABI
// of include/vdnn_b200.h.
#ifndef VDNN_B200_LAYER_H_
#define VDNN_B200_LAYER_H_

#include <assert.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#include <initializer_list>
#include <vector>

#include "cnmem/include/cnmem.h"
#include "vdnn.h"
#include "vdnn_b200.h"

#define CEIL(a, b) (((a) + (b) - 1) / (b))

// State shared by all layers of a network: the role the cuDNN / cuBLAS handles play in the
// reference (layer.h:311,336) plus what the event-ordered memory manager needs.
struct vdnnContext {
    // configuration
    float learning_rate = static_cast<float>(LEARNING_RATE);
    int init_mode = 1;                 // 0 He-normal / zero bias, 1 U(-0.01, 0.01)
    uint64_t weight_seed_base = 3000;
    bool dry_run = false;              // no device: replay allocation / copy schedule only
    bool verbose = true;
    bool host_sync_per_layer = false;  // true = synchronise both streams after every layer
    bool capture = false;
    bool profiling = false;
    bool fix_input_leak = true;
    bool quiet = false;                // trial networks: no message when the pool is exhausted

    // streams and per-layer events (index = layer id)
    cudaStream_t stream_compute = nullptr, stream_d2h = nullptr, stream_h2d = nullptr, stream_comm = nullptr;
    std::vector<cudaEvent_t> ev_fwd_done, ev_bwd_done, ev_offload_done, ev_prefetch_done, ev_weights_ready;
    cudaEvent_t ev_input_ready = nullptr;
    std::vector<char> weights_pending;     // data parallel: an update of layer l is in flight

    // profiling events (created on demand)
    std::vector<cudaEvent_t> pf_fwd_beg, pf_fwd_end, pf_bwd_beg, pf_bwd_end, pf_off_beg, pf_off_end, pf_pre_beg, pf_pre_end;
    cudaEvent_t pf_step_beg = nullptr, pf_step_end = nullptr;

    // allocation / copy trace
    bool trace_enabled = true;
    std::vector<vdnn_trace_event> trace;
    int64_t offload_bytes = 0, prefetch_bytes = 0, pinned_bytes = 0, workspace_bytes_max = 0;
    size_t shared_workspace_bytes = 0;     // BASELINE: size of the one workspace block all layers are handed

    // Offloads whose copy has not been enqueued yet.  The single device-to-host engine serves copies in
    // the order they were enqueued, forward produces layers 0..L and backward needs them L..0; so the copies
    // are enqueued after the last layer's forward, latest layer first: the prefetch of layer l then follows
    // its offload closely and both PCIe directions run at the same time.  Blocks released meanwhile are held
    // in the pool; when only held bytes fit a request, the pool has the oldest copies enqueued at once.
    // `eager_offload_budget` bytes of the first layers are still enqueued in their own layer: the copy engine is idle
    // under the forward kernels, and the first layers are needed last in backward.  By default the budget is what the
    // engine moves during one forward pass (measured: duration of the pass x EAGER_OFFLOAD_RATE; a layer may pass the
    // budget by a quarter); the environment variable VDNN_EAGER_OFFLOAD_BYTES fixes it instead (0 = none).
    struct PendingOffload { int layer; void* host; const void* dev; size_t bytes; };
    bool defer_offloads = false;
    std::vector<PendingOffload> pending_offloads;
    int64_t eager_offload_budget = 0, eager_offload_used = 0, forced_offloads = 0;
    bool eager_offload_auto = false;
    // Copies go out in pieces of this many bytes with an event after each, so that the prefetch of a tensor
    // can start behind the first piece of its offload instead of behind the whole tensor.
    size_t copy_chunk_bytes = static_cast<size_t>(256) << 20;
    std::vector<std::vector<cudaEvent_t>> ev_offload_chunk;      // [layer][piece], created on demand
    cudaEvent_t chunkEvent(int layer, size_t piece);
    bool offloadPending(int layer) const {
        for (const PendingOffload& p : pending_offloads) if (p.layer == layer) return true;
        return false;
    }
    int submitOffload(const PendingOffload& p);      // enqueue the copy, record ev_offload_done, resolve the pool hold
    // layer >= 0: everything pending up to that layer, in forward order (a held block is needed);
    // layer < 0: everything, latest layer first (end of forward)
    int flushOffloads(int layer);

    // data parallelism
    int dp_rank = 0, dp_world = 1;
    void* nccl_comm = nullptr;
    // One allocation holds the flag words of the fused peer all-reduce and every layer's gradient staging buffer
    // (csrc/dp_peer.h); dp_peer[r] is rank r's arena as mapped here when the fused path is on (dp_fused).
    float* dp_arena = nullptr;
    size_t dp_arena_floats = 0;
    float* dp_peer[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    bool dp_fused = false;

    // NULL when the context runs without a device (no events exist)
    static cudaEvent_t event(const std::vector<cudaEvent_t>& v, int id) { return v.empty() ? nullptr : v[id]; }
    void record(int kind, int layer, int tag, int64_t bytes);
    // Pool allocation for use on `streams`; emits a trace event.  Returns 0, -1 (out of memory with
    // isDynamic, as layer.h:119-125) or VDNN_ERR_OUT_OF_MEMORY.
    int alloc(void** ptr, size_t bytes, int layer, int tag, bool isDynamic, std::initializer_list<cudaStream_t> streams);
    // Returns the block to the pool; its bytes stay fenced until the work enqueued so far on `after` is done.
    int release(void* ptr, size_t bytes, int layer, int tag, std::initializer_list<cudaStream_t> after);
    // Same for srcData whose offload copy is still pending: fenced on `after` now, held until the copy is enqueued.
    int releaseHeld(void* ptr, size_t bytes, int layer, int tag, std::initializer_list<cudaStream_t> after);
    int upload(void* dst, const void* src_h, size_t bytes);        // synchronous H2D (initialisation)
};
typedef vdnnContext* vdnnHandle_t;
// Device-to-host rate assumed when forward time is turned into an eager-offload budget (bytes per second): what one
// direction of the link carries while the other is idle, rounded down.
#define EAGER_OFFLOAD_RATE 50e9

/* Handle life cycle for a driver that is not this library's Network: the calls the reference makes on its cuDNN /
   cuBLAS handles (network.cu:39-40, 56-57, 96-97).  vdnnCreate hands out the process-wide context (every "handle"
   is the same object, as all layers of the reference share its two handles); vdnnSetStream names the compute stream
   and creates the per-layer events the layers record. */
int vdnnCreate(vdnnHandle_t* handle);
int vdnnSetStream(vdnnHandle_t handle, cudaStream_t stream_compute);
int vdnnDestroy(vdnnHandle_t handle);

enum {
    TAG_WEIGHT = 0, TAG_BIAS = 1, TAG_DST = 2, TAG_DIFF = 3, TAG_GRAD = 4, TAG_SRC = 5, TAG_WS = 6,
    TAG_ONES = 7, TAG_INPUT = 8, TAG_LABEL = 9, TAG_DXDY = 10, TAG_NONE = 11
};

class Layer {
public:
    Layer(vdnn_t _vdnnMode, vdnnAlgoMode_t _vdnnAlgoMode, Layer_t _layerType, vdnnHandle_t* _handle,
          cudaStream_t* _stream_compute, cudaStream_t* _stream_memory, int _id,
          int _n, int _c, int _h, int _w, int _pad_h, int _pad_w, int _stride_h, int _stride_w,
          int _k, int _r, int _s);
    ~Layer();

    // Seeded initialisation of filter and bias (the reference draws from std::random_device).
    int     initializeConvolutionFilterAndBias();
    int     initializeFullyConnectedFilterAndBias();

    int     forward(bool* _offloaded, DATATYPE** _offloadedSrcData_h, void* workSpace, bool isDynamic);
    int     backward(int _layer_id_to_prefetch, DATATYPE* _prefetchedSrcData_h, void* _srcDataToPrefetch,
                     unsigned long _prefetch_bytes, void* workSpace, bool isDynamic);

    int     convolutionForward(bool* _offloaded, DATATYPE** _offloadedSrcData_h, void* workSpace, bool isDynamic);
    int     convolutionBackward(int _layer_id_to_prefetch, DATATYPE* _prefetchedSrcData_h, void* _srcDataToPrefetch,
                                unsigned long _prefetch_bytes, void* workSpace, bool isDynamic);
    int     fullyConnectedForward(bool* _offloaded, DATATYPE** _offloadedSrcData_h, void* workSpace, bool isDynamic);
    int     fullyConnectedBackward(int _layer_id_to_prefetch, DATATYPE* _prefetchedSrcData_h, void* _srcDataToPrefetch,
                                   unsigned long _prefetch_bytes, void* workSpace, bool isDynamic);
    int     activationForward(bool* _offloaded, DATATYPE** _offloadedSrcData_h, void* workSpace, bool isDynamic);
    int     activationBackward(int _layer_id_to_prefetch, DATATYPE* _prefetchedSrcData_h, void* _srcDataToPrefetch,
                               unsigned long _prefetch_bytes, void* workSpace, bool isDynamic);
    int     softmaxForward(bool* _offloaded, DATATYPE** _offloadedSrcData_h, void* workSpace, bool isDynamic);
    int     softmaxBackward(int _layer_id_to_prefetch, DATATYPE* _prefetchedSrcData_h, void* _srcDataToPrefetch,
                            unsigned long _prefetch_bytes, void* workSpace, bool isDynamic);
    int     poolingForward(bool* _offloaded, DATATYPE** _offloadedSrcData_h, void* workSpace, bool isDynamic);
    int     poolingBackward(int _layer_id_to_prefetch, DATATYPE* _prefetchedSrcData_h, void* _srcDataToPrefetch,
                            unsigned long _prefetch_bytes, void* workSpace, bool isDynamic);
    int     lrnForward(bool* _offloaded, DATATYPE** _offloadedSrcData_h, void* workSpace, bool isDynamic);
    int     lrnBackward(int _layer_id_to_prefetch, DATATYPE* _prefetchedSrcData_h, void* _srcDataToPrefetch,
                        unsigned long _prefetch_bytes, void* workSpace, bool isDynamic);

    int     offloadSrcData(bool* _offloaded, DATATYPE** _offloadedSrcData_h);
    int     prefetchPreviousSrcData(int _layer_id_to_prefetch, DATATYPE* _prefetchedSrcData_h,
                                    void* _srcDataToPrefetch, unsigned long _prefetch_bytes);

    int     cnmemMallocSrcData(bool isDynamic);
    int     cnmemMallocDstData(bool isDynamic);
    int     cnmemMallocDiffData(bool isDynamic);
    int     cnmemMallocGradData(bool isDynamic);

    void    copySrcData(void* _srcData)   { srcData = _srcData;   }
    void    copyDstData(void* _dstData)   { dstData = _dstData;   }
    void    copyDiffData(void* _diffData) { diffData = _diffData; }
    void    copyGradData(void* _gradData) { gradData = _gradData; }

    void    setVdnnMode(vdnn_t _vdnnMode) { vdnnMode = _vdnnMode; }

    Layer_t LayerType()              { assert(layerType < NUM_LAYER_TYPES); return layerType; }
    int     LayerId()                { return layerId;  }
    void*   SrcData()                { return srcData;  }
    void*   DstData()                { return dstData;  }
    void*   DiffData()               { return diffData; }
    void*   GradData()               { return gradData; }
    void*   FilterData()             { return filterData; }
    void*   BiasData()               { return biasData; }
    int     InputN()                 { return n_in;  }
    int     InputC()                 { return c_in;  }
    int     InputH()                 { return h_in;  }
    int     InputW()                 { return w_in;  }
    int     OutputN()                { return n_out; }
    int     OutputC()                { return c_out; }
    int     OutputH()                { return h_out; }
    int     OutputW()                { return w_out; }
    int     SrcDataSize()            { return n_in * c_in * h_in * w_in;     }
    int     DstDataSize()            { return n_out * c_out * h_out * w_out; }
    size_t  FwdWorkSpaceSize()       { return fwdWorkSpaceSize;       }
    size_t  BwdDataWorkSpaceSize()   { return bwdDataWorkSpaceSize;   }
    size_t  BwdFilterWorkSpaceSize() { return bwdFilterWorkSpaceSize; }
    int     FilterDataSize()         { return k * c_in * r * s; }
    bool    HasWeights()             { return layerType == FC_GEMM || layerType == CONV || layerType == FC_CONV; }
    void    spec(vdnn_layer_spec* out);
    bool    ok()                     { return constructed; }

    // Data-parallel staging: gradients are produced in `buffer` (FilterDataSize() + OutputC() floats, owned by the
    // network) instead of being folded into the weights.
    void    setGradientStaging(float* buffer);
    float*  GradFilter()             { return gradFilter; }
    float*  GradBias()               { return gradBias;   }

    /* VDNN_DYNAMIC_ALGO (layer.cu:1091-1147): per operation, the workspace-using algorithm when `use[op]`
       is set, else the zero-workspace one; op = 0 forward, 1 data gradient, 2 filter gradient. */
    void    setOpAlgos(const bool use[3]);
    int     findDynamicAlgo();
    void    opAlgos(int out[3]) const { out[0] = opMode[0]; out[1] = opMode[1]; out[2] = opMode[2]; }
    void    printDstData();
    void    printFilterData();

private:
    vdnn_conv_desc convDesc() const;

    vdnn_t         vdnnMode;
    vdnnAlgoMode_t vdnnAlgoMode;
    Layer_t        layerType;
    int            layerId;
    bool           constructed;

    int n_in, c_in, h_in, w_in;
    int pad_h, pad_w, stride_h, stride_w, k, r, s;
    int n_out, c_out, h_out, w_out;

    size_t fwdWorkSpaceSize, bwdDataWorkSpaceSize, bwdFilterWorkSpaceSize;
    int    opMode[3];          // VDNN_ALGO_MEMORY_OPT / VDNN_ALGO_PERF_OPT per operation

    cudaStream_t* stream_compute;
    cudaStream_t* stream_memory;
    vdnnHandle_t  handle;

    void* srcData;
    void* filterData;
    void* biasData;
    void* dstData;
    void* diffData;
    void* gradData;
    float* gradFilter;
    float* gradBias;
};

#endif
