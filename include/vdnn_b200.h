/*
 * vdnn_b200 -- C ABI of the B200 (sm_100a) implementation of the vDNN training hot path.
 *
 * Every entry point replaces one library call site of james98kr/vDNN_Implementation
 * (cuDNN / cuBLAS / CUDA runtime); the citation beside each declaration is the reference
 * file:line it stands in for.  Conventions shared by all of them:
 *   - plain pointers and sizes only; tensors are fp32, NCHW / KCRS, densely packed
 *     (vdnn.h:11,19), living in device memory unless a name ends in _h;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *     work is enqueued, never synchronised;
 *   - no entry point of sections 1-3 allocates memory: scratch is the caller-provided
 *     `workspace` whose size vdnn_conv_workspace_bytes / vdnn_sgemm_workspace_bytes report;
 *   - alpha / beta follow cuDNN / cuBLAS: out = alpha * op(...) + beta * out;
 *   - the return value is VDNN_OK (0) or a negative vdnn_status; nothing falls back to a
 *     CPU path or to another library.
 */
#ifndef VDNN_B200_H_
#define VDNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    VDNN_OK = 0,
    VDNN_ERR_BAD_ARG = -1,        /* NULL pointer, non-positive extent, unknown enum value   */
    VDNN_ERR_CUDA = -2,           /* a CUDA runtime call failed; see vdnn_last_cuda_error()  */
    VDNN_ERR_WORKSPACE = -3,      /* workspace smaller than vdnn_*_workspace_bytes reports   */
    VDNN_ERR_UNSUPPORTED = -4,    /* shape outside what the selected engine implements       */
    VDNN_ERR_OUT_OF_MEMORY = -5,  /* pool exhausted (network-level calls only)               */
    VDNN_ERR_TIMEOUT = -6,        /* a bounded device-side wait expired                      */
    VDNN_ERR_STATE = -7,          /* call order violated (e.g. backward before forward)      */
    VDNN_ERR_SCRATCH_LIMIT = -8   /* problem needs more than the library's built-in scratch  */
} vdnn_status;

const char* vdnn_status_string(int status);
/* cudaError_t of the most recent failing runtime call on this thread (0 if none). */
int vdnn_last_cuda_error(void);
/* Library version and the compute capability the kernels were built for ("sm_100a"). */
const char* vdnn_build_info(void);

/* -------------------------------------------------------------------------------------------
 * 1. Convolution and GEMM  (reference: cudnnConvolution* and cublasSgemm call sites)
 * ----------------------------------------------------------------------------------------- */

/* vdnnAlgoMode_t of the reference (vdnn.h:31-36).  MEMORY_OPT = zero-workspace kernels,
 * PERF_OPT = kernels that may use workspace (deterministic split-K partial sums). */
typedef enum { VDNN_ALGO_MEMORY_OPT = 0, VDNN_ALGO_PERF_OPT = 1, VDNN_ALGO_DYNAMIC = 2 } vdnn_algo_mode;
typedef enum { VDNN_CONV_FWD = 0, VDNN_CONV_BWD_DATA = 1, VDNN_CONV_BWD_FILTER = 2,
               VDNN_CONV_BWD_ALL = 3 /* the three gradients in one workspace: vdnn_conv_bwd_data_filter_bias */ } vdnn_conv_op;
/* Which contraction engine runs CONV/FC.  AUTO picks TCGEN05 (3xTF32 on the 5th-generation
 * tensor cores, fp32-accurate) when the shape is supported by it and FFMA otherwise.  In PERF_OPT the tensor-core
 * engine has a gather-fed and a TMA-fed kernel family; AUTO uses the TMA-fed one for stride-1 convolutions with
 * enough output tiles to fill the GPU, TCGEN05 for every shape it supports (workspace sizes follow the setting). */
typedef enum { VDNN_ENGINE_AUTO = 0, VDNN_ENGINE_FFMA = 1, VDNN_ENGINE_TCGEN05 = 2 } vdnn_engine;
int vdnn_set_engine(int engine);   /* process-wide; returns the previous value */
int vdnn_get_engine(void);
/* Health of the tensor-core engine.  Its kernels wait on shared-memory barriers with an iteration
 * limit; a wait that expires records a code (101 producer, 102 MMA issuer, 103 epilogue, 104 self-test) instead of
 * spinning for ever.  Synchronises the device, stores the code (0 = healthy) and clears it. */
int vdnn_engine_status(int* code);
/* The same code written to *dst (device memory, or pinned host memory mapped into the device's address space) by a
 * one-thread kernel in stream order: no synchronisation, nothing cleared.  The network driver calls it at the end of
 * every backward pass and vdnn_network_synchronize returns VDNN_ERR_TIMEOUT when the word it left is not 0.
 * No counterpart in the reference (cuDNN reports failures through its return codes, layer.h:73-128). */
int vdnn_engine_status_publish(int* dst, void* stream);
/* Self-test of that path: launches one warp that waits at most `limit_cycles` SM cycles (at most 2e9) on a barrier
 * nothing arrives at.  The wait runs out, code 104 is recorded and the kernel returns; vdnn_engine_status then
 * reports 104.  Nothing faults or hangs.  No counterpart in the reference. */
int vdnn_engine_wait_selftest(unsigned long long limit_cycles, void* stream);
/* Measurement aid: one CTA per SM issues 12 * iterations tcgen05.mma kind::tf32 of 128 x 256 x 8 on zero operands in
 * shared memory (no loads, no epilogue); *flops receives the hardware flops of the launch (2 * 128 * 256 * 8 per MMA).
 * Time it with events on `stream`: flops / time is the dense TF32 rate of the tensor pipe on this device, and a third
 * of it is the ceiling of the fp32-accurate 3xTF32 contraction kernels.  No counterpart in the reference. */
int vdnn_engine_mma_rate_probe(int iterations, double* flops, void* stream);

/* Shape of one convolution: what the reference spreads over srcTensorDesc, filterDesc and
 * convDesc (layer.cu:152-204).  Dilation is 1, mode is cross-correlation (vdnn.h:20). */
typedef struct {
    int n, c, h, w;               /* input  N x C x H x W   */
    int k, r, s;                  /* filter K x C x R x S   */
    int pad_h, pad_w;
    int stride_h, stride_w;
} vdnn_conv_desc;

/* cudnnGetConvolution2dForwardOutputDim (layer.cu:207-215). */
int vdnn_conv_out_dims(const vdnn_conv_desc* d, int* p, int* q);
/* cudnnGetPooling2dForwardOutputDim (layer.cu:431-438); padding is 0 as in the reference. */
int vdnn_pool_out_dims(int h, int w, int win_h, int win_w, int stride_h, int stride_w, int* p, int* q);

/* cudnnGetConvolution{Forward,BackwardData,BackwardFilter}WorkspaceSize (layer.cu:268-294)
 * together with the algorithm choice of find{MemOpt,PerfOpt}*Algo (layer.cu:1013-1089):
 * 0 for VDNN_ALGO_MEMORY_OPT, the split-K scratch of the PERF_OPT kernel otherwise. */
size_t vdnn_conv_workspace_bytes(int op, int algo_mode, const vdnn_conv_desc* d);

/* cudnnConvolutionForward (layer.cu:560-569): y = alpha * (x corr w) + beta * y.
 * `bias` (K floats) may be NULL; when given, bias[k] is added to every y[n][k][p][q] in the
 * same pass, which is what the reference does with a second call, cudnnAddTensor
 * (layer.cu:576-582). */
int vdnn_conv_fwd(const vdnn_conv_desc* d, int algo_mode, float alpha, const float* x,
                  const float* w, const float* bias, float beta, float* y,
                  void* workspace, size_t workspace_bytes, void* stream);
/* cudnnAddTensor with a 1xKx1x1 operand (layer.cu:576-582): y[n][k][*] += alpha * bias[k]. */
int vdnn_add_bias(int n, int k, int pq, float alpha, const float* bias, float* y, void* stream);
/* cudnnConvolutionBackwardData (layer.cu:616-625): dx = alpha * convT(dy, w) + beta * dx. */
int vdnn_conv_bwd_data(const vdnn_conv_desc* d, int algo_mode, float alpha, const float* w,
                       const float* dy, float beta, float* dx,
                       void* workspace, size_t workspace_bytes, void* stream);
/* cudnnConvolutionBackwardBias (layer.cu:631-637): db[k] = alpha * sum_{n,p,q} dy + beta * db[k].
 * The reference passes alpha = -LEARNING_RATE, beta = 1: the SGD step is part of the call. */
int vdnn_conv_bwd_bias(int n, int k, int pq, float alpha, const float* dy, float beta, float* db,
                       void* stream);
/* cudnnConvolutionBackwardFilter (layer.cu:651-660): dw = alpha * (x corr dy) + beta * dw,
 * in place on the weights when alpha = -lr, beta = 1. */
int vdnn_conv_bwd_filter(const vdnn_conv_desc* d, int algo_mode, float alpha, const float* x,
                         const float* dy, float beta, float* dw,
                         void* workspace, size_t workspace_bytes, void* stream);

/* cudnnConvolutionBackwardBias + cudnnConvolutionBackwardFilter (layer.cu:631-660) in one call:
 *   db = alpha_b * sum_{n,p,q} dy + beta_b * db,   dw = alpha * (x corr dy) + beta * dw.
 * In PERF_OPT, for stride-1 convolutions whose channel counts are multiples of 32, the bias sums are formed by the pass
 * that prepares dy for the filter gradient (dy is read once less); otherwise the two separate entry points run. */
int vdnn_conv_bwd_filter_bias(const vdnn_conv_desc* d, int algo_mode, float alpha, const float* x, const float* dy,
                              float beta, float* dw, float alpha_b, float beta_b, float* db,
                              void* workspace, size_t workspace_bytes, void* stream);

/* cudnnConvolutionBackwardData + BackwardBias + BackwardFilter of one layer (layer.cu:616-660) in one call:
 *   dx = alpha_dx * (dy corr^T w) + beta_dx * dx   with the weights as they are on entry (dw may be w),
 *   db = alpha_b * sum dy + beta_b * db,   dw = alpha_w * (x corr dy) + beta_w * dw.
 * Workspace: vdnn_conv_workspace_bytes(VDNN_CONV_BWD_ALL, mode, d); where vdnn_conv_bwd_shares_dy is 1 the figure for
 * VDNN_CONV_BWD_FILTER is at least as large, elsewhere it is the larger of the two separate figures.
 * In PERF_OPT, where both gradients run on the TMA-fed kernels (vdnn_conv_bwd_shares_dy), dy is rewritten into operand
 * images once for both and the bias sums come from the same pass; elsewhere the separate entry points run in the
 * reference's order. */
int vdnn_conv_bwd_data_filter_bias(const vdnn_conv_desc* d, int algo_mode, float alpha_dx, const float* w, const float* x,
                                   const float* dy, float beta_dx, float* dx, float alpha_w, float beta_w, float* dw,
                                   float alpha_b, float beta_b, float* db, void* workspace, size_t workspace_bytes, void* stream);
int vdnn_conv_bwd_shares_dy(const vdnn_conv_desc* d, int algo_mode);

/* Filter gradient for callers that cannot provide workspace.  No counterpart in the reference.
 *
 * Same result as vdnn_conv_bwd_filter with VDNN_ALGO_PERF_OPT (fixed-order, deterministic split-K
 * sums), but the per-split partial sums live in a scratch array that is part of the library image
 * (a file-scope __device__ array of VDNN_STATIC_SCRATCH_BYTES = 16 MiB, resident on every GPU that
 * loads the library until the process exits) instead of caller-provided workspace.  It is meant for
 * hosts that fix their device-memory budget at start-up and must not allocate afterwards -- a
 * plugin loaded into a process whose allocator it cannot reach, or a steady-state loop that must
 * not hit the device-wide synchronisation an allocation or release implies -- and so have no
 * buffer to pass as `workspace`.  The entry point calls no cudaMalloc / cudaFree and no routine
 * that allocates.
 *   - Shapes whose partial sums exceed the array (vdnn_conv_workspace_bytes(VDNN_CONV_BWD_FILTER,
 *     VDNN_ALGO_PERF_OPT, d) > VDNN_STATIC_SCRATCH_BYTES) are refused with VDNN_ERR_SCRATCH_LIMIT;
 *     nothing is launched.
 *   - The first call on a device looks up the array's device address (once per device, with that
 *     device current).  Make that first call before any stream capture begins.
 *   - All calls on a device share the one array, which keeps whatever the last call left in it.
 *     Every element a call reads was written by that same call, so nothing has to be cleared; but
 *     two calls that overlap on the GPU (different streams without ordering) race on it. */
#define VDNN_STATIC_SCRATCH_BYTES (16u << 20)
int vdnn_conv_bwd_filter_static(const vdnn_conv_desc* d, float alpha, const float* x, const float* dy,
                                float beta, float* dw, void* stream);

/* cublasSgemm (layer.cu:677-685, 697-705, 725-733, 736-744, 752-760): column-major
 * C(m x n) = alpha * op(A) * op(B) + beta * C, transa/transb: 0 = N, 1 = T. */
size_t vdnn_sgemm_workspace_bytes(int algo_mode, int m, int n, int k);
int vdnn_sgemm(int transa, int transb, int m, int n, int k, float alpha, const float* A, int lda,
               const float* B, int ldb, float beta, float* C, int ldc,
               int algo_mode, void* workspace, size_t workspace_bytes, void* stream);
/* fillVectorWithOnes (layer.cu:33-38). */
int vdnn_fill(size_t count, float value, float* dst, void* stream);

/* -------------------------------------------------------------------------------------------
 * 2. Bandwidth-bound layers  (reference: cudnnActivation*, cudnnPooling*, cudnnSoftmax*)
 * ----------------------------------------------------------------------------------------- */

/* cudnnActivationForward, RELU, PROPAGATE_NAN, out of place (layer.cu:774-781, 380-385). */
int vdnn_relu_fwd(size_t count, const float* x, float* y, void* stream);
/* cudnnActivationBackward (layer.cu:802-811): dx = dy where x > 0, else 0.  y is accepted
 * for signature parity and not read. */
int vdnn_relu_bwd(size_t count, const float* y, const float* dy, const float* x, float* dx,
                  void* stream);
/* cudnnActivationForward / Backward with the descriptor's mode made an argument (layer.cu:355-385, 774-811):
 * RELU as above; TANH y = tanh(x), dx = dy (1 - y^2); SIGMOID y = 1 / (1 + exp(-x)), dx = dy y (1 - y).
 * No model of the reference uses TANH or SIGMOID; its Layer class accepts them (vdnn.h:28-29). */
#define VDNN_ACT_RELU 0
#define VDNN_ACT_TANH 1
#define VDNN_ACT_SIGMOID 2
int vdnn_activation_fwd(int mode, size_t count, const float* x, float* y, void* stream);
int vdnn_activation_bwd(int mode, size_t count, const float* y, const float* dy, const float* x, float* dx,
                        void* stream);
/* cudnnPoolingForward, MAX, NOT_PROPAGATE_NAN, pad 0 (layer.cu:875-882, 417-428). */
int vdnn_maxpool_fwd(int n, int c, int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                     const float* x, float* y, void* stream);
/* cudnnPoolingBackward (layer.cu:903-912): dy of each window goes to the first element (row-major
 * scan of the window) equal to the window maximum; overlapping windows accumulate. */
int vdnn_maxpool_bwd(int n, int c, int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                     const float* y, const float* dy, const float* x, float* dx, void* stream);
/* cudnnSoftmaxForward, ACCURATE, MODE_INSTANCE over rows x cols (layer.cu:824-832). */
int vdnn_softmax_fwd(int rows, int cols, const float* x, float* y, void* stream);
/* cudnnSoftmaxBackward (layer.cu:853-862): dx = y * (dy - sum_j dy_j y_j). */
int vdnn_softmax_bwd(int rows, int cols, const float* y, const float* dy, float* dx, void* stream);
/* calculateDiffTensor (network.cu:3-8): out = a - b. */
int vdnn_sub(size_t count, const float* a, const float* b, float* out, void* stream);
/* Cross-channel LRN, y = x * (k + alpha/win * sum x^2)^-beta.  No counterpart in the reference
 * (its AlexNet omits LRN, network.cu:156-323); needed by the AlexNet benchmark configuration. */
int vdnn_lrn_fwd(int n, int c, int hw, int win, float alpha, float beta, float k,
                 const float* x, float* y, void* stream);
int vdnn_lrn_bwd(int n, int c, int hw, int win, float alpha, float beta, float k,
                 const float* x, const float* y, const float* dy, float* dx, void* stream);
/* w += alpha * g (the SGD step the reference folds into its backward calls, layer.cu:593,712;
 * used on its own when the gradient is all-reduced across ranks first). */
int vdnn_axpy(size_t count, float alpha, const float* g, float* w, void* stream);
/* out2[0] = 0.5 * sum((y - label)^2) / rows, out2[1] = -mean_rows log y[argmax label]; out2 is
 * two doubles in device memory.  The reference computes no scalar loss (network.cu:1042-1054
 * seeds backward with y - label directly); both figures are defined for parity reports. */
int vdnn_loss(int rows, int cols, const float* y, const float* label, double* out2, void* stream);

/* -------------------------------------------------------------------------------------------
 * 3. Offload / prefetch  (reference: Layer::offloadSrcData, Layer::prefetchPreviousSrcData)
 * ----------------------------------------------------------------------------------------- */

/* cudaMemcpyAsync D2H of a layer's srcData into pinned memory (layer.cu:969-977).  The copy is
 * enqueued on `copy_stream` after `ready_event` (cudaEvent_t as void*, may be NULL) and
 * `done_event` (may be NULL) is recorded behind it. */
int vdnn_offload(void* dst_pinned_h, const void* src, size_t bytes, void* ready_event,
                 void* done_event, void* copy_stream);
/* cudaMemcpyAsync H2D of an offloaded srcData into a fresh buffer (layer.cu:979-987). */
int vdnn_prefetch(void* dst, const void* src_pinned_h, size_t bytes, void* ready_event,
                  void* done_event, void* copy_stream);

/* -------------------------------------------------------------------------------------------
 * 4. Network driver  (reference: class Network, network.h:15-95, and main(), vdnn.cu:56-83)
 *    The C++ classes Network and Layer of this library keep the reference's method names;
 *    these entry points expose them to non-C++ hosts.
 * ----------------------------------------------------------------------------------------- */

/* Layer constructor arguments of the reference (layer.h:133-154). */
typedef struct {
    int type;                     /* Layer_t, vdnn.h:38-50; 9 = LRN */
    int n, c, h, w;
    int pad_h, pad_w, stride_h, stride_w;
    int k, r, s;
} vdnn_layer_spec;

typedef struct {
    int cnn_type;                 /* CNN_t, vdnn.h:52-61; 7 = ALEXNET with two LRN layers      */
    int vdnn_type;                /* vdnn_t, vdnn.h:23-29                                       */
    int algo_mode;                /* vdnnAlgoMode_t, vdnn.h:31-36                               */
    int batch_size;               /* 0 = the reference default for the model (network.cu:142-147) */
    int device;                   /* CUDA device ordinal (vdnn.h:5 hard-codes 0)                 */
    size_t pool_bytes;            /* pool capacity; 0 = 24e9.  The reference takes all of the
                                     device, rounded down to 1e9 (network.cu:49)                 */
    float learning_rate;          /* vdnn.h:8 fixes 1e-5; <= 0 selects that value                */
    int init_mode;                /* 0 = He-normal weights / zero bias, 1 = U(-0.01, 0.01) as
                                     layer.cu:925-967 (seeded instead of std::random_device)     */
    uint64_t weight_seed_base;    /* layer l uses weight_seed_base + l                           */
    int fix_input_leak;           /* 1 = free the superseded input buffer (network.cu:1185 drops it) */
    int host_sync_per_layer;      /* 1 = cudaStreamSynchronize both streams after every layer as
                                     network.cu:1089-1091,1167-1169 do; 0 = event-ordered         */
    int verbose;                  /* 1 = print the reference's banners and per-layer memory lines */
    int capture;                  /* 1 = keep a host copy of every layer's dst / grad for parity  */
    const vdnn_layer_spec* custom_layers;   /* CUSTOM_CNN topology (network.cu:815-817 is empty) */
    int num_custom_layers;
} vdnn_network_config;

typedef struct vdnn_network vdnn_network;

int vdnn_network_create(vdnn_network** out, const vdnn_network_config* cfg);
int vdnn_network_destroy(vdnn_network* net);
int vdnn_network_num_layers(const vdnn_network* net);
int vdnn_network_layer_spec(const vdnn_network* net, int layer, vdnn_layer_spec* out);
size_t vdnn_network_input_size(const vdnn_network* net);    /* Network::getInputSize  */
size_t vdnn_network_output_size(const vdnn_network* net);   /* Network::getOutputSize */
/* Copies one batch from host memory into inputData / labelData on the compute stream; replaces
 * randomInitializeData (network.cu:819-829, 1045, 1059).  Pinned memory makes it asynchronous. */
int vdnn_network_set_input(vdnn_network* net, const float* input_h, const float* label_h);
/* Fills inputData / labelData on the host from the counter-based generator (input ~ N(0,1) with
 * seed input_seed, one-hot labels with seed label_seed) and uploads them. */
int vdnn_network_seed_input(vdnn_network* net, uint64_t input_seed, uint64_t label_seed);
int vdnn_network_forward(vdnn_network* net);    /* Network::forwardPropagation,  network.cu:1056-1110 */
int vdnn_network_backward(vdnn_network* net);   /* Network::backwardPropagation, network.cu:1112-1191 */
int vdnn_network_synchronize(vdnn_network* net);
/* The streams the network enqueues on (cudaStream_t as void*): 0 compute, 1 offload (D2H), 2 prefetch
 * (H2D), 3 collectives.  The reference keeps its two streams private (network.h:67-68). */
void* vdnn_network_stream(vdnn_network* net, int which);
/* Makes the compute stream wait, on the device, for everything enqueued so far on the other three
 * streams; an event recorded on the compute stream afterwards marks the end of all the work. */
int vdnn_network_join(vdnn_network* net);
/* Number of kernels this library has launched in this process (all entry points). */
unsigned long long vdnn_kernel_launch_count(void);
/* Blocks until the loss of the last forward pass is on the host; out2 as in vdnn_loss. */
int vdnn_network_loss(vdnn_network* net, double* out2);

typedef enum { VDNN_TENSOR_DST = 0, VDNN_TENSOR_GRAD = 1, VDNN_TENSOR_WEIGHT = 2, VDNN_TENSOR_BIAS = 3 } vdnn_tensor_kind;
size_t vdnn_network_tensor_size(const vdnn_network* net, int layer, int kind);
/* WEIGHT / BIAS are read from the device; DST / GRAD come from the capture copies (capture = 1). */
int vdnn_network_read_tensor(vdnn_network* net, int layer, int kind, float* dst_h, size_t count);
int vdnn_network_write_tensor(vdnn_network* net, int layer, int kind, const float* src_h, size_t count);

/* Allocation / offload / prefetch trace in program order. */
typedef struct {
    int kind;       /* 0 alloc, 1 free, 2 offload, 3 prefetch, 4 forward of `layer` done, 5 backward done */
    int layer;
    int tag;        /* 0 weight 1 bias 2 dst 3 diff 4 grad 5 src 6 workspace 7 ones 8 input 9 label 10 dx/dy 11 none */
    int64_t bytes;
    int64_t used;   /* pool bytes in use after the event (what total - free of cnmemMemGetInfo gives) */
} vdnn_trace_event;
int vdnn_network_trace(vdnn_network* net, vdnn_trace_event* out, int max_events, int* num_events);
int vdnn_network_trace_reset(vdnn_network* net);

typedef struct {
    int64_t pool_peak_bytes;      /* allocator high-water mark                                   */
    int64_t pool_used_bytes;
    int64_t pool_capacity_bytes;
    int64_t pinned_bytes;         /* host memory pinned for offload                              */
    int64_t offload_bytes;        /* D2H bytes of the last forward                               */
    int64_t prefetch_bytes;       /* H2D bytes of the last backward                              */
    int64_t workspace_bytes_max;
    int64_t grad_buffer_bytes;    /* data-parallel gradient staging (not part of the policy peak) */
    float step_ms;                /* compute-stream time of the last forward + backward           */
    float offload_ms;             /* sum of D2H copy durations                                   */
    float prefetch_ms;            /* sum of H2D copy durations                                   */
    float copy_overlap_ms;        /* part of the copy time that ran under compute kernels        */
    int kernel_launches;          /* launches of this library's kernels in the last step         */
    float contraction_ms;         /* compute-stream time spent in CONV / FC layers (forward + backward) */
    float elementwise_ms;         /* ... in ReLU / pool / LRN / softmax layers                    */
    double contraction_flops;     /* algorithmic FLOPs of those CONV / FC layers: 2*M*N*K each for forward,
                                     data gradient and filter gradient                             */
    double elementwise_bytes;     /* algorithmic bytes of the bandwidth-bound layers, forward + backward */
    int64_t forced_offloads;      /* offload copies of the last forward that had to be enqueued early because
                                     only their (held) bytes fitted an allocation: see vdnn_network_set_offload_order */
} vdnn_network_stats;
/* Fills timing fields only if profiling events were enabled with vdnn_network_set_profiling. */
int vdnn_network_get_stats(vdnn_network* net, vdnn_network_stats* out);
int vdnn_network_set_profiling(vdnn_network* net, int enabled);
/* VDNN_DYNAMIC_ALGO (network.cu:946-1008, layer.cu:1091-1147): the constructor ignores the given policy and
 * settles on the first of VDNN_NONE, VDNN_CONV, VDNN_ALL that trains within the pool with the workspace-using
 * algorithms; failing all three it keeps VDNN_ALL and picks, per convolution and operation, the workspace-using
 * algorithm where the iteration still fits.  A model that does not fit under VDNN_ALL with zero workspace is
 * refused (VDNN_ERR_OUT_OF_MEMORY; the reference asserts).  Candidates are tried by replaying their allocation
 * schedule against a bookkeeping-only pool of the same capacity, not by running them.
 * vdnn_network_selected reports the outcome: *algo_mode is VDNN_DYNAMIC_ALGO (2) when the choice is per layer,
 * and vdnn_network_layer_algos then gives VDNN_ALGO_* for forward, data gradient, filter gradient of a layer. */
int vdnn_network_selected(vdnn_network* net, int* vdnn_type, int* algo_mode);
int vdnn_network_layer_algos(vdnn_network* net, int layer, int* out3);
/* Order in which the offload copies of one forward pass reach the device-to-host copy engine.  The
 * reference enqueues each copy in its own layer (layer.cu:969-977) and waits for it there
 * (network.cu:1090-1091).  Without those waits the engine serves copies first in, first out, while
 * backward needs the last layer's data first; so by default (forward_order = 0) only as many bytes of
 * the first layers as the copy engine moves under the forward kernels (measured from the second step on; the
 * environment variable VDNN_EAGER_OFFLOAD_BYTES fixes the figure, 0 = none) are enqueued in their own layer,
 * and the rest after the last layer's forward, latest layer first.  Which layers are offloaded, the
 * bytes moved, the host-side allocation order and the pool's byte counts are the same either way.
 * forward_order = 1 (or the environment variable VDNN_OFFLOAD_ORDER=forward) restores layer order. */
int vdnn_network_set_offload_order(vdnn_network* net, int forward_order);
/* Lean variant of VDNN_ALL.  Not in the reference and never the default, because it changes the bytes moved and the
 * allocation trace: the srcData of a ReLU layer that follows a CONV / FC layer is released after that ReLU's forward
 * instead of being offloaded, and the ReLU's backward takes its mask from dstData (y > 0 exactly where x > 0), which
 * the prefetch for the next layer brings back anyway; CONV / FC backward never read their own output
 * (layer.cu:616-660, 721-760).  Results are bit-identical to VDNN_ALL; VGG16 moves about half the bytes.
 * on = 1 / 0: networks created from now on follow / do not follow it; on < 0: the environment variable
 * VDNN_LEAN_OFFLOAD decides (the initial state).  vdnn_network_lean reports what a network was built with. */
int vdnn_set_lean_offload(int on);
int vdnn_network_lean(const vdnn_network* net);
/* Per-layer timeline of the last profiled step, in milliseconds from the step's first event:
 * out[8*l + 0..7] = forward begin, forward end, offload begin, offload end, backward begin, backward end,
 * prefetch begin, prefetch end of layer l (negative where the layer has no such event).  `out` holds
 * 8 * vdnn_network_num_layers floats.  Synchronises the network. */
int vdnn_network_timeline(vdnn_network* net, float* out);

/* Data parallelism (no counterpart in the reference, which is single-device: vdnn.h:5).
 * One process per GPU; gradients are written to a staging buffer, all-reduced (sum) with NCCL on
 * a communication stream as each layer's backward finishes, then applied with vdnn_axpy. */
int vdnn_dp_unique_id(char* out128);
int vdnn_network_enable_dp(vdnn_network* net, int rank, int world_size, const char* unique_id128);
/* With VDNN_DP_FUSED=1 in the environment (ranks = processes on one box, at most 8), vdnn_network_enable_dp also maps
 * every rank's gradient arena into this process (CUDA IPC) and the per-layer NCCL all-reduce + axpy is replaced by one
 * kernel per layer: reduce-scatter by peer loads, all-gather by peer stores over NVLink, then the SGD step, ordered by
 * epoch flags in peer memory whose waits are bounded (an expired wait makes vdnn_network_synchronize return
 * VDNN_ERR_TIMEOUT).  Sums are taken in rank order on every rank, so weights stay bit-identical across ranks.
 * vdnn_network_dp_mode: 0 = single device, 1 = NCCL, 2 = fused peer kernel (what the ranks agreed on).
 * vdnn_dp_slice: the part of a `count`-float gradient that `rank` reduces, [*begin, *end) in floats, whole groups of 4. */
int vdnn_network_dp_mode(vdnn_network* net);
int vdnn_dp_slice(size_t count, int world_size, int rank, size_t* begin, size_t* end);
/* 64-bit checksum of all weights and biases (order-dependent FNV over the raw bits). */
int vdnn_network_weight_checksum(vdnn_network* net, uint64_t* out);

/* Host-side generators used by vdnn_network_seed_input and the weight initialiser
 * (Philox4x32-10, element index = counter). */
void vdnn_host_fill_normal(float* dst_h, size_t count, uint64_t seed, float mean, float stddev);
void vdnn_host_fill_uniform(float* dst_h, size_t count, uint64_t seed, float lo, float hi);
void vdnn_host_fill_onehot(float* dst_h, int rows, int cols, uint64_t seed);

#ifdef __cplusplus
}
#endif
#endif /* VDNN_B200_H_ */
