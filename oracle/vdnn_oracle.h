/*
 * CPU oracle for the vDNN training hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * Plain C restatement of the arithmetic that james98kr/vDNN_Implementation
 * obtains from cuDNN / cuBLAS (layer.cu:539-915) and of its allocation /
 * offload / prefetch schedule (network.cu:875-940, 1042-1207).  It is linked
 * by the tests, by the smoke check and by the CPU-baseline leg of the
 * benchmark, never by the product library.
 *
 * Parity status: pinned.  The reference ships no golden vectors and its
 * arithmetic lives in closed libraries (cuDNN, cuBLAS), so the pins were made
 * by running the reference itself: tensors computed by its own Layer class on
 * cuDNN 9.10 / cuBLAS on a B200 and the memory lines its program prints are
 * committed under tests/golden/ (see tests/golden/make_golden.py) and checked by
 * tests/test_golden.py.  LRN has no counterpart in the reference; it is pinned
 * against PyTorch's local_response_norm only.
 *
 * Storage is fp32 NCHW / KCRS (vdnn.h:11,19); accumulation type is
 * ORC_ACC (double for the checker build, float for the timed baseline build).
 */
#ifndef VDNN_ORACLE_H_
#define VDNN_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Layer_t values of the reference (vdnn.h:38-50) plus the LRN extension. */
enum {
    ORC_FC_GEMM = 0, ORC_CONV = 1, ORC_FC_CONV = 2, ORC_RELU = 3, ORC_TANH = 4,
    ORC_SIGMOID = 5, ORC_SOFTMAX = 6, ORC_POOL = 7, ORC_CONCATENATE = 8, ORC_LRN = 9
};
/* vdnn_t (vdnn.h:23-29) */
enum { ORC_BASELINE = 0, ORC_VDNN_NONE = 1, ORC_VDNN_ALL = 2, ORC_VDNN_CONV = 3 };
/* CNN_t (vdnn.h:52-61) plus ALEXNET_LRN (BASELINE config 1) */
enum { ORC_ALEXNET = 0, ORC_OVERFEAT = 1, ORC_GOOGLENET = 2, ORC_VGG16_64 = 3,
       ORC_VGG16_128 = 4, ORC_VGG16_256 = 5, ORC_CUSTOM_CNN = 6, ORC_ALEXNET_LRN = 7 };

/* Same argument list as the reference Layer constructor (layer.h:133-154). */
typedef struct {
    int type;
    int n, c, h, w;
    int pad_h, pad_w, stride_h, stride_w;
    int k, r, s;
} orc_layer_spec;

/* ---- counter-based RNG (Philox4x32-10), element index = counter ---------- */
void orc_fill_uniform(float* dst, size_t n, uint64_t seed, float lo, float hi);
void orc_fill_normal(float* dst, size_t n, uint64_t seed, float mean, float stddev);
void orc_fill_onehot(float* dst, int rows, int cols, uint64_t seed);

/* ---- layer arithmetic ----------------------------------------------------- */
void orc_conv_out_dims(int h, int w, int pad_h, int pad_w, int stride_h, int stride_w,
                       int r, int s, int* p, int* q);
void orc_pool_out_dims(int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                       int* p, int* q);
/* y = alpha*conv(x,w) + beta*y                     (layer.cu:560-569) */
void orc_conv_fwd(int n, int c, int h, int w, int k, int r, int s, int pad_h, int pad_w,
                  int stride_h, int stride_w, float alpha, const float* x, const float* wt,
                  float beta, float* y);
/* y[n][k][p][q] += bias[k]                          (layer.cu:576-582) */
void orc_add_bias(int n, int k, int pq, const float* bias, float* y);
/* dx = alpha*convT(dy,w) + beta*dx                  (layer.cu:616-625) */
void orc_conv_bwd_data(int n, int c, int h, int w, int k, int r, int s, int pad_h, int pad_w,
                       int stride_h, int stride_w, float alpha, const float* wt,
                       const float* dy, float beta, float* dx);
/* db = alpha*sum_{n,p,q} dy + beta*db               (layer.cu:631-637) */
void orc_conv_bwd_bias(int n, int k, int pq, float alpha, const float* dy, float beta, float* db);
/* dw = alpha*(x corr dy) + beta*dw                  (layer.cu:651-660) */
void orc_conv_bwd_filter(int n, int c, int h, int w, int k, int r, int s, int pad_h, int pad_w,
                         int stride_h, int stride_w, float alpha, const float* x,
                         const float* dy, float beta, float* dw);
/* column-major SGEMM with cuBLAS semantics          (layer.cu:677-761) */
void orc_sgemm(int transa, int transb, int m, int n, int k, float alpha, const float* A, int lda,
               const float* B, int ldb, float beta, float* C, int ldc);
void orc_relu_fwd(size_t n, const float* x, float* y);                       /* layer.cu:774-781 */
void orc_relu_bwd(size_t n, const float* y, const float* dy, const float* x, float* dx); /* 802-811 */
/* the other two activation modes the reference's Layer accepts (layer.cu:361-368); mode 1 tanh, 2 sigmoid */
void orc_act_fwd(int mode, size_t n, const float* x, float* y);
void orc_act_bwd(int mode, size_t n, const float* y, const float* dy, float* dx);
void orc_maxpool_fwd(int n, int c, int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                     const float* x, float* y);                              /* layer.cu:875-882 */
void orc_maxpool_bwd(int n, int c, int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                     const float* y, const float* dy, const float* x, float* dx); /* 903-912 */
void orc_softmax_fwd(int rows, int cols, const float* x, float* y);          /* layer.cu:824-832 */
void orc_softmax_bwd(int rows, int cols, const float* y, const float* dy, float* dx); /* 853-862 */
void orc_sub(size_t n, const float* a, const float* b, float* out);          /* network.cu:3-8 */
/* cross-channel LRN (extension; cuDNN convention: alpha is divided by the window) */
void orc_lrn_fwd(int n, int c, int hw, int win, float alpha, float beta, float k,
                 const float* x, float* y);
void orc_lrn_bwd(int n, int c, int hw, int win, float alpha, float beta, float k,
                 const float* x, const float* y, const float* dy, float* dx);
/* out[0] = 0.5*sum((y-t)^2)/rows ; out[1] = -mean_rows log y[argmax t] */
void orc_loss(int rows, int cols, const float* y, const float* label, double* out);

/* ---- topologies (network.cu:156-813) -------------------------------------- */
int orc_model_layers(int cnn_type, int batch, orc_layer_spec* out, int max_layers);
void orc_layer_out_dims(const orc_layer_spec* l, int* n, int* c, int* h, int* w);

/* ---- whole-network training step (network.cu:1056-1191) ------------------- */
typedef struct orc_net orc_net;
/* init_mode 0: He-normal weights, zero bias (seed 3000+layer);
 * init_mode 1: U(-0.01,0.01) for weights and bias (vdnn.h:10, layer.cu:925-967). */
orc_net* orc_net_create(const orc_layer_spec* specs, int num_layers, float lr, int init_mode,
                        uint64_t weight_seed_base);
void orc_net_destroy(orc_net* net);
int orc_net_num_layers(const orc_net* net);
size_t orc_net_input_size(const orc_net* net);
size_t orc_net_output_size(const orc_net* net);
void orc_net_set_input(orc_net* net, const float* input, const float* label);
void orc_net_forward(orc_net* net);
void orc_net_backward(orc_net* net);       /* includes the fused SGD update */
const float* orc_net_dst(const orc_net* net, int layer);
const float* orc_net_grad(const orc_net* net, int layer);
float* orc_net_weights(orc_net* net, int layer);
float* orc_net_bias(orc_net* net, int layer);
size_t orc_net_weight_count(const orc_net* net, int layer);
size_t orc_net_src_size(const orc_net* net, int layer);
size_t orc_net_dst_size(const orc_net* net, int layer);
void orc_net_loss(const orc_net* net, double* out2);

/* ---- allocation / offload / prefetch schedule simulator ------------------- */
enum { ORC_EV_ALLOC = 0, ORC_EV_FREE = 1, ORC_EV_OFFLOAD = 2, ORC_EV_PREFETCH = 3,
       ORC_EV_FWD_DONE = 4, ORC_EV_BWD_DONE = 5 };
enum { ORC_TAG_WEIGHT = 0, ORC_TAG_BIAS = 1, ORC_TAG_DST = 2, ORC_TAG_DIFF = 3, ORC_TAG_GRAD = 4,
       ORC_TAG_SRC = 5, ORC_TAG_WS = 6, ORC_TAG_ONES = 7, ORC_TAG_INPUT = 8, ORC_TAG_LABEL = 9,
       ORC_TAG_DXDY = 10, ORC_TAG_NONE = 11 };
typedef struct {
    int kind;          /* ORC_EV_* */
    int layer;         /* layer id (for OFFLOAD/PREFETCH: the layer whose srcData moves) */
    int tag;           /* ORC_TAG_* */
    int64_t bytes;     /* requested bytes (before rounding) / bytes copied */
    int64_t used;      /* pool bytes in use after the event */
} orc_event;
typedef struct {
    int64_t peak_bytes;
    int64_t static_bytes;
    int64_t offload_bytes;
    int64_t prefetch_bytes;
    int64_t pinned_bytes;
    int num_events;
} orc_trace_summary;
/* ws[3*l+0..2] = fwd / bwd-data / bwd-filter workspace bytes of layer l (may be NULL = 0).
 * Replays construction, `iterations` x (forward, backward).  The reference re-prefetches layer 0
 * into a fresh buffer and drops the old input allocation (network.cu:1156,1185): with
 * fix_input_leak = 0 that leak is replayed, with 1 the old input buffer is freed at the end of
 * backward.  wide_workspace = 0 sizes BASELINE's shared workspace as the reference does, as the maximum kept in an
 * int (network.cu:1025-1040: sizes beyond 2^31 wrap); 1 keeps the maximum in 64 bits.
 * Returns 0, or -1 if max_events was too small (summary still valid). */
int orc_policy_trace(const orc_layer_spec* specs, int num_layers, int vdnn_type,
                     const int64_t* ws, int iterations, int fix_input_leak, orc_event* events,
                     int max_events, orc_trace_summary* summary, int wide_workspace);
/* findPrefetchLayer (network.cu:1198-1207) over explicit tables. */
int orc_find_prefetch_layer(const int* layer_types, const unsigned char* is_offload,
                            unsigned char* is_prefetched, int cur);

#ifdef __cplusplus
}
#endif
#endif
