// C-ABI entry points for the contraction-shaped layers (CONV forward / data gradient / filter
// gradient and SGEMM).  Each call builds the operand views of gemm_operands.cuh over the caller's
// NCHW / KCRS tensors, plans a split along K when the output has too few tiles to fill the GPU,
// and runs the selected engine.  Split results are combined either with fp32 atomics straight
// into the output (MEMORY_OPT: no workspace) or through per-split partial tiles in the caller's
// workspace followed by a fixed-order reduction (PERF_OPT: deterministic).
#include <cuda_pipeline.h>
#include "common.cuh"
#include "gemm_ffma.cuh"
#include "gemm_tc.cuh"
#include "conv_tma.cuh"

namespace vdnn {
namespace {

int g_engine = VDNN_ENGINE_AUTO;
// VDNN_NO_TMA=1 in the environment keeps PERF_OPT forward / data gradient on the gather-fed kernel (A/B measurements).
const bool g_no_tma = []() { const char* v = getenv("VDNN_NO_TMA"); return v && *v && *v != '0'; }();
// VDNN_TMA_BOXES=1: forward / data gradient fetch one box of pixels per tap (conv_kernel) instead of one strip of positions
// per filter row (strip_kernel).
const bool g_tma_boxes = []() { const char* v = getenv("VDNN_TMA_BOXES"); return v && *v && *v != '0'; }();
// VDNN_TMA_WGRAD=0: the PERF_OPT filter gradient stays on the gather-fed kernel (default: TMA-fed where the shape allows).
const bool g_tma_wgrad = []() { const char* v = getenv("VDNN_TMA_WGRAD"); return !(v && *v == '0'); }();

struct SplitPlan { int splits; int k_chunk; };

// Split K so that the grid is as close to two full waves of output tiles as it can get without exceeding them
// (a third, nearly empty wave would cost as much as a full one), keeping at least 64 k per split.
SplitPlan plan_split(int M, int N, int K) {
    const int bn = g_engine == VDNN_ENGINE_FFMA ? 128 : tc::tile_n(N);
    const long tiles = static_cast<long>(ceil_div(M, 128)) * ceil_div(N, bn);
    const int sms = sm_count();
    int splits = 1;
    if (tiles < sms) {
        splits = static_cast<int>((2L * sms) / tiles);
        const int max_by_k = K / 64 > 0 ? K / 64 : 1;
        if (splits > max_by_k) splits = max_by_k;
        if (splits > 1024) splits = 1024;
        if (splits < 1) splits = 1;
    }
    int k_chunk = ceil_div(ceil_div(K, splits), 32) * 32;      // multiple of both engines' k tile
    if (k_chunk < 32) k_chunk = 32;
    SplitPlan p;
    p.k_chunk = k_chunk;
    p.splits = ceil_div(K, k_chunk);
    return p;
}

__global__ void __launch_bounds__(256) scale_dense_kernel(size_t n, float beta, float* __restrict__ out) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = beta == 0.0f ? 0.0f : beta * out[i];
}

__global__ void __launch_bounds__(256) scale_matrix_kernel(int rows, int cols, int ld, float beta, float* __restrict__ out) {
    for (int j = blockIdx.y; j < cols; j += gridDim.y)
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += gridDim.x * blockDim.x) {
            float* p = out + static_cast<size_t>(j) * ld + i;
            *p = beta == 0.0f ? 0.0f : beta * *p;
        }
}

// out[i] = alpha * sum_s partial[s][i] + beta * out[i], splits summed in index order.
__global__ void __launch_bounds__(256) reduce_partials_kernel(size_t n, int splits, float alpha, float beta,
                                                              const float* __restrict__ partial, float* __restrict__ out) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float acc = 0.0f;
        for (int s = 0; s < splits; ++s) acc += partial[static_cast<size_t>(s) * n + i];
        float v = alpha * acc;
        if (beta != 0.0f) v = fmaf(beta, out[i], v);
        out[i] = v;
    }
}

// Data gradient for layers with very few input channels (the first layer: C = 3).  As a contraction it has
// N = C columns, which would leave a 128 x 64 tensor-core tile almost empty; here one thread owns one input pixel
// and all its channels, the filter bank sits in shared memory, and dy is read with unit stride across a warp.
constexpr int SMALL_C_MAX = 4;
constexpr size_t SMALL_C_SMEM_MAX = 200 * 1024;
__global__ void __launch_bounds__(256) dgrad_small_c_kernel(int N, int C, int H, int W, int K, int R, int S, int P, int Q,
                                                            int pad_h, int pad_w, int stride_h, int stride_w, float alpha,
                                                            float beta, const float* __restrict__ w,
                                                            const float* __restrict__ dy, float* __restrict__ dx) {
    extern __shared__ float w_s[];                       // [K][C][R*S], as stored
    const int wcount = K * C * R * S;
    for (int i = threadIdx.x; i < wcount; i += blockDim.x) w_s[i] = w[i];
    __syncthreads();
    const int hw = H * W, pq = P * Q, rs = R * S;
    const long long total = static_cast<long long>(N) * hw;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int n = static_cast<int>(idx / hw), rem = static_cast<int>(idx - static_cast<long long>(n) * hw);
        const int h = rem / W, x = rem - h * W;
        float acc[SMALL_C_MAX] = {0.f, 0.f, 0.f, 0.f};
        const float* dyn = dy + static_cast<size_t>(n) * K * pq;
        // taps that connect this input pixel to an output pixel: (h + pad - r) divisible by the stride and in range
        for (int r = (h + pad_h) % stride_h; r < R; r += stride_h) {
            const int p = (h + pad_h - r) / stride_h;
            if (h + pad_h - r < 0 || p >= P) continue;
            for (int s = (x + pad_w) % stride_w; s < S; s += stride_w) {
                const int q = (x + pad_w - s) / stride_w;
                if (x + pad_w - s < 0 || q >= Q) continue;
                const float* dp = dyn + p * Q + q;
                const float* wp = w_s + r * S + s;
                for (int k = 0; k < K; ++k) {
                    const float g = __ldg(dp + static_cast<size_t>(k) * pq);
#pragma unroll
                    for (int c = 0; c < SMALL_C_MAX; ++c)
                        if (c < C) acc[c] = fmaf(g, wp[(k * C + c) * rs], acc[c]);
                }
            }
        }
        for (int c = 0; c < C; ++c) {
            float* o = dx + (static_cast<size_t>(n) * C + c) * hw + rem;
            float v = alpha * acc[c];
            if (beta != 0.0f) v = fmaf(beta, *o, v);
            *o = v;
        }
    }
}

// The same with dy staged through shared memory, for filters of at most 3 taps per stride step in each direction
// (R <= 3*stride: the first layers of VGG16, 3 x 3 / 1, and of AlexNet and OverFeat, 11 x 11 / 4).  With stride st the
// input pixels fall into st*st phase classes ((h + pad) mod st, (x + pad) mod st); inside a class, pixel (i, j) of the
// class, input (st*i + a - pad, st*j + b - pad), is a stride-1 correlation of dy with the sub-filter
// w[a + st*u][b + st*v], u, v < 3 (zero where that leaves the filter):  dx = sum_{u,v} dy[i - u][j - v] * w[a+st*u][b+st*v].
// A CTA of TW threads owns an 8 x TW tile of one class of one image; dy arrives 8 filters at a time as the tile plus
// its halo; every thread owns one column of the tile and keeps the 10 staged values of a column in registers, so each
// shared-memory load feeds up to 8 rows x 3 taps x C channels.  The sub-filters sit in shared memory as one float4
// (channels 0..3) per filter and tap.
constexpr int S1_TH = 8, S1_KC = 8;
template <int TW, int CC>
__global__ void __launch_bounds__(TW) dgrad_small_c_phase_kernel(int C, int H, int W, int K, int R, int S, int P, int Q, int pad_h,
                                                                 int pad_w, int st, float alpha, float beta,
                                                                 const float* __restrict__ w, const float* __restrict__ dy,
                                                                 float* __restrict__ dx) {
    extern __shared__ float4 s1_smem[];
    constexpr int ROWS = S1_TH + 2, PITCH = TW + 2;
    float4* w_s = s1_smem;                                            // [K][3*3]
    float* dy_s = reinterpret_cast<float*>(s1_smem + K * 9);           // [S1_KC][ROWS][PITCH]
    const int tx = threadIdx.x;
    const int cls = blockIdx.z % (st * st), n = blockIdx.z / (st * st), pa = cls / st, pb = cls - pa * st;
    const int i0 = blockIdx.y * S1_TH, j0 = blockIdx.x * TW;          // tile origin in class coordinates
    const int rs = R * S;
    for (int i = tx; i < K * 9; i += TW) {
        const int k = i / 9, t = i - k * 9, u = t / 3, v = t - u * 3;
        const int r = pa + st * u, sx = pb + st * v;
        float wv[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < R && sx < S)
            for (int c = 0; c < C; ++c) wv[c] = w[(k * C + c) * rs + r * S + sx];
        w_s[i] = make_float4(wv[0], wv[1], wv[2], wv[3]);
    }
    float acc[S1_TH][CC];
#pragma unroll
    for (int i = 0; i < S1_TH; ++i)
#pragma unroll
        for (int c = 0; c < CC; ++c) acc[i][c] = 0.0f;
    // tile row tr holds dy row p0 + tr, tile column tc holds dy column q0 + tc
    const int p0 = i0 - 2, q0 = j0 - 2;
    const float* dyn = dy + static_cast<size_t>(n) * K * P * Q;
    const int q_a = q0 + tx, col_b = TW + tx, q_b = q0 + col_b;
    const bool ok_a = static_cast<unsigned>(q_a) < static_cast<unsigned>(Q);
    const bool has_b = col_b < PITCH, ok_b = has_b && static_cast<unsigned>(q_b) < static_cast<unsigned>(Q);
    for (int k0 = 0; k0 < K; k0 += S1_KC) {
        const int kc = min(S1_KC, K - k0);
        __syncthreads();                                   // the previous chunk has been consumed (first pass: w_s is complete)
        // asynchronous 4-byte copies straight into shared memory (zero-filled outside dy): all of a chunk's loads are
        // in flight at once.  Thread tx copies tile column tx of every row (the first two threads also the halo
        // columns on the right), so the column tests and offsets are computed once.
        for (int kk = 0; kk < kc; ++kk) {
            const float* src = dyn + static_cast<size_t>(k0 + kk) * P * Q;
            float* dst = dy_s + kk * ROWS * PITCH;
#pragma unroll
            for (int tr = 0; tr < ROWS; ++tr) {
                const int p = p0 + tr;
                const bool row_ok = static_cast<unsigned>(p) < static_cast<unsigned>(P);
                const float* rowp = src + (row_ok ? p : 0) * Q;
                const bool a = row_ok && ok_a;
                __pipeline_memcpy_async(dst + tr * PITCH + tx, rowp + (a ? q_a : 0), sizeof(float), a ? 0 : sizeof(float));
                if (has_b) {
                    const bool b2 = row_ok && ok_b;
                    __pipeline_memcpy_async(dst + tr * PITCH + col_b, rowp + (b2 ? q_b : 0), sizeof(float), b2 ? 0 : sizeof(float));
                }
            }
        }
        __pipeline_commit();
        __pipeline_wait_prior(0);
        __syncthreads();
        for (int kk = 0; kk < kc; ++kk) {
            const float* tile = dy_s + kk * ROWS * PITCH;
            const float4* wk = w_s + (k0 + kk) * 9;
#pragma unroll
            for (int v = 0; v < 3; ++v) {
                float colv[ROWS];
#pragma unroll
                for (int tr = 0; tr < ROWS; ++tr) colv[tr] = tile[tr * PITCH + tx + (2 - v)];
#pragma unroll
                for (int u = 0; u < 3; ++u) {
                    const float4 w4 = wk[u * 3 + v];
                    const float wc[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                    for (int i = 0; i < S1_TH; ++i) {
                        const float g = colv[i + 2 - u];
#pragma unroll
                        for (int c = 0; c < CC; ++c) acc[i][c] = fmaf(g, wc[c], acc[i][c]);
                    }
                }
            }
        }
    }
    const int x = st * (j0 + tx) + pb - pad_w;
    if (x < 0 || x >= W) return;
#pragma unroll
    for (int i = 0; i < S1_TH; ++i) {
        const int h = st * (i0 + i) + pa - pad_h;
        if (h < 0 || h >= H) continue;
#pragma unroll
        for (int c = 0; c < CC; ++c) {
            if (c >= C) break;
            float* o = dx + ((static_cast<size_t>(n) * C + c) * H + h) * W + x;
            float v = alpha * acc[i][c];
            if (beta != 0.0f) v = fmaf(beta, *o, v);
            *o = v;
        }
    }
}

template <int TW, int CC>
int launch_dgrad_small_c_phase(const vdnn_conv_desc* d, int P, int Q, float alpha, float beta, const float* w, const float* dy,
                               float* dx, cudaStream_t stream) {
    const int st = d->stride_h;
    const size_t smem = static_cast<size_t>(d->k) * 9 * sizeof(float4) +
                        static_cast<size_t>(S1_KC) * (S1_TH + 2) * (TW + 2) * sizeof(float);
    const long long slices = static_cast<long long>(d->n) * st * st;
    if (smem > 96 * 1024 || slices > 65535) return VDNN_ERR_UNSUPPORTED;
    auto kern = dgrad_small_c_phase_kernel<TW, CC>;
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    if (VDNN_ONCE_PER_DEVICE(dev))
        VDNN_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    // class coordinates run over every i with 0 <= st*i + a - pad < H for some phase a: 0 .. (H - 1 + pad) / st
    const int hv = (d->h - 1 + d->pad_h) / st + 1, wv = (d->w - 1 + d->pad_w) / st + 1;
    dim3 grid(ceil_div(wv, TW), ceil_div(hv, S1_TH), static_cast<unsigned>(slices));
    kern<<<grid, TW, smem, stream>>>(d->c, d->h, d->w, d->k, d->r, d->s, P, Q, d->pad_h, d->pad_w, st, alpha, beta, w, dy, dx);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

// A convolution whose filter covers the whole (unpadded) input produces one output pixel per image: it is a fully
// connected layer, y[n][k] = sum_j w[k][j] x[n][j] with j running over (c, r, s) -- both operands contiguous in j.
bool is_full_extent(const vdnn_conv_desc* d) {
    return d->pad_h == 0 && d->pad_w == 0 && d->h == d->r && d->w == d->s;
}

// PERF_OPT scratch for the weight operand of forward (N = K filters) and data gradient (N = C channels): images of
// its shared-memory tiles, split into tf32 hi / lo halves, that the kernel fetches with bulk copies.
size_t packed_weight_bytes(const vdnn_conv_desc* d, int op) {
    const int red = (op == VDNN_CONV_FWD ? d->c : d->k) * d->r * d->s;
    return tc::bulk_bytes(op == VDNN_CONV_FWD ? d->k : d->c, red);
}

// PERF_OPT scratch for the dy operand of the filter gradient (N = K filters as tile columns, reduction over the
// N*P*Q pixels): the same tile images.  Only where dy fills at least 128 columns: with fewer, the columns are the
// small part of the producers' work and the images (twice the bytes of dy) would not pay for themselves.
size_t packed_dy_bytes(const vdnn_conv_desc* d, int P, int Q) {
    return d->k >= 128 ? tc::bulk_bytes(d->k, d->n * P * Q) : 0;
}

// Forward and data gradient of a stride-1 convolution whose reduction channels (C for forward, K for the data
// gradient) come in whole blocks of 32 run on the TMA-fed engine in PERF_OPT: the gathered tensor is rewritten once into
// two channels-last images (tf32 hi / lo halves) in workspace and the kernel fetches its operand tiles by tensor copies.
bool tma_shape(const vdnn_conv_desc* d, int op) {
    if (op != VDNN_CONV_FWD && op != VDNN_CONV_BWD_DATA) return false;
    if (d->stride_h != 1 || d->stride_w != 1 || is_full_extent(d)) return false;
    if (op == VDNN_CONV_BWD_DATA && d->c <= SMALL_C_MAX) return false;          // the first layer has its own kernels
    if ((op == VDNN_CONV_FWD ? d->c : d->k) % 32 != 0) return false;
    // Only where the output has enough tiles to fill the GPU without splitting the reduction: the few-tile layers (14 x 14
    // maps) stay on the gather kernel, which splits along k at a finer grain and needs no operand images.  With the
    // engine forced to VDNN_ENGINE_TCGEN05 every eligible shape takes the TMA-fed path (small shapes in the tests).
    if (g_engine == VDNN_ENGINE_TCGEN05) return true;
    const int P = (d->h + 2 * d->pad_h - d->r) / d->stride_h + 1, Q = (d->w + 2 * d->pad_w - d->s) / d->stride_w + 1;
    const long long pixels = static_cast<long long>(d->n) * (op == VDNN_CONV_FWD ? P * Q : d->h * d->w);
    const int cols = op == VDNN_CONV_FWD ? d->k : d->c;
    return (pixels + 127) / 128 * ((cols + 255) / 256) >= sm_count();
}

bool tma_wgrad_shape(const vdnn_conv_desc* d) {
    return g_tma_wgrad && !g_no_tma && d->stride_h == 1 && d->stride_w == 1 && !is_full_extent(d) && d->c % 32 == 0 && d->k % 32 == 0;
}

tma::WgradProblem wgrad_problem(const vdnn_conv_desc* d, int P, int Q) {
    return tma::WgradProblem{d->n, d->c, d->h, d->w, d->k, P, Q, d->r, d->s, d->pad_h, d->pad_w};
}

// Operand images of at most this many bytes are kept in workspace at a time.
constexpr size_t TMA_IMAGE_BUDGET = static_cast<size_t>(1) << 30;
int tma_slab_images(int n, size_t bytes_per_image) {
    if (bytes_per_image * n <= TMA_IMAGE_BUDGET) return n;
    const size_t fit = TMA_IMAGE_BUDGET / bytes_per_image;
    return fit > 1 ? static_cast<int>(fit) : 1;
}

tma::Problem tma_problem(const vdnn_conv_desc* d, int op, int P, int Q) {
    if (op == VDNN_CONV_FWD) return tma::Problem{d->n, d->c, d->h, d->w, P, Q, d->k, d->r, d->s, 1, -d->pad_h, -d->pad_w};
    // dx[h][w] = sum over taps of dy[h + pad - r][w + pad - s] (stride 1)
    return tma::Problem{d->n, d->k, P, Q, d->h, d->w, d->c, d->r, d->s, -1, d->pad_h, d->pad_w};
}

bool tma_use_strips(const tma::Problem& q) { return !g_tma_boxes && tma::strip_geometry(q).ok; }

// Bytes of the two operand images of `images` images of the problem, in the layout the chosen kernel reads.
size_t tma_operand_bytes(const tma::Problem& q, int images) {
    tma::Problem part = q;
    part.n = images;
    return tma_use_strips(q) ? tma::strip_image_bytes(part) : tma::image_bytes(images, q.cin, q.in_h, q.in_w);
}

size_t tma_image_bytes(const vdnn_conv_desc* d, int op, int P, int Q) {
    const tma::Problem q = tma_problem(d, op, P, Q);
    return tma_operand_bytes(q, tma_slab_images(d->n, tma_operand_bytes(q, 1)));
}

int stream_blocks(size_t n) {
    size_t want = ceil_div<size_t>(n, 256);
    const size_t cap = static_cast<size_t>(sm_count()) * 8;
    if (want > cap) want = cap;
    return want ? static_cast<int>(want) : 1;
}

template <class OpA, class OpB, bool AKC, bool BKC>
int run_engine(const OpA& a, const OpB& b, const Epilogue& epi, int M, int N, int K, int splits, int k_chunk,
               cudaStream_t stream, char* b_tiles = nullptr) {
    if (g_engine != VDNN_ENGINE_FFMA && tc::supported<OpA, OpB>(M, N, K)) {
        return tc::launch<OpA, OpB, AKC, BKC>(a, b, epi, M, N, K, splits, k_chunk, stream, b_tiles);
    }
    if (g_engine == VDNN_ENGINE_TCGEN05) return VDNN_ERR_UNSUPPORTED;
    return ffma::launch<OpA, OpB, AKC, BKC>(a, b, epi, M, N, K, splits, k_chunk, stream);
}

// `epi` arrives configured for a direct store (out, alpha, beta, bias, addressing).
// dense_elems > 0 says the output is one dense block of that many floats (needed for PARTIAL).
template <class OpA, class OpB, bool AKC, bool BKC>
int contract(const OpA& a, const OpB& b, Epilogue epi, int M, int N, int K, size_t dense_elems, int ld_rows,
             int algo_mode, void* ws, size_t ws_bytes, cudaStream_t stream, char* b_tiles = nullptr) {
    SplitPlan plan = plan_split(M, N, K);
    if (epi.bias) { plan.splits = 1; plan.k_chunk = ceil_div(K, 32) * 32; }
    if (plan.splits == 1) {
        epi.mode = EPI_DIRECT;
        return run_engine<OpA, OpB, AKC, BKC>(a, b, epi, M, N, K, 1, plan.k_chunk, stream, b_tiles);
    }
    if (algo_mode == VDNN_ALGO_PERF_OPT && dense_elems > 0) {
        const size_t need = static_cast<size_t>(plan.splits) * dense_elems * sizeof(float);
        if (!ws || ws_bytes < need) return VDNN_ERR_WORKSPACE;
        Epilogue part = epi;
        part.mode = EPI_PARTIAL;
        part.out = static_cast<float*>(ws);
        part.partial_stride = dense_elems;
        int st = run_engine<OpA, OpB, AKC, BKC>(a, b, part, M, N, K, plan.splits, plan.k_chunk, stream, b_tiles);
        if (st != VDNN_OK) return st;
        reduce_partials_kernel<<<stream_blocks(dense_elems), 256, 0, stream>>>(dense_elems, plan.splits, epi.alpha, epi.beta,
                                                                             static_cast<const float*>(ws), epi.out);
        VDNN_LAUNCHED();
        return VDNN_OK;
    }
    // zero-workspace path: out = beta * out, then every split adds alpha * partial atomically
    if (epi.beta != 1.0f) {
        if (dense_elems > 0) {
            if (epi.beta == 0.0f) VDNN_CUDA(cudaMemsetAsync(epi.out, 0, dense_elems * sizeof(float), stream));
            else {
                scale_dense_kernel<<<stream_blocks(dense_elems), 256, 0, stream>>>(dense_elems, epi.beta, epi.out);
                VDNN_LAUNCHED();
            }
        } else {
            dim3 grid(ceil_div(M, 256), N < 65535 ? N : 65535);
            scale_matrix_kernel<<<grid, 256, 0, stream>>>(M, N, ld_rows, epi.beta, epi.out);
            VDNN_LAUNCHED();
        }
    }
    epi.mode = EPI_ATOMIC;
    return run_engine<OpA, OpB, AKC, BKC>(a, b, epi, M, N, K, plan.splits, plan.k_chunk, stream, b_tiles);
}

// The TMA-fed contraction with the split handling of contract(): `ws` holds the images, then the per-split partials.
// Layers whose images would pass TMA_IMAGE_BUDGET are walked in slabs of whole images (transform a slab, contract it,
// reuse the image buffer), so the workspace stays at the budget whatever the batch size.
int contract_tma(const tma::Problem& q, const float* src, const char* b_tiles, Epilogue epi, size_t out_elems, char* ws,
                 size_t ws_bytes, cudaStream_t stream) {
    const bool strips = tma_use_strips(q);
    const int slab = tma_slab_images(q.n, tma_operand_bytes(q, 1));
    const size_t img = tma_operand_bytes(q, slab);
    if (ws_bytes < img) return VDNN_ERR_WORKSPACE;
    const int M = q.n * q.out_h * q.out_w, K = q.R * q.S * q.cin;
    SplitPlan plan = plan_split(M, q.n_cols, K);
    if (epi.bias || slab < q.n) { plan.splits = 1; plan.k_chunk = K; }
    // the strip kernel splits the reduction between (filter row, channel block) groups of S k blocks
    const int groups = q.R * (q.cin / 32);
    int group_chunk = ceil_div(plan.k_chunk / 32, q.S);
    if (group_chunk < 1) group_chunk = 1;
    const int splits = strips ? ceil_div(groups, group_chunk) : plan.splits;
    auto run = [&](const tma::Problem& part, const float* s, float* o, const float* bias, float alpha, float beta, int mode) {
        return strips ? tma::strip_launch(part, s, ws, b_tiles, o, bias, alpha, beta, mode, out_elems, splits, group_chunk, stream)
                      : tma::launch(part, s, ws, b_tiles, o, bias, alpha, beta, mode, out_elems, splits, plan.k_chunk, stream);
    };
    if (splits == 1) {
        const size_t src_img = static_cast<size_t>(q.cin) * q.in_h * q.in_w, out_img = static_cast<size_t>(q.n_cols) * q.out_h * q.out_w;
        for (int n0 = 0; n0 < q.n; n0 += slab) {
            tma::Problem part = q;
            part.n = min(slab, q.n - n0);
            const int st = run(part, src + n0 * src_img, epi.out + n0 * out_img, epi.bias, epi.alpha, epi.beta, EPI_DIRECT);
            if (st != VDNN_OK) return st;
        }
        return VDNN_OK;
    }
    const size_t need = static_cast<size_t>(splits) * out_elems * sizeof(float);
    if (ws_bytes - img < need) return VDNN_ERR_WORKSPACE;
    float* partial = reinterpret_cast<float*>(ws + img);
    const int st = run(q, src, partial, nullptr, 1.0f, 0.0f, EPI_PARTIAL);
    if (st != VDNN_OK) return st;
    reduce_partials_kernel<<<stream_blocks(out_elems), 256, 0, stream>>>(out_elems, splits, epi.alpha, epi.beta, partial, epi.out);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

// Filter gradient on the TMA-fed engine, in slabs of whole images where the four operand images would pass the budget:
// every slab adds its pixels' share, dw = alpha * (sum over slabs) + beta * dw.
int wgrad_tma(const tma::WgradProblem& q, const float* x, const float* dy, char* ws, size_t ws_bytes, float* dw, float alpha,
              float beta, cudaStream_t stream, float* bias_sums = nullptr, float bias_scale = 0.0f) {
    tma::WgradProblem one = q;
    one.n = 1;
    const int slab = tma_slab_images(q.n, tma::wgrad_image_bytes(one));
    tma::WgradProblem part = q;
    part.n = slab;
    if (ws_bytes < tma::wgrad_image_bytes(part) + tma::wgrad_partial_bytes(part)) return VDNN_ERR_WORKSPACE;
    const size_t x_img = static_cast<size_t>(q.c) * q.h * q.w, dy_img = static_cast<size_t>(q.k) * q.p * q.q;
    const size_t elems = static_cast<size_t>(q.k) * q.c * q.R * q.S;
    for (int n0 = 0; n0 < q.n; n0 += slab) {
        part.n = min(slab, q.n - n0);
        int splits = 1;
        float* partial = nullptr;
        const float b = n0 == 0 ? beta : 1.0f;
        const int st = tma::wgrad_launch(part, x + n0 * x_img, dy + n0 * dy_img, ws, dw, alpha, b, stream, &splits, &partial,
                                         bias_sums, bias_scale);
        if (st != VDNN_OK) return st;
        if (splits > 1) {
            reduce_partials_kernel<<<stream_blocks(elems), 256, 0, stream>>>(elems, splits, alpha, b, partial, dw);
            VDNN_LAUNCHED();
        }
    }
    return VDNN_OK;
}

// Filter gradient (and bias gradient) for layers with very few input channels and a 3 x 3 / stride-1 filter (VGG16's
// first layer: C = 3).  As a contraction it has 27 rows: a 128-row tensor-core tile is four fifths empty and the gather
// that feeds it costs more than the arithmetic.  Here a block walks tiles of 8 x 32 output pixels of one image; dy of
// 64 filters and the x halo lie in shared memory; thread (filter kk, row set g) keeps the sums of its filter for up to
// three (channel, filter row) pairs x three taps in registers, reading four dy values (one LDS.128) and, per pair, six x
// values (warp-uniform, broadcast) for 12 multiply-adds.  Every block leaves its sums as one partial result
// (partial_w[block][K][C][3][3], partial_b[block][K]); reduce_partials_kernel adds the blocks up in index order.
constexpr int WSC_TR = 8, WSC_TC = 32, WSC_KT = 64;
constexpr int WSC_DY_PITCH = WSC_TR * WSC_TC + 4;        // floats per filter in shared memory (+4: conflict-free LDS.128)
constexpr int WSC_X_PITCH = WSC_TC + 4;                  // 34 columns of halo, padded to a multiple of four floats

template <int C>
__global__ void __launch_bounds__(256, 3) wgrad_small_c_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                               float* __restrict__ partial_w, float* __restrict__ partial_b, int N, int H,
                                                               int W, int K, int P, int Q, int pad_h, int pad_w, int tiles_y,
                                                               int tiles_x) {
    extern __shared__ float wsc_smem[];
    float* dyS = wsc_smem;                                               // [WSC_KT][WSC_DY_PITCH]
    float* xS = wsc_smem + WSC_KT * WSC_DY_PITCH;                        // [C][WSC_TR + 2][WSC_X_PITCH]
    constexpr int PAIRS = C * 3;                                         // (channel, filter row)
    constexpr int MINE = (PAIRS + 3) / 4;                                // per row set
    const int t = threadIdx.x, kk = t & 63, g = t >> 6;
    const int k0 = blockIdx.y * WSC_KT;
    float acc[MINE][3];
#pragma unroll
    for (int j = 0; j < MINE; ++j) acc[j][0] = acc[j][1] = acc[j][2] = 0.0f;
    float bsum = 0.0f;
    const long long tiles = static_cast<long long>(N) * tiles_y * tiles_x;
    const size_t pq = static_cast<size_t>(P) * Q, hw = static_cast<size_t>(H) * W;
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int n = static_cast<int>(tile / (tiles_y * tiles_x)), rem = static_cast<int>(tile - static_cast<long long>(n) * tiles_y * tiles_x);
        const int p0 = (rem / tiles_x) * WSC_TR, q0 = (rem % tiles_x) * WSC_TC;
        __syncthreads();                                                 // the last tile has been consumed
        // dy: 64 filters x 8 rows x 32 columns, float4 along a row (Q is a multiple of 4: checked by the host)
        for (int i = t; i < WSC_KT * WSC_TR * (WSC_TC / 4); i += 256) {
            const int c4 = i % (WSC_TC / 4), row = (i / (WSC_TC / 4)) % WSC_TR, k = i / (WSC_TC / 4 * WSC_TR);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + k < K && p0 + row < P && q0 + c4 * 4 < Q)
                v = __ldg(reinterpret_cast<const float4*>(dy + (static_cast<size_t>(n) * K + k0 + k) * pq + static_cast<size_t>(p0 + row) * Q + q0) + c4);
            *reinterpret_cast<float4*>(dyS + k * WSC_DY_PITCH + row * WSC_TC + c4 * 4) = v;
        }
        // x halo: rows p0 - pad_h .. + 9, columns q0 - pad_w .. + 33
        for (int i = t; i < C * (WSC_TR + 2) * (WSC_TC + 2); i += 256) {
            const int col = i % (WSC_TC + 2), row = (i / (WSC_TC + 2)) % (WSC_TR + 2), c = i / ((WSC_TC + 2) * (WSC_TR + 2));
            const int ih = p0 - pad_h + row, iw = q0 - pad_w + col;
            float v = 0.0f;
            if (static_cast<unsigned>(ih) < static_cast<unsigned>(H) && static_cast<unsigned>(iw) < static_cast<unsigned>(W))
                v = __ldg(x + (static_cast<size_t>(n) * C + c) * hw + static_cast<size_t>(ih) * W + iw);
            xS[(c * (WSC_TR + 2) + row) * WSC_X_PITCH + col] = v;
        }
        __syncthreads();
        const float* dk = dyS + kk * WSC_DY_PITCH;
#pragma unroll 2
        for (int pr = 0; pr < WSC_TR; ++pr) {
#pragma unroll
            for (int q4 = 0; q4 < WSC_TC / 4; ++q4) {
                const float4 d = *reinterpret_cast<const float4*>(dk + pr * WSC_TC + q4 * 4);
                if (g == 0) bsum += (d.x + d.y) + (d.z + d.w);
#pragma unroll
                for (int j = 0; j < MINE; ++j) {
                    const int pair = g + 4 * j;                          // warp-uniform
                    if (pair < PAIRS) {
                        const int c = pair / 3, r = pair - c * 3;
                        const float* xr = xS + (c * (WSC_TR + 2) + pr + r) * WSC_X_PITCH + q4 * 4;
                        const float4 a = *reinterpret_cast<const float4*>(xr);
                        const float2 b = *reinterpret_cast<const float2*>(xr + 4);
                        acc[j][0] = fmaf(d.x, a.x, fmaf(d.y, a.y, fmaf(d.z, a.z, fmaf(d.w, a.w, acc[j][0]))));
                        acc[j][1] = fmaf(d.x, a.y, fmaf(d.y, a.z, fmaf(d.z, a.w, fmaf(d.w, b.x, acc[j][1]))));
                        acc[j][2] = fmaf(d.x, a.z, fmaf(d.y, a.w, fmaf(d.z, b.x, fmaf(d.w, b.y, acc[j][2]))));
                    }
                }
            }
        }
    }
    if (k0 + kk < K) {
        float* o = partial_w + (static_cast<size_t>(blockIdx.x) * K + k0 + kk) * (C * 9);
#pragma unroll
        for (int j = 0; j < MINE; ++j) {
            const int pair = g + 4 * j;
            if (pair < PAIRS) { o[pair * 3 + 0] = acc[j][0]; o[pair * 3 + 1] = acc[j][1]; o[pair * 3 + 2] = acc[j][2]; }
        }
        if (g == 0) partial_b[static_cast<size_t>(blockIdx.x) * K + k0 + kk] = bsum;
    }
}

bool wgrad_small_c_shape(const vdnn_conv_desc* d, int Q) {
    return d->c <= SMALL_C_MAX && d->c >= 1 && d->r == 3 && d->s == 3 && d->stride_h == 1 && d->stride_w == 1 && Q % 4 == 0 && d->k % 4 == 0 &&
           !is_full_extent(d);
}
int wgrad_small_c_blocks() { return sm_count() * 3; }
size_t wgrad_small_c_bytes(const vdnn_conv_desc* d) {
    return static_cast<size_t>(wgrad_small_c_blocks()) * d->k * (d->c * 9 + 1) * sizeof(float);
}

// dw = alpha * (x corr dy) + beta * dw and, when db is given, db = alpha_b * sum dy + beta_b * db.
int wgrad_small_c(const vdnn_conv_desc* d, int P, int Q, const float* x, const float* dy, float alpha, float beta, float* dw, float alpha_b,
                  float beta_b, float* db, char* ws, size_t ws_bytes, cudaStream_t s) {
    if (ws_bytes < wgrad_small_c_bytes(d)) return VDNN_ERR_WORKSPACE;
    const int blocks = wgrad_small_c_blocks();
    float* partial_w = reinterpret_cast<float*>(ws);
    float* partial_b = partial_w + static_cast<size_t>(blocks) * d->k * d->c * 9;
    const int tiles_y = ceil_div(P, WSC_TR), tiles_x = ceil_div(Q, WSC_TC);
    const size_t smem = (static_cast<size_t>(WSC_KT) * WSC_DY_PITCH + static_cast<size_t>(d->c) * (WSC_TR + 2) * WSC_X_PITCH) * sizeof(float);
    dim3 grid(blocks, ceil_div(d->k, WSC_KT));
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
#define WSC_LAUNCH(CC)                                                                                                                   \
    {                                                                                                                                   \
        if (VDNN_ONCE_PER_DEVICE(dev)) VDNN_CUDA(cudaFuncSetAttribute(wgrad_small_c_kernel<CC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024)); \
        wgrad_small_c_kernel<CC><<<grid, 256, smem, s>>>(x, dy, partial_w, partial_b, d->n, d->h, d->w, d->k, P, Q, d->pad_h, d->pad_w, tiles_y, tiles_x); \
    }
    switch (d->c) {
    case 1: WSC_LAUNCH(1) break;
    case 2: WSC_LAUNCH(2) break;
    case 3: WSC_LAUNCH(3) break;
    default: WSC_LAUNCH(4) break;
    }
#undef WSC_LAUNCH
    VDNN_LAUNCHED();
    const size_t we = static_cast<size_t>(d->k) * d->c * 9;
    reduce_partials_kernel<<<stream_blocks(we), 256, 0, s>>>(we, blocks, alpha, beta, partial_w, dw);
    VDNN_LAUNCHED();
    if (db) {
        reduce_partials_kernel<<<stream_blocks(d->k), 256, 0, s>>>(static_cast<size_t>(d->k), blocks, alpha_b, beta_b, partial_b, db);
        VDNN_LAUNCHED();
    }
    return VDNN_OK;
}

// Forward for the same few-channel 3 x 3 / stride-1 layers: y[n][k][p][q] = alpha * sum x * w + bias[k] + beta * y.  A block
// computes a tile of 8 x 32 output pixels of one image for 64 filters; the x halo and the 64 x (C * 9) weights (stored
// tap-major, filter innermost) lie in shared memory; a thread owns four neighbouring pixels of one row and 16 filters:
// 64 accumulators, per (channel, filter row) six x values and per tap 16 weights (warp-uniform LDS.128, broadcast) for 64
// multiply-adds.  The reduction has 27 terms: as a tensor-core tile it would be one k block per CTA.
template <int C>
__global__ void __launch_bounds__(256, 2) fwd_small_c_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                             const float* __restrict__ bias, float* __restrict__ y, int N, int H, int W,
                                                             int K, int P, int Q, int pad_h, int pad_w, int tiles_y, int tiles_x, float alpha,
                                                             float beta) {
    extern __shared__ float fsc_smem[];
    float* wS = fsc_smem;                                                // [C * 9][WSC_KT]
    float* xS = fsc_smem + C * 9 * WSC_KT;                               // [C][WSC_TR + 2][WSC_X_PITCH]
    const int t = threadIdx.x, quad = t & 63, kg = t >> 6;               // pixel quad of the tile, group of 16 filters
    const int pr = quad >> 3, q4 = quad & 7;
    const int k0 = blockIdx.y * WSC_KT;
    for (int i = t; i < C * 9 * WSC_KT; i += 256) {
        const int k = i % WSC_KT, tap = i / WSC_KT;                     // tap = c * 9 + r * 3 + s
        wS[i] = k0 + k < K ? __ldg(w + static_cast<size_t>(k0 + k) * (C * 9) + tap) : 0.0f;
    }
    const long long tiles = static_cast<long long>(N) * tiles_y * tiles_x;
    const size_t pq = static_cast<size_t>(P) * Q, hw = static_cast<size_t>(H) * W;
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int n = static_cast<int>(tile / (tiles_y * tiles_x)), rem = static_cast<int>(tile - static_cast<long long>(n) * tiles_y * tiles_x);
        const int p0 = (rem / tiles_x) * WSC_TR, q0 = (rem % tiles_x) * WSC_TC;
        __syncthreads();                                                 // the last tile's halo has been consumed (and wS is written)
        for (int i = t; i < C * (WSC_TR + 2) * (WSC_TC + 2); i += 256) {
            const int col = i % (WSC_TC + 2), row = (i / (WSC_TC + 2)) % (WSC_TR + 2), c = i / ((WSC_TC + 2) * (WSC_TR + 2));
            const int ih = p0 - pad_h + row, iw = q0 - pad_w + col;
            float v = 0.0f;
            if (static_cast<unsigned>(ih) < static_cast<unsigned>(H) && static_cast<unsigned>(iw) < static_cast<unsigned>(W))
                v = __ldg(x + (static_cast<size_t>(n) * C + c) * hw + static_cast<size_t>(ih) * W + iw);
            xS[(c * (WSC_TR + 2) + row) * WSC_X_PITCH + col] = v;
        }
        __syncthreads();
        float acc[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int r = 0; r < 3; ++r) {
                const float* xr = xS + (c * (WSC_TR + 2) + pr + r) * WSC_X_PITCH + q4 * 4;
                const float4 a = *reinterpret_cast<const float4*>(xr);
                const float2 b = *reinterpret_cast<const float2*>(xr + 4);
                const float xv[6] = {a.x, a.y, a.z, a.w, b.x, b.y};
#pragma unroll
                for (int sx = 0; sx < 3; ++sx) {
                    const float* wk = wS + ((c * 3 + r) * 3 + sx) * WSC_KT + kg * 16;
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        const float4 wv = *reinterpret_cast<const float4*>(wk + j4 * 4);
                        const float ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[j4 * 4 + j][i] = fmaf(ww[j], xv[sx + i], acc[j4 * 4 + j][i]);
                    }
                }
            }
        const int p = p0 + pr, q = q0 + q4 * 4;
        if (p < P && q < Q) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int k = k0 + kg * 16 + j;
                if (k >= K) break;
                float4* o = reinterpret_cast<float4*>(y + (static_cast<size_t>(n) * K + k) * pq + static_cast<size_t>(p) * Q + q);
                const float bk = bias ? __ldg(bias + k) : 0.0f;
                float4 v = make_float4(fmaf(alpha, acc[j][0], bk), fmaf(alpha, acc[j][1], bk), fmaf(alpha, acc[j][2], bk), fmaf(alpha, acc[j][3], bk));
                if (beta != 0.0f) { const float4 old = *o; v.x = fmaf(beta, old.x, v.x); v.y = fmaf(beta, old.y, v.y); v.z = fmaf(beta, old.z, v.z); v.w = fmaf(beta, old.w, v.w); }
                *o = v;
            }
        }
    }
}

int fwd_small_c(const vdnn_conv_desc* d, int P, int Q, float alpha, const float* x, const float* w, const float* bias, float beta, float* y,
                cudaStream_t s) {
    const int tiles_y = ceil_div(P, WSC_TR), tiles_x = ceil_div(Q, WSC_TC);
    const size_t smem = (static_cast<size_t>(d->c) * 9 * WSC_KT + static_cast<size_t>(d->c) * (WSC_TR + 2) * WSC_X_PITCH) * sizeof(float);
    const long long tiles = static_cast<long long>(d->n) * tiles_y * tiles_x;
    long long blocks = static_cast<long long>(sm_count()) * 2;
    if (blocks > tiles) blocks = tiles;
    dim3 grid(static_cast<unsigned>(blocks), ceil_div(d->k, WSC_KT));
    switch (d->c) {
    case 1: fwd_small_c_kernel<1><<<grid, 256, smem, s>>>(x, w, bias, y, d->n, d->h, d->w, d->k, P, Q, d->pad_h, d->pad_w, tiles_y, tiles_x, alpha, beta); break;
    case 2: fwd_small_c_kernel<2><<<grid, 256, smem, s>>>(x, w, bias, y, d->n, d->h, d->w, d->k, P, Q, d->pad_h, d->pad_w, tiles_y, tiles_x, alpha, beta); break;
    case 3: fwd_small_c_kernel<3><<<grid, 256, smem, s>>>(x, w, bias, y, d->n, d->h, d->w, d->k, P, Q, d->pad_h, d->pad_w, tiles_y, tiles_x, alpha, beta); break;
    default: fwd_small_c_kernel<4><<<grid, 256, smem, s>>>(x, w, bias, y, d->n, d->h, d->w, d->k, P, Q, d->pad_h, d->pad_w, tiles_y, tiles_x, alpha, beta); break;
    }
    VDNN_LAUNCHED();
    return VDNN_OK;
}

// ---- one image pass over dy for both gradients --------------------------------------------------------------------
// The data gradient's strip engine and the filter gradient both read dy as channels-last tf32 hi / lo images; the strip
// layout (a padded position list) contains the plain image as a strided view, so where both gradients of a layer run on
// the TMA-fed kernels one pass writes dy once (and forms the bias sums), and the two kernels run slab by slab from it.
bool bwd_shared_shape(const vdnn_conv_desc* d, int P, int Q) {
    if (g_no_tma || !tma_shape(d, VDNN_CONV_BWD_DATA) || !tma_wgrad_shape(d)) return false;
    return tma_use_strips(tma_problem(d, VDNN_CONV_BWD_DATA, P, Q));
}

// The filter gradient of layers with at most 128 filters can run on the two position lists themselves
// (conv_tma_wstrip.cuh: one strip of x per filter row instead of one box per tap).  VDNN_WGRAD_STRIPS=0 switches it off.
bool g_wgrad_strips = []() { const char* e = getenv("VDNN_WGRAD_STRIPS"); return !e || e[0] != '0'; }();

bool bwd_wstrip_shape(const vdnn_conv_desc* d, int P, int Q) {
    return g_wgrad_strips && tma::wstrip_filters_ok(d->k, d->c) &&
           tma::wstrip_ok(tma_problem(d, VDNN_CONV_FWD, P, Q), tma_problem(d, VDNN_CONV_BWD_DATA, P, Q));
}

struct BwdSharedPlan { int slab; bool wstrip; size_t pack, strips, ximg, partial, total; };

BwdSharedPlan bwd_shared_plan(const vdnn_conv_desc* d, int P, int Q) {
    BwdSharedPlan plan;
    plan.wstrip = bwd_wstrip_shape(d, P, Q);
    tma::Problem q = tma_problem(d, VDNN_CONV_BWD_DATA, P, Q), fq = tma_problem(d, VDNN_CONV_FWD, P, Q);
    q.n = 1; fq.n = 1;
    const size_t x_one = plan.wstrip ? tma::strip_image_bytes(fq) : tma::image_bytes(1, d->c, d->h, d->w);
    plan.slab = tma_slab_images(d->n, tma::strip_image_bytes(q) + x_one);
    q.n = plan.slab; fq.n = plan.slab;
    plan.pack = packed_weight_bytes(d, VDNN_CONV_BWD_DATA);
    plan.strips = tma::strip_image_bytes(q);
    plan.ximg = plan.wstrip ? tma::strip_image_bytes(fq) : tma::image_bytes(plan.slab, d->c, d->h, d->w);
    tma::WgradProblem wq = wgrad_problem(d, P, Q);
    wq.n = plan.slab;
    plan.partial = plan.wstrip ? tma::wstrip_partial_bytes(fq, d->k) : tma::wgrad_partial_bytes(wq);
    plan.total = plan.pack + plan.strips + plan.ximg + plan.partial;
    return plan;
}

// KCRS weights viewed as [c][(tap, ko)]: offset c*RS + tap + ko*C*RS (the B operand of the data gradient).
SplitDense dgrad_weight_view(const vdnn_conv_desc* d, const float* w) {
    const int rs = d->r * d->s;
    SplitDense B;
    B.p = w; B.rows = d->c; B.cols = d->k * rs;
    B.row_div = FastDiv(1u << 30); B.row_hi = 0;
    B.col_div = FastDiv(d->k);
    B.row_lo = rs; B.col_hi = 1; B.col_lo = d->c * rs;
    return B;
}

int bwd_shared_tma(const vdnn_conv_desc* d, int P, int Q, float alpha_dx, const float* w, const float* x, const float* dy, float beta_dx,
                   float* dx, float alpha_w, float beta_w, float* dw, float alpha_b, float beta_b, float* db, char* ws, size_t ws_bytes,
                   cudaStream_t s) {
    const BwdSharedPlan plan = bwd_shared_plan(d, P, Q);
    if (ws_bytes < plan.total) return VDNN_ERR_WORKSPACE;
    char* tiles = ws;
    char* strips = tiles + plan.pack;
    char* ximg = strips + plan.strips;
    const tma::Problem q = tma_problem(d, VDNN_CONV_BWD_DATA, P, Q);
    const tma::StripGeom g = tma::strip_geometry(q);
    // the weights as they are now: the filter gradient below may update them in place (dw == w)
    int st = tc::pack_b<SplitDense, false>(dgrad_weight_view(d, w), d->c, d->k * d->r * d->s, s, tiles, tma::strip_tile_n(d->c));
    if (st != VDNN_OK) return st;
    if (beta_b == 0.0f) VDNN_CUDA(cudaMemsetAsync(db, 0, sizeof(float) * d->k, s));
    const size_t dy_img = static_cast<size_t>(d->k) * P * Q, x_img = static_cast<size_t>(d->c) * d->h * d->w;
    const size_t dx_elems = static_cast<size_t>(d->n) * x_img, dw_elems = static_cast<size_t>(d->k) * d->c * d->r * d->s;
    const int groups = q.R * (q.cin / 32);
    tma::WgradProblem wq = wgrad_problem(d, P, Q);
    for (int n0 = 0; n0 < d->n; n0 += plan.slab) {
        tma::Problem part = q;
        part.n = min(plan.slab, d->n - n0);
        if ((st = tma::strip_prepare(part, dy + n0 * dy_img, strips, s, db, alpha_b)) != VDNN_OK) return st;
        if ((st = tma::strip_launch(part, nullptr, strips, tiles, dx + n0 * x_img, nullptr, alpha_dx, beta_dx, EPI_DIRECT, dx_elems, 1, groups, s,
                                    false)) != VDNN_OK)
            return st;
        wq.n = part.n;
        const float* hi = reinterpret_cast<const float*>(strips);
        const tma::SharedDy shared{hi, hi + static_cast<size_t>(part.n) * g.lp * q.cin, g.wp, g.lp};
        int splits = 1;
        float* partial = nullptr;
        const float b = n0 == 0 ? beta_w : 1.0f;
        if (plan.wstrip) {
            // x as a position list of the same pitch; the filter gradient runs on the two lists
            tma::Problem fpart = tma_problem(d, VDNN_CONV_FWD, P, Q);
            fpart.n = part.n;
            if ((st = tma::strip_prepare(fpart, x + n0 * x_img, ximg, s)) != VDNN_OK) return st;
            partial = reinterpret_cast<float*>(ximg + tma::strip_image_bytes(fpart));
            if ((st = tma::wstrip_launch(fpart, d->k, ximg, strips, partial, dw, alpha_w, b, s, &splits)) != VDNN_OK) return st;
        } else if ((st = tma::wgrad_launch(wq, x + n0 * x_img, nullptr, ximg, dw, alpha_w, b, s, &splits, &partial, nullptr, 0.0f, &shared)) != VDNN_OK) {
            return st;
        }
        if (splits > 1) {
            reduce_partials_kernel<<<stream_blocks(dw_elems), 256, 0, s>>>(dw_elems, splits, alpha_w, b, partial, dw);
            VDNN_LAUNCHED();
        }
    }
    return VDNN_OK;
}

bool valid_desc(const vdnn_conv_desc* d, int* P, int* Q) {
    if (!d || d->n <= 0 || d->c <= 0 || d->h <= 0 || d->w <= 0 || d->k <= 0 || d->r <= 0 || d->s <= 0 ||
        d->pad_h < 0 || d->pad_w < 0 || d->stride_h <= 0 || d->stride_w <= 0)
        return false;
    if (d->h + 2 * d->pad_h < d->r || d->w + 2 * d->pad_w < d->s) return false;
    *P = (d->h + 2 * d->pad_h - d->r) / d->stride_h + 1;
    *Q = (d->w + 2 * d->pad_w - d->s) / d->stride_w + 1;
    return true;
}

// Offsets are 32-bit inside the kernels: every tensor must stay below 2^31 elements.
bool fits_int32(const vdnn_conv_desc* d, int P, int Q) {
    const long long lim = 0x7fffffffLL;
    return 1LL * d->n * d->c * d->h * d->w < lim && 1LL * d->n * d->k * P * Q < lim &&
           1LL * d->k * d->c * d->r * d->s < lim;
}

XGather make_xgather(const vdnn_conv_desc* d, const float* x, int P, int Q) {
    XGather g;
    g.x = x; g.C = d->c; g.H = d->h; g.W = d->w; g.R = d->r; g.S = d->s;
    g.pad_h = d->pad_h; g.pad_w = d->pad_w; g.stride_h = d->stride_h; g.stride_w = d->stride_w;
    g.n_pix = d->n * P * Q; g.n_filt = d->c * d->r * d->s;
    g.Q = Q;
    g.div_pq = FastDiv(P * Q); g.div_q = FastDiv(Q); g.div_rs = FastDiv(d->r * d->s); g.div_s = FastDiv(d->s);
    g.div_c = FastDiv(d->c);
    g.chw = d->c * d->h * d->w; g.hw = d->h * d->w;
    return g;
}

}  // namespace
}  // namespace vdnn

using namespace vdnn;

extern "C" {

int vdnn_set_engine(int engine) {
    if (engine < VDNN_ENGINE_AUTO || engine > VDNN_ENGINE_TCGEN05) return VDNN_ERR_BAD_ARG;
    const int prev = g_engine;
    g_engine = engine;
    return prev;
}

int vdnn_get_engine(void) { return g_engine; }

int vdnn_engine_status(int* code) {
    if (!code) return VDNN_ERR_BAD_ARG;
    return tc::take_error(code);
}

int vdnn_engine_status_publish(int* dst, void* stream) {
    if (!dst) return VDNN_ERR_BAD_ARG;
    tc::publish_error_kernel<<<1, 1, 0, as_stream(stream)>>>(dst);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_engine_wait_selftest(unsigned long long limit_cycles, void* stream) {
    if (limit_cycles == 0 || limit_cycles > 2000000000ull) return VDNN_ERR_BAD_ARG;      // at most about a second
    tc::wait_probe_kernel<<<1, 32, 0, as_stream(stream)>>>(limit_cycles);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_engine_mma_rate_probe(int iterations, double* flops, void* stream) {
    if (iterations <= 0 || iterations > (1 << 24) || !flops) return VDNN_ERR_BAD_ARG;
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    constexpr int smem = 200 * 1024;            // more than half an SM's shared memory: one CTA per SM
    if (VDNN_ONCE_PER_DEVICE(dev))
        VDNN_CUDA(cudaFuncSetAttribute(tc::mma_rate_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int ctas = sm_count();
    tc::mma_rate_probe_kernel<<<ctas, 128, smem, as_stream(stream)>>>(iterations);
    VDNN_LAUNCHED();
    *flops = 2.0 * 128 * 256 * 8 * 12 * static_cast<double>(iterations) * ctas;
    return VDNN_OK;
}

int vdnn_conv_out_dims(const vdnn_conv_desc* d, int* p, int* q) {
    int P, Q;
    if (!p || !q || !valid_desc(d, &P, &Q)) return VDNN_ERR_BAD_ARG;
    *p = P; *q = Q;
    return VDNN_OK;
}

size_t vdnn_conv_workspace_bytes(int op, int algo_mode, const vdnn_conv_desc* d) {
    int P, Q;
    if (!valid_desc(d, &P, &Q) || algo_mode != VDNN_ALGO_PERF_OPT) return 0;
    int M, N, K;
    size_t out;
    const int crs = d->c * d->r * d->s;
    if (op == VDNN_CONV_BWD_ALL) {
        if (bwd_shared_shape(d, P, Q)) return bwd_shared_plan(d, P, Q).total;
        const size_t a = vdnn_conv_workspace_bytes(VDNN_CONV_BWD_DATA, algo_mode, d), b = vdnn_conv_workspace_bytes(VDNN_CONV_BWD_FILTER, algo_mode, d);
        return a > b ? a : b;
    }
    if (op == VDNN_CONV_BWD_FILTER && tma_wgrad_shape(d)) {
        tma::WgradProblem q = wgrad_problem(d, P, Q);
        q.n = 1;
        q.n = tma_slab_images(d->n, tma::wgrad_image_bytes(q));
        size_t own = tma::wgrad_image_bytes(q) + tma::wgrad_partial_bytes(q);
        // a caller that sizes the filter gradient's workspace by this figure can also run all three gradients in it
        // (vdnn_conv_bwd_data_filter_bias)
        if (bwd_shared_shape(d, P, Q)) { const size_t all = bwd_shared_plan(d, P, Q).total; if (all > own) own = all; }
        return own;
    }
    if (is_full_extent(d)) {        // runs as the corresponding FC product
        switch (op) {
        case VDNN_CONV_FWD: return vdnn_sgemm_workspace_bytes(algo_mode, d->k, d->n, crs);
        case VDNN_CONV_BWD_DATA: return vdnn_sgemm_workspace_bytes(algo_mode, crs, d->n, d->k);
        case VDNN_CONV_BWD_FILTER: return vdnn_sgemm_workspace_bytes(algo_mode, crs, d->k, d->n);
        default: return 0;
        }
    }
    switch (op) {
    case VDNN_CONV_FWD: M = d->n * P * Q; N = d->k; K = crs; out = static_cast<size_t>(M) * N; break;
    case VDNN_CONV_BWD_DATA: M = d->n * d->h * d->w; N = d->c; K = d->k * d->r * d->s; out = static_cast<size_t>(M) * N; break;
    case VDNN_CONV_BWD_FILTER: M = crs; N = d->k; K = d->n * P * Q; out = static_cast<size_t>(M) * N; break;
    default: return 0;
    }
    if (op == VDNN_CONV_BWD_FILTER && wgrad_small_c_shape(d, Q)) return wgrad_small_c_bytes(d);
    const SplitPlan plan = plan_split(M, N, K);
    size_t bytes = plan.splits > 1 ? static_cast<size_t>(plan.splits) * out * sizeof(float) : 0;
    if (op == VDNN_CONV_FWD || op == VDNN_CONV_BWD_DATA) bytes += packed_weight_bytes(d, op);
    else bytes += packed_dy_bytes(d, P, Q);
    if (tma_shape(d, op)) bytes += tma_image_bytes(d, op, P, Q);
    return bytes;
}

int vdnn_conv_fwd(const vdnn_conv_desc* d, int algo_mode, float alpha, const float* x, const float* w,
                  const float* bias, float beta, float* y, void* workspace, size_t workspace_bytes, void* stream) {
    int P, Q;
    if (!x || !w || !y || !valid_desc(d, &P, &Q)) return VDNN_ERR_BAD_ARG;
    if (!fits_int32(d, P, Q)) return VDNN_ERR_UNSUPPORTED;
    const int crs = d->c * d->r * d->s, pq = P * Q, rs = d->r * d->s;
    if (is_full_extent(d)) {    // Y[n][k] = sum_j W[k][j] X[n][j]   (the FC forward product, layer.cu:677-685), then the bias
        const int st = vdnn_sgemm(1, 0, d->k, d->n, crs, alpha, w, crs, x, crs, beta, y, d->k, algo_mode, workspace, workspace_bytes, stream);
        if (st != VDNN_OK || !bias) return st;
        return vdnn_add_bias(d->n, d->k, 1, 1.0f, bias, y, stream);
    }
    // few input channels, 3 x 3, stride 1 (the first layer of VGG16): 27 terms per output, an FFMA kernel of its own
    if (g_engine != VDNN_ENGINE_FFMA && wgrad_small_c_shape(d, Q) && (reinterpret_cast<uintptr_t>(y) & 15u) == 0)
        return fwd_small_c(d, P, Q, alpha, x, w, bias, beta, y, as_stream(stream));
    Epilogue e{};
    e.out = y; e.bias = bias; e.alpha = alpha; e.beta = beta;
    e.row_div = FastDiv(pq); e.row_hi = d->k * pq; e.row_lo = 1; e.col_stride = pq;
    const int M = d->n * pq;
    cudaStream_t s = as_stream(stream);
    if (algo_mode == VDNN_ALGO_PERF_OPT) {
        // workspace variant: reduce tap-major (k = tap*C + c: one bounds test per run of channels); the weights, read
        // through the matching view ko*CRS + c*RS + tap, are packed once into tile images that the kernel bulk-copies
        const size_t pack = packed_weight_bytes(d, VDNN_CONV_FWD);
        if (!workspace || workspace_bytes < pack) return VDNN_ERR_WORKSPACE;
        XGatherPixRowsTap A; A.g = make_xgather(d, x, P, Q);
        SplitDense B = make_dense(w, d->k, crs, crs, 1);
        B.col_div = FastDiv(d->c); B.col_hi = 1; B.col_lo = rs;
        char* tiles = (g_engine != VDNN_ENGINE_FFMA && (reinterpret_cast<uintptr_t>(workspace) & 127u) == 0) ? static_cast<char*>(workspace) : nullptr;
        if (tiles && tma_shape(d, VDNN_CONV_FWD) && !g_no_tma) {
            const tma::Problem q = tma_problem(d, VDNN_CONV_FWD, P, Q);
            int st = tc::pack_b<SplitDense, true>(B, d->k, crs, s, tiles, tma_use_strips(q) ? tma::strip_tile_n(d->k) : 0);
            if (st != VDNN_OK) return st;
            return contract_tma(q, x, tiles, e, static_cast<size_t>(M) * d->k, tiles + pack, workspace_bytes - pack, s);
        }
        return contract<XGatherPixRowsTap, SplitDense, false, true>(A, B, e, M, d->k, crs, static_cast<size_t>(M) * d->k, 0, algo_mode,
                                                                    static_cast<char*>(workspace) + pack, workspace_bytes - pack, s, tiles);
    }
    XGatherPixRows A; A.g = make_xgather(d, x, P, Q);
    SplitDense B = make_dense(w, d->k, crs, crs, 1);
    return contract<XGatherPixRows, SplitDense, false, true>(A, B, e, M, d->k, crs, static_cast<size_t>(M) * d->k, 0,
                                                             algo_mode, workspace, workspace_bytes, s);
}

int vdnn_conv_bwd_data(const vdnn_conv_desc* d, int algo_mode, float alpha, const float* w, const float* dy,
                       float beta, float* dx, void* workspace, size_t workspace_bytes, void* stream) {
    int P, Q;
    if (!w || !dy || !dx || !valid_desc(d, &P, &Q)) return VDNN_ERR_BAD_ARG;
    if (!fits_int32(d, P, Q)) return VDNN_ERR_UNSUPPORTED;
    const int rs = d->r * d->s, hw = d->h * d->w, pq = P * Q;
    if (is_full_extent(d))      // dX[n][j] = sum_k W[k][j] dY[n][k]   (the FC data-gradient product, layer.cu:725-733)
        return vdnn_sgemm(0, 0, d->c * rs, d->n, d->k, alpha, w, d->c * rs, dy, d->k, beta, dx, d->c * rs, algo_mode, workspace,
                          workspace_bytes, stream);
    if (d->c <= SMALL_C_MAX && d->stride_h == d->stride_w && d->r <= 3 * d->stride_h && d->s <= 3 * d->stride_w) {
        const bool narrow = (d->w - 1 + d->pad_w) / d->stride_w + 1 <= 64;      // class coordinates fit a 64-wide tile
        cudaStream_t cs = as_stream(stream);
        int st;
        if (d->c == 3) st = narrow ? launch_dgrad_small_c_phase<64, 3>(d, P, Q, alpha, beta, w, dy, dx, cs)
                                   : launch_dgrad_small_c_phase<128, 3>(d, P, Q, alpha, beta, w, dy, dx, cs);
        else st = narrow ? launch_dgrad_small_c_phase<64, 4>(d, P, Q, alpha, beta, w, dy, dx, cs)
                         : launch_dgrad_small_c_phase<128, 4>(d, P, Q, alpha, beta, w, dy, dx, cs);
        if (st != VDNN_ERR_UNSUPPORTED) return st;
    }
    const size_t small_smem = static_cast<size_t>(d->k) * d->c * rs * sizeof(float);
    if (d->c <= SMALL_C_MAX && small_smem <= SMALL_C_SMEM_MAX) {
        int dev = 0;
        VDNN_CUDA(cudaGetDevice(&dev));
        if (VDNN_ONCE_PER_DEVICE(dev))
            VDNN_CUDA(cudaFuncSetAttribute(dgrad_small_c_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMALL_C_SMEM_MAX)));
        const long long total = static_cast<long long>(d->n) * hw;
        long long blocks = (total + 255) / 256;
        const long long cap = static_cast<long long>(sm_count()) * (small_smem > 100 * 1024 ? 1 : 2) * 2;
        if (blocks > cap) blocks = cap;
        dgrad_small_c_kernel<<<static_cast<int>(blocks), 256, small_smem, as_stream(stream)>>>(
            d->n, d->c, d->h, d->w, d->k, d->r, d->s, P, Q, d->pad_h, d->pad_w, d->stride_h, d->stride_w, alpha, beta, w, dy, dx);
        VDNN_LAUNCHED();
        return VDNN_OK;
    }
    DyGather A;
    A.dy = dy; A.K = d->k; A.P = P; A.Q = Q; A.R = d->r; A.S = d->s;
    A.pad_h = d->pad_h; A.pad_w = d->pad_w; A.stride_h = d->stride_h; A.stride_w = d->stride_w;
    A.n_pix = d->n * hw; A.n_cols = d->k * rs;
    A.div_hw = FastDiv(hw); A.div_w = FastDiv(d->w); A.div_k = FastDiv(d->k); A.div_s = FastDiv(d->s);
    A.div_sh = FastDiv(d->stride_h); A.div_sw = FastDiv(d->stride_w);
    A.kpq = d->k * pq; A.pq = pq;
    Epilogue e{};
    e.out = dx; e.bias = nullptr; e.alpha = alpha; e.beta = beta;
    e.row_div = FastDiv(hw); e.row_hi = d->c * hw; e.row_lo = 1; e.col_stride = hw;
    const int M = d->n * hw;
    cudaStream_t s = as_stream(stream);
    SplitDense B;
    B.p = w; B.rows = d->c; B.cols = d->k * rs;
    B.row_div = FastDiv(1u << 30); B.row_hi = 0;
    B.col_div = FastDiv(d->k);
    B.row_lo = rs; B.col_hi = 1; B.col_lo = d->c * rs;      // KCRS weights viewed as [c][(tap, ko)]: offset c*RS + tap + ko*C*RS
    if (algo_mode == VDNN_ALGO_PERF_OPT) {
        // workspace variant: that view is packed once into tile images that the kernel bulk-copies
        const size_t pack = packed_weight_bytes(d, VDNN_CONV_BWD_DATA);
        if (!workspace || workspace_bytes < pack) return VDNN_ERR_WORKSPACE;
        char* tiles = (g_engine != VDNN_ENGINE_FFMA && (reinterpret_cast<uintptr_t>(workspace) & 127u) == 0) ? static_cast<char*>(workspace) : nullptr;
        if (tiles && tma_shape(d, VDNN_CONV_BWD_DATA) && !g_no_tma) {
            const tma::Problem q = tma_problem(d, VDNN_CONV_BWD_DATA, P, Q);
            int st = tc::pack_b<SplitDense, false>(B, d->c, d->k * rs, s, tiles, tma_use_strips(q) ? tma::strip_tile_n(d->c) : 0);
            if (st != VDNN_OK) return st;
            return contract_tma(q, dy, tiles, e, static_cast<size_t>(M) * d->c, tiles + pack, workspace_bytes - pack, s);
        }
        return contract<DyGather, SplitDense, false, false>(A, B, e, M, d->c, d->k * rs, static_cast<size_t>(M) * d->c, 0, algo_mode,
                                                            static_cast<char*>(workspace) + pack, workspace_bytes - pack, s, tiles);
    }
    // zero-workspace variant: B is walked along its rows (channels, 36-byte stride) by neighbouring threads: along k it
    // would be a whole filter apart.
    return contract<DyGather, SplitDense, false, false>(A, B, e, M, d->c, d->k * rs, static_cast<size_t>(M) * d->c, 0,
                                                        algo_mode, workspace, workspace_bytes, s);
}

int vdnn_conv_bwd_filter(const vdnn_conv_desc* d, int algo_mode, float alpha, const float* x, const float* dy,
                         float beta, float* dw, void* workspace, size_t workspace_bytes, void* stream) {
    int P, Q;
    if (!x || !dy || !dw || !valid_desc(d, &P, &Q)) return VDNN_ERR_BAD_ARG;
    if (!fits_int32(d, P, Q)) return VDNN_ERR_UNSUPPORTED;
    const int crs = d->c * d->r * d->s, pq = P * Q;
    if (is_full_extent(d))      // W[k][j] = alpha * sum_n X[n][j] dY[n][k] + beta * W[k][j]   (layer.cu:736-744)
        return vdnn_sgemm(0, 1, crs, d->k, d->n, alpha, x, crs, dy, d->k, beta, dw, crs, algo_mode, workspace, workspace_bytes, stream);
    if (algo_mode == VDNN_ALGO_PERF_OPT && g_engine != VDNN_ENGINE_FFMA && wgrad_small_c_shape(d, Q) && workspace &&
        (reinterpret_cast<uintptr_t>(dy) & 15u) == 0 && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0)
        return wgrad_small_c(d, P, Q, x, dy, alpha, beta, dw, 0.0f, 0.0f, nullptr, static_cast<char*>(workspace), workspace_bytes, as_stream(stream));
    // D[j][k] = sum over pixels of x(j; pixel) * dy(k; pixel), written to dw[k*CRS + j]: the expensive operand, the
    // gathered input, supplies the 128 tile rows; dy supplies up to 256 columns, so every gathered element feeds up to
    // 256 multiply-adds and layers with few filters (K = 64) still fill the tile's rows.
    XGatherFiltRows A; A.g = make_xgather(d, x, P, Q);
    // dy viewed as [k][(n, pq)]: offset = k*PQ + n*K*PQ + pq
    SplitDense B;
    B.p = dy; B.rows = d->k; B.cols = d->n * pq;
    B.row_div = FastDiv(1u << 30); B.row_hi = 0; B.row_lo = pq;
    B.col_div = FastDiv(pq); B.col_hi = d->k * pq; B.col_lo = 1;
    Epilogue e{};
    e.out = dw; e.bias = nullptr; e.alpha = alpha; e.beta = beta;
    e.row_div = FastDiv(1u << 30); e.row_hi = 0; e.row_lo = 1; e.col_stride = crs;
    if (algo_mode == VDNN_ALGO_PERF_OPT && tma_wgrad_shape(d) && g_engine != VDNN_ENGINE_FFMA && workspace &&
        (reinterpret_cast<uintptr_t>(workspace) & 127u) == 0) {
        // both operands as channels-last tf32 hi / lo images, fetched by tensor copies (conv_tma.cuh)
        return wgrad_tma(wgrad_problem(d, P, Q), x, dy, static_cast<char*>(workspace), workspace_bytes, dw, alpha, beta, as_stream(stream));
    }
    if (algo_mode == VDNN_ALGO_PERF_OPT) {
        // workspace variant: dy, which every row tile of the gathered input needs again, is split into tf32 halves and
        // laid out as tile images once; the kernel's producers then gather x only
        const size_t pack = packed_dy_bytes(d, P, Q);
        if (pack && (!workspace || workspace_bytes < pack)) return VDNN_ERR_WORKSPACE;
        char* tiles = (pack && g_engine != VDNN_ENGINE_FFMA && (reinterpret_cast<uintptr_t>(workspace) & 127u) == 0)
                          ? static_cast<char*>(workspace) : nullptr;
        return contract<XGatherFiltRows, SplitDense, true, true>(A, B, e, crs, d->k, d->n * pq, static_cast<size_t>(d->k) * crs, 0,
                                                                 algo_mode, static_cast<char*>(workspace) + pack,
                                                                 workspace_bytes - pack, as_stream(stream), tiles);
    }
    return contract<XGatherFiltRows, SplitDense, true, true>(A, B, e, crs, d->k, d->n * pq, static_cast<size_t>(d->k) * crs, 0,
                                                             algo_mode, workspace, workspace_bytes, as_stream(stream));
}

// Bias gradient and filter gradient of one convolution in one call (layer.cu:631-660: cudnnConvolutionBackwardBias, then
// cudnnConvolutionBackwardFilter).  Where the filter gradient runs on the TMA-fed engine, the pass that rewrites dy into
// operand images also forms the per-channel sums of dy, so dy is read once less and one kernel launch is saved; anywhere
// else this is vdnn_conv_bwd_bias followed by vdnn_conv_bwd_filter.  beta_b must be 0 or 1 for the combined form.
int vdnn_conv_bwd_filter_bias(const vdnn_conv_desc* d, int algo_mode, float alpha, const float* x, const float* dy, float beta,
                              float* dw, float alpha_b, float beta_b, float* db, void* workspace, size_t workspace_bytes,
                              void* stream) {
    int P, Q;
    if (!x || !dy || !dw || !db || !valid_desc(d, &P, &Q)) return VDNN_ERR_BAD_ARG;
    const bool combined = algo_mode == VDNN_ALGO_PERF_OPT && !is_full_extent(d) && tma_wgrad_shape(d) && g_engine != VDNN_ENGINE_FFMA && workspace &&
                          (reinterpret_cast<uintptr_t>(workspace) & 127u) == 0 && (beta_b == 0.0f || beta_b == 1.0f) &&
                          fits_int32(d, P, Q);
    if (!combined && algo_mode == VDNN_ALGO_PERF_OPT && g_engine != VDNN_ENGINE_FFMA && wgrad_small_c_shape(d, Q) && workspace && fits_int32(d, P, Q) &&
        (reinterpret_cast<uintptr_t>(dy) & 15u) == 0 && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0)
        return wgrad_small_c(d, P, Q, x, dy, alpha, beta, dw, alpha_b, beta_b, db, static_cast<char*>(workspace), workspace_bytes, as_stream(stream));
    if (!combined) {
        const int st = vdnn_conv_bwd_bias(d->n, d->k, P * Q, alpha_b, dy, beta_b, db, stream);
        return st != VDNN_OK ? st : vdnn_conv_bwd_filter(d, algo_mode, alpha, x, dy, beta, dw, workspace, workspace_bytes, stream);
    }
    if (beta_b == 0.0f) VDNN_CUDA(cudaMemsetAsync(db, 0, sizeof(float) * d->k, as_stream(stream)));
    return wgrad_tma(wgrad_problem(d, P, Q), x, dy, static_cast<char*>(workspace), workspace_bytes, dw, alpha, beta, as_stream(stream),
                     db, alpha_b);
}


// cudnnConvolutionBackwardData, BackwardBias and BackwardFilter of one layer (layer.cu:616-660) in one call and one
// workspace (vdnn_conv_workspace_bytes(VDNN_CONV_BWD_ALL, ...), which the figure for VDNN_CONV_BWD_FILTER covers where the
// gradients share an image pass).  The data
// gradient uses the weights as they are on entry, also when dw == w.  Where both gradients run on the TMA-fed engine, dy
// is rewritten into operand images once for both; otherwise the three separate entry points run in the reference's order.
int vdnn_conv_bwd_data_filter_bias(const vdnn_conv_desc* d, int algo_mode, float alpha_dx, const float* w, const float* x, const float* dy,
                                   float beta_dx, float* dx, float alpha_w, float beta_w, float* dw, float alpha_b, float beta_b, float* db,
                                   void* workspace, size_t workspace_bytes, void* stream) {
    int P, Q;
    if (!w || !x || !dy || !dx || !dw || !db || !valid_desc(d, &P, &Q)) return VDNN_ERR_BAD_ARG;
    const bool shared = algo_mode == VDNN_ALGO_PERF_OPT && g_engine != VDNN_ENGINE_FFMA && workspace &&
                        (reinterpret_cast<uintptr_t>(workspace) & 127u) == 0 && (beta_b == 0.0f || beta_b == 1.0f) &&
                        !is_full_extent(d) && fits_int32(d, P, Q) && bwd_shared_shape(d, P, Q);
    if (shared)
        return bwd_shared_tma(d, P, Q, alpha_dx, w, x, dy, beta_dx, dx, alpha_w, beta_w, dw, alpha_b, beta_b, db, static_cast<char*>(workspace),
                              workspace_bytes, as_stream(stream));
    const int st = vdnn_conv_bwd_data(d, algo_mode, alpha_dx, w, dy, beta_dx, dx, workspace, workspace_bytes, stream);
    return st != VDNN_OK ? st
                         : vdnn_conv_bwd_filter_bias(d, algo_mode, alpha_w, x, dy, beta_w, dw, alpha_b, beta_b, db, workspace, workspace_bytes, stream);
}

// 1 where vdnn_conv_bwd_data_filter_bias shares one pass over dy between the gradients (a host that keeps the three calls
// apart loses nothing elsewhere).
int vdnn_conv_bwd_shares_dy(const vdnn_conv_desc* d, int algo_mode) {
    int P, Q;
    return (algo_mode == VDNN_ALGO_PERF_OPT && g_engine != VDNN_ENGINE_FFMA && valid_desc(d, &P, &Q) && !is_full_extent(d) &&
            fits_int32(d, P, Q) && bwd_shared_shape(d, P, Q)) ? 1 : 0;
}

}  // extern "C"

namespace {

// Scratch for vdnn_conv_bwd_filter_static.  In host code this name is only a handle for the
// symbol, not a device address: the address comes from cudaGetSymbolAddress, per device.
static __device__ __align__(256) float g_static_scratch[VDNN_STATIC_SCRATCH_BYTES / sizeof(float)];
constexpr int STATIC_SCRATCH_MAX_DEVICES = 64;
float* g_static_scratch_addr[STATIC_SCRATCH_MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device; resolved on first use per device.  The table is not
// guarded: two host threads making their first call on one device at the same time both look the address up and
// store the same value.  Device ordinals beyond the table are refused, never silently skipped.
int static_scratch_address(float** out) {
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= STATIC_SCRATCH_MAX_DEVICES) return VDNN_ERR_UNSUPPORTED;
    if (!g_static_scratch_addr[dev]) {
        void* p = nullptr;
        VDNN_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        g_static_scratch_addr[dev] = static_cast<float*>(p);
    }
    *out = g_static_scratch_addr[dev];
    return VDNN_OK;
}

}  // namespace

extern "C" {

int vdnn_conv_bwd_filter_static(const vdnn_conv_desc* d, float alpha, const float* x, const float* dy, float beta,
                                float* dw, void* stream) {
    int P, Q;
    if (!x || !dy || !dw || !valid_desc(d, &P, &Q)) return VDNN_ERR_BAD_ARG;
    const size_t need = vdnn_conv_workspace_bytes(VDNN_CONV_BWD_FILTER, VDNN_ALGO_PERF_OPT, d);
    if (need > VDNN_STATIC_SCRATCH_BYTES) return VDNN_ERR_SCRATCH_LIMIT;
    float* scratch = nullptr;
    const int st = static_scratch_address(&scratch);
    if (st != VDNN_OK) return st;
    // The partial sums of every split are written in full before the reduction reads them, so the
    // array's previous contents never matter.
    return vdnn_conv_bwd_filter(d, VDNN_ALGO_PERF_OPT, alpha, x, dy, beta, dw, scratch, VDNN_STATIC_SCRATCH_BYTES, stream);
}

size_t vdnn_sgemm_workspace_bytes(int algo_mode, int m, int n, int k) {
    if (algo_mode != VDNN_ALGO_PERF_OPT || m <= 0 || n <= 0 || k <= 0) return 0;
    const SplitPlan plan = plan_split(m, n, k);
    return plan.splits > 1 ? static_cast<size_t>(plan.splits) * m * n * sizeof(float) : 0;
}

int vdnn_sgemm(int transa, int transb, int m, int n, int k, float alpha, const float* A, int lda, const float* B,
               int ldb, float beta, float* C, int ldc, int algo_mode, void* workspace, size_t workspace_bytes,
               void* stream) {
    if (!A || !B || !C || m <= 0 || n <= 0 || k <= 0 || ldc < m) return VDNN_ERR_BAD_ARG;
    if (lda < (transa ? k : m) || ldb < (transb ? n : k)) return VDNN_ERR_BAD_ARG;
    const long long lim = 0x7fffffffLL;
    if (1LL * lda * (transa ? m : k) >= lim || 1LL * ldb * (transb ? k : n) >= lim || 1LL * ldc * n >= lim)
        return VDNN_ERR_UNSUPPORTED;
    // A'(i, kk) = op(A)[i][kk], B'(j, kk) = op(B)[kk][j]
    SplitDense a = transa ? make_dense(A, m, k, lda, 1) : make_dense(A, m, k, 1, lda);
    SplitDense b = transb ? make_dense(B, n, k, 1, ldb) : make_dense(B, n, k, ldb, 1);
    Epilogue e{};
    e.out = C; e.bias = nullptr; e.alpha = alpha; e.beta = beta;
    e.row_div = FastDiv(1u << 30); e.row_hi = 0; e.row_lo = 1; e.col_stride = ldc;
    const size_t dense = (ldc == m) ? static_cast<size_t>(m) * n : 0;
    cudaStream_t s = as_stream(stream);
    if (transa && !transb) return contract<SplitDense, SplitDense, true, true>(a, b, e, m, n, k, dense, ldc, algo_mode, workspace, workspace_bytes, s);
    if (!transa && !transb) return contract<SplitDense, SplitDense, false, true>(a, b, e, m, n, k, dense, ldc, algo_mode, workspace, workspace_bytes, s);
    if (!transa && transb) return contract<SplitDense, SplitDense, false, false>(a, b, e, m, n, k, dense, ldc, algo_mode, workspace, workspace_bytes, s);
    return contract<SplitDense, SplitDense, true, false>(a, b, e, m, n, k, dense, ldc, algo_mode, workspace, workspace_bytes, s);
}

}  // extern "C"
