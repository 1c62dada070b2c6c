// Bandwidth-bound layers of the vDNN training path for sm_100a: ReLU, max-pool, softmax,
// tensor difference, bias add / bias gradient, LRN, loss, axpy, fill.
// All kernels stream fp32 NCHW tensors with 16-byte accesses where alignment allows and size
// their grids in whole multiples of the SM count.
#include <math.h>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace vdnn {

thread_local int g_last_cuda_error = 0;
unsigned long long g_kernel_launches = 0;

int sm_count() {
    static std::vector<int> cached;                      // indexed by device ordinal, grown on demand
    static std::mutex lock;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 148;
    std::lock_guard<std::mutex> g(lock);
    if (cached.size() <= static_cast<size_t>(dev)) cached.resize(dev + 1, 0);
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

bool first_use_on_device(void** seen_table, int device) {
    static std::mutex lock;
    std::lock_guard<std::mutex> g(lock);
    if (device < 0) return false;
    std::vector<char>* seen = static_cast<std::vector<char>*>(*seen_table);
    if (!seen) { seen = new std::vector<char>(); *seen_table = seen; }     // lives as long as the process
    if (seen->size() <= static_cast<size_t>(device)) seen->resize(device + 1, 0);
    if ((*seen)[device]) return false;
    (*seen)[device] = 1;
    return true;
}

namespace {

constexpr int kThreads = 256;

// Blocks for a streaming kernel in which every thread handles `per_thread` items per loop trip.
inline int stream_grid(size_t items, int per_thread) {
    const size_t want = ceil_div(items, static_cast<size_t>(kThreads) * per_thread);
    const size_t cap = static_cast<size_t>(sm_count()) * 8;     // 8 x 256 threads = a full SM
    size_t g = want < cap ? want : cap;
    if (g > static_cast<size_t>(sm_count())) g = g / sm_count() * sm_count();
    return g ? static_cast<int>(g) : 1;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ float relu1(float v) { return v > 0.0f ? v : (v != v ? v : 0.0f); }

// ---------------------------------------------------------------- ReLU
__global__ void __launch_bounds__(kThreads) relu_fwd_kernel(size_t n4, size_t n, const float* __restrict__ x,
                                                            float* __restrict__ y) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* y4 = reinterpret_cast<float4*>(y);
    for (; i + 3 * stride < n4; i += 4 * stride) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldcs(x4 + i + u * stride);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            v[u].x = relu1(v[u].x); v[u].y = relu1(v[u].y); v[u].z = relu1(v[u].z); v[u].w = relu1(v[u].w);
            y4[i + u * stride] = v[u];
        }
    }
    for (; i < n4; i += stride) {
        float4 v = __ldcs(x4 + i);
        v.x = relu1(v.x); v.y = relu1(v.y); v.z = relu1(v.z); v.w = relu1(v.w);
        y4[i] = v;
    }
    // scalar tail (and the whole tensor when the pointers are not 16-byte aligned: n4 == 0)
    for (size_t j = n4 * 4 + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride)
        y[j] = relu1(x[j]);
}

__global__ void __launch_bounds__(kThreads) relu_bwd_kernel(size_t n4, size_t n, const float* __restrict__ dy,
                                                            const float* __restrict__ x, float* __restrict__ dx) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const float4* d4 = reinterpret_cast<const float4*>(dy);
    float4* o4 = reinterpret_cast<float4*>(dx);
    for (; i + stride < n4; i += 2 * stride) {
        float4 a[2], g[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) { a[u] = __ldcs(x4 + i + u * stride); g[u] = __ldcs(d4 + i + u * stride); }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            float4 r;
            r.x = a[u].x > 0.0f ? g[u].x : 0.0f; r.y = a[u].y > 0.0f ? g[u].y : 0.0f;
            r.z = a[u].z > 0.0f ? g[u].z : 0.0f; r.w = a[u].w > 0.0f ? g[u].w : 0.0f;
            o4[i + u * stride] = r;
        }
    }
    for (; i < n4; i += stride) {
        float4 a = __ldcs(x4 + i), g = __ldcs(d4 + i), r;
        r.x = a.x > 0.0f ? g.x : 0.0f; r.y = a.y > 0.0f ? g.y : 0.0f;
        r.z = a.z > 0.0f ? g.z : 0.0f; r.w = a.w > 0.0f ? g.w : 0.0f;
        o4[i] = r;
    }
    for (size_t j = n4 * 4 + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride)
        dx[j] = x[j] > 0.0f ? dy[j] : 0.0f;
}

// ---------------------------------------------------------------- tanh / sigmoid (mode as in vdnn_b200.h)
template <int MODE> __device__ __forceinline__ float act1(float x) {
    return MODE == VDNN_ACT_TANH ? tanhf(x) : 1.0f / (1.0f + expf(-x));
}
template <int MODE> __device__ __forceinline__ float dact1(float y, float dy) {
    return MODE == VDNN_ACT_TANH ? dy * (1.0f - y * y) : dy * y * (1.0f - y);
}

template <int MODE>
__global__ void __launch_bounds__(kThreads) act_fwd_kernel(size_t n4, size_t n, const float* __restrict__ x,
                                                           float* __restrict__ y) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t first = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* y4 = reinterpret_cast<float4*>(y);
    for (size_t i = first; i < n4; i += stride) {
        float4 v = __ldcs(x4 + i);
        v.x = act1<MODE>(v.x); v.y = act1<MODE>(v.y); v.z = act1<MODE>(v.z); v.w = act1<MODE>(v.w);
        y4[i] = v;
    }
    for (size_t j = n4 * 4 + first; j < n; j += stride) y[j] = act1<MODE>(x[j]);
}

template <int MODE>
__global__ void __launch_bounds__(kThreads) act_bwd_kernel(size_t n4, size_t n, const float* __restrict__ y,
                                                           const float* __restrict__ dy, float* __restrict__ dx) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t first = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const float4* y4 = reinterpret_cast<const float4*>(y);
    const float4* d4 = reinterpret_cast<const float4*>(dy);
    float4* o4 = reinterpret_cast<float4*>(dx);
    for (size_t i = first; i < n4; i += stride) {
        const float4 a = __ldcs(y4 + i), d = __ldcs(d4 + i);
        float4 o;
        o.x = dact1<MODE>(a.x, d.x); o.y = dact1<MODE>(a.y, d.y); o.z = dact1<MODE>(a.z, d.z); o.w = dact1<MODE>(a.w, d.w);
        o4[i] = o;
    }
    for (size_t j = n4 * 4 + first; j < n; j += stride) dx[j] = dact1<MODE>(y[j], dy[j]);
}

// ---------------------------------------------------------------- out = a - b, w += alpha g, fill
__global__ void __launch_bounds__(kThreads) sub_kernel(size_t n, const float* __restrict__ a,
                                                       const float* __restrict__ b, float* __restrict__ out) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = a[i] - b[i];
}

__global__ void __launch_bounds__(kThreads) axpy_kernel(size_t n4, size_t n, float alpha, const float* __restrict__ g,
                                                        float* __restrict__ w) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const float4* g4 = reinterpret_cast<const float4*>(g);
    float4* w4 = reinterpret_cast<float4*>(w);
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 a = g4[i], b = w4[i];
        b.x = fmaf(alpha, a.x, b.x); b.y = fmaf(alpha, a.y, b.y); b.z = fmaf(alpha, a.z, b.z); b.w = fmaf(alpha, a.w, b.w);
        w4[i] = b;
    }
    for (size_t j = n4 * 4 + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride)
        w[j] = fmaf(alpha, g[j], w[j]);
}

__global__ void __launch_bounds__(kThreads) fill_kernel(size_t n, float v, float* __restrict__ dst) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = v;
}

// ---------------------------------------------------------------- bias add, bias gradient
// y[(n*K + k)*pq + i] += alpha * bias[k]; one plane (n,k) per blockIdx.y slice.
__global__ void __launch_bounds__(kThreads) add_bias_kernel(int planes, int k, int pq, float alpha,
                                                            const float* __restrict__ bias, float* __restrict__ y) {
    for (int plane = blockIdx.y; plane < planes; plane += gridDim.y) {
        const float b = alpha * bias[plane % k];
        float* yp = y + static_cast<size_t>(plane) * pq;
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pq; i += gridDim.x * blockDim.x) yp[i] += b;
    }
}

__global__ void __launch_bounds__(kThreads) scale_vec_kernel(int n, float beta, float* __restrict__ v) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] = beta == 0.0f ? 0.0f : beta * v[i];
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// db[k] += alpha * sum over this block's slice of (n, pq) for channel k = blockIdx.x.
// gridDim.y slices share a channel and combine with one atomic each; db was pre-scaled by beta.
__global__ void __launch_bounds__(kThreads) bwd_bias_kernel(int n, int k, int pq, float alpha,
                                                            const float* __restrict__ dy, float* __restrict__ db) {
    const int ch = blockIdx.x;
    float acc = 0.0f;
    const bool vec = (pq % 4 == 0) && ((reinterpret_cast<uintptr_t>(dy) & 15u) == 0);
    for (int in = blockIdx.y; in < n; in += gridDim.y) {
        const float* p = dy + (static_cast<size_t>(in) * k + ch) * pq;
        if (vec) {
            const float4* p4 = reinterpret_cast<const float4*>(p);
            const int n4 = pq / 4, step = blockDim.x;
            int i = threadIdx.x;
            // four independent 16-byte loads in flight per thread
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            for (; i + 3 * step < n4; i += 4 * step) {
                const float4 v0 = __ldcs(p4 + i), v1 = __ldcs(p4 + i + step), v2 = __ldcs(p4 + i + 2 * step), v3 = __ldcs(p4 + i + 3 * step);
                a0 += (v0.x + v0.y) + (v0.z + v0.w); a1 += (v1.x + v1.y) + (v1.z + v1.w);
                a2 += (v2.x + v2.y) + (v2.z + v2.w); a3 += (v3.x + v3.y) + (v3.z + v3.w);
            }
            for (; i < n4; i += step) {
                const float4 v = __ldcs(p4 + i);
                a0 += (v.x + v.y) + (v.z + v.w);
            }
            acc += (a0 + a1) + (a2 + a3);
        } else {
            for (int i = threadIdx.x; i < pq; i += blockDim.x) acc += p[i];
        }
    }
    __shared__ float part[kThreads / 32];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < kThreads / 32 ? part[threadIdx.x] : 0.0f;
        v = warp_sum(v);
        if (threadIdx.x == 0) atomicAdd(db + ch, alpha * v);
    }
}

// ---------------------------------------------------------------- max pooling
__global__ void __launch_bounds__(kThreads) maxpool_fwd_generic(int planes, int h, int w, int P, int Q, int wh, int ww,
                                                                int sh, int sw, const float* __restrict__ x,
                                                                float* __restrict__ y) {
    const size_t total = static_cast<size_t>(planes) * P * Q;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int q = static_cast<int>(idx % Q);
        const size_t t = idx / Q;
        const int p = static_cast<int>(t % P);
        const size_t plane = t / P;
        const float* xp = x + plane * h * w + static_cast<size_t>(p * sh) * w + q * sw;
        float m = -INFINITY;
        for (int i = 0; i < wh; ++i)
            for (int j = 0; j < ww; ++j) {
                const float v = xp[i * w + j];
                if (v > m) m = v;
            }
        y[idx] = m;
    }
}

// 2x2 window, stride 2, even H and W, W % 4 == 0: each thread reads two float4 rows and writes
// two outputs (float2).
__global__ void __launch_bounds__(kThreads) maxpool_fwd_2x2(size_t pairs, int w, int Qh /* Q/2 */,
                                                            const float* __restrict__ x, float* __restrict__ y) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < pairs; idx += stride) {
        const size_t row = idx / Qh;                 // (plane * P + p)
        const int qp = static_cast<int>(idx - row * Qh);
        const float* xr = x + row * 2 * w + qp * 4;
        const float4 a = __ldcs(reinterpret_cast<const float4*>(xr));
        const float4 b = __ldcs(reinterpret_cast<const float4*>(xr + w));
        float m0 = -INFINITY, m1 = -INFINITY;
        if (a.x > m0) m0 = a.x; if (a.y > m0) m0 = a.y; if (b.x > m0) m0 = b.x; if (b.y > m0) m0 = b.y;
        if (a.z > m1) m1 = a.z; if (a.w > m1) m1 = a.w; if (b.z > m1) m1 = b.z; if (b.w > m1) m1 = b.w;
        reinterpret_cast<float2*>(y)[idx] = make_float2(m0, m1);
    }
}

// Gather form: one thread per input element; for each window that contains it, recompute the
// window's first maximum and take dy if this element is it.  No atomics, no pre-zeroing.
__global__ void __launch_bounds__(kThreads) maxpool_bwd_generic(int planes, int h, int w, int P, int Q, int wh, int ww,
                                                                int sh, int sw, const float* __restrict__ dy,
                                                                const float* __restrict__ x, float* __restrict__ dx) {
    const size_t total = static_cast<size_t>(planes) * h * w;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int iw = static_cast<int>(idx % w);
        const size_t t = idx / w;
        const int ih = static_cast<int>(t % h);
        const size_t plane = t / h;
        const float* xp = x + plane * h * w;
        const float* dyp = dy + plane * P * Q;
        int p_lo = ih - wh + 1 <= 0 ? 0 : (ih - wh + 1 + sh - 1) / sh;
        int p_hi = ih / sh; if (p_hi > P - 1) p_hi = P - 1;
        int q_lo = iw - ww + 1 <= 0 ? 0 : (iw - ww + 1 + sw - 1) / sw;
        int q_hi = iw / sw; if (q_hi > Q - 1) q_hi = Q - 1;
        float g = 0.0f;
        for (int p = p_lo; p <= p_hi; ++p)
            for (int q = q_lo; q <= q_hi; ++q) {
                float m = -INFINITY;
                int bi = 0, bj = 0;
                for (int i = 0; i < wh; ++i)
                    for (int j = 0; j < ww; ++j) {
                        const float v = xp[static_cast<size_t>(p * sh + i) * w + q * sw + j];
                        if (v > m) { m = v; bi = i; bj = j; }
                    }
                if (p * sh + bi == ih && q * sw + bj == iw) g += dyp[static_cast<size_t>(p) * Q + q];
            }
        dx[idx] = g;
    }
}

// Overlapping windows (AlexNet's 3x3 / stride 2): one thread per window finds its first maximum once and adds dy
// there; dx is zeroed beforehand.  An input element collects at most four contributions, in arbitrary order.
__global__ void __launch_bounds__(kThreads) maxpool_bwd_scatter(int planes, int h, int w, int P, int Q, int wh, int ww,
                                                                int sh, int sw, const float* __restrict__ dy,
                                                                const float* __restrict__ x, float* __restrict__ dx) {
    const size_t total = static_cast<size_t>(planes) * P * Q;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int q = static_cast<int>(idx % Q);
        const size_t t = idx / Q;
        const int p = static_cast<int>(t % P);
        const size_t plane = t / P;
        const size_t origin = plane * h * w + static_cast<size_t>(p * sh) * w + q * sw;
        float m = -INFINITY;
        int best = 0;
        for (int i = 0; i < wh; ++i)
            for (int j = 0; j < ww; ++j) {
                const float v = x[origin + i * w + j];
                if (v > m) { m = v; best = i * w + j; }
            }
        atomicAdd(dx + origin + best, dy[idx]);
    }
}

__global__ void __launch_bounds__(kThreads) maxpool_bwd_2x2(size_t pairs, int w, int Qh, const float* __restrict__ dy,
                                                            const float* __restrict__ x, float* __restrict__ dx) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < pairs; idx += stride) {
        const size_t row = idx / Qh;
        const int qp = static_cast<int>(idx - row * Qh);
        const size_t off = row * 2 * w + qp * 4;
        const float4 a = __ldcs(reinterpret_cast<const float4*>(x + off));
        const float4 b = __ldcs(reinterpret_cast<const float4*>(x + off + w));
        const float2 g = __ldcs(reinterpret_cast<const float2*>(dy) + idx);
        // first maximum in scan order (row 0: x,y ; row 1: x,y) of each 2x2 window
        int s0 = 0; float m0 = -INFINITY;
        if (a.x > m0) { m0 = a.x; s0 = 0; } if (a.y > m0) { m0 = a.y; s0 = 1; }
        if (b.x > m0) { m0 = b.x; s0 = 2; } if (b.y > m0) { m0 = b.y; s0 = 3; }
        int s1 = 0; float m1 = -INFINITY;
        if (a.z > m1) { m1 = a.z; s1 = 0; } if (a.w > m1) { m1 = a.w; s1 = 1; }
        if (b.z > m1) { m1 = b.z; s1 = 2; } if (b.w > m1) { m1 = b.w; s1 = 3; }
        float4 ra, rb;
        ra.x = s0 == 0 ? g.x : 0.0f; ra.y = s0 == 1 ? g.x : 0.0f; rb.x = s0 == 2 ? g.x : 0.0f; rb.y = s0 == 3 ? g.x : 0.0f;
        ra.z = s1 == 0 ? g.y : 0.0f; ra.w = s1 == 1 ? g.y : 0.0f; rb.z = s1 == 2 ? g.y : 0.0f; rb.w = s1 == 3 ? g.y : 0.0f;
        *reinterpret_cast<float4*>(dx + off) = ra;
        *reinterpret_cast<float4*>(dx + off + w) = rb;
    }
}

// ---------------------------------------------------------------- softmax (one warp per row)
__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The row sums are carried in double: with saturated outputs (y close to one-hot) the backward
// expression dy - sum(dy*y) cancels almost completely, and a float sum would leave only a few
// correct bits.  The tensors stay fp32; the extra cost on N x 1000 elements is nil.
__global__ void __launch_bounds__(128) softmax_fwd_kernel(int rows, int cols, const float* __restrict__ x,
                                                          float* __restrict__ y) {
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* xr = x + static_cast<size_t>(row) * cols;
    float* yr = y + static_cast<size_t>(row) * cols;
    float m = -INFINITY;
    for (int j = lane; j < cols; j += 32) m = fmaxf(m, xr[j]);
    m = warp_max(m);
    double s = 0.0;
    for (int j = lane; j < cols; j += 32) s += static_cast<double>(expf(xr[j] - m));
    s = warp_sum_f64(s);
    for (int j = lane; j < cols; j += 32) yr[j] = static_cast<float>(static_cast<double>(expf(xr[j] - m)) / s);
}

__global__ void __launch_bounds__(128) softmax_bwd_kernel(int rows, int cols, const float* __restrict__ y,
                                                          const float* __restrict__ dy, float* __restrict__ dx) {
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* yr = y + static_cast<size_t>(row) * cols;
    const float* dr = dy + static_cast<size_t>(row) * cols;
    float* xr = dx + static_cast<size_t>(row) * cols;
    double dot = 0.0;
    for (int j = lane; j < cols; j += 32) dot += static_cast<double>(yr[j]) * static_cast<double>(dr[j]);
    dot = warp_sum_f64(dot);
    for (int j = lane; j < cols; j += 32)
        xr[j] = static_cast<float>(static_cast<double>(yr[j]) * (static_cast<double>(dr[j]) - dot));
}

// ---------------------------------------------------------------- loss (single block)
__global__ void __launch_bounds__(1024) loss_kernel(int rows, int cols, const float* __restrict__ y,
                                                    const float* __restrict__ label, double* __restrict__ out2) {
    __shared__ double s_sq[32], s_ce[32];
    double sq = 0.0, ce = 0.0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int r = warp; r < rows; r += nwarps) {
        const float* yr = y + static_cast<size_t>(r) * cols;
        const float* tr = label + static_cast<size_t>(r) * cols;
        float best = -INFINITY; int arg = 0x7fffffff;
        for (int j = lane; j < cols; j += 32) {
            const double d = static_cast<double>(yr[j]) - static_cast<double>(tr[j]);
            sq += d * d;
            if (tr[j] > best) { best = tr[j]; arg = j; }
        }
        // first index of the maximum label across the warp
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (lane == 0) {
            const double p = yr[arg];
            ce += -log(p > 1e-30 ? p : 1e-30);
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
        ce += __shfl_xor_sync(0xffffffffu, ce, o);
    }
    if (lane == 0) { s_sq[warp] = sq; s_ce[warp] = ce; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double a = 0.0, b = 0.0;
        for (int i = 0; i < nwarps; ++i) { a += s_sq[i]; b += s_ce[i]; }
        out2[0] = 0.5 * a / rows;
        out2[1] = b / rows;
    }
}

// ---------------------------------------------------------------- cross-channel LRN
// One thread per (n, spatial position); the channel loop keeps a sliding window of squares so
// every x is read once from DRAM (neighbouring threads read neighbouring positions).
__global__ void __launch_bounds__(kThreads) lrn_fwd_kernel(int n, int c, int hw, int win, float alpha_over_n, float beta,
                                                           float k, const float* __restrict__ x, float* __restrict__ y) {
    const size_t total = static_cast<size_t>(n) * hw;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const int half = win / 2;
    for (size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t in = idx / hw;
        const size_t base = in * c * hw + (idx - in * hw);
        float ss = 0.0f;
        for (int j = 0; j < half && j < c; ++j) { const float v = x[base + static_cast<size_t>(j) * hw]; ss = fmaf(v, v, ss); }
        for (int ic = 0; ic < c; ++ic) {
            if (ic + half < c) { const float v = x[base + static_cast<size_t>(ic + half) * hw]; ss = fmaf(v, v, ss); }
            if (ic - half - 1 >= 0) { const float v = x[base + static_cast<size_t>(ic - half - 1) * hw]; ss = fmaf(-v, v, ss); }
            const float scale = fmaf(alpha_over_n, fmaxf(ss, 0.0f), k);
            y[base + static_cast<size_t>(ic) * hw] = x[base + static_cast<size_t>(ic) * hw] * powf(scale, -beta);
        }
    }
}

__global__ void __launch_bounds__(kThreads) lrn_bwd_kernel(int n, int c, int hw, int win, float alpha_over_n, float beta,
                                                           float k, const float* __restrict__ x, const float* __restrict__ y,
                                                           const float* __restrict__ dy, float* __restrict__ dx) {
    const size_t total = static_cast<size_t>(n) * hw;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const int half = win / 2;
    for (size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t in = idx / hw;
        const size_t base = in * c * hw + (idx - in * hw);
        // dx_i = dy_i * s_i^-beta - 2*alpha*beta/n * x_i * sum_{j: |i-j|<=half} dy_j*y_j/s_j
        for (int ic = 0; ic < c; ++ic) {
            const int lo = ic - half < 0 ? 0 : ic - half, hi = ic + half >= c ? c - 1 : ic + half;
            float t = 0.0f, s_i = k;
            for (int j = lo; j <= hi; ++j) {
                const int l2 = j - half < 0 ? 0 : j - half, h2 = j + half >= c ? c - 1 : j + half;
                float ss = 0.0f;
                for (int m = l2; m <= h2; ++m) { const float v = x[base + static_cast<size_t>(m) * hw]; ss = fmaf(v, v, ss); }
                const float sj = fmaf(alpha_over_n, ss, k);
                if (j == ic) s_i = sj;
                t += dy[base + static_cast<size_t>(j) * hw] * y[base + static_cast<size_t>(j) * hw] / sj;
            }
            const size_t o = base + static_cast<size_t>(ic) * hw;
            dx[o] = dy[o] * powf(s_i, -beta) - 2.0f * alpha_over_n * beta * x[o] * t;
        }
    }
}

// Window of 5 (the AlexNet setting): one pass over the channels per position.  Channel j's scale s_j and
// t_j = dy_j * y_j / s_j are produced once and kept in a five-entry shift register; channel i = j - 2 is finished
// as soon as t_{i+2} exists:  dx_i = dy_i * s_i^-beta - 2*alpha*beta/n * x_i * sum_{|j-i|<=2} t_j.
__global__ void __launch_bounds__(kThreads) lrn_bwd_win5_kernel(int n, int c, int hw, float alpha_over_n, float beta, float k,
                                                                const float* __restrict__ x, const float* __restrict__ y,
                                                                const float* __restrict__ dy, float* __restrict__ dx) {
    const size_t total = static_cast<size_t>(n) * hw;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t in = idx / hw;
        const size_t base = in * c * hw + (idx - in * hw);
        float t[5] = {0.f, 0.f, 0.f, 0.f, 0.f};     // t[4] newest (channel j), t[0] = channel j - 4
        float sc[3] = {k, k, k};                     // scales of channels j-2 (sc[0]), j-1, j
        float xq[5] = {0.f, 0.f, 0.f, 0.f, 0.f};     // x of channels j-2 .. j+2, for the sliding sum of squares
        // prime x window for j = 0: channels 0..2 at xq[2..4]
        for (int m = 0; m < 3; ++m) xq[2 + m] = m < c ? x[base + static_cast<size_t>(m) * hw] : 0.0f;
        for (int j = 0; j < c + 2; ++j) {
            if (j < c) {
                const float ss = xq[0] * xq[0] + xq[1] * xq[1] + xq[2] * xq[2] + xq[3] * xq[3] + xq[4] * xq[4];
                const float sj = fmaf(alpha_over_n, ss, k);
                const size_t o = base + static_cast<size_t>(j) * hw;
                t[0] = t[1]; t[1] = t[2]; t[2] = t[3]; t[3] = t[4];
                t[4] = dy[o] * y[o] / sj;
                sc[0] = sc[1]; sc[1] = sc[2]; sc[2] = sj;
            } else {
                t[0] = t[1]; t[1] = t[2]; t[2] = t[3]; t[3] = t[4]; t[4] = 0.0f;
                sc[0] = sc[1]; sc[1] = sc[2];
            }
            const int i = j - 2;
            if (i >= 0) {
                // x_i sits at xq[0] (the window is centred on j = i + 2)
                const size_t o = base + static_cast<size_t>(i) * hw;
                dx[o] = dy[o] * powf(sc[0], -beta) - 2.0f * alpha_over_n * beta * xq[0] * (t[0] + t[1] + t[2] + t[3] + t[4]);
            }
            // slide the x window to be centred on j + 1
            xq[0] = xq[1]; xq[1] = xq[2]; xq[2] = xq[3]; xq[3] = xq[4];
            xq[4] = (j + 3 < c) ? x[base + static_cast<size_t>(j + 3) * hw] : 0.0f;
        }
    }
}

}  // namespace
}  // namespace vdnn

using namespace vdnn;

extern "C" {

int vdnn_relu_fwd(size_t count, const float* x, float* y, void* stream) {
    if (!x || !y) return VDNN_ERR_BAD_ARG;
    if (count == 0) return VDNN_OK;
    const size_t n4 = (aligned16(x) && aligned16(y)) ? count / 4 : 0;
    relu_fwd_kernel<<<stream_grid(n4 ? n4 : count, 4), kThreads, 0, as_stream(stream)>>>(n4, count, x, y);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_relu_bwd(size_t count, const float* y, const float* dy, const float* x, float* dx, void* stream) {
    (void)y;
    if (!dy || !x || !dx) return VDNN_ERR_BAD_ARG;
    if (count == 0) return VDNN_OK;
    const size_t n4 = (aligned16(x) && aligned16(dy) && aligned16(dx)) ? count / 4 : 0;
    relu_bwd_kernel<<<stream_grid(n4 ? n4 : count, 2), kThreads, 0, as_stream(stream)>>>(n4, count, dy, x, dx);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_activation_fwd(int mode, size_t count, const float* x, float* y, void* stream) {
    if (mode == VDNN_ACT_RELU) return vdnn_relu_fwd(count, x, y, stream);
    if (mode != VDNN_ACT_TANH && mode != VDNN_ACT_SIGMOID) return VDNN_ERR_UNSUPPORTED;
    if (!x || !y) return VDNN_ERR_BAD_ARG;
    if (count == 0) return VDNN_OK;
    const size_t n4 = (aligned16(x) && aligned16(y)) ? count / 4 : 0;
    const int grid = stream_grid(n4 ? n4 : count, 1);
    if (mode == VDNN_ACT_TANH) act_fwd_kernel<VDNN_ACT_TANH><<<grid, kThreads, 0, as_stream(stream)>>>(n4, count, x, y);
    else act_fwd_kernel<VDNN_ACT_SIGMOID><<<grid, kThreads, 0, as_stream(stream)>>>(n4, count, x, y);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_activation_bwd(int mode, size_t count, const float* y, const float* dy, const float* x, float* dx, void* stream) {
    if (mode == VDNN_ACT_RELU) return vdnn_relu_bwd(count, y, dy, x, dx, stream);
    if (mode != VDNN_ACT_TANH && mode != VDNN_ACT_SIGMOID) return VDNN_ERR_UNSUPPORTED;
    if (!y || !dy || !dx) return VDNN_ERR_BAD_ARG;
    if (count == 0) return VDNN_OK;
    const size_t n4 = (aligned16(y) && aligned16(dy) && aligned16(dx)) ? count / 4 : 0;
    const int grid = stream_grid(n4 ? n4 : count, 1);
    if (mode == VDNN_ACT_TANH) act_bwd_kernel<VDNN_ACT_TANH><<<grid, kThreads, 0, as_stream(stream)>>>(n4, count, y, dy, dx);
    else act_bwd_kernel<VDNN_ACT_SIGMOID><<<grid, kThreads, 0, as_stream(stream)>>>(n4, count, y, dy, dx);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_sub(size_t count, const float* a, const float* b, float* out, void* stream) {
    if (!a || !b || !out) return VDNN_ERR_BAD_ARG;
    if (count == 0) return VDNN_OK;
    sub_kernel<<<stream_grid(count, 1), kThreads, 0, as_stream(stream)>>>(count, a, b, out);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_axpy(size_t count, float alpha, const float* g, float* w, void* stream) {
    if (!g || !w) return VDNN_ERR_BAD_ARG;
    if (count == 0) return VDNN_OK;
    const size_t n4 = (aligned16(g) && aligned16(w)) ? count / 4 : 0;
    axpy_kernel<<<stream_grid(n4 ? n4 : count, 1), kThreads, 0, as_stream(stream)>>>(n4, count, alpha, g, w);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_fill(size_t count, float value, float* dst, void* stream) {
    if (!dst) return VDNN_ERR_BAD_ARG;
    if (count == 0) return VDNN_OK;
    fill_kernel<<<stream_grid(count, 1), kThreads, 0, as_stream(stream)>>>(count, value, dst);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_add_bias(int n, int k, int pq, float alpha, const float* bias, float* y, void* stream) {
    if (!bias || !y || n <= 0 || k <= 0 || pq <= 0) return VDNN_ERR_BAD_ARG;
    const int planes = n * k;
    dim3 grid(ceil_div(pq, kThreads * 4) > 0 ? ceil_div(pq, kThreads * 4) : 1, planes < 65535 ? planes : 65535);
    add_bias_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(planes, k, pq, alpha, bias, y);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_conv_bwd_bias(int n, int k, int pq, float alpha, const float* dy, float beta, float* db, void* stream) {
    if (!dy || !db || n <= 0 || k <= 0 || pq <= 0) return VDNN_ERR_BAD_ARG;
    if (beta != 1.0f) {
        scale_vec_kernel<<<ceil_div(k, kThreads), kThreads, 0, as_stream(stream)>>>(k, beta, db);
        VDNN_LAUNCHED();
    }
    // enough (channel, batch-slice) blocks to fill the machine a few times over
    int slices = ceil_div(sm_count() * 4, k);
    if (slices > n) slices = n;
    if (slices < 1) slices = 1;
    bwd_bias_kernel<<<dim3(k, slices), kThreads, 0, as_stream(stream)>>>(n, k, pq, alpha, dy, db);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_pool_out_dims(int h, int w, int win_h, int win_w, int stride_h, int stride_w, int* p, int* q) {
    if (!p || !q || win_h <= 0 || win_w <= 0 || stride_h <= 0 || stride_w <= 0 || h < win_h || w < win_w)
        return VDNN_ERR_BAD_ARG;
    *p = (h - win_h) / stride_h + 1;
    *q = (w - win_w) / stride_w + 1;
    return VDNN_OK;
}

static bool pool_fast_2x2(int h, int w, int wh, int ww, int sh, int sw, const void* a, const void* b, const void* c) {
    return wh == 2 && ww == 2 && sh == 2 && sw == 2 && h % 2 == 0 && w % 4 == 0 && aligned16(a) && aligned16(b) &&
           (c == nullptr || aligned16(c));
}

int vdnn_maxpool_fwd(int n, int c, int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                     const float* x, float* y, void* stream) {
    int P, Q;
    if (!x || !y || n <= 0 || c <= 0) return VDNN_ERR_BAD_ARG;
    if (vdnn_pool_out_dims(h, w, win_h, win_w, stride_h, stride_w, &P, &Q) != VDNN_OK) return VDNN_ERR_BAD_ARG;
    const int planes = n * c;
    if (pool_fast_2x2(h, w, win_h, win_w, stride_h, stride_w, x, y, nullptr)) {
        const size_t pairs = static_cast<size_t>(planes) * P * (Q / 2);
        maxpool_fwd_2x2<<<stream_grid(pairs, 1), kThreads, 0, as_stream(stream)>>>(pairs, w, Q / 2, x, y);
    } else {
        const size_t total = static_cast<size_t>(planes) * P * Q;
        maxpool_fwd_generic<<<stream_grid(total, 1), kThreads, 0, as_stream(stream)>>>(planes, h, w, P, Q, win_h, win_w,
                                                                                       stride_h, stride_w, x, y);
    }
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_maxpool_bwd(int n, int c, int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                     const float* y, const float* dy, const float* x, float* dx, void* stream) {
    (void)y;
    int P, Q;
    if (!dy || !x || !dx || n <= 0 || c <= 0) return VDNN_ERR_BAD_ARG;
    if (vdnn_pool_out_dims(h, w, win_h, win_w, stride_h, stride_w, &P, &Q) != VDNN_OK) return VDNN_ERR_BAD_ARG;
    const int planes = n * c;
    if (pool_fast_2x2(h, w, win_h, win_w, stride_h, stride_w, x, dx, dy)) {
        const size_t pairs = static_cast<size_t>(planes) * P * (Q / 2);
        maxpool_bwd_2x2<<<stream_grid(pairs, 1), kThreads, 0, as_stream(stream)>>>(pairs, w, Q / 2, dy, x, dx);
    } else if (win_h > stride_h || win_w > stride_w) {
        VDNN_CUDA(cudaMemsetAsync(dx, 0, static_cast<size_t>(planes) * h * w * sizeof(float), as_stream(stream)));
        const size_t total = static_cast<size_t>(planes) * P * Q;
        maxpool_bwd_scatter<<<stream_grid(total, 1), kThreads, 0, as_stream(stream)>>>(planes, h, w, P, Q, win_h, win_w,
                                                                                       stride_h, stride_w, dy, x, dx);
    } else {
        const size_t total = static_cast<size_t>(planes) * h * w;
        maxpool_bwd_generic<<<stream_grid(total, 1), kThreads, 0, as_stream(stream)>>>(planes, h, w, P, Q, win_h, win_w,
                                                                                       stride_h, stride_w, dy, x, dx);
    }
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_softmax_fwd(int rows, int cols, const float* x, float* y, void* stream) {
    if (!x || !y || rows <= 0 || cols <= 0) return VDNN_ERR_BAD_ARG;
    softmax_fwd_kernel<<<ceil_div(rows, 4), 128, 0, as_stream(stream)>>>(rows, cols, x, y);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_softmax_bwd(int rows, int cols, const float* y, const float* dy, float* dx, void* stream) {
    if (!y || !dy || !dx || rows <= 0 || cols <= 0) return VDNN_ERR_BAD_ARG;
    softmax_bwd_kernel<<<ceil_div(rows, 4), 128, 0, as_stream(stream)>>>(rows, cols, y, dy, dx);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_loss(int rows, int cols, const float* y, const float* label, double* out2, void* stream) {
    if (!y || !label || !out2 || rows <= 0 || cols <= 0) return VDNN_ERR_BAD_ARG;
    loss_kernel<<<1, 1024, 0, as_stream(stream)>>>(rows, cols, y, label, out2);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_lrn_fwd(int n, int c, int hw, int win, float alpha, float beta, float k, const float* x, float* y,
                 void* stream) {
    if (!x || !y || n <= 0 || c <= 0 || hw <= 0 || win <= 0 || win % 2 == 0) return VDNN_ERR_BAD_ARG;
    lrn_fwd_kernel<<<stream_grid(static_cast<size_t>(n) * hw, 1), kThreads, 0, as_stream(stream)>>>(
        n, c, hw, win, alpha / win, beta, k, x, y);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_lrn_bwd(int n, int c, int hw, int win, float alpha, float beta, float k, const float* x, const float* y,
                 const float* dy, float* dx, void* stream) {
    if (!x || !y || !dy || !dx || n <= 0 || c <= 0 || hw <= 0 || win <= 0 || win % 2 == 0) return VDNN_ERR_BAD_ARG;
    if (win == 5)
        lrn_bwd_win5_kernel<<<stream_grid(static_cast<size_t>(n) * hw, 1), kThreads, 0, as_stream(stream)>>>(
            n, c, hw, alpha / win, beta, k, x, y, dy, dx);
    else
        lrn_bwd_kernel<<<stream_grid(static_cast<size_t>(n) * hw, 1), kThreads, 0, as_stream(stream)>>>(
            n, c, hw, win, alpha / win, beta, k, x, y, dy, dx);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

int vdnn_offload(void* dst_pinned_h, const void* src, size_t bytes, void* ready_event, void* done_event,
                 void* copy_stream) {
    if (!dst_pinned_h || !src) return VDNN_ERR_BAD_ARG;
    cudaStream_t s = as_stream(copy_stream);
    if (ready_event) VDNN_CUDA(cudaStreamWaitEvent(s, static_cast<cudaEvent_t>(ready_event), 0));
    VDNN_CUDA(cudaMemcpyAsync(dst_pinned_h, src, bytes, cudaMemcpyDeviceToHost, s));
    if (done_event) VDNN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(done_event), s));
    return VDNN_OK;
}

int vdnn_prefetch(void* dst, const void* src_pinned_h, size_t bytes, void* ready_event, void* done_event,
                  void* copy_stream) {
    if (!dst || !src_pinned_h) return VDNN_ERR_BAD_ARG;
    cudaStream_t s = as_stream(copy_stream);
    if (ready_event) VDNN_CUDA(cudaStreamWaitEvent(s, static_cast<cudaEvent_t>(ready_event), 0));
    VDNN_CUDA(cudaMemcpyAsync(dst, src_pinned_h, bytes, cudaMemcpyHostToDevice, s));
    if (done_event) VDNN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(done_event), s));
    return VDNN_OK;
}

const char* vdnn_status_string(int status) {
    switch (status) {
    case VDNN_OK: return "VDNN_OK";
    case VDNN_ERR_BAD_ARG: return "VDNN_ERR_BAD_ARG";
    case VDNN_ERR_CUDA: return "VDNN_ERR_CUDA";
    case VDNN_ERR_WORKSPACE: return "VDNN_ERR_WORKSPACE";
    case VDNN_ERR_UNSUPPORTED: return "VDNN_ERR_UNSUPPORTED";
    case VDNN_ERR_OUT_OF_MEMORY: return "VDNN_ERR_OUT_OF_MEMORY";
    case VDNN_ERR_TIMEOUT: return "VDNN_ERR_TIMEOUT";
    case VDNN_ERR_STATE: return "VDNN_ERR_STATE";
    case VDNN_ERR_SCRATCH_LIMIT: return "VDNN_ERR_SCRATCH_LIMIT";
    default: return "VDNN_ERR_UNKNOWN";
    }
}

int vdnn_last_cuda_error(void) { return g_last_cuda_error; }

const char* vdnn_build_info(void) { return "vdnn_b200 0.1 (sm_100a)"; }

}  // extern "C"
