/*
 * CPU oracle for the vDNN training hot path.  TEST INFRASTRUCTURE ONLY: this file is
 * linked by the tests, the smoke check and the CPU-baseline leg of the benchmark and by
 * nothing else.  Every function names the reference lines it restates (paths are
 * relative to james98kr/vDNN_Implementation).  The arithmetic behind those lines is
 * cuDNN / cuBLAS (closed, not in the reference tree); what is restated here is the
 * published definition of each primitive with the reference's arguments.
 *
 * Build flavours:  -DORC_ACC=double  checker (default);  -DORC_ACC=float  timed baseline.
 * Compile with -ffp-contract=off so the RNG matches the product's host generator bit
 * for bit.
 */
#include "vdnn_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifndef ORC_ACC
#define ORC_ACC double
#endif
typedef ORC_ACC acc_t;

/* ------------------------------------------------------------------------- */
/* Philox4x32-10 (Salmon et al., SC'11): counter = element index, key = seed  */
/* ------------------------------------------------------------------------- */
static inline void philox4x32_10(uint64_t ctr, uint64_t key, uint32_t out[4]) {
    uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = 0u, c3 = 0u;
    uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);
    for (int i = 0; i < 10; ++i) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

static inline float u01(uint32_t r) { return (float)(r >> 8) * (1.0f / 16777216.0f); }

void orc_fill_uniform(float* dst, size_t n, uint64_t seed, float lo, float hi) {
    float span = hi - lo;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        uint32_t r[4];
        philox4x32_10((uint64_t)i, seed, r);
        float t = span * u01(r[0]);
        dst[i] = lo + t;
    }
}

void orc_fill_normal(float* dst, size_t n, uint64_t seed, float mean, float stddev) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        uint32_t r[4];
        philox4x32_10((uint64_t)i, seed, r);
        float u1 = (float)((r[0] >> 8) + 1u) * (1.0f / 16777216.0f); /* (0,1] */
        float u2 = u01(r[1]);
        float rad = sqrtf(-2.0f * logf(u1));
        float ang = 6.28318530717958647692f * u2;
        float z = rad * cosf(ang);
        float t = stddev * z;
        dst[i] = mean + t;
    }
}

void orc_fill_onehot(float* dst, int rows, int cols, uint64_t seed) {
    memset(dst, 0, sizeof(float) * (size_t)rows * cols);
    for (int i = 0; i < rows; ++i) {
        uint32_t r[4];
        philox4x32_10((uint64_t)i, seed, r);
        dst[(size_t)i * cols + (r[0] % (uint32_t)cols)] = 1.0f;
    }
}

/* ------------------------------------------------------------------------- */
/* Shapes: cudnnGetConvolution2dForwardOutputDim / cudnnGetPooling2dForward-   */
/* OutputDim with dilation 1 and pooling pad 0 (layer.cu:193-216, 417-439)     */
/* ------------------------------------------------------------------------- */
void orc_conv_out_dims(int h, int w, int pad_h, int pad_w, int stride_h, int stride_w,
                       int r, int s, int* p, int* q) {
    *p = (h + 2 * pad_h - r) / stride_h + 1;
    *q = (w + 2 * pad_w - s) / stride_w + 1;
}

void orc_pool_out_dims(int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                       int* p, int* q) {
    *p = (h - win_h) / stride_h + 1;
    *q = (w - win_w) / stride_w + 1;
}

/* ------------------------------------------------------------------------- */
/* Convolution (cross-correlation, vdnn.h:20)                                 */
/* ------------------------------------------------------------------------- */
void orc_conv_fwd(int n, int c, int h, int w, int k, int r, int s, int pad_h, int pad_w,
                  int stride_h, int stride_w, float alpha, const float* x, const float* wt,
                  float beta, float* y) {
    int P, Q;
    orc_conv_out_dims(h, w, pad_h, pad_w, stride_h, stride_w, r, s, &P, &Q);
    const size_t PQ = (size_t)P * Q;
#pragma omp parallel
    {
        acc_t* acc = (acc_t*)malloc(sizeof(acc_t) * PQ);
#pragma omp for collapse(2) schedule(dynamic)
        for (int in = 0; in < n; ++in)
            for (int ik = 0; ik < k; ++ik) {
                for (size_t i = 0; i < PQ; ++i) acc[i] = 0;
                for (int ic = 0; ic < c; ++ic) {
                    const float* xp = x + ((size_t)in * c + ic) * h * w;
                    for (int ir = 0; ir < r; ++ir)
                        for (int is = 0; is < s; ++is) {
                            const acc_t wv = wt[(((size_t)ik * c + ic) * r + ir) * s + is];
                            for (int p = 0; p < P; ++p) {
                                int ih = p * stride_h - pad_h + ir;
                                if (ih < 0 || ih >= h) continue;
                                const float* xr = xp + (size_t)ih * w;
                                acc_t* ar = acc + (size_t)p * Q;
                                /* q range with 0 <= q*stride - pad + is < w */
                                int q0 = 0, q1 = Q;
                                while (q0 < Q && q0 * stride_w - pad_w + is < 0) ++q0;
                                while (q1 > q0 && (q1 - 1) * stride_w - pad_w + is >= w) --q1;
                                if (stride_w == 1) {
                                    const float* xs = xr - pad_w + is;
                                    for (int q = q0; q < q1; ++q) ar[q] += wv * (acc_t)xs[q];
                                } else {
                                    for (int q = q0; q < q1; ++q)
                                        ar[q] += wv * (acc_t)xr[q * stride_w - pad_w + is];
                                }
                            }
                        }
                }
                float* yp = y + ((size_t)in * k + ik) * PQ;
                if (beta == 0.0f)
                    for (size_t i = 0; i < PQ; ++i) yp[i] = (float)((acc_t)alpha * acc[i]);
                else
                    for (size_t i = 0; i < PQ; ++i)
                        yp[i] = (float)((acc_t)alpha * acc[i] + (acc_t)beta * (acc_t)yp[i]);
            }
        free(acc);
    }
}

void orc_add_bias(int n, int k, int pq, const float* bias, float* y) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int in = 0; in < n; ++in)
        for (int ik = 0; ik < k; ++ik) {
            float* yp = y + ((size_t)in * k + ik) * pq;
            const float b = bias[ik];
            for (int i = 0; i < pq; ++i) yp[i] = yp[i] + b;
        }
}

void orc_conv_bwd_data(int n, int c, int h, int w, int k, int r, int s, int pad_h, int pad_w,
                       int stride_h, int stride_w, float alpha, const float* wt,
                       const float* dy, float beta, float* dx) {
    int P, Q;
    orc_conv_out_dims(h, w, pad_h, pad_w, stride_h, stride_w, r, s, &P, &Q);
    const size_t HW = (size_t)h * w, PQ = (size_t)P * Q;
#pragma omp parallel
    {
        acc_t* acc = (acc_t*)malloc(sizeof(acc_t) * HW);
#pragma omp for collapse(2) schedule(dynamic)
        for (int in = 0; in < n; ++in)
            for (int ic = 0; ic < c; ++ic) {
                for (size_t i = 0; i < HW; ++i) acc[i] = 0;
                for (int ik = 0; ik < k; ++ik) {
                    const float* dyp = dy + ((size_t)in * k + ik) * PQ;
                    for (int ir = 0; ir < r; ++ir)
                        for (int is = 0; is < s; ++is) {
                            const acc_t wv = wt[(((size_t)ik * c + ic) * r + ir) * s + is];
                            for (int p = 0; p < P; ++p) {
                                int ih = p * stride_h - pad_h + ir;
                                if (ih < 0 || ih >= h) continue;
                                acc_t* ar = acc + (size_t)ih * w;
                                const float* dr = dyp + (size_t)p * Q;
                                int q0 = 0, q1 = Q;
                                while (q0 < Q && q0 * stride_w - pad_w + is < 0) ++q0;
                                while (q1 > q0 && (q1 - 1) * stride_w - pad_w + is >= w) --q1;
                                if (stride_w == 1) {
                                    acc_t* as = ar - pad_w + is;
                                    for (int q = q0; q < q1; ++q) as[q] += wv * (acc_t)dr[q];
                                } else {
                                    for (int q = q0; q < q1; ++q)
                                        ar[q * stride_w - pad_w + is] += wv * (acc_t)dr[q];
                                }
                            }
                        }
                }
                float* dxp = dx + ((size_t)in * c + ic) * HW;
                if (beta == 0.0f)
                    for (size_t i = 0; i < HW; ++i) dxp[i] = (float)((acc_t)alpha * acc[i]);
                else
                    for (size_t i = 0; i < HW; ++i)
                        dxp[i] = (float)((acc_t)alpha * acc[i] + (acc_t)beta * (acc_t)dxp[i]);
            }
        free(acc);
    }
}

void orc_conv_bwd_bias(int n, int k, int pq, float alpha, const float* dy, float beta, float* db) {
#pragma omp parallel for schedule(static)
    for (int ik = 0; ik < k; ++ik) {
        acc_t acc = 0;
        for (int in = 0; in < n; ++in) {
            const float* p = dy + ((size_t)in * k + ik) * pq;
            for (int i = 0; i < pq; ++i) acc += (acc_t)p[i];
        }
        acc_t prev = (beta == 0.0f) ? (acc_t)0 : (acc_t)beta * (acc_t)db[ik];
        db[ik] = (float)((acc_t)alpha * acc + prev);
    }
}

void orc_conv_bwd_filter(int n, int c, int h, int w, int k, int r, int s, int pad_h, int pad_w,
                         int stride_h, int stride_w, float alpha, const float* x,
                         const float* dy, float beta, float* dw) {
    int P, Q;
    orc_conv_out_dims(h, w, pad_h, pad_w, stride_h, stride_w, r, s, &P, &Q);
    const size_t HW = (size_t)h * w, PQ = (size_t)P * Q;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int ik = 0; ik < k; ++ik)
        for (int ic = 0; ic < c; ++ic)
            for (int ir = 0; ir < r; ++ir)
                for (int is = 0; is < s; ++is) {
                    acc_t acc = 0;
                    int q0 = 0, q1 = Q;
                    while (q0 < Q && q0 * stride_w - pad_w + is < 0) ++q0;
                    while (q1 > q0 && (q1 - 1) * stride_w - pad_w + is >= w) --q1;
                    for (int in = 0; in < n; ++in) {
                        const float* xp = x + ((size_t)in * c + ic) * HW;
                        const float* dyp = dy + ((size_t)in * k + ik) * PQ;
                        for (int p = 0; p < P; ++p) {
                            int ih = p * stride_h - pad_h + ir;
                            if (ih < 0 || ih >= h) continue;
                            const float* xr = xp + (size_t)ih * w;
                            const float* dr = dyp + (size_t)p * Q;
                            acc_t part = 0;
                            if (stride_w == 1) {
                                const float* xs = xr - pad_w + is;
                                for (int q = q0; q < q1; ++q) part += (acc_t)xs[q] * (acc_t)dr[q];
                            } else {
                                for (int q = q0; q < q1; ++q)
                                    part += (acc_t)xr[q * stride_w - pad_w + is] * (acc_t)dr[q];
                            }
                            acc += part;
                        }
                    }
                    size_t idx = (((size_t)ik * c + ic) * r + ir) * s + is;
                    acc_t prev = (beta == 0.0f) ? (acc_t)0 : (acc_t)beta * (acc_t)dw[idx];
                    dw[idx] = (float)((acc_t)alpha * acc + prev);
                }
}

/* ------------------------------------------------------------------------- */
/* cublasSgemm semantics, column major: C = alpha*op(A)*op(B) + beta*C         */
/* ------------------------------------------------------------------------- */
void orc_sgemm(int transa, int transb, int m, int n, int k, float alpha, const float* A, int lda,
               const float* B, int ldb, float beta, float* C, int ldc) {
#pragma omp parallel
    {
        acc_t* acc = (acc_t*)malloc(sizeof(acc_t) * (size_t)(m > 0 ? m : 1));
#pragma omp for schedule(dynamic)
        for (int j = 0; j < n; ++j) {
            for (int i = 0; i < m; ++i) acc[i] = 0;
            if (!transa) {
                for (int l = 0; l < k; ++l) {
                    const acc_t b = transb ? B[(size_t)j + (size_t)l * ldb] : B[(size_t)l + (size_t)j * ldb];
                    const float* a = A + (size_t)l * lda;
                    for (int i = 0; i < m; ++i) acc[i] += (acc_t)a[i] * b;
                }
            } else {
                for (int i = 0; i < m; ++i) {
                    const float* a = A + (size_t)i * lda;
                    acc_t t = 0;
                    if (!transb) {
                        const float* b = B + (size_t)j * ldb;
                        for (int l = 0; l < k; ++l) t += (acc_t)a[l] * (acc_t)b[l];
                    } else {
                        for (int l = 0; l < k; ++l) t += (acc_t)a[l] * (acc_t)B[(size_t)j + (size_t)l * ldb];
                    }
                    acc[i] = t;
                }
            }
            float* c = C + (size_t)j * ldc;
            if (beta == 0.0f)
                for (int i = 0; i < m; ++i) c[i] = (float)((acc_t)alpha * acc[i]);
            else
                for (int i = 0; i < m; ++i)
                    c[i] = (float)((acc_t)alpha * acc[i] + (acc_t)beta * (acc_t)c[i]);
        }
        free(acc);
    }
}

/* ------------------------------------------------------------------------- */
/* Activation: CUDNN_ACTIVATION_RELU, CUDNN_PROPAGATE_NAN (layer.cu:380-385)   */
/* ------------------------------------------------------------------------- */
void orc_relu_fwd(size_t n, const float* x, float* y) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        float v = x[i];
        y[i] = (v > 0.0f) ? v : ((v != v) ? v : 0.0f);
    }
}

void orc_relu_bwd(size_t n, const float* y, const float* dy, const float* x, float* dx) {
    (void)y;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) dx[i] = (x[i] > 0.0f) ? dy[i] : 0.0f;
}

/* tanh / sigmoid as cudnnActivationForward / Backward define them: the backward reads y only. */
void orc_act_fwd(int mode, size_t n, const float* x, float* y) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const double v = x[i];
        y[i] = (float)(mode == 1 ? tanh(v) : 1.0 / (1.0 + exp(-v)));
    }
}

void orc_act_bwd(int mode, size_t n, const float* y, const float* dy, float* dx) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const double a = y[i], d = dy[i];
        dx[i] = (float)(mode == 1 ? d * (1.0 - a * a) : d * a * (1.0 - a));
    }
}

/* ------------------------------------------------------------------------- */
/* Max pooling, pad 0, NOT_PROPAGATE_NAN (layer.cu:417-428).  Backward routes  */
/* dy to the first window element (row-major scan) equal to the window max.    */
/* ------------------------------------------------------------------------- */
void orc_maxpool_fwd(int n, int c, int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                     const float* x, float* y) {
    int P, Q;
    orc_pool_out_dims(h, w, win_h, win_w, stride_h, stride_w, &P, &Q);
#pragma omp parallel for schedule(static)
    for (long nc = 0; nc < (long)n * c; ++nc) {
        const float* xp = x + (size_t)nc * h * w;
        float* yp = y + (size_t)nc * P * Q;
        for (int p = 0; p < P; ++p)
            for (int q = 0; q < Q; ++q) {
                float m = -INFINITY;
                for (int i = 0; i < win_h; ++i)
                    for (int j = 0; j < win_w; ++j) {
                        float v = xp[(size_t)(p * stride_h + i) * w + q * stride_w + j];
                        if (v > m) m = v;
                    }
                yp[(size_t)p * Q + q] = m;
            }
    }
}

void orc_maxpool_bwd(int n, int c, int h, int w, int win_h, int win_w, int stride_h, int stride_w,
                     const float* y, const float* dy, const float* x, float* dx) {
    int P, Q;
    (void)y;
    orc_pool_out_dims(h, w, win_h, win_w, stride_h, stride_w, &P, &Q);
#pragma omp parallel for schedule(static)
    for (long nc = 0; nc < (long)n * c; ++nc) {
        const float* xp = x + (size_t)nc * h * w;
        const float* dyp = dy + (size_t)nc * P * Q;
        float* dxp = dx + (size_t)nc * h * w;
        for (size_t i = 0; i < (size_t)h * w; ++i) dxp[i] = 0.0f;
        for (int p = 0; p < P; ++p)
            for (int q = 0; q < Q; ++q) {
                float m = -INFINITY;
                int bi = 0, bj = 0;
                for (int i = 0; i < win_h; ++i)
                    for (int j = 0; j < win_w; ++j) {
                        float v = xp[(size_t)(p * stride_h + i) * w + q * stride_w + j];
                        if (v > m) { m = v; bi = i; bj = j; }
                    }
                dxp[(size_t)(p * stride_h + bi) * w + q * stride_w + bj] += dyp[(size_t)p * Q + q];
            }
    }
}

/* ------------------------------------------------------------------------- */
/* Softmax ACCURATE; INSTANCE == CHANNEL when H = W = 1 (layer.cu:824-862)     */
/* ------------------------------------------------------------------------- */
void orc_softmax_fwd(int rows, int cols, const float* x, float* y) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < rows; ++i) {
        const float* xr = x + (size_t)i * cols;
        float* yr = y + (size_t)i * cols;
        float m = xr[0];
        for (int j = 1; j < cols; ++j) if (xr[j] > m) m = xr[j];
        acc_t sum = 0;
        for (int j = 0; j < cols; ++j) sum += (acc_t)expf(xr[j] - m);
        for (int j = 0; j < cols; ++j) yr[j] = (float)((acc_t)expf(xr[j] - m) / sum);
    }
}

void orc_softmax_bwd(int rows, int cols, const float* y, const float* dy, float* dx) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < rows; ++i) {
        const float* yr = y + (size_t)i * cols;
        const float* dr = dy + (size_t)i * cols;
        float* xr = dx + (size_t)i * cols;
        acc_t dot = 0;
        for (int j = 0; j < cols; ++j) dot += (acc_t)yr[j] * (acc_t)dr[j];
        for (int j = 0; j < cols; ++j) xr[j] = (float)((acc_t)yr[j] * ((acc_t)dr[j] - dot));
    }
}

void orc_sub(size_t n, const float* a, const float* b, float* out) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) out[i] = a[i] - b[i];
}

/* ------------------------------------------------------------------------- */
/* Cross-channel LRN: scale_i = k + (alpha/win) * sum_{|j-i|<=win/2} x_j^2,     */
/* y_i = x_i * scale_i^-beta.  Not in the reference (its AlexNet has no LRN).   */
/* ------------------------------------------------------------------------- */
void orc_lrn_fwd(int n, int c, int hw, int win, float alpha, float beta, float k,
                 const float* x, float* y) {
    const int half = win / 2;
#pragma omp parallel for schedule(static)
    for (int in = 0; in < n; ++in)
        for (int ic = 0; ic < c; ++ic) {
            int lo = ic - half < 0 ? 0 : ic - half;
            int hi = ic + half >= c ? c - 1 : ic + half;
            for (int i = 0; i < hw; ++i) {
                acc_t ss = 0;
                for (int j = lo; j <= hi; ++j) {
                    acc_t v = x[((size_t)in * c + j) * hw + i];
                    ss += v * v;
                }
                acc_t scale = (acc_t)k + ((acc_t)alpha / (acc_t)win) * ss;
                size_t idx = ((size_t)in * c + ic) * hw + i;
                y[idx] = (float)((acc_t)x[idx] * pow((double)scale, -(double)beta));
            }
        }
}

void orc_lrn_bwd(int n, int c, int hw, int win, float alpha, float beta, float k,
                 const float* x, const float* y, const float* dy, float* dx) {
    const int half = win / 2;
#pragma omp parallel for schedule(static)
    for (int in = 0; in < n; ++in) {
        acc_t* scale = (acc_t*)malloc(sizeof(acc_t) * (size_t)c);
        for (int i = 0; i < hw; ++i) {
            for (int ic = 0; ic < c; ++ic) {
                int lo = ic - half < 0 ? 0 : ic - half;
                int hi = ic + half >= c ? c - 1 : ic + half;
                acc_t ss = 0;
                for (int j = lo; j <= hi; ++j) {
                    acc_t v = x[((size_t)in * c + j) * hw + i];
                    ss += v * v;
                }
                scale[ic] = (acc_t)k + ((acc_t)alpha / (acc_t)win) * ss;
            }
            for (int ic = 0; ic < c; ++ic) {
                int lo = ic - half < 0 ? 0 : ic - half;
                int hi = ic + half >= c ? c - 1 : ic + half;
                acc_t t = 0;
                for (int j = lo; j <= hi; ++j) {
                    size_t jdx = ((size_t)in * c + j) * hw + i;
                    t += (acc_t)dy[jdx] * (acc_t)y[jdx] / scale[j];
                }
                size_t idx = ((size_t)in * c + ic) * hw + i;
                acc_t g = (acc_t)dy[idx] * pow((double)scale[ic], -(double)beta)
                        - ((acc_t)2 * (acc_t)alpha * (acc_t)beta / (acc_t)win) * (acc_t)x[idx] * t;
                dx[idx] = (float)g;
            }
        }
        free(scale);
    }
}

void orc_loss(int rows, int cols, const float* y, const float* label, double* out) {
    double sq = 0, ce = 0;
    for (int i = 0; i < rows; ++i) {
        const float* yr = y + (size_t)i * cols;
        const float* tr = label + (size_t)i * cols;
        int arg = 0;
        for (int j = 0; j < cols; ++j) {
            double d = (double)yr[j] - (double)tr[j];
            sq += d * d;
            if (tr[j] > tr[arg]) arg = j;
        }
        double p = yr[arg];
        ce += -log(p > 1e-30 ? p : 1e-30);
    }
    out[0] = 0.5 * sq / rows;
    out[1] = ce / rows;
}

/* ------------------------------------------------------------------------- */
/* Topologies (network.cu:156-323 AlexNet, 325-495 OverFeat, 501-813 VGG16)    */
/* ------------------------------------------------------------------------- */
void orc_layer_out_dims(const orc_layer_spec* l, int* n, int* c, int* h, int* w) {
    *n = l->n;
    switch (l->type) {
    case ORC_FC_GEMM: *c = l->k; *h = 1; *w = 1; break;
    case ORC_CONV: case ORC_FC_CONV:
        *c = l->k;
        orc_conv_out_dims(l->h, l->w, l->pad_h, l->pad_w, l->stride_h, l->stride_w, l->r, l->s, h, w);
        break;
    case ORC_POOL:
        *c = l->c;
        orc_pool_out_dims(l->h, l->w, l->r, l->s, l->stride_h, l->stride_w, h, w);
        break;
    default: *c = l->c; *h = l->h; *w = l->w; break;
    }
}

typedef struct { orc_layer_spec* out; int max; int count; int n, c, h, w; } builder;

static void push(builder* b, int type, int pad, int stride, int k, int r) {
    orc_layer_spec l;
    l.type = type; l.n = b->n; l.c = b->c; l.h = b->h; l.w = b->w;
    l.pad_h = l.pad_w = pad; l.stride_h = l.stride_w = stride; l.k = k; l.r = l.s = r;
    if (type == ORC_FC_GEMM) { l.c = b->c * b->h * b->w; l.h = l.w = 1; }
    if (b->count < b->max) b->out[b->count] = l;
    b->count++;
    orc_layer_out_dims(&l, &b->n, &b->c, &b->h, &b->w);
}
static void conv_relu(builder* b, int pad, int stride, int k, int r) {
    push(b, ORC_FC_CONV, pad, stride, k, r);   /* the reference tags every conv FC_CONV */
    push(b, ORC_RELU, 0, 0, 0, 0);
}
static void fc_relu(builder* b, int k) { push(b, ORC_FC_GEMM, 0, 0, k, 1); push(b, ORC_RELU, 0, 0, 0, 0); }

int orc_model_layers(int cnn_type, int batch, orc_layer_spec* out, int max_layers) {
    builder b; b.out = out; b.max = max_layers; b.count = 0; b.n = batch; b.c = 3;
    switch (cnn_type) {
    case ORC_ALEXNET: case ORC_ALEXNET_LRN: {
        int lrn = (cnn_type == ORC_ALEXNET_LRN);
        b.h = b.w = 227;
        conv_relu(&b, 0, 4, 96, 11);  if (lrn) push(&b, ORC_LRN, 0, 0, 0, 5); push(&b, ORC_POOL, 0, 2, 0, 3);
        conv_relu(&b, 2, 1, 256, 5);  if (lrn) push(&b, ORC_LRN, 0, 0, 0, 5); push(&b, ORC_POOL, 0, 2, 0, 3);
        conv_relu(&b, 1, 1, 384, 3);
        conv_relu(&b, 1, 1, 384, 3);
        conv_relu(&b, 1, 1, 256, 3);  push(&b, ORC_POOL, 0, 2, 0, 3);
        fc_relu(&b, 4096); fc_relu(&b, 4096);
        push(&b, ORC_FC_GEMM, 0, 0, 1000, 1);
        push(&b, ORC_SOFTMAX, 0, 0, 0, 0);
    } break;
    case ORC_OVERFEAT:
        b.h = b.w = 231;
        conv_relu(&b, 0, 4, 96, 11);  push(&b, ORC_POOL, 0, 2, 0, 2);
        conv_relu(&b, 0, 1, 256, 5);  push(&b, ORC_POOL, 0, 2, 0, 2);
        conv_relu(&b, 1, 1, 512, 3);
        conv_relu(&b, 1, 1, 1024, 3);
        conv_relu(&b, 1, 1, 1024, 3); push(&b, ORC_POOL, 0, 2, 0, 2);
        conv_relu(&b, 0, 1, 3072, 6);
        conv_relu(&b, 0, 1, 4096, 1);
        push(&b, ORC_FC_CONV, 0, 1, 1000, 1);
        push(&b, ORC_SOFTMAX, 0, 0, 0, 0);
        break;
    case ORC_VGG16_64: case ORC_VGG16_128: case ORC_VGG16_256: {
        static const int width[5] = {64, 128, 256, 512, 512};
        static const int reps[5] = {2, 2, 3, 3, 3};
        b.h = b.w = 224;
        for (int blk = 0; blk < 5; ++blk) {
            for (int i = 0; i < reps[blk]; ++i) conv_relu(&b, 1, 1, width[blk], 3);
            push(&b, ORC_POOL, 0, 2, 0, 2);
        }
        fc_relu(&b, 4096); fc_relu(&b, 4096);
        push(&b, ORC_FC_GEMM, 0, 0, 1000, 1);
        push(&b, ORC_SOFTMAX, 0, 0, 0, 0);
    } break;
    default: return 0;
    }
    return b.count;
}

/* ------------------------------------------------------------------------- */
/* Whole-network step                                                         */
/* ------------------------------------------------------------------------- */
struct orc_net {
    int L;
    float lr;
    orc_layer_spec* spec;
    int (*od)[4];
    float** w; float** b; size_t* wn;
    float** dst; float** grad;
    float* input; float* label;
};

static size_t src_size(const orc_layer_spec* l) { return (size_t)l->n * l->c * l->h * l->w; }

size_t orc_net_src_size(const orc_net* net, int l) { return src_size(&net->spec[l]); }
size_t orc_net_dst_size(const orc_net* net, int l) {
    return (size_t)net->od[l][0] * net->od[l][1] * net->od[l][2] * net->od[l][3];
}
int orc_net_num_layers(const orc_net* net) { return net->L; }
size_t orc_net_input_size(const orc_net* net) { return orc_net_src_size(net, 0); }
size_t orc_net_output_size(const orc_net* net) { return orc_net_dst_size(net, net->L - 1); }
const float* orc_net_dst(const orc_net* net, int l) { return net->dst[l]; }
const float* orc_net_grad(const orc_net* net, int l) { return net->grad[l]; }
float* orc_net_weights(orc_net* net, int l) { return net->w[l]; }
float* orc_net_bias(orc_net* net, int l) { return net->b[l]; }
size_t orc_net_weight_count(const orc_net* net, int l) { return net->wn[l]; }

orc_net* orc_net_create(const orc_layer_spec* specs, int num_layers, float lr, int init_mode,
                        uint64_t weight_seed_base) {
    orc_net* net = (orc_net*)calloc(1, sizeof(orc_net));
    net->L = num_layers; net->lr = lr;
    net->spec = (orc_layer_spec*)malloc(sizeof(orc_layer_spec) * num_layers);
    memcpy(net->spec, specs, sizeof(orc_layer_spec) * num_layers);
    net->od = malloc(sizeof(int[4]) * num_layers);
    net->w = calloc(num_layers, sizeof(float*)); net->b = calloc(num_layers, sizeof(float*));
    net->wn = calloc(num_layers, sizeof(size_t));
    net->dst = calloc(num_layers, sizeof(float*)); net->grad = calloc(num_layers, sizeof(float*));
    for (int l = 0; l < num_layers; ++l) {
        const orc_layer_spec* s = &net->spec[l];
        orc_layer_out_dims(s, &net->od[l][0], &net->od[l][1], &net->od[l][2], &net->od[l][3]);
        net->dst[l] = (float*)malloc(sizeof(float) * orc_net_dst_size(net, l));
        net->grad[l] = (float*)malloc(sizeof(float) * src_size(s));
        if (s->type == ORC_FC_GEMM || s->type == ORC_CONV || s->type == ORC_FC_CONV) {
            size_t fan_in = (size_t)s->c * s->r * s->s;
            net->wn[l] = (size_t)s->k * fan_in;
            net->w[l] = (float*)malloc(sizeof(float) * net->wn[l]);
            net->b[l] = (float*)malloc(sizeof(float) * s->k);
            uint64_t seed = weight_seed_base + (uint64_t)l;
            if (init_mode == 0) {
                orc_fill_normal(net->w[l], net->wn[l], seed, 0.0f, sqrtf(2.0f / (float)fan_in));
                memset(net->b[l], 0, sizeof(float) * s->k);
            } else {
                orc_fill_uniform(net->w[l], net->wn[l], seed, -0.01f, 0.01f);
                orc_fill_uniform(net->b[l], s->k, seed + 0x100000000ull, -0.01f, 0.01f);
            }
        }
    }
    net->input = (float*)malloc(sizeof(float) * orc_net_input_size(net));
    net->label = (float*)malloc(sizeof(float) * orc_net_output_size(net));
    return net;
}

void orc_net_destroy(orc_net* net) {
    if (!net) return;
    for (int l = 0; l < net->L; ++l) { free(net->w[l]); free(net->b[l]); free(net->dst[l]); free(net->grad[l]); }
    free(net->w); free(net->b); free(net->wn); free(net->dst); free(net->grad);
    free(net->od); free(net->spec); free(net->input); free(net->label); free(net);
}

void orc_net_set_input(orc_net* net, const float* input, const float* label) {
    memcpy(net->input, input, sizeof(float) * orc_net_input_size(net));
    memcpy(net->label, label, sizeof(float) * orc_net_output_size(net));
}

/* forward loop of network.cu:1056-1110 with the per-type bodies of layer.cu:539-915 */
void orc_net_forward(orc_net* net) {
    for (int l = 0; l < net->L; ++l) {
        const orc_layer_spec* s = &net->spec[l];
        const float* src = l == 0 ? net->input : net->dst[l - 1];
        float* dst = net->dst[l];
        const int* od = net->od[l];
        switch (s->type) {
        case ORC_CONV: case ORC_FC_CONV:
            orc_conv_fwd(s->n, s->c, s->h, s->w, s->k, s->r, s->s, s->pad_h, s->pad_w, s->stride_h,
                         s->stride_w, 1.0f, src, net->w[l], 0.0f, dst);
            orc_add_bias(s->n, s->k, od[2] * od[3], net->b[l], dst);
            break;
        case ORC_FC_GEMM:
            /* layer.cu:677-685 then the rank-1 bias GEMM of layer.cu:697-705 */
            orc_sgemm(1, 0, s->k, s->n, s->c, 1.0f, net->w[l], s->c, src, s->c, 0.0f, dst, s->k);
            orc_add_bias(s->n, s->k, 1, net->b[l], dst);
            break;
        case ORC_RELU: orc_relu_fwd(src_size(s), src, dst); break;
        case ORC_TANH: orc_act_fwd(1, src_size(s), src, dst); break;
        case ORC_SIGMOID: orc_act_fwd(2, src_size(s), src, dst); break;
        case ORC_POOL:
            orc_maxpool_fwd(s->n, s->c, s->h, s->w, s->r, s->s, s->stride_h, s->stride_w, src, dst);
            break;
        case ORC_SOFTMAX: orc_softmax_fwd(s->n, s->c * s->h * s->w, src, dst); break;
        case ORC_LRN:
            orc_lrn_fwd(s->n, s->c, s->h * s->w, s->r, 1e-4f, 0.75f, 2.0f, src, dst);
            break;
        default: break;
        }
    }
}

/* backward loop of network.cu:1112-1191; update order of layer.cu:615-662, 725-761 */
void orc_net_backward(orc_net* net) {
    const int L = net->L;
    size_t out = orc_net_output_size(net);
    float* diff = (float*)malloc(sizeof(float) * out);
    orc_sub(out, net->dst[L - 1], net->label, diff);          /* network.cu:1042-1054 */
    const float* dy = diff;
    const float nlr = net->lr * -1.0f;
    for (int l = L - 1; l >= 0; --l) {
        const orc_layer_spec* s = &net->spec[l];
        const float* src = l == 0 ? net->input : net->dst[l - 1];
        const float* dst = net->dst[l];
        float* dx = net->grad[l];
        const int* od = net->od[l];
        switch (s->type) {
        case ORC_CONV: case ORC_FC_CONV:
            orc_conv_bwd_data(s->n, s->c, s->h, s->w, s->k, s->r, s->s, s->pad_h, s->pad_w,
                              s->stride_h, s->stride_w, 1.0f, net->w[l], dy, 0.0f, dx);
            orc_conv_bwd_bias(s->n, s->k, od[2] * od[3], nlr, dy, 1.0f, net->b[l]);
            orc_conv_bwd_filter(s->n, s->c, s->h, s->w, s->k, s->r, s->s, s->pad_h, s->pad_w,
                                s->stride_h, s->stride_w, nlr, src, dy, 1.0f, net->w[l]);
            break;
        case ORC_FC_GEMM:
            orc_sgemm(0, 0, s->c, s->n, s->k, 1.0f, net->w[l], s->c, dy, s->k, 0.0f, dx, s->c);
            orc_sgemm(0, 1, s->c, s->k, s->n, nlr, src, s->c, dy, s->k, 1.0f, net->w[l], s->c);
            orc_conv_bwd_bias(s->n, s->k, 1, nlr, dy, 1.0f, net->b[l]);
            break;
        case ORC_RELU: orc_relu_bwd(src_size(s), dst, dy, src, dx); break;
        case ORC_TANH: orc_act_bwd(1, src_size(s), dst, dy, dx); break;
        case ORC_SIGMOID: orc_act_bwd(2, src_size(s), dst, dy, dx); break;
        case ORC_POOL:
            orc_maxpool_bwd(s->n, s->c, s->h, s->w, s->r, s->s, s->stride_h, s->stride_w, dst, dy, src, dx);
            break;
        case ORC_SOFTMAX: orc_softmax_bwd(s->n, s->c * s->h * s->w, dst, dy, dx); break;
        case ORC_LRN:
            orc_lrn_bwd(s->n, s->c, s->h * s->w, s->r, 1e-4f, 0.75f, 2.0f, src, dst, dy, dx);
            break;
        default: break;
        }
        dy = dx;
    }
    free(diff);
}

void orc_net_loss(const orc_net* net, double* out2) {
    const orc_layer_spec* s = &net->spec[net->L - 1];
    orc_loss(s->n, s->c * s->h * s->w, net->dst[net->L - 1], net->label, out2);
}

/* ------------------------------------------------------------------------- */
/* Schedule simulator                                                         */
/* ------------------------------------------------------------------------- */
int orc_find_prefetch_layer(const int* layer_types, const unsigned char* is_offload,
                            unsigned char* is_prefetched, int cur) {
    /* network.cu:1198-1207 */
    for (int id = cur - 1; id >= 0; --id) {
        if (is_offload[id] && !is_prefetched[id]) { is_prefetched[id] = 1; return id; }
        else if (layer_types[id] == ORC_FC_CONV || layer_types[id] == ORC_CONV) return -1;
    }
    return -1;
}

typedef struct {
    orc_event* ev; int max; int n; int overflow;
    int64_t used, peak;
} tracer;

static int64_t round512(int64_t b) { return (b + 511) / 512 * 512; }   /* cnmem granularity */

static void emit(tracer* t, int kind, int layer, int tag, int64_t bytes) {
    if (kind == ORC_EV_ALLOC) { t->used += round512(bytes); if (t->used > t->peak) t->peak = t->used; }
    if (kind == ORC_EV_FREE) t->used -= round512(bytes);
    if (t->n < t->max) {
        orc_event* e = &t->ev[t->n];
        e->kind = kind; e->layer = layer; e->tag = tag; e->bytes = bytes; e->used = t->used;
    } else t->overflow = 1;
    t->n++;
}

int orc_policy_trace(const orc_layer_spec* specs, int L, int vdnn_type, const int64_t* ws,
                     int iterations, int fix_input_leak, orc_event* events, int max_events,
                     orc_trace_summary* sum, int wide_workspace) {
    tracer t; memset(&t, 0, sizeof t); t.ev = events; t.max = events ? max_events : 0;
    int64_t* srcB = malloc(sizeof(int64_t) * L); int64_t* dstB = malloc(sizeof(int64_t) * L);
    int* types = malloc(sizeof(int) * L);
    unsigned char* off = calloc(L, 1); unsigned char* pre = calloc(L, 1);
    int64_t max_dxdy = 0, pinned = 0, offB = 0, preB = 0;
    /* network.cu:1025-1040 keeps the maximum in an int: sizes wrap at 2^31.  wide_workspace = 1 keeps it in 64 bits
       instead (what a driver must do whose kernels really write the workspace they asked for). */
    int64_t max_ws = 0;
    for (int l = 0; l < L; ++l) {
        int n, c, h, w; orc_layer_out_dims(&specs[l], &n, &c, &h, &w);
        srcB[l] = 4 * (int64_t)src_size(&specs[l]); dstB[l] = 4 * (int64_t)n * c * h * w;
        types[l] = specs[l].type;
    }
#define WS(l, j) (ws ? ws[3 * (l) + (j)] : 0)
#define IS_W(l) (types[l] == ORC_CONV || types[l] == ORC_FC_CONV || types[l] == ORC_FC_GEMM)
#define IS_C(l) (types[l] == ORC_CONV || types[l] == ORC_FC_CONV)
    /* construction: Network::Network -> setLayers (layer ctors) -> setVdnnType -> input, label */
    for (int l = 0; l < L; ++l) {
        if (IS_W(l)) {
            emit(&t, ORC_EV_ALLOC, l, ORC_TAG_WEIGHT, 4 * (int64_t)specs[l].k * specs[l].c * specs[l].r * specs[l].s);
            emit(&t, ORC_EV_ALLOC, l, ORC_TAG_BIAS, 4 * (int64_t)specs[l].k);
        }
        if (vdnn_type == ORC_BASELINE) emit(&t, ORC_EV_ALLOC, l, ORC_TAG_DST, dstB[l]);
        if (srcB[l] > max_dxdy) max_dxdy = srcB[l];
        if (IS_C(l)) for (int j = 0; j < 3; ++j) {
            int64_t temp = wide_workspace ? WS(l, j) : (int64_t)(int32_t)(uint32_t)(uint64_t)WS(l, j);
            if (max_ws < temp) max_ws = temp;
        }
    }
    if (dstB[L - 1] > max_dxdy) max_dxdy = dstB[L - 1];
    if (vdnn_type == ORC_BASELINE) {                       /* network.cu:894-906 */
        emit(&t, ORC_EV_ALLOC, -1, ORC_TAG_DXDY, max_dxdy);
        emit(&t, ORC_EV_ALLOC, -1, ORC_TAG_DXDY, max_dxdy);
        if (max_ws > 0) emit(&t, ORC_EV_ALLOC, -1, ORC_TAG_WS, max_ws);
    } else if (vdnn_type == ORC_VDNN_ALL) {                /* network.cu:913-923 */
        for (int l = 0; l < L - 1; ++l) { off[l] = 1; pinned += srcB[l]; }
    } else if (vdnn_type == ORC_VDNN_CONV) {               /* network.cu:926-938 */
        for (int l = 0; l < L - 1; ++l) if (IS_C(l)) { off[l] = 1; pinned += srcB[l]; }
    }
    emit(&t, ORC_EV_ALLOC, -1, ORC_TAG_INPUT, srcB[0]);
    emit(&t, ORC_EV_ALLOC, -1, ORC_TAG_LABEL, dstB[L - 1]);
    int64_t static_bytes = t.used;

    for (int it = 0; it < iterations; ++it) {
        /* ---- forward: network.cu:1056-1110 ---- */
        for (int l = 0; l < L; ++l) {
            if (vdnn_type == ORC_BASELINE) {
                if (types[l] == ORC_FC_GEMM) {
                    emit(&t, ORC_EV_ALLOC, l, ORC_TAG_ONES, 4 * (int64_t)specs[l].n);
                    emit(&t, ORC_EV_FREE, l, ORC_TAG_ONES, 4 * (int64_t)specs[l].n);
                }
            } else {
                int has_ws = IS_C(l) && WS(l, 0) > 0;
                if (has_ws) emit(&t, ORC_EV_ALLOC, l, ORC_TAG_WS, WS(l, 0));
                emit(&t, ORC_EV_ALLOC, l, ORC_TAG_DST, dstB[l]);
                if (off[l]) { emit(&t, ORC_EV_OFFLOAD, l, ORC_TAG_SRC, srcB[l]); offB += srcB[l]; }
                if (types[l] == ORC_FC_GEMM) {
                    emit(&t, ORC_EV_ALLOC, l, ORC_TAG_ONES, 4 * (int64_t)specs[l].n);
                    emit(&t, ORC_EV_FREE, l, ORC_TAG_ONES, 4 * (int64_t)specs[l].n);
                }
                if (has_ws) emit(&t, ORC_EV_FREE, l, ORC_TAG_WS, WS(l, 0));
                if (l != 0 && off[l]) emit(&t, ORC_EV_FREE, l, ORC_TAG_SRC, srcB[l]);
            }
            emit(&t, ORC_EV_FWD_DONE, l, ORC_TAG_NONE, 0);
        }
        /* ---- backward: network.cu:1112-1191 ---- */
        if (vdnn_type != ORC_BASELINE) {
            memset(pre, 0, L);
            emit(&t, ORC_EV_ALLOC, L - 1, ORC_TAG_DIFF, srcB[L - 1]);
        }
        for (int l = L - 1; l >= 0; --l) {
            if (vdnn_type == ORC_BASELINE) {
                if (types[l] == ORC_FC_GEMM) {
                    emit(&t, ORC_EV_ALLOC, l, ORC_TAG_ONES, 4 * (int64_t)specs[l].n);
                    emit(&t, ORC_EV_FREE, l, ORC_TAG_ONES, 4 * (int64_t)specs[l].n);
                }
            } else {
                int prefId = l > 0 ? orc_find_prefetch_layer(types, off, pre, l) : -1;
                if (prefId >= 0) emit(&t, ORC_EV_ALLOC, prefId, ORC_TAG_SRC, srcB[prefId]);
                emit(&t, ORC_EV_ALLOC, l, ORC_TAG_GRAD, srcB[l]);
                if (prefId >= 0) { emit(&t, ORC_EV_PREFETCH, prefId, ORC_TAG_SRC, srcB[prefId]); preB += srcB[prefId]; }
                if (IS_C(l)) {
                    if (WS(l, 1) > 0) { emit(&t, ORC_EV_ALLOC, l, ORC_TAG_WS, WS(l, 1)); emit(&t, ORC_EV_FREE, l, ORC_TAG_WS, WS(l, 1)); }
                    if (WS(l, 2) > 0) { emit(&t, ORC_EV_ALLOC, l, ORC_TAG_WS, WS(l, 2)); emit(&t, ORC_EV_FREE, l, ORC_TAG_WS, WS(l, 2)); }
                }
                if (types[l] == ORC_FC_GEMM) {
                    emit(&t, ORC_EV_ALLOC, l, ORC_TAG_ONES, 4 * (int64_t)specs[l].n);
                    emit(&t, ORC_EV_FREE, l, ORC_TAG_ONES, 4 * (int64_t)specs[l].n);
                }
                emit(&t, ORC_EV_FREE, l, ORC_TAG_DST, dstB[l]);
                emit(&t, ORC_EV_FREE, l, ORC_TAG_DIFF, dstB[l]);
            }
            emit(&t, ORC_EV_BWD_DONE, l, ORC_TAG_NONE, 0);
        }
        if (vdnn_type != ORC_BASELINE) {
            emit(&t, ORC_EV_FREE, 0, ORC_TAG_GRAD, srcB[0]);
            /* network.cu:1185 adopts the prefetched copy of layer 0 as the new input */
            if (fix_input_leak && L > 1 && pre[0]) emit(&t, ORC_EV_FREE, -1, ORC_TAG_INPUT, srcB[0]);
        }
    }
#undef WS
#undef IS_W
#undef IS_C
    if (sum) {
        sum->peak_bytes = t.peak; sum->static_bytes = static_bytes; sum->offload_bytes = offB;
        sum->prefetch_bytes = preB; sum->pinned_bytes = pinned; sum->num_events = t.n;
    }
    free(srcB); free(dstB); free(types); free(off); free(pre);
    return t.overflow ? -1 : 0;
}
