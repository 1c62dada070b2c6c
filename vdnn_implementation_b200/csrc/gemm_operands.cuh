// Operand and output addressing shared by the contraction engines (FFMA and tcgen05).
//
// Every CONV / FC call of the training path is the contraction
//     D[i][j] = sum_kk A(i, kk) * B(j, kk)          i < M, j < N, kk < K
// over fp32 NCHW / KCRS tensors that are never re-laid-out in memory.  An operand is described by a
// "row" coordinate (decoded once per thread) and a "column" (k) coordinate.  Three access forms exist:
//   load(row, col)                  one element (FFMA engine, generic fallbacks)
//   load_run<RUN>(row, kk0, ..)     RUN consecutive k of one row   (thread-per-row producers)
//   cols4(kk0, ..) + load4(row, ..) 4 consecutive k for several rows (thread-per-k-chunk producers)
// Elements outside the tensor (padding, tile tails) read as 0.
//
//   conv forward    A = XGather rows (n,p,q)   k = (r,s,c)       B = weights  K x (r,s,c)
//   conv dgrad      A = DyGather rows (n,h,w)  k = (r,s,ko)      B = weights viewed C x (r,s,ko)
//   conv wgrad      A = dy viewed K x (n,pq)                     B = XGather rows (c,r,s) k = (n,p,q)
//   sgemm           A, B strided views of the column-major operands
// The reduction index of the two convolution products runs tap-major (filter tap outermost, channel
// innermost): a run of consecutive k then stays on one tap, so the bounds test and the address are
// computed once per run and the loads differ by a constant channel stride.  The order of a reduction
// index is free as long as both operands use the same one; the tensors themselves keep KCRS order.
#pragma once

#include "common.cuh"

namespace vdnn {

// Pixel coordinate (n, p, q) of a convolution output / filter coordinate (c, r, s).
struct PixCoord { int base; int ih0; int iw0; int valid; int q; };
struct FiltCoord { int off; int r; int s; int valid; int c; };
struct Pix4 { PixCoord first; int same_row; int count; };     // 4 consecutive pixels; count = how many are in range

// Input tensor x gathered as im2col without materialising it.
struct XGather {
    const float* x;
    int C, H, W, R, S, Q;
    int pad_h, pad_w, stride_h, stride_w;
    int n_pix, n_filt;          // N*P*Q and C*R*S
    FastDiv div_pq, div_q, div_rs, div_s, div_c;
    int chw, hw;

    __device__ __forceinline__ PixCoord pix(int m) const {
        PixCoord pc;
        uint32_t n, pq, p, q;
        div_pq.divmod(static_cast<uint32_t>(m), n, pq);
        div_q.divmod(pq, p, q);
        pc.base = static_cast<int>(n) * chw;
        pc.ih0 = static_cast<int>(p) * stride_h - pad_h;
        pc.iw0 = static_cast<int>(q) * stride_w - pad_w;
        pc.valid = m < n_pix;
        pc.q = static_cast<int>(q);
        return pc;
    }
    // filter coordinate from the KCRS position j = c*RS + r*S + s (rows of the filter gradient)
    __device__ __forceinline__ FiltCoord filt_crs(int j) const {
        FiltCoord fc;
        uint32_t c, rs, r, s;
        div_rs.divmod(static_cast<uint32_t>(j), c, rs);
        div_s.divmod(rs, r, s);
        fc.off = static_cast<int>(c) * hw;
        fc.r = static_cast<int>(r);
        fc.s = static_cast<int>(s);
        fc.c = static_cast<int>(c);
        fc.valid = j < n_filt;
        return fc;
    }
    // filter coordinate from the tap-major reduction index j = (r*S + s)*C + c
    __device__ __forceinline__ FiltCoord filt_tap(int j) const {
        FiltCoord fc;
        uint32_t tap, c, r, s;
        div_c.divmod(static_cast<uint32_t>(j), tap, c);
        div_s.divmod(tap, r, s);
        fc.off = static_cast<int>(c) * hw;
        fc.r = static_cast<int>(r);
        fc.s = static_cast<int>(s);
        fc.c = static_cast<int>(c);
        fc.valid = j < n_filt;
        return fc;
    }
    __device__ __forceinline__ float at(const PixCoord& pc, const FiltCoord& fc) const {
        const int ih = pc.ih0 + fc.r, iw = pc.iw0 + fc.s;
        const bool ok = pc.valid && fc.valid && static_cast<unsigned>(ih) < static_cast<unsigned>(H) &&
                        static_cast<unsigned>(iw) < static_cast<unsigned>(W);
        return ok ? __ldg(x + pc.base + fc.off + ih * W + iw) : 0.0f;
    }
};

// rows are pixels (forward A).  TAP = true: k = (r, s, c) tap-major, which needs the weights in a
// tap-major copy to stay coalesced (PERF_OPT packs one into workspace); TAP = false: k = (c, r, s), the
// order the KCRS weights are stored in (MEMORY_OPT: no workspace).
template <bool TAP>
struct XGatherPixRowsT {
    XGather g;
    typedef PixCoord Row;
    typedef FiltCoord Col;
    __device__ __forceinline__ Row row(int i) const { return g.pix(i); }
    __device__ __forceinline__ Col col(int kk) const { return TAP ? g.filt_tap(kk) : g.filt_crs(kk); }
    __device__ __forceinline__ float load(const Row& r, const Col& c) const { return g.at(r, c); }
    template <int RUN>
    __device__ __forceinline__ void load_run(const Row& pc, int kk0, int kend, float (&v)[RUN]) const {
        const int lim = min(kend, g.n_filt) - kk0;            // elements of the run that exist
        if (TAP) {
            const FiltCoord f = g.filt_tap(kk0);
            if (f.c + RUN <= g.C) {                           // one tap: one bounds test, constant channel stride
                const int ih = pc.ih0 + f.r, iw = pc.iw0 + f.s;
                const bool ok = pc.valid && static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) &&
                                static_cast<unsigned>(iw) < static_cast<unsigned>(g.W);
                const float* p = g.x + pc.base + f.off + ih * g.W + iw;
                if (lim >= RUN) {                                 // every k block but the last: no test per element
#pragma unroll
                    for (int e = 0; e < RUN; ++e) v[e] = ok ? __ldg(p + e * g.hw) : 0.0f;
                } else {
#pragma unroll
                    for (int e = 0; e < RUN; ++e) v[e] = (ok && e < lim) ? __ldg(p + e * g.hw) : 0.0f;
                }
            } else {
#pragma unroll
                for (int e = 0; e < RUN; ++e) v[e] = e < lim ? g.at(pc, g.filt_tap(kk0 + e)) : 0.0f;
            }
        } else {
            FiltCoord f = g.filt_crs(kk0);                    // then step (c, r, s) without dividing
#pragma unroll
            for (int e = 0; e < RUN; ++e) {
                f.valid = e < lim;                            // folded into the load's predicate: no branch per element
                v[e] = g.at(pc, f);
                if (++f.s == g.S) { f.s = 0; if (++f.r == g.R) { f.r = 0; f.off += g.hw; } }
            }
        }
    }
};
typedef XGatherPixRowsT<false> XGatherPixRows;
typedef XGatherPixRowsT<true> XGatherPixRowsTap;

struct XGatherFiltRows {           // rows are filter coordinates in KCRS order, k = pixels (wgrad B)
    XGather g;
    typedef FiltCoord Row;
    typedef PixCoord Col;
    typedef Pix4 Cols4;
    __device__ __forceinline__ Row row(int i) const { return g.filt_crs(i); }
    __device__ __forceinline__ Col col(int kk) const { return g.pix(kk); }
    __device__ __forceinline__ float load(const Row& r, const Col& c) const { return g.at(c, r); }
    __device__ __forceinline__ Cols4 cols4(int kk0, int kend) const {
        Cols4 c;
        c.first = g.pix(kk0);
        c.count = min(kend, g.n_pix) - kk0;
        c.same_row = c.first.q + 3 < g.Q;                     // the 4 pixels are neighbours in one output row
        return c;
    }
    __device__ __forceinline__ void load4(const Row& f, const Cols4& c, int kk0, float* v) const {
        if (c.same_row && c.count >= 4) {
            const int ih = c.first.ih0 + f.r, iw = c.first.iw0 + f.s;
            const bool ok = f.valid && static_cast<unsigned>(ih) < static_cast<unsigned>(g.H);
            const float* p = g.x + c.first.base + f.off + ih * g.W + iw;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int w = iw + e * g.stride_w;
                v[e] = (ok && static_cast<unsigned>(w) < static_cast<unsigned>(g.W)) ? __ldg(p + e * g.stride_w) : 0.0f;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = e < c.count ? g.at(g.pix(kk0 + e), f) : 0.0f;
        }
    }
};

// Output gradient dy gathered for the data gradient: rows are input pixels (n,h,w), k = (r, s, ko)
// tap-major; element = dy[n][ko][(h+pad-r)/stride][(w+pad-s)/stride] when that is integral and in range.
struct DyGather {
    const float* dy;
    int K, P, Q, R, S;
    int pad_h, pad_w, stride_h, stride_w;
    int n_pix, n_cols;          // N*H*W and K*R*S
    FastDiv div_hw, div_w, div_k, div_s, div_sh, div_sw;
    int kpq, pq;

    typedef PixCoord Row;
    typedef FiltCoord Col;
    __device__ __forceinline__ Row row(int m) const {
        Row pc;
        uint32_t n, hw, h, w;
        div_hw.divmod(static_cast<uint32_t>(m), n, hw);
        div_w.divmod(hw, h, w);
        pc.base = static_cast<int>(n) * kpq;
        pc.ih0 = static_cast<int>(h) + pad_h;
        pc.iw0 = static_cast<int>(w) + pad_w;
        pc.valid = m < n_pix;
        pc.q = static_cast<int>(w);
        return pc;
    }
    __device__ __forceinline__ Col col(int j) const {
        Col fc;
        uint32_t tap, k, r, s;
        div_k.divmod(static_cast<uint32_t>(j), tap, k);
        div_s.divmod(tap, r, s);
        fc.off = static_cast<int>(k) * pq;
        fc.r = static_cast<int>(r);
        fc.s = static_cast<int>(s);
        fc.c = static_cast<int>(k);
        fc.valid = j < n_cols;
        return fc;
    }
    // position inside dy of the output pixel that tap (r, s) connects to this input pixel; false if none
    __device__ __forceinline__ bool locate(const Row& pc, const Col& fc, int* pos) const {
        const int t = pc.ih0 - fc.r, u = pc.iw0 - fc.s;
        if (!pc.valid || t < 0 || u < 0) return false;
        uint32_t p, pr, q, qr;
        div_sh.divmod(static_cast<uint32_t>(t), p, pr);
        div_sw.divmod(static_cast<uint32_t>(u), q, qr);
        *pos = static_cast<int>(p) * Q + static_cast<int>(q);
        return pr == 0 && qr == 0 && static_cast<int>(p) < P && static_cast<int>(q) < Q;
    }
    __device__ __forceinline__ float load(const Row& pc, const Col& fc) const {
        int pos = 0;
        const bool ok = fc.valid && locate(pc, fc, &pos);
        return ok ? __ldg(dy + pc.base + fc.off + pos) : 0.0f;
    }
    template <int RUN>
    __device__ __forceinline__ void load_run(const Row& pc, int kk0, int kend, float (&v)[RUN]) const {
        const Col f = col(kk0);
        const int lim = min(kend, n_cols) - kk0;
        if (f.c + RUN <= K) {
            int pos = 0;
            const bool ok = locate(pc, f, &pos);
            const float* p = dy + pc.base + f.off + pos;
            if (lim >= RUN) {
#pragma unroll
                for (int e = 0; e < RUN; ++e) v[e] = ok ? __ldg(p + e * pq) : 0.0f;
            } else {
#pragma unroll
                for (int e = 0; e < RUN; ++e) v[e] = (ok && e < lim) ? __ldg(p + e * pq) : 0.0f;
            }
        } else {
#pragma unroll
            for (int e = 0; e < RUN; ++e) v[e] = e < lim ? load(pc, col(kk0 + e)) : 0.0f;
        }
    }
};

// Dense operand whose row and column indices each split once:
//   offset = (i / row_div) * row_hi + (i % row_div) * row_lo + (kk / col_div) * col_hi + (kk % col_div) * col_lo
struct SplitDense {
    const float* p;
    int rows, cols;
    FastDiv row_div, col_div;
    int row_hi, row_lo, col_hi, col_lo;

    struct Row { int off; int valid; };
    struct Col { int off; int valid; int rem; };
    struct Cols4 { int off0; int step; int count; int contiguous; };   // contiguous: the 4 k share one segment
    __device__ __forceinline__ Row row(int i) const {
        uint32_t a, b;
        row_div.divmod(static_cast<uint32_t>(i), a, b);
        Row r;
        r.off = static_cast<int>(a) * row_hi + static_cast<int>(b) * row_lo;
        r.valid = i < rows;
        return r;
    }
    __device__ __forceinline__ Col col(int kk) const {
        uint32_t a, b;
        col_div.divmod(static_cast<uint32_t>(kk), a, b);
        Col c;
        c.off = static_cast<int>(a) * col_hi + static_cast<int>(b) * col_lo;
        c.valid = kk < cols;
        c.rem = static_cast<int>(b);
        return c;
    }
    __device__ __forceinline__ float load(const Row& r, const Col& c) const {
        return (r.valid && c.valid) ? __ldg(p + r.off + c.off) : 0.0f;
    }
    template <int RUN>
    __device__ __forceinline__ void load_run(const Row& r, int kk0, int kend, float (&v)[RUN]) const {
        const Col c0 = col(kk0);
        const int lim = min(kend, cols) - kk0;
        if (c0.rem + RUN <= static_cast<int>(col_div.d)) {    // the run stays inside one column segment
            const float* q = p + r.off + c0.off;
            if (lim >= RUN) {
#pragma unroll
                for (int e = 0; e < RUN; ++e) v[e] = r.valid ? __ldg(q + e * col_lo) : 0.0f;
            } else {
#pragma unroll
                for (int e = 0; e < RUN; ++e) v[e] = (r.valid && e < lim) ? __ldg(q + e * col_lo) : 0.0f;
            }
        } else {
#pragma unroll
            for (int e = 0; e < RUN; ++e) v[e] = e < lim ? load(r, col(kk0 + e)) : 0.0f;
        }
    }
    __device__ __forceinline__ Cols4 cols4(int kk0, int kend) const {
        const Col c0 = col(kk0);
        Cols4 c;
        c.off0 = c0.off;
        c.step = col_lo;
        c.count = min(kend, cols) - kk0;
        c.contiguous = c0.rem + 4 <= static_cast<int>(col_div.d);
        return c;
    }
    __device__ __forceinline__ void load4(const Row& r, const Cols4& c, int kk0, float* v) const {
        if (c.contiguous && c.count >= 4) {
            const float* q = p + r.off + c.off0;
#ifndef VDNN_NO_VEC4
            if (c.step == 1 && (reinterpret_cast<uintptr_t>(q) & 15u) == 0) {     // one 16-byte load
                const float4 t = r.valid ? __ldg(reinterpret_cast<const float4*>(q)) : make_float4(0.f, 0.f, 0.f, 0.f);
                v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
            } else
#endif
            {
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = r.valid ? __ldg(q + e * c.step) : 0.0f;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = e < c.count ? load(r, col(kk0 + e)) : 0.0f;
        }
    }
};

inline SplitDense make_dense(const float* p, int rows, int cols, int row_stride, int col_stride) {
    SplitDense d;
    d.p = p; d.rows = rows; d.cols = cols;
    d.row_div = FastDiv(1u << 30); d.col_div = FastDiv(1u << 30);   // never splits
    d.row_hi = 0; d.row_lo = row_stride; d.col_hi = 0; d.col_lo = col_stride;
    return d;
}

// Where D[i][j] goes:  offset = (i / row_div) * row_hi + (i % row_div) * row_lo + j * col_stride.
enum EpilogueMode { EPI_DIRECT = 0, EPI_ATOMIC = 1, EPI_PARTIAL = 2 };
struct Epilogue {
    float* out;
    const float* bias;          // indexed by j; DIRECT mode only
    float alpha, beta;
    int mode;
    FastDiv row_div;
    int row_hi, row_lo, col_stride;
    size_t partial_stride;      // elements between the partial results of consecutive k splits

    __device__ __forceinline__ int row_off(int i) const {
        uint32_t a, b;
        row_div.divmod(static_cast<uint32_t>(i), a, b);
        return static_cast<int>(a) * row_hi + static_cast<int>(b) * row_lo;
    }
    __device__ __forceinline__ void store(int roff, int j, float acc, int split) const {
        const size_t o = static_cast<size_t>(roff) + static_cast<size_t>(j) * col_stride;
        if (mode == EPI_DIRECT) {
            float v = alpha * acc;
            if (bias) v += bias[j];
            if (beta != 0.0f) v = fmaf(beta, out[o], v);
            out[o] = v;
        } else if (mode == EPI_ATOMIC) {
            atomicAdd(out + o, alpha * acc);
        } else {
            out[static_cast<size_t>(split) * partial_stride + o] = acc;
        }
    }
};

}  // namespace vdnn
