// Operand and output addressing shared by the contraction engines (FFMA and tcgen05).
//
// Every CONV / FC call of the training path is the contraction
//     D[i][j] = sum_kk A(i, kk) * B(j, kk)          i < M, j < N, kk < K
// over fp32 NCHW / KCRS tensors that are never re-laid-out in memory.  An operand is described
// by a "row" coordinate (decoded once per thread) and a "column" coordinate (decoded once per
// k step); load(row, col) returns the element or 0 outside the tensor (padding, tile tails).
//
//   conv forward    A = XGather rows (n,p,q)   cols (c,r,s)      B = weights  K x CRS
//   conv dgrad      A = DyGather rows (n,h,w)  cols (k,r,s)      B = weights viewed C x (K,RS)
//   conv wgrad      A = dy viewed K x (n,pq)                     B = XGather rows (c,r,s) cols (n,p,q)
//   sgemm           A, B strided views of the column-major operands
#pragma once

#include "common.cuh"

namespace vdnn {

// Pixel coordinate (n, p, q) of a convolution output / filter coordinate (c, r, s).
struct PixCoord { int base; int ih0; int iw0; int valid; };
struct FiltCoord { int off; int r; int s; int valid; };

// Input tensor x gathered as im2col without materialising it.
struct XGather {
    const float* x;
    int C, H, W, R, S;
    int pad_h, pad_w, stride_h, stride_w;
    int n_pix, n_filt;          // N*P*Q and C*R*S
    FastDiv div_pq, div_q, div_rs, div_s;
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
        return pc;
    }
    __device__ __forceinline__ FiltCoord filt(int j) const {
        FiltCoord fc;
        uint32_t c, rs, r, s;
        div_rs.divmod(static_cast<uint32_t>(j), c, rs);
        div_s.divmod(rs, r, s);
        fc.off = static_cast<int>(c) * hw;
        fc.r = static_cast<int>(r);
        fc.s = static_cast<int>(s);
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

struct XGatherPixRows {            // rows are pixels, columns are filter taps (forward A)
    XGather g;
    typedef PixCoord Row;
    typedef FiltCoord Col;
    __device__ __forceinline__ Row row(int i) const { return g.pix(i); }
    __device__ __forceinline__ Col col(int kk) const { return g.filt(kk); }
    // column kk + 1 from column kk without a division
    __device__ __forceinline__ void next_col(Col& c, int kk_next) const {
        if (++c.s == g.S) { c.s = 0; if (++c.r == g.R) { c.r = 0; c.off += g.hw; } }
        c.valid = kk_next < g.n_filt;
    }
    __device__ __forceinline__ float load(const Row& r, const Col& c) const { return g.at(r, c); }
};

struct XGatherFiltRows {           // rows are filter taps, columns are pixels (wgrad B)
    XGather g;
    typedef FiltCoord Row;
    typedef PixCoord Col;
    __device__ __forceinline__ Row row(int i) const { return g.filt(i); }
    __device__ __forceinline__ Col col(int kk) const { return g.pix(kk); }
    __device__ __forceinline__ void next_col(Col& c, int kk_next) const { c = g.pix(kk_next); }
    __device__ __forceinline__ float load(const Row& r, const Col& c) const { return g.at(c, r); }
};

// Output gradient dy gathered for the data gradient: rows are input pixels (n,h,w), columns are
// (k, r, s); element = dy[n][k][(h+pad-r)/stride][(w+pad-s)/stride] when that is integral and in range.
struct DyGather {
    const float* dy;
    int K, P, Q, R, S;
    int pad_h, pad_w, stride_h, stride_w;
    int n_pix, n_cols;          // N*H*W and K*R*S
    FastDiv div_hw, div_w, div_rs, div_s, div_sh, div_sw;
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
        return pc;
    }
    __device__ __forceinline__ Col col(int j) const {
        Col fc;
        uint32_t k, rs, r, s;
        div_rs.divmod(static_cast<uint32_t>(j), k, rs);
        div_s.divmod(rs, r, s);
        fc.off = static_cast<int>(k) * pq;
        fc.r = static_cast<int>(r);
        fc.s = static_cast<int>(s);
        fc.valid = j < n_cols;
        return fc;
    }
    __device__ __forceinline__ void next_col(Col& c, int kk_next) const {
        if (++c.s == S) { c.s = 0; if (++c.r == R) { c.r = 0; c.off += pq; } }
        c.valid = kk_next < n_cols;
    }
    __device__ __forceinline__ float load(const Row& pc, const Col& fc) const {
        const int t = pc.ih0 - fc.r, u = pc.iw0 - fc.s;
        if (!(pc.valid && fc.valid) || t < 0 || u < 0) return 0.0f;
        uint32_t p, pr, q, qr;
        div_sh.divmod(static_cast<uint32_t>(t), p, pr);
        div_sw.divmod(static_cast<uint32_t>(u), q, qr);
        const bool ok = pr == 0 && qr == 0 && static_cast<int>(p) < P && static_cast<int>(q) < Q;
        return ok ? __ldg(dy + pc.base + fc.off + static_cast<int>(p) * Q + static_cast<int>(q)) : 0.0f;
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
    __device__ __forceinline__ void next_col(Col& c, int kk_next) const {
        if (++c.rem == static_cast<int>(col_div.d)) { c.rem = 0; c.off += col_hi - (static_cast<int>(col_div.d) - 1) * col_lo; }
        else c.off += col_lo;
        c.valid = kk_next < cols;
    }
    __device__ __forceinline__ float load(const Row& r, const Col& c) const {
        return (r.valid && c.valid) ? __ldg(p + r.off + c.off) : 0.0f;
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
