// TMA-fed convolution engines for sm_100a (PERF_OPT, stride-1 convolutions whose channel counts are multiples of 32).
//
// The gathered operands are first rewritten once, by bandwidth-bound passes, into channels-last images in workspace:
// hi = tf32(x) and lo = x - hi, fp32 containers, 32-channel blocks of 128 bytes.  The contraction kernels then spend no
// instruction on operand elements: a warp of its own issues cp.async.bulk.tensor loads that complete the stage's
// "full" barrier by byte count, one thread issues the 3xTF32 tcgen05.mma sequence of gemm_tc.cuh, and 16 warps add each
// finished accumulator buffer (two k blocks = 24 chained MMAs) into fp32 registers and run the epilogue.  In this file:
//   conv_kernel          forward / data gradient, one set of four 32-pixel boxes per filter tap (the first design; the
//                        fallback for filters wider than nine taps);
//   strip_kernel         forward / data gradient on a padded position list: one strip per filter row serves its taps
//                        through shifted descriptors; persistent CTAs; tiles of 128 x 64, 256 x 128 or 128 x 256;
//   wgrad_kernel         filter gradient, both operands MN-major, one box per (tap, channel block) row group;
//   conv_tma_pair.cuh    (included below) the 256-column cases of the last two on CTA pairs (tcgen05 cta_group::2);
//   conv_tma_wstrip.cuh  (included below) the filter gradient on two position lists, taps as 128-byte shifts of a
//                        tile's row groups;
//   the image passes (nchw_to_split_*), tensor-map construction and the launch plans.
// The box kernel in detail:
//   warp 16    one thread issues, per 32-wide k block (one filter tap, 32 channels), eight tiled
//              cp.async.bulk.tensor loads -- four 32-pixel boxes of the hi image and of the lo image, shifted by the
//              tap, zero-filled by the TMA unit outside the image (that is the padding) -- plus one cp.async.bulk for
//              the packed weight tile; all nine complete the stage's "full" barrier by byte count;
//   warp 17    allocates TMEM and issues the 3xTF32 tcgen05.mma sequence of gemm_tc.cuh on the stage;
//   warps 0-15 add each finished accumulator buffer into fp32 registers and run the epilogue (alpha / beta / bias /
//              split-K partials), as in gemm_tc.cuh.
// An output tile is 128 pixels = four boxes of bw x bh = 32 pixels of one image; the box shape is chosen per layer
// so that the boxes cover the output grid with the least overhang.  Every barrier wait is bounded.
//
// No load carries a cluster multicast qualifier, and every tensor map covers this GPU's own workspace only.
#pragma once

#include <cuda.h>

#include "gemm_tc.cuh"

namespace vdnn {
namespace tma {

using tc::A_TILE_BYTES;
using tc::BK;
using tc::BM;

constexpr int DRAIN_WARPS = 16;
constexpr int THREADS = (DRAIN_WARPS + 2) * 32;      // + the TMA warp and the MMA warp
constexpr int BOX_PIXELS = 32, BOXES = BM / BOX_PIXELS;
constexpr int BOX_BYTES = BOX_PIXELS * BK * 4;       // 4 KB: four swizzle atoms
constexpr int TR_PIX = 128;                          // pixels per block of the image transform passes

template <int BN> struct Config {
    static constexpr int B_TILE_BYTES = BN * BK * 4;
    static constexpr int STAGE_BYTES = 2 * A_TILE_BYTES + 2 * B_TILE_BYTES;
    static constexpr int STAGES = BN == 256 ? 2 : (BN == 128 ? 3 : 4);
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    static constexpr uint32_t IDESC = tc::Config<BN>::IDESC;
};

struct Params {
    // output pixel grid, covered by boxes of (1 << bw_log2) x bh pixels
    int n_img, out_h, out_w, bw_log2, bh;
    int boxes_w, total_boxes;
    FastDiv div_boxes_img, div_boxes_w;
    // reduction index k = tap * channels + channel, walked in blocks of 32 channels
    FastDiv div_cblocks, div_s;
    int tap_sign, off_h, off_w;          // image row of output row y under tap (r, s): y + tap_sign * r + off_h
    int K, k_chunk, kblocks_total;
    const char* b_tiles;                 // packed weight tiles (tc::pack_b_tiles_kernel)
    // output: NCHW tensor of n_cols channels over the output grid
    float* out;
    const float* bias;
    float alpha, beta;
    int mode, n_cols;
    size_t partial_stride;
};

// One contraction: image row of output row y under tap r is y + tap_sign * r + off_h (columns likewise).
struct Problem {
    int n, cin, in_h, in_w;        // the gathered tensor (x for forward, dy for the data gradient)
    int out_h, out_w, n_cols;      // output grid and channels
    int R, S, tap_sign, off_h, off_w;
};

__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int x, int y, int n) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(x), "r"(y), "r"(n) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
conv_kernel(const __grid_constant__ CUtensorMap map_hi, const __grid_constant__ CUtensorMap map_lo, const Params p) {
    typedef Config<BN> Cfg;
    constexpr int S = Cfg::STAGES;
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + S * Cfg::STAGE_BYTES);
    // bars[0..S) stage full, [S..2S) stage empty, [2S..2S+2) accumulator buffer ready, [2S+2..2S+4) buffer drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int n0 = blockIdx.y * BN;
    const int kbeg = blockIdx.z * p.k_chunk;
    const int kend = min(p.K, kbeg + p.k_chunk);
    const int nkb = kbeg < kend ? (kend - kbeg) / BK : 0;
    const int npairs = (nkb + 1) / 2;

    if (t == 0) {
        for (int s = 0; s < S; ++s) {
            tc::mbar_init(tc::smem_u32(&bars[s]), 1);
            tc::mbar_init(tc::smem_u32(&bars[S + s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(tc::smem_u32(&bars[2 * S + b]), 1);
            tc::mbar_init(tc::smem_u32(&bars[2 * S + 2 + b]), DRAIN_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp < DRAIN_WARPS) {
        // ------------------------------------------------------------------ accumulator drain + epilogue
        constexpr int NACC = BN / (DRAIN_WARPS / 4);
        const int col_beg = (warp >> 2) * NACC;
        const uint32_t tmem_mine = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(col_beg);
        float acc[NACC];
#pragma unroll
        for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;
        bool alive = true;
        for (int pair = 0; pair < npairs && alive; ++pair) {
            const int b = pair & 1;
            bool ok = tc::mbar_wait(tc::smem_u32(&bars[2 * S + b]), static_cast<uint32_t>(pair >> 1) & 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { atomicCAS(&tc::g_tc_error, 0, 103); alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < NACC; c += 16) {
                float v[16];
                tc::tmem_ld16(tmem_mine + static_cast<uint32_t>(b * BN + c), v);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c + j] += v[j];
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(&bars[2 * S + 2 + b]));      // this warp's part of the buffer is free again
        }
        // this thread's pixel: box (warp & 3) of the tile, pixel `lane` of the box
        const int box = blockIdx.x * BOXES + (warp & 3);
        if (alive && box < p.total_boxes) {
            uint32_t n, rem, by, bx;
            p.div_boxes_img.divmod(static_cast<uint32_t>(box), n, rem);
            p.div_boxes_w.divmod(rem, by, bx);
            const int y = static_cast<int>(by) * p.bh + (lane >> p.bw_log2);
            const int x = (static_cast<int>(bx) << p.bw_log2) + (lane & ((1 << p.bw_log2) - 1));
            if (y < p.out_h && x < p.out_w) {
                const size_t plane = static_cast<size_t>(p.out_h) * p.out_w;
                float* o = p.out + (static_cast<size_t>(n) * p.n_cols) * plane + static_cast<size_t>(y) * p.out_w + x;
                if (p.mode == EPI_PARTIAL) o += static_cast<size_t>(blockIdx.z) * p.partial_stride;
#pragma unroll
                for (int j = 0; j < NACC; ++j) {
                    const int col = n0 + col_beg + j;
                    if (col < p.n_cols) {
                        float* q = o + static_cast<size_t>(col) * plane;
                        if (p.mode == EPI_DIRECT) {
                            float v = p.alpha * acc[j];
                            if (p.bias) v += p.bias[col];
                            if (p.beta != 0.0f) v = fmaf(p.beta, *q, v);
                            *q = v;
                        } else if (p.mode == EPI_ATOMIC) {
                            atomicAdd(q, p.alpha * acc[j]);
                        } else {
                            *q = acc[j];
                        }
                    }
                }
            }
        }
    } else if (warp == DRAIN_WARPS) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int bx0[BOXES], by0[BOXES], bn[BOXES];
#pragma unroll
            for (int j = 0; j < BOXES; ++j) {
                const int box = blockIdx.x * BOXES + j;
                if (box < p.total_boxes) {
                    uint32_t n, rem, by, bx;
                    p.div_boxes_img.divmod(static_cast<uint32_t>(box), n, rem);
                    p.div_boxes_w.divmod(rem, by, bx);
                    bn[j] = static_cast<int>(n); by0[j] = static_cast<int>(by) * p.bh; bx0[j] = static_cast<int>(bx) << p.bw_log2;
                } else {
                    bn[j] = p.n_img; by0[j] = 0; bx0[j] = 0;       // past the last image: the whole box reads as zeros
                }
            }
            const char* b_src = p.b_tiles + (static_cast<size_t>(blockIdx.y) * p.kblocks_total + kbeg / BK) * (2 * Cfg::B_TILE_BYTES);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % S;
                const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
                if (!tc::mbar_wait(tc::smem_u32(&bars[S + s]), phase ^ 1u)) { atomicCAS(&tc::g_tc_error, 0, 101); break; }
                uint32_t tap, cb, r, sx;
                p.div_cblocks.divmod(static_cast<uint32_t>(kbeg / BK + i), tap, cb);
                p.div_s.divmod(tap, r, sx);
                const int dy = p.tap_sign * static_cast<int>(r) + p.off_h, dx = p.tap_sign * static_cast<int>(sx) + p.off_w;
                const uint32_t bar = tc::smem_u32(&bars[s]);
                const uint32_t st = tc::smem_u32(tiles + s * Cfg::STAGE_BYTES);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(Cfg::STAGE_BYTES) : "memory");
#pragma unroll
                for (int j = 0; j < BOXES; ++j) {
                    tma_load_box(st + j * BOX_BYTES, &map_hi, bar, static_cast<int>(cb) * BK, bx0[j] + dx, by0[j] + dy, bn[j]);
                    tma_load_box(st + A_TILE_BYTES + j * BOX_BYTES, &map_lo, bar, static_cast<int>(cb) * BK, bx0[j] + dx, by0[j] + dy, bn[j]);
                }
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(st + 2 * A_TILE_BYTES), "l"(b_src + static_cast<size_t>(i) * (2 * Cfg::B_TILE_BYTES)),
                               "r"(2 * Cfg::B_TILE_BYTES), "r"(bar) : "memory");
            }
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        for (int i = 0; i < nkb; ++i) {
            const int s = i % S, pair = i >> 1, b = pair & 1;
            const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
            // pairs p and p - 2 share an accumulator buffer: the drain warps must have emptied it
            if (!(i & 1) && pair >= 2 &&
                !tc::mbar_wait(tc::smem_u32(&bars[2 * S + 2 + b]), static_cast<uint32_t>((pair >> 1) - 1) & 1u)) {
                atomicCAS(&tc::g_tc_error, 0, 102);
                break;
            }
            if (!tc::mbar_wait(tc::smem_u32(&bars[s]), phase)) { atomicCAS(&tc::g_tc_error, 0, 102); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = tc::smem_u32(tiles + s * Cfg::STAGE_BYTES);
            const uint32_t a_lo = a_hi + A_TILE_BYTES;
            const uint32_t b_hi = a_hi + 2 * A_TILE_BYTES;
            const uint32_t b_lo = b_hi + Cfg::B_TILE_BYTES;
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(b * BN);
            tc::mma_block_3xtf32(d_tmem, tc::make_desc(a_hi), tc::make_desc(a_lo), tc::make_desc(b_hi), tc::make_desc(b_lo), Cfg::IDESC, !(i & 1));
            tc::mma_commit(tc::smem_u32(&bars[S + s]));
            if ((i & 1) || i == nkb - 1) tc::mma_commit(tc::smem_u32(&bars[2 * S + b]));
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Strip engine: the same contraction with every operand row fetched once per filter row instead of once per tap.
//
// The gathered tensor is laid out as ONE long list of pixel positions: image after image, row after row, each row
// followed by `gap_w` zero pixels and each image by `gap_h` zero rows, wide enough that a tap's shift never reaches
// real data of a neighbouring row or image (the zeros are the padding).  Position q of the list holds 32-channel
// blocks of 128 bytes, so a filter tap is a constant shift of the position: the operand tile of tap (r, s) for the 128
// output positions m0 .. m0 + 127 is rows  m0 + dh(r) * Wp + dw(s) ...  of the list, and the tiles of the S taps of
// one filter row are windows, one row apart, of a single strip of 128 + S - 1 rows.  The TMA unit fetches that strip
// once (two copies: hi and lo image); the MMA reads tap s through a shared-memory descriptor whose start address is s
// rows into the strip.  (Measured on B200: the tensor core derives the 128-byte swizzle phase of every operand row from
// the row's shared-memory address, so a window that starts inside a swizzle period needs nothing but its start
// address; putting the phase into the descriptor's base-offset field as well gives wrong operands.)
// Shared-memory fill per k block drops from 32 KB to about 11 KB for the gathered operand; the packed weight tiles
// (their own, deeper ring) are fetched as before.  Output tiles are 128 consecutive positions; results at gap
// positions are computed and dropped.
struct StripParams {
    int n_img, img_h, img_w;             // gathered tensor: images, rows, columns
    int wp, lp;                          // padded row length and positions per image: lp = (img_h + gap_h) * wp
    long long total_pos;                 // n_img * lp
    FastDiv div_lp, div_wp;
    int out_h, out_w, n_cols;            // output grid (inside the padded geometry) and channels
    int R, S, cblocks;                   // taps and 32-channel blocks of the reduction
    int dh0, dh_step, row0, row_step;    // tap (r, s): strip starts dh0 + dh_step * r rows of wp above/below, tap window at row row0 + row_step * s
    int dw_min;                          // column shift of the strip's first row
    int groups_total, group_chunk;       // groups = (r, channel block); each split walks group_chunk of them
    int inner;                           // taps served by one strip: S, or 1 (one strip per tap: groups = (tap, channel block))
    int use_base_offset;                 // descriptors of shifted windows carry the swizzle phase in their base-offset field
    int kblocks_total;
    const char* b_tiles;
    float* out;
    const float* bias;
    float alpha, beta;
    int mode;
    size_t partial_stride;
};

constexpr int STRIP_MAX_TAPS = 9;                                  // taps per filter row the strip buffer has room for
constexpr int STRIP_HALF_BYTES = (BM + 8) * BK * 4;                // 136 rows of 128 bytes, a multiple of the swizzle period

// MH = 128-row halves of an output tile.  The packed weight tile of a k block (BN * 256 bytes) costs three times the
// shared-memory fill of a 128-row strip's share of it (~11 KB), and the SM's ingest rate is what bounds these kernels, so
// a tile of 256 positions x 128 columns (two MMAs per k slice sharing the weight operand) moves a third fewer bytes per
// flop than 128 x 256: MH = 2 wherever the tensor memory holds the four accumulators (BN <= 128).
template <int BN, int MH> struct StripConfig {
    static_assert(MH == 1 || (MH == 2 && BN <= 128), "two row halves need 4 * BN <= 512 columns of tensor memory");
    static constexpr int B_TILE_BYTES = BN * BK * 4;
    static constexpr int A_STAGE_BYTES = MH * 2 * STRIP_HALF_BYTES;
    static constexpr int B_STAGE_BYTES = 2 * B_TILE_BYTES;
    // MERGED (64-column tiles): the hi and the lo weight tile lie back to back, so ONE MMA of 2 * BN columns forms
    // a_hi * b_hi and a_hi * b_lo side by side, and a second one of BN columns adds a_lo * b_hi to the first half: two
    // instructions per k slice instead of three, and the A operand is read from shared memory twice instead of three
    // times -- what bounds the 64-column kernels is the tensor core's operand reads and the one issuing thread.  The
    // accumulator is 2 * BN columns wide; the drain adds the halves.
    static constexpr bool MERGED = (BN == 64 && MH == 1);
    static constexpr int ACC_COLS = MERGED ? 2 * BN : BN;
    static constexpr int TMEM_COLS = 2 * MH * ACC_COLS;
    // Ring depths.  A strip is in use for S k blocks, i.e. S * 6 * BN clocks of MMA work, and its refill (a TMA box of
    // ~130 rows gathered from rows C * 4 bytes apart) takes a few thousand clocks to land: narrow tiles need more strips
    // in flight than wide ones.  Measured with two strips: 256 columns 77 % tensor-pipe activity (bound by the SM's ingest
    // rate), 128 columns 54 %, 64 columns 47 % (both waiting for strips).
    // (Measured, 128-row tiles: deeper strip rings or L2 prefetches of the next tile's strips did not help; two CTAs per
    // SM for 64-column tiles did, because one thread issues a tile's MMAs and 12 per 384 clocks of tensor work is about
    // its limit.)
    static constexpr int SA = 2;
    static constexpr int SB = MH == 2 ? (BN == 128 ? 2 : 4) : (BN == 256 ? 2 : (BN == 128 ? 4 : 2));
    static constexpr int CTAS_PER_SM = (MH == 1 && BN == 64) ? 2 : 1;
    static constexpr int SMEM_BYTES = SA * A_STAGE_BYTES + SB * B_STAGE_BYTES + 1024 + 256;
    static constexpr uint32_t IDESC = tc::Config<BN>::IDESC;
    static constexpr uint32_t IDESC_WIDE = tc::Config<2 * BN <= 256 ? 2 * BN : 256>::IDESC;
};

// One 32-wide k block with the hi and lo tiles of B taken as one operand of twice the columns (StripConfig::MERGED):
// d[:, 0:BN] = a_hi * b_hi + a_lo * b_hi, d[:, BN:2BN] = a_hi * b_lo.  dbh is the descriptor of the hi tile; the lo tile
// follows it in shared memory.
__device__ __forceinline__ void mma_block_merged(uint32_t d_tmem, uint64_t dah, uint64_t dal, uint64_t dbh, uint32_t idesc, uint32_t idesc_wide,
                                                 bool fresh) {
    tc::mma_tf32(d_tmem, dah, dbh, idesc_wide, fresh ? 0u : 1u);
    tc::mma_tf32_acc(d_tmem, dal, dbh, idesc);
#pragma unroll
    for (int ks = 1; ks < BK / 8; ++ks) {
        dah += 2; dal += 2; dbh += 2;
        tc::mma_tf32_acc(d_tmem, dah, dbh, idesc_wide);
        tc::mma_tf32_acc(d_tmem, dal, dbh, idesc);
    }
}

// The same descriptor with the row's position inside the 1024-byte swizzle period, (address >> 7) & 7, in the
// base-offset field (bits 49-51).  Kept for the diagnostic mode only: see the note on the strip engine above.
__device__ __forceinline__ uint64_t make_desc_at(uint32_t saddr) {
    return tc::make_desc(saddr) | (static_cast<uint64_t>((saddr >> 7) & 7u) << 49);
}

__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int row) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(row) : "memory");
}

template <int BN, int MH>
__global__ void __launch_bounds__(THREADS, StripConfig<BN, MH>::CTAS_PER_SM)
strip_kernel(const __grid_constant__ CUtensorMap map_hi, const __grid_constant__ CUtensorMap map_lo, const StripParams p) {
    typedef StripConfig<BN, MH> Cfg;
    constexpr int SA = Cfg::SA, SB = Cfg::SB;
    constexpr int TILE_ROWS = BM * MH;
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    char* b_ring = tiles + SA * Cfg::A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(b_ring + SB * Cfg::B_STAGE_BYTES);
    uint64_t* a_full = bars;               // [SA]
    uint64_t* a_empty = a_full + SA;       // [SA]
    uint64_t* b_full = a_empty + SA;       // [SB]
    uint64_t* b_empty = b_full + SB;       // [SB]
    uint64_t* acc_ready = b_empty + SB;    // [2]
    uint64_t* acc_free = acc_ready + 2;    // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);

    // The CTA is persistent along x: it walks output tiles blockIdx.x, blockIdx.x + gridDim.x, ... of its column tile
    // (blockIdx.y) and reduction split (blockIdx.z).  The three roles loop over the tiles independently and keep their
    // ring / accumulator counters running, so the loads of the next tile are in flight, and its first MMAs issued, while
    // the previous tile's results are still being stored: barrier set-up, TMEM allocation and the pipeline fill are paid
    // once per CTA, not once per tile.
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int n0 = blockIdx.y * BN;
    const long long num_tiles = (p.total_pos + TILE_ROWS - 1) / TILE_ROWS;
    const int g_beg = blockIdx.z * p.group_chunk;
    const int g_end = min(p.groups_total, g_beg + p.group_chunk);
    const int ngroups = g_beg < g_end ? g_end - g_beg : 0;
    const int nkb = ngroups * p.inner;                 // k blocks per tile
    const int npairs = (nkb + 1) / 2;                  // accumulator hand-overs per tile
    const uint32_t strip_bytes = static_cast<uint32_t>(BM + p.inner - 1) * BK * 4;

    if (t == 0) {
        for (int s = 0; s < SA; ++s) { tc::mbar_init(tc::smem_u32(&a_full[s]), 1); tc::mbar_init(tc::smem_u32(&a_empty[s]), 1); }
        for (int s = 0; s < SB; ++s) { tc::mbar_init(tc::smem_u32(&b_full[s]), 1); tc::mbar_init(tc::smem_u32(&b_empty[s]), 1); }
        for (int b = 0; b < 2; ++b) { tc::mbar_init(tc::smem_u32(&acc_ready[b]), 1); tc::mbar_init(tc::smem_u32(&acc_free[b]), DRAIN_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp < DRAIN_WARPS) {
        // ------------------------------------------------------------------ accumulator drain + epilogue
        constexpr int NACC = BN / (DRAIN_WARPS / 4);
        const int col_beg = (warp >> 2) * NACC;
        const uint32_t tmem_mine = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(col_beg);
        const size_t plane = static_cast<size_t>(p.out_h) * p.out_w;
        bool alive = true;
        unsigned pair = 0;                                  // running count of accumulator hand-overs
        for (long long tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
            float acc[MH][NACC];
#pragma unroll
            for (int h = 0; h < MH; ++h)
#pragma unroll
                for (int j = 0; j < NACC; ++j) acc[h][j] = 0.0f;
            for (int pp = 0; pp < npairs && alive; ++pp, ++pair) {
                const int b = pair & 1;
                bool ok = tc::mbar_wait(tc::smem_u32(&acc_ready[b]), (pair >> 1) & 1u);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { atomicCAS(&tc::g_tc_error, 0, 103); alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int h = 0; h < MH; ++h)
#pragma unroll
                    for (int c = 0; c < NACC; c += 16) {
                        float v[16];
                        tc::tmem_ld16(tmem_mine + static_cast<uint32_t>((b * MH + h) * Cfg::ACC_COLS + c), v);
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[h][c + j] += v[j];
                        if (Cfg::MERGED) {      // the a_hi * b_lo half of the accumulator
                            tc::tmem_ld16(tmem_mine + static_cast<uint32_t>((b * MH + h) * Cfg::ACC_COLS + BN + c), v);
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[h][c + j] += v[j];
                        }
                    }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(tc::smem_u32(&acc_free[b]));
            }
#pragma unroll
            for (int h = 0; h < MH; ++h) {
                const long long q = tile * TILE_ROWS + h * BM + (warp & 3) * 32 + lane;      // this thread's position in the padded list
                if (!alive || q >= p.total_pos) continue;
                const uint32_t n = static_cast<uint32_t>(q / p.lp), rem = static_cast<uint32_t>(q - static_cast<long long>(n) * p.lp);
                uint32_t y, x;
                p.div_wp.divmod(rem, y, x);
                if (static_cast<int>(y) >= p.out_h || static_cast<int>(x) >= p.out_w) continue;
                float* o = p.out + (static_cast<size_t>(n) * p.n_cols) * plane + static_cast<size_t>(y) * p.out_w + x;
                if (p.mode == EPI_PARTIAL) o += static_cast<size_t>(blockIdx.z) * p.partial_stride;
#pragma unroll
                for (int j = 0; j < NACC; ++j) {
                    const int col = n0 + col_beg + j;
                    if (col < p.n_cols) {
                        float* dst = o + static_cast<size_t>(col) * plane;
                        if (p.mode == EPI_DIRECT) {
                            float v = p.alpha * acc[h][j];
                            if (p.bias) v += p.bias[col];
                            if (p.beta != 0.0f) v = fmaf(p.beta, *dst, v);
                            *dst = v;
                        } else if (p.mode == EPI_ATOMIC) {
                            atomicAdd(dst, p.alpha * acc[h][j]);
                        } else {
                            *dst = acc[h][j];
                        }
                    }
                }
            }
        }
    } else if (warp == DRAIN_WARPS) {
        // ------------------------------------------------------------------ TMA producer: strips and weight tiles
        if (lane == 0) {
            const char* b_col = p.b_tiles + static_cast<size_t>(blockIdx.y) * p.kblocks_total * Cfg::B_STAGE_BYTES;
            unsigned i = 0, gcount = 0;                     // running k-block and strip counts (ring positions)
            bool ok = true;
            for (long long tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const long long m0 = tile * TILE_ROWS;
                for (int g = 0; g < ngroups && ok; ++g, ++gcount) {
                    const int group = g_beg + g;
                    const int outer = group / p.cblocks, cb = group - outer * p.cblocks;
                    const int r = p.inner == 1 ? outer / p.S : outer, s_first = p.inner == 1 ? outer - r * p.S : 0;
                    const int sa = gcount % SA;
                    if (!tc::mbar_wait(tc::smem_u32(&a_empty[sa]), ((gcount / SA) & 1u) ^ 1u)) { ok = false; break; }
                    // first row of the strip: position m0 shifted by the filter row and by the leftmost tap (or, with
                    // one strip per tap, by that tap)
                    const long long row = m0 + static_cast<long long>(p.dh0 + p.dh_step * r) * p.wp + p.dw_min +
                                          (p.inner == 1 ? p.row0 + p.row_step * s_first : 0);
                    const uint32_t abar = tc::smem_u32(&a_full[sa]);
                    const uint32_t ast = tc::smem_u32(tiles + sa * Cfg::A_STAGE_BYTES);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(abar), "r"(MH * 2u * strip_bytes) : "memory");
#pragma unroll
                    for (int h = 0; h < MH; ++h) {      // one strip pair (hi, lo) per 128-row half of the tile
                        tma_load_rows(ast + h * 2 * STRIP_HALF_BYTES, &map_hi, abar, cb * BK, static_cast<int>(row) + h * BM);
                        tma_load_rows(ast + h * 2 * STRIP_HALF_BYTES + STRIP_HALF_BYTES, &map_lo, abar, cb * BK, static_cast<int>(row) + h * BM);
                    }
                    for (int sx = 0; sx < p.inner; ++sx, ++i) {
                        const int sb = i % SB;
                        if (!tc::mbar_wait(tc::smem_u32(&b_empty[sb]), ((i / SB) & 1u) ^ 1u)) { ok = false; break; }
                        const int kb = (r * p.S + s_first + sx) * p.cblocks + cb;
                        const uint32_t bbar = tc::smem_u32(&b_full[sb]);
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bbar), "r"(Cfg::B_STAGE_BYTES) : "memory");
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(tc::smem_u32(b_ring + sb * Cfg::B_STAGE_BYTES)), "l"(b_col + static_cast<size_t>(kb) * Cfg::B_STAGE_BYTES),
                                       "r"(Cfg::B_STAGE_BYTES), "r"(bbar) : "memory");
                    }
                }
            }
            if (!ok) atomicCAS(&tc::g_tc_error, 0, 101);
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        unsigned i = 0, gcount = 0, pair = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int kb_in_tile = 0;
            for (int g = 0; g < ngroups && ok; ++g, ++gcount) {
                const int sa = gcount % SA;
                if (!tc::mbar_wait(tc::smem_u32(&a_full[sa]), (gcount / SA) & 1u)) { ok = false; break; }
                const uint32_t a_hi0 = tc::smem_u32(tiles + sa * Cfg::A_STAGE_BYTES);
                for (int sx = 0; sx < p.inner; ++sx, ++i, ++kb_in_tile) {
                    const int sb = i % SB, b = pair & 1;
                    const bool first_of_pair = !(kb_in_tile & 1);
                    // hand-overs `pair` and `pair - 2` share an accumulator buffer: the drain warps must have emptied it
                    if (first_of_pair && pair >= 2 && !tc::mbar_wait(tc::smem_u32(&acc_free[b]), ((pair >> 1) - 1) & 1u)) { ok = false; break; }
                    if (!tc::mbar_wait(tc::smem_u32(&b_full[sb]), (i / SB) & 1u)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_hi = a_hi0 + (p.inner == 1 ? 0u : static_cast<uint32_t>(p.row0 + p.row_step * sx) * (BK * 4));
                    const uint32_t a_lo = a_hi + STRIP_HALF_BYTES;
                    const uint32_t b_hi = tc::smem_u32(b_ring + sb * Cfg::B_STAGE_BYTES);
                    const uint32_t b_lo = b_hi + Cfg::B_TILE_BYTES;
                    const uint64_t dbh = tc::make_desc(b_hi), dbl = tc::make_desc(b_lo);
#pragma unroll
                    for (int h = 0; h < MH; ++h) {      // the row halves share the weight operand
                        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>((b * MH + h) * Cfg::ACC_COLS);
                        const uint32_t ah = a_hi + h * 2 * STRIP_HALF_BYTES, al = a_lo + h * 2 * STRIP_HALF_BYTES;
                        if (Cfg::MERGED)
                            mma_block_merged(d_tmem, tc::make_desc(ah), tc::make_desc(al), dbh, Cfg::IDESC, Cfg::IDESC_WIDE, first_of_pair);
                        else if (p.use_base_offset)      // diagnostic mode only
                            tc::mma_block_3xtf32(d_tmem, make_desc_at(ah), make_desc_at(al), dbh, dbl, Cfg::IDESC, first_of_pair);
                        else
                            tc::mma_block_3xtf32(d_tmem, tc::make_desc(ah), tc::make_desc(al), dbh, dbl, Cfg::IDESC, first_of_pair);
                    }
                    tc::mma_commit(tc::smem_u32(&b_empty[sb]));
                    if (sx == p.inner - 1) tc::mma_commit(tc::smem_u32(&a_empty[sa]));
                    if (!first_of_pair || kb_in_tile == nkb - 1) { tc::mma_commit(tc::smem_u32(&acc_ready[b])); ++pair; }
                }
            }
        }
        if (!ok) atomicCAS(&tc::g_tc_error, 0, 102);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
    }
}

// NCHW fp32 -> the padded position list of the strip engine, as two images (tf32 hi, lo): position q of image n is
// (row q / wp, column q % wp); rows >= h and columns >= w are the zero gaps.  A block takes `tiles_per_block` consecutive
// tiles of 32 channels x 128 PIXELS of one image (reads in full, aligned 128-byte lines along the pixels of a channel),
// written to the pixels' positions (one 128-byte line per pixel and image half); the thread that writes the last pixel
// of an image row also zeroes the gap columns behind it, and the first block of every (image, channel block) zeroes the
// gap rows.  SUMS: also adds scale * (per-channel sums of the block's pixels) into sums[channel] (see
// nchw_to_split_nhwc_kernel).
template <bool SUMS>
__global__ void __launch_bounds__(256) nchw_to_split_strip_kernel(const float* __restrict__ x, float* __restrict__ hi,
                                                                  float* __restrict__ lo, int C, int H, int W, int wp, int lp,
                                                                  int tiles_per_block, float* __restrict__ sums, float scale) {
    __shared__ float tile[32][TR_PIX + 1];
    const int n = blockIdx.z, c0 = blockIdx.y * 32;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int HW = H * W;
    const int quad = t & 7;                     // channels 4 * quad .. + 3
    const size_t base = static_cast<size_t>(n) * lp * C + c0 + quad * 4;
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int it = 0; it < tiles_per_block; ++it) {
        const int p0 = (blockIdx.x * tiles_per_block + it) * TR_PIX;
        if (p0 >= HW) break;
        if (it) __syncthreads();                // the tile of the last round has been written out
        const int npix = min(TR_PIX, HW - p0);
        const float* src = x + (static_cast<size_t>(n) * C + c0) * HW + p0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = warp * 4 + j;
#pragma unroll
            for (int q = 0; q < TR_PIX / 32; ++q) {
                const int pix = q * 32 + lane;
                const float v = pix < npix ? __ldg(src + static_cast<size_t>(c) * HW + pix) : 0.0f;
                tile[c][pix] = v;
                if (SUMS) part[j] += v;
            }
        }
        __syncthreads();
#pragma unroll
        for (int pass = 0; pass < TR_PIX / 32; ++pass) {
            const int pix = pass * 32 + (t >> 3);
            if (pix < npix) {
                const int pidx = p0 + pix, row = pidx / W, col = pidx - row * W;
                const size_t q = static_cast<size_t>(row) * wp + col;
                float4 h, l;
                tc::split_tf32_safe(tile[quad * 4 + 0][pix], h.x, l.x);
                tc::split_tf32_safe(tile[quad * 4 + 1][pix], h.y, l.y);
                tc::split_tf32_safe(tile[quad * 4 + 2][pix], h.z, l.z);
                tc::split_tf32_safe(tile[quad * 4 + 3][pix], h.w, l.w);
                *reinterpret_cast<float4*>(hi + base + q * C) = h;
                *reinterpret_cast<float4*>(lo + base + q * C) = l;
                if (col == W - 1)
                    for (int g = 1; g <= wp - W; ++g) {
                        *reinterpret_cast<float4*>(hi + base + (q + g) * C) = zero;
                        *reinterpret_cast<float4*>(lo + base + (q + g) * C) = zero;
                    }
            }
        }
    }
    if (blockIdx.x == 0)
        for (int q = H * wp + (t >> 3); q < lp; q += 32) {
            *reinterpret_cast<float4*>(hi + base + static_cast<size_t>(q) * C) = zero;
            *reinterpret_cast<float4*>(lo + base + static_cast<size_t>(q) * C) = zero;
        }
    if (SUMS) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v = part[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) atomicAdd(sums + c0 + warp * 4 + j, scale * v);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Filter gradient on the same images:  dw[k][c][r][s] = sum over pixels of x[pixel + tap][c] * dy[pixel][k].
// The reduction runs over pixels, and in channels-last images the channels are the contiguous direction, so both
// operands are "MN-major" for the tensor core: a box of 32 pixels x 32 channels, as the TMA unit drops it (one pixel
// per 128-byte row, 128-byte swizzle), is four 8-pixel k slices of a 32-wide strip of rows (x) or columns (dy).
//   rows     128 per tile = four "row groups" of 32 channels; row group g = tap * (C / 32) + channel block, so layers
//            with few channels fill the tile with several taps (each group is fetched with its own tap shift);
//   columns  up to 256 filters = up to eight boxes of the dy image, unshifted, shared by the four row groups;
//   k        boxes of bw x bh = 32 pixels of one image; the reduction over all boxes is split across blockIdx.z.
// (The images are the ones forward and data gradient use; only the swizzle the TMA unit applies on the way into
// shared memory differs, see make_desc_mn.)
struct WgradParams {
    int n_img, bw_log2, bh, boxes_w, total_boxes, box_chunk;
    FastDiv div_boxes_img, div_boxes_w;
    int row_groups, cblocks, taps_s;         // row_groups = R * S * cblocks
    int off_h, off_w;                        // image row of grid row y under tap r: y + r + off_h
    int C, taps, n_cols;                     // dw is [n_cols][C][taps]
    float* out;
    float alpha, beta;
    int mode;
    size_t partial_stride;
};

// Shared-memory descriptor of an MN-major tf32 operand made of 32-wide strips.  32-bit operands can only be read
// MN-major in the "128-byte swizzle with 32-byte atoms" layout: rows of 128 bytes (one pixel, 32 channels) whose
// 32-byte quarters are XORed with the row number modulo 4, the pattern repeating every 4 rows (512 bytes); the TMA
// unit writes exactly that with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.  One MMA takes 8 pixels = two such groups, 512
// bytes apart (stride dimension); strips of 32 rows / columns (one TMA box each) follow each other at BOX_BYTES
// (leading dimension).  Descriptor version 1, layout type 1.
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(BOX_BYTES >> 4) << 16;
    d |= static_cast<uint64_t>(512 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(1) << 61;
    return d;
}

// MH = 128-row halves of a tile (MH * four row groups).  A tile's dy slice (BN * 256 bytes per k block) is fetched once
// for all its rows, and the SM's ingest rate is what bounds the narrow tiles: with 128 or 64 filters a CTA takes two
// halves (a quarter / a sixth fewer bytes per flop); with 256 filters the tensor memory holds one (2 * MH * BN <= 512).
template <int BN, int MH> struct WgradConfig {
    static_assert(MH == 1 || (MH == 2 && BN <= 128), "two row halves need 4 * BN <= 512 columns of tensor memory");
    static constexpr int B_TILE_BYTES = BN * BK * 4;
    static constexpr int A_BYTES = MH * 2 * A_TILE_BYTES;                 // hi and lo of every half
    static constexpr int STAGE_BYTES = A_BYTES + 2 * B_TILE_BYTES;
    static constexpr int STAGES = MH == 2 ? 2 : (BN == 256 ? 2 : (BN == 128 ? 3 : 4));
    static constexpr int TMEM_COLS = 2 * MH * BN;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    static constexpr uint32_t IDESC = tc::Config<BN>::IDESC;
};

template <int BN, int MH>
__global__ void __launch_bounds__(THREADS, 1)
wgrad_kernel(const __grid_constant__ CUtensorMap x_hi, const __grid_constant__ CUtensorMap x_lo,
             const __grid_constant__ CUtensorMap dy_hi, const __grid_constant__ CUtensorMap dy_lo, const WgradParams p) {
    typedef WgradConfig<BN, MH> Cfg;
    constexpr int S = Cfg::STAGES;
    constexpr int GROUPS = MH * BOXES;                                       // row groups of a tile
    constexpr uint32_t IDESC_MN = Cfg::IDESC | (1u << 15) | (1u << 16);      // both operands MN-major
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + S * Cfg::STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int n0 = blockIdx.y * BN;
    const int box_beg = blockIdx.z * p.box_chunk;
    const int box_end = min(p.total_boxes, box_beg + p.box_chunk);
    const int nkb = box_beg < box_end ? box_end - box_beg : 0;
    const int npairs = (nkb + 1) / 2;

    if (t == 0) {
        for (int s = 0; s < S; ++s) {
            tc::mbar_init(tc::smem_u32(&bars[s]), 1);
            tc::mbar_init(tc::smem_u32(&bars[S + s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(tc::smem_u32(&bars[2 * S + b]), 1);
            tc::mbar_init(tc::smem_u32(&bars[2 * S + 2 + b]), DRAIN_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp < DRAIN_WARPS) {
        constexpr int NACC = BN / (DRAIN_WARPS / 4);
        const int col_beg = (warp >> 2) * NACC;
        const uint32_t tmem_mine = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(col_beg);
        float acc[MH][NACC];
#pragma unroll
        for (int h = 0; h < MH; ++h)
#pragma unroll
            for (int j = 0; j < NACC; ++j) acc[h][j] = 0.0f;
        bool alive = true;
        for (int pair = 0; pair < npairs && alive; ++pair) {
            const int b = pair & 1;
            bool ok = tc::mbar_wait(tc::smem_u32(&bars[2 * S + b]), static_cast<uint32_t>(pair >> 1) & 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { atomicCAS(&tc::g_tc_error, 0, 103); alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < MH; ++h)
#pragma unroll
                for (int c = 0; c < NACC; c += 16) {
                    float v[16];
                    tc::tmem_ld16(tmem_mine + static_cast<uint32_t>((b * MH + h) * BN + c), v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[h][c + j] += v[j];
                }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(&bars[2 * S + 2 + b]));
        }
        // this thread's rows: row group (warp & 3) of every half of the tile, channel `lane` of its block
#pragma unroll
        for (int h = 0; h < MH; ++h) {
            const int group = (blockIdx.x * MH + h) * BOXES + (warp & 3);
            if (!alive || group >= p.row_groups) continue;
            const int tap = group / p.cblocks, cb = group - tap * p.cblocks;
            const size_t crs = static_cast<size_t>(p.C) * p.taps;
            float* o = p.out + static_cast<size_t>(cb * 32 + lane) * p.taps + tap;
            if (p.mode == EPI_PARTIAL) o += static_cast<size_t>(blockIdx.z) * p.partial_stride;
#pragma unroll
            for (int j = 0; j < NACC; ++j) {
                const int col = n0 + col_beg + j;
                if (col < p.n_cols) {
                    float* q = o + static_cast<size_t>(col) * crs;
                    if (p.mode == EPI_DIRECT) {
                        float v = p.alpha * acc[h][j];
                        if (p.beta != 0.0f) v = fmaf(p.beta, *q, v);
                        *q = v;
                    } else if (p.mode == EPI_ATOMIC) {
                        atomicAdd(q, p.alpha * acc[h][j]);
                    } else {
                        *q = acc[h][j];
                    }
                }
            }
        }
    } else if (warp == DRAIN_WARPS) {
        if (lane == 0) {
            int gc[GROUPS], gdy[GROUPS], gdx[GROUPS];
            int groups = 0;
#pragma unroll
            for (int j = 0; j < GROUPS; ++j) {
                const int group = blockIdx.x * GROUPS + j;
                if (group < p.row_groups) {
                    const int tap = group / p.cblocks, cb = group - tap * p.cblocks;
                    const int r = tap / p.taps_s, sx = tap - r * p.taps_s;
                    gc[j] = cb * 32; gdy[j] = r + p.off_h; gdx[j] = sx + p.off_w;
                    groups = j + 1;
                } else {
                    gc[j] = 0; gdy[j] = 0; gdx[j] = 0;
                }
            }
            const int col_boxes = min(BN, p.n_cols - n0) / 32;
            const uint32_t stage_tx = static_cast<uint32_t>(2 * (groups + col_boxes) * BOX_BYTES);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % S;
                const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
                if (!tc::mbar_wait(tc::smem_u32(&bars[S + s]), phase ^ 1u)) { atomicCAS(&tc::g_tc_error, 0, 101); break; }
                uint32_t n, rem, by, bx;
                p.div_boxes_img.divmod(static_cast<uint32_t>(box_beg + i), n, rem);
                p.div_boxes_w.divmod(rem, by, bx);
                const int y0 = static_cast<int>(by) * p.bh, x0 = static_cast<int>(bx) << p.bw_log2;
                const uint32_t bar = tc::smem_u32(&bars[s]);
                const uint32_t st = tc::smem_u32(tiles + s * Cfg::STAGE_BYTES);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(stage_tx) : "memory");
#pragma unroll
                for (int j = 0; j < GROUPS; ++j) {
                    if (j < groups) {
                        // half j / BOXES: [hi tile][lo tile], group j % BOXES inside each
                        const uint32_t a = st + (j / BOXES) * 2 * A_TILE_BYTES + (j % BOXES) * BOX_BYTES;
                        tma_load_box(a, &x_hi, bar, gc[j], x0 + gdx[j], y0 + gdy[j], static_cast<int>(n));
                        tma_load_box(a + A_TILE_BYTES, &x_lo, bar, gc[j], x0 + gdx[j], y0 + gdy[j], static_cast<int>(n));
                    }
                }
                for (int j = 0; j < col_boxes; ++j) {
                    tma_load_box(st + Cfg::A_BYTES + j * BOX_BYTES, &dy_hi, bar, n0 + j * 32, x0, y0, static_cast<int>(n));
                    tma_load_box(st + Cfg::A_BYTES + Cfg::B_TILE_BYTES + j * BOX_BYTES, &dy_lo, bar, n0 + j * 32, x0, y0, static_cast<int>(n));
                }
            }
        }
    } else if (lane == 0) {
        for (int i = 0; i < nkb; ++i) {
            const int s = i % S, pair = i >> 1, b = pair & 1;
            const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
            if (!(i & 1) && pair >= 2 &&
                !tc::mbar_wait(tc::smem_u32(&bars[2 * S + 2 + b]), static_cast<uint32_t>((pair >> 1) - 1) & 1u)) {
                atomicCAS(&tc::g_tc_error, 0, 102);
                break;
            }
            if (!tc::mbar_wait(tc::smem_u32(&bars[s]), phase)) { atomicCAS(&tc::g_tc_error, 0, 102); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a0 = tc::smem_u32(tiles + s * Cfg::STAGE_BYTES);
            const uint32_t b_hi = a0 + Cfg::A_BYTES;
            const uint32_t b_lo = b_hi + Cfg::B_TILE_BYTES;
            const uint64_t dbh = make_desc_mn(b_hi), dbl = make_desc_mn(b_lo);
#pragma unroll
            for (int h = 0; h < MH; ++h) {      // the row halves share the dy slice
                const uint32_t a_hi = a0 + h * 2 * A_TILE_BYTES, a_lo = a_hi + A_TILE_BYTES;
                // one k slice = 8 pixels = 1024 bytes further into every strip
                tc::mma_block_3xtf32<1024 / 16>(tmem_base + static_cast<uint32_t>((b * MH + h) * BN), make_desc_mn(a_hi), make_desc_mn(a_lo),
                                                dbh, dbl, IDESC_MN, !(i & 1));
            }
            tc::mma_commit(tc::smem_u32(&bars[S + s]));
            if ((i & 1) || i == nkb - 1) tc::mma_commit(tc::smem_u32(&bars[2 * S + b]));
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
    }
}

// NCHW fp32 -> two channels-last images: hi = tf32(x) (round to nearest), lo = x - hi.  One block moves 32 channels x
// 128 pixels of one image through shared memory: reads run along the pixels of a channel, writes along the channels
// of a pixel, both in full 128-byte lines.  A block takes `tiles_per_block` consecutive 128-pixel tiles.
// SUMS: the pass also adds scale * (sum over the block's pixels) of every channel into sums[channel] (fp32 atomics): the
// bias gradient of a convolution is the per-channel sum of dy, and this pass reads all of dy anyway.  One atomic per
// channel and block: with several tiles per block the atomics on one address stay a small part of the pass.
template <bool SUMS>
__global__ void __launch_bounds__(256) nchw_to_split_nhwc_kernel(const float* __restrict__ x, float* __restrict__ hi,
                                                                 float* __restrict__ lo, int C, int HW, int tiles_per_block,
                                                                 float* __restrict__ sums, float scale) {
    __shared__ float tile[32][TR_PIX + 1];
    const int n = blockIdx.z, c0 = blockIdx.y * 32;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int quad = t & 7;                     // channels 4 * quad .. + 3
    float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int it = 0; it < tiles_per_block; ++it) {
        const int p0 = (blockIdx.x * tiles_per_block + it) * TR_PIX;
        if (p0 >= HW) break;
        if (it) __syncthreads();                // the tile of the last round has been written out
        const float* src = x + (static_cast<size_t>(n) * C + c0) * HW + p0;
        const int npix = min(TR_PIX, HW - p0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = warp * 4 + j;
#pragma unroll
            for (int q = 0; q < TR_PIX / 32; ++q) {
                const int pix = q * 32 + lane;
                const float v = pix < npix ? __ldg(src + static_cast<size_t>(c) * HW + pix) : 0.0f;
                tile[c][pix] = v;
                if (SUMS) part[j] += v;
            }
        }
        __syncthreads();
        float* dh = hi + (static_cast<size_t>(n) * HW + p0) * C + c0 + quad * 4;
        float* dl = lo + (static_cast<size_t>(n) * HW + p0) * C + c0 + quad * 4;
#pragma unroll
        for (int pass = 0; pass < TR_PIX / 32; ++pass) {
            const int pix = pass * 32 + (t >> 3);
            if (pix < npix) {
                float4 h, l;
                tc::split_tf32_safe(tile[quad * 4 + 0][pix], h.x, l.x);
                tc::split_tf32_safe(tile[quad * 4 + 1][pix], h.y, l.y);
                tc::split_tf32_safe(tile[quad * 4 + 2][pix], h.z, l.z);
                tc::split_tf32_safe(tile[quad * 4 + 3][pix], h.w, l.w);
                *reinterpret_cast<float4*>(dh + static_cast<size_t>(pix) * C) = h;
                *reinterpret_cast<float4*>(dl + static_cast<size_t>(pix) * C) = l;
            }
        }
    }
    if (SUMS) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v = part[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) atomicAdd(sums + c0 + warp * 4 + j, scale * v);
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled from the driver the runtime is bound to (the library links no libcuda stub).
inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

// Tensor map over a channels-last image [n][h][w][c] (fp32, dense) with boxes of 32 channels x bw x bh pixels of one
// image, 128-byte swizzle, zeros outside the image.
// row_pitch / image_pitch (pixels; 0 = dense): the image may be a view of a larger one, e.g. the h x w pixels of a padded
// position list whose rows are row_pitch positions apart and whose images are image_pitch positions apart.
inline int make_image_map(CUtensorMap* map, const float* image, int n, int h, int w, int c, int bw, int bh,
                          CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, int row_pitch = 0, long long image_pitch = 0) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return VDNN_ERR_UNSUPPORTED;
    const cuuint64_t rp = row_pitch ? row_pitch : w, ip = image_pitch ? static_cast<cuuint64_t>(image_pitch) : static_cast<cuuint64_t>(h) * w;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(c), static_cast<cuuint64_t>(w), static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(n)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(c) * 4, rp * c * 4, ip * c * 4};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(bw), static_cast<cuuint32_t>(bh), 1u};
    const cuuint32_t elem[4] = {1u, 1u, 1u, 1u};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(image), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? VDNN_OK : VDNN_ERR_CUDA;
}

// Box shape (bw x bh = 32 pixels, bw a power of two) that covers a grid of out_h x out_w pixels with the fewest boxes.
inline void pick_box(int out_h, int out_w, int* bw_log2, int* bh) {
    long best = -1;
    for (int lg = 5; lg >= 2; --lg) {
        const int bw = 1 << lg, h = BOX_PIXELS / bw;
        const long boxes = static_cast<long>(ceil_div(out_w, bw)) * ceil_div(out_h, h);
        if (best < 0 || boxes < best) { best = boxes; *bw_log2 = lg; *bh = h; }
    }
}

// Bytes of the two images of an n x c x h x w tensor.
inline size_t image_bytes(int n, int c, int h, int w) { return 2 * sizeof(float) * static_cast<size_t>(n) * c * h * w; }

// Transforms `src` (NCHW) into images at `images` (image_bytes() bytes, 128-byte aligned) and runs the contraction
// against packed weight tiles.  `splits` / `k_chunk` as planned by the caller (k_chunk a multiple of 32).
template <int BN>
int launch_bn(const Problem& q, const float* src, char* images, const char* b_tiles, float* out, const float* bias, float alpha,
              float beta, int mode, size_t partial_stride, int splits, int k_chunk, cudaStream_t stream) {
    typedef Config<BN> Cfg;
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    auto kern = conv_kernel<BN>;
    if (VDNN_ONCE_PER_DEVICE(dev))
        VDNN_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    const size_t elems = static_cast<size_t>(q.n) * q.cin * q.in_h * q.in_w;
    float* hi = reinterpret_cast<float*>(images);
    float* lo = hi + elems;
    Params p;
    p.n_img = q.n; p.out_h = q.out_h; p.out_w = q.out_w;
    pick_box(q.out_h, q.out_w, &p.bw_log2, &p.bh);
    const int bw = 1 << p.bw_log2;
    p.boxes_w = ceil_div(q.out_w, bw);
    const int boxes_h = ceil_div(q.out_h, p.bh);
    const long total = static_cast<long>(q.n) * boxes_h * p.boxes_w;
    if (total > 0x7fffffffL / 2) return VDNN_ERR_UNSUPPORTED;
    p.total_boxes = static_cast<int>(total);
    p.div_boxes_img = FastDiv(boxes_h * p.boxes_w); p.div_boxes_w = FastDiv(p.boxes_w);
    p.div_cblocks = FastDiv(q.cin / BK); p.div_s = FastDiv(q.S);
    p.tap_sign = q.tap_sign; p.off_h = q.off_h; p.off_w = q.off_w;
    p.K = q.R * q.S * q.cin; p.k_chunk = k_chunk; p.kblocks_total = p.K / BK;
    p.b_tiles = b_tiles;
    p.out = out; p.bias = bias; p.alpha = alpha; p.beta = beta; p.mode = mode; p.n_cols = q.n_cols;
    p.partial_stride = partial_stride;
    CUtensorMap map_hi, map_lo;
    int st = make_image_map(&map_hi, hi, q.n, q.in_h, q.in_w, q.cin, bw, p.bh);
    if (st != VDNN_OK) return st;
    st = make_image_map(&map_lo, lo, q.n, q.in_h, q.in_w, q.cin, bw, p.bh);
    if (st != VDNN_OK) return st;
    const int hw = q.in_h * q.in_w;
    dim3 tgrid(ceil_div(hw, TR_PIX), q.cin / 32, q.n);
    if (tgrid.y > 65535u || tgrid.z > 65535u) return VDNN_ERR_UNSUPPORTED;
    nchw_to_split_nhwc_kernel<false><<<tgrid, 256, 0, stream>>>(src, hi, lo, q.cin, hw, 1, nullptr, 0.0f);
    VDNN_LAUNCHED();
    dim3 grid(ceil_div(p.total_boxes, BOXES), ceil_div(q.n_cols, BN), splits);
    if (grid.y > 65535u || grid.z > 65535u) return VDNN_ERR_UNSUPPORTED;
    kern<<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(map_hi, map_lo, p);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

inline int launch(const Problem& q, const float* src, char* images, const char* b_tiles, float* out, const float* bias, float alpha,
                  float beta, int mode, size_t partial_stride, int splits, int k_chunk, cudaStream_t stream) {
    const int bn = tc::tile_n(q.n_cols);
    if (bn == 64) return launch_bn<64>(q, src, images, b_tiles, out, bias, alpha, beta, mode, partial_stride, splits, k_chunk, stream);
    if (bn == 128) return launch_bn<128>(q, src, images, b_tiles, out, bias, alpha, beta, mode, partial_stride, splits, k_chunk, stream);
    return launch_bn<256>(q, src, images, b_tiles, out, bias, alpha, beta, mode, partial_stride, splits, k_chunk, stream);
}

// Geometry of the strip engine's padded position list for one problem.
struct StripGeom { int wp, hp, lp, dh0, dh_step, row0, row_step, dw_min; bool ok; };

inline StripGeom strip_geometry(const Problem& q) {
    StripGeom g;
    // row shift of tap r: off_h + tap_sign * r; column shift of tap s likewise
    const int dh_a = q.off_h, dh_b = q.off_h + q.tap_sign * (q.R - 1);
    const int dw_a = q.off_w, dw_b = q.off_w + q.tap_sign * (q.S - 1);
    const int dh_min = dh_a < dh_b ? dh_a : dh_b, dh_max = dh_a < dh_b ? dh_b : dh_a;
    const int dw_min = dw_a < dw_b ? dw_a : dw_b, dw_max = dw_a < dw_b ? dw_b : dw_a;
    int gap_h = -dh_min > dh_max ? -dh_min : dh_max, gap_w = -dw_min > dw_max ? -dw_min : dw_max;
    if (gap_h < 0) gap_h = 0;
    if (gap_w < 0) gap_w = 0;
    g.wp = q.in_w + gap_w; g.hp = q.in_h + gap_h; g.lp = g.hp * g.wp;
    g.dh0 = q.off_h; g.dh_step = q.tap_sign;
    g.dw_min = dw_min;
    g.row0 = q.tap_sign > 0 ? 0 : q.S - 1; g.row_step = q.tap_sign;
    g.ok = q.S <= STRIP_MAX_TAPS && q.out_w <= g.wp && q.out_h <= g.hp && static_cast<long long>(q.n) * g.lp < 0x7fffff00LL;
    return g;
}

inline size_t strip_image_bytes(const Problem& q) {
    const StripGeom g = strip_geometry(q);
    return 2 * sizeof(float) * static_cast<size_t>(q.n) * g.lp * q.cin;
}

// Writes the operand images of the strip engine for problem q (strip_image_bytes(q) bytes at `images`).  sums (may be
// null): cin floats that receive += scale * (per-channel sums of src).
inline int strip_prepare(const Problem& q, const float* src, char* images, cudaStream_t stream, float* sums = nullptr, float scale = 0.0f) {
    const StripGeom g = strip_geometry(q);
    if (!g.ok) return VDNN_ERR_UNSUPPORTED;
    const size_t elems = static_cast<size_t>(q.n) * g.lp * q.cin;
    float* hi = reinterpret_cast<float*>(images);
    float* lo = hi + elems;
    const int tiles = ceil_div(q.in_h * q.in_w, TR_PIX);
    if (q.cin / 32 > 65535 || q.n > 65535) return VDNN_ERR_UNSUPPORTED;
    if (sums) {
        const int per_block = tiles < 8 ? tiles : 8;        // fewer atomics per channel
        nchw_to_split_strip_kernel<true><<<dim3(ceil_div(tiles, per_block), q.cin / 32, q.n), 256, 0, stream>>>(
            src, hi, lo, q.cin, q.in_h, q.in_w, g.wp, g.lp, per_block, sums, scale);
    } else {
        nchw_to_split_strip_kernel<false><<<dim3(tiles, q.cin / 32, q.n), 256, 0, stream>>>(src, hi, lo, q.cin, q.in_h, q.in_w, g.wp, g.lp, 1,
                                                                                           nullptr, 0.0f);
    }
    VDNN_LAUNCHED();
    return VDNN_OK;
}

// group_chunk: (filter row, channel block) groups per split; splits = ceil(R * cin / 32 / group_chunk).
template <int BN, int MH>
int strip_launch_bn(const Problem& q, const float* src, char* images, const char* b_tiles, float* out, const float* bias, float alpha,
                    float beta, int mode, size_t partial_stride, int splits, int group_chunk, cudaStream_t stream, bool prepare) {
    typedef StripConfig<BN, MH> Cfg;
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    auto kern = strip_kernel<BN, MH>;
    if (VDNN_ONCE_PER_DEVICE(dev))
        VDNN_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    const StripGeom g = strip_geometry(q);
    if (!g.ok) return VDNN_ERR_UNSUPPORTED;
    const size_t elems = static_cast<size_t>(q.n) * g.lp * q.cin;
    float* hi = reinterpret_cast<float*>(images);
    float* lo = hi + elems;
    StripParams p;
    p.n_img = q.n; p.img_h = q.in_h; p.img_w = q.in_w; p.wp = g.wp; p.lp = g.lp;
    p.total_pos = static_cast<long long>(q.n) * g.lp;
    p.div_lp = FastDiv(g.lp); p.div_wp = FastDiv(g.wp);
    p.out_h = q.out_h; p.out_w = q.out_w; p.n_cols = q.n_cols;
    p.R = q.R; p.S = q.S; p.cblocks = q.cin / BK;
    p.dh0 = g.dh0; p.dh_step = g.dh_step; p.row0 = g.row0; p.row_step = g.row_step; p.dw_min = g.dw_min;
    // VDNN_STRIP_MODE (diagnostics): unset / 1 = one strip per filter row, tap windows by start address alone;
    // 0 = the same with the swizzle phase also in the descriptors' base-offset field (gives wrong results on B200);
    // 2 = one strip per tap (no shifted windows)
    static const int strip_mode = []() { const char* v = getenv("VDNN_STRIP_MODE"); return v ? atoi(v) : 1; }();
    p.inner = strip_mode == 2 ? 1 : q.S;
    p.use_base_offset = strip_mode == 0 ? 1 : 0;
    p.groups_total = (strip_mode == 2 ? q.R * q.S : q.R) * p.cblocks;
    p.group_chunk = strip_mode == 2 ? group_chunk * q.S : group_chunk;
    p.kblocks_total = q.R * q.S * p.cblocks;
    p.b_tiles = b_tiles;
    p.out = out; p.bias = bias; p.alpha = alpha; p.beta = beta; p.mode = mode; p.partial_stride = partial_stride;
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return VDNN_ERR_UNSUPPORTED;
    CUtensorMap map_hi, map_lo;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(q.cin), static_cast<cuuint64_t>(p.total_pos)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(q.cin) * 4};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(BM + p.inner - 1)};
    const cuuint32_t elem[2] = {1u, 1u};
    for (int half = 0; half < 2; ++half) {
        const CUresult r = enc(half ? &map_lo : &map_hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, half ? lo : hi, dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return VDNN_ERR_CUDA;
    }
    if (prepare) {
        const int st = strip_prepare(q, src, images, stream);
        if (st != VDNN_OK) return st;
    }
    // persistent along x: as many CTAs as the GPU holds at once (all column tiles and splits of an output tile run side
    // by side, so that they share its strips through L2), each walking every gridDim.x-th output tile
    const long long tiles = ceil_div<long long>(p.total_pos, BM * MH);
    const int ny = ceil_div(q.n_cols, BN);
    if (ny > 65535 || splits > 65535) return VDNN_ERR_UNSUPPORTED;
    long long gx = static_cast<long long>(sm_count()) * Cfg::CTAS_PER_SM / (static_cast<long long>(ny) * splits);
    if (gx < 1) gx = 1;
    if (gx > tiles) gx = tiles;
    dim3 grid(static_cast<unsigned>(gx), ny, splits);
    kern<<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(map_hi, map_lo, p);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

// Tile shape of the strip engine by the number of output columns (measured on B200, VGG16 shapes at batch 32):
//   up to 64 columns    128 positions x 64, two CTAs per SM   (one thread can issue about 12 MMAs per 384 clocks of
//                        tensor work: two CTAs give two issuers)
//   65 .. 128 columns   256 positions x 128: the two 128-row halves share the weight tile (a third fewer bytes per flop)
//   more                128 positions x 256: with 256-column MMAs the tensor core reads the fewest operand bytes per
//                        flop from shared memory, which is what bounds the narrower shapes
// VDNN_STRIP_SHAPE=tall / wide forces 256 x 128 (256 x 64) or 128-row tiles everywhere (comparison runs).
inline int strip_shape_override() {
    static const int v = []() { const char* e = getenv("VDNN_STRIP_SHAPE"); return !e ? 0 : (e[0] == 't' ? 2 : (e[0] == 'w' ? 1 : 0)); }();
    return v;
}
inline int strip_halves(int n_cols) {
    const int o = strip_shape_override();
    if (o) return o;
    return (n_cols > 64 && n_cols <= 128) ? 2 : 1;
}
inline int strip_tile_n(int n_cols) {
    if (strip_halves(n_cols) == 2) return n_cols <= 64 ? 64 : 128;
    return tc::tile_n(n_cols);
}

#include "conv_tma_pair.cuh"

// 256-column tiles of the strip engine run on CTA pairs (conv_tma_pair.cuh); VDNN_STRIP_PAIRS=0: on single CTAs
// (comparison runs).  Pair tiles of 128 and 64 columns were measured too and are slower than what single CTAs do there
// (128 -> 128 @ 112 x 112 forward, batch 32: 0.735 ms against 0.647 for 256 x 128 tiles on one CTA; 64 -> 64 @ 224 x 224:
// 1.35 ms against 0.90 for two CTAs per SM).
inline bool strip_pairs_enabled() {
    static const bool v = []() { const char* e = getenv("VDNN_STRIP_PAIRS"); return !e || e[0] != '0'; }();
    return v;
}

// prepare = false: the images at `images` have been written already (strip_prepare) and src is not read.
inline int strip_launch(const Problem& q, const float* src, char* images, const char* b_tiles, float* out, const float* bias,
                        float alpha, float beta, int mode, size_t partial_stride, int splits, int group_chunk, cudaStream_t stream,
                        bool prepare = true) {
    const int bn = strip_tile_n(q.n_cols);
    if (bn == 256 && strip_halves(q.n_cols) == 1 && strip_pairs_enabled()) {
        const int st = pair::strip_pair_launch<256>(q, src, images, b_tiles, out, bias, alpha, beta, mode, partial_stride, splits, group_chunk, stream, prepare);
        if (st != VDNN_ERR_UNSUPPORTED) return st;
    }
    if (strip_halves(q.n_cols) == 2) {
        if (bn == 64) return strip_launch_bn<64, 2>(q, src, images, b_tiles, out, bias, alpha, beta, mode, partial_stride, splits, group_chunk, stream, prepare);
        return strip_launch_bn<128, 2>(q, src, images, b_tiles, out, bias, alpha, beta, mode, partial_stride, splits, group_chunk, stream, prepare);
    }
    if (bn == 64) return strip_launch_bn<64, 1>(q, src, images, b_tiles, out, bias, alpha, beta, mode, partial_stride, splits, group_chunk, stream, prepare);
    if (bn == 128) return strip_launch_bn<128, 1>(q, src, images, b_tiles, out, bias, alpha, beta, mode, partial_stride, splits, group_chunk, stream, prepare);
    return strip_launch_bn<256, 1>(q, src, images, b_tiles, out, bias, alpha, beta, mode, partial_stride, splits, group_chunk, stream, prepare);
}

#include "conv_tma_wstrip.cuh"

struct WgradProblem {
    int n, c, h, w;          // x
    int k, p, q;             // dy: n x k x p x q
    int R, S, pad_h, pad_w;
};

// The filter gradient of layers with more than 128 filters runs on CTA pairs (conv_tma_pair.cuh); VDNN_WGRAD_PAIRS=0:
// on single CTAs (comparison runs).  Pair tiles of 128 and 64 filters were measured too and are slower than single
// CTAs (128 -> 128 @ 112 x 112, batch 32: 1.13 ms against 0.84; 64 -> 64 @ 224 x 224: 2.14 against 1.48).
inline bool wgrad_pairs_enabled(int bn) {
    static const bool on = []() { const char* e = getenv("VDNN_WGRAD_PAIRS"); return !e || e[0] != '0'; }();
    return on && bn == 256;
}

// Reduction split for the filter gradient: the tiles (row-group quadruples x column tiles) are few, the reduction over
// pixel boxes is long; as many splits as fill two waves of CTAs, at least two boxes each.
// Row halves of a filter-gradient tile.  Measured (B200, batch 128): 128 -> 128 @ 112 x 112 (36 row groups) 3.39 ms with
// one half, 3.20 with two; 64 -> 128 @ 112 x 112 (18 groups: the third two-half tile is mostly padding) 2.03 / 2.05;
// 64 -> 64 @ 224 x 224 5.86 / 6.02.  So: two halves for 128-filter tiles with at least 32 row groups.
// VDNN_WGRAD_SHAPE=flat / tall: one half everywhere / two wherever the tensor memory holds them (comparison runs).
inline int wgrad_halves(int bn, int row_groups) {
    static const int force = []() { const char* e = getenv("VDNN_WGRAD_SHAPE"); return !e ? 0 : (e[0] == 'f' ? 1 : (e[0] == 't' ? 2 : 0)); }();
    if (force == 1 || bn > 128) return 1;
    if (force == 2) return 2;
    return (bn == 128 && row_groups >= 32) ? 2 : 1;
}

inline void wgrad_plan(const WgradProblem& q, int total_boxes, int* splits, int* box_chunk) {
    const int bn = tc::tile_n(q.k);
    const int row_groups = q.R * q.S * (q.c / 32);
    int row_tiles = ceil_div(row_groups, BOXES * wgrad_halves(bn, row_groups));
    if (wgrad_pairs_enabled(bn)) row_tiles = (row_tiles + 1) / 2 * 2;          // CTA pairs take two row tiles each
    const long tiles = static_cast<long>(row_tiles) * ceil_div(q.k, bn);
    long s = (2L * sm_count()) / tiles;
    if (s > total_boxes / 2) s = total_boxes / 2;
    if (s > 1024) s = 1024;
    if (s < 1) s = 1;
    *box_chunk = ceil_div(total_boxes, static_cast<int>(s));
    *splits = ceil_div(total_boxes, *box_chunk);
}

inline int wgrad_boxes(const WgradProblem& q, int* bw_log2, int* bh) {
    pick_box(q.p, q.q, bw_log2, bh);
    return q.n * ceil_div(q.p, *bh) * ceil_div(q.q, 1 << *bw_log2);
}

// Bytes of split partials the filter gradient needs behind its four images.
inline size_t wgrad_partial_bytes(const WgradProblem& q) {
    int lg, bh, splits, chunk;
    const int total = wgrad_boxes(q, &lg, &bh);
    wgrad_plan(q, total, &splits, &chunk);
    return splits > 1 ? static_cast<size_t>(splits) * q.k * q.c * q.R * q.S * sizeof(float) : 0;
}

// The images of dy as the data gradient's strip engine has written them (padded position list: rows wp positions apart,
// images lp positions apart): the filter gradient reads the h x w pixels of every image through a strided tensor map, so
// one pass over dy serves both gradients.
struct SharedDy { const float* hi; const float* lo; int wp; long long lp; };

// bias_sums (may be null): K floats that receive += bias_scale * (per-channel sums of dy) from the dy transform pass.
// shared (may be null): dy has been written as images already (then dy, bias_sums are not used, and ws holds the x images
// and the partial sums only).
template <int BN, int MH>
int wgrad_launch_bn(const WgradProblem& q, const float* x, const float* dy, char* ws, float* dw, float alpha, float beta,
                    cudaStream_t stream, int* splits_out, float** partial_out, float* bias_sums, float bias_scale, const SharedDy* shared) {
    typedef WgradConfig<BN, MH> Cfg;
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    auto kern = wgrad_kernel<BN, MH>;
    if (VDNN_ONCE_PER_DEVICE(dev))
        VDNN_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    const size_t xe = static_cast<size_t>(q.n) * q.c * q.h * q.w, ye = static_cast<size_t>(q.n) * q.k * q.p * q.q;
    float* xh = reinterpret_cast<float*>(ws);
    float* xl = xh + xe;
    float* yh = shared ? const_cast<float*>(shared->hi) : xl + xe;
    float* yl = shared ? const_cast<float*>(shared->lo) : yh + ye;
    float* partial = shared ? xl + xe : yl + ye;
    WgradParams p;
    p.n_img = q.n;
    p.total_boxes = wgrad_boxes(q, &p.bw_log2, &p.bh);
    const int bw = 1 << p.bw_log2;
    p.boxes_w = ceil_div(q.q, bw);
    p.div_boxes_img = FastDiv(ceil_div(q.p, p.bh) * p.boxes_w); p.div_boxes_w = FastDiv(p.boxes_w);
    int splits = 1;
    wgrad_plan(q, p.total_boxes, &splits, &p.box_chunk);
    p.cblocks = q.c / 32; p.taps_s = q.S; p.row_groups = q.R * q.S * p.cblocks;
    p.off_h = -q.pad_h; p.off_w = -q.pad_w;
    p.C = q.c; p.taps = q.R * q.S; p.n_cols = q.k;
    p.partial_stride = static_cast<size_t>(q.k) * q.c * q.R * q.S;
    if (splits > 1) { p.out = partial; p.alpha = 1.0f; p.beta = 0.0f; p.mode = EPI_PARTIAL; }
    else { p.out = dw; p.alpha = alpha; p.beta = beta; p.mode = EPI_DIRECT; }
    CUtensorMap mxh, mxl, myh, myl;
    int st;
    const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    if ((st = make_image_map(&mxh, xh, q.n, q.h, q.w, q.c, bw, p.bh, sw)) != VDNN_OK) return st;
    if ((st = make_image_map(&mxl, xl, q.n, q.h, q.w, q.c, bw, p.bh, sw)) != VDNN_OK) return st;
    if ((st = make_image_map(&myh, yh, q.n, q.p, q.q, q.k, bw, p.bh, sw, shared ? shared->wp : 0, shared ? shared->lp : 0)) != VDNN_OK) return st;
    if ((st = make_image_map(&myl, yl, q.n, q.p, q.q, q.k, bw, p.bh, sw, shared ? shared->wp : 0, shared ? shared->lp : 0)) != VDNN_OK) return st;
    dim3 tx(ceil_div(q.h * q.w, TR_PIX), q.c / 32, q.n), ty(ceil_div(q.p * q.q, TR_PIX), q.k / 32, q.n);
    if (tx.y > 65535u || tx.z > 65535u || ty.y > 65535u) return VDNN_ERR_UNSUPPORTED;
    nchw_to_split_nhwc_kernel<false><<<tx, 256, 0, stream>>>(x, xh, xl, q.c, q.h * q.w, 1, nullptr, 0.0f);
    VDNN_LAUNCHED();
    if (shared) {
        // dy is there already
    } else if (bias_sums) {
        // several tiles per block: fewer atomics per channel; the grid stays above two waves for every layer of interest
        const int tiles = static_cast<int>(ty.x), per_block = tiles < 8 ? tiles : 8;
        const dim3 tys((tiles + per_block - 1) / per_block, ty.y, ty.z);
        nchw_to_split_nhwc_kernel<true><<<tys, 256, 0, stream>>>(dy, yh, yl, q.k, q.p * q.q, per_block, bias_sums, bias_scale);
    } else {
        nchw_to_split_nhwc_kernel<false><<<ty, 256, 0, stream>>>(dy, yh, yl, q.k, q.p * q.q, 1, nullptr, 0.0f);
    }
    VDNN_LAUNCHED();
    dim3 grid(ceil_div(p.row_groups, BOXES * MH), ceil_div(q.k, BN), splits);
    if (grid.y > 65535u || grid.z > 65535u) return VDNN_ERR_UNSUPPORTED;
    if constexpr (BN == 256) {
        if (wgrad_pairs_enabled(BN)) {
            const int st = pair::wgrad_pair_launch<BN>(mxh, mxl, myh, myl, p, grid.x, grid.y, grid.z, stream);
            if (st != VDNN_OK) return st;
            *splits_out = splits;
            *partial_out = partial;
            return VDNN_OK;
        }
    }
    {
        kern<<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(mxh, mxl, myh, myl, p);
        VDNN_LAUNCHED();
    }
    *splits_out = splits;
    *partial_out = partial;
    return VDNN_OK;
}

// Bytes of the four images of the filter gradient's operands.
inline size_t wgrad_image_bytes(const WgradProblem& q) {
    return image_bytes(q.n, q.c, q.h, q.w) + image_bytes(q.n, q.k, q.p, q.q);
}

inline int wgrad_launch(const WgradProblem& q, const float* x, const float* dy, char* ws, float* dw, float alpha, float beta,
                        cudaStream_t stream, int* splits, float** partial, float* bias_sums = nullptr, float bias_scale = 0.0f,
                        const SharedDy* shared = nullptr) {
    const int bn = tc::tile_n(q.k);
    if (wgrad_halves(bn, q.R * q.S * (q.c / 32)) == 2) {
        if (bn == 64) return wgrad_launch_bn<64, 2>(q, x, dy, ws, dw, alpha, beta, stream, splits, partial, bias_sums, bias_scale, shared);
        return wgrad_launch_bn<128, 2>(q, x, dy, ws, dw, alpha, beta, stream, splits, partial, bias_sums, bias_scale, shared);
    }
    if (bn == 64) return wgrad_launch_bn<64, 1>(q, x, dy, ws, dw, alpha, beta, stream, splits, partial, bias_sums, bias_scale, shared);
    if (bn == 128) return wgrad_launch_bn<128, 1>(q, x, dy, ws, dw, alpha, beta, stream, splits, partial, bias_sums, bias_scale, shared);
    return wgrad_launch_bn<256, 1>(q, x, dy, ws, dw, alpha, beta, stream, splits, partial, bias_sums, bias_scale, shared);
}

}  // namespace tma
}  // namespace vdnn
