// tcgen05 contraction engine for sm_100a: fp32-accurate products on the 5th-generation tensor
// cores by the 3xTF32 split
//        a*b ~= a_hi*b_hi + a_hi*b_lo + a_lo*b_hi,      x_hi = tf32(x), x_lo = x - x_hi  (exact),
// with fp32 accumulation in tensor memory (TMEM).
//
// One CTA computes a 128 x BN tile of D (BN = 64, 128 or 256) over a K range in steps of 32:
//   warps 0-15 producers: gather the 128 x 32 A tile and BN x 32 B tile straight from the NCHW /
//              KCRS tensors (gemm_operands.cuh), split every value into hi / lo, and store both
//              into shared memory in the K-major, 128-byte-swizzled layout tcgen05.mma reads;
//              they also collect the per-stage sums from TMEM (tcgen05.ld) and run the epilogue:
//              alpha / beta / bias / split-K handling, coalesced stores.
//   warp 16    allocates TMEM; one elected lane issues tcgen05.mma (3 per 8-wide k slice, 12 per
//              stage) into one of two TMEM accumulator buffers and tcgen05.commit to hand the stage
//              back and to publish that buffer.  The producers add each finished buffer into fp32
//              registers (round-to-nearest adds), so no accumulation chain inside the tensor core
//              is longer than two stages (24 MMAs).
// Stages are handed over with mbarriers (full: one arrival per producer thread, empty: one commit).  Every
// wait is bounded: on expiry the thread records an error code in g_tc_error, stops waiting, and
// the CTA still runs its common exit path (barrier, TMEM release).
#pragma once

#include "gemm_operands.cuh"

namespace vdnn {
namespace tc {

#ifndef VDNN_TC_PRODUCERS
#define VDNN_TC_PRODUCERS 512
#endif
constexpr int BM = 128, BK = 32, PRODUCERS = VDNN_TC_PRODUCERS, THREADS = PRODUCERS + 32;
constexpr int PRODUCER_WARPS = PRODUCERS / 32;      // 8 or 16; the MMA warp comes after them
static_assert(PRODUCERS == 256 || PRODUCERS == 512, "producer mappings are written for 256 or 512 threads");
constexpr int A_TILE_BYTES = BM * BK * 4;              // 16 KB, one per hi / lo
constexpr unsigned long long SPIN_CYCLES = 4000000000ull;   // ~2 s at 1.9 GHz
constexpr unsigned SPIN_TRIES = 1u << 26;

// 0 = healthy; otherwise 100 + role of the first wait that expired (1 producer, 2 mma, 3 epilogue, 4 the self-test).
__device__ int g_tc_error = 0;

// PAIRED: two CTAs of this configuration share an SM (see STAGES).
template <int BN, bool PAIRED = false> struct Config {
    static constexpr int B_TILE_BYTES = BN * BK * 4;
    static constexpr int STAGE_BYTES = 2 * A_TILE_BYTES + 2 * B_TILE_BYTES;
    // The 64-column tile with one gathered operand is bound by its producers (the tensor core needs a quarter of
    // their time per k block), so two of its CTAs share an SM: two stages each, and the producers of one fill the
    // issue slots the other leaves (64 -> 64 @ 224x224 forward: 1.65 -> 1.34 ms).  With both operands gathered (the
    // filter gradient of 64-filter layers) the deeper pipeline of a single CTA was the faster one.
    static constexpr int STAGES = BN == 256 ? 2 : (BN == 128 ? 3 : (PAIRED ? 2 : 4));
    static constexpr int CTAS_PER_SM = PAIRED ? 2 : 1;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    // instruction descriptor: D = F32, A = B = TF32, both K-major, N = BN, M = 128
    static constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                      (static_cast<uint32_t>(BM >> 4) << 24);
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false when the limit expired.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, unsigned long long cycles, unsigned tries) {
    if (mbar_try(bar, parity)) return true;                  // the common case costs one instruction
    const unsigned long long t0 = clock64();
    for (unsigned it = 0; it < tries; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 1023u) == 1023u && clock64() - t0 > cycles) break;
    }
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    return mbar_wait_for(bar, parity, SPIN_CYCLES, SPIN_TRIES);
}

// K-major operand tile with 128-byte swizzle: row r is 128 bytes (32 fp32), 8 rows form a 1 KB atom,
// the 16-byte chunk index is XORed with (r & 7).
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return static_cast<uint32_t>((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

// Shared-memory matrix descriptor: start address, stride between 8-row atoms = 1024 B, descriptor
// version 1 (sm_100), layout = SWIZZLE_128B.  The leading-dimension offset is unused for a K-major
// tile that is exactly one swizzle atom wide.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the accumulate flag known at compile time (no predicate set-up): D += A * B.
__device__ __forceinline__ void mma_tf32_acc(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 1;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
// One 32-wide k block of the 3xTF32 product: for each of the four 8-wide k slices, lo*hi, hi*lo, hi*hi (small terms
// first).  The four descriptors are built once; a k slice is 32 bytes further into the swizzle atom, which is 2 in the
// descriptors' 16-byte address units.  `fresh` = the first MMA overwrites the accumulator instead of adding to it.
// (K-major tiles: STEP = 2.  MN-major strips step a whole 8-row group per k slice: STEP = bytes / 16.)
template <int STEP = 2>
__device__ __forceinline__ void mma_block_3xtf32(uint32_t d_tmem, uint64_t dah, uint64_t dal, uint64_t dbh, uint64_t dbl,
                                                 uint32_t idesc, bool fresh) {
    mma_tf32(d_tmem, dal, dbh, idesc, fresh ? 0u : 1u);
    mma_tf32_acc(d_tmem, dah, dbl, idesc);
    mma_tf32_acc(d_tmem, dah, dbh, idesc);
#pragma unroll
    for (int ks = 1; ks < BK / 8; ++ks) {
        dah += STEP; dal += STEP; dbh += STEP; dbl += STEP;
        mma_tf32_acc(d_tmem, dal, dbh, idesc);
        mma_tf32_acc(d_tmem, dah, dbl, idesc);
        mma_tf32_acc(d_tmem, dah, dbh, idesc);
    }
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// x = hi + lo with hi representable in tf32 (10 explicit mantissa bits, round to nearest, ties away from zero).
// Two integer instructions: cvt.rna.tf32.f32 does the same in one, but on the quarter-rate conversion pipe,
// and measured slower in the producers.
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
    hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
    lo = x - hi;
}
// The same for the passes that prepare operand images (bandwidth-bound, so two more instructions are free): an
// infinite x, or one that rounds up to infinity, keeps lo = 0, so that the three partial products give +-inf as one
// fp32 product would, not inf - inf.
__device__ __forceinline__ void split_tf32_safe(float x, float& hi, float& lo) {
    hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
    lo = (__float_as_uint(hi) & 0x7F800000u) == 0x7F800000u ? 0.0f : x - hi;
}

// Gathers a ROWS x 32 operand tile into registers and stores its hi / lo images.
//   KC = true : the operand is contiguous along k.  Thread t handles the 16-byte chunk (t & 7) of rows
//               (t >> 3) + 32*j: a quarter warp reads one 128-byte row segment.
//   KC = false: the operand is contiguous along its rows.  Thread t handles row t % ROWS and a run of
//               32 / (256 / ROWS) consecutive k: a warp reads 32 consecutive rows of one k.
template <class Op, bool KC, int ROWS>
struct Gather {
    static constexpr int ROWS_PER_PASS = PRODUCERS / 8;      // KC: 8 threads cover one 128-byte row
    static constexpr int PASSES = ROWS / ROWS_PER_PASS;
    static constexpr int KRUN = BK / (PRODUCERS / ROWS);     // !KC: consecutive k per thread (4 .. 16)
    static_assert(PASSES >= 1 && KRUN >= 4, "tile too small for the producer count");
    static constexpr int COUNT = KC ? PASSES * 4 : KRUN;
    typename Op::Row rows[KC ? PASSES : 1];
    float v[COUNT];

    __device__ __forceinline__ void init(const Op& op, int row0, int t) {
        if (KC) {
#pragma unroll
            for (int j = 0; j < PASSES; ++j) rows[j] = op.row(row0 + (t >> 3) + ROWS_PER_PASS * j);
        } else {
            rows[0] = op.row(row0 + t % ROWS);
        }
    }
    __device__ __forceinline__ void fetch(const Op& op, int k0, int kend, int t) {
        if constexpr (KC) {
            const int kk = k0 + (t & 7) * 4;
            const auto c = op.cols4(kk, kend);
#pragma unroll
            for (int j = 0; j < PASSES; ++j) op.load4(rows[j], c, kk, &v[j * 4]);
        } else {
            op.template load_run<KRUN>(rows[0], k0 + (t / ROWS) * KRUN, kend, v);
        }
    }
    __device__ __forceinline__ void stash(char* hi_tile, char* lo_tile, int t) const {
        if (KC) {
#pragma unroll
            for (int j = 0; j < PASSES; ++j) {
                float4 h, l;
                split_tf32(v[j * 4 + 0], h.x, l.x); split_tf32(v[j * 4 + 1], h.y, l.y);
                split_tf32(v[j * 4 + 2], h.z, l.z); split_tf32(v[j * 4 + 3], h.w, l.w);
                const uint32_t o = swz((t >> 3) + ROWS_PER_PASS * j, t & 7);
                *reinterpret_cast<float4*>(hi_tile + o) = h;
                *reinterpret_cast<float4*>(lo_tile + o) = l;
            }
        } else {
            const int row = t % ROWS, chunk0 = (t / ROWS) * (KRUN / 4);
#pragma unroll
            for (int q = 0; q < KRUN / 4; ++q) {
                float4 h, l;
                split_tf32(v[q * 4 + 0], h.x, l.x); split_tf32(v[q * 4 + 1], h.y, l.y);
                split_tf32(v[q * 4 + 2], h.z, l.z); split_tf32(v[q * 4 + 3], h.w, l.w);
                const uint32_t o = swz(row, chunk0 + q);
                *reinterpret_cast<float4*>(hi_tile + o) = h;
                *reinterpret_cast<float4*>(lo_tile + o) = l;
            }
        }
    }
};

// BBULK: the B operand was packed beforehand into images of its shared-memory tiles (hi and lo halves,
// swizzled, zero-padded; see pack_b_tiles_kernel), one image per (n tile, k block).  A producer thread then
// fetches a stage's B tiles with a single bulk asynchronous copy (the TMA engine, no tensor map needed for a
// contiguous image) that reports its bytes to the stage's "full" barrier; the producers only gather A.
template <class OpA, class OpB, bool AKC, bool BKC, int BN, bool BBULK>
__global__ void __launch_bounds__(THREADS, Config<BN, BN == 64 && !(AKC && BKC)>::CTAS_PER_SM)
gemm_kernel(const OpA opa, const OpB opb, const Epilogue epi, int M, int N, int K, int k_chunk,
            const char* __restrict__ b_tiles, int kblocks_total) {
    typedef Config<BN, BN == 64 && !(AKC && BKC)> Cfg;
    constexpr int S = Cfg::STAGES;
    extern __shared__ char smem_raw[];
    // operand tiles need 1 KB alignment (swizzle atoms); barriers and the TMEM slot follow them
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + S * Cfg::STAGE_BYTES);
    // bars[0..S) stage full, bars[S..2S) stage empty, bars[2S..2S+2) accumulator buffer ready; then the TMEM base
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 2);

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int kbeg = blockIdx.z * k_chunk;
    const int kend = min(K, kbeg + k_chunk);
    const int nkb = kbeg < kend ? (kend - kbeg + BK - 1) / BK : 0;

    if (t == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars[s]), PRODUCERS);
            mbar_init(smem_u32(&bars[S + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * S]), 1);
        mbar_init(smem_u32(&bars[2 * S + 1]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Two accumulator buffers of BN columns each: the tensor core sums two 32-wide k blocks into a
    // buffer (a chain of 24 MMAs) while the previous pair's buffer is added into fp32 registers.
    // Keeping the in-TMEM chains short matters for accuracy: the tensor core truncates when it adds
    // into its accumulator, and over thousands of chained MMAs that bias reaches 1e-5 relative.
    if (warp == PRODUCER_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp < PRODUCER_WARPS) {
        // ------------------------------------------------------------------ producers
        Gather<OpA, AKC, BM> ga;
        Gather<OpB, BKC, BN> gb;
        ga.init(opa, m0, t);
        if (!BBULK) gb.init(opb, n0, t);
        const char* b_src = BBULK ? b_tiles + (static_cast<size_t>(blockIdx.y) * kblocks_total + kbeg / BK) * (2 * Cfg::B_TILE_BYTES)
                                  : nullptr;
        // this thread owns row (warp & 3) * 32 + lane of the tile and a slice of its columns
        constexpr int NACC = BN / (PRODUCER_WARPS / 4);
        const int col_beg = (warp >> 2) * NACC;
        const uint32_t tmem_mine = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(col_beg);
        float acc[NACC];
#pragma unroll
        for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;
        bool alive = true;
        int next_drain = 0;

        // adds the finished pair of k blocks `pair` from its TMEM buffer into the register accumulators
        auto drain = [&](int pair) {
            const int b = pair & 1;
            bool ok = mbar_wait(smem_u32(&bars[2 * S + b]), static_cast<uint32_t>(pair >> 1) & 1u);
            ok = __all_sync(0xffffffffu, ok);               // tcgen05.ld is warp-collective
            if (!ok) { atomicCAS(&g_tc_error, 0, 103); alive = false; return; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < NACC; c += 16) {
                float v[16];
                tmem_ld16(tmem_mine + static_cast<uint32_t>(b * BN + c), v);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c + j] += v[j];
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        };

        if (nkb > 0) { ga.fetch(opa, kbeg, kend, t); if (!BBULK) gb.fetch(opb, kbeg, kend, t); }
        for (int i = 0; i < nkb && alive; ++i) {
            const int s = i % S;
            const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
            // blocks i, i+1 (i even) reuse the accumulator buffer of blocks i-4, i-3: empty it first (every producer
            // does, and the MMA of block i cannot start before all of them have arrived on full[s])
            if (i >= 4 && !(i & 1)) { drain(next_drain++); if (!alive) break; }
            bool ok = mbar_wait(smem_u32(&bars[S + s]), phase ^ 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { atomicCAS(&g_tc_error, 0, 101); alive = false; break; }
            char* st = tiles + s * Cfg::STAGE_BYTES;
            if (BBULK) {
                // the stage is free: one thread announces the bytes and starts the copy of both B halves
                if (t == 0) {
                    const uint32_t bar = smem_u32(&bars[s]), dst = smem_u32(st + 2 * A_TILE_BYTES);
                    const char* src = b_src + static_cast<size_t>(i) * (2 * Cfg::B_TILE_BYTES);
                    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(2 * Cfg::B_TILE_BYTES) : "memory");
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(dst), "l"(src), "r"(2 * Cfg::B_TILE_BYTES), "r"(bar) : "memory");
                }
            } else {
                gb.stash(st + 2 * A_TILE_BYTES, st + 2 * A_TILE_BYTES + Cfg::B_TILE_BYTES, t);
            }
            ga.stash(st, st + A_TILE_BYTES, t);
            // make the generic-proxy stores visible to the tensor core (async proxy), then publish
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_u32(&bars[s]));
            if (i + 1 < nkb) {
                ga.fetch(opa, kbeg + (i + 1) * BK, kend, t);
                if (!BBULK) gb.fetch(opb, kbeg + (i + 1) * BK, kend, t);
            }
        }
        while (alive && next_drain < (nkb + 1) / 2) drain(next_drain++);

        // ------------------------------------------------------------------ epilogue
        const int m = m0 + (warp & 3) * 32 + lane;
        if (alive && m < M) {
            const int roff = epi.row_off(m);
#pragma unroll
            for (int j = 0; j < NACC; ++j) {
                const int n = n0 + col_beg + j;
                if (n < N) epi.store(roff, n, acc[j], blockIdx.z);
            }
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        for (int i = 0; i < nkb; ++i) {
            const int s = i % S;
            const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
            if (!mbar_wait(smem_u32(&bars[s]), phase)) { atomicCAS(&g_tc_error, 0, 102); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(tiles + s * Cfg::STAGE_BYTES);
            const uint32_t a_lo = a_hi + A_TILE_BYTES;
            const uint32_t b_hi = a_hi + 2 * A_TILE_BYTES;
            const uint32_t b_lo = b_hi + Cfg::B_TILE_BYTES;
            // two consecutive k blocks share an accumulator buffer (a chain of 24 MMAs), then the other buffer is used
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(((i >> 1) & 1) * BN);
            mma_block_3xtf32(d_tmem, make_desc(a_hi), make_desc(a_lo), make_desc(b_hi), make_desc(b_lo), Cfg::IDESC, !(i & 1));
            mma_commit(smem_u32(&bars[S + s]));             // stage s may be overwritten once these finish
            if ((i & 1) || i == nkb - 1)
                mma_commit(smem_u32(&bars[2 * S + ((i >> 1) & 1)]));   // and this pair's sums may be collected
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == PRODUCER_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

template <class OpA, class OpB>
inline bool supported(int M, int N, int K) { return M >= 1 && N >= 1 && K >= 1; }

// Writes the shared-memory images of all B tiles: image (nt, kb) = [hi tile | lo tile], each BN rows of 128 bytes,
// 16-byte chunks swizzled as the kernel's own stash() does, zero where n >= N or k >= K.
// BKC: the operand is contiguous along k (a run of 4 k is one 16-byte load where aligned).
template <class OpB, int BN, bool BKC>
__global__ void __launch_bounds__(256) pack_b_tiles_kernel(const OpB opb, int N, int K, int n_tiles, int kblocks, char* __restrict__ out) {
    typedef Config<BN> Cfg;
    const size_t total = static_cast<size_t>(n_tiles) * kblocks * BN * 8;          // one thread per 16-byte chunk
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int chunk = static_cast<int>(i & 7);
        const int row = static_cast<int>((i >> 3) % BN);
        const size_t tile = (i >> 3) / BN;                                         // nt * kblocks + kb
        const int kb = static_cast<int>(tile % kblocks), nt = static_cast<int>(tile / kblocks);
        const typename OpB::Row r = opb.row(nt * BN + row);
        const int kk = kb * BK + chunk * 4;
        float4 h, l;
        float v[4];
        if constexpr (BKC) {
            if (kk < K) opb.load4(r, opb.cols4(kk, K), kk, v);
            else v[0] = v[1] = v[2] = v[3] = 0.0f;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = (kk + e < K) ? opb.load(r, opb.col(kk + e)) : 0.0f;
        }
        split_tf32_safe(v[0], h.x, l.x); split_tf32_safe(v[1], h.y, l.y); split_tf32_safe(v[2], h.z, l.z); split_tf32_safe(v[3], h.w, l.w);
        char* img = out + tile * (2 * Cfg::B_TILE_BYTES);
        *reinterpret_cast<float4*>(img + swz(row, chunk)) = h;
        *reinterpret_cast<float4*>(img + Cfg::B_TILE_BYTES + swz(row, chunk)) = l;
    }
}

// Column tile: wide tiles amortise the A gather over more columns (the producers' cost per flop goes with 1/BN).
inline int tile_n(int N) { return N <= 64 ? 64 : (N < 256 ? 128 : 256); }

// Bytes of packed B tile images for an N x K operand.
inline size_t bulk_bytes(int N, int K) {
    const int bn = tile_n(N);
    return static_cast<size_t>(ceil_div(N, bn)) * ceil_div(K, BK) * 2 * bn * BK * sizeof(float);
}

// Packs all B tiles of an N x K operand for the column tile tile_n(N) into `b_tiles` (bulk_bytes(N, K) bytes).
template <class OpB, bool BKC, int BN>
int pack_b_bn(const OpB& b, int N, int K, cudaStream_t stream, char* b_tiles) {
    const int n_tiles = ceil_div(N, BN), kblocks = ceil_div(K, BK);
    const size_t chunks = static_cast<size_t>(n_tiles) * kblocks * BN * 8;
    size_t blocks = ceil_div<size_t>(chunks, 256);
    const size_t cap = static_cast<size_t>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    pack_b_tiles_kernel<OpB, BN, BKC><<<static_cast<int>(blocks), 256, 0, stream>>>(b, N, K, n_tiles, kblocks, b_tiles);
    VDNN_LAUNCHED();
    return VDNN_OK;
}
// bn: the column tile the consuming kernel uses (0 = tile_n(N)).
template <class OpB, bool BKC>
int pack_b(const OpB& b, int N, int K, cudaStream_t stream, char* b_tiles, int bn = 0) {
    if (bn == 0) bn = tile_n(N);
    if (bn == 64) return pack_b_bn<OpB, BKC, 64>(b, N, K, stream, b_tiles);
    if (bn == 128) return pack_b_bn<OpB, BKC, 128>(b, N, K, stream, b_tiles);
    return pack_b_bn<OpB, BKC, 256>(b, N, K, stream, b_tiles);
}

template <class OpA, class OpB, bool AKC, bool BKC, int BN, bool BBULK>
int launch_bn(const OpA& a, const OpB& b, const Epilogue& epi, int M, int N, int K, int splits, int k_chunk, cudaStream_t stream,
              char* b_tiles) {
    typedef Config<BN, BN == 64 && !(AKC && BKC)> Cfg;
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    auto kern = gemm_kernel<OpA, OpB, AKC, BKC, BN, BBULK>;
    if (VDNN_ONCE_PER_DEVICE(dev))
        VDNN_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    dim3 grid(ceil_div(M, BM), ceil_div(N, BN), splits);
    if (grid.y > 65535u || grid.z > 65535u) return VDNN_ERR_UNSUPPORTED;
    const int kblocks = ceil_div(K, BK);
    if (BBULK) {
        const size_t chunks = static_cast<size_t>(grid.y) * kblocks * BN * 8;
        size_t blocks = ceil_div<size_t>(chunks, 256);
        const size_t cap = static_cast<size_t>(sm_count()) * 8;
        if (blocks > cap) blocks = cap;
        pack_b_tiles_kernel<OpB, BN, BKC><<<static_cast<int>(blocks), 256, 0, stream>>>(b, N, K, static_cast<int>(grid.y), kblocks, b_tiles);
        VDNN_LAUNCHED();
    }
    kern<<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(a, b, epi, M, N, K, k_chunk, b_tiles, kblocks);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

// k_chunk must be a multiple of 32.  b_tiles: nullptr, or bulk_bytes(N, K) bytes of 128-byte-aligned scratch: B is then
// packed into tile images first and fetched by bulk copies.
template <class OpA, class OpB, bool AKC, bool BKC>
int launch(const OpA& a, const OpB& b, const Epilogue& epi, int M, int N, int K, int splits, int k_chunk, cudaStream_t stream,
           char* b_tiles = nullptr) {
    const int bn = tile_n(N);
    if (b_tiles) {
        if (bn == 64) return launch_bn<OpA, OpB, AKC, BKC, 64, true>(a, b, epi, M, N, K, splits, k_chunk, stream, b_tiles);
        if (bn == 128) return launch_bn<OpA, OpB, AKC, BKC, 128, true>(a, b, epi, M, N, K, splits, k_chunk, stream, b_tiles);
        return launch_bn<OpA, OpB, AKC, BKC, 256, true>(a, b, epi, M, N, K, splits, k_chunk, stream, b_tiles);
    }
    if (bn == 64) return launch_bn<OpA, OpB, AKC, BKC, 64, false>(a, b, epi, M, N, K, splits, k_chunk, stream, nullptr);
    if (bn == 128) return launch_bn<OpA, OpB, AKC, BKC, 128, false>(a, b, epi, M, N, K, splits, k_chunk, stream, nullptr);
    return launch_bn<OpA, OpB, AKC, BKC, 256, false>(a, b, epi, M, N, K, splits, k_chunk, stream, nullptr);
}

// One warp waits, with a short limit, on a barrier that nothing ever arrives at: the wait runs out, the code 104 is
// recorded like any expired wait of the engine, and the kernel returns normally.  Exists so that the path
// "a bounded wait expired -> status word -> host" can be exercised without disturbing the GPU.
__global__ void wait_probe_kernel(unsigned long long cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait_for(smem_u32(&bar), 0u, cycles, 1u << 20)) atomicCAS(&g_tc_error, 0, 104);
}

// Tensor-pipe rate probe: every CTA (one per SM, 227 KB of shared memory so that no second one fits) issues
// `iterations` groups of 12 tcgen05.mma kind::tf32 128 x 256 x 8 on whatever its shared memory holds, with no loads
// and no epilogue, and waits (bounded) for the last commit.  2 * 128 * 256 * 8 * 12 * iterations * CTAs flops over the
// kernel's duration is what the tensor pipe sustains when nothing else limits it: the ceiling the contraction
// kernels are measured against (a product that is exact to fp32 costs three of these MMAs).
__global__ void __launch_bounds__(128, 1) mma_rate_probe_kernel(int iterations) {
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // operands: finite values (zeros) so that no NaN handling path is involved
    for (int i = threadIdx.x; i < (16384 + 32768) / 16; i += blockDim.x) reinterpret_cast<float4*>(tiles)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    if (warp == 1 && lane == 0) {
        const uint32_t a = smem_u32(tiles), b = a + 16384;
        for (int it = 0; it < iterations; ++it) {
#pragma unroll
            for (int j = 0; j < 12; ++j)
                mma_tf32(tmem_base, make_desc(a + (j & 3) * 32), make_desc(b + (j & 3) * 32), Config<256>::IDESC, (it | j) ? 1u : 0u);
        }
        mma_commit(smem_u32(&bar));
        if (!mbar_wait(smem_u32(&bar), 0u)) atomicCAS(&g_tc_error, 0, 105);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
    }
}

// Copies the error word to *dst (device memory or mapped pinned host memory) in stream order, without clearing it.
__global__ void publish_error_kernel(int* dst) { *dst = g_tc_error; }

// Reads and clears the device-side error word (synchronises the device).
inline int take_error(int* code) {
    int v = 0, zero = 0;
    VDNN_CUDA(cudaDeviceSynchronize());
    VDNN_CUDA(cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)));
    if (v != 0) VDNN_CUDA(cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int)));
    *code = v;
    return VDNN_OK;
}

}  // namespace tc
}  // namespace vdnn
