// Strip engine on CTA pairs (tcgen05.mma.cta_group::2): included at the end of conv_tma.cuh, inside vdnn::tma.
//
// What bounds the 128 x 256 strip kernel is the path from L2 into the SM, and 85 % of the bytes it pulls are weight
// tiles that every CTA fetches again.  A cluster of two CTAs on neighbouring SMs computes a tile of 256 positions x 256
// columns with one MMA: each CTA stages the strip of its own 128 positions and HALF of the weight tile (128 of the 256
// columns); the tensor cores of the pair read each other's half.  Per filter row and channel block a CTA then takes in
// 34 KB of strip + 3 x 32 KB of weights instead of 34 + 3 x 64.
//
// Protocol (same stage rings as strip_kernel, all waits bounded):
//   * both CTAs run a TMA producer for their own operands; every copy is a tensor copy with .cta_group::2 (no
//     multicast) whose completion bytes go to the LEADER's "full" barrier (rank 0 of the pair), which the leader's
//     producer arms with the bytes of both CTAs;
//   * one thread of the leader issues the MMAs for the pair; its commits arrive on the "empty" and "accumulator
//     ready" barriers of BOTH CTAs (tcgen05.commit with a CTA mask);
//   * each CTA drains the accumulator rows of its own 128 positions from its own tensor memory; the peer's drain
//     warps hand the buffer back with a remote arrive on the leader's "accumulator free" barrier;
//   * tensor memory is allocated and released by the same warp of both CTAs, with a cluster barrier before the
//     release; every thread of both CTAs reaches that barrier on every path (roles leave their loops, never the kernel).

namespace pair {

// BNP = columns of a pair tile (256, 128 or 64); each CTA stages BNP / 2 of them.
template <int BNP> struct PairCfg {
    static_assert(BNP == 256 || BNP == 128 || BNP == 64, "pair tiles of 256, 128 or 64 columns");
    static constexpr int HALF = BNP / 2;
    static constexpr int SA = 2, SB = 4;
    static constexpr int B_TILE_BYTES = HALF * BK * 4;                      // one half (hi or lo) of this CTA's columns
    static constexpr int A_STAGE_BYTES = 2 * STRIP_HALF_BYTES;
    static constexpr int B_STAGE_BYTES = 2 * B_TILE_BYTES;
    static constexpr int TMEM_COLS = 2 * BNP;
    static constexpr int CTAS_PER_SM = BNP == 64 ? 2 : 1;                   // as for single CTAs: two issuers per SM at 64 columns
    static constexpr int SMEM_BYTES = SA * A_STAGE_BYTES + SB * B_STAGE_BYTES + 1024 + 256;
    // instruction descriptor: D = F32, A = B = TF32, both K-major, N = BNP, M = 256 (128 rows in each CTA)
    static constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(BNP >> 3) << 17) |
                                      (static_cast<uint32_t>(256 >> 4) << 24);
};

__device__ __forceinline__ uint32_t cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tensor copy into this CTA's shared memory whose completion bytes go to a barrier that may live in the peer CTA.
__device__ __forceinline__ void tma_load_rows_2cta(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int row) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(row) : "memory");
}
__device__ __forceinline__ void mma_tf32_2cta(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// One 32-wide k block of the 3xTF32 product on the pair (order and descriptors as tc::mma_block_3xtf32; STEP = what a
// k slice adds to the descriptors' address field: 2 for K-major tiles, 64 for MN-major strips).
template <int STEP>
__device__ __forceinline__ void mma_block_3xtf32_2cta(uint32_t d_tmem, uint64_t dah, uint64_t dal, uint64_t dbh, uint64_t dbl, bool fresh,
                                                      uint32_t idesc) {
    mma_tf32_2cta(d_tmem, dal, dbh, idesc, fresh ? 0u : 1u);
    mma_tf32_2cta(d_tmem, dah, dbl, idesc, 1u);
    mma_tf32_2cta(d_tmem, dah, dbh, idesc, 1u);
#pragma unroll
    for (int ks = 1; ks < BK / 8; ++ks) {
        dah += STEP; dal += STEP; dbh += STEP; dbl += STEP;
        mma_tf32_2cta(d_tmem, dal, dbh, idesc, 1u);
        mma_tf32_2cta(d_tmem, dah, dbl, idesc, 1u);
        mma_tf32_2cta(d_tmem, dah, dbh, idesc, 1u);
    }
}
// Arrive on the barrier at this offset in both CTAs of the pair once the MMAs issued so far have completed.
__device__ __forceinline__ void mma_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}

template <int BNP>
__global__ void __launch_bounds__(THREADS, PairCfg<BNP>::CTAS_PER_SM)
strip_pair_kernel(const __grid_constant__ CUtensorMap map_hi, const __grid_constant__ CUtensorMap map_lo,
                  const __grid_constant__ CUtensorMap map_b, const StripParams p) {
    typedef PairCfg<BNP> Cfg;
    constexpr int SA = Cfg::SA, SB = Cfg::SB;
    constexpr int TILE_ROWS = 2 * BM;               // positions per pair tile
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    char* b_ring = tiles + SA * Cfg::A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(b_ring + SB * Cfg::B_STAGE_BYTES);
    uint64_t* a_full = bars;               // [SA]  used in the leader: bytes of both CTAs
    uint64_t* a_empty = a_full + SA;       // [SA]  in each CTA, from the leader's commits
    uint64_t* b_full = a_empty + SA;       // [SB]
    uint64_t* b_empty = b_full + SB;       // [SB]
    uint64_t* acc_ready = b_empty + SB;    // [2]   in each CTA
    uint64_t* acc_free = acc_ready + 2;    // [2]   used in the leader: drain warps of both CTAs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t rank = cta_rank();
    const bool leader = rank == 0;
    const unsigned pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int n0 = blockIdx.y * BNP;
    const long long num_tiles = (p.total_pos + TILE_ROWS - 1) / TILE_ROWS;
    const int g_beg = blockIdx.z * p.group_chunk;
    const int g_end = min(p.groups_total, g_beg + p.group_chunk);
    const int ngroups = g_beg < g_end ? g_end - g_beg : 0;
    const int nkb = ngroups * p.S;                     // k blocks per tile
    const int npairs = (nkb + 1) / 2;                  // accumulator hand-overs per tile
    const uint32_t strip_bytes = static_cast<uint32_t>(BM + p.S - 1) * BK * 4;

    if (t == 0) {
        for (int s = 0; s < SA; ++s) { tc::mbar_init(tc::smem_u32(&a_full[s]), 1); tc::mbar_init(tc::smem_u32(&a_empty[s]), 1); }
        for (int s = 0; s < SB; ++s) { tc::mbar_init(tc::smem_u32(&b_full[s]), 1); tc::mbar_init(tc::smem_u32(&b_empty[s]), 1); }
        for (int b = 0; b < 2; ++b) { tc::mbar_init(tc::smem_u32(&acc_ready[b]), 1); tc::mbar_init(tc::smem_u32(&acc_free[b]), 2 * DRAIN_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync();                                     // barriers of both CTAs initialised, tensor memory allocated
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp < DRAIN_WARPS) {
        // ------------------------------------------------------------------ accumulator drain + epilogue (own 128 rows)
        constexpr int NACC = BNP / (DRAIN_WARPS / 4);
        const int col_beg = (warp >> 2) * NACC;
        const uint32_t tmem_mine = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(col_beg);
        const size_t plane = static_cast<size_t>(p.out_h) * p.out_w;
        const uint32_t free0 = map_to_cta(tc::smem_u32(&acc_free[0]), 0), free1 = map_to_cta(tc::smem_u32(&acc_free[1]), 0);
        bool alive = true;
        unsigned pair = 0;
        for (long long tile = pair_id; tile < num_tiles && alive; tile += num_pairs) {
            float acc[NACC];
#pragma unroll
            for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;
            for (int pp = 0; pp < npairs && alive; ++pp, ++pair) {
                const int b = pair & 1;
                bool ok = tc::mbar_wait(tc::smem_u32(&acc_ready[b]), (pair >> 1) & 1u);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { atomicCAS(&tc::g_tc_error, 0, 103); alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c = 0; c < NACC; c += 16) {
                    float v[16];
                    tc::tmem_ld16(tmem_mine + static_cast<uint32_t>(b * BNP + c), v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[c + j] += v[j];
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(b ? free1 : free0);
            }
            const long long q = tile * TILE_ROWS + rank * BM + (warp & 3) * 32 + lane;
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
                        float v = p.alpha * acc[j];
                        if (p.bias) v += p.bias[col];
                        if (p.beta != 0.0f) v = fmaf(p.beta, *dst, v);
                        *dst = v;
                    } else if (p.mode == EPI_ATOMIC) {
                        atomicAdd(dst, p.alpha * acc[j]);
                    } else {
                        *dst = acc[j];
                    }
                }
            }
        }
    } else if (warp == DRAIN_WARPS) {
        // ------------------------------------------------------------------ TMA producer: own strip, own half of the weights
        if (lane == 0) {
            // rows of the weight tile images: per (column tile, k block) 256 rows of the hi half, then 256 of the lo half
            const long long b_row0 = static_cast<long long>(blockIdx.y) * p.kblocks_total * (2 * BNP) + rank * Cfg::HALF;
            unsigned i = 0, gcount = 0;
            bool ok = true;
            for (long long tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
                const long long m0 = tile * TILE_ROWS + rank * BM;
                for (int g = 0; g < ngroups && ok; ++g, ++gcount) {
                    const int group = g_beg + g;
                    const int r = group / p.cblocks, cb = group - r * p.cblocks;
                    const int sa = gcount % SA;
                    if (!tc::mbar_wait(tc::smem_u32(&a_empty[sa]), ((gcount / SA) & 1u) ^ 1u)) { ok = false; break; }
                    const long long row = m0 + static_cast<long long>(p.dh0 + p.dh_step * r) * p.wp + p.dw_min;
                    const uint32_t abar = map_to_cta(tc::smem_u32(&a_full[sa]), 0);
                    const uint32_t ast = tc::smem_u32(tiles + sa * Cfg::A_STAGE_BYTES);
                    if (leader)     // the strips of both CTAs complete on this barrier
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc::smem_u32(&a_full[sa])), "r"(4u * strip_bytes) : "memory");
                    tma_load_rows_2cta(ast, &map_hi, abar, cb * BK, static_cast<int>(row));
                    tma_load_rows_2cta(ast + STRIP_HALF_BYTES, &map_lo, abar, cb * BK, static_cast<int>(row));
                    for (int sx = 0; sx < p.S; ++sx, ++i) {
                        const int sb = i % SB;
                        if (!tc::mbar_wait(tc::smem_u32(&b_empty[sb]), ((i / SB) & 1u) ^ 1u)) { ok = false; break; }
                        const int kb = (r * p.S + sx) * p.cblocks + cb;
                        const uint32_t bbar = map_to_cta(tc::smem_u32(&b_full[sb]), 0);
                        const uint32_t bst = tc::smem_u32(b_ring + sb * Cfg::B_STAGE_BYTES);
                        if (leader)
                            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc::smem_u32(&b_full[sb])), "r"(2u * Cfg::B_STAGE_BYTES) : "memory");
                        const long long brow = b_row0 + static_cast<long long>(kb) * (2 * BNP);
                        tma_load_rows_2cta(bst, &map_b, bbar, 0, static_cast<int>(brow));
                        tma_load_rows_2cta(bst + Cfg::B_TILE_BYTES, &map_b, bbar, 0, static_cast<int>(brow + BNP));
                    }
                }
            }
            if (!ok) atomicCAS(&tc::g_tc_error, 0, 101);
        }
    } else if (lane == 0 && leader) {
        // ------------------------------------------------------------------ MMA issuer of the pair
        unsigned i = 0, gcount = 0, pair = 0;
        bool ok = true;
        for (long long tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
            int kb_in_tile = 0;
            for (int g = 0; g < ngroups && ok; ++g, ++gcount) {
                const int sa = gcount % SA;
                if (!tc::mbar_wait(tc::smem_u32(&a_full[sa]), (gcount / SA) & 1u)) { ok = false; break; }
                const uint32_t a_hi0 = tc::smem_u32(tiles + sa * Cfg::A_STAGE_BYTES);
                for (int sx = 0; sx < p.S; ++sx, ++i, ++kb_in_tile) {
                    const int sb = i % SB, b = pair & 1;
                    const bool first_of_pair = !(kb_in_tile & 1);
                    if (first_of_pair && pair >= 2 && !tc::mbar_wait(tc::smem_u32(&acc_free[b]), ((pair >> 1) - 1) & 1u)) { ok = false; break; }
                    if (!tc::mbar_wait(tc::smem_u32(&b_full[sb]), (i / SB) & 1u)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_hi = a_hi0 + static_cast<uint32_t>(p.row0 + p.row_step * sx) * (BK * 4);
                    const uint32_t a_lo = a_hi + STRIP_HALF_BYTES;
                    const uint32_t b_hi = tc::smem_u32(b_ring + sb * Cfg::B_STAGE_BYTES);
                    const uint32_t b_lo = b_hi + Cfg::B_TILE_BYTES;
                    mma_block_3xtf32_2cta<2>(tmem_base + static_cast<uint32_t>(b * BNP), tc::make_desc(a_hi), tc::make_desc(a_lo),
                                             tc::make_desc(b_hi), tc::make_desc(b_lo), first_of_pair, Cfg::IDESC);
                    mma_commit_both(tc::smem_u32(&b_empty[sb]));
                    if (sx == p.S - 1) mma_commit_both(tc::smem_u32(&a_empty[sa]));
                    if (!first_of_pair || kb_in_tile == nkb - 1) { mma_commit_both(tc::smem_u32(&acc_ready[b])); ++pair; }
                }
            }
        }
        if (!ok) atomicCAS(&tc::g_tc_error, 0, 102);
    }

    // both CTAs are through with each other's shared memory, barriers and tensor memory before either leaves
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync();
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
    }
}

// Same arguments as strip_launch_bn; the tile is 256 positions x BNP columns per CTA pair.
template <int BNP>
int strip_pair_launch(const Problem& q, const float* src, char* images, const char* b_tiles, float* out, const float* bias,
                      float alpha, float beta, int mode, size_t partial_stride, int splits, int group_chunk, cudaStream_t stream, bool prepare) {
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    typedef PairCfg<BNP> Cfg;
    auto kern = strip_pair_kernel<BNP>;
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
    p.inner = q.S; p.use_base_offset = 0;
    p.groups_total = q.R * p.cblocks;
    p.group_chunk = group_chunk;
    p.kblocks_total = q.R * q.S * p.cblocks;
    p.b_tiles = b_tiles;
    p.out = out; p.bias = bias; p.alpha = alpha; p.beta = beta; p.mode = mode; p.partial_stride = partial_stride;
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return VDNN_ERR_UNSUPPORTED;
    CUtensorMap map_hi, map_lo, map_b;
    const cuuint32_t elem[2] = {1u, 1u};
    {
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(q.cin), static_cast<cuuint64_t>(p.total_pos)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(q.cin) * 4};
        const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(BM + q.S - 1)};
        for (int half = 0; half < 2; ++half) {
            const CUresult r = enc(half ? &map_lo : &map_hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, half ? lo : hi, dims, strides, box, elem,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return VDNN_ERR_CUDA;
        }
    }
    const int ny = ceil_div(q.n_cols, BNP);
    {
        // the packed weight tiles as rows of 128 bytes (they are stored swizzled already: the copy must not swizzle again)
        const cuuint64_t rows = static_cast<cuuint64_t>(ny) * p.kblocks_total * (2 * BNP);
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(BK), rows};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(BK) * 4};
        const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(Cfg::HALF)};
        const CUresult r = enc(&map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<char*>(b_tiles), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return VDNN_ERR_CUDA;
    }
    if (prepare) {
        const int st = strip_prepare(q, src, images, stream);
        if (st != VDNN_OK) return st;
    }
    if (ny > 65535 || splits > 65535) return VDNN_ERR_UNSUPPORTED;
    // persistent along x: as many CTA pairs as the GPU holds at once
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cfg.gridDim = dim3(2 * (sm_count() / 2) * Cfg::CTAS_PER_SM, 1, 1);
    int resident = 0;
    if (cudaOccupancyMaxActiveClusters(&resident, kern, &cfg) != cudaSuccess || resident < 1) { (void)cudaGetLastError(); return VDNN_ERR_UNSUPPORTED; }
    const long long tiles = ceil_div<long long>(p.total_pos, 2 * BM);
    long long pairs = resident / (static_cast<long long>(ny) * splits);
    if (pairs < 1) pairs = 1;
    if (pairs > tiles) pairs = tiles;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), ny, splits);
    VDNN_CUDA(cudaLaunchKernelEx(&cfg, kern, map_hi, map_lo, map_b, p));
    VDNN_LAUNCHED();
    return VDNN_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// Filter gradient on CTA pairs: the two CTAs of a pair take neighbouring row tiles (128 rows = four (tap, channel block)
// groups each) of the same column tile and pixel range, so they need the same 256-filter slice of dy; each stages its
// own rows of x and half of that slice (four of the eight 32-filter boxes).  64 KB per CTA and k block instead of 96.
// BNP = filters per pair tile (256, 128 or 64); each CTA stages BNP / 2 of them (BNP / 64 boxes of 32).
template <int BNP> struct WgradCfg {
    static_assert(BNP == 256 || BNP == 128 || BNP == 64, "pair tiles of 256, 128 or 64 filters");
    static constexpr int HALF = BNP / 2;
    static constexpr int HALF_BOXES = HALF / 32;
    static constexpr int B_TILE_BYTES = HALF * BK * 4;
    static constexpr int STAGE_BYTES = 2 * A_TILE_BYTES + 2 * B_TILE_BYTES;                 // 64 / 48 / 40 KB
    static constexpr int S = BNP == 256 ? 3 : (BNP == 128 ? 4 : 5);
    static constexpr int TMEM_COLS = 2 * BNP;
    static constexpr int SMEM_BYTES = S * STAGE_BYTES + 1024 + 256;
    // D = F32, A = B = TF32, both MN-major, N = BNP, M = 256 (128 rows in each CTA)
    static constexpr uint32_t IDESC_MN = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) |
                                         (static_cast<uint32_t>(BNP >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
};

__device__ __forceinline__ void tma_load_box_2cta(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int x, int y, int n) {
    asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(x), "r"(y), "r"(n) : "memory");
}

template <int BNP>
__global__ void __launch_bounds__(THREADS, 1)
wgrad_pair_kernel(const __grid_constant__ CUtensorMap x_hi, const __grid_constant__ CUtensorMap x_lo,
                  const __grid_constant__ CUtensorMap dy_hi, const __grid_constant__ CUtensorMap dy_lo, const WgradParams p) {
    typedef WgradCfg<BNP> WCfg;
    constexpr int S = WCfg::S;
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + S * WCfg::STAGE_BYTES);
    uint64_t* full = bars;                  // [S]  used in the leader: bytes of both CTAs
    uint64_t* empty = full + S;             // [S]  in each CTA
    uint64_t* acc_ready = empty + S;        // [2]  in each CTA
    uint64_t* acc_free = acc_ready + 2;     // [2]  used in the leader: drain warps of both CTAs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t rank = cta_rank();
    const bool leader = rank == 0;
    const int n0 = blockIdx.y * BNP;
    const int box_beg = blockIdx.z * p.box_chunk;
    const int box_end = min(p.total_boxes, box_beg + p.box_chunk);
    const int nkb = box_beg < box_end ? box_end - box_beg : 0;
    const int npairs = (nkb + 1) / 2;

    if (t == 0) {
        for (int s = 0; s < S; ++s) { tc::mbar_init(tc::smem_u32(&full[s]), 1); tc::mbar_init(tc::smem_u32(&empty[s]), 1); }
        for (int b = 0; b < 2; ++b) { tc::mbar_init(tc::smem_u32(&acc_ready[b]), 1); tc::mbar_init(tc::smem_u32(&acc_free[b]), 2 * DRAIN_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(WCfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp < DRAIN_WARPS) {
        constexpr int NACC = BNP / (DRAIN_WARPS / 4);
        const int col_beg = (warp >> 2) * NACC;
        const uint32_t tmem_mine = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(col_beg);
        const uint32_t free0 = map_to_cta(tc::smem_u32(&acc_free[0]), 0), free1 = map_to_cta(tc::smem_u32(&acc_free[1]), 0);
        float acc[NACC];
#pragma unroll
        for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;
        bool alive = true;
        for (int pair = 0; pair < npairs && alive; ++pair) {
            const int b = pair & 1;
            bool ok = tc::mbar_wait(tc::smem_u32(&acc_ready[b]), static_cast<uint32_t>(pair >> 1) & 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { atomicCAS(&tc::g_tc_error, 0, 103); alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < NACC; c += 16) {
                float v[16];
                tc::tmem_ld16(tmem_mine + static_cast<uint32_t>(b * BNP + c), v);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c + j] += v[j];
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(b ? free1 : free0);
        }
        // this thread's row: row group (warp & 3) of this CTA's tile, channel `lane` of its block
        const int group = blockIdx.x * BOXES + (warp & 3);
        if (alive && group < p.row_groups) {
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
                        float v = p.alpha * acc[j];
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
    } else if (warp == DRAIN_WARPS) {
        if (lane == 0) {
            int gc[BOXES], gdy[BOXES], gdx[BOXES];
            int groups = 0;
#pragma unroll
            for (int j = 0; j < BOXES; ++j) {
                const int group = blockIdx.x * BOXES + j;
                if (group < p.row_groups) {
                    const int tap = group / p.cblocks, cb = group - tap * p.cblocks;
                    const int r = tap / p.taps_s, sx = tap - r * p.taps_s;
                    gc[j] = cb * 32; gdy[j] = r + p.off_h; gdx[j] = sx + p.off_w;
                    groups = j + 1;
                } else {
                    gc[j] = 0; gdy[j] = 0; gdx[j] = 0;
                }
            }
            // the peer's tile is the next one along x (the leader has the even tile of the pair)
            const int peer_first = (static_cast<int>(blockIdx.x) + 1) * BOXES;
            const int groups_peer = leader ? max(0, min(BOXES, p.row_groups - peer_first)) : 0;
            const int col_boxes = min(BNP, p.n_cols - n0) / 32;                         // of the pair
            const int box_first = leader ? 0 : WCfg::HALF_BOXES;                        // this CTA's boxes of the dy slice
            const int my_boxes = max(0, min(WCfg::HALF_BOXES, col_boxes - box_first));
            const uint32_t stage_tx = static_cast<uint32_t>(2 * (groups + groups_peer + col_boxes) * BOX_BYTES);    // armed by the leader
            for (int i = 0; i < nkb; ++i) {
                const int s = i % S;
                const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
                if (!tc::mbar_wait(tc::smem_u32(&empty[s]), phase ^ 1u)) { atomicCAS(&tc::g_tc_error, 0, 101); break; }
                uint32_t n, rem, by, bx;
                p.div_boxes_img.divmod(static_cast<uint32_t>(box_beg + i), n, rem);
                p.div_boxes_w.divmod(rem, by, bx);
                const int y0 = static_cast<int>(by) * p.bh, x0 = static_cast<int>(bx) << p.bw_log2;
                const uint32_t bar = map_to_cta(tc::smem_u32(&full[s]), 0);
                const uint32_t st = tc::smem_u32(tiles + s * WCfg::STAGE_BYTES);
                if (leader)
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc::smem_u32(&full[s])), "r"(stage_tx) : "memory");
#pragma unroll
                for (int j = 0; j < BOXES; ++j) {
                    if (j < groups) {
                        tma_load_box_2cta(st + j * BOX_BYTES, &x_hi, bar, gc[j], x0 + gdx[j], y0 + gdy[j], static_cast<int>(n));
                        tma_load_box_2cta(st + A_TILE_BYTES + j * BOX_BYTES, &x_lo, bar, gc[j], x0 + gdx[j], y0 + gdy[j], static_cast<int>(n));
                    }
                }
                for (int j = 0; j < my_boxes; ++j) {
                    const int c0 = n0 + (box_first + j) * 32;
                    tma_load_box_2cta(st + 2 * A_TILE_BYTES + j * BOX_BYTES, &dy_hi, bar, c0, x0, y0, static_cast<int>(n));
                    tma_load_box_2cta(st + 2 * A_TILE_BYTES + WCfg::B_TILE_BYTES + j * BOX_BYTES, &dy_lo, bar, c0, x0, y0, static_cast<int>(n));
                }
            }
        }
    } else if (lane == 0 && leader) {
        for (int i = 0; i < nkb; ++i) {
            const int s = i % S, pair = i >> 1, b = pair & 1;
            const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
            if (!(i & 1) && pair >= 2 && !tc::mbar_wait(tc::smem_u32(&acc_free[b]), static_cast<uint32_t>((pair >> 1) - 1) & 1u)) {
                atomicCAS(&tc::g_tc_error, 0, 102);
                break;
            }
            if (!tc::mbar_wait(tc::smem_u32(&full[s]), phase)) { atomicCAS(&tc::g_tc_error, 0, 102); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = tc::smem_u32(tiles + s * WCfg::STAGE_BYTES);
            const uint32_t a_lo = a_hi + A_TILE_BYTES;
            const uint32_t b_hi = a_hi + 2 * A_TILE_BYTES;
            const uint32_t b_lo = b_hi + WCfg::B_TILE_BYTES;
            // one k slice = 8 pixels = 1024 bytes further into every strip
            mma_block_3xtf32_2cta<1024 / 16>(tmem_base + static_cast<uint32_t>(b * BNP), make_desc_mn(a_hi), make_desc_mn(a_lo),
                                             make_desc_mn(b_hi), make_desc_mn(b_lo), !(i & 1), WCfg::IDESC_MN);
            mma_commit_both(tc::smem_u32(&empty[s]));
            if ((i & 1) || i == nkb - 1) mma_commit_both(tc::smem_u32(&acc_ready[b]));
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync();
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(WCfg::TMEM_COLS) : "memory");
    }
}

// Launch of the pair kernel on the grid of the single-CTA kernel with x rounded up to whole pairs.
template <int BNP>
int wgrad_pair_launch(const CUtensorMap& mxh, const CUtensorMap& mxl, const CUtensorMap& myh, const CUtensorMap& myl,
                      const WgradParams& p, unsigned row_tiles, unsigned col_tiles, unsigned splits, cudaStream_t stream) {
    typedef WgradCfg<BNP> WCfg;
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    auto kern = wgrad_pair_kernel<BNP>;
    if (VDNN_ONCE_PER_DEVICE(dev))
        VDNN_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WCfg::SMEM_BYTES));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3((row_tiles + 1u) / 2u * 2u, col_tiles, splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = WCfg::SMEM_BYTES;
    cfg.stream = stream;
    cfg.attrs = attr; cfg.numAttrs = 1;
    VDNN_CUDA(cudaLaunchKernelEx(&cfg, kern, mxh, mxl, myh, myl, p));
    VDNN_LAUNCHED();
    return VDNN_OK;
}

}  // namespace pair
