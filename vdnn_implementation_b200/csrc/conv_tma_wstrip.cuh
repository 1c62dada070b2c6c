// Filter gradient on the strip engine's position lists: included from conv_tma.cuh, inside vdnn::tma.
//
//   dw[k][c][r][s] = sum over positions q of dy[q][k] * x[q + (r - pad_h) * wp + (s - pad_w)][c]
//
// Both tensors lie as padded position lists (rows wp positions apart, zero gaps: see strip_geometry) with the SAME
// pitch, so the sum may run over all positions (dy is zero in the gaps) and a filter tap is a constant shift of the x
// list.  The reduction runs over positions, so both operands are MN-major for the tensor core (one position = one
// 128-byte row of 32 channels, TMA swizzle 128B_ATOM_32B as in wgrad_kernel).  What this layout buys: the S taps of a
// filter row are the SAME strip of 32 + S - 1 positions read from S starting rows, and the four 32-row groups of an
// MMA's 128 rows may start any number of bytes apart (the descriptor's leading-dimension stride) -- 128 bytes = one
// position here.  A 128-row tile is therefore (filter row r, channel block cb) with its rows = taps s = 0 .. 3 of that
// filter row (the groups past S are computed and dropped), fed by ONE strip of 4.4 KB per image half instead of one
// 4 KB box per tap: a third of the bytes for 3 x 3 filters.  A CTA takes RT such tiles (consecutive (cb, r)) against one
// slice of dy, which they share.
//
// Needs: stride 1, S <= 4, and the input and output grids in one padded geometry (3 x 3 / pad 1 and the like).

struct WstripParams {
    long long total_pos;                 // positions of the lists (images * lp)
    int wp;                              // positions per padded row
    int R, S, cblocks;                   // filter rows, taps per row, 32-channel blocks of x
    int off_h, off_w;                    // x position of dy position q under tap (r, s): q + (r + off_h) * wp + (s + off_w)
    int tiles;                           // R * cblocks row tiles, tile t = (cb = t / R, r = t % R)
    int kb_total, kb_chunk;              // 32-position blocks of the reduction, and how many of them one split walks
    int C, n_cols;                       // dw is [n_cols][C][R * S]
    float* out;
    float alpha, beta;
    int mode;
    size_t partial_stride;
};

constexpr int WSTRIP_A_HALF = 5 * 1024;          // 32 + 3 rows of 128 bytes, padded to whole kilobytes (the junk group reads on)

// CPS = CTAs per SM: with 64 filters the MMAs are short and one issuing thread per SM is the limit (as in the forward
// kernel), so two CTAs of two tiles each share an SM.
template <int BN, int RT> struct WstripConfig {
    static_assert(2 * RT * BN <= 512, "the accumulators of RT tiles, twice, must fit the tensor memory");
    static constexpr int CPS = (2 * RT * BN <= 256) ? 2 : 1;
    static constexpr int B_TILE_BYTES = BN * BK * 4;
    static constexpr int A_BYTES = RT * 2 * WSTRIP_A_HALF;
    static constexpr int STAGE_BYTES = A_BYTES + 2 * B_TILE_BYTES;
    static constexpr int SMEM_BUDGET = (CPS == 2 ? 108 : 200) * 1024;
    static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES > 6 ? 6 : SMEM_BUDGET / STAGE_BYTES;
    static constexpr int TMEM_COLS = (2 * RT * BN <= 128) ? 128 : (2 * RT * BN <= 256 ? 256 : 512);
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
    static constexpr uint32_t IDESC_MN = tc::Config<BN>::IDESC | (1u << 15) | (1u << 16);
};

// MN-major descriptor (see make_desc_mn) with the stride between an operand's 32-wide strips given in bytes.
__device__ __forceinline__ uint64_t make_desc_mn_lbo(uint32_t saddr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
    d |= static_cast<uint64_t>(512 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(1) << 61;
    return d;
}

template <int BN, int RT>
__global__ void __launch_bounds__(THREADS, WstripConfig<BN, RT>::CPS)
wgrad_strip_kernel(const __grid_constant__ CUtensorMap x_hi, const __grid_constant__ CUtensorMap x_lo,
                   const __grid_constant__ CUtensorMap dy_hi, const __grid_constant__ CUtensorMap dy_lo, const WstripParams p) {
    typedef WstripConfig<BN, RT> Cfg;
    constexpr int S = Cfg::STAGES;
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + S * Cfg::STAGE_BYTES);
    uint64_t* full = bars;                  // [S]
    uint64_t* empty = full + S;             // [S]
    uint64_t* acc_ready = empty + S;        // [2]
    uint64_t* acc_free = acc_ready + 2;     // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int tile0 = blockIdx.x * RT;                       // first row tile of this CTA
    const int my_tiles = min(RT, p.tiles - tile0);
    const int n0 = blockIdx.y * BN;
    const int kb_beg = blockIdx.z * p.kb_chunk;
    const int kb_end = min(p.kb_total, kb_beg + p.kb_chunk);
    const int nkb = kb_beg < kb_end ? kb_end - kb_beg : 0;
    const int npairs = (nkb + 1) / 2;

    if (t == 0) {
        for (int s = 0; s < S; ++s) { tc::mbar_init(tc::smem_u32(&full[s]), 1); tc::mbar_init(tc::smem_u32(&empty[s]), 1); }
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
        constexpr int NACC = BN / (DRAIN_WARPS / 4);
        const int col_beg = (warp >> 2) * NACC;
        const uint32_t tmem_mine = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(col_beg);
        float acc[RT][NACC];
#pragma unroll
        for (int h = 0; h < RT; ++h)
#pragma unroll
            for (int j = 0; j < NACC; ++j) acc[h][j] = 0.0f;
        bool alive = true;
        for (int pair = 0; pair < npairs && alive; ++pair) {
            const int b = pair & 1;
            bool ok = tc::mbar_wait(tc::smem_u32(&acc_ready[b]), static_cast<uint32_t>(pair >> 1) & 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { atomicCAS(&tc::g_tc_error, 0, 103); alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < RT; ++h)
#pragma unroll
                for (int c = 0; c < NACC; c += 16) {
                    float v[16];
                    tc::tmem_ld16(tmem_mine + static_cast<uint32_t>((b * RT + h) * BN + c), v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[h][c + j] += v[j];
                }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(&acc_free[b]));
        }
        // this thread's rows: tap s = warp & 3 of every tile's filter row, channel `lane` of its block
        const int sx = warp & 3;
#pragma unroll
        for (int h = 0; h < RT; ++h) {
            if (!alive || h >= my_tiles || sx >= p.S) continue;
            const int tile = tile0 + h, cb = tile / p.R, r = tile - cb * p.R;
            const int taps = p.R * p.S;
            const size_t crs = static_cast<size_t>(p.C) * taps;
            float* o = p.out + static_cast<size_t>(cb * 32 + lane) * taps + r * p.S + sx;
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
            const int col_boxes = min(BN, p.n_cols - n0) / 32;
            const uint32_t strip_bytes = static_cast<uint32_t>(32 + p.S - 1) * BK * 4;
            const uint32_t stage_tx = static_cast<uint32_t>(my_tiles) * 2u * strip_bytes + static_cast<uint32_t>(2 * col_boxes * BOX_BYTES);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % S;
                const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
                if (!tc::mbar_wait(tc::smem_u32(&empty[s]), phase ^ 1u)) { atomicCAS(&tc::g_tc_error, 0, 101); break; }
                const long long q0 = static_cast<long long>(kb_beg + i) * 32;           // first dy position of the block
                const uint32_t bar = tc::smem_u32(&full[s]);
                const uint32_t st = tc::smem_u32(tiles + s * Cfg::STAGE_BYTES);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(stage_tx) : "memory");
                for (int h = 0; h < my_tiles; ++h) {
                    const int tile = tile0 + h, cb = tile / p.R, r = tile - cb * p.R;
                    const long long row = q0 + static_cast<long long>(r + p.off_h) * p.wp + p.off_w;
                    tma_load_rows(st + h * 2 * WSTRIP_A_HALF, &x_hi, bar, cb * 32, static_cast<int>(row));
                    tma_load_rows(st + h * 2 * WSTRIP_A_HALF + WSTRIP_A_HALF, &x_lo, bar, cb * 32, static_cast<int>(row));
                }
                for (int j = 0; j < col_boxes; ++j) {
                    tma_load_rows(st + Cfg::A_BYTES + j * BOX_BYTES, &dy_hi, bar, n0 + j * 32, static_cast<int>(q0));
                    tma_load_rows(st + Cfg::A_BYTES + Cfg::B_TILE_BYTES + j * BOX_BYTES, &dy_lo, bar, n0 + j * 32, static_cast<int>(q0));
                }
            }
        }
    } else if (lane == 0) {
        for (int i = 0; i < nkb; ++i) {
            const int s = i % S, pair = i >> 1, b = pair & 1;
            const uint32_t phase = static_cast<uint32_t>(i / S) & 1u;
            if (!(i & 1) && pair >= 2 && !tc::mbar_wait(tc::smem_u32(&acc_free[b]), static_cast<uint32_t>((pair >> 1) - 1) & 1u)) {
                atomicCAS(&tc::g_tc_error, 0, 102);
                break;
            }
            if (!tc::mbar_wait(tc::smem_u32(&full[s]), phase)) { atomicCAS(&tc::g_tc_error, 0, 102); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a0 = tc::smem_u32(tiles + s * Cfg::STAGE_BYTES);
            const uint32_t b_hi = a0 + Cfg::A_BYTES;
            const uint32_t b_lo = b_hi + Cfg::B_TILE_BYTES;
            const uint64_t dbh = make_desc_mn(b_hi), dbl = make_desc_mn(b_lo);
            for (int h = 0; h < my_tiles; ++h) {        // the tiles share the dy slice
                const uint32_t a_hi = a0 + h * 2 * WSTRIP_A_HALF, a_lo = a_hi + WSTRIP_A_HALF;
                // the four 32-row groups of the tile start one position (128 bytes) apart: taps s = 0 .. 3; one k slice =
                // 8 positions = 1024 bytes further
                tc::mma_block_3xtf32<1024 / 16>(tmem_base + static_cast<uint32_t>((b * RT + h) * BN), make_desc_mn_lbo(a_hi, 128),
                                                make_desc_mn_lbo(a_lo, 128), dbh, dbl, Cfg::IDESC_MN, !(i & 1));
            }
            tc::mma_commit(tc::smem_u32(&empty[s]));
            if ((i & 1) || i == nkb - 1) tc::mma_commit(tc::smem_u32(&acc_ready[b]));
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == DRAIN_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
    }
}

// Geometry test: the filter gradient may run on the two position lists.
inline bool wstrip_ok(const Problem& fwd, const Problem& dgrad) {
    const StripGeom a = strip_geometry(fwd), b = strip_geometry(dgrad);
    return a.ok && b.ok && a.wp == b.wp && a.lp == b.lp && fwd.S <= 4 && fwd.in_h == dgrad.in_h && fwd.in_w == dgrad.in_w;
}

// Reduction split: as many splits as fill two waves of CTAs, at least four 32-position blocks each.
template <int BN, int RT>
void wstrip_plan(int tiles, int n_cols, int kb_total, int* splits, int* kb_chunk) {
    const long ctas = static_cast<long>(ceil_div(tiles, RT)) * ceil_div(n_cols, BN);
    long s = (2L * sm_count() * WstripConfig<BN, RT>::CPS) / ctas;
    if (s > kb_total / 4) s = kb_total / 4;
    if (s > 1024) s = 1024;
    if (s < 1) s = 1;
    *kb_chunk = ceil_div(kb_total, static_cast<int>(s));
    *splits = ceil_div(kb_total, *kb_chunk);
}

template <int BN, int RT>
size_t wstrip_partial_bytes_bn(const Problem& fwd, int n_filters) {
    const StripGeom g = strip_geometry(fwd);
    const int kb_total = static_cast<int>((static_cast<long long>(fwd.n) * g.lp + 31) / 32);
    int splits, chunk;
    wstrip_plan<BN, RT>(fwd.R * (fwd.cin / 32), n_filters, kb_total, &splits, &chunk);
    return splits > 1 ? static_cast<size_t>(splits) * n_filters * fwd.cin * fwd.R * fwd.S * sizeof(float) : 0;
}

// x_images / dy_images: the strip images (hi then lo) of `fwd.n` images as strip_prepare writes them for the forward and
// the data-gradient problem of the layer.  partial: wstrip_partial_bytes() bytes.
template <int BN, int RT>
int wstrip_launch_bn(const Problem& fwd, int n_filters, const char* x_images, const char* dy_images, float* partial, float* dw,
                     float alpha, float beta, cudaStream_t stream, int* splits_out) {
    typedef WstripConfig<BN, RT> Cfg;
    int dev = 0;
    VDNN_CUDA(cudaGetDevice(&dev));
    auto kern = wgrad_strip_kernel<BN, RT>;
    if (VDNN_ONCE_PER_DEVICE(dev))
        VDNN_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    const StripGeom g = strip_geometry(fwd);
    WstripParams p;
    p.total_pos = static_cast<long long>(fwd.n) * g.lp;
    p.wp = g.wp;
    p.R = fwd.R; p.S = fwd.S; p.cblocks = fwd.cin / 32;
    p.off_h = fwd.off_h; p.off_w = fwd.off_w;
    p.tiles = p.R * p.cblocks;
    p.kb_total = static_cast<int>((p.total_pos + 31) / 32);
    int splits = 1;
    wstrip_plan<BN, RT>(p.tiles, n_filters, p.kb_total, &splits, &p.kb_chunk);
    p.C = fwd.cin; p.n_cols = n_filters;
    p.partial_stride = static_cast<size_t>(n_filters) * fwd.cin * fwd.R * fwd.S;
    if (splits > 1) { p.out = partial; p.alpha = 1.0f; p.beta = 0.0f; p.mode = EPI_PARTIAL; }
    else { p.out = dw; p.alpha = alpha; p.beta = beta; p.mode = EPI_DIRECT; }
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return VDNN_ERR_UNSUPPORTED;
    CUtensorMap maps[4];
    const cuuint32_t elem[2] = {1u, 1u};
    for (int m = 0; m < 4; ++m) {
        const bool is_x = m < 2;
        const int ch = is_x ? fwd.cin : n_filters;
        const float* base = reinterpret_cast<const float*>(is_x ? x_images : dy_images) + ((m & 1) ? static_cast<size_t>(p.total_pos) * ch : 0);
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(ch), static_cast<cuuint64_t>(p.total_pos)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ch) * 4};
        const cuuint32_t box[2] = {32u, static_cast<cuuint32_t>(is_x ? 32 + fwd.S - 1 : 32)};
        const CUresult r = enc(&maps[m], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return VDNN_ERR_CUDA;
    }
    dim3 grid(ceil_div(p.tiles, RT), ceil_div(n_filters, BN), splits);
    if (grid.y > 65535u || grid.z > 65535u) return VDNN_ERR_UNSUPPORTED;
    kern<<<grid, THREADS, Cfg::SMEM_BYTES, stream>>>(maps[0], maps[1], maps[2], maps[3], p);
    VDNN_LAUNCHED();
    *splits_out = splits;
    return VDNN_OK;
}

// Where this kernel is the faster filter gradient (measured, B200, batch 128, data + filter gradient of the layer):
// 64 -> 64 @ 224 x 224 7.87 ms against 8.91 with one box per tap; 64 -> 128 @ 112 x 112 3.38 / 3.49; 128 -> 128 @ 112 x 112
// 5.67 / 5.52 (there the 128-filter tile with two halves wins).  So: 64-filter tiles, and 128-filter tiles of layers with
// at most 64 input channels.
inline bool wstrip_filters_ok(int n_filters, int cin) {
    const int bn = tc::tile_n(n_filters);
    return bn == 64 || (bn == 128 && cin <= 64);
}

inline size_t wstrip_partial_bytes(const Problem& fwd, int n_filters) {
    return tc::tile_n(n_filters) == 64 ? wstrip_partial_bytes_bn<64, 2>(fwd, n_filters) : wstrip_partial_bytes_bn<128, 2>(fwd, n_filters);
}

inline int wstrip_launch(const Problem& fwd, int n_filters, const char* x_images, const char* dy_images, float* partial, float* dw,
                         float alpha, float beta, cudaStream_t stream, int* splits) {
    if (tc::tile_n(n_filters) == 64) return wstrip_launch_bn<64, 2>(fwd, n_filters, x_images, dy_images, partial, dw, alpha, beta, stream, splits);
    return wstrip_launch_bn<128, 2>(fwd, n_filters, x_images, dy_images, partial, dw, alpha, beta, stream, splits);
}
