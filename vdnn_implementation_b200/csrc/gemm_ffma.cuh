// FFMA contraction engine: 128x128x8 block tile, 256 threads, 8x8 register tile per thread,
// operands gathered straight from the NCHW / KCRS tensors (see gemm_operands.cuh), global loads
// of the next k step in flight while the current one is multiplied, optional split along K
// (blockIdx.z).  Exact fp32 multiply-add: this is the engine used for shapes the tensor-core
// engine does not take, and the numerical cross-check for it.
#pragma once

#include "gemm_operands.cuh"

namespace vdnn {
namespace ffma {

constexpr int BM = 128, BN = 128, BK = 8, THREADS = 256, LDS = BM + 4;

// Moves one 128 x 8 operand tile from global memory to shared memory [k][row].
//   K_CONTIG = true : consecutive threads walk k      (operand is contiguous along k)
//   K_CONTIG = false: consecutive threads walk rows   (operand is contiguous along its rows)
template <class Op, bool K_CONTIG>
struct TileLoader {
    typename Op::Row rows[K_CONTIG ? 4 : 1];
    float v[4];

    __device__ __forceinline__ void init(const Op& op, int row0) {
        if (K_CONTIG) {
#pragma unroll
            for (int j = 0; j < 4; ++j) rows[j] = op.row(row0 + (threadIdx.x >> 3) + 32 * j);
        } else {
            rows[0] = op.row(row0 + (threadIdx.x & 127));
        }
    }
    __device__ __forceinline__ void fetch(const Op& op, int k0, int kend) {
        if (K_CONTIG) {
            const int kk = k0 + (threadIdx.x & 7);
            typename Op::Col c = op.col(kk);
            c.valid = c.valid && kk < kend;
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = op.load(rows[j], c);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kk = k0 + (threadIdx.x >> 7) + 2 * j;
                typename Op::Col c = op.col(kk);
                c.valid = c.valid && kk < kend;
                v[j] = op.load(rows[0], c);
            }
        }
    }
    __device__ __forceinline__ void stash(float (*smem)[LDS]) const {
        if (K_CONTIG) {
#pragma unroll
            for (int j = 0; j < 4; ++j) smem[threadIdx.x & 7][(threadIdx.x >> 3) + 32 * j] = v[j];
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) smem[(threadIdx.x >> 7) + 2 * j][threadIdx.x & 127] = v[j];
        }
    }
};

template <class OpA, class OpB, bool A_KC, bool B_KC>
__global__ void __launch_bounds__(THREADS, 2)
gemm_kernel(const OpA opa, const OpB opb, const Epilogue epi, int M, int N, int K, int k_chunk) {
    __shared__ __align__(16) float As[2][BK][LDS];
    __shared__ __align__(16) float Bs[2][BK][LDS];

    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int kbeg = blockIdx.z * k_chunk;
    const int kend = min(K, kbeg + k_chunk);

    TileLoader<OpA, A_KC> la;
    TileLoader<OpB, B_KC> lb;
    la.init(opa, m0);
    lb.init(opb, n0);

    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    if (kbeg < kend) {
        la.fetch(opa, kbeg, kend);
        lb.fetch(opb, kbeg, kend);
        la.stash(As[0]);
        lb.stash(Bs[0]);
    }
    __syncthreads();

    int buf = 0;
    for (int k0 = kbeg; k0 < kend; k0 += BK) {
        const bool more = k0 + BK < kend;
        if (more) {
            la.fetch(opa, k0 + BK, kend);
            lb.fetch(opb, k0 + BK, kend);
        }
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) {
            la.stash(As[buf ^ 1]);
            lb.stash(Bs[buf ^ 1]);
        }
        __syncthreads();
        buf ^= 1;
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= M) continue;
        const int roff = epi.row_off(m);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (n < N) epi.store(roff, n, acc[i][j], blockIdx.z);
        }
    }
}

// k_chunk must be a multiple of BK; splits = ceil(K / k_chunk) (see plan_split in conv_api.cu).
template <class OpA, class OpB, bool A_KC, bool B_KC>
int launch(const OpA& a, const OpB& b, const Epilogue& epi, int M, int N, int K, int splits, int k_chunk,
           cudaStream_t stream) {
    dim3 grid(ceil_div(M, BM), ceil_div(N, BN), splits);
    if (grid.y > 65535u || grid.z > 65535u) return VDNN_ERR_UNSUPPORTED;
    gemm_kernel<OpA, OpB, A_KC, B_KC><<<grid, THREADS, 0, stream>>>(a, b, epi, M, N, K, k_chunk);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

}  // namespace ffma
}  // namespace vdnn
