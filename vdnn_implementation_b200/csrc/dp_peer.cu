// Gradient all-reduce fused with the SGD step, over peer-mapped memory (NVLink / NVSwitch), for the data-parallel
// path: the alternative to ncclAllReduce + two axpy kernels per layer.  No counterpart in the reference (single device).
//
// Every rank keeps the gradients of all its layers in one arena that the other ranks of the box map into their own
// address space (CUDA IPC).  For one layer, every rank launches the same kernel on its communication stream as soon as
// that layer's backward has finished:
//   1. announce: write this step's epoch into every peer's "ready" flag for (layer, this rank);
//   2. wait (bounded) until all ranks have announced; then reduce slice `rank` of the gradient -- read it from every
//      rank's arena with plain loads, add in rank order (the same order everywhere: results are bit-identical across
//      ranks), write the sum back into every rank's arena with plain stores (a two-shot all-reduce: reduce-scatter by
//      loads, all-gather by stores);
//   3. the last CTA to finish announces "done" to every peer; all CTAs wait (bounded) until every rank is done, i.e. the
//      local arena holds the complete sum;
//   4. SGD: w += -lr * sum, b likewise, from the local arena.
// Flags only grow (epoch = step number), so nothing is reset between steps.  Every wait has a cycle limit; on expiry the
// CTA writes a code into the host-visible status word, skips its remaining work and returns.  No multimem, no TMA.
#include "common.cuh"
#include "dp_peer.h"

namespace vdnn {
namespace {

constexpr int THREADS = 256, BLOCKS = 64;

struct PeerTable { float* base[DP_MAX_RANKS]; int world, rank; };

__device__ __forceinline__ bool wait_flags(const volatile unsigned* flags, int world, unsigned epoch, unsigned long long cycles) {
    const unsigned long long t0 = clock64();
    for (int r = 0; r < world; ++r) {
        while (flags[r] < epoch) {
            if (clock64() - t0 > cycles) return false;
            __nanosleep(200);
        }
    }
    return true;
}

__global__ void __launch_bounds__(THREADS) peer_allreduce_sgd_kernel(PeerTable t, size_t off, size_t count, size_t slice_beg,
                                                                     size_t slice_end, int layer, unsigned epoch, float neg_lr,
                                                                     float* __restrict__ w, size_t wn, float* __restrict__ b,
                                                                     int* status_h, unsigned long long cycles) {
    __shared__ int failed;
    unsigned* mine = reinterpret_cast<unsigned*>(t.base[t.rank]);
    if (threadIdx.x == 0) failed = 0;
    // 1. this rank's gradient of the layer is complete (the kernel was enqueued behind the layer's backward)
    if (blockIdx.x == 0 && threadIdx.x < t.world) {
        __threadfence_system();
        reinterpret_cast<volatile unsigned*>(t.base[threadIdx.x])[DP_FLAG_READY + layer * DP_MAX_RANKS + t.rank] = epoch;
    }
    __syncthreads();
    // 2. everybody's is: reduce this rank's slice
    if (threadIdx.x == 0 && !wait_flags(mine + DP_FLAG_READY + layer * DP_MAX_RANKS, t.world, epoch, cycles)) {
        failed = 1;
        *status_h = 201;
    }
    __syncthreads();
    if (failed) return;
    __threadfence_system();
    for (size_t i = slice_beg / 4 + static_cast<size_t>(blockIdx.x) * THREADS + threadIdx.x; i < slice_end / 4;
         i += static_cast<size_t>(BLOCKS) * THREADS) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < t.world; ++r) {
            const float4 v = __ldcv(reinterpret_cast<const float4*>(t.base[r] + off) + i);       // never from a stale L1 line
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        for (int r = 0; r < t.world; ++r) reinterpret_cast<float4*>(t.base[r] + off)[i] = acc;
    }
    // 3. this rank's slice has been delivered everywhere once all its CTAs are through
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned prev = atomicAdd(mine + DP_FLAG_COUNTER + layer, 1u);
        if (prev == gridDim.x - 1) {
            atomicExch(mine + DP_FLAG_COUNTER + layer, 0u);
            __threadfence_system();
            for (int r = 0; r < t.world; ++r)
                reinterpret_cast<volatile unsigned*>(t.base[r])[DP_FLAG_DONE + layer * DP_MAX_RANKS + t.rank] = epoch;
        }
        if (!wait_flags(mine + DP_FLAG_DONE + layer * DP_MAX_RANKS, t.world, epoch, cycles)) {
            failed = 1;
            *status_h = 202;
        }
    }
    __syncthreads();
    if (failed) return;
    __threadfence_system();
    // 4. the SGD step from the local copy of the sum
    const float* g = t.base[t.rank] + off;
    for (size_t i = static_cast<size_t>(blockIdx.x) * THREADS + threadIdx.x; i < count; i += static_cast<size_t>(BLOCKS) * THREADS) {
        const float v = __ldcg(g + i);
        if (i < wn) w[i] = fmaf(neg_lr, v, w[i]);
        else b[i - wn] = fmaf(neg_lr, v, b[i - wn]);
    }
}

}  // namespace

void dp_slice(size_t count, int world, int rank, size_t* begin, size_t* end) {
    const size_t quads = (count + 3) / 4, per = (quads + world - 1) / world;
    const size_t b = per * rank < quads ? per * rank : quads;
    const size_t e = b + per < quads ? b + per : quads;
    *begin = b * 4;
    *end = e * 4;
}

int dp_peer_allreduce_sgd(float* const* arenas, int world, int rank, size_t offset_floats, size_t count, int layer,
                          unsigned epoch, float neg_lr, float* w, size_t wn, float* b, int* status_h, cudaStream_t stream) {
    if (world < 2 || world > DP_MAX_RANKS || rank < 0 || rank >= world || layer < 0 || layer >= DP_MAX_LAYERS || !status_h)
        return VDNN_ERR_BAD_ARG;
    PeerTable t;
    for (int r = 0; r < DP_MAX_RANKS; ++r) t.base[r] = r < world ? arenas[r] : nullptr;
    t.world = world; t.rank = rank;
    size_t beg = 0, end = 0;
    dp_slice(count, world, rank, &beg, &end);
    // waits give up after about two seconds
    peer_allreduce_sgd_kernel<<<BLOCKS, THREADS, 0, stream>>>(t, offset_floats, count, beg, end, layer, epoch, neg_lr, w, wn, b,
                                                              status_h, 4000000000ull);
    VDNN_LAUNCHED();
    return VDNN_OK;
}

}  // namespace vdnn

extern "C" int vdnn_dp_slice(size_t count, int world, int rank, size_t* begin, size_t* end) {
    if (world < 1 || rank < 0 || rank >= world || !begin || !end) return VDNN_ERR_BAD_ARG;
    vdnn::dp_slice(count, world, rank, begin, end);
    return VDNN_OK;
}
