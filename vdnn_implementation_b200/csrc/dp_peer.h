// Fused peer all-reduce + SGD of the data-parallel path (dp_peer.cu) and the layout of the gradient arena it works on.
#ifndef VDNN_B200_DP_PEER_H_
#define VDNN_B200_DP_PEER_H_

#include <cuda_runtime.h>
#include <stddef.h>

namespace vdnn {

constexpr int DP_MAX_RANKS = 8, DP_MAX_LAYERS = 40;
// The arena starts with DP_FLAG_WORDS 32-bit words of flags (peers write "ready" and "done" epochs per layer and source
// rank; a local counter per layer finds the last CTA), then the layers' gradient staging buffers.
constexpr int DP_FLAG_READY = 0, DP_FLAG_DONE = DP_MAX_LAYERS * DP_MAX_RANKS, DP_FLAG_COUNTER = 2 * DP_MAX_LAYERS * DP_MAX_RANKS;
constexpr int DP_FLAG_WORDS = 1024;

// Slice of a `count`-float gradient that rank `rank` reduces: whole groups of 4 floats, [begin, end) in floats (end may
// pass `count` by up to 3: staging buffers are padded to a multiple of 4).
void dp_slice(size_t count, int world, int rank, size_t* begin, size_t* end);

// Enqueues the fused kernel for one layer.  arenas[r] = base of rank r's arena as mapped in this process.
int dp_peer_allreduce_sgd(float* const* arenas, int world, int rank, size_t offset_floats, size_t count, int layer, unsigned epoch,
                          float neg_lr, float* w, size_t wn, float* b, int* status_h, cudaStream_t stream);

}  // namespace vdnn

#endif
