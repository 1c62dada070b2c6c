// Data-parallel plumbing: one NCCL communicator per process, resolved at run time from the NCCL
// shared library that is already in the process (or the system one).  The reference is
// single-device (vdnn.h:5); nothing here has a counterpart in it.
#ifndef VDNN_B200_DP_NCCL_H_
#define VDNN_B200_DP_NCCL_H_

#include <cuda_runtime.h>
#include <stddef.h>

struct vdnnContext;

namespace vdnn {
int dp_unique_id(char* out128);
int dp_init(vdnnContext* ctx, int rank, int world, const char* unique_id128);
int dp_allreduce_sum(vdnnContext* ctx, float* buf, size_t count, cudaStream_t stream);
int dp_map_peers(vdnnContext* ctx, cudaStream_t stream);
void dp_shutdown(vdnnContext* ctx);
}

#endif
