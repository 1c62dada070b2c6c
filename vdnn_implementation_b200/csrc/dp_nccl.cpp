// NCCL binding for the gradient all-reduce (sum over ranks, fp32).  Sum, not mean: the filter and
// bias gradients of the single-device path are batch sums without a 1/N factor, so summing the
// per-rank gradients of a split batch reproduces exactly the update of one big batch.
#include "dp_nccl.h"

#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include <vector>

#include "dp_peer.h"
#include "layer.h"

namespace {

// Minimal slice of the NCCL ABI (stable across 2.x): 128-byte opaque id passed by value.
struct NcclUniqueId { char internal[128]; };
typedef void* NcclComm;
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(NcclComm*, int, NcclUniqueId, int);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, NcclComm, cudaStream_t);
typedef int (*CommDestroyFn)(NcclComm);
typedef const char* (*GetErrorStringFn)(int);
constexpr int kNcclFloat32 = 7, kNcclSum = 0, kNcclChar = 0;

struct Api {
    void* lib = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    AllReduceFn all_reduce = nullptr;
    AllGatherFn all_gather = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    GetErrorStringFn error_string = nullptr;
} g_api;

bool load_api() {
    if (g_api.lib) return true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);      // the copy torch already mapped, if any
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { fprintf(stderr, "libnccl.so.2 not found: %s\n", dlerror()); return false; }
    g_api.get_unique_id = reinterpret_cast<GetUniqueIdFn>(dlsym(h, "ncclGetUniqueId"));
    g_api.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(h, "ncclCommInitRank"));
    g_api.all_reduce = reinterpret_cast<AllReduceFn>(dlsym(h, "ncclAllReduce"));
    g_api.all_gather = reinterpret_cast<AllGatherFn>(dlsym(h, "ncclAllGather"));
    g_api.comm_destroy = reinterpret_cast<CommDestroyFn>(dlsym(h, "ncclCommDestroy"));
    g_api.error_string = reinterpret_cast<GetErrorStringFn>(dlsym(h, "ncclGetErrorString"));
    if (!g_api.get_unique_id || !g_api.comm_init_rank || !g_api.all_reduce || !g_api.comm_destroy) return false;
    g_api.lib = h;
    return true;
}

int fail(const char* what, int rc) {
    fprintf(stderr, "NCCL %s failed: %s\n", what, g_api.error_string ? g_api.error_string(rc) : "?");
    return VDNN_ERR_CUDA;
}

}  // namespace

namespace vdnn {

int dp_unique_id(char* out128) {
    if (!out128) return VDNN_ERR_BAD_ARG;
    if (!load_api()) return VDNN_ERR_UNSUPPORTED;
    NcclUniqueId id;
    const int rc = g_api.get_unique_id(&id);
    if (rc != 0) return fail("ncclGetUniqueId", rc);
    memcpy(out128, id.internal, 128);
    return VDNN_OK;
}

int dp_init(vdnnContext* ctx, int rank, int world, const char* unique_id128) {
    if (!unique_id128) return VDNN_ERR_BAD_ARG;
    if (!load_api()) return VDNN_ERR_UNSUPPORTED;
    NcclUniqueId id;
    memcpy(id.internal, unique_id128, 128);
    NcclComm comm = nullptr;
    const int rc = g_api.comm_init_rank(&comm, world, id, rank);
    if (rc != 0) return fail("ncclCommInitRank", rc);
    ctx->nccl_comm = comm;
    ctx->dp_rank = rank;
    ctx->dp_world = world;
    return VDNN_OK;
}

int dp_allreduce_sum(vdnnContext* ctx, float* buf, size_t count, cudaStream_t stream) {
    if (!ctx->nccl_comm) return VDNN_ERR_STATE;
    const int rc = g_api.all_reduce(buf, buf, count, kNcclFloat32, kNcclSum, ctx->nccl_comm, stream);
    return rc == 0 ? VDNN_OK : fail("ncclAllReduce", rc);
}

// Maps every rank's gradient arena into this process (CUDA IPC; all ranks are processes on one box).  The 64-byte IPC
// handles travel through an NCCL all-gather.  Fills ctx->dp_peer[]; any failure leaves the NCCL path in charge.
int dp_map_peers(vdnnContext* ctx, cudaStream_t stream) {
    if (!ctx->nccl_comm || !g_api.all_gather || !ctx->dp_arena) return VDNN_ERR_STATE;
    if (ctx->dp_world > vdnn::DP_MAX_RANKS) return VDNN_ERR_UNSUPPORTED;
    const int world = ctx->dp_world;
    cudaIpcMemHandle_t mine;
    if (cudaIpcGetMemHandle(&mine, ctx->dp_arena) != cudaSuccess) { (void)cudaGetLastError(); return VDNN_ERR_UNSUPPORTED; }
    char* d_buf = nullptr;
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    if (cudaMalloc(reinterpret_cast<void**>(&d_buf), hb * (world + 1)) != cudaSuccess) return VDNN_ERR_CUDA;
    std::vector<cudaIpcMemHandle_t> all(world);
    int st = VDNN_OK;
    if (cudaMemcpyAsync(d_buf + hb * world, &mine, hb, cudaMemcpyHostToDevice, stream) != cudaSuccess) st = VDNN_ERR_CUDA;
    if (st == VDNN_OK) {
        const int rc = g_api.all_gather(d_buf + hb * world, d_buf, hb, kNcclChar, ctx->nccl_comm, stream);
        if (rc != 0) st = fail("ncclAllGather", rc);
    }
    if (st == VDNN_OK && (cudaMemcpyAsync(all.data(), d_buf, hb * world, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
                          cudaStreamSynchronize(stream) != cudaSuccess))
        st = VDNN_ERR_CUDA;
    cudaFree(d_buf);
    if (st != VDNN_OK) return st;
    for (int r = 0; r < world; ++r) {
        if (r == ctx->dp_rank) { ctx->dp_peer[r] = ctx->dp_arena; continue; }
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            (void)cudaGetLastError();
            for (int q = 0; q < r; ++q)
                if (q != ctx->dp_rank && ctx->dp_peer[q]) { cudaIpcCloseMemHandle(ctx->dp_peer[q]); ctx->dp_peer[q] = nullptr; }
            return VDNN_ERR_UNSUPPORTED;
        }
        ctx->dp_peer[r] = static_cast<float*>(p);
    }
    return VDNN_OK;
}

void dp_shutdown(vdnnContext* ctx) {
    for (int r = 0; r < vdnn::DP_MAX_RANKS; ++r) {
        if (ctx->dp_peer[r] && r != ctx->dp_rank) cudaIpcCloseMemHandle(ctx->dp_peer[r]);
        ctx->dp_peer[r] = nullptr;
    }
    if (ctx->nccl_comm && g_api.comm_destroy) g_api.comm_destroy(ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
}

}  // namespace vdnn
