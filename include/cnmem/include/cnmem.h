/*
 * Pool sub-allocator with the call interface of NVIDIA cnmem, written from scratch for this
 * library (the reference includes "./cnmem/include/cnmem.h" at layer.h:21 and links -lcnmem at
 * build.sh:2, but vendors neither).  Only the behaviour the reference relies on is implemented:
 * one device, one root pool reserved up front, 512-byte granularity, best-fit allocation with
 * coalescing on free, and "used = total - free" accounting (network.cu:1069,1098,1129,1176).
 * The stream arguments are accepted and ignored, as the reference always passes NULL.
 *
 * The vdnnPool* functions below the cnmem block are extensions used by the event-ordered
 * memory manager; the reference has no counterpart for them.
 */
#ifndef VDNN_B200_CNMEM_COMPAT_H_
#define VDNN_B200_CNMEM_COMPAT_H_

#include <stddef.h>
#include <stdio.h>
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    CNMEM_STATUS_SUCCESS = 0,
    CNMEM_STATUS_CUDA_ERROR,
    CNMEM_STATUS_INVALID_ARGUMENT,
    CNMEM_STATUS_NOT_INITIALIZED,
    CNMEM_STATUS_OUT_OF_MEMORY,
    CNMEM_STATUS_UNKNOWN_ERROR
} cnmemStatus_t;

typedef enum {
    CNMEM_FLAGS_DEFAULT = 0,
    CNMEM_FLAGS_CANNOT_GROW = 1,
    CNMEM_FLAGS_CANNOT_STEAL = 2,
    CNMEM_FLAGS_MANAGED = 4
} cnmemManagerFlags_t;

typedef struct cnmemDevice_t_ {
    int device;
    size_t size;
    int numStreams;
    cudaStream_t* streams;
    size_t* streamSizes;
} cnmemDevice_t;

/* network.cu:47-53, 113-118.  The requested size is clamped to the environment variable
 * VDNN_POOL_BYTES when that is set (the reference asks for the whole device). */
cnmemStatus_t cnmemInit(int numDevices, const cnmemDevice_t* devices, unsigned flags);
cnmemStatus_t cnmemFinalize(void);                                             /* network.cu:103 */
cnmemStatus_t cnmemMalloc(void** ptr, size_t size, cudaStream_t stream);       /* layer.cu:549,989-1011 */
cnmemStatus_t cnmemFree(void* ptr, cudaStream_t stream);                       /* network.cu:1095,1172 */
cnmemStatus_t cnmemMemGetInfo(size_t* freeMem, size_t* totalMem, cudaStream_t stream);
cnmemStatus_t cnmemPrintMemoryState(FILE* file, cudaStream_t stream);
cnmemStatus_t cnmemRegisterStream(cudaStream_t stream);
const char* cnmemGetErrorString(cnmemStatus_t status);                         /* layer.h:114 */

/* ---- extensions --------------------------------------------------------------------------- */
/* Same as cnmemFree, but remembers that the bytes are still in use on the device until everything
 * enqueued so far on each of `streams` has completed (the pool records a private event on each).  A later
 * allocation that lands on those bytes makes its streams wait for those events first, so the host can
 * free in the reference's order without synchronising. */
cnmemStatus_t vdnnPoolFreeAfter(void* ptr, const cudaStream_t* streams, int numStreams);
/* cnmemMalloc followed by cudaStreamWaitEvent(streams[i], e) for every pending event e that
 * covers part of the returned block.  Among the free blocks that fit, the one that becomes usable
 * soonest is chosen (no pending event, else the oldest pending events), then the tightest fit. */
cnmemStatus_t vdnnPoolMallocFor(void** ptr, size_t size, const cudaStream_t* streams, int numStreams);
/* The same with a hint: transient != 0 marks a block that is given back within the same layer call (workspace).  A pool
 * that is not packed places those at the end of a free range, highest address first, so that they do not cut the
 * ranges the long-lived tensors grow into.  Byte counts are the same. */
/* Keeps the top `bytes` of a pool that is not packed for transient blocks: other blocks go there only when they fit
 * nowhere else.  With the reserve at least as large as the largest workspace, that workspace always finds its bytes in
 * one piece, however the tensors below are spread by placement by pending events. */
cnmemStatus_t vdnnPoolSetTransientReserve(size_t bytes);
cnmemStatus_t vdnnPoolMallocKindFor(void** ptr, size_t size, const cudaStream_t* streams, int numStreams, int transient);
/* Same as vdnnPoolFreeAfter, for bytes whose last reader has not been enqueued yet (a copy that the
 * host will submit later, in an order of its own choosing).  The bytes count as free, but carry a "hold"
 * named by `token` (> 0).  vdnnPoolResolve(token, stream), called once that reader has been enqueued on
 * `stream`, turns the hold into an ordinary pending event.  Allocations avoid held bytes while anything
 * else fits; when only held bytes fit, the pool calls the resolver (lowest token first), which must
 * enqueue the reader and call vdnnPoolResolve for that token before it returns. */
typedef void (*vdnnPoolResolver_t)(void* user, unsigned long long token);
cnmemStatus_t vdnnPoolSetResolver(vdnnPoolResolver_t resolver, void* user);
cnmemStatus_t vdnnPoolFreeHeld(void* ptr, const cudaStream_t* streams, int numStreams, unsigned long long token);
cnmemStatus_t vdnnPoolResolve(unsigned long long token, cudaStream_t stream);
/* packed != 0: allocations take the tightest-fitting free block from its start, whatever events are pending on it
 * (the streams still wait for them): the placement of plain cnmemMalloc, and of the bookkeeping-only pool, so a
 * schedule that was replayed there fits here too.  Default 0: placement by pending events as described above. */
cnmemStatus_t vdnnPoolSetPacked(int packed);
cnmemStatus_t vdnnPoolHighWater(size_t* peakBytes, int reset);
/* Makes the k-th allocation from now fail with CNMEM_STATUS_OUT_OF_MEMORY (k >= 1; 0 disarms).
 * Host-side fault injection for the soft-OOM return path (layer.h:119-125). */
cnmemStatus_t vdnnPoolFailAfter(int k);
int vdnnPoolIsInitialized(void);
/* Size in bytes of the live block that starts at `ptr` (what the request was rounded up to). */
cnmemStatus_t vdnnPoolBlockBytes(const void* ptr, size_t* bytes);
/* Bookkeeping-only pool: hands out addresses from a range that is never backed by memory and
 * never dereferenced.  Lets the allocation schedule of a network be replayed on a machine
 * without a GPU (dry-run networks, allocator unit tests). */
cnmemStatus_t vdnnPoolInitVirtual(size_t size);

#ifdef __cplusplus
}
#endif
#endif
