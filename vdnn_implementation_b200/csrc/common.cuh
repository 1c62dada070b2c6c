// Shared helpers for the sm_100a kernels: status plumbing, launch sizing, fast integer division.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "vdnn_b200.h"

namespace vdnn {

// Last failing runtime call of this thread, reported by vdnn_last_cuda_error().
extern thread_local int g_last_cuda_error;
// Launch counter (all kernels of this library), reported through vdnn_network_stats.
extern unsigned long long g_kernel_launches;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = static_cast<int>(e);
    (void)cudaGetLastError();
    return VDNN_ERR_CUDA;
}

#define VDNN_CUDA(call)                                              \
    do {                                                             \
        cudaError_t _e = (call);                                     \
        if (_e != cudaSuccess) return ::vdnn::cuda_fail(_e);         \
    } while (0)

// After a <<<>>> launch: count it and surface launch-configuration errors.
#define VDNN_LAUNCHED()                                              \
    do {                                                             \
        ++::vdnn::g_kernel_launches;                                 \
        cudaError_t _e = cudaPeekAtLastError();                      \
        if (_e != cudaSuccess) return ::vdnn::cuda_fail(_e);         \
    } while (0)

// B200 has 148 SMs; grids of the bandwidth kernels are sized in whole multiples of the SM count
// (queried once per device) so that every SM gets the same number of resident blocks.
int sm_count();

// True exactly once per device and call site (`seen` is the site's own table): kernels raise their dynamic shared
// memory limit the first time they run on a device.  The table grows with the device ordinal.
bool first_use_on_device(void** seen_table, int device);
#define VDNN_ONCE_PER_DEVICE(dev) ([&]() { static void* _tbl = nullptr; return ::vdnn::first_use_on_device(&_tbl, (dev)); }())

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

template <typename T>
__host__ __device__ constexpr T ceil_div(T a, T b) { return (a + b - 1) / b; }

// Division by a run-time constant with one mul.hi (valid for dividends below 2^31).
struct FastDiv {
    uint32_t d, mul, shr;
    FastDiv() : d(1), mul(0), shr(0) {}
    explicit FastDiv(uint32_t denom) : d(denom), mul(0), shr(0) {
        if (denom > 1) {
            uint32_t lg = 0;
            while ((1u << lg) < denom) ++lg;
            const uint32_t p = 31 + lg;
            mul = static_cast<uint32_t>(((1ull << p) + denom - 1) / denom);
            shr = p - 32;
        }
    }
    __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
        return d == 1 ? n : (__umulhi(n, mul) >> shr);
#else
        return n / d;
#endif
    }
    __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
        q = div(n);
        r = n - q * d;
    }
};

}  // namespace vdnn
