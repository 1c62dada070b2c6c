// Host-side counter-based generators (Philox4x32-10, element index = counter) for inputs, labels
// and weights.  Compiled with -ffp-contract=off so that every value is reproducible bit for bit
// by any other implementation of the same formulas.
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "vdnn_b200.h"

namespace {

inline void philox(uint64_t ctr, uint64_t key, uint32_t out[4]) {
    uint32_t c[4] = {static_cast<uint32_t>(ctr), static_cast<uint32_t>(ctr >> 32), 0u, 0u};
    uint32_t k[2] = {static_cast<uint32_t>(key), static_cast<uint32_t>(key >> 32)};
    for (int round = 0; round < 10; ++round) {
        const uint64_t a = 0xD2511F53ull * c[0], b = 0xCD9E8D57ull * c[2];
        const uint32_t n0 = static_cast<uint32_t>(b >> 32) ^ c[1] ^ k[0];
        const uint32_t n2 = static_cast<uint32_t>(a >> 32) ^ c[3] ^ k[1];
        c[1] = static_cast<uint32_t>(b);
        c[3] = static_cast<uint32_t>(a);
        c[0] = n0;
        c[2] = n2;
        k[0] += 0x9E3779B9u;
        k[1] += 0xBB67AE85u;
    }
    std::memcpy(out, c, sizeof c);
}

constexpr float kInv24 = 1.0f / 16777216.0f;

template <class F>
void parallel_for(size_t n, F body) {
    unsigned workers = std::thread::hardware_concurrency();
    if (workers == 0) workers = 1;
    if (workers > 16) workers = 16;
    if (n < (1u << 16) || workers == 1) { body(0, n); return; }
    std::vector<std::thread> pool;
    const size_t chunk = (n + workers - 1) / workers;
    for (unsigned t = 0; t < workers; ++t) {
        const size_t lo = t * chunk, hi = lo + chunk < n ? lo + chunk : n;
        if (lo < hi) pool.emplace_back(body, lo, hi);
    }
    for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

void vdnn_host_fill_uniform(float* dst, size_t count, uint64_t seed, float lo, float hi) {
    const float span = hi - lo;
    parallel_for(count, [=](size_t a, size_t b) {
        for (size_t i = a; i < b; ++i) {
            uint32_t r[4];
            philox(i, seed, r);
            const float t = span * (static_cast<float>(r[0] >> 8) * kInv24);
            dst[i] = lo + t;
        }
    });
}

void vdnn_host_fill_normal(float* dst, size_t count, uint64_t seed, float mean, float stddev) {
    parallel_for(count, [=](size_t a, size_t b) {
        for (size_t i = a; i < b; ++i) {
            uint32_t r[4];
            philox(i, seed, r);
            const float u1 = static_cast<float>((r[0] >> 8) + 1u) * kInv24;   // (0, 1]
            const float u2 = static_cast<float>(r[1] >> 8) * kInv24;          // [0, 1)
            const float radius = sqrtf(-2.0f * logf(u1));
            const float angle = 6.28318530717958647692f * u2;
            const float z = radius * cosf(angle);
            const float t = stddev * z;
            dst[i] = mean + t;
        }
    });
}

void vdnn_host_fill_onehot(float* dst, int rows, int cols, uint64_t seed) {
    std::memset(dst, 0, sizeof(float) * static_cast<size_t>(rows) * cols);
    for (int i = 0; i < rows; ++i) {
        uint32_t r[4];
        philox(static_cast<uint64_t>(i), seed, r);
        dst[static_cast<size_t>(i) * cols + r[0] % static_cast<uint32_t>(cols)] = 1.0f;
    }
}

}  // extern "C"
