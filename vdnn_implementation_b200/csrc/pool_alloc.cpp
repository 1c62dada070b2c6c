// Pool sub-allocator behind the cnmem-compatible interface (include/cnmem/include/cnmem.h).
// One root pool per process, reserved with a single cudaMalloc; blocks are kept in an
// address-ordered map, allocation is best-fit, neighbours coalesce on free.
#include "cnmem/include/cnmem.h"

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <vector>

namespace {

constexpr size_t kGranularity = 512;   // cnmem rounds every request up to 512 bytes

struct Block { size_t size; bool free; };
struct Fence { size_t begin, end; cudaEvent_t event; unsigned long long seq; cudaStream_t stream; };
// Bytes whose last reader the host has not enqueued yet (vdnnPoolFreeHeld).
struct Hold { size_t begin, end; unsigned long long token; };
constexpr unsigned long long kHeldRank = 1ull << 62;   // held bytes rank behind every pending event

struct Pool {
    std::recursive_mutex mu;            // the resolver re-enters through vdnnPoolResolve
    bool ready = false;
    bool is_virtual = false;
    int device = 0;
    char* base = nullptr;
    size_t capacity = 0, used = 0, peak = 0;
    std::map<size_t, Block> blocks;     // offset -> block
    std::vector<Fence> fences;
    std::vector<Hold> holds;
    vdnnPoolResolver_t resolver = nullptr;
    void* resolver_user = nullptr;
    int fail_countdown = 0;
    bool packed = false;                // tightest fit only (vdnnPoolSetPacked)
    size_t reserve = 0;                 // top bytes kept for transient blocks while the pool is not packed
    unsigned long long next_seq = 1;
    std::vector<cudaEvent_t> spare_events;   // recycled fence events
};
Pool g_pool;

void drop_finished_fences_locked();

size_t round_up(size_t n) { return (n + kGranularity - 1) / kGranularity * kGranularity; }

// 0 when no pending event covers any byte of [begin, end); otherwise the issue number of the youngest
// such event.  Events are issued in program order, so a smaller number means "usable sooner".
// Events recorded on one of the consumer's own streams cost nothing (stream order already covers them).
bool is_consumer(cudaStream_t s, const cudaStream_t* consumers, int n) {
    for (int i = 0; i < n; ++i) if (consumers[i] == s) return true;
    return false;
}

unsigned long long range_readiness_locked(size_t begin, size_t end, const cudaStream_t* consumers, int n, bool events = true) {
    unsigned long long youngest = 0;
    if (events) for (const Fence& f : g_pool.fences)
        if (f.begin < end && begin < f.end && f.seq > youngest && !is_consumer(f.stream, consumers, n)) youngest = f.seq;
    for (const Hold& h : g_pool.holds)
        if (h.begin < end && begin < h.end && kHeldRank + h.token > youngest) youngest = kHeldRank + h.token;
    return youngest;
}

// Has the host enqueue the readers that still hold bytes of [begin, end), lowest token first.
cnmemStatus_t resolve_holds_locked(size_t begin, size_t end) {
    for (;;) {
        unsigned long long lowest = 0;
        for (const Hold& h : g_pool.holds)
            if (h.begin < end && begin < h.end && (lowest == 0 || h.token < lowest)) lowest = h.token;
        if (lowest == 0) return CNMEM_STATUS_SUCCESS;
        if (!g_pool.resolver) return CNMEM_STATUS_INVALID_ARGUMENT;
        const size_t before = g_pool.holds.size();
        g_pool.resolver(g_pool.resolver_user, lowest);
        if (g_pool.holds.size() >= before) return CNMEM_STATUS_UNKNOWN_ERROR;   // the resolver did not resolve
    }
}

// Best fit.  With consumer streams given, the block whose bytes those streams can use soonest wins even
// when it is larger: first blocks with no pending event on another stream, then those whose youngest such
// event was issued earliest.  The consumer then starts at once, or waits for old work that has probably
// finished, instead of queueing behind the copy or kernel that just released the tightest-fitting block
// (a prefetch target must not wait for compute, nor an activation for an offload).  The byte accounting
// (used / peak) is the same either way; only the placement differs.
//
// transient: a block that is given back within the same layer call (workspace).  In a roomy pool those are placed at
// the END of a free block, highest address first among the equally ready: long-lived tensors grow from the low end of
// the free ranges, and a large workspace that is cut out of the middle of one would leave two short ranges behind.
cnmemStatus_t alloc_locked(void** ptr, size_t size, size_t* off_out, size_t* len_out,
                           const cudaStream_t* consumers = nullptr, int num_consumers = 0, bool transient = false) {
    if (!g_pool.ready) return CNMEM_STATUS_NOT_INITIALIZED;
    if (!ptr) return CNMEM_STATUS_INVALID_ARGUMENT;
    if (size == 0) { *ptr = nullptr; return CNMEM_STATUS_SUCCESS; }
    if (g_pool.fail_countdown > 0 && --g_pool.fail_countdown == 0) return CNMEM_STATUS_OUT_OF_MEMORY;
    const size_t need = round_up(size);
    auto best = g_pool.blocks.end();
    unsigned long long best_ready = 0;
    size_t best_at = 0;
    const bool rank = (num_consumers > 0 && !g_pool.fences.empty()) || !g_pool.holds.empty();
    // A candidate is a start offset inside a free block: the block's own start, or the edge of a pending
    // event's (or hold's) byte range inside it: after a long-lived copy has been queued on the first bytes of
    // a large coalesced block, the bytes behind it are still usable at once.  Both refinements -- ranking by
    // pending events and cutting a block in the middle -- trade packing for waiting time; a pool set to
    // "packed" (vdnnPoolSetPacked) uses neither and places exactly like the bookkeeping-only pool.
    const bool roomy = !g_pool.packed;
    auto consider = [&](std::map<size_t, Block>::iterator it, size_t at) {
        const unsigned long long ready = rank ? range_readiness_locked(at, at + need, consumers, num_consumers, roomy) : 0;
        const bool better = best == g_pool.blocks.end() || ready < best_ready ||
            (ready == best_ready && ((at == it->first) > (best_at == best->first) ||
                                     ((at == it->first) == (best_at == best->first) && it->second.size < best->second.size)));
        if (better) { best = it; best_ready = ready; best_at = at; }
    };
    const bool top_down = transient && roomy && !g_pool.is_virtual;
    // Long-lived blocks keep out of the reserve at the top of a roomy pool as long as they fit below it (second pass:
    // anywhere), so that the largest workspace always finds its bytes in one piece there.
    const size_t fence_line = (roomy && !g_pool.is_virtual && !transient && g_pool.reserve < g_pool.capacity)
                                  ? g_pool.capacity - g_pool.reserve : g_pool.capacity;
    for (int pass = 0; pass < 2 && best == g_pool.blocks.end(); ++pass) {
        const size_t limit = pass == 0 ? fence_line : g_pool.capacity;
        if (pass == 1 && fence_line == g_pool.capacity) break;
        for (auto it = g_pool.blocks.begin(); it != g_pool.blocks.end(); ++it) {
            if (!it->second.free || it->second.size < need) continue;
            const size_t block_end = it->first + it->second.size < limit ? it->first + it->second.size : limit;
            if (block_end < it->first + need) continue;
            const size_t lo = it->first, hi = block_end - need;   // admissible starts: [lo, hi]
            if (top_down) {
                const unsigned long long ready = rank ? range_readiness_locked(hi, hi + need, consumers, num_consumers, true) : 0;
                if (best == g_pool.blocks.end() || ready < best_ready || (ready == best_ready && hi > best_at)) {
                    best = it; best_ready = ready; best_at = hi;
                }
                continue;
            }
            consider(it, lo);
            if (!rank || !roomy || (best == it && best_ready == 0)) continue;
            for (const Fence& f : g_pool.fences) {
                if (f.end > lo && f.end <= hi) consider(it, f.end);
                if (f.begin > lo && f.begin <= hi) consider(it, f.begin);
            }
            for (const Hold& h : g_pool.holds) {
                if (h.end > lo && h.end <= hi) consider(it, h.end);
                if (h.begin > lo && h.begin <= hi) consider(it, h.begin);
            }
        }
    }
    if (best == g_pool.blocks.end()) return CNMEM_STATUS_OUT_OF_MEMORY;
    size_t off = best->first;
    const size_t total = best->second.size;
    if (best_at > off) {                       // keep the bytes in front as a free block of their own
        best->second.size = best_at - off;
        g_pool.blocks[best_at] = Block{need, false};
        off = best_at;
    } else {
        best->second.size = need;
        best->second.free = false;
    }
    const size_t rest = (best->first + total) - (off + need);
    if (rest) g_pool.blocks[off + need] = Block{rest, true};
    g_pool.used += need;
    if (g_pool.used > g_pool.peak) g_pool.peak = g_pool.used;
    *ptr = g_pool.base + off;
    if (off_out) { *off_out = off; *len_out = need; }
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t free_locked(void* ptr, size_t* off_out, size_t* len_out) {
    if (!g_pool.ready) return CNMEM_STATUS_NOT_INITIALIZED;
    if (!ptr) return CNMEM_STATUS_SUCCESS;
    const size_t off = static_cast<char*>(ptr) - g_pool.base;
    auto it = g_pool.blocks.find(off);
    if (it == g_pool.blocks.end() || it->second.free) return CNMEM_STATUS_INVALID_ARGUMENT;
    if (off_out) { *off_out = off; *len_out = it->second.size; }
    g_pool.used -= it->second.size;
    it->second.free = true;
    auto next = std::next(it);
    if (next != g_pool.blocks.end() && next->second.free) {
        it->second.size += next->second.size;
        g_pool.blocks.erase(next);
    }
    if (it != g_pool.blocks.begin()) {
        auto prev = std::prev(it);
        if (prev->second.free) {
            prev->second.size += it->second.size;
            g_pool.blocks.erase(it);
        }
    }
    return CNMEM_STATUS_SUCCESS;
}

void drop_finished_fences_locked() {
    size_t keep = 0;
    for (size_t i = 0; i < g_pool.fences.size(); ++i) {
        if (cudaEventQuery(g_pool.fences[i].event) == cudaErrorNotReady) g_pool.fences[keep++] = g_pool.fences[i];
        else g_pool.spare_events.push_back(g_pool.fences[i].event);
    }
    (void)cudaGetLastError();
    g_pool.fences.resize(keep);
}

void destroy_events_locked() {
    for (const Fence& f : g_pool.fences) cudaEventDestroy(f.event);
    for (cudaEvent_t e : g_pool.spare_events) cudaEventDestroy(e);
    g_pool.fences.clear();
    g_pool.spare_events.clear();
}

}  // namespace

extern "C" {

cnmemStatus_t cnmemInit(int numDevices, const cnmemDevice_t* devices, unsigned) {
    if (numDevices != 1 || !devices) return CNMEM_STATUS_INVALID_ARGUMENT;
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (g_pool.ready) return CNMEM_STATUS_INVALID_ARGUMENT;
    size_t size = devices[0].size;
    if (const char* cap = std::getenv("VDNN_POOL_BYTES")) {
        const size_t limit = std::strtoull(cap, nullptr, 10);
        if (limit && limit < size) size = limit;
    }
    size = size / kGranularity * kGranularity;
    if (size == 0) return CNMEM_STATUS_INVALID_ARGUMENT;
    if (cudaSetDevice(devices[0].device) != cudaSuccess) return CNMEM_STATUS_CUDA_ERROR;
    void* p = nullptr;
    if (cudaMalloc(&p, size) != cudaSuccess) { (void)cudaGetLastError(); return CNMEM_STATUS_OUT_OF_MEMORY; }
    g_pool.base = static_cast<char*>(p);
    g_pool.is_virtual = false;
    g_pool.device = devices[0].device;
    g_pool.capacity = size;
    g_pool.used = g_pool.peak = 0;
    g_pool.reserve = 0;
    g_pool.blocks.clear();
    g_pool.blocks[0] = Block{size, true};
    g_pool.fences.clear();
    g_pool.holds.clear();
    g_pool.fail_countdown = 0;
    g_pool.ready = true;
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t cnmemFinalize(void) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (!g_pool.ready) return CNMEM_STATUS_NOT_INITIALIZED;
    if (!g_pool.is_virtual) destroy_events_locked();
    cudaError_t e = g_pool.is_virtual ? cudaSuccess : cudaFree(g_pool.base);
    g_pool.base = nullptr;
    g_pool.blocks.clear();
    g_pool.fences.clear();
    g_pool.holds.clear();
    g_pool.resolver = nullptr;
    g_pool.packed = false;
    g_pool.capacity = g_pool.used = 0;
    g_pool.ready = false;
    return e == cudaSuccess ? CNMEM_STATUS_SUCCESS : CNMEM_STATUS_CUDA_ERROR;
}

cnmemStatus_t cnmemMalloc(void** ptr, size_t size, cudaStream_t) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    size_t off = 0, len = 0;
    const cnmemStatus_t st = alloc_locked(ptr, size, &off, &len);
    if (st != CNMEM_STATUS_SUCCESS || size == 0 || g_pool.holds.empty()) return st;
    return resolve_holds_locked(off, off + len);
}

cnmemStatus_t cnmemFree(void* ptr, cudaStream_t) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    return free_locked(ptr, nullptr, nullptr);
}

cnmemStatus_t cnmemMemGetInfo(size_t* freeMem, size_t* totalMem, cudaStream_t) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (!g_pool.ready) return CNMEM_STATUS_NOT_INITIALIZED;
    if (!freeMem || !totalMem) return CNMEM_STATUS_INVALID_ARGUMENT;
    *totalMem = g_pool.capacity;
    *freeMem = g_pool.capacity - g_pool.used;
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t cnmemPrintMemoryState(FILE* file, cudaStream_t) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (!g_pool.ready) return CNMEM_STATUS_NOT_INITIALIZED;
    if (!file) return CNMEM_STATUS_INVALID_ARGUMENT;
    std::fprintf(file, "pool device=%d capacity=%zu used=%zu peak=%zu blocks=%zu\n", g_pool.device,
                 g_pool.capacity, g_pool.used, g_pool.peak, g_pool.blocks.size());
    for (const auto& kv : g_pool.blocks)
        std::fprintf(file, "  [%12zu, %12zu) %s\n", kv.first, kv.first + kv.second.size,
                     kv.second.free ? "free" : "used");
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t cnmemRegisterStream(cudaStream_t) { return CNMEM_STATUS_SUCCESS; }

const char* cnmemGetErrorString(cnmemStatus_t status) {
    switch (status) {
    case CNMEM_STATUS_SUCCESS: return "CNMEM_STATUS_SUCCESS";
    case CNMEM_STATUS_CUDA_ERROR: return "CNMEM_STATUS_CUDA_ERROR";
    case CNMEM_STATUS_INVALID_ARGUMENT: return "CNMEM_STATUS_INVALID_ARGUMENT";
    case CNMEM_STATUS_NOT_INITIALIZED: return "CNMEM_STATUS_NOT_INITIALIZED";
    case CNMEM_STATUS_OUT_OF_MEMORY: return "CNMEM_STATUS_OUT_OF_MEMORY";
    default: return "CNMEM_STATUS_UNKNOWN_ERROR";
    }
}

cnmemStatus_t vdnnPoolFreeAfter(void* ptr, const cudaStream_t* streams, int numStreams) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    size_t off = 0, len = 0;
    cnmemStatus_t st = free_locked(ptr, &off, &len);
    if (st != CNMEM_STATUS_SUCCESS || !ptr || g_pool.is_virtual) return st;
    // one private event per stream, recorded now: it stands for "everything enqueued on that stream so far".
    // Private events are never re-recorded while a fence holds them, so a fence cannot be extended by
    // later work.
    for (int i = 0; i < numStreams; ++i) {
        cudaEvent_t ev = nullptr;
        if (!g_pool.spare_events.empty()) { ev = g_pool.spare_events.back(); g_pool.spare_events.pop_back(); }
        else if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return CNMEM_STATUS_CUDA_ERROR;
        if (cudaEventRecord(ev, streams[i]) != cudaSuccess) return CNMEM_STATUS_CUDA_ERROR;
        g_pool.fences.push_back(Fence{off, off + len, ev, g_pool.next_seq++, streams[i]});
    }
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t vdnnPoolMallocFor(void** ptr, size_t size, const cudaStream_t* streams, int numStreams) {
    return vdnnPoolMallocKindFor(ptr, size, streams, numStreams, 0);
}

cnmemStatus_t vdnnPoolMallocKindFor(void** ptr, size_t size, const cudaStream_t* streams, int numStreams, int transient) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    size_t off = 0, len = 0;
    if (!g_pool.is_virtual && g_pool.ready) drop_finished_fences_locked();
    cnmemStatus_t st = alloc_locked(ptr, size, &off, &len, streams, g_pool.is_virtual ? 0 : numStreams, transient != 0);
    if (st != CNMEM_STATUS_SUCCESS || size == 0) return st;
    if (!g_pool.holds.empty()) {
        st = resolve_holds_locked(off, off + len);
        if (st != CNMEM_STATUS_SUCCESS) return st;
    }
    if (g_pool.is_virtual) return CNMEM_STATUS_SUCCESS;
    for (const Fence& f : g_pool.fences)
        if (f.begin < off + len && off < f.end)
            for (int s = 0; s < numStreams; ++s)
                if (streams[s] != f.stream && cudaStreamWaitEvent(streams[s], f.event, 0) != cudaSuccess) return CNMEM_STATUS_CUDA_ERROR;
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t vdnnPoolSetPacked(int packed) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    g_pool.packed = packed != 0;
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t vdnnPoolSetTransientReserve(size_t bytes) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (!g_pool.ready) return CNMEM_STATUS_NOT_INITIALIZED;
    g_pool.reserve = round_up(bytes);
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t vdnnPoolSetResolver(vdnnPoolResolver_t resolver, void* user) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    g_pool.resolver = resolver;
    g_pool.resolver_user = user;
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t vdnnPoolFreeHeld(void* ptr, const cudaStream_t* streams, int numStreams, unsigned long long token) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (token == 0 || token >= kHeldRank) return CNMEM_STATUS_INVALID_ARGUMENT;
    if (!ptr || !g_pool.ready) return vdnnPoolFreeAfter(ptr, streams, numStreams);
    const size_t off = static_cast<char*>(ptr) - g_pool.base;
    auto it = g_pool.blocks.find(off);
    if (it == g_pool.blocks.end() || it->second.free) return CNMEM_STATUS_INVALID_ARGUMENT;
    const size_t len = it->second.size;
    const cnmemStatus_t st = vdnnPoolFreeAfter(ptr, streams, numStreams);
    if (st == CNMEM_STATUS_SUCCESS) g_pool.holds.push_back(Hold{off, off + len, token});
    return st;
}

cnmemStatus_t vdnnPoolResolve(unsigned long long token, cudaStream_t stream) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (!g_pool.ready) return CNMEM_STATUS_NOT_INITIALIZED;
    size_t keep = 0;
    for (size_t i = 0; i < g_pool.holds.size(); ++i) {
        const Hold h = g_pool.holds[i];
        if (h.token != token) { g_pool.holds[keep++] = h; continue; }
        if (g_pool.is_virtual) continue;           // bookkeeping only: the hold just goes away
        cudaEvent_t ev = nullptr;
        if (!g_pool.spare_events.empty()) { ev = g_pool.spare_events.back(); g_pool.spare_events.pop_back(); }
        else if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return CNMEM_STATUS_CUDA_ERROR;
        if (cudaEventRecord(ev, stream) != cudaSuccess) return CNMEM_STATUS_CUDA_ERROR;
        g_pool.fences.push_back(Fence{h.begin, h.end, ev, g_pool.next_seq++, stream});
    }
    g_pool.holds.resize(keep);
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t vdnnPoolHighWater(size_t* peakBytes, int reset) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (!g_pool.ready) return CNMEM_STATUS_NOT_INITIALIZED;
    if (peakBytes) *peakBytes = g_pool.peak;
    if (reset) g_pool.peak = g_pool.used;
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t vdnnPoolFailAfter(int k) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    g_pool.fail_countdown = k > 0 ? k : 0;
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t vdnnPoolInitVirtual(size_t size) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (g_pool.ready) return CNMEM_STATUS_INVALID_ARGUMENT;
    size = size / kGranularity * kGranularity;
    if (size == 0) return CNMEM_STATUS_INVALID_ARGUMENT;
    g_pool.base = reinterpret_cast<char*>(static_cast<uintptr_t>(1) << 40);
    g_pool.is_virtual = true;
    g_pool.device = -1;
    g_pool.capacity = size;
    g_pool.used = g_pool.peak = 0;
    g_pool.reserve = 0;
    g_pool.blocks.clear();
    g_pool.blocks[0] = Block{size, true};
    g_pool.fences.clear();
    g_pool.holds.clear();
    g_pool.fail_countdown = 0;
    g_pool.ready = true;
    return CNMEM_STATUS_SUCCESS;
}

cnmemStatus_t vdnnPoolBlockBytes(const void* ptr, size_t* bytes) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    if (!g_pool.ready) return CNMEM_STATUS_NOT_INITIALIZED;
    if (!ptr || !bytes) return CNMEM_STATUS_INVALID_ARGUMENT;
    auto it = g_pool.blocks.find(static_cast<size_t>(static_cast<const char*>(ptr) - g_pool.base));
    if (it == g_pool.blocks.end() || it->second.free) return CNMEM_STATUS_INVALID_ARGUMENT;
    *bytes = it->second.size;
    return CNMEM_STATUS_SUCCESS;
}

int vdnnPoolIsInitialized(void) {
    std::lock_guard<std::recursive_mutex> lock(g_pool.mu);
    return g_pool.ready ? 1 : 0;
}

}  // extern "C"
