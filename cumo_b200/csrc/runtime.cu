// Runtime glue of libcumo_b200: the launch stream, per-device facts, the launch
// counter, and weak default definitions of the three callbacks that the host
// program owns in the reference (ext/cumo/include/cumo/template_kernel.h:83-90,
// ext/cumo/cuda/runtime.c:16-20, ext/cumo/cuda/memory_pool.cpp:64-123).
//
// The default scratch pool follows the shape of the reference's pool
// (ext/cumo/cuda/memory_pool_impl.hpp:23,160-288): sizes rounded up to 512
// bytes, freed blocks cached per device AND per stream and handed out best-fit,
// everything released and the allocation retried once when the device is out of memory.
// It backs only reduction scratch here, so it is small; it hands out plain
// device memory (cudaMalloc), not managed memory.
#include "common.cuh"

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>

namespace cb200 {

static thread_local cudaStream_t tl_stream = nullptr;
static std::atomic<uint64_t> g_launches{0};

cudaStream_t current_stream() { return tl_stream; }

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int sm_count() {
    static std::atomic<int> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int v = cache[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cache[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

// ---- error latch ---------------------------------------------------------------------
static thread_local int tl_err = 0;
static thread_local std::string tl_msg;

static void latch(cudaError_t e, const char* what) {
    if (e == cudaSuccess || tl_err != 0) return;
    tl_err = (int)e;
    tl_msg = std::string(what) + ": " + cudaGetErrorString(e);
}

// ---- scratch pool --------------------------------------------------------------------
// One pool per device, one arena of cached blocks per (device, stream), like the reference's
// per-stream arenas (ext/cumo/cuda/memory_pool_impl.hpp:222-244): a block goes back to the arena of
// the stream that was current when it was taken, so the next taker queues behind the kernels that
// may still be reading it.  A block remembers its device, so it finds its way home even when
// another device is current at the time it is freed.
struct Pool {
    struct Block { size_t size; int dev; cudaStream_t stream; };
    std::map<cudaStream_t, std::multimap<size_t, char*>> arenas;   // stream -> (size -> block)
    size_t total = 0, used = 0;
};

static std::mutex g_pool_mu;                                        // guards every pool and the table of live blocks
static Pool g_pools[64];
static std::unordered_map<char*, Pool::Block> g_live;               // handed out, any device

static int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    return dev;
}

static void release_locked(Pool& p) {
    for (auto& arena : p.arenas)
        for (auto& kv : arena.second) { cudaFree(kv.second); p.total -= kv.first; }
    p.arenas.clear();
}

static char* pool_take(size_t size) {
    size_t need = (size + 511) / 512 * 512;
    if (need == 0) need = 512;
    const int dev = current_device();
    const cudaStream_t st = tl_stream;
    std::lock_guard<std::mutex> lk(g_pool_mu);
    Pool& p = g_pools[dev];
    auto& arena = p.arenas[st];
    auto it = arena.lower_bound(need);
    // reuse a cached block unless it wastes more than half of itself
    if (it != arena.end() && it->first <= need * 2) {
        char* b = it->second;
        const size_t sz = it->first;
        arena.erase(it);
        g_live[b] = {sz, dev, st};
        p.used += sz;
        return b;
    }
    void* b = nullptr;
    cudaError_t e = cudaMalloc(&b, need);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        release_locked(p);                                          // cudaFree synchronises the device: nothing still reads the blocks
        e = cudaMalloc(&b, need);
    }
    if (e != cudaSuccess) { (void)cudaGetLastError(); latch(e, "cumo_cuda_runtime_malloc"); return nullptr; }
    g_live[(char*)b] = {need, dev, st};
    p.total += need;
    p.used += need;
    return (char*)b;
}

static void pool_give(char* b) {
    if (!b) return;
    std::lock_guard<std::mutex> lk(g_pool_mu);
    auto it = g_live.find(b);
    if (it == g_live.end()) return;
    const Pool::Block blk = it->second;
    g_live.erase(it);
    Pool& p = g_pools[blk.dev];
    p.used -= blk.size;
    p.arenas[blk.stream].emplace(blk.size, b);
}

}  // namespace cb200

extern "C" {

__attribute__((weak)) void cumo_cuda_runtime_check_kernel_launch(void) {
    cb200::latch(cudaGetLastError(), "kernel launch");
}

__attribute__((weak)) char* cumo_cuda_runtime_malloc(size_t size) {
    return cb200::pool_take(size);
}

__attribute__((weak)) void cumo_cuda_runtime_free(char* ptr) {
    // Stream-ordered reuse: the block goes back while kernels that read it may still be
    // queued; it returns to the arena of the stream it was taken on, so whoever takes it
    // next queues behind them on that same stream.
    cb200::pool_give(ptr);
}

void cb200_set_stream(void* s) { cb200::tl_stream = (cudaStream_t)s; }
void* cb200_get_stream(void) { return (void*)cb200::tl_stream; }

int cb200_last_error(const char** message) {
    int e = cb200::tl_err;
    if (message) *message = e ? cb200::tl_msg.c_str() : "";
    cb200::tl_err = 0;
    return e;
}

uint64_t cb200_launch_count(void) { return cb200::g_launches.load(std::memory_order_relaxed); }

size_t cb200_pool_total_bytes(void) { std::lock_guard<std::mutex> lk(cb200::g_pool_mu); return cb200::g_pools[cb200::current_device()].total; }
size_t cb200_pool_used_bytes(void) { std::lock_guard<std::mutex> lk(cb200::g_pool_mu); return cb200::g_pools[cb200::current_device()].used; }
void cb200_pool_free_all_blocks(void) { std::lock_guard<std::mutex> lk(cb200::g_pool_mu); cb200::release_locked(cb200::g_pools[cb200::current_device()]); }

const char* cb200_version(void) { return "cumo_b200 0.1 (sm_100a)"; }

}  // extern "C"
