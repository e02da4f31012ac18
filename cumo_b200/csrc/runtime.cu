// Runtime glue of libcumo_b200: the launch stream, per-device facts, the launch
// counter, and weak default definitions of the three callbacks that the host
// program owns in the reference (ext/cumo/include/cumo/template_kernel.h:83-90,
// ext/cumo/cuda/runtime.c:16-20, ext/cumo/cuda/memory_pool.cpp:64-123).
//
// The default scratch pool follows the shape of the reference's pool
// (ext/cumo/cuda/memory_pool_impl.hpp:23,160-288): sizes rounded up to 512
// bytes, freed blocks cached per device and handed out best-fit, everything
// released and the allocation retried once when the device is out of memory.
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
struct Pool {
    std::mutex mu;
    std::multimap<size_t, char*> free_blocks;           // size -> block
    std::unordered_map<char*, size_t> live;             // handed out
    size_t total = 0, used = 0;

    char* take(size_t size) {
        size_t need = (size + 511) / 512 * 512;
        if (need == 0) need = 512;
        std::lock_guard<std::mutex> lk(mu);
        auto it = free_blocks.lower_bound(need);
        // reuse a cached block unless it wastes more than half of itself
        if (it != free_blocks.end() && it->first <= need * 2) {
            char* p = it->second;
            size_t sz = it->first;
            free_blocks.erase(it);
            live[p] = sz;
            used += sz;
            return p;
        }
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, need);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            release_locked();
            e = cudaMalloc(&p, need);
        }
        if (e != cudaSuccess) { (void)cudaGetLastError(); latch(e, "cumo_cuda_runtime_malloc"); return nullptr; }
        live[(char*)p] = need;
        total += need;
        used += need;
        return (char*)p;
    }
    void give(char* p) {
        if (!p) return;
        std::lock_guard<std::mutex> lk(mu);
        auto it = live.find(p);
        if (it == live.end()) return;
        used -= it->second;
        free_blocks.emplace(it->second, p);
        live.erase(it);
    }
    void release_locked() {
        for (auto& kv : free_blocks) { cudaFree(kv.second); total -= kv.first; }
        free_blocks.clear();
    }
};

static Pool& pool_of_current_device() {
    static Pool pools[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    return pools[dev];
}

}  // namespace cb200

extern "C" {

__attribute__((weak)) void cumo_cuda_runtime_check_kernel_launch(void) {
    cb200::latch(cudaGetLastError(), "kernel launch");
}

__attribute__((weak)) char* cumo_cuda_runtime_malloc(size_t size) {
    return cb200::pool_of_current_device().take(size);
}

__attribute__((weak)) void cumo_cuda_runtime_free(char* ptr) {
    // Stream-ordered reuse: the block goes back while kernels that read it may
    // still be queued; whoever takes it next queues behind them on the same stream.
    cb200::pool_of_current_device().give(ptr);
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

size_t cb200_pool_total_bytes(void) { auto& p = cb200::pool_of_current_device(); std::lock_guard<std::mutex> lk(p.mu); return p.total; }
size_t cb200_pool_used_bytes(void) { auto& p = cb200::pool_of_current_device(); std::lock_guard<std::mutex> lk(p.mu); return p.used; }
void cb200_pool_free_all_blocks(void) { auto& p = cb200::pool_of_current_device(); std::lock_guard<std::mutex> lk(p.mu); p.release_locked(); }

const char* cb200_version(void) { return "cumo_b200 0.1 (sm_100a)"; }

}  // extern "C"
