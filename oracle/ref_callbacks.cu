// TEST / BENCH INFRASTRUCTURE, not product.  The three callbacks that the reference's kernel units expect
// from their host program (ext/cumo/include/cumo/template_kernel.h:83-90), for the build of those units
// outside the Ruby extension (oracle/build_ref_kernels.py): the launch check latches the first error for
// refk_last_error(), and scratch comes from a small cache over cudaMalloc (the extension's pool caches
// too, so a split reduction pays no cudaMalloc per call there either).
#include <cuda_runtime.h>
#include <map>
#include <mutex>
#include <unordered_map>

static int g_err = 0;
static std::mutex g_mu;
static std::multimap<size_t, char*> g_free;
static std::unordered_map<char*, size_t> g_live;

extern "C" {

void cumo_cuda_runtime_check_kernel_launch(void) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess && g_err == 0) g_err = (int)e;
}

char* cumo_cuda_runtime_malloc(size_t size) {
    size_t need = (size + 511) / 512 * 512;
    if (need == 0) need = 512;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_free.lower_bound(need);
    if (it != g_free.end() && it->first <= 2 * need) {
        char* p = it->second;
        g_live[p] = it->first;
        g_free.erase(it);
        return p;
    }
    void* p = nullptr;
    if (cudaMalloc(&p, need) != cudaSuccess) { (void)cudaGetLastError(); if (g_err == 0) g_err = (int)cudaErrorMemoryAllocation; return nullptr; }
    g_live[(char*)p] = need;
    return (char*)p;
}

void cumo_cuda_runtime_free(char* ptr) {
    if (!ptr) return;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_live.find(ptr);
    if (it == g_live.end()) return;
    g_free.emplace(it->second, ptr);        // everything runs on the legacy default stream: reuse is stream ordered
    g_live.erase(it);
}

// first launch error seen since the last call (a cudaError_t value), 0 if none
int refk_last_error(void) { int e = g_err; g_err = 0; return e; }

}
