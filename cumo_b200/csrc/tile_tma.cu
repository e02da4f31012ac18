// Host pieces of the copy-engine tile kernel (tile_tma.cuh): the tensor-map encoder, looked up through the runtime
// so that the library does not link against the driver library; the status word of the kernel's bounded waits; knobs.
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <set>
#include <utility>

#include "tile_tma.cuh"

namespace cb200 {

static __device__ int g_tile_pipeline_status_word;

TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            p = nullptr;
        }
        return reinterpret_cast<TensorMapEncodeFn>(p);
    }();
    return fn;
}

int* tile_status_word() {
    static std::mutex m;
    static int* word[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(m);
    if (!word[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_tile_pipeline_status_word) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        word[dev] = static_cast<int*>(p);
    }
    return word[dev];
}

static std::atomic<unsigned long long> g_tile_tma_launches{0};
void note_tile_tma_launch() { g_tile_tma_launches.fetch_add(1, std::memory_order_relaxed); }

static int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

// CB200_TILE_STAGES: depth of the ring (2..6); default 4 tiles of one input, 3 of two
int tile_tma_stages(int n_inputs) {
    static const int forced = env_int("CB200_TILE_STAGES", 0);
    int s = forced > 0 ? forced : (n_inputs <= 1 ? 4 : 3);
    if (s < 2) s = 2;
    if (s > kTmaMaxStages) s = kTmaMaxStages;
    return s;
}

// Kernels that take more than 48 KiB of dynamic shared memory must say so once per device.
bool tile_tma_raise_smem_limit(const void* kernel) {
    static std::mutex m;
    static std::set<std::pair<const void*, int>> done;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(m);
    if (done.count({kernel, dev})) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) { cudaGetLastError(); return false; }
    done.insert({kernel, dev});
    return true;
}

// CB200_TILE_TMA: 0 sends transposed operands through the register-staged tile kernels, 1 through the copy-engine
// kernel whenever it can take them; unset (or 2): each where it measured faster
int tile_tma_mode() {
    static const int v = env_int("CB200_TILE_TMA", 2);
    return v;
}

}  // namespace cb200

// 0: no bounded wait of the copy-engine tile kernel has run out on the current device since the library was loaded (or
// since the last call); 1: one did, and the results of that launch are not valid; 2: the kernel found its shared memory
// misaligned and did nothing; -1: the word could not be read.  Synchronises the device; clears the word.
extern "C" int cb200_tile_pipeline_status(void) {
    int* w = cb200::tile_status_word();
    if (!w) return -1;
    int v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpy(&v, w, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(w, 0, sizeof v);
    return v;
}

// Launches of the copy-engine tile kernel in this process.
extern "C" unsigned long long cb200_tile_pipeline_launches(void) {
    return cb200::g_tile_tma_launches.load(std::memory_order_relaxed);
}
