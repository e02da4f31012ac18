// cb200_sfloat_sum_noalloc_kernel_launch: the float32 `sum` reduction for callers that
// must not allocate device memory.
//
// The regular entry point (cumo_sfloat_sum_kernel_launch) takes its [output][segment]
// scratch from the host program's cumo_cuda_runtime_malloc callback.  Some callers cannot
// go there at the moment they need a sum:
//   * inside the Ruby extension that callback may run the garbage collector and raise
//     (longjmp) when the pool is exhausted, which is not allowed in a finalizer or while a
//     C++ object with a destructor is live on the caller's stack;
//   * an embedder that hands out all device memory at start-up (a fixed budget per tenant
//     or per job) has no allocator left to call later, and a bare cudaMalloc would both
//     break its accounting and synchronise the whole device;
//   * a latency-critical loop that must not take the allocator's lock or risk the
//     cudaMalloc/cudaFree fallback of an empty pool.
// This variant runs the same two kernels (red_row_kernel, then red_fold_kernel) but keeps
// the scratch in a fixed array that is part of the library image, so it never allocates or
// frees anything, on the device or through any library.  It always cuts long rows into
// 32 KiB segments, where the regular entry point keeps rows of up to 256 KiB whole when there
// are many of them, so the two agree to rounding (the additions are grouped differently), not
// bit for bit.
//
// Limits and rules, all of them consequences of the fixed array:
//   * the array holds kNoAllocScratchFloats partial sums (1 MiB); a reduction that needs
//     more outputs x segments than that is refused with an error, nothing is launched;
//   * every GPU that loads the library carries the 1 MiB until the process exits;
//   * only the layout the ROW plan covers is accepted: the reduced axes must collapse to
//     one contiguous run (a full sum of a contiguous array, or sums along the last axes);
//   * all calls on a device share the one array and find the previous call's partials in
//     it.  Nothing in it has to start at zero -- every partial a fold reads was written by
//     the pass before it -- but two calls whose kernels overlap on the GPU (different
//     streams, no ordering between them) race on it.  Issue them on one stream;
//   * the first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current).  Make that first call outside any
//     stream capture; later calls only launch kernels.
#include "reduce.cuh"

#include <atomic>
#include <cstdio>
#include <mutex>

namespace cb200 {

constexpr int64_t kNoAllocScratchFloats = 1 << 18;

// In host code this name is only a handle for the runtime's symbol table, not a device
// address; kernels get the address looked up below.
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

// device address of the array, per device, looked up once
static float* noalloc_scratch_address(char* err, size_t errlen) {
    static std::mutex mu;
    static float* addr[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        snprintf(err, errlen, "cudaGetDevice failed: %s", cudaGetErrorString(e));
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(mu);
    if (!addr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            snprintf(err, errlen, "cudaGetSymbolAddress(scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
            return nullptr;
        }
        addr[dev] = p;
    }
    return addr[dev];
}

}  // namespace cb200

extern "C" int cb200_sfloat_sum_noalloc_kernel_launch(cumo_na_reduction_arg_t* arg, char* errbuf, size_t errlen) {
    using namespace cb200;
    using R = red::SumLike<float, false, false>;
    char local[8];
    if (!errbuf || errlen == 0) { errbuf = local; errlen = sizeof local; }
    errbuf[0] = 0;
    constexpr int ES = 4, VMAX = 4;
    RedPlan p;
    if (!make_red_plan(&p, arg, nullptr)) return 0;                  // an empty output: nothing to do
    if (!(p.n_rd == 1 && (p.in_rstep[0] == ES || p.n_red <= 1))) {
        snprintf(errbuf, errlen, "the no-allocation sum needs the reduced axes to form one contiguous run "
                                 "(innermost reduce step %lld bytes, %d reduce dims after merging)",
                 (long long)p.in_rstep[p.n_rd - 1], p.n_rd);
        return 1;
    }
    // The array's address is looked up on the first call on each device, whatever that call's shape, so that a
    // small warm-up call made before a stream capture covers the segmented calls that follow.
    float* const scratch = noalloc_scratch_address(errbuf, errlen);
    if (!scratch) return 3;
    const R r{0, 0.0f};
    RedLaunch q;
    q.n_split = 1;
    q.n_strips = 0;
    q.flat_index = 0;
    q.ordered = 1;
    const int64_t L = p.n_red;
    const char* in = arg->in.ptr;
    bool vec = aligned16(in);
    for (int d = 0; d < p.n_od && vec; ++d) if (!mult16(p.in_ostep[d])) vec = false;
    const bool wide = L >= 4096;
    q.seg_len = L > 0 ? L : 1;
    if (wide) {
        int64_t seg = (32 << 10) / ES;
        int64_t ns = (L + seg - 1) / seg;
        while (ns > 8192) { seg *= 2; ns = (L + seg - 1) / seg; }
        if (ns > 1) { q.seg_len = seg; q.n_split = (int)ns; }
    }
    float* partial = nullptr;
    if (q.n_split > 1) {
        const int64_t need = p.n_out * q.n_split;
        if (need > kNoAllocScratchFloats) {
            snprintf(errbuf, errlen, "the no-allocation sum needs %lld partial sums (%lld outputs x %d segments) "
                                     "but its fixed scratch holds %lld; use cumo_sfloat_sum_kernel_launch",
                     (long long)need, (long long)p.n_out, q.n_split, (long long)kNoAllocScratchFloats);
            return 2;
        }
        partial = scratch;
    }
    cudaStream_t st = current_stream();
    const int64_t items = p.n_out * q.n_split;
    char* out = arg->out.ptr;
    if (wide) {
        if (vec) red_row_kernel<R, VMAX, kBlock><<<red_grid(items), kBlock, 0, st>>>(p, r, q, in, out, nullptr, partial);
        else     red_row_kernel<R, 1, kBlock><<<red_grid(items), kBlock, 0, st>>>(p, r, q, in, out, nullptr, partial);
    } else {
        const unsigned grid = red_grid((items + kWarpsPerBlock - 1) / kWarpsPerBlock);
        if (vec) red_row_kernel<R, VMAX, 32><<<grid, kBlock, 0, st>>>(p, r, q, in, out, nullptr, partial);
        else     red_row_kernel<R, 1, 32><<<grid, kBlock, 0, st>>>(p, r, q, in, out, nullptr, partial);
    }
    int launches = 1;
    if (q.n_split > 1) {
        if (q.n_split > 256 && p.n_out < 4096)
            red_fold_kernel<R, kBlock><<<red_grid(p.n_out), kBlock, 0, st>>>(p, r, partial, q.n_split, out, nullptr);
        else
            red_fold_kernel<R, 32><<<red_grid((p.n_out + kWarpsPerBlock - 1) / kWarpsPerBlock), kBlock, 0, st>>>(p, r, partial, q.n_split, out, nullptr);
        ++launches;
    }
    count_launch(launches);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(errbuf, errlen, "kernel launch failed: %s", cudaGetErrorString(e));
        return 4;
    }
    return 0;
}
