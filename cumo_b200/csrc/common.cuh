// Shared device/host helpers for the libcumo_b200 kernels.
//
// Everything a kernel needs to address its operands is worked out on the host
// into small read-only plan structs that travel as kernel parameters (constant
// bank, never written by a thread), instead of the reference's by-value
// indexer that every thread mutates (ext/cumo/include/cumo/indexer.h:224-300).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include <sys/types.h>

#include "../../include/cumo_b200.h"

namespace cb200 {

constexpr int kMaxDim = CUMO_NA_MAX_DIMENSION;
constexpr int kBlock = 256;          // threads per CTA for every streaming kernel
constexpr int kWarpsPerBlock = kBlock / 32;
constexpr int kUnroll = 4;           // 16-byte packets per operand in flight per thread

// ---- runtime (runtime.cu) -------------------------------------------------
cudaStream_t current_stream();
int sm_count();                       // SMs of the current device (cached per device)
void count_launch(int n = 1);

// grid size for a persistent-style launch: `per_sm` CTAs per SM, capped by work
inline unsigned grid_for(int64_t work_items, int per_sm) {
    int64_t cap = (int64_t)sm_count() * per_sm;
    if (work_items < 1) work_items = 1;
    return (unsigned)(work_items < cap ? work_items : cap);
}

// ---- tracing ----------------------------------------------------------------
// The reference has no tracer (its `NArray.profile` is a stub).  A build with -DCB200_NVTX brackets every host-side launch
// function with an NVTX range named after the function and its template arguments, which a timeline tool then shows
// around the kernels it launched; the default build has none of it.
#ifdef CB200_NVTX
}  // namespace cb200
#include <nvtx3/nvToolsExt.h>
namespace cb200 {
struct TraceRange {
    explicit TraceRange(const char* name) { nvtxRangePushA(name); }
    ~TraceRange() { nvtxRangePop(); }
    TraceRange(const TraceRange&) = delete;
    TraceRange& operator=(const TraceRange&) = delete;
};
#else
struct TraceRange {
    explicit TraceRange(const char*) {}
};
#endif
#define CB200_TRACE_LAUNCH() ::cb200::TraceRange cb200_trace_range_(__PRETTY_FUNCTION__)

// ---- vector access ----------------------------------------------------------
// 16-byte packets: 4 x 32-bit or 2 x 64-bit elements.
template <typename T> struct VecOf { static constexpr int n = 16 / sizeof(T); };

template <typename T> struct alignas(16) Pack { T v[16 / sizeof(T)]; };

// Streaming (evict-first) 16-byte load/store.  ld.global.cs stays coherent, so
// an in-place operation (output aliasing an input) is safe.
template <typename T>
__device__ __forceinline__ Pack<T> ld_pack(const void* p) {
    Pack<T> r;
    int4 q = __ldcs(reinterpret_cast<const int4*>(p));
    *reinterpret_cast<int4*>(&r) = q;
    return r;
}
template <typename T>
__device__ __forceinline__ void st_pack(void* p, const Pack<T>& v) {
    __stcs(reinterpret_cast<int4*>(p), *reinterpret_cast<const int4*>(&v));
}
template <typename T>
__device__ __forceinline__ T ld_one(const void* p) { return __ldcs(reinterpret_cast<const T*>(p)); }
template <>
__device__ __forceinline__ int64_t ld_one<int64_t>(const void* p) {
    return (int64_t)__ldcs(reinterpret_cast<const long long*>(p));
}
template <typename T>
__device__ __forceinline__ void st_one(void* p, T v) { __stcs(reinterpret_cast<T*>(p), v); }
template <>
__device__ __forceinline__ void st_one<int64_t>(void* p, int64_t v) {
    __stcs(reinterpret_cast<long long*>(p), (long long)v);
}

// ---- index decomposition ------------------------------------------------------
// An extent as the 32-bit divisor of an index below 2^31: anything of 2^32 or more divides such an index to
// zero and leaves it as the remainder, and so does 2^32 - 1, so huge extents are clamped instead of truncated.
__device__ __forceinline__ uint32_t extent32(int64_t n) { return n > 0xffffffffLL ? 0xffffffffu : (uint32_t)n; }

// Row-major split of a flat index over `nd` extents into a byte offset, 32-bit
// arithmetic when the index fits (integer division on 64-bit operands is an
// order of magnitude more instructions).
__device__ __forceinline__ int64_t offset_of(int64_t flat, int nd, const int64_t* shape, const int64_t* step) {
    int64_t off = 0;
    if (flat < 0x7fffffffLL) {
        uint32_t i = (uint32_t)flat;
        for (int d = nd - 1; d > 0; --d) {
            uint32_t n = extent32(shape[d]);
            uint32_t q = i / n;
            off += (int64_t)(i - q * n) * step[d];
            i = q;
        }
        if (nd > 0) off += (int64_t)i * step[0];
    } else {
        int64_t i = flat;
        for (int d = nd - 1; d > 0; --d) {
            int64_t n = shape[d];
            int64_t q = i / n;
            off += (i - q * n) * step[d];
            i = q;
        }
        if (nd > 0) off += i * step[0];
    }
    return off;
}

// Same split, producing up to three offsets that share the extents.
template <int NA>
__device__ __forceinline__ void offsets_of(int64_t flat, int nd, const int64_t* shape,
                                           const int64_t (*step)[kMaxDim], int64_t* off) {
#pragma unroll
    for (int a = 0; a < NA; ++a) off[a] = 0;
    if (flat < 0x7fffffffLL) {
        uint32_t i = (uint32_t)flat;
        for (int d = nd - 1; d > 0; --d) {
            uint32_t n = extent32(shape[d]);
            uint32_t q = i / n;
            int64_t r = (int64_t)(i - q * n);
#pragma unroll
            for (int a = 0; a < NA; ++a) off[a] += r * step[a][d];
            i = q;
        }
        if (nd > 0) {
#pragma unroll
            for (int a = 0; a < NA; ++a) off[a] += (int64_t)i * step[a][0];
        }
    } else {
        int64_t i = flat;
        for (int d = nd - 1; d > 0; --d) {
            int64_t n = shape[d];
            int64_t q = i / n;
            int64_t r = i - q * n;
#pragma unroll
            for (int a = 0; a < NA; ++a) off[a] += r * step[a][d];
            i = q;
        }
        if (nd > 0) {
#pragma unroll
            for (int a = 0; a < NA; ++a) off[a] += i * step[a][0];
        }
    }
}

// ---- programmatic dependent launch ----------------------------------------------------------
// A first-pass kernel says early that the kernel queued behind it may be launched (pdl_trigger); that second
// kernel, launched with launch_dependent(), becomes resident while the first still runs and waits in pdl_wait()
// until the first has finished and its writes are visible.  The launch latency of the second pass then overlaps the
// tail of the first instead of following it.  Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline void launch_dependent(void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...) != cudaSuccess) {
        (void)cudaGetLastError();                      // e.g. a stream mode that does not take the attribute: plain launch
        kernel<<<grid, block, 0, st>>>(KArgs(args)...);
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool mult16(int64_t s) { return (s & 15) == 0; }

}  // namespace cb200
