// bincount: occurrences (or summed weights) of each non-negative integer value along one run.
//
// Entry points and argument meaning are the reference's (narray/gen/tmpl/bincount.c:18,70 declare
// them, bincount_kernel.cu:32-97 defines them): the output is cleared, then every element x of
// the run adds 1 (or its weight) to out[x]; an element outside [0, n) raises `*oor`, leaves its
// value in `*item` and is skipped.  The reference does one global atomicAdd per element.  Here a
// CTA counts into private histograms in shared memory (up to kSmemBins bins; several copies picked
// by lane when the bins are few, so that equal values within a warp collide less), reading the run
// with 16-byte loads when it is contiguous, and adds each non-empty bin to the output once, so
// global atomics drop from one per element to one per (CTA, occupied bin).  Integer counts are
// exact in any order; weighted sums use floating-point atomics, as in the reference, so their
// last bits may differ from run to run.
#include "common.cuh"

#include <limits>
#include <type_traits>

namespace cb200 {

constexpr int kSmemBins = 8192;              // 32 KiB of 32-bit counters (or of floats; 64 KiB of doubles)
constexpr int kBinsPerThreadLoads = 16;      // elements per thread per pass

template <typename TC>
__global__ void __launch_bounds__(kBlock)
bincount_clear_kernel(char* out, int64_t so, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (uint64_t)gridDim.x * kBlock)
        *reinterpret_cast<TC*>(out + (int64_t)i * so) = TC(0);
}

template <typename TI>
__device__ __forceinline__ TI load_item(const char* p1, int64_t s1, const size_t* idx1, uint64_t i) {
    return *reinterpret_cast<const TI*>(idx1 ? p1 + idx1[i] : p1 + (int64_t)i * s1);
}

// TS: the shared-memory counter type (uint32_t for counts, the weight type for weighted sums)
template <typename TI, typename TC, typename TW, bool SMEM>
__global__ void __launch_bounds__(kBlock)
bincount_kernel(const char* __restrict__ p1, int64_t s1, const size_t* __restrict__ idx1, uint64_t count,
                const char* __restrict__ pw, int64_t sw, char* out, int64_t so, uint64_t n, int copies, int* oor, size_t* item) {
    constexpr bool WEIGHTED = !std::is_same<TW, void>::value;
    using TS = typename std::conditional<WEIGHTED, TC, uint32_t>::type;
    extern __shared__ __align__(16) char smem_raw[];
    TS* hist = reinterpret_cast<TS*>(smem_raw);
    // `copies` private histograms, picked by lane: threads of a warp that meet the same value collide less often
    TS* my_hist = hist + (size_t)(threadIdx.x % copies) * n;
    if (SMEM) {
        for (uint32_t b = threadIdx.x; b < n * copies; b += kBlock) hist[b] = TS(0);
        __syncthreads();
    }
    auto add = [&](TI x, uint64_t i) {
        if (x < 0 || (uint64_t)x >= n) { *item = (size_t)x; *oor = 1; return; }     // any offender will do: the stores race harmlessly
        if constexpr (WEIGHTED) {
            const TC w = (TC)*reinterpret_cast<const typename std::conditional<WEIGHTED, TW, float>::type*>(pw + (int64_t)i * sw);
            if (SMEM) atomicAdd(my_hist + x, w); else atomicAdd(reinterpret_cast<TC*>(out + (int64_t)x * so), w);
        } else {
            if (SMEM) atomicAdd(my_hist + x, 1u);
            else atomicAdd(reinterpret_cast<typename std::conditional<sizeof(TC) == 8, unsigned long long, unsigned>::type*>(out + (int64_t)x * so), 1);
        }
    };
    constexpr int V = 16 / sizeof(TI);
    const bool packed = !idx1 && s1 == (int64_t)sizeof(TI) && (reinterpret_cast<uintptr_t>(p1) & 15) == 0;
    const uint64_t per_cta = (uint64_t)kBlock * kBinsPerThreadLoads;
    for (uint64_t base = (uint64_t)blockIdx.x * per_cta; base < count; base += (uint64_t)gridDim.x * per_cta) {
        if (packed && base + per_cta <= count) {
            // whole tile, contiguous: 16-byte loads, all issued before the first use
            Pack<TI> v[kBinsPerThreadLoads / V];
#pragma unroll
            for (int j = 0; j < kBinsPerThreadLoads / V; ++j)
                v[j] = ld_pack<TI>(p1 + (base + ((uint64_t)j * kBlock + threadIdx.x) * V) * sizeof(TI));
#pragma unroll
            for (int j = 0; j < kBinsPerThreadLoads / V; ++j)
#pragma unroll
                for (int e = 0; e < V; ++e) add(v[j].v[e], base + ((uint64_t)j * kBlock + threadIdx.x) * V + e);
        } else {
            for (int j = 0; j < kBinsPerThreadLoads; ++j) {
                const uint64_t i = base + (uint64_t)j * kBlock + threadIdx.x;
                if (i < count) add(load_item<TI>(p1, s1, idx1, i), i);
            }
        }
    }
    if (SMEM) {
        __syncthreads();
        for (uint32_t b = threadIdx.x; b < n; b += kBlock) {
            TS c = hist[b];
            for (int r = 1; r < copies; ++r) c += hist[(size_t)r * n + b];
            if (c != TS(0)) {
                if constexpr (WEIGHTED) atomicAdd(reinterpret_cast<TC*>(out + (int64_t)b * so), c);
                else atomicAdd(reinterpret_cast<typename std::conditional<sizeof(TC) == 8, unsigned long long, unsigned>::type*>(out + (int64_t)b * so), c);
            }
        }
    }
}

template <typename TI, typename TC, typename TW>
void launch_bincount(char* p1, ssize_t s1, size_t* idx1, uint64_t count, char* pw, ssize_t sw, char* out, ssize_t so,
                     uint64_t n, int* oor, size_t* item) {
    CB200_TRACE_LAUNCH();
    constexpr bool WEIGHTED = !std::is_same<TW, void>::value;
    cudaStream_t st = current_stream();
    int launches = 0;
    if (n > 0) {
        bincount_clear_kernel<TC><<<grid_for((int64_t)((n + kBlock - 1) / kBlock), 8), kBlock, 0, st>>>(out, so, n);
        ++launches;
    }
    if (count > 0 && n > 0) {
        const uint64_t per_cta = (uint64_t)kBlock * kBinsPerThreadLoads;
        const unsigned grid = grid_for((int64_t)((count + per_cta - 1) / per_cta), 8);
        const size_t ts = WEIGHTED ? sizeof(TC) : sizeof(uint32_t);
        if (n <= (uint64_t)kSmemBins) {
            int copies = (int)(kSmemBins / n);           // as many private histograms as fit the budget, at most 8
            if (copies > 8) copies = 8;
            if (copies < 1) copies = 1;
            const size_t smem = (size_t)n * copies * ts;
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(bincount_kernel<TI, TC, TW, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kSmemBins * sizeof(double)));
            bincount_kernel<TI, TC, TW, true><<<grid, kBlock, smem, st>>>(p1, s1, idx1, count, pw, sw, out, so, n, copies, oor, item);
        } else {
            bincount_kernel<TI, TC, TW, false><<<grid, kBlock, 0, st>>>(p1, s1, idx1, count, pw, sw, out, so, n, 1, oor, item);
        }
        ++launches;
    }
    count_launch(launches);
    cumo_cuda_runtime_check_kernel_launch();
}

// ---- counting and sizing in one pass ---------------------------------------------------------------------------------------
// The output of bincount is as long as the largest value says, so the reference reads the run twice: a min/max reduction to
// size the output (bincount.c:99-131), then the counting kernel.  This probe does both at once for the common case of small
// values: it counts every value in [0, kProbeBins) into a fixed histogram and records the extremes of ALL values.  A host that
// finds 0 <= min and max < kProbeBins has its counts; otherwise it falls back to the two passes.  Values below kProbeFast go
// to per-CTA histograms in shared memory (eight copies picked by lane), the rest of the range to global atomics.
constexpr int kProbeBins = 8192;
constexpr int kProbeFast = 1024;
constexpr int kProbeCopies = 8;

__global__ void bincount_probe_init_kernel(uint32_t* hist, long long* extremes) {
    for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < kProbeBins; b += gridDim.x * blockDim.x) hist[b] = 0u;
    if (blockIdx.x == 0 && threadIdx.x == 0) { extremes[0] = 0x7fffffffffffffffLL; extremes[1] = -0x7fffffffffffffffLL - 1; }
}

template <typename TI>
__global__ void __launch_bounds__(kBlock)
bincount_probe_kernel(const char* __restrict__ p1, int64_t s1, uint64_t count, uint32_t* hist, long long* extremes) {
    __shared__ uint32_t local[kProbeFast * kProbeCopies];
    __shared__ long long lo_s[kWarpsPerBlock], hi_s[kWarpsPerBlock];
    for (int b = threadIdx.x; b < kProbeFast * kProbeCopies; b += kBlock) local[b] = 0u;
    __syncthreads();
    uint32_t* mine = local + (threadIdx.x % kProbeCopies) * kProbeFast;
    // extremes in the element type (one min and one max instruction per element for 32-bit items); range tests as unsigned,
    // so that a negative value fails both
    using TU = typename std::make_unsigned<TI>::type;
    TI lo_t = std::numeric_limits<TI>::max(), hi_t = std::numeric_limits<TI>::min();
    auto add = [&](TI x) {
        lo_t = x < lo_t ? x : lo_t;
        hi_t = x > hi_t ? x : hi_t;
        const TU u = (TU)x;
        if (u < (TU)kProbeFast) atomicAdd(mine + u, 1u);
        else if (u < (TU)kProbeBins) atomicAdd(hist + u, 1u);
    };
    constexpr int V = 16 / sizeof(TI);
    const bool packed = s1 == (int64_t)sizeof(TI) && (reinterpret_cast<uintptr_t>(p1) & 15) == 0;
    const uint64_t per_cta = (uint64_t)kBlock * kBinsPerThreadLoads;
    for (uint64_t base = (uint64_t)blockIdx.x * per_cta; base < count; base += (uint64_t)gridDim.x * per_cta) {
        if (packed && base + per_cta <= count) {
            Pack<TI> v[kBinsPerThreadLoads / V];
#pragma unroll
            for (int j = 0; j < kBinsPerThreadLoads / V; ++j)
                v[j] = ld_pack<TI>(p1 + (base + ((uint64_t)j * kBlock + threadIdx.x) * V) * sizeof(TI));
#pragma unroll
            for (int j = 0; j < kBinsPerThreadLoads / V; ++j)
#pragma unroll
                for (int e = 0; e < V; ++e) add(v[j].v[e]);
        } else {
            for (int j = 0; j < kBinsPerThreadLoads; ++j) {
                const uint64_t i = base + (uint64_t)j * kBlock + threadIdx.x;
                if (i < count) add(*reinterpret_cast<const TI*>(p1 + (int64_t)i * s1));
            }
        }
    }
    long long lo = (long long)lo_t, hi = (long long)hi_t;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const long long ol = __shfl_xor_sync(0xffffffffu, lo, d), oh = __shfl_xor_sync(0xffffffffu, hi, d);
        lo = ol < lo ? ol : lo;
        hi = oh > hi ? oh : hi;
    }
    if ((threadIdx.x & 31) == 0) { lo_s[threadIdx.x >> 5] = lo; hi_s[threadIdx.x >> 5] = hi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kWarpsPerBlock; ++w) { lo = lo_s[w] < lo ? lo_s[w] : lo; hi = hi_s[w] > hi ? hi_s[w] : hi; }
        atomicMin(extremes, lo);
        atomicMax(extremes + 1, hi);
    }
    for (int b = threadIdx.x; b < kProbeFast; b += kBlock) {
        uint32_t c = 0;
#pragma unroll
        for (int r = 0; r < kProbeCopies; ++r) c += local[r * kProbeFast + b];
        if (c) atomicAdd(hist + b, c);
    }
}

template <typename TI>
void launch_bincount_probe(char* p1, ssize_t s1, uint64_t count, uint32_t* hist, long long* extremes) {
    CB200_TRACE_LAUNCH();
    cudaStream_t st = current_stream();
    bincount_probe_init_kernel<<<8, 256, 0, st>>>(hist, extremes);
    int launches = 1;
    if (count > 0) {
        const uint64_t per_cta = (uint64_t)kBlock * kBinsPerThreadLoads;
        bincount_probe_kernel<TI><<<grid_for((int64_t)((count + per_cta - 1) / per_cta), 8), kBlock, 0, st>>>(p1, s1, count, hist, extremes);
        ++launches;
    }
    count_launch(launches);
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200

using namespace cb200;

extern "C" int cb200_bincount_probe_bins(void) { return kProbeBins; }
extern "C" void cb200_int32_bincount_probe_kernel_launch(char* p1, ssize_t s1, uint64_t count, uint32_t* hist, long long* extremes) {
    launch_bincount_probe<int32_t>(p1, s1, count, hist, extremes);
}
extern "C" void cb200_int64_bincount_probe_kernel_launch(char* p1, ssize_t s1, uint64_t count, uint32_t* hist, long long* extremes) {
    launch_bincount_probe<int64_t>(p1, s1, count, hist, extremes);
}

#define CB200_DEF_BINCOUNT(T, C)                                                                                                   \
    extern "C" void cumo_iter_##T##_bincount_32_kernel_launch(char* p1, ssize_t s1, size_t* idx1, uint64_t count, char* p2,        \
                                                             ssize_t s2, uint64_t n, int* oor, size_t* item) {                     \
        launch_bincount<C, uint32_t, void>(p1, s1, idx1, count, nullptr, 0, p2, s2, n, oor, item); }                               \
    extern "C" void cumo_iter_##T##_bincount_64_kernel_launch(char* p1, ssize_t s1, size_t* idx1, uint64_t count, char* p2,        \
                                                             ssize_t s2, uint64_t n, int* oor, size_t* item) {                     \
        launch_bincount<C, uint64_t, void>(p1, s1, idx1, count, nullptr, 0, p2, s2, n, oor, item); }                               \
    extern "C" void cumo_iter_##T##_bincount_sf_kernel_launch(char* p1, ssize_t s1, char* p2, ssize_t s2, uint64_t count, char* p3, \
                                                             ssize_t s3, uint64_t n, int* oor, size_t* item) {                     \
        launch_bincount<C, float, float>(p1, s1, nullptr, count, p2, s2, p3, s3, n, oor, item); }                                  \
    extern "C" void cumo_iter_##T##_bincount_df_kernel_launch(char* p1, ssize_t s1, char* p2, ssize_t s2, uint64_t count, char* p3, \
                                                             ssize_t s3, uint64_t n, int* oor, size_t* item) {                     \
        launch_bincount<C, double, double>(p1, s1, nullptr, count, p2, s2, p3, s3, n, oor, item); }

CB200_DEF_BINCOUNT(int32, int32_t)
CB200_DEF_BINCOUNT(int64, int64_t)
