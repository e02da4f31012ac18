// cumsum / cumprod along one strided run: out[i] = x[0] (+|*) ... (+|*) x[i].
//
// Entry points are the reference's (narray/gen/tmpl/cum.c:3 declares them, cum_kernel.cu:56-80
// defines them on top of thrust::inclusive_scan): (p1, p2, s1, s2, n) with byte steps of any sign,
// returning a cudaError_t; the host side calls once per run (ndloop walks the other axes).
// The `_nan` forms use the reference's operator (include/cumo/types/real_accum_kernel.h:12-26):
// a NaN accumulator is replaced by the next value and a NaN value is skipped, i.e. NaN means
// "nothing yet" -- which makes it associative, so it can be scanned in parallel as it stands.
//
// Plan: tiles of 4096 elements, 16 consecutive elements per thread (staged through shared memory so
// that global memory sees coalesced 16-byte accesses when the run is contiguous).  Short runs are one
// CTA.  Longer runs take three launches with no waiting between CTAs: (1) every CTA folds its run of
// consecutive tiles into one value, (2) one CTA scans those (at most 4096) values, (3) every CTA scans
// its tiles again starting from the value before it.  No identity element is
// ever combined in, so out[0] is x[0] bit for bit (a -0.0 stays -0.0) and integer overflow wraps
// exactly as in the sequential loop; floating-point results differ from it only by association.
#include "common.cuh"

namespace cb200 {

constexpr int kScanItems = 16;
constexpr int kScanTile = kBlock * kScanItems;

template <typename T, bool PROD, bool NANSKIP>
struct ScanOp {
    __device__ __forceinline__ static T combine(T a, T b) {
        if constexpr (NANSKIP) {
            if (a != a) return b;             // nothing yet: take the next value, whatever it is
            if (b != b) return a;             // a NaN value is skipped
        }
        return PROD ? a * b : a + b;
    }
};

// inclusive scan of one value per thread across the CTA, in thread order; returns the value of the
// thread before this one in `*before` (valid when threadIdx.x > 0) and the CTA's total in `*total`
template <typename T, typename Op>
__device__ __forceinline__ void block_scan(T v, T* before, T* total, T* smem /* [2 * warps] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const T o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc = Op::combine(o, inc);
    }
    if (lane == 31) smem[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        T w = lane < kWarpsPerBlock ? smem[lane] : smem[0];
#pragma unroll
        for (int d = 1; d < kWarpsPerBlock; d <<= 1) {
            const T o = __shfl_up_sync(0xffffffffu, w, d);
            if (lane >= d) w = Op::combine(o, w);
        }
        if (lane < kWarpsPerBlock) smem[kWarpsPerBlock + lane] = w;      // inclusive over warps
    }
    __syncthreads();
    T prev = __shfl_up_sync(0xffffffffu, inc, 1);                        // inclusive value of the lane before
    if (warp > 0) prev = lane > 0 ? Op::combine(smem[kWarpsPerBlock + warp - 1], prev) : smem[kWarpsPerBlock + warp - 1];
    *before = prev;
    *total = smem[2 * kWarpsPerBlock - 1];
    __syncthreads();                                                      // smem is reused by the caller's next tile
}

template <typename T>
__device__ __forceinline__ void load_items(const char* p, int64_t s, int64_t first, int64_t n, bool packed, T (&x)[kScanItems]) {
    constexpr int V = 16 / sizeof(T);
    if (packed && first + kScanItems <= n) {
#pragma unroll
        for (int j = 0; j < kScanItems / V; ++j) {
            const Pack<T> v = ld_pack<T>(p + (first + j * V) * (int64_t)sizeof(T));
#pragma unroll
            for (int e = 0; e < V; ++e) x[j * V + e] = v.v[e];
        }
    } else {
#pragma unroll
        for (int j = 0; j < kScanItems; ++j)
            x[j] = first + j < n ? *reinterpret_cast<const T*>(p + (first + j) * s) : T();
    }
}

// Whole, contiguous, 16-byte-aligned tiles go through shared memory so that global memory sees a warp's
// 32 packets side by side (512 bytes per instruction) while each thread still ends up with its 16 consecutive
// elements.  A thread's chunk is followed by 16 bytes of padding: with that stride the 16-byte accesses of a
// quarter-warp fall on disjoint banks.
template <typename T>
struct ScanStage {
    static constexpr int kChunk = kScanItems * (int)sizeof(T);
    static constexpr int kStride = kChunk + 16;
    static constexpr int kBytes = kBlock * kStride;
    static constexpr int kPacksPerThread = kChunk / 16;
};

template <typename T>
__device__ __forceinline__ void load_tile_staged(const char* tile_ptr, char* stage, T (&x)[kScanItems]) {
    constexpr int PPT = ScanStage<T>::kPacksPerThread;
    constexpr int V = 16 / sizeof(T);
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
        const int q = j * kBlock + threadIdx.x;                              // packet of the tile
        const int4 v = __ldcs(reinterpret_cast<const int4*>(tile_ptr) + q);
        *reinterpret_cast<int4*>(stage + (q / PPT) * ScanStage<T>::kStride + (q % PPT) * 16) = v;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
        Pack<T> v;
        *reinterpret_cast<int4*>(&v) = *reinterpret_cast<const int4*>(stage + threadIdx.x * ScanStage<T>::kStride + j * 16);
#pragma unroll
        for (int e = 0; e < V; ++e) x[j * V + e] = v.v[e];
    }
    __syncthreads();                                                          // the stage is reused for the way out
}

template <typename T>
__device__ __forceinline__ void store_tile_staged(char* tile_ptr, char* stage, const T (&x)[kScanItems]) {
    constexpr int PPT = ScanStage<T>::kPacksPerThread;
    constexpr int V = 16 / sizeof(T);
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
        Pack<T> v;
#pragma unroll
        for (int e = 0; e < V; ++e) v.v[e] = x[j * V + e];
        *reinterpret_cast<int4*>(stage + threadIdx.x * ScanStage<T>::kStride + j * 16) = *reinterpret_cast<const int4*>(&v);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
        const int q = j * kBlock + threadIdx.x;
        __stcs(reinterpret_cast<int4*>(tile_ptr) + q,
               *reinterpret_cast<const int4*>(stage + (q / PPT) * ScanStage<T>::kStride + (q % PPT) * 16));
    }
}

// pass 1: the fold of every CTA's run of `tiles_per_cta` consecutive tiles, in element order
template <typename T, typename Op>
__global__ void __launch_bounds__(kBlock)
scan_fold_kernel(const char* __restrict__ p1, int64_t s1, int64_t n, bool packed, int64_t tiles_per_cta, int64_t n_tiles, T* cta_sums) {
    __shared__ T smem[2 * kWarpsPerBlock];
    __shared__ T tile_fold_s;
    T running = T();                            // thread 0's: the fold of the tiles so far
    const int64_t t_begin = (int64_t)blockIdx.x * tiles_per_cta;
    int64_t t_end = t_begin + tiles_per_cta; if (t_end > n_tiles) t_end = n_tiles;
    for (int64_t tile = t_begin; tile < t_end; ++tile) {
        const int64_t first = tile * kScanTile + (int64_t)threadIdx.x * kScanItems;
        T x[kScanItems];
        load_items<T>(p1, s1, first, n, packed, x);           // (staging through shared memory measured slower for this read-only pass)
        T acc = x[0];                           // threads past the end hold zeros that never flow backwards
#pragma unroll
        for (int j = 1; j < kScanItems; ++j)
            if (first + j < n) acc = Op::combine(acc, x[j]);
        T before, total;
        block_scan<T, Op>(acc, &before, &total, smem);
        // the tile's fold is the inclusive value at the last thread that holds an element
        const int64_t last_elem = (tile + 1) * kScanTile <= n ? (tile + 1) * kScanTile - 1 : n - 1;
        const int last_thread = (int)((last_elem - tile * kScanTile) / kScanItems);
        if ((int)threadIdx.x == last_thread) tile_fold_s = threadIdx.x > 0 ? Op::combine(before, acc) : acc;
        __syncthreads();
        if (threadIdx.x == 0) running = tile == t_begin ? tile_fold_s : Op::combine(running, tile_fold_s);
        __syncthreads();
    }
    if (threadIdx.x == 0) cta_sums[blockIdx.x] = running;
}

// pass 2: inclusive scan of the tile folds, one CTA, kScanTile values per round
template <typename T, typename Op>
__global__ void __launch_bounds__(kBlock)
scan_tiles_kernel(T* tile_sums, int64_t n_tiles) {
    __shared__ T smem[2 * kWarpsPerBlock];
    __shared__ T carry_s;
    bool have_carry = false;
    T carry = T();
    for (int64_t base = 0; base < n_tiles; base += kScanTile) {
        const int64_t first = base + (int64_t)threadIdx.x * kScanItems;
        T x[kScanItems];
        load_items<T>(reinterpret_cast<const char*>(tile_sums), sizeof(T), first, n_tiles, false, x);
        T acc[kScanItems];
        acc[0] = x[0];
#pragma unroll
        for (int j = 1; j < kScanItems; ++j) acc[j] = first + j < n_tiles ? Op::combine(acc[j - 1], x[j]) : acc[j - 1];
        T before, total;
        block_scan<T, Op>(acc[kScanItems - 1], &before, &total, smem);
#pragma unroll
        for (int j = 0; j < kScanItems; ++j) {
            if (first + j >= n_tiles) break;
            T v = acc[j];
            if (threadIdx.x > 0) v = Op::combine(before, v);
            if (have_carry) v = Op::combine(carry, v);
            tile_sums[first + j] = v;
        }
        // the round's last value carries into the next round
        const int64_t last = base + kScanTile <= n_tiles ? base + kScanTile - 1 : n_tiles - 1;
        __syncthreads();
        if (first <= last && last < first + kScanItems) carry_s = tile_sums[last];
        __syncthreads();
        carry = carry_s;
        have_carry = true;
    }
}

// pass 3 (or the only pass of a short run): the scan itself, a CTA walking its tiles with the fold so far
template <typename T, typename Op>
__global__ void __launch_bounds__(kBlock, sizeof(T) <= 4 ? 4 : 3)      // 4 CTAs per SM measured 8 % faster than 3 for 4-byte elements
scan_write_kernel(const char* __restrict__ p1, int64_t s1, char* p2, int64_t s2, int64_t n, bool packed_in, bool packed_out,
                  int64_t tiles_per_cta, int64_t n_tiles, const T* __restrict__ cta_sums) {
    __shared__ T smem[2 * kWarpsPerBlock];
    __shared__ __align__(16) char stage[ScanStage<T>::kBytes];
    const int64_t t_begin = (int64_t)blockIdx.x * tiles_per_cta;
    int64_t t_end = t_begin + tiles_per_cta; if (t_end > n_tiles) t_end = n_tiles;
    bool have_carry = blockIdx.x > 0;            // everything before this CTA's first tile
    T carry = have_carry ? cta_sums[blockIdx.x - 1] : T();
    for (int64_t tile = t_begin; tile < t_end; ++tile) {
        const int64_t first = tile * kScanTile + (int64_t)threadIdx.x * kScanItems;
        const bool whole = (tile + 1) * kScanTile <= n;       // the same for every thread of the CTA
        T acc[kScanItems];                           // the elements, then their running fold in place
        if (packed_in && whole) load_tile_staged<T>(p1 + tile * kScanTile * (int64_t)sizeof(T), stage, acc);
        else load_items<T>(p1, s1, first, n, packed_in, acc);
#pragma unroll
        for (int j = 1; j < kScanItems; ++j) acc[j] = first + j < n ? Op::combine(acc[j - 1], acc[j]) : acc[j - 1];
        T before, total;
        block_scan<T, Op>(acc[kScanItems - 1], &before, &total, smem);
        T prefix = T();
        bool have_prefix = false;
        if (threadIdx.x > 0) { prefix = before; have_prefix = true; }
        if (have_carry) {
            prefix = have_prefix ? Op::combine(carry, prefix) : carry;
            have_prefix = true;
        }
        constexpr int V = 16 / sizeof(T);
        if (packed_out && whole) {
#pragma unroll
            for (int j = 0; j < kScanItems; ++j) acc[j] = have_prefix ? Op::combine(prefix, acc[j]) : acc[j];
            store_tile_staged<T>(p2 + tile * kScanTile * (int64_t)sizeof(T), stage, acc);
            __syncthreads();                             // the stage is loaded again for the next tile
        } else if (packed_out && first + kScanItems <= n) {
#pragma unroll
            for (int j = 0; j < kScanItems / V; ++j) {
                Pack<T> o;
#pragma unroll
                for (int e = 0; e < V; ++e) o.v[e] = have_prefix ? Op::combine(prefix, acc[j * V + e]) : acc[j * V + e];
                st_pack<T>(p2 + (first + j * V) * (int64_t)sizeof(T), o);
            }
        } else {
#pragma unroll
            for (int j = 0; j < kScanItems; ++j)
                if (first + j < n) *reinterpret_cast<T*>(p2 + (first + j) * s2) = have_prefix ? Op::combine(prefix, acc[j]) : acc[j];
        }
        // a whole tile's total is the inclusive value of its last thread (only the run's last tile can be partial)
        carry = have_carry ? Op::combine(carry, total) : total;
        have_carry = true;
    }
}

template <typename T, bool PROD, bool NANSKIP>
cudaError_t launch_scan(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n64) {
    using Op = ScanOp<T, PROD, NANSKIP>;
    if (n64 == 0) return cudaSuccess;
    const int64_t n = (int64_t)n64;
    cudaStream_t st = current_stream();
    const bool packed_in = s1 == (ssize_t)sizeof(T) && aligned16(p1);
    const bool packed_out = s2 == (ssize_t)sizeof(T) && aligned16(p2);
    const int64_t n_tiles = (n + kScanTile - 1) / kScanTile;
    if (n_tiles == 1) {
        scan_write_kernel<T, Op><<<1, kBlock, 0, st>>>(p1, s1, p2, s2, n, packed_in, packed_out, 1, 1, nullptr);
        count_launch();
        return cudaGetLastError();
    }
    // at most kScanTile CTAs, so that the middle pass is a single round of one CTA
    const int64_t tiles_per_cta = (n_tiles + kScanTile - 1) / kScanTile;
    const int64_t n_ctas = (n_tiles + tiles_per_cta - 1) / tiles_per_cta;
    T* cta_sums = reinterpret_cast<T*>(cumo_cuda_runtime_malloc(sizeof(T) * (size_t)n_ctas));
    if (!cta_sums) return cudaErrorMemoryAllocation;
    scan_fold_kernel<T, Op><<<(unsigned)n_ctas, kBlock, 0, st>>>(p1, s1, n, packed_in, tiles_per_cta, n_tiles, cta_sums);
    scan_tiles_kernel<T, Op><<<1, kBlock, 0, st>>>(cta_sums, n_ctas);
    scan_write_kernel<T, Op><<<(unsigned)n_ctas, kBlock, 0, st>>>(p1, s1, p2, s2, n, packed_in, packed_out, tiles_per_cta, n_tiles, cta_sums);
    count_launch(3);
    const cudaError_t e = cudaGetLastError();
    cumo_cuda_runtime_free(reinterpret_cast<char*>(cta_sums));      // stream-ordered reuse: later kernels queue behind these
    return e;
}

}  // namespace cb200

using namespace cb200;

#define CB200_DEF_CUM(T, C)                                                                                          \
    extern "C" cudaError_t cumo_##T##_cumsum_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n) {  \
        return launch_scan<C, false, false>(p1, p2, s1, s2, n); }                                                    \
    extern "C" cudaError_t cumo_##T##_cumprod_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n) { \
        return launch_scan<C, true, false>(p1, p2, s1, s2, n); }
#define CB200_DEF_CUM_NAN(T, C)                                                                                          \
    extern "C" cudaError_t cumo_##T##_cumsum_nan_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n) {  \
        return launch_scan<C, false, true>(p1, p2, s1, s2, n); }                                                         \
    extern "C" cudaError_t cumo_##T##_cumprod_nan_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n) { \
        return launch_scan<C, true, true>(p1, p2, s1, s2, n); }

CB200_DEF_CUM(sfloat, float)
CB200_DEF_CUM(dfloat, double)
CB200_DEF_CUM(int32, int32_t)
CB200_DEF_CUM(int64, int64_t)
CB200_DEF_CUM_NAN(sfloat, float)
CB200_DEF_CUM_NAN(dfloat, double)
