// cumsum / cumprod along one strided run: out[i] = x[0] (+|*) ... (+|*) x[i].
//
// Entry points are the reference's (narray/gen/tmpl/cum.c:3 declares them, cum_kernel.cu:56-80
// defines them on top of thrust::inclusive_scan): (p1, p2, s1, s2, n) with byte steps of any sign,
// returning a cudaError_t; the host side calls once per run (ndloop walks the other axes).
// The `_nan` forms use the reference's operator (include/cumo/types/real_accum_kernel.h:12-26):
// a NaN accumulator is replaced by the next value and a NaN value is skipped, i.e. NaN means
// "nothing yet" -- which makes it associative, so it can be scanned in parallel as it stands.
//
// Plan: tiles of 4096 elements, 16 consecutive elements per thread (four 16-byte loads when the
// run is contiguous).  Short runs are one CTA.  Longer runs take three launches with no waiting
// between CTAs: (1) every CTA folds its tile into one value, (2) one CTA scans those values,
// (3) every CTA scans its tile again starting from the value before it.  No identity element is
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

// pass 1: the fold of every tile, in element order
template <typename T, typename Op>
__global__ void __launch_bounds__(kBlock)
scan_fold_kernel(const char* __restrict__ p1, int64_t s1, int64_t n, bool packed, T* tile_sums) {
    __shared__ T smem[2 * kWarpsPerBlock];
    const int64_t tile = blockIdx.x;
    const int64_t first = tile * kScanTile + (int64_t)threadIdx.x * kScanItems;
    T x[kScanItems];
    load_items<T>(p1, s1, first, n, packed, x);
    T acc = x[0];                               // threads past the end carry garbage that never flows backwards
#pragma unroll
    for (int j = 1; j < kScanItems; ++j)
        if (first + j < n) acc = Op::combine(acc, x[j]);
    T before, total;
    block_scan<T, Op>(acc, &before, &total, smem);
    // the tile's fold is the inclusive value at the last thread that holds an element
    const int64_t last_elem = (tile + 1) * kScanTile <= n ? (tile + 1) * kScanTile - 1 : n - 1;
    const int last_thread = (int)((last_elem - tile * kScanTile) / kScanItems);
    if ((int)threadIdx.x == last_thread) tile_sums[tile] = threadIdx.x > 0 ? Op::combine(before, acc) : acc;
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

// pass 3 (or the only pass of a short run): the scan itself
template <typename T, typename Op>
__global__ void __launch_bounds__(kBlock)
scan_write_kernel(const char* __restrict__ p1, int64_t s1, char* p2, int64_t s2, int64_t n, bool packed_in, bool packed_out,
                  const T* __restrict__ tile_sums) {
    __shared__ T smem[2 * kWarpsPerBlock];
    const int64_t tile = blockIdx.x;
    const int64_t first = tile * kScanTile + (int64_t)threadIdx.x * kScanItems;
    T x[kScanItems];
    load_items<T>(p1, s1, first, n, packed_in, x);
    T acc[kScanItems];
    acc[0] = x[0];
#pragma unroll
    for (int j = 1; j < kScanItems; ++j) acc[j] = first + j < n ? Op::combine(acc[j - 1], x[j]) : acc[j - 1];
    T before, total;
    block_scan<T, Op>(acc[kScanItems - 1], &before, &total, smem);
    const bool have_tile = tile > 0;
    T prefix = T();
    bool have_prefix = false;
    if (threadIdx.x > 0) { prefix = before; have_prefix = true; }
    if (have_tile) {
        const T t = tile_sums[tile - 1];
        prefix = have_prefix ? Op::combine(t, prefix) : t;
        have_prefix = true;
    }
    constexpr int V = 16 / sizeof(T);
    if (packed_out && first + kScanItems <= n) {
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
    if (n_tiles > 0x7fffffffLL) return cudaErrorInvalidValue;
    if (n_tiles == 1) {
        scan_write_kernel<T, Op><<<1, kBlock, 0, st>>>(p1, s1, p2, s2, n, packed_in, packed_out, nullptr);
        count_launch();
        return cudaGetLastError();
    }
    T* tile_sums = reinterpret_cast<T*>(cumo_cuda_runtime_malloc(sizeof(T) * (size_t)n_tiles));
    if (!tile_sums) return cudaErrorMemoryAllocation;
    scan_fold_kernel<T, Op><<<(unsigned)n_tiles, kBlock, 0, st>>>(p1, s1, n, packed_in, tile_sums);
    scan_tiles_kernel<T, Op><<<1, kBlock, 0, st>>>(tile_sums, n_tiles);
    scan_write_kernel<T, Op><<<(unsigned)n_tiles, kBlock, 0, st>>>(p1, s1, p2, s2, n, packed_in, packed_out, tile_sums);
    count_launch(3);
    const cudaError_t e = cudaGetLastError();
    cumo_cuda_runtime_free(reinterpret_cast<char*>(tile_sums));      // stream-ordered reuse: later kernels queue behind these
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
