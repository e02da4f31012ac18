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
// tiles [t_begin, t_end) of one run, scanned in order by the CTA, starting from `carry` when there is one
template <typename T, typename Op>
__device__ __forceinline__ void scan_tiles_of_run(const char* __restrict__ p1, int64_t s1, char* p2, int64_t s2, int64_t n, bool packed_in,
                                                  bool packed_out, int64_t t_begin, int64_t t_end, bool have_carry, T carry, T* smem, char* stage) {
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

template <typename T, typename Op>
__global__ void __launch_bounds__(kBlock, sizeof(T) <= 4 ? 4 : 3)      // 4 CTAs per SM measured 8 % faster than 3 for 4-byte elements
scan_write_kernel(const char* __restrict__ p1, int64_t s1, char* p2, int64_t s2, int64_t n, bool packed_in, bool packed_out,
                  int64_t tiles_per_cta, int64_t n_tiles, const T* __restrict__ cta_sums) {
    __shared__ T smem[2 * kWarpsPerBlock];
    __shared__ __align__(16) char stage[ScanStage<T>::kBytes];
    const int64_t t_begin = (int64_t)blockIdx.x * tiles_per_cta;
    int64_t t_end = t_begin + tiles_per_cta; if (t_end > n_tiles) t_end = n_tiles;
    const bool have_carry = blockIdx.x > 0;      // everything before this CTA's first tile
    const T carry = have_carry ? cta_sums[blockIdx.x - 1] : T();
    scan_tiles_of_run<T, Op>(p1, s1, p2, s2, n, packed_in, packed_out, t_begin, t_end, have_carry, carry, smem, stage);
}

template <typename T, bool PROD, bool NANSKIP>
cudaError_t launch_scan(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n64);

// ---- many runs in one launch ---------------------------------------------------------------------------------------------
// `cumsum(axis: k)` of an array with other dimensions is one scan per run along k.  The reference's ndloop launches its
// scan once per run (cum.c:9-24); here the whole loop is one launch.  The other dimensions arrive as extents with the byte
// step of input and output; run r (row-major over them) starts at the two offsets they give.
struct ScanRuns {
    int nd;
    int64_t runs;
    int64_t shape[kMaxDim], step1[kMaxDim], step2[kMaxDim];
};

__device__ __forceinline__ void run_offsets(const ScanRuns& o, int64_t r, int64_t* off1, int64_t* off2) {
    int64_t a = 0, b = 0;
    for (int d = o.nd - 1; d >= 0; --d) {
        const int64_t n = o.shape[d];
        const int64_t k = d > 0 ? r % n : r;
        r = d > 0 ? r / n : 0;
        a += k * o.step1[d];
        b += k * o.step2[d];
    }
    *off1 = a;
    *off2 = b;
}

// ROWS: a CTA per run, walking the run's tiles in order with the fold so far (runs of a few hundred elements or more)
template <typename T, typename Op>
__global__ void __launch_bounds__(kBlock, sizeof(T) <= 4 ? 4 : 3)
scan_rows_kernel(const ScanRuns o, const char* __restrict__ p1, int64_t s1, char* p2, int64_t s2, int64_t n, bool packed_in, bool packed_out) {
    __shared__ T smem[2 * kWarpsPerBlock];
    __shared__ __align__(16) char stage[ScanStage<T>::kBytes];
    const int64_t n_tiles = (n + kScanTile - 1) / kScanTile;
    for (int64_t r = blockIdx.x; r < o.runs; r += gridDim.x) {
        int64_t off1, off2;
        run_offsets(o, r, &off1, &off2);
        scan_tiles_of_run<T, Op>(p1 + off1, s1, p2 + off2, s2, n, packed_in, packed_out, 0, n_tiles, false, T(), smem, stage);
        __syncthreads();
    }
}

// SHORT ROWS: runs of fewer than 256 elements that do not lie side by side (a scan along the contiguous axis of a matrix
// with short rows).  G lanes per run (the smallest power of two that covers the run, at most a warp), 32/G runs per warp at
// a time; the lanes of a group take consecutive elements, so a warp's loads and stores are consecutive memory when the rows
// are; runs longer than a warp go in chunks of 32 with the fold so far carried along.  Every chunk of a lane is loaded
// before the first shuffle.  No shared memory, no barrier.
constexpr int kShortMax = 256;
template <typename T, typename Op, int G, int CH>
__global__ void __launch_bounds__(kBlock)
scan_short_rows_kernel(const ScanRuns o, const char* __restrict__ p1, int64_t s1, char* p2, int64_t s2, int64_t n) {
    constexpr int R = 32 / G;                              // runs per warp and slot
    constexpr int U = 8 / CH;                              // slots per round: eight loads per lane in flight either way
    const int lane = threadIdx.x & 31, sub = lane % G;
    const int64_t warp = ((int64_t)blockIdx.x * kBlock + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * kBlock) >> 5;
    for (int64_t r0 = warp * (R * U); r0 < o.runs; r0 += n_warps * (R * U)) {
        T x[U][CH];
        int64_t off2[U];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t r = r0 + u * R + lane / G;
            live[u] = r < o.runs;
            int64_t off1 = 0;
            off2[u] = 0;
            if (live[u]) run_offsets(o, r, &off1, &off2[u]);
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                const int64_t j = (int64_t)k * G + sub;
                x[u][k] = (live[u] && j < n) ? *reinterpret_cast<const T*>(p1 + off1 + j * s1) : T();
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            T carry = T();
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                if ((int64_t)k * G >= n) break;            // the same for every lane
                const int64_t j = (int64_t)k * G + sub;
                T v = x[u][k];
#pragma unroll
                for (int d = 1; d < G; d <<= 1) {
                    const T before = __shfl_up_sync(0xffffffffu, v, d, G);
                    if (sub >= d) v = Op::combine(before, v);
                }
                if (k > 0) v = Op::combine(carry, v);
                if (live[u] && j < n) *reinterpret_cast<T*>(p2 + off2[u] + j * s2) = v;
                carry = __shfl_sync(0xffffffffu, v, G - 1, G);  // a chunk that is followed by another is a whole one
            }
        }
    }
}

// ... and when such short rows are contiguous, whole packets long and 16-byte aligned, a thread per run reading and writing
// its own run by packets, four at a time: a warp then has 32 neighbouring rows in flight instead of one to sixteen.
template <typename T, typename Op>
__global__ void __launch_bounds__(kBlock)
scan_thread_rows_kernel(const ScanRuns o, const char* __restrict__ p1, char* p2, int64_t n) {
    constexpr int V = 16 / (int)sizeof(T);
    const int64_t packets = n / V;
    for (int64_t r = (int64_t)blockIdx.x * kBlock + threadIdx.x; r < o.runs; r += (int64_t)gridDim.x * kBlock) {
        int64_t off1, off2;
        run_offsets(o, r, &off1, &off2);
        const char* src = p1 + off1;
        char* dst = p2 + off2;
        T acc = T();
        for (int64_t k0 = 0; k0 < packets; k0 += 4) {
            Pack<T> x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (k0 + u < packets) x[u] = ld_pack<T>(src + (k0 + u) * 16);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (k0 + u >= packets) break;
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    acc = (k0 + u == 0 && e == 0) ? x[u].v[e] : Op::combine(acc, x[u].v[e]);
                    x[u].v[e] = acc;
                }
                st_pack<T>(dst + (k0 + u) * 16, x[u]);
            }
        }
    }
}

// COLUMNS: a thread per run, in element order; consecutive threads are consecutive runs, so when the runs lie side by
// side in memory (a scan along an outer axis) every step of a warp is one coalesced access.  Loads run kColAhead
// elements ahead of the dependent chain of combines.
// V > 1: V runs that lie side by side per thread, one 16-byte packet of them per step (the launch checks the alignment).
constexpr int kColAhead = 8;

template <typename T, int V>
__device__ __forceinline__ void load_group(const char* q, T (&x)[V]) {
    if constexpr (V > 1) {
        const Pack<T> v = ld_pack<T>(q);
#pragma unroll
        for (int e = 0; e < V; ++e) x[e] = v.v[e];
    } else {
        x[0] = *reinterpret_cast<const T*>(q);
    }
}
template <typename T, int V>
__device__ __forceinline__ void store_group(char* q, const T (&x)[V]) {
    if constexpr (V > 1) {
        Pack<T> v;
#pragma unroll
        for (int e = 0; e < V; ++e) v.v[e] = x[e];
        st_pack<T>(q, v);
    } else {
        *reinterpret_cast<T*>(q) = x[0];
    }
}

template <typename T, typename Op, int V>
__global__ void __launch_bounds__(kBlock)
scan_columns_kernel(const ScanRuns o, const char* __restrict__ p1, int64_t s1, char* p2, int64_t s2, int64_t n) {
    constexpr int AHEAD = V > 1 ? kColAhead / 2 : kColAhead;
    const int64_t groups = o.runs / V;
    for (int64_t g = (int64_t)blockIdx.x * kBlock + threadIdx.x; g < groups; g += (int64_t)gridDim.x * kBlock) {
        int64_t off1, off2;
        run_offsets(o, g * V, &off1, &off2);
        const char* src = p1 + off1;
        char* dst = p2 + off2;
        T acc[V];
        for (int64_t j0 = 0; j0 < n; j0 += AHEAD) {
            T x[AHEAD][V];
#pragma unroll
            for (int k = 0; k < AHEAD; ++k)
                if (j0 + k < n) load_group<T, V>(src + (j0 + k) * s1, x[k]);
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                if (j0 + k >= n) break;
#pragma unroll
                for (int e = 0; e < V; ++e) acc[e] = (j0 + k == 0) ? x[k][e] : Op::combine(acc[e], x[k][e]);
                store_group<T, V>(dst + (j0 + k) * s2, acc);
            }
        }
    }
}

// COLUMNS with few runs (a scan down the rows of a matrix with a few thousand columns): a thread per run leaves most of
// the GPU idle, so every run is cut into `segs` segments of `seg_len` elements and a thread takes one (segment, run):
// (1) fold of each segment, (2) per run, the folds become the fold of everything before each segment, (3) the scan of
// each segment starting from that.  Consecutive threads are still consecutive runs, so every access stays coalesced.
template <typename T, typename Op, int V>
__global__ void __launch_bounds__(kBlock)
scan_columns_fold_kernel(const ScanRuns o, const char* __restrict__ p1, int64_t s1, int64_t n, int64_t seg_len, int64_t segs, T* partial) {
    constexpr int AHEAD = V > 1 ? kColAhead / 2 : kColAhead;
    const int64_t groups = o.runs / V;
    const int64_t total = segs * groups;
    for (int64_t t = (int64_t)blockIdx.x * kBlock + threadIdx.x; t < total; t += (int64_t)gridDim.x * kBlock) {
        const int64_t seg = t / groups, r = (t - seg * groups) * V;
        int64_t off1, off2;
        run_offsets(o, r, &off1, &off2);
        const char* src = p1 + off1;
        const int64_t j_begin = seg * seg_len;
        const int64_t j_end = j_begin + seg_len < n ? j_begin + seg_len : n;
        T acc[V];
        for (int64_t j0 = j_begin; j0 < j_end; j0 += AHEAD) {
            T x[AHEAD][V];
#pragma unroll
            for (int k = 0; k < AHEAD; ++k)
                if (j0 + k < j_end) load_group<T, V>(src + (j0 + k) * s1, x[k]);
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                if (j0 + k >= j_end) break;
#pragma unroll
                for (int e = 0; e < V; ++e) acc[e] = (j0 + k == j_begin) ? x[k][e] : Op::combine(acc[e], x[k][e]);
            }
        }
#pragma unroll
        for (int e = 0; e < V; ++e) partial[seg * o.runs + r + e] = acc[e];
    }
}

template <typename T, typename Op>
__global__ void __launch_bounds__(kBlock)
scan_columns_carry_kernel(int64_t runs, int64_t segs, T* partial) {
    for (int64_t r = (int64_t)blockIdx.x * kBlock + threadIdx.x; r < runs; r += (int64_t)gridDim.x * kBlock) {
        T acc = partial[r];
        for (int64_t seg0 = 1; seg0 < segs; seg0 += kColAhead) {
            T mine[kColAhead];                              // the loads do not depend on the chain of combines: fetch ahead
#pragma unroll
            for (int k = 0; k < kColAhead; ++k)
                if (seg0 + k < segs) mine[k] = partial[(seg0 + k) * runs + r];
#pragma unroll
            for (int k = 0; k < kColAhead; ++k) {
                if (seg0 + k >= segs) break;
                partial[(seg0 + k) * runs + r] = acc;      // everything before this segment
                acc = Op::combine(acc, mine[k]);
            }
        }
    }
}

template <typename T, typename Op, int V>
__global__ void __launch_bounds__(kBlock)
scan_columns_write_kernel(const ScanRuns o, const char* __restrict__ p1, int64_t s1, char* p2, int64_t s2, int64_t n, int64_t seg_len, int64_t segs,
                          const T* __restrict__ partial) {
    constexpr int AHEAD = V > 1 ? kColAhead / 2 : kColAhead;
    const int64_t groups = o.runs / V;
    const int64_t total = segs * groups;
    for (int64_t t = (int64_t)blockIdx.x * kBlock + threadIdx.x; t < total; t += (int64_t)gridDim.x * kBlock) {
        const int64_t seg = t / groups, r = (t - seg * groups) * V;
        int64_t off1, off2;
        run_offsets(o, r, &off1, &off2);
        const char* src = p1 + off1;
        char* dst = p2 + off2;
        const int64_t j_begin = seg * seg_len;
        const int64_t j_end = j_begin + seg_len < n ? j_begin + seg_len : n;
        const bool have_carry = seg > 0;
        T acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = have_carry ? partial[seg * o.runs + r + e] : T();
        for (int64_t j0 = j_begin; j0 < j_end; j0 += AHEAD) {
            T x[AHEAD][V];
#pragma unroll
            for (int k = 0; k < AHEAD; ++k)
                if (j0 + k < j_end) load_group<T, V>(src + (j0 + k) * s1, x[k]);
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                if (j0 + k >= j_end) break;
#pragma unroll
                for (int e = 0; e < V; ++e) acc[e] = (j0 + k == j_begin && !have_carry) ? x[k][e] : Op::combine(acc[e], x[k][e]);
                store_group<T, V>(dst + (j0 + k) * s2, acc);
            }
        }
    }
}

template <typename T, bool PROD, bool NANSKIP>
cudaError_t launch_scan_runs(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n64, int n_outer, const size_t* oshape,
                             const ssize_t* ostep1, const ssize_t* ostep2) {
    using Op = ScanOp<T, PROD, NANSKIP>;
    if (n64 == 0 || n_outer < 0 || n_outer > kMaxDim) return n64 == 0 ? cudaSuccess : cudaErrorInvalidValue;
    ScanRuns o;
    o.nd = 0;
    o.runs = 1;
    bool steps16 = true, side_by_side = false;
    for (int d = 0; d < kMaxDim; ++d) { o.shape[d] = 1; o.step1[d] = o.step2[d] = 0; }
    for (int d = 0; d < n_outer; ++d) {
        if (oshape[d] == 0) return cudaSuccess;
        if (oshape[d] == 1) continue;
        o.shape[o.nd] = (int64_t)oshape[d]; o.step1[o.nd] = (int64_t)ostep1[d]; o.step2[o.nd] = (int64_t)ostep2[d];
        o.runs *= o.shape[o.nd];
        if (!mult16(o.step1[o.nd]) || !mult16(o.step2[o.nd])) steps16 = false;
        ++o.nd;
    }
    if (o.nd > 0) side_by_side = o.step1[o.nd - 1] == (int64_t)sizeof(T) && o.step2[o.nd - 1] == (int64_t)sizeof(T);
    const int64_t n = (int64_t)n64;
    cudaStream_t st = current_stream();
    if (o.runs == 1) return launch_scan<T, PROD, NANSKIP>(p1, p2, s1, s2, n64);
    if (!side_by_side && n < kShortMax && s1 == (ssize_t)sizeof(T) && s2 == (ssize_t)sizeof(T) && n % (16 / (int64_t)sizeof(T)) == 0 && steps16 &&
        aligned16(p1) && aligned16(p2) && o.runs >= (int64_t)sm_count() * 512) {
        scan_thread_rows_kernel<T, Op><<<grid_for((o.runs + kBlock - 1) / kBlock, 8), kBlock, 0, st>>>(o, p1, p2, n);
    } else if (!side_by_side && n < kShortMax) {
        int g = 1;
        while (g < 32 && g < n) g <<= 1;
        const int chunks = g < 32 ? 1 : (int)((n + 31) / 32);
        const int ch = chunks <= 1 ? 1 : chunks <= 2 ? 2 : chunks <= 4 ? 4 : 8;
        const int64_t per_warp = (int64_t)(32 / g) * (8 / ch);
        const int64_t warps = (o.runs + per_warp - 1) / per_warp;
        const unsigned grid = grid_for((warps + kBlock / 32 - 1) / (kBlock / 32), 8);
        switch (g) {
        case 1: case 2: scan_short_rows_kernel<T, Op, 2, 1><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n); break;
        case 4:  scan_short_rows_kernel<T, Op, 4, 1><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n); break;
        case 8:  scan_short_rows_kernel<T, Op, 8, 1><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n); break;
        case 16: scan_short_rows_kernel<T, Op, 16, 1><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n); break;
        default:
            if (ch == 1)      scan_short_rows_kernel<T, Op, 32, 1><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n);
            else if (ch == 2) scan_short_rows_kernel<T, Op, 32, 2><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n);
            else if (ch == 4) scan_short_rows_kernel<T, Op, 32, 4><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n);
            else              scan_short_rows_kernel<T, Op, 32, 8><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n);
            break;
        }
    } else if (!side_by_side && n >= 256) {
        const bool packed_in = s1 == (ssize_t)sizeof(T) && aligned16(p1) && steps16;
        const bool packed_out = s2 == (ssize_t)sizeof(T) && aligned16(p2) && steps16;
        scan_rows_kernel<T, Op><<<grid_for(o.runs, sizeof(T) <= 4 ? 4 : 3), kBlock, 0, st>>>(o, p1, s1, p2, s2, n, packed_in, packed_out);
    } else {
        // groups of V runs that lie side by side go by 16-byte packets when every access stays aligned
        constexpr int VMAX = 16 / (int)sizeof(T);
        bool wide = side_by_side && o.shape[o.nd - 1] % VMAX == 0 && aligned16(p1) && aligned16(p2) && mult16(s1) && mult16(s2);
        for (int d = 0; d + 1 < o.nd && wide; ++d) wide = mult16(o.step1[d]) && mult16(o.step2[d]);
        const int64_t groups = wide ? o.runs / VMAX : o.runs;
        // enough threads to fill the GPU: cut the runs into segments of at least 64 elements when the runs alone are too few
        const int64_t wanted = (int64_t)sm_count() * 2048;
        int64_t segs = (wanted + groups - 1) / groups;
        if (segs > n / 64) segs = n / 64;
        if (segs >= 2) {
            const int64_t seg_len = (n + segs - 1) / segs;
            segs = (n + seg_len - 1) / seg_len;
            const int64_t total = segs * groups;
            T* partial = reinterpret_cast<T*>(cumo_cuda_runtime_malloc(sizeof(T) * (size_t)(segs * o.runs)));
            if (!partial) return cudaErrorMemoryAllocation;
            const unsigned grid = grid_for((total + kBlock - 1) / kBlock, 8);
            if (wide) scan_columns_fold_kernel<T, Op, VMAX><<<grid, kBlock, 0, st>>>(o, p1, s1, n, seg_len, segs, partial);
            else scan_columns_fold_kernel<T, Op, 1><<<grid, kBlock, 0, st>>>(o, p1, s1, n, seg_len, segs, partial);
            scan_columns_carry_kernel<T, Op><<<grid_for((o.runs + kBlock - 1) / kBlock, 8), kBlock, 0, st>>>(o.runs, segs, partial);
            if (wide) scan_columns_write_kernel<T, Op, VMAX><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n, seg_len, segs, partial);
            else scan_columns_write_kernel<T, Op, 1><<<grid, kBlock, 0, st>>>(o, p1, s1, p2, s2, n, seg_len, segs, partial);
            count_launch(3);
            const cudaError_t e = cudaGetLastError();
            cumo_cuda_runtime_free(reinterpret_cast<char*>(partial));     // stream-ordered reuse: later kernels queue behind these
            return e;
        }
        if (wide) scan_columns_kernel<T, Op, VMAX><<<grid_for((groups + kBlock - 1) / kBlock, 8), kBlock, 0, st>>>(o, p1, s1, p2, s2, n);
        else scan_columns_kernel<T, Op, 1><<<grid_for((groups + kBlock - 1) / kBlock, 8), kBlock, 0, st>>>(o, p1, s1, p2, s2, n);
    }
    count_launch();
    return cudaGetLastError();
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

#define CB200_RUNS_ARGS char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n, int n_outer, const size_t* outer_shape, const ssize_t* outer_step1, const ssize_t* outer_step2
#define CB200_RUNS_PASS p1, p2, s1, s2, n, n_outer, outer_shape, outer_step1, outer_step2
#define CB200_DEF_CUM(T, C)                                                                                          \
    extern "C" cudaError_t cb200_##T##_cumsum_runs_kernel_launch(CB200_RUNS_ARGS) { return launch_scan_runs<C, false, false>(CB200_RUNS_PASS); }  \
    extern "C" cudaError_t cb200_##T##_cumprod_runs_kernel_launch(CB200_RUNS_ARGS) { return launch_scan_runs<C, true, false>(CB200_RUNS_PASS); }  \
    extern "C" cudaError_t cumo_##T##_cumsum_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n) {  \
        return launch_scan<C, false, false>(p1, p2, s1, s2, n); }                                                    \
    extern "C" cudaError_t cumo_##T##_cumprod_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n) { \
        return launch_scan<C, true, false>(p1, p2, s1, s2, n); }
#define CB200_DEF_CUM_NAN(T, C)                                                                                          \
    extern "C" cudaError_t cb200_##T##_cumsum_nan_runs_kernel_launch(CB200_RUNS_ARGS) { return launch_scan_runs<C, false, true>(CB200_RUNS_PASS); }  \
    extern "C" cudaError_t cb200_##T##_cumprod_nan_runs_kernel_launch(CB200_RUNS_ARGS) { return launch_scan_runs<C, true, true>(CB200_RUNS_PASS); }  \
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
