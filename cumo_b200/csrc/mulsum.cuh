// mulsum: sum of elementwise products along one axis (the non-BLAS `dot`).
// Replaces ext/cumo/narray/gen/tmpl/accum_binary_kernel.cu:27-92 (<=1024 blocks of
// 512 threads with scalar loads, then a one-block combine).  Here: 16-byte loads
// when both operands are contiguous and aligned, a CTA per segment with enough
// segments to fill the device, partials folded in segment order by one warp.
// The accumulator has the element type, as in the reference (integers wrap).
#pragma once

#include "common.cuh"
#include "reduce.cuh"

namespace cb200 {

template <typename T, bool NAN_SKIP>
struct MulSumR {     // only the pieces group_fold/warp_fold need
    using In = T;
    using Acc = T;
    __device__ __forceinline__ Acc identity() const { return (T)0; }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return a + b; }
    __device__ __forceinline__ static void fma_into(T x, T y, T& acc) {
        if (NAN_SKIP) { if (x == x && y == y) acc = x * y + acc; }
        else acc = x * y + acc;
    }
};

template <typename T, bool NAN_SKIP, int V>
__global__ void __launch_bounds__(kBlock)
mulsum_partial_kernel(const char* __restrict__ p1, const char* __restrict__ p2, int64_t s1, int64_t s2,
                      int64_t n, int64_t seg_len, T* partial, T* out) {
    using R = MulSumR<T, NAN_SKIP>;
    constexpr int ES = sizeof(T);
    __shared__ T smem[kWarpsPerBlock];
    R r;
    const int64_t begin = (int64_t)blockIdx.x * seg_len;
    int64_t end = begin + seg_len; if (end > n) end = n;
    T acc = 0;
    for (int64_t e0 = begin + (int64_t)threadIdx.x * V; e0 < end; e0 += (int64_t)kBlock * V * kUnroll) {
        Pack<T> x[kUnroll], y[kUnroll];
        int nv[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            int64_t e = e0 + (int64_t)j * kBlock * V;
            int64_t left = end - e;
            nv[j] = left >= V ? V : (left > 0 ? (int)left : 0);
            if (V > 1 && nv[j] == V) { x[j] = ld_pack<T>(p1 + e * ES); y[j] = ld_pack<T>(p2 + e * ES); }
            else {
#pragma unroll
                for (int k = 0; k < V; ++k) if (k < nv[j]) {
                    x[j].v[k] = ld_one<T>(p1 + (e + k) * s1);
                    y[j].v[k] = ld_one<T>(p2 + (e + k) * s2);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kUnroll; ++j)
#pragma unroll
            for (int k = 0; k < V; ++k) if (k < nv[j]) R::fma_into(x[j].v[k], y[j].v[k], acc);
    }
    acc = group_fold<R, kBlock>(r, acc, smem);
    if (threadIdx.x == 0) {
        if (partial) partial[blockIdx.x] = acc;
        else *out = *out + acc;
    }
}

template <typename T, bool NAN_SKIP>
__global__ void __launch_bounds__(32)
mulsum_fold_kernel(const T* __restrict__ partial, int n_seg, T* out) {
    MulSumR<T, NAN_SKIP> r;
    const int lane = threadIdx.x;
    const int per = (n_seg + 31) / 32;
    T acc = 0;
    for (int k = 0; k < per; ++k) { int s = lane * per + k; if (s < n_seg) acc += partial[s]; }
    acc = warp_fold(r, acc);
    if (lane == 0) *out = *out + acc;
}

template <typename T, bool NAN_SKIP>
__global__ void __launch_bounds__(kBlock)
mulsum_each_kernel(const char* __restrict__ p1, const char* __restrict__ p2, char* p3, int64_t s1, int64_t s2,
                   int64_t s3, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (int64_t)gridDim.x * kBlock) {
        T x = ld_one<T>(p1 + i * s1), y = ld_one<T>(p2 + i * s2);
        T* z = reinterpret_cast<T*>(p3 + i * s3);
        T acc = *z;
        MulSumR<T, NAN_SKIP>::fma_into(x, y, acc);
        *z = acc;
    }
}

template <typename T, bool NAN_SKIP>
void launch_mulsum_reduce(char* p1, char* p2, char* p3, ssize_t s1, ssize_t s2, uint64_t n) {
    CB200_TRACE_LAUNCH();
    constexpr int ES = sizeof(T);
    constexpr int VMAX = 16 / ES;
    cudaStream_t st = current_stream();
    const bool vec = s1 == ES && s2 == ES && aligned16(p1) && aligned16(p2);
    // fixed 32 KiB segments, one CTA each, doubled until one warp can fold the partials
    int64_t seg_len = (32 << 10) / ES;
    int64_t n_seg = ((int64_t)n + seg_len - 1) / seg_len;
    while (n_seg > 4096) { seg_len *= 2; n_seg = ((int64_t)n + seg_len - 1) / seg_len; }
    if (n_seg < 1) n_seg = 1;
    T* partial = nullptr;
    if (n_seg > 1) {
        partial = reinterpret_cast<T*>(cumo_cuda_runtime_malloc(sizeof(T) * n_seg));
        if (!partial) return;          // the allocator reported it; several CTAs adding into *p3 without partials would be wrong
    }
    if (vec) mulsum_partial_kernel<T, NAN_SKIP, VMAX><<<(unsigned)n_seg, kBlock, 0, st>>>(p1, p2, s1, s2, (int64_t)n, seg_len, partial, reinterpret_cast<T*>(p3));
    else     mulsum_partial_kernel<T, NAN_SKIP, 1><<<(unsigned)n_seg, kBlock, 0, st>>>(p1, p2, s1, s2, (int64_t)n, seg_len, partial, reinterpret_cast<T*>(p3));
    int launches = 1;
    if (partial) {
        mulsum_fold_kernel<T, NAN_SKIP><<<1, 32, 0, st>>>(partial, (int)n_seg, reinterpret_cast<T*>(p3));
        cumo_cuda_runtime_free(reinterpret_cast<char*>(partial));
        ++launches;
    }
    count_launch(launches);
    cumo_cuda_runtime_check_kernel_launch();
}

template <typename T, bool NAN_SKIP>
void launch_mulsum_each(char* p1, char* p2, char* p3, ssize_t s1, ssize_t s2, ssize_t s3, uint64_t n) {
    CB200_TRACE_LAUNCH();
    if (n == 0) return;
    int64_t blocks = ((int64_t)n + kBlock - 1) / kBlock;
    mulsum_each_kernel<T, NAN_SKIP><<<grid_for(blocks, 8), kBlock, 0, current_stream()>>>(p1, p2, p3, s1, s2, s3, (int64_t)n);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200

// ---- many outputs in one launch ----------------------------------------------------------------------------------------------
// `a.mulsum(b, axis: k)` of arrays with other dimensions is one sum of products per output element.  The reference's
// ndloop calls its iterator once per innermost run (gen/tmpl/accum_binary.c:9-46): the integer `dot` of two matrices,
// which is a mulsum over a new axis (lib/cumo/narray/extra.rb:1145-1196), is one launch per element of the result.
// Here the whole loop is one launch: the kept dimensions with the byte steps of both inputs and of the output, the summed
// dimensions with the byte steps of both inputs; each output gets the sum added to it.
namespace cb200 {

struct MulSumAxes {
    int n_keep, n_red;
    int64_t outputs, reduced;
    int64_t kshape[kMaxDim], ks1[kMaxDim], ks2[kMaxDim], ks3[kMaxDim];
    int64_t rshape[kMaxDim], rs1[kMaxDim], rs2[kMaxDim];
};

__device__ __forceinline__ void mulsum_output_of(const MulSumAxes& c, int64_t o, int64_t* o1, int64_t* o2, int64_t* o3) {
    int64_t a = 0, b = 0, q = 0, r = o;
    for (int d = c.n_keep - 1; d >= 0; --d) {
        const int64_t n = c.kshape[d];
        const int64_t k = d > 0 ? r % n : r;
        r = d > 0 ? r / n : 0;
        a += k * c.ks1[d]; b += k * c.ks2[d]; q += k * c.ks3[d];
    }
    *o1 = a; *o2 = b; *o3 = q;
}

__device__ __forceinline__ void mulsum_reduced_of(const MulSumAxes& c, int64_t j, int upto, int64_t* o1, int64_t* o2) {
    int64_t a = 0, b = 0, r = j;
    for (int d = upto; d >= 0; --d) {
        const int64_t n = c.rshape[d];
        const int64_t k = d > 0 ? r % n : r;
        r = d > 0 ? r / n : 0;
        a += k * c.rs1[d]; b += k * c.rs2[d];
    }
    *o1 = a; *o2 = b;
}

// ROWS: the innermost summed dimension is long: G threads per output (a warp, or the whole CTA for long sums) stride over it
// VEC: both inputs contiguous along the summed dimension with every run starting on a 16-byte boundary and holding whole
// packets: 16-byte loads, two packets per input in flight per thread.
template <typename T, bool NAN_SKIP, int G, bool VEC>
__global__ void __launch_bounds__(kBlock)
mulsum_rows_kernel(const MulSumAxes c, const char* __restrict__ p1, const char* __restrict__ p2, char* p3) {
    using R = MulSumR<T, NAN_SKIP>;
    __shared__ T smem[kWarpsPerBlock];
    R r;
    const int last = c.n_red - 1;
    const int64_t run = c.rshape[last];
    const int64_t runs = c.reduced / run;
    const int64_t s1 = c.rs1[last], s2 = c.rs2[last];
    const int member = threadIdx.x % G;
    const int64_t group = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / G;
    const int64_t n_groups = (int64_t)gridDim.x * kBlock / G;
    for (int64_t o = group; o < c.outputs; o += n_groups) {
        int64_t o1, o2, o3;
        mulsum_output_of(c, o, &o1, &o2, &o3);
        T acc = 0;
        for (int64_t j = 0; j < runs; ++j) {
            int64_t a = 0, b = 0;
            if (last > 0) mulsum_reduced_of(c, j, last - 1, &a, &b);
            const char* q1 = p1 + o1 + a;
            const char* q2 = p2 + o2 + b;
            if constexpr (VEC) {
                constexpr int V = 16 / (int)sizeof(T);
                const int64_t packets = run / V;
                for (int64_t k0 = member; k0 < packets; k0 += (int64_t)G * 2) {
                    Pack<T> x[2], y[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int64_t k = k0 + (int64_t)u * G;
                        if (k < packets) { x[u] = ld_pack<T>(q1 + k * 16); y[u] = ld_pack<T>(q2 + k * 16); }
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        if (k0 + (int64_t)u * G >= packets) break;
#pragma unroll
                        for (int e = 0; e < V; ++e) R::fma_into(x[u].v[e], y[u].v[e], acc);
                    }
                }
                continue;
            }
            for (int64_t e0 = member; e0 < run; e0 += (int64_t)G * 4) {
                T x[4], y[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int64_t e = e0 + (int64_t)u * G;
                    if (e < run) { x[u] = ld_one<T>(q1 + e * s1); y[u] = ld_one<T>(q2 + e * s2); }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (e0 + (int64_t)u * G < run) R::fma_into(x[u], y[u], acc);
            }
        }
        if (G == 32) acc = warp_fold(r, acc);
        else { acc = group_fold<R, kBlock>(r, acc, smem); __syncthreads(); }
        if (member == 0) {
            T* z = reinterpret_cast<T*>(p3 + o3);
            *z = *z + acc;
        }
    }
}

// COLUMNS: a thread per (slice, V consecutive outputs) walking its part of the summed elements in order; consecutive threads
// are consecutive outputs.  V > 1 when the innermost kept dimension is contiguous (or repeated) in both inputs and in the
// output and everything is 16-byte aligned: one packet of each input per step.  With one slice the sums are added to the
// outputs; with more the partial sums go to `partial` (V per thread, side by side) for the fold below.
template <typename T, bool NAN_SKIP, int V>
__global__ void __launch_bounds__(kBlock)
mulsum_columns_kernel(const MulSumAxes c, const char* __restrict__ p1, const char* __restrict__ p2, char* p3, int64_t slice_len, int64_t slices, T* partial) {
    using R = MulSumR<T, NAN_SKIP>;
    const int64_t groups = c.outputs / V;
    const int64_t total = slices * groups;
    const bool wide1 = V > 1 && c.ks1[c.n_keep - 1] != 0, wide2 = V > 1 && c.ks2[c.n_keep - 1] != 0;
    for (int64_t t = (int64_t)blockIdx.x * kBlock + threadIdx.x; t < total; t += (int64_t)gridDim.x * kBlock) {
        const int64_t sl = t / groups, o = (t - sl * groups) * V;
        int64_t o1, o2, o3;
        mulsum_output_of(c, o, &o1, &o2, &o3);
        const int64_t j_begin = sl * slice_len;
        const int64_t j_end = j_begin + slice_len < c.reduced ? j_begin + slice_len : c.reduced;
        T acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0;
        for (int64_t j0 = j_begin; j0 < j_end; j0 += 4) {
            Pack<T> x[4], y[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (j0 + u >= j_end) break;
                int64_t a, b;
                if (c.n_red == 1) { a = (j0 + u) * c.rs1[0]; b = (j0 + u) * c.rs2[0]; }
                else mulsum_reduced_of(c, j0 + u, c.n_red - 1, &a, &b);
                if (wide1) x[u] = ld_pack<T>(p1 + o1 + a);
                else { const T v = ld_one<T>(p1 + o1 + a);
#pragma unroll
                       for (int e = 0; e < V; ++e) x[u].v[e] = v; }
                if (wide2) y[u] = ld_pack<T>(p2 + o2 + b);
                else { const T v = ld_one<T>(p2 + o2 + b);
#pragma unroll
                       for (int e = 0; e < V; ++e) y[u].v[e] = v; }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (j0 + u >= j_end) break;
#pragma unroll
                for (int e = 0; e < V; ++e) R::fma_into(x[u].v[e], y[u].v[e], acc[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < V; ++e) {
            if (partial) partial[sl * c.outputs + o + e] = acc[e];
            else { T* z = reinterpret_cast<T*>(p3 + o3) + e; *z = *z + acc[e]; }
        }
    }
}

// SHORT ROWS: one summed dimension, contiguous in both inputs, of fewer than 64 elements in whole 16-byte packets: a thread per
// output reading its own run by packets, four of each input in flight (a warp then covers 32 neighbouring rows).
template <typename T, bool NAN_SKIP>
__global__ void __launch_bounds__(kBlock)
mulsum_shortrows_kernel(const MulSumAxes c, const char* __restrict__ p1, const char* __restrict__ p2, char* p3) {
    using R = MulSumR<T, NAN_SKIP>;
    constexpr int V = 16 / (int)sizeof(T);
    const int64_t packets = c.rshape[0] / V;
    for (int64_t o = (int64_t)blockIdx.x * kBlock + threadIdx.x; o < c.outputs; o += (int64_t)gridDim.x * kBlock) {
        int64_t o1, o2, o3;
        mulsum_output_of(c, o, &o1, &o2, &o3);
        const char* q1 = p1 + o1;
        const char* q2 = p2 + o2;
        T acc = 0;
        for (int64_t k0 = 0; k0 < packets; k0 += 4) {
            Pack<T> x[4], y[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (k0 + u < packets) { x[u] = ld_pack<T>(q1 + (k0 + u) * 16); y[u] = ld_pack<T>(q2 + (k0 + u) * 16); }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (k0 + u >= packets) break;
#pragma unroll
                for (int e = 0; e < V; ++e) R::fma_into(x[u].v[e], y[u].v[e], acc);
            }
        }
        T* z = reinterpret_cast<T*>(p3 + o3);
        *z = *z + acc;
    }
}

template <typename T>
__global__ void __launch_bounds__(kBlock)
mulsum_slices_fold_kernel(const MulSumAxes c, const T* __restrict__ partial, int64_t slices, char* p3) {
    for (int64_t o = (int64_t)blockIdx.x * kBlock + threadIdx.x; o < c.outputs; o += (int64_t)gridDim.x * kBlock) {
        int64_t o1, o2, o3;
        mulsum_output_of(c, o, &o1, &o2, &o3);
        T acc = partial[o];
        for (int64_t sl = 1; sl < slices; ++sl) acc += partial[sl * c.outputs + o];         // slice order: the same sum every run
        T* z = reinterpret_cast<T*>(p3 + o3);
        *z = *z + acc;
    }
}

template <typename T, bool NAN_SKIP>
void launch_mulsum_axes(char* p1, char* p2, char* p3, int n_keep, const size_t* kshape, const ssize_t* ks1, const ssize_t* ks2, const ssize_t* ks3,
                        int n_red, const size_t* rshape, const ssize_t* rs1, const ssize_t* rs2) {
    CB200_TRACE_LAUNCH();
    if (n_keep < 0 || n_red < 0 || n_keep > kMaxDim || n_red > kMaxDim) return;
    MulSumAxes c;
    c.n_keep = 0; c.n_red = 0; c.outputs = 1; c.reduced = 1;
    for (int d = 0; d < kMaxDim; ++d) { c.kshape[d] = c.rshape[d] = 1; c.ks1[d] = c.ks2[d] = c.ks3[d] = c.rs1[d] = c.rs2[d] = 0; }
    for (int d = 0; d < n_keep; ++d) {
        if (kshape[d] == 0) return;
        if (kshape[d] == 1) continue;
        c.kshape[c.n_keep] = (int64_t)kshape[d]; c.ks1[c.n_keep] = ks1[d]; c.ks2[c.n_keep] = ks2[d]; c.ks3[c.n_keep] = ks3[d];
        c.outputs *= c.kshape[c.n_keep++];
    }
    for (int d = 0; d < n_red; ++d) {
        if (rshape[d] == 0) return;                         // an empty sum adds nothing
        if (rshape[d] == 1) continue;
        c.rshape[c.n_red] = (int64_t)rshape[d]; c.rs1[c.n_red] = rs1[d]; c.rs2[c.n_red] = rs2[d];
        c.reduced *= c.rshape[c.n_red++];
    }
    if (c.n_red == 0) c.n_red = 1;                          // every output is one product
    cudaStream_t st = current_stream();
    const int last = c.n_red - 1;
    int launches = 1;
    // rows only when the lanes' consecutive elements are consecutive in memory (or repeated) in both inputs; a summed
    // dimension with a long step is better walked by one thread per output, whose neighbours then share each line
    constexpr int64_t ES = sizeof(T);
    const bool along = (c.rs1[last] == ES || c.rs1[last] == 0) && (c.rs2[last] == ES || c.rs2[last] == 0);
    if (along && c.rshape[last] >= 64) {
        bool vec = c.rs1[last] == ES && c.rs2[last] == ES && aligned16(p1) && aligned16(p2) && c.rshape[last] % (16 / ES) == 0;
        for (int d = 0; d < c.n_keep && vec; ++d) vec = mult16(c.ks1[d]) && mult16(c.ks2[d]);
        for (int d = 0; d < last && vec; ++d) vec = mult16(c.rs1[d]) && mult16(c.rs2[d]);
        const unsigned g_cta = grid_for(c.outputs, 8), g_warp = grid_for((c.outputs + kBlock / 32 - 1) / (kBlock / 32), 8);
        if (c.rshape[last] >= 8192) {
            if (vec) mulsum_rows_kernel<T, NAN_SKIP, kBlock, true><<<g_cta, kBlock, 0, st>>>(c, p1, p2, p3);
            else mulsum_rows_kernel<T, NAN_SKIP, kBlock, false><<<g_cta, kBlock, 0, st>>>(c, p1, p2, p3);
        } else {
            if (vec) mulsum_rows_kernel<T, NAN_SKIP, 32, true><<<g_warp, kBlock, 0, st>>>(c, p1, p2, p3);
            else mulsum_rows_kernel<T, NAN_SKIP, 32, false><<<g_warp, kBlock, 0, st>>>(c, p1, p2, p3);
        }
    } else if (along && c.n_red == 1 && c.rs1[0] == ES && c.rs2[0] == ES && c.rshape[0] % (16 / ES) == 0 && aligned16(p1) && aligned16(p2) &&
               c.outputs >= (int64_t)sm_count() * 512 && [&] {
                   for (int d = 0; d < c.n_keep; ++d) if (!mult16(c.ks1[d]) || !mult16(c.ks2[d])) return false;
                   return true; }()) {
        mulsum_shortrows_kernel<T, NAN_SKIP><<<grid_for((c.outputs + kBlock - 1) / kBlock, 8), kBlock, 0, st>>>(c, p1, p2, p3);
    } else {
        const int64_t wanted = (int64_t)sm_count() * 2048;
        int64_t slices = (wanted + c.outputs - 1) / c.outputs;
        if (slices > c.reduced / 64) slices = c.reduced / 64;
        if (slices < 1) slices = 1;
        const int64_t slice_len = (c.reduced + slices - 1) / slices;
        slices = (c.reduced + slice_len - 1) / slice_len;
        T* partial = nullptr;
        if (slices > 1) {
            partial = reinterpret_cast<T*>(cumo_cuda_runtime_malloc(sizeof(T) * (size_t)(slices * c.outputs)));
            if (!partial) return;
        }
        constexpr int VMAX = 16 / (int)ES;
        const int lk = c.n_keep - 1;
        bool wide = lk >= 0 && c.ks3[lk] == ES && (c.ks1[lk] == ES || c.ks1[lk] == 0) && (c.ks2[lk] == ES || c.ks2[lk] == 0) &&
                    (c.ks1[lk] != 0 || c.ks2[lk] != 0) && c.kshape[lk] % VMAX == 0 && aligned16(p1) && aligned16(p2) && aligned16(p3);
        for (int d = 0; d < lk && wide; ++d) wide = mult16(c.ks1[d]) && mult16(c.ks2[d]) && mult16(c.ks3[d]);
        for (int d = 0; d < c.n_red && wide; ++d) wide = mult16(c.rs1[d]) && mult16(c.rs2[d]);
        if (wide) mulsum_columns_kernel<T, NAN_SKIP, VMAX><<<grid_for((slices * (c.outputs / VMAX) + kBlock - 1) / kBlock, 8), kBlock, 0, st>>>(c, p1, p2, p3, slice_len, slices, partial);
        else mulsum_columns_kernel<T, NAN_SKIP, 1><<<grid_for((slices * c.outputs + kBlock - 1) / kBlock, 8), kBlock, 0, st>>>(c, p1, p2, p3, slice_len, slices, partial);
        if (partial) {
            mulsum_slices_fold_kernel<T><<<grid_for((c.outputs + kBlock - 1) / kBlock, 8), kBlock, 0, st>>>(c, partial, slices, p3);
            cumo_cuda_runtime_free(reinterpret_cast<char*>(partial));
            ++launches;
        }
    }
    count_launch(launches);
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200
