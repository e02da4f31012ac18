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
