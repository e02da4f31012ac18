// k-means assignment step, fused: nearest centroid of every point without ever
// writing the (N, K) distance matrix.
//
// The reference has no such kernel; its k-means benchmark builds the step from
// array operations (bench/kmeans_bench.rb:108-126: d = x.dot(c^T) * -2 + |c|^2, then
// min_index(axis: 1)), which materialises N*K floats and reads them back twice.
// Here a CTA owns 128 points, keeps the whole centroid table in shared memory and
// computes, per point, dist[k] = |c_k|^2 - 2 <x, c_k> in 8x8 register tiles (the
// |x|^2 term is constant per point and cannot change the argmin, as the reference
// notes), folding the running (smallest distance, lowest index) as it goes.  The
// label, optionally the winning distance, and a per-cluster population count leave
// the kernel: 4*D bytes read and 4 bytes written per point.
//
// This is the fp32 CUDA-core form: the contraction is done with FMAs in float, in
// increasing order of the feature index.
#include "common.cuh"

#include <cstdio>

namespace cb200 {

constexpr int kKmPoints = 128;       // points per CTA tile
constexpr int kKmCentTile = 128;     // centroids per register-tile sweep
constexpr int kKmPad = 4;            // floats of row padding in shared memory (keeps 16-byte alignment)

// smem: cs[k_pad][d + pad] | xs[128][d + pad] | cnorm[k_pad] | hist[k_pad]
__global__ void __launch_bounds__(256)
kmeans_assign_kernel(const float* __restrict__ x, int64_t n, int d, const float* __restrict__ c, int k, int k_pad,
                     int32_t* __restrict__ labels, float* __restrict__ min_dist, unsigned long long* __restrict__ counts,
                     int64_t n_tiles) {
    extern __shared__ __align__(16) float smem[];
    const int ld = d + kKmPad;
    float* cs = smem;
    float* xs = cs + (size_t)k_pad * ld;
    float* cnorm = xs + (size_t)kKmPoints * ld;
    unsigned* hist = reinterpret_cast<unsigned*>(cnorm + k_pad);
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;      // 16 x 16 threads: tx over centroids, ty over points
    const int d4 = d >> 2;

    // centroid table and its squared norms, once per CTA
    for (int i = tid; i < k_pad * d4; i += 256) {
        const int kk = i / d4, q = i - kk * d4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kk < k) v = *reinterpret_cast<const float4*>(c + (size_t)kk * d + q * 4);
        *reinterpret_cast<float4*>(cs + (size_t)kk * ld + q * 4) = v;
    }
    for (int i = tid; i < k_pad; i += 256) hist[i] = 0;
    __syncthreads();
    for (int kk = tid; kk < k_pad; kk += 256) {
        float s = 0.f;
        for (int q = 0; q < d; ++q) { const float v = cs[(size_t)kk * ld + q]; s = fmaf(v, v, s); }
        cnorm[kk] = kk < k ? s : INFINITY;       // padding centroids can never win
    }
    __syncthreads();

    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t p0 = tile * kKmPoints;
        // the tile of points is one contiguous run of 128*d floats
        for (int i = tid; i < kKmPoints * d4; i += 256) {
            const int pp = i / d4, q = i - pp * d4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p0 + pp < n) v = __ldcs(reinterpret_cast<const float4*>(x + (size_t)(p0 + pp) * d + q * 4));
            *reinterpret_cast<float4*>(xs + (size_t)pp * ld + q * 4) = v;
        }
        __syncthreads();

        float best[8];
        int best_k[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { best[i] = INFINITY; best_k[i] = 0x7fffffff; }

        for (int ct = 0; ct < k_pad; ct += kKmCentTile) {
            float acc[8][8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
            // my points: ty*8 + i;  my centroids: ct + tx + 16*j (ascending in j)
            for (int q = 0; q < d4; ++q) {
                float4 xv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) xv[i] = *reinterpret_cast<const float4*>(xs + (size_t)(ty * 8 + i) * ld + q * 4);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 cv = *reinterpret_cast<const float4*>(cs + (size_t)(ct + tx + 16 * j) * ld + q * 4);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        acc[i][j] = fmaf(xv[i].x, cv.x, acc[i][j]);
                        acc[i][j] = fmaf(xv[i].y, cv.y, acc[i][j]);
                        acc[i][j] = fmaf(xv[i].z, cv.z, acc[i][j]);
                        acc[i][j] = fmaf(xv[i].w, cv.w, acc[i][j]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int kk = ct + tx + 16 * j;
                const float cn = cnorm[kk];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float dist = fmaf(-2.f, acc[i][j], cn);
                    if (dist < best[i]) { best[i] = dist; best_k[i] = kk; }    // strict: the earlier index stays
                }
            }
        }
        // fold across the 16 threads that share my points: smaller distance, then lower index
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int m = 1; m < 16; m <<= 1) {
                const float od = __shfl_xor_sync(0xffffffffu, best[i], m);
                const int ok = __shfl_xor_sync(0xffffffffu, best_k[i], m);
                if (od < best[i] || (od == best[i] && ok < best_k[i])) { best[i] = od; best_k[i] = ok; }
            }
        }
        if (tx == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int64_t p = p0 + ty * 8 + i;
                if (p < n) {
                    labels[p] = best_k[i];
                    if (min_dist) min_dist[p] = best[i];
                    atomicAdd(&hist[best_k[i]], 1u);
                }
            }
        }
        __syncthreads();            // xs is reused by the next tile
    }
    if (counts) {
        __syncthreads();
        for (int kk = tid; kk < k; kk += 256)
            if (hist[kk]) atomicAdd(counts + kk, (unsigned long long)hist[kk]);
    }
}

}  // namespace cb200

extern "C" int cb200_kmeans_assign_sfloat(const float* x, int64_t n, int d, const float* c, int k, int32_t* labels,
                                          float* min_dist, unsigned long long* counts, char* errbuf, size_t errlen) {
    using namespace cb200;
    char local[8];
    if (!errbuf || errlen == 0) { errbuf = local; errlen = sizeof local; }
    errbuf[0] = 0;
    if (n <= 0) return 0;
    if (d < 4 || d % 4 != 0 || k < 1) {
        snprintf(errbuf, errlen, "kmeans_assign: D must be a positive multiple of 4 and K >= 1 (D=%d, K=%d)", d, k);
        return 1;
    }
    if (!aligned16(x) || !aligned16(c)) {
        snprintf(errbuf, errlen, "kmeans_assign: x and c must be 16-byte aligned");
        return 1;
    }
    const int k_pad = (k + kKmCentTile - 1) / kKmCentTile * kKmCentTile;
    const size_t smem = ((size_t)k_pad * (d + kKmPad) + (size_t)kKmPoints * (d + kKmPad) + 2 * (size_t)k_pad) * sizeof(float);
    if (smem > 200 * 1024) {
        snprintf(errbuf, errlen, "kmeans_assign: K=%d centroids of D=%d need %zu bytes of shared memory (limit 204800)", k, d, smem);
        return 2;
    }
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kmeans_assign_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) { snprintf(errbuf, errlen, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return 3; }
        attr_set[dev] = true;
    }
    const int64_t n_tiles = (n + kKmPoints - 1) / kKmPoints;
    const int per_sm = smem > 110 * 1024 ? 1 : 2;
    const unsigned grid = grid_for(n_tiles, per_sm);
    kmeans_assign_kernel<<<grid, 256, smem, current_stream()>>>(x, n, d, c, k, k_pad, labels, min_dist, counts, n_tiles);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { snprintf(errbuf, errlen, "kmeans_assign launch: %s", cudaGetErrorString(e)); return 4; }
    return 0;
}
