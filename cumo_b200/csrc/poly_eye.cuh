// poly (Horner over any number of coefficient operands) and eye (a value on one diagonal of a matrix, zero elsewhere).
// Entry points are the reference's: cumo_iter_<T>_poly_kernel_launch (narray/gen/tmpl/poly.c:2, poly_kernel.cu:22-44) and
// cumo_iter_<T>_eye_stride_kernel_launch (narray/gen/tmpl/eye.c:2, eye_kernel.cu:12-19).
//
// poly: the descriptors of x, z and the coefficients are canonicalised together on the host (extent-1 dims dropped,
// dims merged where every operand walks them with one stride) and the coefficients' part goes to the device as an array,
// since their number is the caller's.  One element per thread slot, the index split done once and shared by all operands;
// a coefficient that is a single repeated element costs one cached load per element.
#pragma once

#include "common.cuh"

#include <vector>

namespace cb200 {

struct PolyOperand {
    const char* ptr;
    int64_t step[kMaxDim];
};
struct PolyPlan {
    int nd;
    int64_t total;
    int64_t shape[kMaxDim];
    PolyOperand x, z;
};

template <typename T>
__global__ void __launch_bounds__(kBlock)
poly_kernel(const PolyPlan p, const PolyOperand* __restrict__ coef, int ncoef) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < p.total; i += (int64_t)gridDim.x * kBlock) {
        int64_t k[kMaxDim];
        int64_t r = i;
        for (int d = p.nd - 1; d >= 0; --d) {
            const int64_t n = p.shape[d];
            k[d] = d > 0 ? r % n : r;
            r = d > 0 ? r / n : 0;
        }
        auto at = [&](const PolyOperand& o) {
            int64_t off = 0;
            for (int d = 0; d < p.nd; ++d) off += k[d] * o.step[d];
            return o.ptr + off;
        };
        const T xv = *reinterpret_cast<const T*>(at(p.x));
        T y = ncoef > 0 ? *reinterpret_cast<const T*>(at(coef[ncoef - 1])) : xv;       // no coefficient at all answers x itself
        for (int c = ncoef - 2; c >= 0; --c) {
            y = xv * y;
            y = y + *reinterpret_cast<const T*>(at(coef[c]));
        }
        *reinterpret_cast<T*>(const_cast<char*>(at(p.z))) = y;
    }
}

// FLAT: x and z contiguous, every coefficient either contiguous like them or one repeated element, everything 16-byte
// aligned, at most kPolyFlatMax coefficients.  A thread keeps the repeated coefficients in registers and takes two packets
// of x (and of each array coefficient) per round.
constexpr int kPolyFlatMax = 8;
struct PolyFlat {
    int ncoef;
    const char* ptr[kPolyFlatMax];
    bool is_array[kPolyFlatMax];
};

template <typename T, int NC>
__global__ void __launch_bounds__(kBlock)
poly_flat_kernel(const char* __restrict__ x, char* z, int64_t n_packets, const PolyFlat c) {
    constexpr int V = 16 / (int)sizeof(T);
    constexpr int U = 2;                                   // packets per thread, all loads issued before the first use
    T held[NC > 0 ? NC : 1];
#pragma unroll
    for (int k = 0; k < NC; ++k) held[k] = c.is_array[k] ? T(0) : *reinterpret_cast<const T*>(c.ptr[k]);
    for (int64_t tile = blockIdx.x; tile * (kBlock * U) < n_packets; tile += gridDim.x) {
        int64_t q[U];
        Pack<T> xv[U], cv[U][NC > 0 ? NC : 1];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            q[u] = tile * (kBlock * U) + u * kBlock + threadIdx.x;
            if (q[u] >= n_packets) continue;
            xv[u] = ld_pack<T>(x + q[u] * 16);
#pragma unroll
            for (int k = 0; k < NC; ++k)
                if (c.is_array[k]) cv[u][k] = ld_pack<T>(c.ptr[k] + q[u] * 16);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (q[u] >= n_packets) continue;
            Pack<T> y = xv[u];                             // no coefficient at all answers x itself
#pragma unroll
            for (int k = NC - 1; k >= 0; --k) {
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    const T ck = c.is_array[k] ? cv[u][k].v[e] : held[k];
                    if (k == NC - 1) y.v[e] = ck;
                    else { const T t = xv[u].v[e] * y.v[e]; y.v[e] = t + ck; }
                }
            }
            st_pack<T>(z + q[u] * 16, y);
        }
    }
}

template <typename T>
void launch_poly_flat(const char* x, char* z, int64_t n_packets, const PolyFlat& c, cudaStream_t st) {
    const int64_t tiles = (n_packets + kBlock * 2 - 1) / (kBlock * 2);
    const unsigned grid = (unsigned)(tiles > 0x7fffffffLL ? 0x7fffffffLL : tiles);
    switch (c.ncoef) {
    case 0: poly_flat_kernel<T, 0><<<grid, kBlock, 0, st>>>(x, z, n_packets, c); break;
    case 1: poly_flat_kernel<T, 1><<<grid, kBlock, 0, st>>>(x, z, n_packets, c); break;
    case 2: poly_flat_kernel<T, 2><<<grid, kBlock, 0, st>>>(x, z, n_packets, c); break;
    case 3: poly_flat_kernel<T, 3><<<grid, kBlock, 0, st>>>(x, z, n_packets, c); break;
    case 4: poly_flat_kernel<T, 4><<<grid, kBlock, 0, st>>>(x, z, n_packets, c); break;
    case 5: poly_flat_kernel<T, 5><<<grid, kBlock, 0, st>>>(x, z, n_packets, c); break;
    case 6: poly_flat_kernel<T, 6><<<grid, kBlock, 0, st>>>(x, z, n_packets, c); break;
    case 7: poly_flat_kernel<T, 7><<<grid, kBlock, 0, st>>>(x, z, n_packets, c); break;
    default: poly_flat_kernel<T, 8><<<grid, kBlock, 0, st>>>(x, z, n_packets, c); break;
    }
}

template <typename T>
void launch_poly(const cumo_na_iarray_t* x, const cumo_na_iarray_t* coef, int ncoef, const cumo_na_iarray_t* z, const cumo_na_indexer_t* ix) {
    CB200_TRACE_LAUNCH();
    if (ncoef < 0) ncoef = 0;
    const int nops = ncoef + 2;
    std::vector<const cumo_na_iarray_t*> ops(nops);
    ops[0] = x; ops[1] = z;
    for (int c = 0; c < ncoef; ++c) ops[2 + c] = &coef[c];
    std::vector<PolyOperand> plan(nops);
    for (int o = 0; o < nops; ++o) { plan[o].ptr = ops[o]->ptr; for (int d = 0; d < kMaxDim; ++d) plan[o].step[d] = 0; }
    PolyPlan p;
    p.nd = 0;
    p.total = 1;
    for (int d = 0; d < ix->ndim; ++d) {
        const int64_t n = (int64_t)ix->shape[d];
        if (n == 0) return;
        if (n == 1) continue;
        bool merge = p.nd > 0;
        for (int o = 0; o < nops && merge; ++o) merge = plan[o].step[p.nd - 1] == (int64_t)ops[o]->step[d] * n;
        if (merge) {
            p.shape[p.nd - 1] *= n;
            for (int o = 0; o < nops; ++o) plan[o].step[p.nd - 1] = (int64_t)ops[o]->step[d];
        } else {
            p.shape[p.nd] = n;
            for (int o = 0; o < nops; ++o) plan[o].step[p.nd] = (int64_t)ops[o]->step[d];
            ++p.nd;
        }
        p.total *= n;
    }
    p.x = plan[0];
    p.z = plan[1];
    cudaStream_t st = current_stream();
    constexpr int64_t ES = sizeof(T);
    constexpr int V = 16 / (int)sizeof(T);
    bool flat = p.nd <= 1 && ncoef <= kPolyFlatMax && p.total >= V && (p.nd == 0 || (plan[0].step[0] == ES && plan[1].step[0] == ES)) &&
                aligned16(plan[0].ptr) && aligned16(plan[1].ptr);
    PolyFlat fc;
    fc.ncoef = ncoef;
    for (int c = 0; c < kPolyFlatMax; ++c) { fc.ptr[c] = nullptr; fc.is_array[c] = false; }
    for (int c = 0; c < ncoef && flat; ++c) {
        const int64_t stp = p.nd == 0 ? 0 : plan[2 + c].step[0];
        fc.ptr[c] = plan[2 + c].ptr;
        fc.is_array[c] = stp != 0;
        if (stp != 0 && (stp != ES || !aligned16(plan[2 + c].ptr))) flat = false;
    }
    if (flat) {
        const int64_t n_packets = p.total / V;
        launch_poly_flat<T>(plan[0].ptr, const_cast<char*>(plan[1].ptr), n_packets, fc, st);
        count_launch();
        const int64_t done = n_packets * V;
        if (done == p.total) { cumo_cuda_runtime_check_kernel_launch(); return; }
        // the few elements after the last whole packet: the general kernel on the shifted operands
        for (int o = 0; o < nops; ++o) plan[o].ptr += done * plan[o].step[0];
        p.total -= done;
        p.shape[0] = p.total;
        p.x = plan[0];
        p.z = plan[1];
    }
    PolyOperand* d_coef = reinterpret_cast<PolyOperand*>(cumo_cuda_runtime_malloc(sizeof(PolyOperand) * (size_t)(ncoef > 0 ? ncoef : 1)));
    if (!d_coef) return;
    if (ncoef > 0) cudaMemcpyAsync(d_coef, plan.data() + 2, sizeof(PolyOperand) * (size_t)ncoef, cudaMemcpyHostToDevice, st);
    poly_kernel<T><<<grid_for((p.total + kBlock - 1) / kBlock, 16), kBlock, 0, st>>>(p, d_coef, ncoef);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
    cumo_cuda_runtime_free(reinterpret_cast<char*>(d_coef));          // stream-ordered reuse: later kernels queue behind this one
}

template <typename T>
__global__ void __launch_bounds__(kBlock)
eye_kernel(char* ptr, int64_t s0, int64_t s1, int64_t kofs, T data, uint64_t n0, uint64_t n1) {
    const uint64_t n = n0 * n1;
    for (uint64_t i = (uint64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (uint64_t)gridDim.x * kBlock) {
        const uint64_t i0 = i / n1, i1 = i - i0 * n1;
        *reinterpret_cast<T*>(ptr + (int64_t)i0 * s0 + (int64_t)i1 * s1) = ((int64_t)i0 + kofs == (int64_t)i1) ? data : T(0);
    }
}

template <typename T>
void launch_eye(char* ptr, ssize_t s0, ssize_t s1, ssize_t kofs, T data, uint64_t n0, uint64_t n1) {
    CB200_TRACE_LAUNCH();
    if (n0 == 0 || n1 == 0) return;
    eye_kernel<T><<<grid_for((int64_t)((n0 * n1 + kBlock - 1) / kBlock), 16), kBlock, 0, current_stream()>>>(ptr, s0, s1, kofs, data, n0, n1);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200
