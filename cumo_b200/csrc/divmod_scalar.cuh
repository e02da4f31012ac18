// Integer `a / s` and `a % s` with a host scalar on the right (binary_kernel.cu:83-99 with scalar_is_left == 0).
//
// The general kernels divide with the hardware's sequence for a divisor they know nothing about (some twenty
// instructions per 32-bit element, far more per 64-bit one): measured, `a % 7` over 2^26 Int32 ran at 0.52 of nominal
// HBM bandwidth, bound by instruction issue.  The divisor of this form is one number for the whole launch, so the host
// turns it into a multiplier and two shifts (Granlund & Montgomery, "Division by invariant integers using
// multiplication", 1994, figure 4.1: for 1 <= d < 2^N, L = ceil(log2 d), m' = floor(2^N (2^L - d) / d) + 1,
// q = (t + ((n - t) >> min(L, 1))) >> max(L - 1, 0) with t = the high word of m' * n) and the kernel works on
// magnitudes: a multiply-high, a subtract, an add, two shifts, then the signs of C's truncating division.
// Flat contiguous 16-byte-aligned arrays only (what `a % 7` is); everything else takes the general path.
#pragma once

#include <type_traits>

#include "elementwise.cuh"

namespace cb200 {

template <typename U> struct InvariantDivisor {
    U d;            // |divisor|
    U m;            // m'
    int sh1, sh2;
    int negative;   // the divisor's sign
};

template <typename U>
inline InvariantDivisor<U> make_invariant_divisor(U d, bool negative) {
    constexpr int N = 8 * sizeof(U);
    InvariantDivisor<U> r;
    r.d = d;
    int L = 0;
    while (L < N && ((U)1 << L) < d) ++L;                 // ceil(log2 d); d <= 2^(N-1) here (a magnitude of a signed value)
    const unsigned __int128 two_n = (unsigned __int128)1 << N;
    r.m = (U)((two_n * (((unsigned __int128)1 << L) - d)) / d + 1);
    r.sh1 = L < 1 ? L : 1;
    r.sh2 = L > 1 ? L - 1 : 0;
    r.negative = negative ? 1 : 0;
    return r;
}

__device__ __forceinline__ uint32_t mul_high(uint32_t a, uint32_t b) { return __umulhi(a, b); }
__device__ __forceinline__ uint64_t mul_high(uint64_t a, uint64_t b) { return __umul64hi(a, b); }

template <typename T, bool MOD>
__device__ __forceinline__ T divmod_invariant(T x, const InvariantDivisor<typename std::make_unsigned<T>::type>& k) {
    using U = typename std::make_unsigned<T>::type;
    const bool xneg = x < 0;
    const U n = xneg ? (U)0 - (U)x : (U)x;
    const U t = mul_high(k.m, n);
    const U q = (t + ((n - t) >> k.sh1)) >> k.sh2;
    if (MOD) {
        const U r = n - q * k.d;
        return (T)(xneg ? (U)0 - r : r);                        // the remainder takes the dividend's sign
    }
    return (T)((xneg != (k.negative != 0)) ? (U)0 - q : q);      // the quotient truncates toward zero
}

template <typename T, bool MOD>
__global__ void __launch_bounds__(kBlock)
int_divmod_scalar_kernel(const char* __restrict__ in, char* out, int64_t n_packets,
                         const InvariantDivisor<typename std::make_unsigned<T>::type> k) {
    constexpr int V = 16 / sizeof(T);
    constexpr int U = 4;                                   // packets in flight per thread
    const int64_t base = (int64_t)blockIdx.x * (kBlock * U) + threadIdx.x;
    Pack<T> x[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int64_t i = base + (int64_t)j * kBlock;
        if (i < n_packets) x[j] = ld_pack<T>(in + i * 16);
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int64_t i = base + (int64_t)j * kBlock;
        if (i >= n_packets) continue;
        Pack<T> z;
#pragma unroll
        for (int e = 0; e < V; ++e) z.v[e] = divmod_invariant<T, MOD>(x[j].v[e], k);
        st_pack<T>(out + i * 16, z);
    }
}

template <typename T, bool MOD>
__global__ void int_divmod_scalar_tail_kernel(const T* __restrict__ in, T* out, int n,
                                              const InvariantDivisor<typename std::make_unsigned<T>::type> k) {
    const int i = threadIdx.x;
    if (i < n) out[i] = divmod_invariant<T, MOD>(in[i], k);
}

// True when it launched; false sends the call down the general path (zero and -1 divisors, whose flag and overflow
// rules live there; views; unaligned arrays).
template <typename T, bool MOD>
bool launch_int_divmod_by_scalar(const cumo_na_iarray_t* a1, T sv, cumo_na_iarray_t* a3, const cumo_na_indexer_t* ix) {
    using U = typename std::make_unsigned<T>::type;
    constexpr int64_t ES = sizeof(T);
    constexpr int V = 16 / sizeof(T);
    if (sv == 0 || sv == (T)-1) return false;
    EwPlan p;
    if (!make_plan(&p, ix, a1->step, nullptr, a3->step)) return true;          // nothing to do
    if (p.nd != 1 || p.step[0][0] != ES || p.step[2][0] != ES) return false;
    if (!aligned16(a1->ptr) || !aligned16(a3->ptr) || p.total < 4 * V) return false;
    const U mag = sv < 0 ? (U)0 - (U)sv : (U)sv;
    const InvariantDivisor<U> k = make_invariant_divisor<U>(mag, sv < 0);
    cudaStream_t st = current_stream();
    const int64_t n_packets = p.total / V;
    const int64_t per_cta = (int64_t)kBlock * 4;
    const int64_t ctas = (n_packets + per_cta - 1) / per_cta;
    if (ctas > 0x7fffffffLL) return false;
    int_divmod_scalar_kernel<T, MOD><<<(unsigned)ctas, kBlock, 0, st>>>(a1->ptr, a3->ptr, n_packets, k);
    int launches = 1;
    const int tail = (int)(p.total - n_packets * V);
    if (tail > 0) {
        int_divmod_scalar_tail_kernel<T, MOD><<<1, 32, 0, st>>>(reinterpret_cast<const T*>(a1->ptr) + n_packets * V,
                                                                reinterpret_cast<T*>(a3->ptr) + n_packets * V, tail, k);
        ++launches;
    }
    count_launch(launches);
    cumo_cuda_runtime_check_kernel_launch();
    return true;
}

}  // namespace cb200
