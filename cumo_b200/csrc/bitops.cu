// Bit o Bit operations and the all? / any? reductions: what stands between a comparison's Bit result and the count,
// where and mask kernels when masks are combined (`(a > 0) & (b < 1)`).
//
// Entry points are the reference's (narray/gen/tmpl_bit/binary.c:1-2, unary.c:1-2, bit_reduce.c:1-3 declare them;
// binary_kernel.cu, unary_kernel.cu and bit_reduce_kernel.cu define them):
//   cumo_iter_bit_{and,or,xor,eq}_kernel_launch(a1, a2, a3, indexer)         operands addressed per dimension by a bit step
//   cumo_iter_bit_{copy,not}_kernel_launch(a1, a3, indexer)                  or an index array (cumo_na_bit_iarray_stridx_t)
//   ..._contiguous_kernel_launch(words, bit offset, ..., n)                   every operand a run of consecutive bits
//   cumo_iter_bit_{all_p,any_p}_{elementwise,reduce,contiguous_reduce}_kernel_launch
//
// Plan.  Contiguous: a thread produces FOUR consecutive words of the output; an operand whose run starts at another bit
// offset than the output's is realigned with a funnel shift over the five words that cover them; interior groups leave as
// one 16-byte store, the partial words at either end are merged under a mask by the one thread that owns them (the
// reference's rule, types/bit_kernel.h:73-83).  A whole array of 2^28 bits is 32 MiB, so these are launch-bound long before
// they are bandwidth-bound; the point of the packets is only that the kernel is not the slower side of that.
// General views: one bit per thread, the position looked up per dimension, the store an atomic AND / OR on the word
// (the reference's CUMO_STORE_BIT, template_kernel.h:26-35) because neighbouring bits belong to other threads.
// Reductions: the output bit starts at the identity (the host fills it) and can only flip, so stores are idempotent and
// need no order (bit_reduce_kernel.cu:1-3); a CTA ORs its threads' findings and at most one thread touches the bit.
#include "common.cuh"

namespace cb200 {

enum BitOp { kBitAnd, kBitOr, kBitXor, kBitEq, kBitCopy, kBitNot };

template <int OP>
__device__ __forceinline__ uint32_t bit_apply(uint32_t x, uint32_t y) {
    switch (OP) {
    case kBitAnd: return x & y;
    case kBitOr: return x | y;
    case kBitXor: return x ^ y;
    case kBitEq: return ~(x ^ y);
    case kBitCopy: return x;
    default: return ~x;
    }
}

// word w (counted from the output's first word) of an operand whose run starts `o` bits after (o > 0) or before (o < 0)
// the output's within their first words; words outside [0, nw) read as zero (their bits are outside the store mask)
__device__ __forceinline__ uint32_t gather_word(const uint32_t* __restrict__ a, int o, int64_t nw, int64_t w) {
    if (o == 0) return w < nw ? a[w] : 0u;
    if (o > 0) {
        const uint32_t lo = w < nw ? a[w] : 0u, hi = w + 1 < nw ? a[w + 1] : 0u;
        return __funnelshift_r(lo, hi, o);
    }
    const uint32_t lo = w > 0 ? a[w - 1] : 0u, hi = w < nw ? a[w] : 0u;
    return __funnelshift_r(lo, hi, 32 + o);
}

__device__ __forceinline__ uint32_t word_mask(uint32_t p, uint64_t n, int64_t w) {
    const uint64_t lb = w == 0 ? p : 0;
    const uint64_t end = (uint64_t)p + n;
    const uint64_t hb = (uint64_t)(w + 1) * 32 <= end ? 32 : end - (uint64_t)w * 32;
    const uint32_t upto_hb = hb >= 32 ? 0xffffffffu : ((1u << hb) - 1u);
    const uint32_t upto_lb = lb >= 32 ? 0xffffffffu : ((1u << lb) - 1u);
    return upto_hb & ~upto_lb;
}

template <int OP, bool BINARY>
__global__ void __launch_bounds__(kBlock)
bit_contiguous_kernel(const uint32_t* __restrict__ a1, int o1, int64_t w1, const uint32_t* __restrict__ a2, int o2, int64_t w2,
                      uint32_t* a3, uint32_t p3, uint64_t n, int64_t w3) {
    const bool aligned = (reinterpret_cast<uintptr_t>(a3) & 15u) == 0;
    for (int64_t g = ((int64_t)blockIdx.x * kBlock + threadIdx.x) * 4; g < w3; g += (int64_t)gridDim.x * kBlock * 4) {
        uint32_t z[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t w = g + k;
            const uint32_t x = gather_word(a1, o1, w1, w);
            const uint32_t y = BINARY ? gather_word(a2, o2, w2, w) : 0u;
            z[k] = bit_apply<OP>(x, y);
        }
        const bool interior = g > 0 && (uint64_t)(g + 4) * 32 <= (uint64_t)p3 + n;          // four whole words, none of them the first
        if (interior && aligned) {
            *reinterpret_cast<uint4*>(a3 + g) = make_uint4(z[0], z[1], z[2], z[3]);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int64_t w = g + k;
                if (w >= w3) break;
                const uint32_t m = word_mask(p3, n, w);
                a3[w] = m == 0xffffffffu ? z[k] : ((z[k] & m) | (a3[w] & ~m));
            }
        }
    }
}

// ---- general views ------------------------------------------------------------------------------------------------------
struct BitView {
    const uint32_t* ptr;
    uint64_t pos;
    int64_t step[kMaxDim];                // bit steps; unused where idx is set
    const size_t* idx[kMaxDim];           // bit offsets per position, or null
};
struct BitPlan {
    int nd;
    int64_t total;
    int64_t shape[kMaxDim];
};

template <int OP, bool BINARY>
__global__ void __launch_bounds__(kBlock)
bit_general_kernel(const BitPlan p, const BitView v1, const BitView v2, const BitView v3) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < p.total; i += (int64_t)gridDim.x * kBlock) {
        uint64_t q1 = v1.pos, q2 = v2.pos, q3 = v3.pos;
        int64_t r = i;
        for (int d = p.nd - 1; d >= 0; --d) {
            const int64_t n = p.shape[d];
            const int64_t k = d > 0 ? r % n : r;
            r = d > 0 ? r / n : 0;
            q1 += v1.idx[d] ? (uint64_t)v1.idx[d][k] : (uint64_t)(k * v1.step[d]);
            if (BINARY) q2 += v2.idx[d] ? (uint64_t)v2.idx[d][k] : (uint64_t)(k * v2.step[d]);
            q3 += v3.idx[d] ? (uint64_t)v3.idx[d][k] : (uint64_t)(k * v3.step[d]);
        }
        const uint32_t x = (v1.ptr[q1 >> 5] >> (q1 & 31)) & 1u;
        const uint32_t y = BINARY ? (v2.ptr[q2 >> 5] >> (q2 & 31)) & 1u : 0u;
        const uint32_t z = bit_apply<OP>(x, y) & 1u;
        uint32_t* word = const_cast<uint32_t*>(v3.ptr) + (q3 >> 5);
        if (z) atomicOr(word, 1u << (q3 & 31));
        else atomicAnd(word, ~(1u << (q3 & 31)));
    }
}

static bool make_bit_view(BitView* v, const cumo_na_bit_iarray_stridx_t* a, int nd) {
    v->ptr = a->ptr;
    v->pos = a->pos;
    for (int d = 0; d < kMaxDim; ++d) { v->step[d] = 0; v->idx[d] = nullptr; }
    for (int d = 0; d < nd; ++d) {
        const uintptr_t word = (uintptr_t)a->stridx[d].index;
        if (word & 1u) v->step[d] = (int64_t)(a->stridx[d].stride >> 1);      // a step s is stored as (s << 1) | 1
        else v->idx[d] = a->stridx[d].index;
    }
    return true;
}

template <int OP, bool BINARY>
static void launch_bit_general(const cumo_na_bit_iarray_stridx_t* a1, const cumo_na_bit_iarray_stridx_t* a2, const cumo_na_bit_iarray_stridx_t* a3,
                               const cumo_na_indexer_t* ix) {
    CB200_TRACE_LAUNCH();
    if (ix->total_size == 0) return;
    BitPlan p;
    p.nd = ix->ndim;
    p.total = (int64_t)ix->total_size;
    for (int d = 0; d < kMaxDim; ++d) p.shape[d] = d < ix->ndim ? (int64_t)ix->shape[d] : 1;
    BitView v1, v2, v3;
    make_bit_view(&v1, a1, ix->ndim);
    make_bit_view(&v2, BINARY ? a2 : a1, ix->ndim);
    make_bit_view(&v3, a3, ix->ndim);
    bit_general_kernel<OP, BINARY><<<grid_for((p.total + kBlock - 1) / kBlock, 8), kBlock, 0, current_stream()>>>(p, v1, v2, v3);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

template <int OP, bool BINARY>
static void launch_bit_contiguous(uint32_t* a1, size_t p1, uint32_t* a2, size_t p2, uint32_t* a3, size_t p3, uint64_t n) {
    CB200_TRACE_LAUNCH();
    if (n == 0) return;
    const int64_t w1 = (int64_t)((p1 + n + 31) / 32), w2 = (int64_t)((p2 + n + 31) / 32), w3 = (int64_t)((p3 + n + 31) / 32);
    const int o1 = (int)p1 - (int)p3, o2 = (int)p2 - (int)p3;                      // bit offsets are below 32
    const int64_t groups = (w3 + 3) / 4;
    bit_contiguous_kernel<OP, BINARY><<<grid_for((groups + kBlock - 1) / kBlock, 8), kBlock, 0, current_stream()>>>(
        a1, o1, w1, BINARY ? a2 : a1, BINARY ? o2 : o1, BINARY ? w2 : w1, a3, (uint32_t)p3, n, w3);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

// ---- all? / any? ----------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t bit_pos(uint64_t p, int64_t s, const size_t* idx, uint64_t i) {
    return idx ? p + idx[i] : (uint64_t)((int64_t)p + (int64_t)i * s);
}
__device__ __forceinline__ uint32_t load_bit(const uint32_t* a, uint64_t q) { return (a[q >> 5] >> (q & 31)) & 1u; }
__device__ __forceinline__ void store_bit(uint32_t* a, uint64_t q, uint32_t x) {
    if (x) atomicOr(a + (q >> 5), 1u << (q & 31));
    else atomicAnd(a + (q >> 5), ~(1u << (q & 31)));
}

// INIT: the identity the output starts from (1 for all?, 0 for any?)
template <uint32_t INIT>
__global__ void __launch_bounds__(kBlock)
bit_reduce_elementwise_kernel(const uint32_t* __restrict__ a1, uint64_t p1, int64_t s1, const size_t* __restrict__ idx1, uint32_t* a2, uint64_t p2,
                              int64_t s2, const size_t* __restrict__ idx2, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (uint64_t)gridDim.x * kBlock) {
        const uint64_t q2 = bit_pos(p2, s2, idx2, i);
        if (load_bit(a2, q2) == INIT) {
            const uint32_t x = load_bit(a1, bit_pos(p1, s1, idx1, i));
            if (x != INIT) store_bit(a2, q2, x);
        }
    }
}

template <uint32_t INIT>
__device__ __forceinline__ void store_flip(int flip, uint32_t* a2, uint64_t p2) {
    if (__syncthreads_or(flip) && threadIdx.x == 0 && load_bit(a2, p2) == INIT) store_bit(a2, p2, 1u - INIT);
}

template <uint32_t INIT>
__global__ void __launch_bounds__(kBlock)
bit_reduce_strided_kernel(const uint32_t* __restrict__ a1, uint64_t p1, int64_t s1, const size_t* __restrict__ idx1, uint32_t* a2, uint64_t p2, uint64_t n) {
    int flip = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * kBlock + threadIdx.x; i < n && !flip; i += (uint64_t)gridDim.x * kBlock)
        flip = load_bit(a1, bit_pos(p1, s1, idx1, i)) != INIT;
    store_flip<INIT>(flip, a2, p2);
}

// contiguous input: 16-byte packets of words, the partial words at either end under their masks
template <uint32_t INIT>
__global__ void __launch_bounds__(kBlock)
bit_reduce_contiguous_kernel(const uint32_t* __restrict__ a1, uint32_t p1, uint32_t* a2, uint64_t p2, uint64_t n, int64_t w1) {
    const uint32_t init_word = INIT ? 0xffffffffu : 0u;
    const bool aligned = (reinterpret_cast<uintptr_t>(a1) & 15u) == 0;
    int flip = 0;
    for (int64_t g = ((int64_t)blockIdx.x * kBlock + threadIdx.x) * 4; g < w1 && !flip; g += (int64_t)gridDim.x * kBlock * 4) {
        const bool interior = g > 0 && (uint64_t)(g + 4) * 32 <= (uint64_t)p1 + n;
        if (interior && aligned) {
            const uint4 v = *reinterpret_cast<const uint4*>(a1 + g);
            flip = ((v.x ^ init_word) | (v.y ^ init_word) | (v.z ^ init_word) | (v.w ^ init_word)) != 0;
        } else {
            for (int k = 0; k < 4 && g + k < w1; ++k) flip |= ((a1[g + k] ^ init_word) & word_mask(p1, n, g + k)) != 0;
        }
    }
    store_flip<INIT>(flip, a2, p2);
}

template <uint32_t INIT>
static void launch_bit_reduce_elementwise(uint32_t* a1, size_t p1, ssize_t s1, size_t* idx1, uint32_t* a2, size_t p2, ssize_t s2, size_t* idx2, uint64_t n) {
    CB200_TRACE_LAUNCH();
    if (n == 0) return;
    bit_reduce_elementwise_kernel<INIT><<<grid_for((int64_t)((n + kBlock - 1) / kBlock), 8), kBlock, 0, current_stream()>>>(a1, p1, s1, idx1, a2, p2, s2, idx2, n);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}
template <uint32_t INIT>
static void launch_bit_reduce_strided(uint32_t* a1, size_t p1, ssize_t s1, size_t* idx1, uint32_t* a2, size_t p2, uint64_t n) {
    CB200_TRACE_LAUNCH();
    if (n == 0) return;
    bit_reduce_strided_kernel<INIT><<<grid_for((int64_t)((n + kBlock - 1) / kBlock), 8), kBlock, 0, current_stream()>>>(a1, p1, s1, idx1, a2, p2, n);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}
template <uint32_t INIT>
static void launch_bit_reduce_contiguous(uint32_t* a1, size_t p1, uint32_t* a2, size_t p2, uint64_t n) {
    CB200_TRACE_LAUNCH();
    if (n == 0) return;
    const int64_t w1 = (int64_t)((p1 + n + 31) / 32);
    const int64_t groups = (w1 + 3) / 4;
    bit_reduce_contiguous_kernel<INIT><<<grid_for((groups + kBlock - 1) / kBlock, 8), kBlock, 0, current_stream()>>>(a1, (uint32_t)p1, a2, p2, n, w1);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200

using namespace cb200;

#define CB200_DEF_BIT_BINARY(name, OP)                                                                                                   \
    extern "C" void cumo_iter_bit_##name##_kernel_launch(cumo_na_bit_iarray_stridx_t* a1, cumo_na_bit_iarray_stridx_t* a2,                \
                                                         cumo_na_bit_iarray_stridx_t* a3, cumo_na_indexer_t* indexer) {                   \
        launch_bit_general<OP, true>(a1, a2, a3, indexer); }                                                                              \
    extern "C" void cumo_iter_bit_##name##_contiguous_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, CUMO_BIT_DIGIT* a2, size_t p2,         \
                                                                    CUMO_BIT_DIGIT* a3, size_t p3, uint64_t n) {                          \
        launch_bit_contiguous<OP, true>(a1, p1, a2, p2, a3, p3, n); }
#define CB200_DEF_BIT_UNARY(name, OP)                                                                                                    \
    extern "C" void cumo_iter_bit_##name##_kernel_launch(cumo_na_bit_iarray_stridx_t* a1, cumo_na_bit_iarray_stridx_t* a3,                \
                                                         cumo_na_indexer_t* indexer) {                                                    \
        launch_bit_general<OP, false>(a1, nullptr, a3, indexer); }                                                                        \
    extern "C" void cumo_iter_bit_##name##_contiguous_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, CUMO_BIT_DIGIT* a3, size_t p3,         \
                                                                    uint64_t n) {                                                         \
        launch_bit_contiguous<OP, false>(a1, p1, nullptr, 0, a3, p3, n); }
#define CB200_DEF_BIT_REDUCE(name, INIT)                                                                                                 \
    extern "C" void cumo_iter_bit_##name##_elementwise_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, ssize_t s1, size_t* idx1,             \
                                                                     CUMO_BIT_DIGIT* a2, size_t p2, ssize_t s2, size_t* idx2, uint64_t n) { \
        launch_bit_reduce_elementwise<INIT>(a1, p1, s1, idx1, a2, p2, s2, idx2, n); }                                                     \
    extern "C" void cumo_iter_bit_##name##_reduce_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, ssize_t s1, size_t* idx1,                  \
                                                                CUMO_BIT_DIGIT* a2, size_t p2, uint64_t n) {                              \
        launch_bit_reduce_strided<INIT>(a1, p1, s1, idx1, a2, p2, n); }                                                                   \
    extern "C" void cumo_iter_bit_##name##_contiguous_reduce_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, CUMO_BIT_DIGIT* a2, size_t p2,  \
                                                                           uint64_t n) {                                                  \
        launch_bit_reduce_contiguous<INIT>(a1, p1, a2, p2, n); }

CB200_DEF_BIT_BINARY(and, kBitAnd)
CB200_DEF_BIT_BINARY(or, kBitOr)
CB200_DEF_BIT_BINARY(xor, kBitXor)
CB200_DEF_BIT_BINARY(eq, kBitEq)
CB200_DEF_BIT_UNARY(copy, kBitCopy)
CB200_DEF_BIT_UNARY(store_bit, kBitCopy)      // Bit#store(Bit): tmpl_bit/store_bit.c, store_bit_kernel.cu:22-46 -- the same walk as copy
CB200_DEF_BIT_UNARY(not, kBitNot)
CB200_DEF_BIT_REDUCE(all_p, 1u)
CB200_DEF_BIT_REDUCE(any_p, 0u)
