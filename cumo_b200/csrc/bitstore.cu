// Conversions between Bit arrays and value arrays, and Bit#fill: how a comparison's result re-enters arithmetic
// (`SFloat.cast(a > 0) * a`) and how a value array becomes a mask (`Bit.cast(labels)`).
//
// Entry points are the reference's:
//   cumo_iter_<T>_store_bit_kernel_launch(dst values, src bits, indexer)   narray/gen/tmpl/store_bit.c, store_bit_kernel.cu:14-30
//   cumo_iter_bit_store_<S>_kernel_launch(dst bits, src values, indexer)   narray/gen/tmpl_bit/store_from.c, store_from_kernel.cu:14-29
//       S = dfloat sfloat int64 int32 int16 int8 uint64 uint32 uint16 uint8; a bit is set where the value is not zero
//       (types/bit_kernel.h:13-19), so a NaN sets it
//   cumo_iter_bit_fill_kernel_launch(dst bits, y, indexer), ..._contiguous_kernel_launch(words, bit offset, n, y)
//                                                                          narray/gen/tmpl_bit/fill.c, fill_kernel.cu:21-41
// Every operand is addressed per dimension by a step (bytes for values, bits for Bit) or through an index array
// (cumo_stridx_t: the low bit of the word says which, narray_kernel.h:168-176).
//
// Plan.  When both sides collapse to one run laid end to end:
//   * Bit -> values: a warp takes 32 words of the mask (1024 elements); lane l loads word l, then in 32/V steps every lane
//     fetches the word holding its V consecutive elements by shuffle and stores them as one 16-byte packet: the stores of
//     a step are 512 consecutive bytes.  Traffic is the output, n*s bytes (+n/8 read).
//   * values -> Bit: as in the comparison kernels, each lane loads ONE element per step, so the warp's ballot is the output
//     word; several steps' loads are in flight per thread.  An output run that starts inside a word is walked by output
//     word, the lanes outside the run sit out and the two partial words are merged under their masks.
//   * fill: whole words, the partial ones merged.
// Anything else: one element per thread, positions from the steps / index arrays, the bit set with an atomic OR / AND on
// its word (the reference's CUMO_STORE_BIT, template_kernel.h:26-35) because neighbouring bits belong to other threads.
#include "common.cuh"

namespace cb200 {

namespace {

struct MixPlan {
    int nd;
    int64_t total;
    int64_t shape[kMaxDim];
    int64_t vstep[kMaxDim];              // value operand: byte steps, unused where vidx is set
    const size_t* vidx[kMaxDim];
    int64_t bstep[kMaxDim];              // Bit operand: bit steps, unused where bidx is set
    const size_t* bidx[kMaxDim];
};

// fills the plan; *flat says whether both operands are single runs laid end to end (element size `es`)
void make_mix_plan(MixPlan* p, const cumo_na_iarray_stridx_t* v, const cumo_na_bit_iarray_stridx_t* b, const cumo_na_indexer_t* ix,
                   int64_t es, bool* flat) {
    p->nd = ix->ndim;
    p->total = 1;
    *flat = true;
    for (int d = 0; d < kMaxDim; ++d) { p->shape[d] = 1; p->vstep[d] = p->bstep[d] = 0; p->vidx[d] = p->bidx[d] = nullptr; }
    for (int d = 0; d < ix->ndim; ++d) {
        p->shape[d] = (int64_t)ix->shape[d];
        p->total *= p->shape[d];
        if (v->stridx[d].stride & 1) p->vstep[d] = (int64_t)(v->stridx[d].stride >> 1); else { p->vidx[d] = v->stridx[d].index; *flat = false; }
        if (b->stridx[d].stride & 1) p->bstep[d] = (int64_t)(b->stridx[d].stride >> 1); else { p->bidx[d] = b->stridx[d].index; *flat = false; }
    }
    int64_t ve = es, be = 1;
    for (int d = ix->ndim - 1; d >= 0 && *flat; --d) {
        if (p->shape[d] == 1) continue;
        if (p->vstep[d] != ve || p->bstep[d] != be) *flat = false;
        ve *= p->shape[d];
        be *= p->shape[d];
    }
}

__device__ __forceinline__ void mix_offsets(const MixPlan& p, int64_t i, int64_t* vo, uint64_t* bo) {
    int64_t r = i, v = 0;
    uint64_t b = 0;
    for (int d = p.nd - 1; d >= 0; --d) {
        const int64_t n = p.shape[d];
        const int64_t k = d > 0 ? r % n : r;
        r = d > 0 ? r / n : 0;
        v += p.vidx[d] ? (int64_t)p.vidx[d][k] : k * p.vstep[d];
        b += p.bidx[d] ? (uint64_t)p.bidx[d][k] : (uint64_t)(k * p.bstep[d]);
    }
    *vo = v;
    *bo = b;
}

__device__ __forceinline__ void put_bit(uint32_t* a, uint64_t q, uint32_t x) {
    if (x) atomicOr(a + (q >> 5), 1u << (q & 31));
    else atomicAnd(a + (q >> 5), ~(1u << (q & 31)));
}

// bits [p, p+n) of a run whose first word is word 0: the bits of word w that belong to it
__device__ __forceinline__ uint32_t run_mask(uint32_t p, uint64_t n, int64_t w) {
    const uint64_t lb = w == 0 ? p : 0;
    const uint64_t end = (uint64_t)p + n;
    const uint64_t hb = (uint64_t)(w + 1) * 32 <= end ? 32 : end - (uint64_t)w * 32;
    const uint32_t upto_hb = hb >= 32 ? 0xffffffffu : ((1u << hb) - 1u);
    const uint32_t upto_lb = lb >= 32 ? 0xffffffffu : ((1u << lb) - 1u);
    return upto_hb & ~upto_lb;
}

// ---- Bit -> values ----------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBlock)
bits_to_values_flat_kernel(T* __restrict__ dst, const uint32_t* __restrict__ words, uint32_t p, uint64_t n, int64_t nw) {
    constexpr int V = 16 / (int)sizeof(T);
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * kBlock + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * kBlock) >> 5;
    const int64_t chunks = (int64_t)((n + 1023) / 1024);
    for (int64_t c = warp; c < chunks; c += n_warps) {
        // word `lane` of the chunk, realigned so that its bit 0 is element c*1024 + lane*32
        const int64_t w = c * 32 + lane;
        uint32_t mine = 0;
        if (w < nw) {
            mine = words[w];
            if (p) mine = __funnelshift_r(mine, w + 1 < nw ? words[w + 1] : 0u, p);
        }
#pragma unroll
        for (int s = 0; s < 32 / V; ++s) {
            const uint32_t wv = __shfl_sync(0xffffffffu, mine, s * V + ((lane * V) >> 5));
            const uint32_t bits = wv >> ((lane * V) & 31);
            const uint64_t e = (uint64_t)c * 1024 + (uint64_t)s * 32 * V + (uint64_t)lane * V;
            if (e + V <= n) {
                Pack<T> out;
#pragma unroll
                for (int k = 0; k < V; ++k) out.v[k] = (T)((bits >> k) & 1u);
                st_pack<T>(dst + e, out);
            } else {
                for (int k = 0; k < V && e + k < n; ++k) dst[e + k] = (T)((bits >> k) & 1u);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kBlock)
bits_to_values_gen_kernel(const MixPlan p, char* dst, const uint32_t* __restrict__ words, uint64_t pos) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < p.total; i += (int64_t)gridDim.x * kBlock) {
        int64_t vo;
        uint64_t bo;
        mix_offsets(p, i, &vo, &bo);
        const uint64_t q = pos + bo;
        *reinterpret_cast<T*>(dst + vo) = (T)((words[q >> 5] >> (q & 31)) & 1u);
    }
}

template <typename T>
void launch_bits_to_values(const cumo_na_iarray_stridx_t* a1, const cumo_na_bit_iarray_stridx_t* a2, const cumo_na_indexer_t* ix) {
    CB200_TRACE_LAUNCH();
    MixPlan p;
    bool flat;
    make_mix_plan(&p, a1, a2, ix, (int64_t)sizeof(T), &flat);
    if (p.total <= 0) return;
    cudaStream_t st = current_stream();
    if (flat && aligned16(a1->ptr)) {
        const uint32_t* words = a2->ptr + (a2->pos >> 5);
        const uint32_t off = (uint32_t)(a2->pos & 31);
        const int64_t nw = (int64_t)((off + (uint64_t)p.total + 31) / 32);
        const int64_t chunks = (p.total + 1023) / 1024;
        bits_to_values_flat_kernel<T><<<grid_for((chunks + kBlock / 32 - 1) / (kBlock / 32), 16), kBlock, 0, st>>>(
            reinterpret_cast<T*>(a1->ptr), words, off, (uint64_t)p.total, nw);
    } else {
        bits_to_values_gen_kernel<T><<<grid_for((p.total + kBlock - 1) / kBlock, 16), kBlock, 0, st>>>(p, a1->ptr, a2->ptr, (uint64_t)a2->pos);
    }
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

// ---- values -> Bit ----------------------------------------------------------------------------------------------------
template <typename S> constexpr int v2b_steps() { return sizeof(S) >= 8 ? 8 : 16; }      // loads in flight per thread

template <typename S>
__global__ void __launch_bounds__(kBlock)
values_to_bits_flat_kernel(uint32_t* words, uint32_t p, uint64_t n, int64_t nw, const S* __restrict__ src) {
    constexpr int U = v2b_steps<S>();
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * kBlock + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * kBlock) >> 5;
    for (int64_t w0 = warp * U; w0 < nw; w0 += n_warps * U) {
        S x[U];
        bool ok[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int64_t i = (w0 + j) * 32 + lane - (int64_t)p;            // my element of output word w0 + j
            ok[j] = i >= 0 && (uint64_t)i < n;
            x[j] = ok[j] ? src[i] : S();
        }
        // lane j keeps the word of step j, so that the first U lanes store the warp's U words as one access
        uint32_t my_z = 0, my_m = 0;
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const uint32_t z = __ballot_sync(0xffffffffu, ok[j] && x[j] != S());
            const uint32_t m = __ballot_sync(0xffffffffu, ok[j]);
            if (lane == j) { my_z = z; my_m = m; }
        }
        if (lane < U && my_m) words[w0 + lane] = my_m == 0xffffffffu ? my_z : ((my_z & my_m) | (words[w0 + lane] & ~my_m));
    }
}

// The interior of a run whose output starts on a word boundary: a warp per group of U whole words, no bounds to test,
// one pass (a grid of as many CTAs as there are groups streams faster than a persistent loop here).
template <typename S>
__global__ void __launch_bounds__(kBlock)
values_to_bits_full_kernel(uint32_t* words, const S* __restrict__ src, int64_t groups) {
    constexpr int U = v2b_steps<S>();
    const int lane = threadIdx.x & 31;
    const int64_t g = (int64_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5);
    if (g >= groups) return;
    const S* q = src + g * (32 * U) + lane;
    S x[U];
#pragma unroll
    for (int j = 0; j < U; ++j) x[j] = ld_one<S>(q + j * 32);
    uint32_t mine = 0;
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const uint32_t z = __ballot_sync(0xffffffffu, x[j] != S());
        if (lane == j) mine = z;
    }
    if (lane < U) words[g * U + lane] = mine;
}

template <typename S>
__global__ void __launch_bounds__(kBlock)
values_to_bits_gen_kernel(const MixPlan p, uint32_t* words, uint64_t pos, const char* __restrict__ src) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < p.total; i += (int64_t)gridDim.x * kBlock) {
        int64_t vo;
        uint64_t bo;
        mix_offsets(p, i, &vo, &bo);
        put_bit(words, pos + bo, *reinterpret_cast<const S*>(src + vo) != S() ? 1u : 0u);
    }
}

template <typename S>
void launch_values_to_bits(const cumo_na_bit_iarray_stridx_t* a1, const cumo_na_iarray_stridx_t* a2, const cumo_na_indexer_t* ix) {
    CB200_TRACE_LAUNCH();
    MixPlan p;
    bool flat;
    make_mix_plan(&p, a2, a1, ix, (int64_t)sizeof(S), &flat);
    if (p.total <= 0) return;
    cudaStream_t st = current_stream();
    if (flat) {
        uint32_t* words = a1->ptr + (a1->pos >> 5);
        const uint32_t off = (uint32_t)(a1->pos & 31);
        const int64_t nw = (int64_t)((off + (uint64_t)p.total + 31) / 32);
        constexpr int U = v2b_steps<S>();
        const S* src = reinterpret_cast<const S*>(a2->ptr);
        uint64_t n = (uint64_t)p.total;
        int64_t nwords = nw;
        const int64_t groups = off == 0 ? (int64_t)(n / 32) / U : 0;
        int launches = 0;
        if (groups > 0 && groups <= 0x7fffffffLL * (kBlock / 32)) {
            values_to_bits_full_kernel<S><<<(unsigned)((groups + kBlock / 32 - 1) / (kBlock / 32)), kBlock, 0, st>>>(words, src, groups);
            ++launches;
            words += groups * U;
            src += groups * U * 32;
            n -= (uint64_t)groups * U * 32;
            nwords -= groups * U;
        }
        if (n > 0) {
            const int64_t per_cta = (int64_t)(kBlock / 32) * U;
            values_to_bits_flat_kernel<S><<<grid_for((nwords + per_cta - 1) / per_cta, 16), kBlock, 0, st>>>(words, off, n, nwords, src);
            ++launches;
        }
        count_launch(launches);
        cumo_cuda_runtime_check_kernel_launch();
        return;
    } else {
        values_to_bits_gen_kernel<S><<<grid_for((p.total + kBlock - 1) / kBlock, 16), kBlock, 0, st>>>(p, a1->ptr, (uint64_t)a1->pos, a2->ptr);
    }
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

// ---- fill -------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBlock)
bit_fill_flat_kernel(uint32_t* words, uint32_t p, uint64_t n, int64_t nw, uint32_t value) {
    for (int64_t w = (int64_t)blockIdx.x * kBlock + threadIdx.x; w < nw; w += (int64_t)gridDim.x * kBlock) {
        const uint32_t m = run_mask(p, n, w);
        words[w] = m == 0xffffffffu ? value : ((value & m) | (words[w] & ~m));
    }
}

struct BitOnly {
    int nd;
    int64_t total;
    int64_t shape[kMaxDim];
    int64_t step[kMaxDim];
    const size_t* idx[kMaxDim];
};

__global__ void __launch_bounds__(kBlock)
bit_fill_gen_kernel(const BitOnly p, uint32_t* words, uint64_t pos, uint32_t y) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < p.total; i += (int64_t)gridDim.x * kBlock) {
        int64_t r = i;
        uint64_t q = pos;
        for (int d = p.nd - 1; d >= 0; --d) {
            const int64_t n = p.shape[d];
            const int64_t k = d > 0 ? r % n : r;
            r = d > 0 ? r / n : 0;
            q += p.idx[d] ? (uint64_t)p.idx[d][k] : (uint64_t)(k * p.step[d]);
        }
        put_bit(words, q, y);
    }
}

// `word` is stored as given (the reference's caller passes 0 or ~0, tmpl_bit/fill.c:19-33)
void launch_bit_fill_flat(uint32_t* a3, size_t p3, uint64_t n, uint32_t word) {
    CB200_TRACE_LAUNCH();
    if (n == 0) return;
    uint32_t* words = a3 + (p3 >> 5);
    const uint32_t off = (uint32_t)(p3 & 31);
    const int64_t nw = (int64_t)((off + n + 31) / 32);
    bit_fill_flat_kernel<<<grid_for((nw + kBlock - 1) / kBlock, 8), kBlock, 0, current_stream()>>>(words, off, n, nw, word);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

void launch_bit_fill(const cumo_na_bit_iarray_stridx_t* a3, uint32_t y, const cumo_na_indexer_t* ix) {
    BitOnly p;
    p.nd = ix->ndim;
    p.total = 1;
    bool flat = true;
    for (int d = 0; d < kMaxDim; ++d) { p.shape[d] = 1; p.step[d] = 0; p.idx[d] = nullptr; }
    for (int d = 0; d < ix->ndim; ++d) {
        p.shape[d] = (int64_t)ix->shape[d];
        p.total *= p.shape[d];
        if (a3->stridx[d].stride & 1) p.step[d] = (int64_t)(a3->stridx[d].stride >> 1); else { p.idx[d] = a3->stridx[d].index; flat = false; }
    }
    if (p.total <= 0) return;
    int64_t be = 1;
    for (int d = ix->ndim - 1; d >= 0 && flat; --d) {
        if (p.shape[d] == 1) continue;
        if (p.step[d] != be) flat = false;
        be *= p.shape[d];
    }
    if (flat) { launch_bit_fill_flat(a3->ptr, a3->pos, (uint64_t)p.total, (y & 1u) ? 0xffffffffu : 0u); return; }
    CB200_TRACE_LAUNCH();
    bit_fill_gen_kernel<<<grid_for((p.total + kBlock - 1) / kBlock, 8), kBlock, 0, current_stream()>>>(p, a3->ptr, (uint64_t)a3->pos, y & 1u);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace
}  // namespace cb200

using namespace cb200;

#define CB200_DEF_STORE_BIT(T, C)                                                                                                       \
    extern "C" void cumo_iter_##T##_store_bit_kernel_launch(cumo_na_iarray_stridx_t* a1, cumo_na_bit_iarray_stridx_t* a2,                \
                                                            cumo_na_indexer_t* indexer) { launch_bits_to_values<C>(a1, a2, indexer); }
CB200_DEF_STORE_BIT(sfloat, float)
CB200_DEF_STORE_BIT(dfloat, double)
CB200_DEF_STORE_BIT(int32, int32_t)
CB200_DEF_STORE_BIT(int64, int64_t)

#define CB200_DEF_BIT_STORE(S, C)                                                                                                       \
    extern "C" void cumo_iter_bit_store_##S##_kernel_launch(cumo_na_bit_iarray_stridx_t* a1, cumo_na_iarray_stridx_t* a2,                \
                                                            cumo_na_indexer_t* indexer) { launch_values_to_bits<C>(a1, a2, indexer); }
CB200_DEF_BIT_STORE(dfloat, double)
CB200_DEF_BIT_STORE(sfloat, float)
CB200_DEF_BIT_STORE(int64, int64_t)
CB200_DEF_BIT_STORE(int32, int32_t)
CB200_DEF_BIT_STORE(int16, int16_t)
CB200_DEF_BIT_STORE(int8, int8_t)
CB200_DEF_BIT_STORE(uint64, uint64_t)
CB200_DEF_BIT_STORE(uint32, uint32_t)
CB200_DEF_BIT_STORE(uint16, uint16_t)
CB200_DEF_BIT_STORE(uint8, uint8_t)

extern "C" void cumo_iter_bit_fill_kernel_launch(cumo_na_bit_iarray_stridx_t* a3, CUMO_BIT_DIGIT y, cumo_na_indexer_t* indexer) {
    launch_bit_fill(a3, y, indexer);
}
extern "C" void cumo_iter_bit_fill_contiguous_kernel_launch(CUMO_BIT_DIGIT* a3, size_t p3, uint64_t n, CUMO_BIT_DIGIT y) {
    launch_bit_fill_flat(a3, p3, n, y);
}
