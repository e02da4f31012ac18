// Population counts over Cumo::Bit arrays: count_true / count_false.
//
// Replaces ext/cumo/narray/gen/tmpl_bit/bit_count_kernel.cu:4-78, where one thread
// looks at one bit and every set bit costs an atomicAdd on the single output word.
// Here a contiguous run of bits (bit step 1) is read as 16-byte packets of four
// 32-bit words, each masked at the run's two ends and counted with __popc; every
// CTA folds its count in registers/shared memory and adds it to the output with
// ONE atomicAdd (integer addition commutes, so the total is exact in any order;
// no scratch, no second launch).  Strided bit runs take one bit per thread but
// fold the same way.  The output is accumulated into (`+=`), as the reference
// does, because ndloop pre-fills it with 0 and may call once per outer index.
#include "common.cuh"
#include "reduce.cuh"

namespace cb200 {

struct CountR {
    using Acc = unsigned long long;
    __device__ __forceinline__ Acc identity() const { return 0ull; }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return a + b; }
};

// count_false: CTA 0 adds the number of bits looked at and every CTA subtracts its
// own count of set bits (arithmetic modulo 2^64, so the order still does not matter).
__device__ __forceinline__ void add_count(unsigned long long* out, unsigned long long acc, unsigned long long n_bits, int want_false) {
    if (want_false) {
        if (blockIdx.x == 0) atomicAdd(out, n_bits);
        if (acc) atomicAdd(out, 0ull - acc);
    } else if (acc) {
        atomicAdd(out, acc);
    }
}

// bits [first, first+n) of the word array, contiguous.  Words are visited as
// 16-byte packets starting from the 16-byte-aligned address at or below the first word.
__global__ void __launch_bounds__(kBlock)
bitcount_run_kernel(const uint32_t* __restrict__ words16, int64_t w_base, int64_t w_first, int64_t w_last,
                    uint32_t head_mask, uint32_t tail_mask, int64_t n_packets, int64_t per_cta,
                    unsigned long long n_bits, int want_false, unsigned long long* out) {
    __shared__ unsigned long long smem[kWarpsPerBlock];
    CountR r;
    unsigned long long acc = 0;
    const int64_t p_begin = (int64_t)blockIdx.x * per_cta;
    int64_t p_end = p_begin + per_cta; if (p_end > n_packets) p_end = n_packets;
    for (int64_t q0 = p_begin + threadIdx.x; q0 < p_end; q0 += (int64_t)kBlock * kUnroll) {
        Pack<uint32_t> v[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            int64_t q = q0 + (int64_t)j * kBlock;
            if (q < p_end) v[j] = ld_pack<uint32_t>(words16 + q * 4);
        }
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            int64_t q = q0 + (int64_t)j * kBlock;
            if (q >= p_end) continue;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                int64_t w = w_base + q * 4 + k;
                uint32_t x = v[j].v[k];
                if (w < w_first || w > w_last) x = 0;
                if (w == w_first) x &= head_mask;
                if (w == w_last) x &= tail_mask;
                acc += __popc(x);
            }
        }
    }
    acc = group_fold<CountR, kBlock>(r, acc, smem);
    if (threadIdx.x == 0) add_count(out, acc, n_bits, want_false);
}

// bits at first + i*step (or first + idx[i]), one per thread
__global__ void __launch_bounds__(kBlock)
bitcount_strided_kernel(const uint32_t* __restrict__ words, uint64_t first, int64_t step, const size_t* __restrict__ idx,
                        int64_t n, int64_t per_cta, int want_false, unsigned long long* out) {
    __shared__ unsigned long long smem[kWarpsPerBlock];
    CountR r;
    unsigned long long acc = 0;
    const int64_t begin = (int64_t)blockIdx.x * per_cta;
    int64_t end = begin + per_cta; if (end > n) end = n;
    for (int64_t i = begin + threadIdx.x; i < end; i += kBlock) {
        uint64_t b = idx ? first + idx[i] : first + (uint64_t)(i * step);
        acc += (words[b >> 5] >> (b & 31)) & 1u;
    }
    acc = group_fold<CountR, kBlock>(r, acc, smem);
    if (threadIdx.x == 0) add_count(out, acc, (unsigned long long)n, want_false);
}

// out[i] += bit_i (or its complement): the loop dimension is not reduced
__global__ void __launch_bounds__(kBlock)
bitcount_each_kernel(const uint32_t* __restrict__ words, uint64_t first, int64_t step, const size_t* __restrict__ idx,
                     char* out, int64_t out_step, int64_t n, int want_false) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (int64_t)gridDim.x * kBlock) {
        uint64_t b = idx ? first + idx[i] : first + (uint64_t)(i * step);
        unsigned bit = (words[b >> 5] >> (b & 31)) & 1u;
        if (want_false) bit ^= 1u;
        if (bit) *reinterpret_cast<unsigned long long*>(out + i * out_step) += 1ull;
    }
}

// CTAs for `units` units of work at `base` units per CTA, growing the share so that at
// most kMaxCtas CTAs (= atomics on the one output word) are launched
static int64_t share_per_cta(int64_t units, int64_t base) {
    constexpr int64_t kMaxCtas = 8192;
    int64_t per = base;
    if ((units + per - 1) / per > kMaxCtas) per = ((units + kMaxCtas - 1) / kMaxCtas + base - 1) / base * base;
    return per;
}

static void count_total(size_t p1, char* p2, const uint32_t* a1, ssize_t s1, const size_t* idx, uint64_t n, int want_false) {
    if (n == 0) return;
    cudaStream_t st = current_stream();
    unsigned long long* out = reinterpret_cast<unsigned long long*>(p2);
    if (!idx && s1 == 1) {
        const int64_t w_first = (int64_t)(p1 >> 5), w_last = (int64_t)((p1 + n - 1) >> 5);
        const uint32_t head = 0xffffffffu << (p1 & 31);
        const unsigned tb = (unsigned)((p1 + n - 1) & 31);
        const uint32_t tail = tb == 31 ? 0xffffffffu : ((1u << (tb + 1)) - 1u);
        // back up to a 16-byte boundary; the packet holding the last word ends on one too.
        // Bit arrays are allocated in whole 512-byte blocks, so both stay inside the allocation.
        uintptr_t addr = reinterpret_cast<uintptr_t>(a1 + w_first);
        const int back = (int)((addr & 15u) / 4);
        const uint32_t* words16 = a1 + w_first - back;
        const int64_t w_base = w_first - back;
        const int64_t n_packets = (w_last - w_base) / 4 + 1;
        const int64_t per_cta = share_per_cta(n_packets, (int64_t)kBlock * kUnroll);
        const int64_t ctas = (n_packets + per_cta - 1) / per_cta;
        bitcount_run_kernel<<<(unsigned)ctas, kBlock, 0, st>>>(words16, w_base, w_first, w_last, head, tail, n_packets, per_cta,
                                                               (unsigned long long)n, want_false, out);
    } else {
        const int64_t per_cta = share_per_cta((int64_t)n, (int64_t)kBlock * kUnroll);
        const int64_t ctas = ((int64_t)n + per_cta - 1) / per_cta;
        bitcount_strided_kernel<<<(unsigned)ctas, kBlock, 0, st>>>(a1, (uint64_t)p1, (int64_t)s1, idx, (int64_t)n, per_cta, want_false, out);
    }
    count_launch(1);
    cumo_cuda_runtime_check_kernel_launch();
}

static void count_each(size_t p1, char* p2, const uint32_t* a1, ssize_t s1, const size_t* idx, ssize_t s2, uint64_t n, int want_false) {
    if (n == 0) return;
    int64_t blocks = ((int64_t)n + kBlock - 1) / kBlock;
    bitcount_each_kernel<<<grid_for(blocks, 8), kBlock, 0, current_stream()>>>(a1, (uint64_t)p1, (int64_t)s1, idx, p2, (int64_t)s2, (int64_t)n, want_false);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200

#define CB_BITCOUNT(name, want_false)                                                                                       \
    extern "C" void cumo_iter_bit_##name##_index_kernel_launch(size_t p1, char* p2, CUMO_BIT_DIGIT* a1, size_t* idx1, uint64_t n) { \
        cb200::count_total(p1, p2, a1, 0, idx1, n, want_false); }                                                           \
    extern "C" void cumo_iter_bit_##name##_stride_kernel_launch(size_t p1, char* p2, CUMO_BIT_DIGIT* a1, ssize_t s1, uint64_t n) { \
        cb200::count_total(p1, p2, a1, s1, nullptr, n, want_false); }                                                       \
    extern "C" void cumo_iter_bit_##name##_index_stride_kernel_launch(size_t p1, char* p2, CUMO_BIT_DIGIT* a1, size_t* idx1, ssize_t s2, uint64_t n) { \
        cb200::count_each(p1, p2, a1, 0, idx1, s2, n, want_false); }                                                        \
    extern "C" void cumo_iter_bit_##name##_stride_stride_kernel_launch(size_t p1, char* p2, CUMO_BIT_DIGIT* a1, ssize_t s1, ssize_t s2, uint64_t n) { \
        cb200::count_each(p1, p2, a1, s1, nullptr, s2, n, want_false); }

CB_BITCOUNT(count_true, 0)
CB_BITCOUNT(count_false, 1)
