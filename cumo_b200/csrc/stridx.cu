// Same-type store between operands that may be addressed through index arrays.
//
// Entry points: cumo_iter_<T>_store_<T>_stridx_kernel_launch, declared by the reference in
// narray/gen/tmpl/store_from.c:5 and defined in store_from_kernel.cu:21-36.  The reference reaches them
// from store_array's own loop, and they are how a view made by `x[index_array, true]` or by Bit#mask is
// materialised: per dimension an operand either steps by a byte stride or looks its byte offset up in a
// device array of size_t (cumo_stridx_t: the low bit of the word says which, narray_kernel.h:168-176).
// A same-type store moves elements unchanged, so there is one kernel per element width (4 or 8 bytes),
// shared by sfloat/int32 and by dfloat/int64.
//
// Plan: one element per thread slot, consecutive threads on consecutive logical elements, the flat index
// split over the extents in 32-bit arithmetic where it fits; an index lookup is one extra 8-byte load per
// indexed dimension.  Gathers are bound by the randomness of the offsets, not by this arithmetic.
#include "common.cuh"

namespace cb200 {

struct StridxPlan {
    int nd;
    int64_t total;
    int64_t shape[kMaxDim];
    int64_t step[2][kMaxDim];            // byte steps ([0] destination, [1] source); unused where idx is set
    const size_t* idx[2][kMaxDim];       // byte offsets per position, or null
};

template <typename W>
__global__ void __launch_bounds__(kBlock)
stridx_copy_kernel(const StridxPlan p, char* dst, const char* __restrict__ src) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < p.total; i += (int64_t)gridDim.x * kBlock) {
        int64_t od = 0, os = 0;
        auto add = [&](int d, int64_t k) {
            od += p.idx[0][d] ? (int64_t)p.idx[0][d][k] : k * p.step[0][d];
            os += p.idx[1][d] ? (int64_t)p.idx[1][d][k] : k * p.step[1][d];
        };
        if (i < 0x7fffffffLL) {
            uint32_t r = (uint32_t)i;
            for (int d = p.nd - 1; d > 0; --d) {
                const uint32_t n = extent32(p.shape[d]);
                const uint32_t q = r / n;
                add(d, (int64_t)(r - q * n));
                r = q;
            }
            if (p.nd > 0) add(0, (int64_t)r);
        } else {
            int64_t r = i;
            for (int d = p.nd - 1; d > 0; --d) {
                const int64_t n = p.shape[d];
                const int64_t q = r / n;
                add(d, r - q * n);
                r = q;
            }
            if (p.nd > 0) add(0, r);
        }
        *reinterpret_cast<W*>(dst + od) = *reinterpret_cast<const W*>(src + os);
    }
}

template <typename W>
static void launch_stridx_store(const cumo_na_iarray_stridx_t* a1, const cumo_na_iarray_stridx_t* a2, const cumo_na_indexer_t* ix) {
    CB200_TRACE_LAUNCH();
    StridxPlan p;
    p.nd = ix->ndim;
    p.total = 1;
    for (int d = 0; d < ix->ndim; ++d) {
        p.shape[d] = (int64_t)ix->shape[d];
        p.total *= p.shape[d];
        const cumo_stridx_t* both[2] = {&a1->stridx[d], &a2->stridx[d]};
        for (int a = 0; a < 2; ++a) {
            if (both[a]->stride & 1) { p.step[a][d] = (int64_t)(both[a]->stride >> 1); p.idx[a][d] = nullptr; }
            else { p.step[a][d] = 0; p.idx[a][d] = both[a]->index; }
        }
    }
    if (p.total <= 0) return;
    const int64_t blocks = (p.total + kBlock - 1) / kBlock;
    stridx_copy_kernel<W><<<grid_for(blocks, 16), kBlock, 0, current_stream()>>>(p, a1->ptr, a2->ptr);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200

#define CB200_DEF_STRIDX(T, W)                                                                                         \
    extern "C" void cumo_iter_##T##_store_##T##_stridx_kernel_launch(cumo_na_iarray_stridx_t* a1, cumo_na_iarray_stridx_t* a2, \
                                                                     cumo_na_indexer_t* indexer) {                     \
        cb200::launch_stridx_store<W>(a1, a2, indexer);                                                                \
    }
CB200_DEF_STRIDX(sfloat, uint32_t)
CB200_DEF_STRIDX(int32, uint32_t)
CB200_DEF_STRIDX(dfloat, uint64_t)
CB200_DEF_STRIDX(int64, uint64_t)
