// Elementwise operations that do not fit the two-inputs-one-output mould of elementwise.cuh: three inputs
// (clip against two arrays of bounds), two outputs (divmod, modf, frexp) or a value that depends on the element's
// position (seq).  They stand where the reference's per-ndim indexer kernels of
// ext/cumo/narray/gen/tmpl/clip_kernel.cu:8-22, binary2_kernel.cu:13-25, unary_ret2_kernel.cu:1-14,
// frexp_kernel.cu:1-13 and seq_kernel.cu:13-35 stand.
//
// An operation F names its element types and how many inputs and outputs it has; every input and the first output
// are of type F::Elem, the second output of type F::O1.  Two kernels:
//   * FLAT: every operand contiguous and 16-byte aligned.  A thread takes kMultiUnroll packets of 16 bytes per
//     operand of type T, all loads issued before the first use;
//   * GEN: any steps (views, repeated operands).  One element per slot, consecutive threads on consecutive
//     logical elements, the row-major index split shared by all operands.
// An element whose operation answers false (integer division by zero, an empty clip range) is left unwritten and
// raises the caller's flag, as in the reference.
#pragma once

#include "common.cuh"
#include "ops.cuh"

namespace cb200 {

constexpr int kMultiOps = 4;                       // operands of the widest operation
constexpr int kMultiUnroll = 2;

struct MultiPlan {
    int nd;
    int64_t total;
    int64_t shape[kMaxDim];
    int64_t step[kMultiOps][kMaxDim];
};

// Canonical plan over `n` operands (drops extent-1 dims, merges dims that every operand walks with one stride).
inline bool make_multi_plan(MultiPlan* p, const cumo_na_indexer_t* ix, const cumo_na_iarray_t* const* a, int n) {
    int nd = 0;
    p->total = 1;
    for (int d = 0; d < ix->ndim; ++d) {
        const int64_t len = (int64_t)ix->shape[d];
        if (len == 0) return false;
        if (len == 1) continue;
        int64_t t[kMultiOps] = {0, 0, 0, 0};
        for (int k = 0; k < n; ++k) t[k] = (int64_t)a[k]->step[d];
        bool merge = nd > 0;
        for (int k = 0; k < n && merge; ++k) merge = p->step[k][nd - 1] == t[k] * len;
        if (merge) {
            p->shape[nd - 1] *= len;
            for (int k = 0; k < kMultiOps; ++k) p->step[k][nd - 1] = t[k];
        } else {
            p->shape[nd] = len;
            for (int k = 0; k < kMultiOps; ++k) p->step[k][nd] = t[k];
            ++nd;
        }
        p->total *= len;
    }
    if (nd == 0) {
        nd = 1;
        p->shape[0] = 1;
        for (int k = 0; k < kMultiOps; ++k) p->step[k][0] = 0;
    }
    p->nd = nd;
    return true;
}

struct MultiPtrs { char* p[kMultiOps]; };

// V elements of type O, stored as one access when they make 8 or 16 bytes
template <typename O, int V>
__device__ __forceinline__ void st_group(char* q, const O* v) {
    if constexpr (sizeof(O) * V == 16) {
        __stcs(reinterpret_cast<int4*>(q), *reinterpret_cast<const int4*>(v));
    } else if constexpr (sizeof(O) * V == 8) {
        __stcs(reinterpret_cast<int2*>(q), *reinterpret_cast<const int2*>(v));
    } else {
#pragma unroll
        for (int e = 0; e < V; ++e) st_one<O>(q + e * sizeof(O), v[e]);
    }
}

template <typename F>
__global__ void __launch_bounds__(kBlock)
multi_flat_kernel(const MultiPtrs ptr, int64_t n_packets, int64_t base, const typename F::Params prm, int* flag) {
    using T = typename F::Elem;
    using O1 = typename F::O1;
    constexpr int V = 16 / (int)sizeof(T);
    constexpr int U = kMultiUnroll;
    constexpr int NIN = F::NIN;
    for (int64_t tile = blockIdx.x; tile * (kBlock * U) < n_packets; tile += gridDim.x) {
        Pack<T> in[U][NIN > 0 ? NIN : 1];
        int64_t k[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            k[j] = tile * (kBlock * U) + j * kBlock + threadIdx.x;
            if (k[j] < n_packets) {
#pragma unroll
                for (int a = 0; a < NIN; ++a) in[j][a] = ld_pack<T>(ptr.p[a] + k[j] * 16);
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (k[j] >= n_packets) continue;
            alignas(16) T o0[V];
            alignas(16) O1 o1[V];
            unsigned keep = 0;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                T x[NIN > 0 ? NIN : 1];
#pragma unroll
                for (int a = 0; a < NIN; ++a) x[a] = in[j][a].v[e];
                o0[e] = T(); o1[e] = O1();
                if (F::apply(x, base + k[j] * V + e, prm, o0[e], o1[e], flag)) keep |= 1u << e;
            }
            char* q0 = ptr.p[NIN] + k[j] * 16;
            char* q1 = F::NOUT == 2 ? ptr.p[NIN + 1] + k[j] * (int64_t)(V * sizeof(O1)) : nullptr;
            if (keep == (1u << V) - 1u) {
                st_group<T, V>(q0, o0);
                if (F::NOUT == 2) st_group<O1, V>(q1, o1);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    if (!(keep & (1u << e))) continue;
                    st_one<T>(q0 + e * sizeof(T), o0[e]);
                    if (F::NOUT == 2) st_one<O1>(q1 + e * sizeof(O1), o1[e]);
                }
            }
        }
    }
}

template <typename F>
__global__ void __launch_bounds__(kBlock)
multi_gen_kernel(const MultiPlan p, const MultiPtrs ptr, int64_t n_tiles, int64_t base, const typename F::Params prm, int* flag) {
    using T = typename F::Elem;
    using O1 = typename F::O1;
    constexpr int U = kMultiUnroll;
    constexpr int NIN = F::NIN;
    constexpr int NOPS = F::NIN + F::NOUT;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        int64_t off[U][NOPS];
        int64_t i[U];
        T x[U][NIN > 0 ? NIN : 1];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            i[j] = tile * (kBlock * U) + j * kBlock + threadIdx.x;
            if (i[j] < p.total) {
                offsets_of<NOPS>(i[j], p.nd, p.shape, p.step, off[j]);
#pragma unroll
                for (int a = 0; a < NIN; ++a) x[j][a] = ld_one<T>(ptr.p[a] + off[j][a]);
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (i[j] >= p.total) continue;
            T o0 = T();
            O1 o1 = O1();
            if (F::apply(x[j], base + i[j], prm, o0, o1, flag)) {
                st_one<T>(ptr.p[NIN] + off[j][NIN], o0);
                if (F::NOUT == 2) st_one<O1>(ptr.p[NIN + 1] + off[j][NIN + 1], o1);
            }
        }
    }
}

// `a` lists the inputs, then the outputs.
template <typename F>
void launch_multi(const cumo_na_iarray_t* const* a, const cumo_na_indexer_t* ix, const typename F::Params& prm, int* flag) {
    CB200_TRACE_LAUNCH();
    using T = typename F::Elem;
    using O1 = typename F::O1;
    constexpr int NOPS = F::NIN + F::NOUT;
    constexpr int V = 16 / (int)sizeof(T);
    MultiPlan p;
    if (!make_multi_plan(&p, ix, a, NOPS)) return;
    MultiPtrs ptr = {};
    for (int k = 0; k < NOPS; ++k) ptr.p[k] = a[k]->ptr;
    cudaStream_t st = current_stream();
    constexpr int64_t kPer = (int64_t)kBlock * kMultiUnroll;
    auto grid_for = [](int64_t tiles) { return (unsigned)(tiles < 1 ? 1 : (tiles > 0x7fffffffLL ? 0x7fffffffLL : tiles)); };

    bool flat = p.nd == 1;
    for (int k = 0; k < NOPS && flat; ++k) {
        const int64_t es = (F::NOUT == 2 && k == NOPS - 1) ? (int64_t)sizeof(O1) : (int64_t)sizeof(T);
        flat = p.step[k][0] == es && aligned16(ptr.p[k]);
    }
    int launches = 0;
    int64_t done = 0;
    if (flat && p.total >= V) {
        const int64_t n_packets = p.total / V;
        multi_flat_kernel<F><<<grid_for((n_packets + kPer - 1) / kPer), kBlock, 0, st>>>(ptr, n_packets, 0, prm, flag);
        ++launches;
        done = n_packets * V;
        for (int k = 0; k < NOPS; ++k) ptr.p[k] += done * p.step[k][0];
    }
    if (done < p.total) {
        // the elements after the last whole packet of a flat array, or everything of a view
        if (done) { p.total -= done; p.shape[0] = p.total; }
        const int64_t n_tiles = (p.total + kPer - 1) / kPer;
        multi_gen_kernel<F><<<grid_for(n_tiles), kBlock, 0, st>>>(p, ptr, n_tiles, done, prm, flag);
        ++launches;
    }
    count_launch(launches);
    cumo_cuda_runtime_check_kernel_launch();
}

namespace op {

struct NoParams {};

// x limited to [lo, hi], both from arrays; an empty range raises the flag and leaves the element (clip_kernel.cu:16-20)
template <typename T> struct ClipArrays {
    using Elem = T; using O1 = T; using Params = NoParams;
    static constexpr int NIN = 3, NOUT = 1;
    __device__ __forceinline__ static bool apply(const T* in, int64_t, const Params&, T& o0, O1&, int* flag) {
        T x = in[0];
        const T lo = in[1], hi = in[2];
        if (lo > hi) { if (flag) *flag = 1; return false; }
        if (x < lo) x = lo;
        if (x > hi) x = hi;
        o0 = x;
        return true;
    }
};

// quotient and remainder together (binary2_kernel.cu:13-25 with m_divmod: the quotient of `/`, the remainder of `%`)
template <typename T> struct DivMod {
    using Elem = T; using O1 = T; using Params = NoParams;
    static constexpr int NIN = 2, NOUT = 2;
    __device__ __forceinline__ static bool apply(const T* in, int64_t, const Params&, T& o0, O1& o1, int* flag) {
        const bool q = Div<T>::apply(in[0], in[1], o0, flag);
        const bool r = Mod<T>::apply(in[0], in[1], o1, flag);
        return q && r;
    }
};

// fractional and integral part (unary_ret2_kernel.cu:1-14 with m_modf, which goes through double for either type)
template <typename T> struct Modf {
    using Elem = T; using O1 = T; using Params = NoParams;
    static constexpr int NIN = 1, NOUT = 2;
    __device__ __forceinline__ static bool apply(const T* in, int64_t, const Params&, T& o0, O1& o1, int*) {
        double whole;
        o0 = (T)modf((double)in[0], &whole);
        o1 = (T)whole;
        return true;
    }
};

// mantissa and binary exponent (frexp_kernel.cu:1-13); the exponent goes to an Int32 array
template <typename T> struct Frexp {
    using Elem = T; using O1 = int32_t; using Params = NoParams;
    static constexpr int NIN = 1, NOUT = 2;
    __device__ __forceinline__ static bool apply(const T* in, int64_t, const Params&, T& o0, O1& o1, int*) {
        int e;
        o0 = frexp(in[0], &e);
        o1 = e;
        return true;
    }
};

// beg + step * (count + position) (seq_kernel.cu:13-35): the integer types compute in double and come back through
// a signed 64-bit integer, so that an out-of-range value wraps the way a cast does
template <typename T> struct SeqParams {
    using Data = typename std::conditional<std::is_integral<T>::value, double, T>::type;
    Data beg, step;
    double count;
};
template <typename T> struct Seq {
    using Elem = T; using O1 = T; using Params = SeqParams<T>;
    static constexpr int NIN = 0, NOUT = 1;
    __device__ __forceinline__ static bool apply(const T*, int64_t i, const Params& s, T& o0, O1&, int*) {
        const double c = s.count + (double)(uint64_t)i;
        if constexpr (std::is_integral<T>::value) o0 = (T)(int64_t)(s.beg + s.step * c);
        else o0 = (T)(s.beg + s.step * c);
        return true;
    }
};

}  // namespace op
}  // namespace cb200
