// Elementwise kernels: strided / broadcast binary and unary operations, and
// comparisons into a Bit array.
//
// They stand where the reference's per-ndim indexer kernels stand
// (ext/cumo/narray/gen/tmpl/binary_kernel.cu:14-49, unary_kernel.cu:14-25,
// unary_s_kernel.cu:2-12, cond_binary_kernel.cu:7-22, pow_kernel.cu:6-33,
// ewcomp_kernel.cu:5-14), with a different execution plan:
//
//   * the host canonicalises the descriptor (drops extent-1 dims, merges dims
//     that every operand walks with one stride) and classifies it;
//   * ROW kernel: every operand's innermost step is the element size or 0
//     (broadcast).  A CTA tile is 1024 "slots" of one 16-byte packet each,
//     laid over (row, column-packet); outer dims are decomposed once per slot
//     (one multiply when only one outer dim is left), never per element.
//     Covers contiguous, (R,C)o(R,1), (R,C)o(1,C), (R,1)o(1,C), sliced views
//     with a contiguous inner dim.  16-byte streaming loads/stores, 4 packets
//     per operand in flight per thread;
//   * GEN kernel: anything else (transposed operands, negative or non-unit
//     inner steps).  One element per slot, consecutive threads on consecutive
//     logical elements, index split in 32-bit arithmetic.
//   * comparisons write whole 32-bit words assembled with a warp OR-reduce /
//     ballot when the Bit output is contiguous and word aligned; one atomic per
//     element (the reference's CUMO_STORE_BIT, template_kernel.h:26-35) only
//     for strided or unaligned Bit outputs.
#pragma once

#include "common.cuh"
#include "ops.cuh"

namespace cb200 {

constexpr int kSlots = kBlock * kUnroll;      // slots per CTA tile

struct EwPlan {
    int nd;                                   // canonical dims, >= 1
    int64_t total;                            // elements
    int64_t shape[kMaxDim];
    int64_t step[3][kMaxDim];                 // [0],[1] inputs, [2] output (bit steps for a Bit output)
};

struct RowGeom {
    int64_t L;                                // inner extent (elements)
    int64_t R;                                // rows = total / L
    int64_t vpr;                              // slots per row = ceil(L / V)
    int64_t n_tiles;
    int32_t rows_per_tile;                    // >1: several rows per tile; 1 and chunks>1: chunked rows
    int32_t chunks_per_row;
    int32_t inner[3];                         // inner step in elements: 1 or 0
};

// Canonical plan from up to two input descriptors and an output step array.
// Returns false when there is nothing to do (an extent is 0).
inline bool make_plan(EwPlan* p, const cumo_na_indexer_t* ix, const ssize_t* s1, const ssize_t* s2,
                      const ssize_t* s3) {
    int nd = 0;
    p->total = 1;
    for (int d = 0; d < ix->ndim; ++d) {
        int64_t n = (int64_t)ix->shape[d];
        if (n == 0) return false;
        if (n == 1) continue;
        int64_t t1 = s1 ? (int64_t)s1[d] : 0, t2 = s2 ? (int64_t)s2[d] : 0, t3 = s3 ? (int64_t)s3[d] : 0;
        if (nd > 0 && p->step[0][nd - 1] == t1 * n && p->step[1][nd - 1] == t2 * n &&
            p->step[2][nd - 1] == t3 * n) {
            // previous dim strides exactly over this one for every operand: merge
            p->shape[nd - 1] *= n;
            p->step[0][nd - 1] = t1; p->step[1][nd - 1] = t2; p->step[2][nd - 1] = t3;
        } else {
            p->shape[nd] = n;
            p->step[0][nd] = t1; p->step[1][nd] = t2; p->step[2][nd] = t3;
            ++nd;
        }
        p->total *= n;
    }
    if (nd == 0) {
        nd = 1;
        p->shape[0] = 1;
        p->step[0][0] = p->step[1][0] = p->step[2][0] = 0;
    }
    p->nd = nd;
    return true;
}

// ----------------------------------------------------------------------------
// ROW kernel
// ----------------------------------------------------------------------------
template <typename Op, int V>
__global__ void __launch_bounds__(kBlock)
ew_row_kernel(const EwPlan p, const RowGeom g, const char* __restrict__ a1, const char* __restrict__ a2,
              char* a3, typename Op::In1 sx, typename Op::In2 sy, int use_scalar, int* flag) {
    using T1 = typename Op::In1;
    using T2 = typename Op::In2;
    using TO = typename Op::Out;
    static_assert(sizeof(T1) == sizeof(TO) && sizeof(T2) == sizeof(TO), "row kernel needs equal element sizes");
    constexpr int ES = sizeof(TO);
    const bool have1 = use_scalar != 2;
    const bool have2 = Op::arity == 2 && use_scalar != 1;
    const int nd_outer = p.nd - 1;

    for (int64_t tile = blockIdx.x; tile < g.n_tiles; tile += gridDim.x) {
        int64_t off[kUnroll][3];
        int64_t col[kUnroll];
        bool ok[kUnroll];
        // where each of my slots lies
        if (g.rows_per_tile == 1) {
            int64_t row = tile / g.chunks_per_row;
            int64_t c0 = (tile - row * g.chunks_per_row) * kSlots;
            int64_t ro[3];
            offsets_of<3>(row, nd_outer, p.shape, p.step, ro);
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                int64_t c = c0 + j * kBlock + threadIdx.x;
                col[j] = c * V;
                ok[j] = col[j] < g.L;
                off[j][0] = ro[0]; off[j][1] = ro[1]; off[j][2] = ro[2];
            }
        } else {
            const uint32_t vpr = (uint32_t)g.vpr;
            const uint32_t live = vpr * (uint32_t)g.rows_per_tile;
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                uint32_t k = j * kBlock + threadIdx.x;
                uint32_t r = k / vpr;
                uint32_t c = k - r * vpr;
                int64_t row = tile * g.rows_per_tile + r;
                col[j] = (int64_t)c * V;
                ok[j] = k < live && row < g.R;
                if (ok[j]) offsets_of<3>(row, nd_outer, p.shape, p.step, off[j]);
            }
        }

        // issue every load of the tile before the first use
        Pack<TO> x[kUnroll], y[kUnroll];
        int nv[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            nv[j] = 0;
            if (!ok[j]) continue;
            int64_t left = g.L - col[j];
            nv[j] = left < V ? (int)left : V;
            if (have1) {
                const char* q = a1 + off[j][0] + col[j] * g.inner[0] * ES;
                if (g.inner[0] == 0) {
                    T1 s = ld_one<T1>(q);
#pragma unroll
                    for (int e = 0; e < V; ++e) reinterpret_cast<T1*>(&x[j])[e] = s;
                } else if (V > 1 && nv[j] == V) {
                    *reinterpret_cast<Pack<T1>*>(&x[j]) = ld_pack<T1>(q);
                } else {
#pragma unroll
                    for (int e = 0; e < V; ++e)
                        if (e < nv[j]) reinterpret_cast<T1*>(&x[j])[e] = ld_one<T1>(q + e * ES);
                }
            }
            if (have2) {
                const char* q = a2 + off[j][1] + col[j] * g.inner[1] * ES;
                if (g.inner[1] == 0) {
                    T2 s = ld_one<T2>(q);
#pragma unroll
                    for (int e = 0; e < V; ++e) reinterpret_cast<T2*>(&y[j])[e] = s;
                } else if (V > 1 && nv[j] == V) {
                    *reinterpret_cast<Pack<T2>*>(&y[j]) = ld_pack<T2>(q);
                } else {
#pragma unroll
                    for (int e = 0; e < V; ++e)
                        if (e < nv[j]) reinterpret_cast<T2*>(&y[j])[e] = ld_one<T2>(q + e * ES);
                }
            }
        }

#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            if (!ok[j]) continue;
            char* q = a3 + off[j][2] + col[j] * ES;
            Pack<TO> z;
            unsigned keep = 0;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                T1 xv = have1 ? reinterpret_cast<T1*>(&x[j])[e] : sx;
                T2 yv = have2 ? reinterpret_cast<T2*>(&y[j])[e] : sy;
                TO zv = TO();
                if (e < nv[j] && Op::apply(xv, yv, zv, flag)) keep |= 1u << e;
                z.v[e] = zv;
            }
            if (V > 1 && keep == (1u << V) - 1u) {
                st_pack<TO>(q, z);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e)
                    if (keep & (1u << e)) st_one<TO>(q + e * ES, z.v[e]);
            }
        }
    }
}

// ----------------------------------------------------------------------------
// GEN kernel: any strides, any element sizes
// ----------------------------------------------------------------------------
template <typename Op>
__global__ void __launch_bounds__(kBlock)
ew_gen_kernel(const EwPlan p, int64_t n_tiles, const char* __restrict__ a1, const char* __restrict__ a2,
              char* a3, typename Op::In1 sx, typename Op::In2 sy, int use_scalar, int* flag) {
    using T1 = typename Op::In1;
    using T2 = typename Op::In2;
    using TO = typename Op::Out;
    const bool have1 = use_scalar != 2;
    const bool have2 = Op::arity == 2 && use_scalar != 1;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        int64_t off[kUnroll][3];
        bool ok[kUnroll];
        T1 x[kUnroll];
        T2 y[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            int64_t i = tile * kSlots + j * kBlock + threadIdx.x;
            ok[j] = i < p.total;
            if (ok[j]) {
                offsets_of<3>(i, p.nd, p.shape, p.step, off[j]);
                x[j] = have1 ? ld_one<T1>(a1 + off[j][0]) : sx;
                y[j] = have2 ? ld_one<T2>(a2 + off[j][1]) : sy;
            }
        }
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            if (!ok[j]) continue;
            TO z;
            if (Op::apply(x[j], y[j], z, flag)) st_one<TO>(a3 + off[j][2], z);
        }
    }
}

// host side ---------------------------------------------------------------
template <typename Op>
void launch_elementwise(const cumo_na_iarray_t* a1, const cumo_na_iarray_t* a2, cumo_na_iarray_t* a3,
                        const cumo_na_indexer_t* ix, typename Op::In1 sx, typename Op::In2 sy,
                        int use_scalar, int* flag) {
    using T1 = typename Op::In1;
    using T2 = typename Op::In2;
    using TO = typename Op::Out;
    constexpr int ES = sizeof(TO);
    const bool have1 = use_scalar != 2 && a1 != nullptr;
    const bool have2 = Op::arity == 2 && use_scalar != 1 && a2 != nullptr;
    EwPlan p;
    if (!make_plan(&p, ix, have1 ? a1->step : nullptr, have2 ? a2->step : nullptr, a3->step)) return;
    const char* p1 = have1 ? a1->ptr : nullptr;
    const char* p2 = have2 ? a2->ptr : nullptr;
    char* p3 = a3->ptr;
    cudaStream_t st = current_stream();

    constexpr bool same_size = sizeof(T1) == ES && sizeof(T2) == ES;
    const int in = p.nd - 1;
    bool row_ok = same_size && p.step[2][in] == ES &&
                  (!have1 || p.step[0][in] == ES || p.step[0][in] == 0) &&
                  (!have2 || p.step[1][in] == ES || p.step[1][in] == 0);
    // a short inner dim under several outer dims pays the outer decomposition
    // per packet; the generic kernel is the better plan there
    if (row_ok && p.nd > 2 && p.shape[in] * ES < 64) row_ok = false;

    if constexpr (same_size) {
        if (row_ok) {
            constexpr int VMAX = 16 / ES;
            bool vec = aligned16(p3) && (!have1 || p.step[0][in] == 0 || aligned16(p1)) &&
                       (!have2 || p.step[1][in] == 0 || aligned16(p2));
            for (int d = 0; d < in && vec; ++d) {
                if (!mult16(p.step[2][d])) vec = false;
                if (have1 && p.step[0][in] != 0 && !mult16(p.step[0][d])) vec = false;
                if (have2 && p.step[1][in] != 0 && !mult16(p.step[1][d])) vec = false;
            }
            const int V = vec ? VMAX : 1;
            RowGeom g;
            g.L = p.shape[in];
            g.R = p.total / g.L;
            g.vpr = (g.L + V - 1) / V;
            g.inner[0] = have1 && p.step[0][in] != 0;
            g.inner[1] = have2 && p.step[1][in] != 0;
            g.inner[2] = 1;
            if (g.vpr >= kSlots) {
                g.rows_per_tile = 1;
                g.chunks_per_row = (int32_t)((g.vpr + kSlots - 1) / kSlots);
                g.n_tiles = g.R * g.chunks_per_row;
            } else {
                g.rows_per_tile = (int32_t)(kSlots / g.vpr);
                g.chunks_per_row = 1;
                g.n_tiles = (g.R + g.rows_per_tile - 1) / g.rows_per_tile;
            }
            unsigned grid = grid_for(g.n_tiles, 8);
            if (vec)
                ew_row_kernel<Op, VMAX><<<grid, kBlock, 0, st>>>(p, g, p1, p2, p3, sx, sy, use_scalar, flag);
            else
                ew_row_kernel<Op, 1><<<grid, kBlock, 0, st>>>(p, g, p1, p2, p3, sx, sy, use_scalar, flag);
            count_launch();
            cumo_cuda_runtime_check_kernel_launch();
            return;
        }
    }
    int64_t n_tiles = (p.total + kSlots - 1) / kSlots;
    ew_gen_kernel<Op><<<grid_for(n_tiles, 8), kBlock, 0, st>>>(p, n_tiles, p1, p2, p3, sx, sy, use_scalar, flag);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

// ----------------------------------------------------------------------------
// Comparisons -> Bit
// ----------------------------------------------------------------------------
// Flat kernel: inputs contiguous (or broadcast scalars), Bit output contiguous
// and starting on a word boundary.  Each lane tests V consecutive elements;
// the 32/V lanes that share an output word OR their bit groups together.
template <typename Op, int V>
__global__ void __launch_bounds__(kBlock)
cmp_flat_kernel(int64_t total, int64_t n_tiles, const char* __restrict__ a1, const char* __restrict__ a2,
                uint32_t* out, int st1, int st2, typename Op::In1 sx, typename Op::In2 sy, int use_scalar) {
    using T1 = typename Op::In1;
    using T2 = typename Op::In2;
    constexpr int ES = sizeof(T1);
    constexpr int LPW = 32 / V;               // lanes per output word
    const bool have1 = use_scalar != 2;
    const bool have2 = Op::arity == 2 && use_scalar != 1;
    const int lane = threadIdx.x & 31;
    const unsigned group_mask = (LPW == 32) ? 0xffffffffu : (((1u << LPW) - 1u) << (lane / LPW * LPW));
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        Pack<T1> x[kUnroll];
        Pack<T2> y[kUnroll];
        int64_t e0[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            e0[j] = (tile * kSlots + j * kBlock + threadIdx.x) * (int64_t)V;
            int64_t left = total - e0[j];
            if (left <= 0) continue;
            if (have1) {
                if (st1 == 0) { T1 s = ld_one<T1>(a1);
#pragma unroll
                    for (int e = 0; e < V; ++e) x[j].v[e] = s; }
                else if (V > 1 && left >= V) x[j] = ld_pack<T1>(a1 + e0[j] * ES);
                else {
#pragma unroll
                    for (int e = 0; e < V; ++e) if (e < left) x[j].v[e] = ld_one<T1>(a1 + (e0[j] + e) * ES); }
            }
            if (have2) {
                if (st2 == 0) { T2 s = ld_one<T2>(a2);
#pragma unroll
                    for (int e = 0; e < V; ++e) y[j].v[e] = s; }
                else if (V > 1 && left >= V) y[j] = ld_pack<T2>(a2 + e0[j] * ES);
                else {
#pragma unroll
                    for (int e = 0; e < V; ++e) if (e < left) y[j].v[e] = ld_one<T2>(a2 + (e0[j] + e) * ES); }
            }
        }
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            int64_t left = total - e0[j];
            uint32_t bits = 0;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                if (e < left) {
                    T1 xv = have1 ? x[j].v[e] : sx;
                    T2 yv = have2 ? y[j].v[e] : sy;
                    bits |= (Op::test(xv, yv) ? 1u : 0u) << e;
                }
            }
            bits <<= (lane % LPW) * V;
            uint32_t word = __reduce_or_sync(group_mask, bits);
            if (lane % LPW == 0 && left > 0) {
                int64_t w = e0[j] >> 5;
                if (left >= 32) out[w] = word;
                else {                         // last, partial word: keep the bits past the end
                    uint32_t m = (1u << left) - 1u;
                    out[w] = (out[w] & ~m) | (word & m);
                }
            }
        }
    }
}

// Generic comparison kernel.  word_store: the Bit output is contiguous and word
// aligned, so a warp's ballot is one whole output word.
template <typename Op>
__global__ void __launch_bounds__(kBlock)
cmp_gen_kernel(const EwPlan p, int64_t n_tiles, const char* __restrict__ a1, const char* __restrict__ a2,
               uint32_t* out, uint64_t pos, int word_store, typename Op::In1 sx, typename Op::In2 sy,
               int use_scalar) {
    using T1 = typename Op::In1;
    using T2 = typename Op::In2;
    const bool have1 = use_scalar != 2;
    const bool have2 = Op::arity == 2 && use_scalar != 1;
    const int lane = threadIdx.x & 31;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            int64_t i = tile * kSlots + j * kBlock + threadIdx.x;
            bool ok = i < p.total;
            bool r = false;
            int64_t off[3] = {0, 0, 0};
            if (ok) {
                offsets_of<3>(i, p.nd, p.shape, p.step, off);
                T1 x = have1 ? ld_one<T1>(a1 + off[0]) : sx;
                T2 y = have2 ? ld_one<T2>(a2 + off[1]) : sy;
                r = Op::test(x, y);
            }
            if (word_store) {
                uint32_t word = __ballot_sync(0xffffffffu, r);
                int64_t i0 = i - lane;        // multiple of 32
                if (lane == 0 && i0 < p.total) {
                    int64_t left = p.total - i0;
                    int64_t w = (int64_t)(pos >> 5) + (i0 >> 5);
                    if (left >= 32) out[w] = word;
                    else {
                        uint32_t m = (1u << left) - 1u;
                        out[w] = (out[w] & ~m) | (word & m);
                    }
                }
            } else if (ok) {
                uint64_t b = pos + (uint64_t)off[2];
                if (r) atomicOr(out + (b >> 5), 1u << (b & 31));
                else atomicAnd(out + (b >> 5), ~(1u << (b & 31)));
            }
        }
    }
}

template <typename Op>
void launch_compare(const cumo_na_iarray_t* a1, const cumo_na_iarray_t* a2, cumo_na_bit_iarray_t* a3,
                    const cumo_na_indexer_t* ix, typename Op::In1 sx, typename Op::In2 sy, int use_scalar) {
    using T1 = typename Op::In1;
    constexpr int ES = sizeof(T1);
    const bool have1 = use_scalar != 2 && a1 != nullptr;
    const bool have2 = Op::arity == 2 && use_scalar != 1 && a2 != nullptr;
    EwPlan p;
    if (!make_plan(&p, ix, have1 ? a1->step : nullptr, have2 ? a2->step : nullptr, a3->step)) return;
    const char* p1 = have1 ? a1->ptr : nullptr;
    const char* p2 = have2 ? a2->ptr : nullptr;
    cudaStream_t st = current_stream();
    const bool out_flat = p.nd == 1 && (p.step[2][0] == 1 || p.total == 1) && (a3->pos & 31) == 0;
    const bool in_flat = p.nd == 1 && (!have1 || p.step[0][0] == ES || p.step[0][0] == 0) &&
                         (!have2 || p.step[1][0] == ES || p.step[1][0] == 0);
    if (out_flat && in_flat) {
        uint32_t* out = a3->ptr + (a3->pos >> 5);
        int st1 = have1 && p.step[0][0] != 0, st2 = have2 && p.step[1][0] != 0;
        constexpr int VMAX = 16 / ES;
        bool vec = (!st1 || aligned16(p1)) && (!st2 || aligned16(p2));
        if (vec) {
            int64_t n_tiles = (p.total + (int64_t)kSlots * VMAX - 1) / ((int64_t)kSlots * VMAX);
            cmp_flat_kernel<Op, VMAX><<<grid_for(n_tiles, 8), kBlock, 0, st>>>(p.total, n_tiles, p1, p2, out, st1, st2, sx, sy, use_scalar);
        } else {
            int64_t n_tiles = (p.total + kSlots - 1) / kSlots;
            cmp_flat_kernel<Op, 1><<<grid_for(n_tiles, 8), kBlock, 0, st>>>(p.total, n_tiles, p1, p2, out, st1, st2, sx, sy, use_scalar);
        }
    } else {
        // is the output still one run of bits in logical order?
        bool word_store = (a3->pos & 31) == 0;
        int64_t run = 1;
        for (int d = p.nd - 1; d >= 0 && word_store; --d) {
            if (p.step[2][d] != run) word_store = false;
            run *= p.shape[d];
        }
        int64_t n_tiles = (p.total + kSlots - 1) / kSlots;
        cmp_gen_kernel<Op><<<grid_for(n_tiles, 8), kBlock, 0, st>>>(p, n_tiles, p1, p2, a3->ptr, (uint64_t)a3->pos, word_store ? 1 : 0, sx, sy, use_scalar);
    }
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200
