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
//     (broadcast).  One CTA = one tile of 512 "slots" of one 16-byte packet each,
//     laid over (row, column-packet), two packets per operand in flight per
//     thread, a grid of as many CTAs as there are tiles (measured on B200: many
//     small CTAs stream ~10% faster than a persistent grid-stride loop).  Index
//     arithmetic is 32-bit and per slot, never per element: one multiply per
//     operand when at most one outer dim is left (contiguous, (R,C)o(R,1),
//     (R,C)o(1,C), (R,1)o(1,C), row-sliced views), a short division chain when
//     several outer dims survive canonicalisation;
//   * TILE kernel: an input whose contiguous axis is not the output's (a transposed
//     operand): staged through a padded shared-memory tile so that every operand is
//     read and written along its own contiguous axis;
//   * GEN kernel: anything else (negative or non-unit inner steps, short extents,
//     index patterns with no contiguous axis).  One element per slot, consecutive
//     threads on consecutive logical elements.
//   * comparisons write whole 32-bit words assembled with a warp OR-reduce /
//     ballot when the Bit output is contiguous and word aligned; one atomic per
//     element (the reference's CUMO_STORE_BIT, template_kernel.h:26-35) only
//     for strided or unaligned Bit outputs.
#pragma once

#include "common.cuh"
#include "ops.cuh"
#include "tile_tma.cuh"

namespace cb200 {

constexpr int kEwUnroll = 2;                     // packets per operand in flight per thread
constexpr int kEwSlots = kBlock * kEwUnroll;     // slots per CTA tile
constexpr int64_t kMaxGrid = 0x7fffffffLL;

struct EwPlan {
    int nd;                                   // canonical dims, >= 1
    int64_t total;                            // elements
    int64_t shape[kMaxDim];
    int64_t step[3][kMaxDim];                 // [0],[1] inputs, [2] output (bit steps for a Bit output)
};

struct RowGeom {
    int64_t L;                                // inner extent (elements)
    int64_t R;                                // rows = total / L
    int64_t n_tiles;
    int64_t rs[3];                            // row step (bytes) per operand when one outer dim is left
    uint32_t vpr;                             // slots per row = ceil(L / V)
    uint32_t rows_per_tile;                   // >1: several rows per tile
    uint32_t chunks_per_row;                  // >1: several tiles per row
    int32_t inner[2];                         // inner step of the inputs in elements: 1 or 0
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
// ROW kernel.  ND: more than one outer dim (offsets from an index split).
// ----------------------------------------------------------------------------
template <typename Op, int V, bool ND>
__global__ void __launch_bounds__(kBlock)
ew_row_kernel(const EwPlan p, const RowGeom g, const char* __restrict__ a1, const char* __restrict__ a2,
              char* a3, typename Op::In1 sx, typename Op::In2 sy, int use_scalar, int* flag) {
    using T1 = typename Op::In1;
    using T2 = typename Op::In2;
    using TO = typename Op::Out;
    static_assert(sizeof(T1) == sizeof(TO) && sizeof(T2) == sizeof(TO), "row kernel needs equal element sizes");
    constexpr int ES = sizeof(TO);
    constexpr int U = kEwUnroll;
    const bool have1 = use_scalar != 2;
    const bool have2 = Op::arity == 2 && use_scalar != 1;

    for (int64_t tile = blockIdx.x; tile < g.n_tiles; tile += gridDim.x) {   // one pass unless the grid was capped
        int64_t row[U];
        uint32_t col[U];                       // first element of my packet within the row
        bool ok[U];
        if (g.rows_per_tile == 1) {
            int64_t r;
            uint32_t ch;
            if (tile <= 0xffffffffLL) {        // 32-bit division: this sits on every CTA's critical path
                const uint32_t t = (uint32_t)tile, rr = t / g.chunks_per_row;
                r = rr; ch = t - rr * g.chunks_per_row;
            } else {
                r = tile / g.chunks_per_row; ch = (uint32_t)(tile - r * g.chunks_per_row);
            }
#pragma unroll
            for (int j = 0; j < U; ++j) {
                row[j] = r;
                uint64_t c = ((uint64_t)ch * kEwSlots + j * kBlock + threadIdx.x) * V;
                ok[j] = c < (uint64_t)g.L;
                col[j] = (uint32_t)c;
            }
        } else {
            const uint32_t live = g.vpr * g.rows_per_tile;
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const uint32_t k = j * kBlock + threadIdx.x;
                const uint32_t r = k / g.vpr;
                col[j] = (k - r * g.vpr) * V;
                row[j] = tile * g.rows_per_tile + r;
                ok[j] = k < live && row[j] < g.R;
            }
        }
        int64_t off[U][3];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (ND) {
                if (ok[j]) offsets_of<3>(row[j], p.nd - 1, p.shape, p.step, off[j]);
            } else {
                off[j][0] = row[j] * g.rs[0]; off[j][1] = row[j] * g.rs[1]; off[j][2] = row[j] * g.rs[2];
            }
        }

        // issue every load of the tile before the first use.  The host only picks V > 1 when
        // the inner extent is a multiple of V, so a live slot always holds a whole packet.
        Pack<T1> x[U];
        Pack<T2> y[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (!ok[j]) continue;
            if (have1) {
                const char* q = a1 + off[j][0] + (int64_t)col[j] * (g.inner[0] * ES);
                if (g.inner[0] == 0) {
                    T1 s = ld_one<T1>(q);
#pragma unroll
                    for (int e = 0; e < V; ++e) x[j].v[e] = s;
                } else {
                    if (V > 1) x[j] = ld_pack<T1>(q); else x[j].v[0] = ld_one<T1>(q);
                }
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) x[j].v[e] = sx;
            }
            if (have2) {
                const char* q = a2 + off[j][1] + (int64_t)col[j] * (g.inner[1] * ES);
                if (g.inner[1] == 0) {
                    T2 s = ld_one<T2>(q);
#pragma unroll
                    for (int e = 0; e < V; ++e) y[j].v[e] = s;
                } else {
                    if (V > 1) y[j] = ld_pack<T2>(q); else y[j].v[0] = ld_one<T2>(q);
                }
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) y[j].v[e] = sy;
            }
        }

#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (!ok[j]) continue;
            char* q = a3 + off[j][2] + (int64_t)col[j] * ES;
            Pack<TO> z;
            unsigned keep = 0;                 // folds to a constant for operations that never skip
#pragma unroll
            for (int e = 0; e < V; ++e) {
                TO zv = TO();
                if (ew_apply<Op>(x[j].v[e], y[j].v[e], sx, zv, flag)) keep |= 1u << e;
                z.v[e] = zv;
            }
            if (keep == (1u << V) - 1u) {
                if (V > 1) st_pack<TO>(q, z); else st_one<TO>(q, z.v[0]);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e)
                    if (keep & (1u << e)) st_one<TO>(q + e * ES, z.v[e]);
            }
        }
    }
}

// ----------------------------------------------------------------------------
// ROW-SHARE kernel.  Two canonical dims (rows x L) where an input is a row vector
// repeated down the rows (row step 0, inner step one element) and the other input
// is one element per row, another such vector or a scalar: x(R,1) + y(1,C).  The
// output is the only real traffic, and the plain row kernel spends ~100 instructions
// per 16-byte store on index arithmetic that is the same for every row; here a CTA
// keeps its packets of the vector in registers and walks kShareRows rows with them.
// ----------------------------------------------------------------------------
constexpr int kShareRows = 16;                   // rows per CTA
constexpr int kShareBatch = 4;                   // rows whose loads are issued together

// How an input reaches a row of the tile.  The kernel is compiled per pair of modes so that
// its inner loop carries no tests and no copies.
enum : int { kHeld = 0,      // same packets for every row: the shared row vector, or a scalar argument
             kRowScalar = 1, // one element per row (inner step 0)
             kRowPack = 2 }; // a packet per row and slot

template <typename Op, int V, int M1, int M2>
__global__ void __launch_bounds__(kBlock)
ew_rowshare_kernel(const RowGeom g, const char* __restrict__ a1, const char* __restrict__ a2, char* a3,
                   typename Op::In1 sx, typename Op::In2 sy, int* flag) {
    using T1 = typename Op::In1;
    using T2 = typename Op::In2;
    using TO = typename Op::Out;
    constexpr int ES = sizeof(TO);
    constexpr int U = kEwUnroll;
    constexpr int B = kShareBatch;
    // an input that is one element per row: the first kShareRows threads fetch the tile's values once and everyone
    // reads them back from shared memory (a broadcast read), instead of every thread loading every row's element
    __shared__ T1 row1[M1 == kRowScalar ? kShareRows : 1];
    __shared__ T2 row2[M2 == kRowScalar ? kShareRows : 1];

    for (int64_t tile = blockIdx.x; tile < g.n_tiles; tile += gridDim.x) {   // one pass unless the grid was capped
        int64_t rg;
        uint32_t ch;
        if (tile <= 0xffffffffLL) {
            const uint32_t t = (uint32_t)tile, q = t / g.chunks_per_row;
            rg = q; ch = t - q * g.chunks_per_row;
        } else {
            rg = tile / g.chunks_per_row; ch = (uint32_t)(tile - rg * g.chunks_per_row);
        }
        uint32_t col[U];                       // byte offset of my packet within a row
        bool ok[U];
        Pack<T1> xs[U];
        Pack<T2> ys[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const uint64_t c = ((uint64_t)ch * kEwSlots + j * kBlock + threadIdx.x) * V;
            ok[j] = c < (uint64_t)g.L;
            col[j] = (uint32_t)c * ES;
#pragma unroll
            for (int e = 0; e < V; ++e) { xs[j].v[e] = sx; ys[j].v[e] = sy; }
            if (ok[j]) {
                if (M1 == kHeld && a1) xs[j] = ld_pack<T1>(a1 + col[j]);
                if (M2 == kHeld && a2) ys[j] = ld_pack<T2>(a2 + col[j]);
            }
        }
        const int64_t row0 = rg * kShareRows;
        const int rows = (int)(g.R - row0 < kShareRows ? g.R - row0 : kShareRows);
        const char* q1 = a1 + row0 * g.rs[0];
        const char* q2 = a2 + row0 * g.rs[1];
        char* q3 = a3 + row0 * g.rs[2];
        if (M1 == kRowScalar || M2 == kRowScalar) {
            __syncthreads();                   // the previous tile's values may still be read
            if ((int)threadIdx.x < rows) {
                if (M1 == kRowScalar) row1[threadIdx.x] = ld_one<T1>(q1 + (int64_t)threadIdx.x * g.rs[0]);
                if (M2 == kRowScalar) row2[threadIdx.x] = ld_one<T2>(q2 + (int64_t)threadIdx.x * g.rs[1]);
            }
            __syncthreads();
        }
        for (int rb = 0; rb < rows; rb += B) {
            T1 xr[B];
            T2 yr[B];
            Pack<T1> xp[B][U];
            Pack<T2> yp[B][U];
#pragma unroll
            for (int r = 0; r < B; ++r) {
                if (rb + r >= rows) continue;
                if (M1 == kRowScalar) xr[r] = row1[rb + r];
                if (M2 == kRowScalar) yr[r] = row2[rb + r];
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    if (!ok[j]) continue;
                    if (M1 == kRowPack) xp[r][j] = ld_pack<T1>(q1 + r * g.rs[0] + col[j]);
                    if (M2 == kRowPack) yp[r][j] = ld_pack<T2>(q2 + r * g.rs[1] + col[j]);
                }
            }
#pragma unroll
            for (int r = 0; r < B; ++r) {
                if (rb + r >= rows) continue;
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    if (!ok[j]) continue;
                    char* q = q3 + r * g.rs[2] + col[j];
                    Pack<TO> z;
                    unsigned keep = 0;
#pragma unroll
                    for (int e = 0; e < V; ++e) {
                        const T1 xv = M1 == kHeld ? xs[j].v[e] : M1 == kRowScalar ? xr[r] : xp[r][j].v[e];
                        const T2 yv = M2 == kHeld ? ys[j].v[e] : M2 == kRowScalar ? yr[r] : yp[r][j].v[e];
                        TO zv = TO();
                        if (ew_apply<Op>(xv, yv, sx, zv, flag)) keep |= 1u << e;
                        z.v[e] = zv;
                    }
                    if (keep == (1u << V) - 1u) {
                        st_pack<TO>(q, z);
                    } else {
#pragma unroll
                        for (int e = 0; e < V; ++e)
                            if (keep & (1u << e)) st_one<TO>(q + e * ES, z.v[e]);
                    }
                }
            }
            q1 += B * g.rs[0];
            q2 += B * g.rs[1];
            q3 += B * g.rs[2];
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
    constexpr int U = kEwUnroll;
    const bool have1 = use_scalar != 2;
    const bool have2 = Op::arity == 2 && use_scalar != 1;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        int64_t off[U][3];
        bool ok[U];
        T1 x[U];
        T2 y[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            int64_t i = tile * kEwSlots + j * kBlock + threadIdx.x;
            ok[j] = i < p.total;
            if (ok[j]) {
                offsets_of<3>(i, p.nd, p.shape, p.step, off[j]);
                x[j] = have1 ? ld_one<T1>(a1 + off[j][0]) : sx;
                y[j] = have2 ? ld_one<T2>(a2 + off[j][1]) : sy;
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (!ok[j]) continue;
            TO z;
            if (ew_apply<Op>(x[j], y[j], sx, z, flag)) st_one<TO>(a3 + off[j][2], z);
        }
    }
}

// ----------------------------------------------------------------------------
// TILE kernel: operands whose contiguous axes differ (a transposed operand).
// ----------------------------------------------------------------------------
// out[r][c] = op(x[r][c], y[r][c]) over a plane (r, c) in which the output is contiguous along c and at least one
// input is contiguous along r instead (`a + b.transpose`, `b.transpose.dup`, `SFloat.cast(m.transpose)`).  The generic
// kernel reads such an input with a stride between neighbouring lanes: one 32-byte sector fetched per element used.
// Here a CTA takes a tile of kTileR x TC elements; a transposed input's tile is first read with the lanes running
// along ITS contiguous axis (r) and parked in shared memory, rows padded by one element; then the lanes run along c,
// pick the parked values column-wise (conflict-free thanks to the padding), load the row-like operands, and store
// the result -- every global access of every operand is a run of consecutive elements per warp.  Dimensions other
// than the two of the plane are walked as a batch index.  Works for any element sizes and alignments.
constexpr int kTileR = 64;

template <typename Op, bool T1, bool T2, int TC>
__global__ void __launch_bounds__(kBlock)
ew_tile_kernel(const TilePlan t, const char* __restrict__ a1, const char* __restrict__ a2, char* a3,
               typename Op::In1 sx, typename Op::In2 sy, int use_scalar, int* flag) {
    using X = typename Op::In1;
    using Y = typename Op::In2;
    using TO = typename Op::Out;
    constexpr int TR = kTileR;
    __shared__ X tile1[T1 ? TC : 1][T1 ? TR + 1 : 1];
    __shared__ Y tile2[T2 ? TC : 1][T2 ? TR + 1 : 1];
    const bool have1 = use_scalar != 2;
    const bool have2 = Op::arity == 2 && use_scalar != 1;
    for (int64_t tile = blockIdx.x; tile < t.n_tiles; tile += gridDim.x) {
        // tiles along c vary fastest (the CTAs resident at one time write long runs of each output row), then r, then the batch
        const int64_t tc = tile % t.tiles_c;
        const int64_t rest = tile / t.tiles_c;
        const int64_t tr = rest % t.tiles_r;
        const int64_t batch = rest / t.tiles_r;
        int64_t off[3];
        offsets_of<3>(batch, t.n_outer, t.oshape, t.ostep, off);
        const int64_t r0 = tr * TR, c0 = tc * TC;
        if (T1 || T2) {
            // lanes along r: element (r0 + lr, c0 + lc) of a transposed input sits lr elements on from the start of its line.
            // All of a thread's loads are issued before the first is parked, so that they are in flight together.
            constexpr int CP = kBlock / TR;        // lines per pass
            constexpr int NL = TC / CP;            // loads per thread and operand
            const int lr = threadIdx.x % TR;
            const int lc0 = threadIdx.x / TR;
            const bool r_ok = r0 + lr < t.R;
            X xv[T1 ? NL : 1];
            Y yv[T2 ? NL : 1];
            const char* q1 = a1 + off[0] + (r0 + lr) * t.rstep[0] + (c0 + lc0) * t.cstep[0];
            const char* q2 = a2 + off[1] + (r0 + lr) * t.rstep[1] + (c0 + lc0) * t.cstep[1];
#pragma unroll
            for (int j = 0; j < NL; ++j) {
                const bool ok = r_ok && c0 + lc0 + j * CP < t.C;
                if (T1) xv[j] = ok ? ld_one<X>(q1 + (int64_t)j * CP * t.cstep[0]) : X();
                if (T2) yv[j] = ok ? ld_one<Y>(q2 + (int64_t)j * CP * t.cstep[1]) : Y();
            }
            __syncthreads();                   // the previous tile may still be read
#pragma unroll
            for (int j = 0; j < NL; ++j) {
                if (T1) tile1[lc0 + j * CP][lr] = xv[j];
                if (T2) tile2[lc0 + j * CP][lr] = yv[j];
            }
            __syncthreads();
        }
        // lanes along c
        const int lc = threadIdx.x % TC;
        const bool c_ok = c0 + lc < t.C;
        constexpr int RP = kBlock / TC;        // rows per pass
        constexpr int UN = 8;                  // loads of the row-like operands in flight per thread
        const int lrt = threadIdx.x / TC;
        const char* w1 = a1 + off[0] + (r0 + lrt) * t.rstep[0] + (c0 + lc) * t.cstep[0];
        const char* w2 = a2 + off[1] + (r0 + lrt) * t.rstep[1] + (c0 + lc) * t.cstep[1];
        char* w3 = a3 + off[2] + (r0 + lrt) * t.rstep[2] + (c0 + lc) * t.cstep[2];
        for (int lr0 = lrt; lr0 < TR; lr0 += RP * UN) {
            X x[UN];
            Y y[UN];
            bool ok[UN];
#pragma unroll
            for (int j = 0; j < UN; ++j) {
                const int lr = lr0 + j * RP;
                ok[j] = c_ok && lr < TR && r0 + lr < t.R;
                x[j] = sx; y[j] = sy;
                if (!ok[j]) continue;
                if (T1) x[j] = tile1[lc][lr];
                else if (have1) x[j] = ld_one<X>(w1 + (int64_t)(lr - lrt) * t.rstep[0]);
                if (T2) y[j] = tile2[lc][lr];
                else if (have2) y[j] = ld_one<Y>(w2 + (int64_t)(lr - lrt) * t.rstep[1]);
            }
#pragma unroll
            for (int j = 0; j < UN; ++j) {
                if (!ok[j]) continue;
                const int lr = lr0 + j * RP;
                TO z;
                if (ew_apply<Op>(x[j], y[j], sx, z, flag)) st_one<TO>(w3 + (int64_t)(lr - lrt) * t.rstep[2], z);
            }
        }
    }
}

// The same plan with 16-byte global accesses, for operands of one element size whose lines are 16-byte aligned and
// whose plane extents are whole packets: the transposed input is read a packet (V elements along r) at a time and parked
// element by element; the output phase gathers V parked elements (along c) per thread, loads one packet of each row-like
// operand and stores one packet.  About a fifth of the instructions per element of the element-wise form, which is
// bound by instruction issue, not by DRAM (75 % of issue slots busy at 57 % of DRAM throughput when measured).
template <typename Op, bool T1, bool T2, int TC>
__global__ void __launch_bounds__(kBlock)
ew_tile_vec_kernel(const TilePlan t, const char* __restrict__ a1, const char* __restrict__ a2, char* a3,
                   typename Op::In1 sx, typename Op::In2 sy, int use_scalar, int* flag) {
    using X = typename Op::In1;
    using Y = typename Op::In2;
    using TO = typename Op::Out;
    static_assert(sizeof(X) == sizeof(TO) && sizeof(Y) == sizeof(TO), "one element size");
    constexpr int ES = sizeof(TO);
    constexpr int V = 16 / ES;
    constexpr int TR = kTileR;
    constexpr int PR = TR / V;                 // packets along r per line
    constexpr int LP = kBlock / PR;            // lines per pass of the load phase
    constexpr int NL = TC / LP;                // passes
    constexpr int PC = TC / V;                 // packets along c per row
    constexpr int RP = kBlock / PC;            // rows per pass of the output phase
    constexpr int NR = TR / RP;                // passes
    __shared__ X tile1[T1 ? TC : 1][T1 ? TR + 1 : 1];
    __shared__ Y tile2[T2 ? TC : 1][T2 ? TR + 1 : 1];
    const bool have1 = use_scalar != 2;
    const bool have2 = Op::arity == 2 && use_scalar != 1;
    for (int64_t tile = blockIdx.x; tile < t.n_tiles; tile += gridDim.x) {
        const int64_t tc = tile % t.tiles_c;
        const int64_t rest = tile / t.tiles_c;
        const int64_t tr = rest % t.tiles_r;
        const int64_t batch = rest / t.tiles_r;
        int64_t off[3];
        offsets_of<3>(batch, t.n_outer, t.oshape, t.ostep, off);
        const int64_t r0 = tr * TR, c0 = tc * TC;
        if (T1 || T2) {
            const int pk = threadIdx.x % PR;                     // packet along r
            const int l0 = threadIdx.x / PR;                     // first line
            const bool r_ok = r0 + pk * V < t.R;                 // extents are whole packets: a packet is in or out
            Pack<X> xv[T1 ? NL : 1];
            Pack<Y> yv[T2 ? NL : 1];
            const char* q1 = a1 + off[0] + (r0 + pk * V) * ES + (c0 + l0) * t.cstep[0];
            const char* q2 = a2 + off[1] + (r0 + pk * V) * ES + (c0 + l0) * t.cstep[1];
            const int64_t inc1 = (int64_t)LP * t.cstep[0], inc2 = (int64_t)LP * t.cstep[1];
#pragma unroll
            for (int j = 0; j < NL; ++j) {
                const bool ok = r_ok && c0 + l0 + j * LP < t.C;
                if (T1 && ok) xv[j] = ld_pack<X>(q1 + j * inc1);
                if (T2 && ok) yv[j] = ld_pack<Y>(q2 + j * inc2);
            }
            __syncthreads();                   // the previous tile may still be read
#pragma unroll
            for (int j = 0; j < NL; ++j) {
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    if (T1) tile1[l0 + j * LP][pk * V + e] = xv[j].v[e];
                    if (T2) tile2[l0 + j * LP][pk * V + e] = yv[j].v[e];
                }
            }
            __syncthreads();
        }
        const int pc = threadIdx.x % PC;                         // packet along c
        const int lr0 = threadIdx.x / PC;                        // first row
        const bool c_ok = c0 + pc * V < t.C;
        const char* w1 = a1 + off[0] + (r0 + lr0) * t.rstep[0] + (c0 + pc * V) * (t.cstep[0] ? ES : 0);
        const char* w2 = a2 + off[1] + (r0 + lr0) * t.rstep[1] + (c0 + pc * V) * (t.cstep[1] ? ES : 0);
        char* w3 = a3 + off[2] + (r0 + lr0) * t.rstep[2] + (c0 + pc * V) * ES;
        const int64_t i1 = (int64_t)RP * t.rstep[0], i2 = (int64_t)RP * t.rstep[1], i3 = (int64_t)RP * t.rstep[2];
        Pack<X> x[NR];
        Pack<Y> y[NR];
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            const int lr = lr0 + j * RP;
            const bool ok = c_ok && r0 + lr < t.R;
#pragma unroll
            for (int e = 0; e < V; ++e) { x[j].v[e] = sx; y[j].v[e] = sy; }
            if (!ok) continue;
            if (T1) {
#pragma unroll
                for (int e = 0; e < V; ++e) x[j].v[e] = tile1[pc * V + e][lr];
            } else if (have1) {
                if (t.cstep[0]) x[j] = ld_pack<X>(w1 + j * i1);
                else { const X s = ld_one<X>(w1 + j * i1);
#pragma unroll
                       for (int e = 0; e < V; ++e) x[j].v[e] = s; }
            }
            if (T2) {
#pragma unroll
                for (int e = 0; e < V; ++e) y[j].v[e] = tile2[pc * V + e][lr];
            } else if (have2) {
                if (t.cstep[1]) y[j] = ld_pack<Y>(w2 + j * i2);
                else { const Y s = ld_one<Y>(w2 + j * i2);
#pragma unroll
                       for (int e = 0; e < V; ++e) y[j].v[e] = s; }
            }
        }
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            const int lr = lr0 + j * RP;
            if (!(c_ok && r0 + lr < t.R)) continue;
            Pack<TO> z;
            unsigned keep = 0;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                TO zv = TO();
                if (ew_apply<Op>(x[j].v[e], y[j].v[e], sx, zv, flag)) keep |= 1u << e;
                z.v[e] = zv;
            }
            char* q = w3 + j * i3;
            if (keep == (1u << V) - 1u) st_pack<TO>(q, z);
            else {
#pragma unroll
                for (int e = 0; e < V; ++e)
                    if (keep & (1u << e)) st_one<TO>(q + e * ES, z.v[e]);
            }
        }
    }
}

// Plans the tile kernel for `p`; false when the operation is not of that shape (the generic kernel takes it).
template <typename Op>
bool launch_tiled(const EwPlan& p, const char* p1, const char* p2, char* p3, bool have1, bool have2,
                  typename Op::In1 sx, typename Op::In2 sy, int use_scalar, int* flag, cudaStream_t st) {
    constexpr int64_t ES[3] = {(int64_t)sizeof(typename Op::In1), (int64_t)sizeof(typename Op::In2), (int64_t)sizeof(typename Op::Out)};
    if (p.nd < 2 || p.total < (1 << 14)) return false;
    // the output's contiguous axis becomes c (an elementwise operation may walk its dims in any order)
    int dc = -1;
    for (int d = p.nd - 1; d >= 0; --d) if (p.step[2][d] == ES[2]) { dc = d; break; }
    if (dc < 0) return false;
    // inputs: row-like (contiguous or repeated along c) or transposed (contiguous along one other axis, the same for all)
    const bool have[2] = {have1, have2};
    bool tr[2] = {false, false};
    int dr = -1;
    for (int a = 0; a < 2; ++a) {
        if (!have[a]) continue;
        if (p.step[a][dc] == ES[a] || p.step[a][dc] == 0) continue;
        int d_in = -1;
        for (int d = p.nd - 1; d >= 0; --d) if (d != dc && p.step[a][d] == ES[a]) { d_in = d; break; }
        if (d_in < 0 || (dr >= 0 && d_in != dr)) return false;
        dr = d_in;
        tr[a] = true;
    }
    if (dr < 0) return false;                                  // nothing is transposed
    if (p.shape[dr] < 16 || p.shape[dc] < 16) return false;     // slivers: not worth a tile
    constexpr bool wide = sizeof(typename Op::In1) > 4 || sizeof(typename Op::In2) > 4;
    constexpr int TC = wide ? 32 : 64;                          // the parked tiles stay within 34 KiB of shared memory
    TilePlan t;
    t.n_outer = 0;
    for (int d = 0; d < p.nd; ++d) {
        if (d == dr || d == dc) continue;
        t.oshape[t.n_outer] = p.shape[d];
        for (int a = 0; a < 3; ++a) t.ostep[a][t.n_outer] = p.step[a][d];
        ++t.n_outer;
    }
    t.R = p.shape[dr]; t.C = p.shape[dc];
    for (int a = 0; a < 3; ++a) { t.rstep[a] = p.step[a][dr]; t.cstep[a] = p.step[a][dc]; }
    t.tiles_r = (t.R + kTileR - 1) / kTileR;
    t.tiles_c = (t.C + TC - 1) / TC;
    int64_t batch = 1;
    for (int d = 0; d < t.n_outer; ++d) batch *= t.oshape[d];
    t.n_tiles = t.tiles_r * t.tiles_c * batch;
    const unsigned grid = (unsigned)(t.n_tiles > kMaxGrid ? kMaxGrid : t.n_tiles);
    // 16-byte accesses when every operand has the same element size, the plane's extents are whole packets, and every
    // line of every operand starts on a 16-byte boundary
    if constexpr (sizeof(typename Op::In1) == sizeof(typename Op::Out) && sizeof(typename Op::In2) == sizeof(typename Op::Out)) {
        constexpr int V = 16 / (int)sizeof(typename Op::Out);
        bool vec = t.R % V == 0 && t.C % V == 0 && aligned16(p3) && mult16(t.rstep[2]);
        const char* bases[2] = {p1, p2};
        for (int a = 0; a < 2 && vec; ++a) {
            if (!have[a]) continue;
            if (!aligned16(bases[a])) vec = false;
            if (tr[a]) { if (!mult16(t.cstep[a])) vec = false; }                     // lines of a transposed input
            else if (t.cstep[a] != 0 && !mult16(t.rstep[a])) vec = false;            // rows of a row-like input read by packets
        }
        for (int d = 0; d < t.n_outer && vec; ++d)
            for (int a = 0; a < 3; ++a) if ((a == 2 || have[a]) && !mult16(t.ostep[a][d])) vec = false;
        if (vec && launch_tiled_tma<Op>(t, tr, p1, p2, p3, have1, have2, sx, sy, flag, st)) return true;
        if (vec) {
            if constexpr (Op::arity == 1) {
                ew_tile_vec_kernel<Op, true, false, TC><<<grid, kBlock, 0, st>>>(t, p1, p2, p3, sx, sy, use_scalar, flag);
            } else {
                if (tr[0] && tr[1])  ew_tile_vec_kernel<Op, true, true, TC><<<grid, kBlock, 0, st>>>(t, p1, p2, p3, sx, sy, use_scalar, flag);
                else if (tr[0])      ew_tile_vec_kernel<Op, true, false, TC><<<grid, kBlock, 0, st>>>(t, p1, p2, p3, sx, sy, use_scalar, flag);
                else                 ew_tile_vec_kernel<Op, false, true, TC><<<grid, kBlock, 0, st>>>(t, p1, p2, p3, sx, sy, use_scalar, flag);
            }
            return true;
        }
    }
    if constexpr (Op::arity == 1) {
        ew_tile_kernel<Op, true, false, TC><<<grid, kBlock, 0, st>>>(t, p1, p2, p3, sx, sy, use_scalar, flag);
    } else {
        if (tr[0] && tr[1])  ew_tile_kernel<Op, true, true, TC><<<grid, kBlock, 0, st>>>(t, p1, p2, p3, sx, sy, use_scalar, flag);
        else if (tr[0])      ew_tile_kernel<Op, true, false, TC><<<grid, kBlock, 0, st>>>(t, p1, p2, p3, sx, sy, use_scalar, flag);
        else                 ew_tile_kernel<Op, false, true, TC><<<grid, kBlock, 0, st>>>(t, p1, p2, p3, sx, sy, use_scalar, flag);
    }
    return true;
}

inline unsigned grid_of(int64_t n_tiles) { return (unsigned)(n_tiles < 1 ? 1 : (n_tiles > kMaxGrid ? kMaxGrid : n_tiles)); }

// host side ---------------------------------------------------------------
template <typename Op>
void launch_elementwise(const cumo_na_iarray_t* a1, const cumo_na_iarray_t* a2, cumo_na_iarray_t* a3,
                        const cumo_na_indexer_t* ix, typename Op::In1 sx, typename Op::In2 sy,
                        int use_scalar, int* flag) {
    CB200_TRACE_LAUNCH();
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
    // a short inner dim under several outer dims pays an index split per packet;
    // the generic kernel is the better plan there
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
            const int64_t L = p.shape[in];
            // whole packets only: a ragged inner extent takes the scalar form, except for a flat
            // array, whose few trailing elements get a launch of their own
            int64_t tail = 0;
            if (vec && L % VMAX != 0) {
                if (p.nd == 1 && L > VMAX) tail = L % VMAX; else vec = false;
            }
            if (p.nd > 2 && !vec) row_ok = false;      // the split-index form exists for 16-byte packets only
            int launches = 0;
            auto run = [&](bool v16, int64_t len, const char* q1, const char* q2, char* q3) {
                const int V = v16 ? VMAX : 1;
                RowGeom g;
                g.L = len;
                g.R = p.total / L;
                const int64_t vpr = (len + V - 1) / V;
                g.inner[0] = have1 && p.step[0][in] != 0;
                g.inner[1] = have2 && p.step[1][in] != 0;
                for (int a = 0; a < 3; ++a) g.rs[a] = p.nd == 2 ? p.step[a][0] : 0;
                // a row vector repeated down the rows is worth holding in registers
                const bool shared_row = p.nd == 2 && ((g.inner[0] == 1 && g.rs[0] == 0) || (g.inner[1] == 1 && g.rs[1] == 0));
                // ... and so is one element per row against a full array, (R,C) o (R,1): the per-row value is fetched once per CTA
                const bool row_scalar = p.nd == 2 && have1 && have2 && ((g.inner[0] == 0 && g.inner[1] == 1) || (g.inner[0] == 1 && g.inner[1] == 0));
                if constexpr (Op::arity == 2)
                if (v16 && (shared_row || row_scalar) && vpr >= kBlock && g.R >= 2 * kShareRows && len * ES <= 0xffffffffLL) {
                    const int64_t chunks = (vpr + kEwSlots - 1) / kEwSlots;
                    g.rows_per_tile = 1;
                    g.chunks_per_row = (uint32_t)chunks;
                    g.vpr = kEwSlots;
                    g.n_tiles = (g.R + kShareRows - 1) / kShareRows * chunks;
                    // mode of each input: held (shared row vector, or the scalar argument: null pointer), one element per row, a packet per row
                    const int m1 = !have1 || (g.inner[0] == 1 && g.rs[0] == 0) ? kHeld : g.inner[0] == 0 ? kRowScalar : kRowPack;
                    const int m2 = !have2 || (g.inner[1] == 1 && g.rs[1] == 0) ? kHeld : g.inner[1] == 0 ? kRowScalar : kRowPack;
                    const unsigned grid = grid_of(g.n_tiles);
                    const char* h1 = have1 ? q1 : nullptr;
                    const char* h2 = have2 ? q2 : nullptr;
                    bool done = true;
                    if (m1 == kHeld && m2 == kHeld)           ew_rowshare_kernel<Op, VMAX, kHeld, kHeld><<<grid, kBlock, 0, st>>>(g, h1, h2, q3, sx, sy, flag);
                    else if (m1 == kHeld && m2 == kRowScalar) ew_rowshare_kernel<Op, VMAX, kHeld, kRowScalar><<<grid, kBlock, 0, st>>>(g, h1, h2, q3, sx, sy, flag);
                    else if (m1 == kRowScalar && m2 == kHeld) ew_rowshare_kernel<Op, VMAX, kRowScalar, kHeld><<<grid, kBlock, 0, st>>>(g, h1, h2, q3, sx, sy, flag);
                    else if (m1 == kRowPack && m2 == kRowScalar) ew_rowshare_kernel<Op, VMAX, kRowPack, kRowScalar><<<grid, kBlock, 0, st>>>(g, h1, h2, q3, sx, sy, flag);
                    else if (m1 == kRowScalar && m2 == kRowPack) ew_rowshare_kernel<Op, VMAX, kRowScalar, kRowPack><<<grid, kBlock, 0, st>>>(g, h1, h2, q3, sx, sy, flag);
                    else done = false;        // a full array against a row vector: the plain row kernel measures faster (fewer registers)
                    if (done) { ++launches; return true; }
                }
                if (vpr >= kEwSlots) {
                    g.rows_per_tile = 1;
                    const int64_t chunks = (vpr + kEwSlots - 1) / kEwSlots;
                    if (chunks > 0xffffffffLL) return false;
                    g.chunks_per_row = (uint32_t)chunks;
                    g.vpr = kEwSlots;
                    g.n_tiles = g.R * chunks;
                } else {
                    g.vpr = (uint32_t)vpr;
                    g.rows_per_tile = (uint32_t)(kEwSlots / vpr);
                    g.chunks_per_row = 1;
                    g.n_tiles = (g.R + g.rows_per_tile - 1) / g.rows_per_tile;
                }
                const unsigned grid = grid_of(g.n_tiles);
                if (p.nd > 2) ew_row_kernel<Op, VMAX, true><<<grid, kBlock, 0, st>>>(p, g, q1, q2, q3, sx, sy, use_scalar, flag);
                else if (v16) ew_row_kernel<Op, VMAX, false><<<grid, kBlock, 0, st>>>(p, g, q1, q2, q3, sx, sy, use_scalar, flag);
                else          ew_row_kernel<Op, 1, false><<<grid, kBlock, 0, st>>>(p, g, q1, q2, q3, sx, sy, use_scalar, flag);
                ++launches;
                return true;
            };
            // the row kernels address a slot's column with 32 bits: an inner extent beyond that goes in slices
            // (a multiple of every packet size, so each slice keeps the alignment of the whole)
            constexpr int64_t kMaxInner = 1LL << 31;
            auto run_sliced = [&](bool v16, int64_t len, const char* q1, const char* q2, char* q3) {
                for (int64_t done = 0; done < len; done += kMaxInner) {
                    const int64_t part = len - done < kMaxInner ? len - done : kMaxInner;
                    if (!run(v16, part, q1 ? q1 + done * p.step[0][in] : q1, q2 ? q2 + done * p.step[1][in] : q2, q3 + done * ES)) return false;
                }
                return true;
            };
            if (row_ok && run_sliced(vec, L - tail, p1, p2, p3)) {
                if (tail) {
                    const int64_t done = L - tail;
                    run(false, tail, p1 ? p1 + done * p.step[0][in] : p1, p2 ? p2 + done * p.step[1][in] : p2, p3 + done * ES);
                }
                count_launch(launches);
                cumo_cuda_runtime_check_kernel_launch();
                return;
            }
        }
    }
    if (launch_tiled<Op>(p, p1, p2, p3, have1, have2, sx, sy, use_scalar, flag, st)) {
        count_launch();
        cumo_cuda_runtime_check_kernel_launch();
        return;
    }
    int64_t n_tiles = (p.total + kEwSlots - 1) / kEwSlots;
    ew_gen_kernel<Op><<<grid_of(n_tiles), kBlock, 0, st>>>(p, n_tiles, p1, p2, p3, sx, sy, use_scalar, flag);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

// ----------------------------------------------------------------------------
// Comparisons -> Bit
// ----------------------------------------------------------------------------
// Flat kernel: inputs contiguous (or broadcast scalars), Bit output contiguous
// and starting on a word boundary.  Each lane tests V consecutive elements;
// the 32/V lanes that share an output word OR their bit groups together.
// Whole-tile kernel for the flat case: each lane loads one element per step, so a warp's
// ballot IS the output word (no bit assembly across lanes); lane j keeps the word of step j
// and the first U lanes store the warp's U words together.  Array-or-scalar is a template
// argument so the loop carries no tests.  Elements past the last whole tile go to
// cmp_flat_kernel below.
template <typename T> constexpr int cmp_steps() { return 64 / (int)sizeof(T); }     // 16 (4-byte) or 8 (8-byte) loads in flight per thread

template <typename Op, bool A1, bool A2>
__global__ void __launch_bounds__(kBlock)
cmp_full_kernel(const typename Op::In1* __restrict__ a1, const typename Op::In2* __restrict__ a2, uint32_t* out,
                typename Op::In1 sx, typename Op::In2 sy) {
    using T1 = typename Op::In1;
    using T2 = typename Op::In2;
    constexpr int U = cmp_steps<T1>();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t first = ((size_t)blockIdx.x * (kBlock / 32) + warp) * (32 * U) + lane;
    T1 x[U];
    T2 y[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        x[j] = A1 ? ld_one<T1>(a1 + first + j * 32) : sx;
        y[j] = A2 ? ld_one<T2>(a2 + first + j * 32) : sy;
    }
    uint32_t mine = 0;
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const uint32_t w = __ballot_sync(0xffffffffu, Op::test(x[j], y[j]));
        if (lane == j) mine = w;
    }
    if (lane < U) out[((size_t)blockIdx.x * (kBlock / 32) + warp) * U + lane] = mine;
}

template <typename Op, int V>
__global__ void __launch_bounds__(kBlock)
cmp_flat_kernel(int64_t total, int64_t n_tiles, const char* __restrict__ a1, const char* __restrict__ a2,
                uint32_t* out, int st1, int st2, typename Op::In1 sx, typename Op::In2 sy, int use_scalar) {
    using T1 = typename Op::In1;
    using T2 = typename Op::In2;
    constexpr int ES = sizeof(T1);
    constexpr int LPW = 32 / V;               // lanes per output word
    constexpr int U = kEwUnroll;
    const bool have1 = use_scalar != 2 && st1 != 0;
    const bool have2 = Op::arity == 2 && use_scalar != 1 && st2 != 0;
    // a one-element (broadcast) array operand behaves like a scalar: read it once
    if (use_scalar != 2 && st1 == 0) sx = ld_one<T1>(a1);
    if (Op::arity == 2 && use_scalar != 1 && st2 == 0) sy = ld_one<T2>(a2);
    const int lane = threadIdx.x & 31;
    unsigned group_mask = 0xffffffffu;
    if (LPW < 32) group_mask = ((1u << (LPW & 31)) - 1u) << (lane / LPW * LPW);
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        Pack<T1> x[U];
        Pack<T2> y[U];
        int64_t e0[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            e0[j] = (tile * kEwSlots + j * kBlock + threadIdx.x) * (int64_t)V;
            const int64_t left = total - e0[j];
#pragma unroll
            for (int e = 0; e < V; ++e) { x[j].v[e] = sx; y[j].v[e] = sy; }
            if (left >= V) {
                if (have1) { if (V > 1) x[j] = ld_pack<T1>(a1 + e0[j] * ES); else x[j].v[0] = ld_one<T1>(a1 + e0[j] * ES); }
                if (have2) { if (V > 1) y[j] = ld_pack<T2>(a2 + e0[j] * ES); else y[j].v[0] = ld_one<T2>(a2 + e0[j] * ES); }
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    if (have1 && e < left) x[j].v[e] = ld_one<T1>(a1 + (e0[j] + e) * ES);
                    if (have2 && e < left) y[j].v[e] = ld_one<T2>(a2 + (e0[j] + e) * ES);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int64_t left = total - e0[j];
            uint32_t bits = 0;
#pragma unroll
            for (int e = 0; e < V; ++e)
                bits |= (Op::test(x[j].v[e], y[j].v[e]) ? 1u : 0u) << e;
            if (left < V) bits &= left > 0 ? (1u << left) - 1u : 0u;     // elements past the end
            bits <<= (lane % LPW) * V;
            const uint32_t word = LPW == 32 ? __ballot_sync(0xffffffffu, bits != 0) : __reduce_or_sync(group_mask, bits);
            if (lane % LPW == 0 && left > 0) {
                const int64_t w = e0[j] >> 5;
                if (left >= 32) out[w] = word;
                else {                         // last, partial word: keep the bits past the end
                    const uint32_t m = (1u << left) - 1u;
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
        for (int j = 0; j < kEwUnroll; ++j) {
            int64_t i = tile * kEwSlots + j * kBlock + threadIdx.x;
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
    CB200_TRACE_LAUNCH();
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
        int launches = 0;
        // whole tiles: every operand is an array that steps or a scalar argument (a one-element
        // array that is broadcast has its value on the device and stays with the kernel below)
        constexpr int64_t kTile = (int64_t)kBlock * cmp_steps<T1>();
        const int64_t full = p.total / kTile;
        int64_t done = 0;
        if (full > 0 && full <= kMaxGrid && (st1 || st2) && (st1 || !have1) && (st2 || !have2)) {
            using T2 = typename Op::In2;
            const T1* q1 = reinterpret_cast<const T1*>(p1);
            const T2* q2 = reinterpret_cast<const T2*>(p2);
            if (st1 && st2)  cmp_full_kernel<Op, true, true><<<(unsigned)full, kBlock, 0, st>>>(q1, q2, out, sx, sy);
            else if (st1)    cmp_full_kernel<Op, true, false><<<(unsigned)full, kBlock, 0, st>>>(q1, q2, out, sx, sy);
            else             cmp_full_kernel<Op, false, true><<<(unsigned)full, kBlock, 0, st>>>(q1, q2, out, sx, sy);
            ++launches;
            done = full * kTile;
        }
        if (done < p.total) {
            const int64_t rest = p.total - done;
            const char* r1 = st1 ? p1 + done * ES : p1;
            const char* r2 = st2 ? p2 + done * ES : p2;
            uint32_t* ro = out + (done >> 5);
            bool vec = (!st1 || aligned16(r1)) && (!st2 || aligned16(r2));
            if (vec) {
                int64_t n_tiles = (rest + (int64_t)kEwSlots * VMAX - 1) / ((int64_t)kEwSlots * VMAX);
                cmp_flat_kernel<Op, VMAX><<<grid_of(n_tiles), kBlock, 0, st>>>(rest, n_tiles, r1, r2, ro, st1, st2, sx, sy, use_scalar);
            } else {
                int64_t n_tiles = (rest + kEwSlots - 1) / kEwSlots;
                cmp_flat_kernel<Op, 1><<<grid_of(n_tiles), kBlock, 0, st>>>(rest, n_tiles, r1, r2, ro, st1, st2, sx, sy, use_scalar);
            }
            ++launches;
        }
        count_launch(launches);
        cumo_cuda_runtime_check_kernel_launch();
        return;
    } else {
        // is the output still one run of bits in logical order?
        bool word_store = (a3->pos & 31) == 0;
        int64_t run = 1;
        for (int d = p.nd - 1; d >= 0 && word_store; --d) {
            if (p.step[2][d] != run) word_store = false;
            run *= p.shape[d];
        }
        int64_t n_tiles = (p.total + kEwSlots - 1) / kEwSlots;
        cmp_gen_kernel<Op><<<grid_of(n_tiles), kBlock, 0, st>>>(p, n_tiles, p1, p2, a3->ptr, (uint64_t)a3->pos, word_store ? 1 : 0, sx, sy, use_scalar);
    }
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200
