// Reduction engine: axis and full reductions over a cumo_na_reduction_arg_t.
//
// Stands where the reference's CuPy-style engine stands
// (ext/cumo/include/cumo/reduce_kernel.h:250-611: one 512-thread block per
// output, shared-memory tree, scalar loads, a split into at most 1024 chunks
// only when fewer than 256 blocks would run).  Plan here:
//
//   ROW  the reduce axes collapse to one contiguous run (step == element size).
//        A "group" (a warp for short rows, a whole CTA for long ones) owns one
//        (output, segment) item and streams it with 16-byte loads, 4 packets in
//        flight per thread.  A long row is cut into fixed 32 KiB segments, one CTA
//        each, consecutive CTAs on consecutive segments: B200 streams fastest with
//        very many small CTAs marching through memory together.
//   COL  the innermost OUTPUT axis is the contiguous one (a column / "transposed"
//        reduction).  A CTA owns a strip of 32 lanes x 16 bytes of columns and a
//        segment of 256 rows; its 8 warps walk different rows with 16-byte loads
//        and keep one accumulator per column in registers.
//   GEN  any other stride pattern: a group per (output, segment), offsets from a
//        32-bit index split.
//   Segmented plans write accumulators to scratch ([output][segment]) and a
//   second launch folds the segments of each output in index order, so a result
//   depends only on shape and strides, never on scheduling or on the device.
//
// Index reductions get, per element, either its position along the reduce axes
// or its element offset from arg->in.ptr (reduce_kernel.h:219-239).
#pragma once

#include "common.cuh"
#include "reducers.cuh"

namespace cb200 {

struct RedPlan {
    int n_od, n_rd;                       // canonical out dims / reduce dims (each >= 1)
    int64_t n_out, n_red;
    int64_t oshape[kMaxDim], in_ostep[kMaxDim], out_step[kMaxDim], out2_step[kMaxDim];
    int64_t rshape[kMaxDim], in_rstep[kMaxDim];
};

// arg->in carries the reduce dims last (ndloop transposed them there); dims of
// extent 1 are dropped and neighbours that one stride covers are merged, out and
// reduce groups separately.
inline bool make_red_plan(RedPlan* p, const cumo_na_reduction_arg_t* arg, const cumo_na_iarray_t* out2) {
    const int in_nd = arg->in_indexer.ndim;
    const int out_nd = arg->out_indexer.ndim;
    p->n_od = p->n_rd = 0;
    p->n_out = p->n_red = 1;
    for (int d = 0; d < out_nd; ++d) {
        int64_t n = (int64_t)arg->out_indexer.shape[d];
        if (n == 0) return false;
        p->n_out *= n;
        if (n == 1) continue;
        int64_t si = arg->in.step[d], so = arg->out.step[d], s2 = out2 ? (int64_t)out2->step[d] : 0;
        int k = p->n_od;
        if (k > 0 && p->in_ostep[k - 1] == si * n && p->out_step[k - 1] == so * n && p->out2_step[k - 1] == s2 * n) {
            p->oshape[k - 1] *= n; p->in_ostep[k - 1] = si; p->out_step[k - 1] = so; p->out2_step[k - 1] = s2;
        } else {
            p->oshape[k] = n; p->in_ostep[k] = si; p->out_step[k] = so; p->out2_step[k] = s2;
            ++p->n_od;
        }
    }
    for (int d = out_nd; d < in_nd; ++d) {
        int64_t n = (int64_t)arg->in_indexer.shape[d];
        p->n_red *= n;
        if (n == 1) continue;
        int64_t si = arg->in.step[d];
        int k = p->n_rd;
        if (k > 0 && p->in_rstep[k - 1] == si * n) { p->rshape[k - 1] *= n; p->in_rstep[k - 1] = si; }
        else { p->rshape[k] = n; p->in_rstep[k] = si; ++p->n_rd; }
    }
    if (p->n_od == 0) { p->n_od = 1; p->oshape[0] = 1; p->in_ostep[0] = p->out_step[0] = p->out2_step[0] = 0; }
    if (p->n_rd == 0) { p->n_rd = 1; p->rshape[0] = p->n_red ? 1 : 0; p->in_rstep[0] = 0; }
    return true;
}

// ---- moving accumulators between lanes ------------------------------------------------
template <typename A>
__device__ __forceinline__ A shfl_down_acc(A v, int delta) {
    constexpr int W = (sizeof(A) + 3) / 4;
    union { A a; uint32_t w[W]; } u;
    u.a = v;
#pragma unroll
    for (int i = 0; i < W; ++i) u.w[i] = __shfl_down_sync(0xffffffffu, u.w[i], delta);
    return u.a;
}

// Index reductions on 4-byte element types: the warp's extreme value by one integer reduce instruction on an
// order-preserving key, then the lowest index among the lanes that hold it by a second one -- instead of five rounds
// of 16-byte shuffles and comparisons.  Same total order as R::combine (NaN rule, better value, lower index).
template <typename R, typename = void> struct redux_fold : std::false_type {};
template <typename R> struct redux_fold<R, std::void_t<decltype(R::kReduxFold)>> : std::integral_constant<bool, R::kReduxFold> {};

template <typename R>
__device__ __forceinline__ typename R::Acc warp_fold_redux(const R& r, typename R::Acc a) {
    const uint32_t key = r.order_key(a.value);                       // larger key = better; the losing NaN class maps to 0
    const uint32_t best = __reduce_max_sync(0xffffffffu, key);
    // indices of one warp's accumulators are distinct (or INT64_MAX for identities), so the minimum picks one lane;
    // the sign bit is flipped so that the unsigned minimum follows the signed order
    constexpr unsigned long long kBias = 0x8000000000000000ull;
    const unsigned long long mine = key == best ? ((unsigned long long)a.index ^ kBias) : ~0ull;
    const uint32_t lo = __reduce_min_sync(0xffffffffu, (uint32_t)(mine >> 32));
    const uint32_t lo2 = __reduce_min_sync(0xffffffffu, (uint32_t)(mine >> 32) == lo ? (uint32_t)mine : 0xffffffffu);
    const unsigned long long win = ((unsigned long long)lo << 32) | lo2;
    const unsigned holder = __ballot_sync(0xffffffffu, mine == win);
    const int src = __ffs(holder) - 1;
    typename R::Acc out;
    out.value = __shfl_sync(0xffffffffu, a.value, src);
    out.index = (int64_t)(win ^ kBias);
    return out;
}

template <typename R>
__device__ __forceinline__ typename R::Acc warp_fold(const R& r, typename R::Acc a) {
    if constexpr (redux_fold<R>::value) return warp_fold_redux(r, a);
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {      // lane i folds in lane i+d: earlier positions stay on the left
        typename R::Acc b = shfl_down_acc(a, d);
        a = r.combine(a, b);
    }
    return a;                                // lane 0 holds the warp's result
}

// Result valid in thread 0 of the group.  G < 32: G neighbouring lanes of a warp; G == 32: a warp; G == kBlock: the CTA.
template <typename R, int G>
__device__ __forceinline__ typename R::Acc group_fold(const R& r, typename R::Acc a, typename R::Acc* smem) {
    if constexpr (G < 32) {
        // lane i folds in lane i+d for d < G: the first lane of a group only ever reaches lanes of its own group
#pragma unroll
        for (int d = 1; d < G; d <<= 1) {
            typename R::Acc b = shfl_down_acc(a, d);
            a = r.combine(a, b);
        }
        return a;
    }
    a = warp_fold(r, a);
    if (G == 32) return a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                         // smem may still be read from the previous item
    if (lane == 0) smem[warp] = a;
    __syncthreads();
    if (threadIdx.x == 0) {
        a = smem[0];
#pragma unroll
        for (int w = 1; w < kWarpsPerBlock; ++w) a = r.combine(a, smem[w]);
    }
    return a;
}

// A thread's private accumulation over the elements it visits, addressed by a 32-bit
// position inside the thread's segment; `idx_of(pos)` turns a position into the index
// the functor wants and is only evaluated when it is needed.  Reducers with a private
// scan (the index reductions) use it when positions are visited in increasing index
// order; everything else folds combine(map()).
template <typename R, bool SCAN>
struct Runner;
template <typename R>
struct Runner<R, false> {
    typename R::Acc a;
    __device__ __forceinline__ void init(const R& r) { a = r.identity(); }
    template <typename F>
    __device__ __forceinline__ void step(const R& r, typename R::In v, int32_t pos, F idx_of) {
        a = r.combine(a, r.map(v, R::kIndexed ? idx_of(pos) : (int64_t)0));
    }
    __device__ __forceinline__ void merge(const R& r, const Runner& o) { a = r.combine(a, o.a); }
    __device__ __forceinline__ void settle(int32_t) {}
    template <typename F>
    __device__ __forceinline__ typename R::Acc finish(const R&, F) { return a; }
};
template <typename R>
struct Runner<R, true> {
    typename R::Local l;
    __device__ __forceinline__ void init(const R& r) { l = r.local_identity(); }
    template <typename F>
    __device__ __forceinline__ void step(const R& r, typename R::In v, int32_t pos, F) { r.local_scan(l, v, pos); }
    __device__ __forceinline__ void merge(const R& r, const Runner& o) { r.local_merge(l, o.l); }
    // first: the first position this scan visited, negative if it visited nothing
    __device__ __forceinline__ void settle(int32_t first) { if (l.pos < 0 && first >= 0) l.pos = first; }
    template <typename F>
    __device__ __forceinline__ typename R::Acc finish(const R& r, F idx_of) {
        if (l.pos < 0) return r.identity();
        return typename R::Acc{l.value, idx_of(l.pos)};
    }
};

template <typename R>
__device__ __forceinline__ void emit(const R& r, const RedPlan& p, int64_t o, int n_split, int64_t s,
                                     typename R::Acc a, char* out, char* out2, typename R::Acc* partial) {
    if (n_split > 1) { partial[o * n_split + s] = a; return; }
    int64_t oo = offset_of(o, p.n_od, p.oshape, p.out_step);
    int64_t o2 = out2 ? offset_of(o, p.n_od, p.oshape, p.out2_step) : 0;
    r.store(out + oo, out2 ? out2 + o2 : nullptr, a);
}

// what every first-pass kernel is told besides the plan
struct RedLaunch {
    int64_t seg_len;       // elements (ROW/GEN) or rows (COL) per segment
    int64_t n_strips;      // COL only
    int n_split;
    int flat_index;        // 1: feed the element offset; 0: the position along the reduce axes
    int ordered;           // indices grow with the position inside a segment
};

// ---- ROW ------------------------------------------------------------------------------
// one (output, segment) item reduced by a group of G threads; returns the group's result in its thread 0
template <typename R, int V, int G, bool SCAN>
__device__ __forceinline__ typename R::Acc row_item(const R& r, const char* base, int64_t begin, int64_t end,
                                                    int64_t idx_base, int gl, typename R::Acc* smem) {
    using T = typename R::In;
    constexpr int ES = sizeof(T);
    // a scan spends longer on each packet than a sum does, so it keeps twice as many loads in flight
    constexpr int UN = SCAN ? 2 * kUnroll : kUnroll;
    constexpr int64_t SPAN = (int64_t)G * V * UN;          // elements per group iteration
    // a private scan is a chain of dependent compares: one chain per packet lane keeps V of them in flight
    constexpr int NR = SCAN ? V : 1;
    Runner<R, SCAN> run[NR];
#pragma unroll
    for (int k = 0; k < NR; ++k) run[k].init(r);
    auto idx_of = [&](int32_t pos) { return idx_base + begin + pos; };
    int64_t eb = begin;
    // whole iterations: every packet of every lane lies inside the segment, no tests per element
    for (; eb + SPAN <= end; eb += SPAN) {
        Pack<T> v[UN];
#pragma unroll
        for (int j = 0; j < UN; ++j) {
            const char* q = base + (eb + (int64_t)(j * G + gl) * V) * ES;
            if (V > 1) v[j] = ld_pack<T>(q); else v[j].v[0] = ld_one<T>(q);
        }
        const int32_t p0 = (int32_t)(eb - begin);
#pragma unroll
        for (int j = 0; j < UN; ++j)
#pragma unroll
            for (int k = 0; k < V; ++k) run[SCAN ? k : 0].step(r, v[j].v[k], p0 + (j * G + gl) * V + k, idx_of);
    }
    // the ragged end of the segment: its whole packets, strided over the group (four loads issued
    // before the first use while four remain), then the few elements past the last whole packet
    if (eb < end) {
        const char* rb = base + eb * ES;
        const int32_t p0 = (int32_t)(eb - begin);
        const int32_t n_pk = (int32_t)((end - eb) / V);            // < UN * G
        int32_t pk = gl;
        for (; pk + 3 * G < n_pk; pk += 4 * G) {
            Pack<T> v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const char* q = rb + (int64_t)(pk + j * G) * (V * ES);
                if (V > 1) v[j] = ld_pack<T>(q); else v[j].v[0] = ld_one<T>(q);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int k = 0; k < V; ++k) run[SCAN ? k : 0].step(r, v[j].v[k], p0 + (pk + j * G) * V + k, idx_of);
        }
        for (; pk < n_pk; pk += G) {
            Pack<T> v;
            const char* q = rb + (int64_t)pk * (V * ES);
            if (V > 1) v = ld_pack<T>(q); else v.v[0] = ld_one<T>(q);
#pragma unroll
            for (int k = 0; k < V; ++k) run[SCAN ? k : 0].step(r, v.v[k], p0 + pk * V + k, idx_of);
        }
        if (V > 1 && gl == 0) {                                    // thread 0's positions stay in rising order
            const int32_t rest = (int32_t)(end - eb) - n_pk * V;
#pragma unroll
            for (int k = 0; k < V; ++k)
                if (k < rest) run[SCAN ? k : 0].step(r, ld_one<T>(rb + (int64_t)(n_pk * V + k) * ES), p0 + n_pk * V + k, idx_of);
        }
    }
#pragma unroll
    for (int k = 0; k < NR; ++k) run[k].settle(begin + gl * V + k < end ? gl * V + k : -1);
#pragma unroll
    for (int k = 1; k < NR; ++k) run[0].merge(r, run[k]);
    return group_fold<R, G>(r, run[0].finish(r, idx_of), smem);
}

template <typename R, int V, int G>
__global__ void __launch_bounds__(kBlock)
red_row_kernel(const RedPlan p, const R r, const RedLaunch q, const char* __restrict__ in, char* out, char* out2,
               typename R::Acc* partial) {
    using T = typename R::In;
    using Acc = typename R::Acc;
    constexpr int ES = sizeof(T);
    constexpr int GPB = kBlock / G;          // groups per CTA
    pdl_trigger();                           // a second (folding) pass may be launched while this one runs
    __shared__ Acc smem[kWarpsPerBlock];
    const int gid = threadIdx.x / G, gl = threadIdx.x % G;
    const int64_t L = p.n_red;
    const int64_t items = p.n_out * q.n_split;
    for (int64_t item0 = (int64_t)blockIdx.x * GPB; item0 < items; item0 += (int64_t)gridDim.x * GPB) {
        int64_t item = item0 + gid;
        const bool live = item < items;      // whole groups go idle together; G==kBlock: always live
        if (!live) item = items - 1;         // idle groups of the last CTA redo the last item and drop it
        int64_t o, s;
        if (item <= 0xffffffffLL) { uint32_t oo = (uint32_t)item / (uint32_t)q.n_split; o = oo; s = (uint32_t)item - oo * (uint32_t)q.n_split; }
        else { o = item / q.n_split; s = item - o * q.n_split; }
        const int64_t in_off = offset_of(o, p.n_od, p.oshape, p.in_ostep);
        const int64_t begin = s * q.seg_len;
        int64_t end = begin + q.seg_len; if (end > L) end = L;
        const int64_t idx_base = q.flat_index ? in_off / ES : 0;
        Acc acc = row_item<R, V, G, R::kHasScan>(r, in + in_off, begin, end, idx_base, gl, smem);
        if (live && gl == 0) emit(r, p, o, q.n_split, s, acc, out, out2, partial);
    }
}

// ---- COL ------------------------------------------------------------------------------
template <typename R, int V, bool SCAN>
__device__ __forceinline__ void col_item(const R& r, const RedPlan& p, const RedLaunch& q, const char* base, int64_t in_b,
                                         int64_t col0, int nv, int64_t r_begin, int64_t r_end, int warp,
                                         typename R::Acc* acc_out) {
    using T = typename R::In;
    constexpr int ES = sizeof(T);
    Runner<R, SCAN> run[V];
#pragma unroll
    for (int k = 0; k < V; ++k) run[k].init(r);
    auto row_off = [&](int64_t row) { return row * p.in_rstep[0]; };
    int64_t r0 = r_begin + warp;
    if (nv == V) {
        // whole iterations: four rows of this warp inside the segment, whole packets
        for (; r0 + (kUnroll - 1) * kWarpsPerBlock < r_end; r0 += kWarpsPerBlock * kUnroll) {
            Pack<T> v[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const char* a = base + row_off(r0 + j * kWarpsPerBlock);
                if (V > 1) v[j] = ld_pack<T>(a); else v[j].v[0] = ld_one<T>(a);
            }
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int32_t pos = (int32_t)(r0 + j * kWarpsPerBlock - r_begin);
#pragma unroll
                for (int k = 0; k < V; ++k)
                    run[k].step(r, v[j].v[k], pos, [&](int32_t ps) {
                        const int64_t row = r_begin + ps;
                        return q.flat_index ? (in_b + row_off(row)) / ES + col0 + k : row; });
            }
        }
    }
    for (; r0 < r_end; r0 += kWarpsPerBlock) {
        const char* a = base + row_off(r0);
        const int32_t pos = (int32_t)(r0 - r_begin);
#pragma unroll
        for (int k = 0; k < V; ++k)
            if (k < nv)
                run[k].step(r, ld_one<T>(a + k * ES), pos, [&](int32_t ps) {
                    const int64_t row = r_begin + ps;
                    return q.flat_index ? (in_b + row_off(row)) / ES + col0 + k : row; });
    }
#pragma unroll
    for (int k = 0; k < V; ++k) run[k].settle(k < nv && r_begin + warp < r_end ? warp : -1);
#pragma unroll
    for (int k = 0; k < V; ++k)
        acc_out[k] = run[k].finish(r, [&](int32_t ps) {
            const int64_t row = r_begin + ps;
            return q.flat_index ? (in_b + row_off(row)) / ES + col0 + k : row; });
}

template <typename R, int V>
__global__ void __launch_bounds__(kBlock)
red_col_kernel(const RedPlan p, const R r, const RedLaunch q, const char* __restrict__ in, char* out, char* out2,
               typename R::Acc* partial) {
    using T = typename R::In;
    using Acc = typename R::Acc;
    constexpr int ES = sizeof(T);
    constexpr int W = 32 * V;                // columns per strip
    pdl_trigger();                           // a second (folding) pass may be launched while this one runs
    __shared__ Acc smem[kWarpsPerBlock][W];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int od_in = p.n_od - 1;            // innermost out dim = the columns
    const int64_t C = p.oshape[od_in];
    const int64_t n_batch = p.n_out / C;
    const int64_t items = n_batch * q.n_strips * q.n_split;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        // strips vary fastest: neighbouring CTAs read neighbouring columns of the same rows
        int64_t strip, s, b;
        if (item <= 0xffffffffLL) {
            uint32_t it = (uint32_t)item, t = it / (uint32_t)q.n_strips;
            strip = it - t * (uint32_t)q.n_strips;
            uint32_t bb = t / (uint32_t)q.n_split;
            s = t - bb * (uint32_t)q.n_split; b = bb;
        } else {
            strip = item % q.n_strips;
            const int64_t t = item / q.n_strips;
            s = t % q.n_split; b = t / q.n_split;
        }
        const int64_t col0 = strip * W + (int64_t)lane * V;
        const int64_t cleft = C - col0;
        const int nv = cleft >= V ? V : (cleft > 0 ? (int)cleft : 0);
        const int64_t in_b = offset_of(b, od_in, p.oshape, p.in_ostep);
        const int64_t r_begin = s * q.seg_len;
        int64_t r_end = r_begin + q.seg_len; if (r_end > p.n_red) r_end = p.n_red;
        Acc acc[V];
        if (nv > 0) {
            const char* base = in + in_b + col0 * ES;
            col_item<R, V, R::kHasScan>(r, p, q, base, in_b, col0, nv, r_begin, r_end, warp, acc);
        } else {
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] = r.identity();
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < V; ++k) smem[warp][lane * V + k] = acc[k];
        __syncthreads();
        if (warp == 0 && nv > 0) {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                if (k >= nv) break;
                Acc a = smem[0][lane * V + k];
#pragma unroll
                for (int w = 1; w < kWarpsPerBlock; ++w) a = r.combine(a, smem[w][lane * V + k]);
                emit(r, p, b * C + col0 + k, q.n_split, s, a, out, out2, partial);
            }
        }
    }
}

// ---- COL, wide rows ---------------------------------------------------------------------
// When a row of output columns is at least half a CTA's width of packets, every thread owns
// V columns outright: the CTA reads kBlock contiguous packets of each row (4 KiB), walks its rows
// with kColUnroll loads in flight per thread, and nothing is folded across threads at all.
// The rows are dealt to the n_split segments in blocks of kColUnroll, round robin: segment s takes
// row blocks s, s + n_split, s + 2 n_split, ...  So at any moment the resident CTAs read one compact
// window of the array that slides through memory (B200 streams measurably faster that way than with
// every CTA walking a far-apart region of its own), and all segments are equally long to within one block.
constexpr int kColUnroll = 8;

template <typename R, int V>
__global__ void __launch_bounds__(kBlock, 4)
red_colwide_kernel(const RedPlan p, const R r, const RedLaunch q, const char* __restrict__ in, char* out, char* out2,
                   typename R::Acc* partial) {
    using T = typename R::In;
    constexpr int ES = sizeof(T);
    constexpr int W = kBlock * V;            // columns per strip
    constexpr int U = kColUnroll;
    pdl_trigger();                           // a second (folding) pass may be launched while this one runs
    const int od_in = p.n_od - 1;            // innermost out dim = the columns
    const int64_t C = p.oshape[od_in];
    const int64_t n_batch = p.n_out / C;
    const int64_t items = n_batch * q.n_strips * q.n_split;
    const int64_t rstep = p.in_rstep[0];
    const int64_t n_rows = p.n_red;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        // strips vary fastest: neighbouring CTAs read neighbouring columns of the same rows
        int64_t strip, s, b;
        if (item <= 0xffffffffLL) {
            uint32_t it = (uint32_t)item, t = it / (uint32_t)q.n_strips;
            strip = it - t * (uint32_t)q.n_strips;
            uint32_t bb = t / (uint32_t)q.n_split;
            s = t - bb * (uint32_t)q.n_split; b = bb;
        } else {
            strip = item % q.n_strips;
            const int64_t t = item / q.n_strips;
            s = t % q.n_split; b = t / q.n_split;
        }
        const int64_t col0 = strip * W + (int64_t)threadIdx.x * V;
        const int64_t cleft = C - col0;
        const int nv = cleft >= V ? V : (cleft > 0 ? (int)cleft : 0);
        if (nv == 0) continue;
        const int64_t in_b = offset_of(b, od_in, p.oshape, p.in_ostep);
        const char* base = in + in_b + col0 * ES;
        Runner<R, R::kHasScan> run[V];
#pragma unroll
        for (int k = 0; k < V; ++k) run[k].init(r);
        // positions are row numbers (the host keeps the row count of this plan below 2^31)
        auto idx_of = [&](int32_t row, int k) {
            return q.flat_index ? (in_b + (int64_t)row * rstep) / ES + col0 + k : (int64_t)row;
        };
        const int64_t first = s * U;
        for (int64_t rb = first; rb < n_rows; rb += (int64_t)q.n_split * U) {
            const char* a0 = base + rb * rstep;
            if (nv == V && rb + U <= n_rows) {
                Pack<T> v[U];
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    const char* a = a0 + (int64_t)j * rstep;
                    if (V > 1) v[j] = ld_pack<T>(a); else v[j].v[0] = ld_one<T>(a);
                }
#pragma unroll
                for (int j = 0; j < U; ++j)
#pragma unroll
                    for (int k = 0; k < V; ++k)
                        run[k].step(r, v[j].v[k], (int32_t)(rb + j), [&](int32_t ps) { return idx_of(ps, k); });
            } else {
                for (int j = 0; j < U && rb + j < n_rows; ++j) {
                    const char* a = a0 + (int64_t)j * rstep;
#pragma unroll
                    for (int k = 0; k < V; ++k)
                        if (k < nv) run[k].step(r, ld_one<T>(a + k * ES), (int32_t)(rb + j), [&](int32_t ps) { return idx_of(ps, k); });
                }
            }
        }
#pragma unroll
        for (int k = 0; k < V; ++k) run[k].settle(k < nv && first < n_rows ? (int32_t)first : -1);
#pragma unroll
        for (int k = 0; k < V; ++k)
            if (k < nv)
                emit(r, p, b * C + col0 + k, q.n_split, s, run[k].finish(r, [&](int32_t ps) { return idx_of(ps, k); }), out, out2, partial);
    }
}

// ---- GEN ------------------------------------------------------------------------------
template <typename R, int G>
__global__ void __launch_bounds__(kBlock)
red_gen_kernel(const RedPlan p, const R r, const RedLaunch q, const char* __restrict__ in, char* out, char* out2,
               typename R::Acc* partial) {
    using T = typename R::In;
    using Acc = typename R::Acc;
    constexpr int ES = sizeof(T);
    pdl_trigger();                           // a second (folding) pass may be launched while this one runs
    constexpr int GPB = kBlock / G;
    __shared__ Acc smem[kWarpsPerBlock];
    const int gid = threadIdx.x / G, gl = threadIdx.x % G;
    const int64_t items = p.n_out * q.n_split;
    for (int64_t item0 = (int64_t)blockIdx.x * GPB; item0 < items; item0 += (int64_t)gridDim.x * GPB) {
        const int64_t item = item0 + gid;
        const bool live = item < items;
        Acc acc = r.identity();
        int64_t o = 0, s = 0;
        if (live) {
            o = item / q.n_split;
            s = item - o * q.n_split;
            const int64_t in_off = offset_of(o, p.n_od, p.oshape, p.in_ostep);
            const int64_t begin = s * q.seg_len;
            int64_t end = begin + q.seg_len; if (end > p.n_red) end = p.n_red;
            for (int64_t e0 = begin + gl; e0 < end; e0 += (int64_t)G * kUnroll) {
                T v[kUnroll];
                int64_t off[kUnroll];
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    int64_t e = e0 + (int64_t)j * G;
                    if (e < end) {
                        off[j] = in_off + offset_of(e, p.n_rd, p.rshape, p.in_rstep);
                        v[j] = ld_one<T>(in + off[j]);
                    }
                }
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    int64_t e = e0 + (int64_t)j * G;
                    if (e < end) acc = r.combine(acc, r.map(v[j], q.flat_index ? off[j] / ES : e));
                }
            }
        }
        acc = group_fold<R, G>(r, acc, smem);
        if (live && gl == 0) emit(r, p, o, q.n_split, s, acc, out, out2, partial);
    }
}

// ---- second pass: fold the segments of each output, in segment order -------------------
// G == 32: a warp per output; G == kBlock: a CTA per output (many segments, few outputs).
template <typename R, int G>
__global__ void __launch_bounds__(kBlock)
red_fold_kernel(const RedPlan p, const R r, const typename R::Acc* __restrict__ partial, int n_split,
                char* out, char* out2) {
    using Acc = typename R::Acc;
    constexpr int GPB = kBlock / G;
    __shared__ Acc smem[kWarpsPerBlock];
    const int gid = threadIdx.x / G, gl = threadIdx.x % G;
    pdl_wait();                              // the first pass has finished and its partials are visible
    for (int64_t o0 = (int64_t)blockIdx.x * GPB; o0 < p.n_out; o0 += (int64_t)gridDim.x * GPB) {
        const int64_t o = o0 + gid;
        const bool live = o < p.n_out;
        // thread t takes the contiguous run of segments [t*per, (t+1)*per): thread order == segment order
        const int per = (n_split + G - 1) / G;
        Acc acc = r.identity();
        if (live) {
            // eight independent loads at a time, folded in order
            const Acc* run = partial + o * n_split;
            for (int k = 0; k < per; k += 8) {
                Acc buf[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    int s = gl * per + k + i;
                    if (k + i < per && s < n_split) buf[i] = run[s];
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    int s = gl * per + k + i;
                    if (k + i < per && s < n_split) acc = r.combine(acc, buf[i]);
                }
            }
        }
        acc = group_fold<R, G>(r, acc, smem);
        if (live && gl == 0) emit(r, p, o, 1, 0, acc, out, out2, (Acc*)nullptr);
    }
}

// Many segments, few outputs: a CTA of 1024 threads per output, so that even 8192 segments are
// one batch of eight independent loads per thread.  Thread order == segment order throughout.
template <typename R>
__global__ void __launch_bounds__(1024)
red_fold_big_kernel(const RedPlan p, const R r, const typename R::Acc* __restrict__ partial, int n_split,
                    char* out, char* out2) {
    using Acc = typename R::Acc;
    __shared__ Acc smem[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per = (n_split + 1023) / 1024;
    pdl_wait();                              // the first pass has finished and its partials are visible
    for (int64_t o = blockIdx.x; o < p.n_out; o += gridDim.x) {
        const Acc* run = partial + o * n_split;
        Acc acc = r.identity();
        for (int k = 0; k < per; k += 8) {
            Acc buf[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int s = (int)threadIdx.x * per + k + i;
                if (k + i < per && s < n_split) buf[i] = run[s];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int s = (int)threadIdx.x * per + k + i;
                if (k + i < per && s < n_split) acc = r.combine(acc, buf[i]);
            }
        }
        acc = warp_fold(r, acc);
        __syncthreads();                     // smem may still be read from the previous output
        if (lane == 0) smem[warp] = acc;
        __syncthreads();
        if (warp == 0) {
            acc = warp_fold(r, smem[lane]);
            if (lane == 0) emit(r, p, o, 1, 0, acc, out, out2, (Acc*)nullptr);
        }
    }
}

// Scratch for the [output][segment] partials from the host program's allocator.  A null answer means the
// allocator has already reported the failure its own way (an exception in the extension, the error latch in the
// library's default): the caller launches nothing, because a first pass would write through the null pointer.
template <typename Acc>
inline Acc* take_partials(int64_t count) {
    return reinterpret_cast<Acc*>(cumo_cuda_runtime_malloc(sizeof(Acc) * (size_t)count));
}

inline unsigned red_grid(int64_t ctas) { return (unsigned)(ctas < 1 ? 1 : (ctas > 0x7fffffffLL ? 0x7fffffffLL : ctas)); }

// ---- host ----------------------------------------------------------------------------------
// flat_index: 0 = feed the position along the reduce axes, 1 = feed the element offset.
template <typename R>
void launch_reduce(const cumo_na_reduction_arg_t* arg, const cumo_na_iarray_t* out2_arr, const R& r, int flat_index) {
    CB200_TRACE_LAUNCH();
    using T = typename R::In;
    using Acc = typename R::Acc;
    constexpr int ES = sizeof(T);
    constexpr int VMAX = 16 / ES;
    constexpr int64_t kSegBytes = 32 << 10;           // one CTA's share of a long row
    constexpr int64_t kManyRows = 148 * 64;           // rows enough to fill a B200 with a warp each
    constexpr int64_t kColSegRows = 256;              // one CTA's share of a column strip
    constexpr int64_t kColWideSegRows = 256;          // the same when the strip is a CTA wide (4 KiB per row)
    constexpr int64_t kColWideRound = 148 * 4;        // CTAs of that plan resident at once on a B200: 148 SMs x 4
    constexpr size_t kColWideSmem = 48 << 10;
    RedPlan p;
    if (!make_red_plan(&p, arg, out2_arr)) return;
    const char* in = arg->in.ptr;
    char* out = arg->out.ptr;
    char* out2 = out2_arr ? out2_arr->ptr : nullptr;
    cudaStream_t st = current_stream();
    Acc* partial = nullptr;
    RedLaunch q;
    q.n_split = 1;
    q.n_strips = 0;
    q.flat_index = flat_index;
    q.ordered = 1;
    if (flat_index)                                   // element offsets grow along a run only with positive steps
        for (int d = 0; d < p.n_rd; ++d) if (p.in_rstep[d] < 0) q.ordered = 0;
    for (int d = 0; d + 1 < p.n_rd; ++d) if (flat_index && p.in_rstep[d] < p.in_rstep[d + 1] * p.rshape[d + 1]) q.ordered = 0;

    const bool row = p.n_rd == 1 && (p.in_rstep[0] == ES || p.n_red <= 1);
    // the column plan takes one strided reduce dim and index-ordered runs; anything else is GEN's
    const bool col = !row && p.n_rd == 1 && q.ordered && p.in_ostep[p.n_od - 1] == ES && p.oshape[p.n_od - 1] >= 8;

    if (row) {
        const int64_t L = p.n_red;
        bool vec = aligned16(in);
        for (int d = 0; d < p.n_od && vec; ++d) if (!mult16(p.in_ostep[d])) vec = false;
        // a warp per row while there are rows enough to fill the device that way (no CTA-wide fold per
        // 16 KiB of input); a CTA per (row, segment) for long or few rows
        // (these thresholds are constants of the plan, not read from the device: a result never depends on where it ran)
        const bool wide = L >= 4096 && !(L * ES <= kSegBytes && p.n_out >= kManyRows);
        q.seg_len = L > 0 ? L : 1;
        // rows of up to 256 KiB stay whole, one CTA each, when there are CTAs enough without cutting them
        const bool whole_rows = p.n_out >= kManyRows / 8 && L * ES <= 8 * kSegBytes;
        if (wide && !whole_rows) {
            // a multiple of 32 elements: segment starts stay 16-byte aligned.  Index reductions fold 16-byte {value, index}
            // accumulators across the CTA, which costs about as much as scanning 32 KiB, so their segments are longer
            int64_t seg = kSegBytes / ES;
            if (R::kHasScan) {
                // about two and a half rounds of resident CTAs (148 SMs x 8) over the row, in whole multiples of
                // kSegBytes, at most 16 of them: a function of the row length only
                int64_t mult = (L * ES / 3000 + kSegBytes - 1) / kSegBytes;
                mult = mult < 1 ? 1 : (mult > 16 ? 16 : mult);
                seg *= mult;
            }
            int64_t ns = (L + seg - 1) / seg;
            while (ns > 8192) { seg *= 2; ns = (L + seg - 1) / seg; }
            if (ns > 1) { q.seg_len = seg; q.n_split = (int)ns; }
        }
        if (q.n_split > 1 && !(partial = take_partials<Acc>(p.n_out * q.n_split))) return;
        const int64_t items = p.n_out * q.n_split;
        if (wide) {
            if (vec) red_row_kernel<R, VMAX, kBlock><<<red_grid(items), kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
            else     red_row_kernel<R, 1, kBlock><<<red_grid(items), kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
        } else {
            // short rows: one lane (up to 4 packets) or 4 lanes (up to 16) per row instead of a warp (a warp per 16-element row
            // leaves 28 lanes idle and pays a five-step fold per 64 bytes); every lane then has up to four loads in flight and
            // a warp covers 32 or 8 neighbouring rows
            const int64_t units = vec ? (L + VMAX - 1) / VMAX : L;
            if (units <= 4 && q.n_split == 1) {
                const unsigned grid = red_grid((items + kBlock - 1) / kBlock);
                if (vec) red_row_kernel<R, VMAX, 1><<<grid, kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
                else     red_row_kernel<R, 1, 1><<<grid, kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
            } else if (units <= 16 && q.n_split == 1) {
                const unsigned grid = red_grid((items + kBlock / 4 - 1) / (kBlock / 4));
                if (vec) red_row_kernel<R, VMAX, 4><<<grid, kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
                else     red_row_kernel<R, 1, 4><<<grid, kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
            } else {
                const unsigned grid = red_grid((items + kWarpsPerBlock - 1) / kWarpsPerBlock);
                if (vec) red_row_kernel<R, VMAX, 32><<<grid, kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
                else     red_row_kernel<R, 1, 32><<<grid, kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
            }
        }
    } else if (col) {
        const int od_in = p.n_od - 1;
        const int64_t C = p.oshape[od_in];
        bool vec = aligned16(in);
        for (int d = 0; d < od_in && vec; ++d) if (!mult16(p.in_ostep[d])) vec = false;
        for (int d = 0; d < p.n_rd && vec; ++d) if (!mult16(p.in_rstep[d])) vec = false;
        // thread-owned columns when a row of columns fills at least half a CTA; else a warp-wide strip with rows spread over warps
        const bool wide_cols = C >= (int64_t)kBlock * (vec ? VMAX : 1) / 2 && p.n_red < 0x7fffffffLL;
        const int64_t W = (wide_cols ? kBlock : 32) * (vec ? VMAX : 1);
        const int64_t seg_rows = wide_cols ? kColWideSegRows : kColSegRows;
        q.n_strips = (C + W - 1) / W;
        q.seg_len = p.n_red > 0 ? p.n_red : 1;
        if (p.n_red > seg_rows + seg_rows / 2) {
            int64_t seg = seg_rows;
            int64_t ns = (p.n_red + seg - 1) / seg;
            while (ns > 8192) { seg *= 2; ns = (p.n_red + seg - 1) / seg; }
            if (wide_cols) {
                // These CTAs are large (half a MiB of input) and all alike, so they run in rounds of
                // kColWideRound; a last round that is mostly empty costs as much as a full one.  Pick the
                // segment count so that the CTA count is just under a whole number of rounds (the rows are
                // dealt to the segments in blocks of kColUnroll, round robin, so any count balances).  The
                // round size is a constant of the plan, not a property read from the device, so results stay
                // the same anywhere.
                const int64_t lanes = (p.n_out / C) * q.n_strips;           // CTAs per segment index
                const int64_t rounds = (lanes * ns + kColWideRound - 1) / kColWideRound;
                const int64_t want = rounds * kColWideRound / lanes;
                const int64_t blocks = (p.n_red + kColUnroll - 1) / kColUnroll;
                if (want >= 2 && want <= 8192) ns = want < blocks ? want : blocks;
                seg = (p.n_red + ns - 1) / ns;                              // (not used by this kernel)
            }
            q.seg_len = seg;
            q.n_split = (int)ns;
        }
        if (q.n_split > 1 && !(partial = take_partials<Acc>(p.n_out * q.n_split))) return;
        const unsigned grid = red_grid((p.n_out / C) * q.n_strips * q.n_split);
        if (wide_cols) {
            // 48 KiB of (unused) dynamic shared memory per CTA holds residency at 4 CTAs per SM for every functor
            if (vec) red_colwide_kernel<R, VMAX><<<grid, kBlock, kColWideSmem, st>>>(p, r, q, in, out, out2, partial);
            else     red_colwide_kernel<R, 1><<<grid, kBlock, kColWideSmem, st>>>(p, r, q, in, out, out2, partial);
        } else {
            if (vec) red_col_kernel<R, VMAX><<<grid, kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
            else     red_col_kernel<R, 1><<<grid, kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
        }
    } else {
        const bool wide = p.n_red >= 2048;
        q.seg_len = p.n_red > 0 ? p.n_red : 1;
        if (wide) {
            int64_t seg = (int64_t)kBlock * kUnroll * 4;
            int64_t ns = (p.n_red + seg - 1) / seg;
            while (ns > 8192) { seg *= 2; ns = (p.n_red + seg - 1) / seg; }
            if (ns > 1) { q.seg_len = seg; q.n_split = (int)ns; }
        }
        if (q.n_split > 1 && !(partial = take_partials<Acc>(p.n_out * q.n_split))) return;
        const int64_t items = p.n_out * q.n_split;
        if (wide) red_gen_kernel<R, kBlock><<<red_grid(items), kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
        else      red_gen_kernel<R, 32><<<red_grid((items + kWarpsPerBlock - 1) / kWarpsPerBlock), kBlock, 0, st>>>(p, r, q, in, out, out2, partial);
    }
    int launches = 1;
    if (q.n_split > 1) {
        const Acc* cpartial = partial;
        if (q.n_split > 1024 && p.n_out <= 64)
            launch_dependent(red_fold_big_kernel<R>, red_grid(p.n_out), 1024, st, p, r, cpartial, q.n_split, out, out2);
        else if (q.n_split > 256 && p.n_out < 4096)
            launch_dependent(red_fold_kernel<R, kBlock>, red_grid(p.n_out), kBlock, st, p, r, cpartial, q.n_split, out, out2);
        else
            launch_dependent(red_fold_kernel<R, 32>, red_grid((p.n_out + kWarpsPerBlock - 1) / kWarpsPerBlock), kBlock, st, p, r, cpartial, q.n_split, out, out2);
        ++launches;
        cumo_cuda_runtime_free(reinterpret_cast<char*>(partial));
    }
    count_launch(launches);
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200
