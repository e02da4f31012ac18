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
//        flight per thread; long rows with few outputs are cut into segments so
//        that every SM has several CTAs to run.
//   COL  the innermost OUTPUT axis is the contiguous one (a column / "transposed"
//        reduction).  A CTA owns a strip of 32 lanes x 16 bytes of columns; its
//        8 warps walk different rows with 16-byte loads and keep one accumulator
//        per column in registers; rows are cut into segments across CTAs.
//   GEN  any other stride pattern: a group per (output, segment), offsets from a
//        32-bit index split.
//   Segmented plans write accumulators to scratch ([output][segment]) and a
//   second launch folds the segments of each output in index order, so a result
//   depends only on (shape, strides, SM count), never on scheduling.
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

template <typename R>
__device__ __forceinline__ typename R::Acc warp_fold(const R& r, typename R::Acc a) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {      // lane i folds in lane i+d: earlier positions stay on the left
        typename R::Acc b = shfl_down_acc(a, d);
        a = r.combine(a, b);
    }
    return a;                                // lane 0 holds the warp's result
}

// Result valid in thread 0 of the group.  G == 32: a warp; G == kBlock: the CTA.
template <typename R, int G>
__device__ __forceinline__ typename R::Acc group_fold(const R& r, typename R::Acc a, typename R::Acc* smem) {
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

template <typename R>
__device__ __forceinline__ void emit(const R& r, const RedPlan& p, int64_t o, int n_split, int64_t s,
                                     typename R::Acc a, char* out, char* out2, typename R::Acc* partial) {
    if (n_split > 1) { partial[o * n_split + s] = a; return; }
    int64_t oo = offset_of(o, p.n_od, p.oshape, p.out_step);
    int64_t o2 = out2 ? offset_of(o, p.n_od, p.oshape, p.out2_step) : 0;
    r.store(out + oo, out2 ? out2 + o2 : nullptr, a);
}

// ---- ROW ------------------------------------------------------------------------------
template <typename R, int V, int G>
__global__ void __launch_bounds__(kBlock)
red_row_kernel(const RedPlan p, const R r, const char* __restrict__ in, char* out, char* out2,
               typename R::Acc* partial, int64_t seg_len, int n_split, int flat_index) {
    using T = typename R::In;
    using Acc = typename R::Acc;
    constexpr int ES = sizeof(T);
    constexpr int GPB = kBlock / G;          // groups per CTA
    __shared__ Acc smem[kWarpsPerBlock];
    const int gid = threadIdx.x / G, gl = threadIdx.x % G;
    const int64_t L = p.n_red;
    const int64_t items = p.n_out * n_split;
    for (int64_t item0 = (int64_t)blockIdx.x * GPB; item0 < items; item0 += (int64_t)gridDim.x * GPB) {
        const int64_t item = item0 + gid;
        const bool live = item < items;      // whole groups go idle together; G==kBlock: always live
        Acc acc = r.identity();
        int64_t o = 0, s = 0;
        if (live) {
            o = item / n_split;
            s = item - o * n_split;
            const int64_t in_off = offset_of(o, p.n_od, p.oshape, p.in_ostep);
            const int64_t begin = s * seg_len;
            int64_t end = begin + seg_len; if (end > L) end = L;
            const char* base = in + in_off;
            const int64_t idx_base = flat_index ? in_off / ES : 0;
            for (int64_t e0 = begin + (int64_t)gl * V; e0 < end; e0 += (int64_t)G * V * kUnroll) {
                Pack<T> v[kUnroll];
                int nv[kUnroll];
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    int64_t e = e0 + (int64_t)j * G * V;
                    int64_t left = end - e;
                    nv[j] = left >= V ? V : (left > 0 ? (int)left : 0);
                    if (V > 1 && nv[j] == V) v[j] = ld_pack<T>(base + e * ES);
                    else {
#pragma unroll
                        for (int k = 0; k < V; ++k) if (k < nv[j]) v[j].v[k] = ld_one<T>(base + (e + k) * ES);
                    }
                }
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    int64_t e = e0 + (int64_t)j * G * V;
#pragma unroll
                    for (int k = 0; k < V; ++k)
                        if (k < nv[j]) acc = r.combine(acc, r.map(v[j].v[k], idx_base + e + k));
                }
            }
        }
        acc = group_fold<R, G>(r, acc, smem);
        if (live && gl == 0) emit(r, p, o, n_split, s, acc, out, out2, partial);
    }
}

// ---- COL ------------------------------------------------------------------------------
template <typename R, int V>
__global__ void __launch_bounds__(kBlock)
red_col_kernel(const RedPlan p, const R r, const char* __restrict__ in, char* out, char* out2,
               typename R::Acc* partial, int64_t rows_per_seg, int n_split, int64_t n_strips, int flat_index) {
    using T = typename R::In;
    using Acc = typename R::Acc;
    constexpr int ES = sizeof(T);
    constexpr int W = 32 * V;                // columns per strip
    __shared__ Acc smem[kWarpsPerBlock][W];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int od_in = p.n_od - 1;            // innermost out dim = the columns
    const int64_t C = p.oshape[od_in];
    const int64_t n_batch = p.n_out / C;
    const int64_t items = n_batch * n_strips * n_split;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t s = item % n_split;
        const int64_t t = item / n_split;
        const int64_t strip = t % n_strips;
        const int64_t b = t / n_strips;
        const int64_t col0 = strip * W + (int64_t)lane * V;
        const int64_t cleft = C - col0;
        const int nv = cleft >= V ? V : (cleft > 0 ? (int)cleft : 0);
        const int64_t in_b = offset_of(b, od_in, p.oshape, p.in_ostep);
        const int64_t r_begin = s * rows_per_seg;
        int64_t r_end = r_begin + rows_per_seg; if (r_end > p.n_red) r_end = p.n_red;
        Acc acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = r.identity();
        if (nv > 0) {
            const char* base = in + in_b + col0 * ES;
            for (int64_t r0 = r_begin + warp; r0 < r_end; r0 += kWarpsPerBlock * kUnroll) {
                Pack<T> v[kUnroll];
                int64_t roff[kUnroll];
                bool ok[kUnroll];
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    int64_t row = r0 + j * kWarpsPerBlock;
                    ok[j] = row < r_end;
                    if (!ok[j]) continue;
                    roff[j] = (p.n_rd == 1) ? row * p.in_rstep[0] : offset_of(row, p.n_rd, p.rshape, p.in_rstep);
                    if (V > 1 && nv == V) v[j] = ld_pack<T>(base + roff[j]);
                    else {
#pragma unroll
                        for (int k = 0; k < V; ++k) if (k < nv) v[j].v[k] = ld_one<T>(base + roff[j] + k * ES);
                    }
                }
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    if (!ok[j]) continue;
                    int64_t row = r0 + j * kWarpsPerBlock;
                    int64_t idx = flat_index ? (in_b + roff[j]) / ES + col0 : row;
#pragma unroll
                    for (int k = 0; k < V; ++k)
                        if (k < nv) acc[k] = r.combine(acc[k], r.map(v[j].v[k], flat_index ? idx + k : idx));
                }
            }
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
                emit(r, p, b * C + col0 + k, n_split, s, a, out, out2, partial);
            }
        }
    }
}

// ---- GEN ------------------------------------------------------------------------------
template <typename R, int G>
__global__ void __launch_bounds__(kBlock)
red_gen_kernel(const RedPlan p, const R r, const char* __restrict__ in, char* out, char* out2,
               typename R::Acc* partial, int64_t seg_len, int n_split, int flat_index) {
    using T = typename R::In;
    using Acc = typename R::Acc;
    constexpr int ES = sizeof(T);
    constexpr int GPB = kBlock / G;
    __shared__ Acc smem[kWarpsPerBlock];
    const int gid = threadIdx.x / G, gl = threadIdx.x % G;
    const int64_t items = p.n_out * n_split;
    for (int64_t item0 = (int64_t)blockIdx.x * GPB; item0 < items; item0 += (int64_t)gridDim.x * GPB) {
        const int64_t item = item0 + gid;
        const bool live = item < items;
        Acc acc = r.identity();
        int64_t o = 0, s = 0;
        if (live) {
            o = item / n_split;
            s = item - o * n_split;
            const int64_t in_off = offset_of(o, p.n_od, p.oshape, p.in_ostep);
            const int64_t begin = s * seg_len;
            int64_t end = begin + seg_len; if (end > p.n_red) end = p.n_red;
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
                    if (e < end) acc = r.combine(acc, r.map(v[j], flat_index ? off[j] / ES : e));
                }
            }
        }
        acc = group_fold<R, G>(r, acc, smem);
        if (live && gl == 0) emit(r, p, o, n_split, s, acc, out, out2, partial);
    }
}

// ---- second pass: fold the segments of each output, in segment order -------------------
template <typename R>
__global__ void __launch_bounds__(kBlock)
red_fold_kernel(const RedPlan p, const R r, const typename R::Acc* __restrict__ partial, int n_split,
                char* out, char* out2) {
    using Acc = typename R::Acc;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int64_t o = (int64_t)blockIdx.x * kWarpsPerBlock + warp; o < p.n_out; o += (int64_t)gridDim.x * kWarpsPerBlock) {
        // lane l takes the contiguous run of segments [l*per, (l+1)*per): lane order == segment order
        const int per = (n_split + 31) / 32;
        Acc acc = r.identity();
        for (int k = 0; k < per; ++k) {
            int s = lane * per + k;
            if (s < n_split) acc = r.combine(acc, partial[o * n_split + s]);
        }
        acc = warp_fold(r, acc);
        if (lane == 0) emit(r, p, o, 1, 0, acc, out, out2, (Acc*)nullptr);
    }
}

// ---- host ----------------------------------------------------------------------------------
// flat_index: 0 = feed the position along the reduce axes, 1 = feed the element offset.
template <typename R>
void launch_reduce(const cumo_na_reduction_arg_t* arg, const cumo_na_iarray_t* out2_arr, const R& r, int flat_index) {
    using T = typename R::In;
    using Acc = typename R::Acc;
    constexpr int ES = sizeof(T);
    constexpr int VMAX = 16 / ES;
    RedPlan p;
    if (!make_red_plan(&p, arg, out2_arr)) return;
    const char* in = arg->in.ptr;
    char* out = arg->out.ptr;
    char* out2 = out2_arr ? out2_arr->ptr : nullptr;
    cudaStream_t st = current_stream();
    const int64_t target = (int64_t)sm_count() * 8;   // CTAs wanted in flight
    Acc* partial = nullptr;
    int n_split = 1;
    int launches = 1;

    const bool row = p.n_rd == 1 && (p.in_rstep[0] == ES || p.n_red <= 1);
    const bool col = !row && p.in_ostep[p.n_od - 1] == ES && p.oshape[p.n_od - 1] >= 8;

    if (row) {
        const int64_t L = p.n_red;
        bool vec = aligned16(in);
        for (int d = 0; d < p.n_od && vec; ++d) if (!mult16(p.in_ostep[d])) vec = false;
        const int V = vec ? VMAX : 1;
        const bool wide = L >= 4096;                    // a CTA per item, else a warp per item
        int64_t seg_len = L > 0 ? L : 1;
        if (wide && p.n_out < target) {
            const int64_t min_seg = (int64_t)kBlock * VMAX * kUnroll * 2;
            int64_t want = (target + p.n_out - 1) / p.n_out;
            int64_t fits = L / min_seg;
            int64_t ns = want < fits ? want : fits;
            if (ns > 1) {
                seg_len = (L + ns - 1) / ns;
                seg_len = (seg_len + 31) / 32 * 32;     // keeps every segment start 16-byte aligned
                n_split = (int)((L + seg_len - 1) / seg_len);
            }
        }
        if (n_split > 1) partial = reinterpret_cast<Acc*>(cumo_cuda_runtime_malloc(sizeof(Acc) * p.n_out * n_split));
        const int64_t items = p.n_out * n_split;
        if (wide) {
            unsigned grid = grid_for(items, 8);
            if (vec) red_row_kernel<R, VMAX, kBlock><<<grid, kBlock, 0, st>>>(p, r, in, out, out2, partial, seg_len, n_split, flat_index);
            else     red_row_kernel<R, 1, kBlock><<<grid, kBlock, 0, st>>>(p, r, in, out, out2, partial, seg_len, n_split, flat_index);
        } else {
            unsigned grid = grid_for((items + kWarpsPerBlock - 1) / kWarpsPerBlock, 8);
            if (vec) red_row_kernel<R, VMAX, 32><<<grid, kBlock, 0, st>>>(p, r, in, out, out2, partial, seg_len, n_split, flat_index);
            else     red_row_kernel<R, 1, 32><<<grid, kBlock, 0, st>>>(p, r, in, out, out2, partial, seg_len, n_split, flat_index);
        }
    } else if (col) {
        const int od_in = p.n_od - 1;
        const int64_t C = p.oshape[od_in];
        bool vec = aligned16(in);
        for (int d = 0; d < od_in && vec; ++d) if (!mult16(p.in_ostep[d])) vec = false;
        for (int d = 0; d < p.n_rd && vec; ++d) if (!mult16(p.in_rstep[d])) vec = false;
        const int V = vec ? VMAX : 1;
        const int64_t W = 32 * V;
        const int64_t n_strips = (C + W - 1) / W;
        const int64_t base_items = (p.n_out / C) * n_strips;
        int64_t rows_per_seg = p.n_red > 0 ? p.n_red : 1;
        if (base_items < target) {
            const int64_t min_rows = kWarpsPerBlock * kUnroll * 2;
            int64_t want = (target + base_items - 1) / base_items;
            int64_t fits = p.n_red / min_rows;
            int64_t ns = want < fits ? want : fits;
            if (ns > 1) {
                rows_per_seg = (p.n_red + ns - 1) / ns;
                n_split = (int)((p.n_red + rows_per_seg - 1) / rows_per_seg);
            }
        }
        if (n_split > 1) partial = reinterpret_cast<Acc*>(cumo_cuda_runtime_malloc(sizeof(Acc) * p.n_out * n_split));
        unsigned grid = grid_for(base_items * n_split, 8);
        if (vec) red_col_kernel<R, VMAX><<<grid, kBlock, 0, st>>>(p, r, in, out, out2, partial, rows_per_seg, n_split, n_strips, flat_index);
        else     red_col_kernel<R, 1><<<grid, kBlock, 0, st>>>(p, r, in, out, out2, partial, rows_per_seg, n_split, n_strips, flat_index);
    } else {
        const bool wide = p.n_red >= 2048;
        int64_t seg_len = p.n_red > 0 ? p.n_red : 1;
        if (wide && p.n_out < target) {
            const int64_t min_seg = (int64_t)kBlock * kUnroll * 2;
            int64_t want = (target + p.n_out - 1) / p.n_out;
            int64_t fits = p.n_red / min_seg;
            int64_t ns = want < fits ? want : fits;
            if (ns > 1) {
                seg_len = (p.n_red + ns - 1) / ns;
                n_split = (int)((p.n_red + seg_len - 1) / seg_len);
            }
        }
        if (n_split > 1) partial = reinterpret_cast<Acc*>(cumo_cuda_runtime_malloc(sizeof(Acc) * p.n_out * n_split));
        const int64_t items = p.n_out * n_split;
        if (wide) red_gen_kernel<R, kBlock><<<grid_for(items, 8), kBlock, 0, st>>>(p, r, in, out, out2, partial, seg_len, n_split, flat_index);
        else      red_gen_kernel<R, 32><<<grid_for((items + kWarpsPerBlock - 1) / kWarpsPerBlock, 8), kBlock, 0, st>>>(p, r, in, out, out2, partial, seg_len, n_split, flat_index);
    }
    if (n_split > 1) {
        red_fold_kernel<R><<<grid_for((p.n_out + kWarpsPerBlock - 1) / kWarpsPerBlock, 8), kBlock, 0, st>>>(p, r, partial, n_split, out, out2);
        ++launches;
        cumo_cuda_runtime_free(reinterpret_cast<char*>(partial));
    }
    count_launch(launches);
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200
