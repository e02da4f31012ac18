// Rank-order folds of per-GPU partial results: the last step of a row-sharded reduction.
//
// The reference has no multi-GPU code; these entry points have no counterpart there.  Every rank reduces its own
// rows with the ordinary kernels, the per-rank partials are gathered (NCCL all_gather: a few bytes per output),
// and each rank folds the `world` rows of the gathered block with the kernels below, in rank order, so the answer
// is the same on every rank and does not depend on the collective's algorithm:
//   * float sums / means: partials of the element type are added in float64 and rounded once;
//   * min / max: the per-rank answers merged with red::MinMax::combine (the single-GPU NaN rules);
//   * index reductions: {value, global index} pairs are merged with the same total order the single-GPU kernels
//     use (red::ArgMinMax::combine: NaN rule first, then the better value, then the lower index), so NaN handling
//     and first-occurrence ties hold across GPUs exactly as they hold across CTAs.
// One thread per output, `world` coalesced loads each; the gathered block is a few KiB.
#include "reducers.cuh"

namespace cb200 {

template <typename T>
__global__ void __launch_bounds__(kBlock)
rank_fold_sum_kernel(const char* __restrict__ partials, int64_t rank_stride, int world, int64_t n_out, double divisor, T* out) {
    pdl_wait();            // launched as a dependent of the exchange (or of whatever precedes it): resident early, reads late
    for (int64_t o = (int64_t)blockIdx.x * kBlock + threadIdx.x; o < n_out; o += (int64_t)gridDim.x * kBlock) {
        double acc = 0.0;
        for (int r = 0; r < world; ++r) acc += (double)reinterpret_cast<const T*>(partials + r * rank_stride)[o];
        if (divisor != 0.0) acc /= divisor;
        out[o] = (T)acc;
    }
}

template <typename T, bool IS_MAX, bool NAN_WINS>
__global__ void __launch_bounds__(kBlock)
rank_fold_arg_kernel(const char* __restrict__ indices, const char* __restrict__ values, int64_t rank_stride, int world, int64_t n_out,
                     int64_t* out_index, T* out_value) {
    using R = red::ArgMinMax<T, IS_MAX, NAN_WINS>;
    const R r{1};
    pdl_wait();
    for (int64_t o = (int64_t)blockIdx.x * kBlock + threadIdx.x; o < n_out; o += (int64_t)gridDim.x * kBlock) {
        typename R::Acc acc = r.identity();
        for (int k = 0; k < world; ++k) {
            typename R::Acc b;
            b.value = reinterpret_cast<const T*>(values + k * rank_stride)[o];
            b.index = reinterpret_cast<const int64_t*>(indices + k * rank_stride)[o];
            acc = r.combine(acc, b);
        }
        out_index[o] = acc.index;
        if (out_value) out_value[o] = acc.value;
    }
}

// min / max of the per-rank answers with the single-GPU functor's rules (plain form: a NaN loses unless all are NaN;
// _nan form: a NaN wins)
template <typename T, bool IS_MAX, bool NAN_WINS>
__global__ void __launch_bounds__(kBlock)
rank_fold_extreme_kernel(const char* __restrict__ partials, int64_t rank_stride, int world, int64_t n_out, T* out) {
    using R = red::MinMax<T, IS_MAX, NAN_WINS>;
    const R r{};
    pdl_wait();
    for (int64_t o = (int64_t)blockIdx.x * kBlock + threadIdx.x; o < n_out; o += (int64_t)gridDim.x * kBlock) {
        typename R::Acc acc = reinterpret_cast<const T*>(partials)[o];
        for (int k = 1; k < world; ++k) acc = r.combine(acc, reinterpret_cast<const T*>(partials + k * rank_stride)[o]);
        out[o] = acc;
    }
}

template <typename T>
static void launch_rank_fold_extreme(const char* partials, int64_t rank_stride, int world, int64_t n_out, int is_max, int nan_wins, char* out) {
    if (n_out <= 0 || world <= 0) return;
    const unsigned grid = grid_for((n_out + kBlock - 1) / kBlock, 8);
    cudaStream_t st = current_stream();
    T* o = reinterpret_cast<T*>(out);
    if constexpr (!red::is_fp<T>::value) nan_wins = 0;
    if (is_max) {
        if (nan_wins) launch_dependent(rank_fold_extreme_kernel<T, true, red::is_fp<T>::value>, grid, kBlock, st, partials, rank_stride, world, n_out, o);
        else          launch_dependent(rank_fold_extreme_kernel<T, true, false>, grid, kBlock, st, partials, rank_stride, world, n_out, o);
    } else {
        if (nan_wins) launch_dependent(rank_fold_extreme_kernel<T, false, red::is_fp<T>::value>, grid, kBlock, st, partials, rank_stride, world, n_out, o);
        else          launch_dependent(rank_fold_extreme_kernel<T, false, false>, grid, kBlock, st, partials, rank_stride, world, n_out, o);
    }
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

template <typename T>
static void launch_rank_fold_sum(const char* partials, int64_t rank_stride, int world, int64_t n_out, double divisor, char* out) {
    if (n_out <= 0 || world <= 0) return;
    launch_dependent(rank_fold_sum_kernel<T>, grid_for((n_out + kBlock - 1) / kBlock, 8), kBlock, current_stream(), partials, rank_stride, world, n_out, divisor, reinterpret_cast<T*>(out));
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

template <typename T>
static void launch_rank_fold_arg(const char* indices, const char* values, int64_t rank_stride, int world, int64_t n_out, int is_max, int nan_wins,
                                 int64_t* out_index, char* out_value) {
    if (n_out <= 0 || world <= 0) return;
    const unsigned grid = grid_for((n_out + kBlock - 1) / kBlock, 8);
    cudaStream_t st = current_stream();
    T* ov = reinterpret_cast<T*>(out_value);
    if constexpr (!red::is_fp<T>::value) nan_wins = 0;
    if (is_max) {
        if (nan_wins) launch_dependent(rank_fold_arg_kernel<T, true, red::is_fp<T>::value>, grid, kBlock, st, indices, values, rank_stride, world, n_out, out_index, ov);
        else          launch_dependent(rank_fold_arg_kernel<T, true, false>, grid, kBlock, st, indices, values, rank_stride, world, n_out, out_index, ov);
    } else {
        if (nan_wins) launch_dependent(rank_fold_arg_kernel<T, false, red::is_fp<T>::value>, grid, kBlock, st, indices, values, rank_stride, world, n_out, out_index, ov);
        else          launch_dependent(rank_fold_arg_kernel<T, false, false>, grid, kBlock, st, indices, values, rank_stride, world, n_out, out_index, ov);
    }
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
}

}  // namespace cb200

extern "C" {
void cb200_sfloat_rank_fold_sum_kernel_launch(const char* partials, int64_t rank_stride, int world, int64_t n_out, double divisor, char* out) {
    cb200::launch_rank_fold_sum<float>(partials, rank_stride, world, n_out, divisor, out);
}
void cb200_dfloat_rank_fold_sum_kernel_launch(const char* partials, int64_t rank_stride, int world, int64_t n_out, double divisor, char* out) {
    cb200::launch_rank_fold_sum<double>(partials, rank_stride, world, n_out, divisor, out);
}
#define CB200_DEF_FOLD_ARG(T, C)                                                                                                        \
    void cb200_##T##_rank_fold_arg_kernel_launch(const char* indices, const char* values, int64_t rank_stride, int world, int64_t n_out, \
                                                 int is_max, int nan_wins, int64_t* out_index, char* out_value) {                       \
        cb200::launch_rank_fold_arg<C>(indices, values, rank_stride, world, n_out, is_max, nan_wins, out_index, out_value);              \
    }
#define CB200_DEF_FOLD_EXTREME(T, C)                                                                                                    \
    void cb200_##T##_rank_fold_extreme_kernel_launch(const char* partials, int64_t rank_stride, int world, int64_t n_out, int is_max,   \
                                                     int nan_wins, char* out) {                                                         \
        cb200::launch_rank_fold_extreme<C>(partials, rank_stride, world, n_out, is_max, nan_wins, out);                                  \
    }
CB200_DEF_FOLD_EXTREME(sfloat, float)
CB200_DEF_FOLD_EXTREME(dfloat, double)
CB200_DEF_FOLD_EXTREME(int32, int32_t)
CB200_DEF_FOLD_EXTREME(int64, int64_t)
CB200_DEF_FOLD_ARG(sfloat, float)
CB200_DEF_FOLD_ARG(dfloat, double)
CB200_DEF_FOLD_ARG(int32, int32_t)
CB200_DEF_FOLD_ARG(int64, int64_t)
}
