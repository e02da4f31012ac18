// Definitions of the reduction entry points `cumo_<T>_<op>_kernel_launch` for one
// element type.  Included by abi_<type>_red.cu after defining CB_T, CB_C, CB_FLOAT
// (and CB_DOUBLE for the double-precision type).  Signatures are the reference's
// (include/cumo_b200.h gives the file:line of each declaration).
#include "reduce.cuh"
#include "mulsum.cuh"

using namespace cb200;

#define CB_RSYM_(t, name) cumo_##t##_##name##_kernel_launch
#define CB_RSYM(t, name) CB_RSYM_(t, name)
#define CB_RED(name) CB_RSYM(CB_T, name)

static inline CB_C reduce_length(const cumo_na_reduction_arg_t* arg) {
    size_t o = arg->out_indexer.total_size;
    return (CB_C)(o ? arg->in_indexer.total_size / o : 0);
}

#define DEF_ACCUM(name, ...)                                                           \
    extern "C" void CB_RED(name)(cumo_na_reduction_arg_t* arg) {                        \
        auto r = __VA_ARGS__;                                                           \
        launch_reduce(arg, nullptr, r, 0);                                              \
    }
// (max|min)_index feed the element offset, arg(max|min) the position along the axes
#define DEF_INDEX(name, IS_MAX, NANW)                                                  \
    extern "C" void CB_RED(name##_int32)(cumo_na_reduction_arg_t* arg) {                \
        launch_reduce(arg, nullptr, red::ArgMinMax<CB_C, IS_MAX, NANW>{0, 0}, 1); }        \
    extern "C" void CB_RED(name##_int64)(cumo_na_reduction_arg_t* arg) {                \
        launch_reduce(arg, nullptr, red::ArgMinMax<CB_C, IS_MAX, NANW>{1, 0}, 1); }
#define DEF_ARG(name, IS_MAX, NANW)                                                    \
    extern "C" void CB_RED(name##_int32)(cumo_na_reduction_arg_t* arg) {                \
        launch_reduce(arg, nullptr, red::ArgMinMax<CB_C, IS_MAX, NANW>{0, 0}, 0); }        \
    extern "C" void CB_RED(name##_int64)(cumo_na_reduction_arg_t* arg) {                \
        launch_reduce(arg, nullptr, red::ArgMinMax<CB_C, IS_MAX, NANW>{1, 0}, 0); }

// Index and value from one pass (no reference counterpart: the reference has no multi-GPU
// reductions, whose per-rank partial is exactly this pair).  Indices are int64_t; index_base is added to each
// (the shard's offset in the global array).
#define CB_VSYM_(t, name) cb200_##t##_##name##_with_value_kernel_launch
#define CB_VSYM(t, name) CB_VSYM_(t, name)
#define DEF_WITH_VALUE(name, IS_MAX, NANW, FLAT)                                                           \
    extern "C" void CB_VSYM(CB_T, name)(cumo_na_reduction_arg_t* arg, cumo_na_iarray_t* values, int64_t index_base) { \
        launch_reduce(arg, values, red::ArgMinMax<CB_C, IS_MAX, NANW>{1, index_base}, FLAT); }
DEF_WITH_VALUE(max_index, true, false, 1)
DEF_WITH_VALUE(min_index, false, false, 1)
DEF_WITH_VALUE(argmax, true, false, 0)
DEF_WITH_VALUE(argmin, false, false, 0)
#if CB_FLOAT
DEF_WITH_VALUE(max_index_nan, true, true, 1)
DEF_WITH_VALUE(min_index_nan, false, true, 1)
DEF_WITH_VALUE(argmax_nan, true, true, 0)
DEF_WITH_VALUE(argmin_nan, false, true, 0)
#endif

DEF_ACCUM(sum, red::SumLike<CB_C, false, false>{0, CB_C(0)})
DEF_ACCUM(prod, red::SumLike<CB_C, false, true>{0, CB_C(0)})
DEF_ACCUM(min, red::MinMax<CB_C, false, false>{})
DEF_ACCUM(max, red::MinMax<CB_C, true, false>{})
DEF_ACCUM(ptp, red::MinAndMax<CB_C, false, false>{})
extern "C" void CB_RED(minmax)(cumo_na_reduction_arg_t* arg, cumo_na_iarray_t* out2) {
    launch_reduce(arg, out2, red::MinAndMax<CB_C, false, true>{}, 0);
}
DEF_INDEX(max_index, true, false)
DEF_INDEX(min_index, false, false)
DEF_ARG(argmax, true, false)
DEF_ARG(argmin, false, false)

#if CB_FLOAT
DEF_ACCUM(mean, red::SumLike<CB_C, false, false>{1, reduce_length(arg)})
DEF_ACCUM(var, red::Moments<CB_C, false>{0})
DEF_ACCUM(stddev, red::Moments<CB_C, false>{1})
DEF_ACCUM(rms, red::Rms<CB_C, false>{reduce_length(arg)})
DEF_ACCUM(sum_nan, red::SumLike<CB_C, true, false>{0, CB_C(0)})
DEF_ACCUM(prod_nan, red::SumLike<CB_C, true, true>{0, CB_C(0)})
DEF_ACCUM(min_nan, red::MinMax<CB_C, false, true>{})
DEF_ACCUM(max_nan, red::MinMax<CB_C, true, true>{})
DEF_ACCUM(ptp_nan, red::MinAndMax<CB_C, true, false>{})
DEF_ACCUM(mean_nan, red::MeanNan<CB_C>{})
DEF_ACCUM(var_nan, red::Moments<CB_C, true>{0})
DEF_ACCUM(stddev_nan, red::Moments<CB_C, true>{1})
DEF_ACCUM(rms_nan, red::Rms<CB_C, true>{CB_C(0)})
extern "C" void CB_RED(minmax_nan)(cumo_na_reduction_arg_t* arg, cumo_na_iarray_t* out2) {
    launch_reduce(arg, out2, red::MinAndMax<CB_C, true, true>{}, 0);
}
DEF_INDEX(max_index_nan, true, true)
DEF_INDEX(min_index_nan, false, true)
DEF_ARG(argmax_nan, true, true)
DEF_ARG(argmin_nan, false, true)
#ifdef CB_DOUBLE
DEF_ACCUM(kahan_sum, red::Kahan<CB_C, false>{})
DEF_ACCUM(kahan_sum_nan, red::Kahan<CB_C, true>{})
#endif
#endif

// ---- mulsum ---------------------------------------------------------------------------
#define CB_MSYM_(t, sfx, tail) cumo_##t##_mulsum##sfx##tail
#define CB_MSYM(t, sfx, tail) CB_MSYM_(t, sfx, tail)
extern "C" void CB_MSYM(CB_T, , _reduce_kernel_launch)(char* p1, char* p2, char* p3, ssize_t s1, ssize_t s2, uint64_t n) {
    launch_mulsum_reduce<CB_C, false>(p1, p2, p3, s1, s2, n);
}
extern "C" void CB_MSYM(CB_T, , _kernel_launch)(char* p1, char* p2, char* p3, ssize_t s1, ssize_t s2, ssize_t s3, uint64_t n) {
    launch_mulsum_each<CB_C, false>(p1, p2, p3, s1, s2, s3, n);
}
#define CB_MAXES_(t, sfx) cb200_##t##_mulsum##sfx##_axes_kernel_launch
#define CB_MAXES(t, sfx) CB_MAXES_(t, sfx)
#define CB_MAXES_ARGS char* p1, char* p2, char* p3, int n_keep, const size_t* keep_shape, const ssize_t* keep_step1, const ssize_t* keep_step2, \
                      const ssize_t* keep_step3, int n_red, const size_t* red_shape, const ssize_t* red_step1, const ssize_t* red_step2
#define CB_MAXES_PASS p1, p2, p3, n_keep, keep_shape, keep_step1, keep_step2, keep_step3, n_red, red_shape, red_step1, red_step2
extern "C" void CB_MAXES(CB_T, )(CB_MAXES_ARGS) { launch_mulsum_axes<CB_C, false>(CB_MAXES_PASS); }
#if CB_FLOAT
extern "C" void CB_MAXES(CB_T, _nan)(CB_MAXES_ARGS) { launch_mulsum_axes<CB_C, true>(CB_MAXES_PASS); }
extern "C" void CB_MSYM(CB_T, _nan, _reduce_kernel_launch)(char* p1, char* p2, char* p3, ssize_t s1, ssize_t s2, uint64_t n) {
    launch_mulsum_reduce<CB_C, true>(p1, p2, p3, s1, s2, n);
}
extern "C" void CB_MSYM(CB_T, _nan, _kernel_launch)(char* p1, char* p2, char* p3, ssize_t s1, ssize_t s2, ssize_t s3, uint64_t n) {
    launch_mulsum_each<CB_C, true>(p1, p2, p3, s1, s2, s3, n);
}
#endif
