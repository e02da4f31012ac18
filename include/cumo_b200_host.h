/*
 * cumo_b200_host.h -- a small C++-implemented, C-callable host layer that plays the
 * part of the reference's host code ABOVE the kernel-launch ABI when the Ruby
 * extension is not there: an NArray object (typed device buffer + shape + byte
 * steps, views), and an ndloop that casts, broadcasts, allocates the output,
 * moves reduce dimensions last, builds the cumo_na_* descriptors and calls the
 * `cumo_..._kernel_launch` symbol of include/cumo_b200.h that the reference's
 * generated iterator would call for the same method.
 *
 * It mirrors, for the hot path only:
 *   ext/cumo/narray/ndloop.c:494-516   broadcast rule (extent 1 repeats, else must match)
 *   ext/cumo/narray/ndloop.c:523-595   per-operand byte steps, 0 on repeated dims
 *   ext/cumo/narray/ndloop.c:750-815   output allocation / in-place output
 *   ext/cumo/narray/ndloop.c:421-451   reduce dimensions transposed to the end
 *   ext/cumo/narray/gen/tmpl/binary.c:113-220, unary.c, unary_s.c, cond_binary.c,
 *   accum.c:62-90, accum_index.c:51-137, accum_arg.c:50-128, tmpl_bit/bit_count.c:49-69
 *   ext/cumo/narray/narray.c:1313-1333 upcast table (restricted to the four types)
 *   ext/cumo/cuda/runtime.c:22-69      integer div-by-zero flag protocol
 *
 * Errors: functions that return a handle return NULL on error, others return
 * non-zero; cb200_host_error() then gives the class and message, named after the
 * Ruby exception the reference raises ("ShapeError", "ZeroDivisionError",
 * "ValueError", "TypeError", "CudaError").
 */
#ifndef CUMO_B200_HOST_H
#define CUMO_B200_HOST_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cb200_na cb200_na_t;

enum {
    CB200_SFLOAT = 0, CB200_DFLOAT = 1, CB200_INT32 = 2, CB200_INT64 = 3,
    CB200_BIT = 4,      /* 1 bit per element, 32-bit words, LSB first; steps/offset in bits */
    CB200_UINT64 = 5,   /* result container of count_true/count_false and bincount */
    CB200_UINT32 = 6    /* result container of bincount */
};

const char* cb200_host_error(const char** klass);   /* message (and class) of the last error on this thread */

/* ---- arrays ---- */
cb200_na_t* cb200_na_new(int dtype, int ndim, const int64_t* shape);                 /* uninitialised, contiguous */
cb200_na_t* cb200_na_zeros(int dtype, int ndim, const int64_t* shape);
/* borrow device memory owned by someone else (steps in bytes; bits for CB200_BIT) */
cb200_na_t* cb200_na_wrap(int dtype, int ndim, const int64_t* shape, const int64_t* step, void* device_ptr, int64_t offset);
/* a view of `a`: new shape/steps/offset (offset relative to a's first element, same unit as steps) */
cb200_na_t* cb200_na_view(cb200_na_t* a, int ndim, const int64_t* shape, const int64_t* step, int64_t offset);
void cb200_na_release(cb200_na_t* a);
int  cb200_na_dtype(const cb200_na_t* a);
int  cb200_na_ndim(const cb200_na_t* a);
int64_t cb200_na_size(const cb200_na_t* a);
void cb200_na_shape(const cb200_na_t* a, int64_t* shape);
void cb200_na_steps(const cb200_na_t* a, int64_t* step);
int64_t cb200_na_offset(const cb200_na_t* a);
void* cb200_na_base(const cb200_na_t* a);              /* start of the underlying buffer */
int  cb200_na_is_contiguous(const cb200_na_t* a);
void cb200_na_set_inplace(cb200_na_t* a, int on);      /* `x.inplace`: the next operation writes into x */
/* host <-> device, contiguous arrays only; `bytes` must be the array's byte size
 * (Bit: 4 * ceil(size/32)).  store is asynchronous on the launch stream when
 * `host` is pinned; read synchronises the stream. */
int cb200_na_store_host(cb200_na_t* a, const void* host, size_t bytes);
int cb200_na_read_host(cb200_na_t* a, void* host, size_t bytes);
/* The same read queued on `copy_stream` (a cudaStream_t) behind the work queued so far on the launch stream; does not
 * synchronise: the caller keeps `a` and `host` (pinned) alive and synchronises copy_stream before reading `host`. */
int cb200_na_read_host_async(cb200_na_t* a, void* host, size_t bytes, void* copy_stream);
int cb200_synchronize(void);

/* ---- operations (names are the reference's method names) ---- */
/* binary: add sub mul div mod pow copysign bit_and bit_or bit_xor left_shift right_shift
 *         maximum minimum maximum_nan minimum_nan atan2 hypot ldexp.  Operands of different
 *         types are cast to the upcast type first. */
cb200_na_t* cb200_na_binary(const char* op, cb200_na_t* a, cb200_na_t* b);
/* array (op) host numeric; the numeric is converted to the array's type, as the reference's
 * `_s` path does for a Float/Integer operand.  scalar_is_left: numeric (op) array. */
cb200_na_t* cb200_na_binary_scalar(const char* op, cb200_na_t* a, double sv_f, int64_t sv_i, int scalar_is_left);
/* `x ** Integer` with repeated multiplication (pow_int32 path) */
cb200_na_t* cb200_na_pow_int(cb200_na_t* a, int32_t exponent);
/* unary: minus reciprocal sign square abs floor round ceil trunc rint bit_not and the
 *        NMath functions sqrt cbrt log log2 log10 exp exp2 exp10 sin cos tan asin acos atan
 *        sinh cosh tanh asinh acosh atanh sinc erf erfc log1p expm1 */
cb200_na_t* cb200_na_unary(const char* op, cb200_na_t* a);
/* comparisons -> Bit: eq ne gt ge lt le nearly_eq; classifications: isnan isinf isposinf
 * isneginf isfinite signbit (b == NULL) */
cb200_na_t* cb200_na_compare(const char* op, cb200_na_t* a, cb200_na_t* b);
cb200_na_t* cb200_na_compare_scalar(const char* op, cb200_na_t* a, double sv_f, int64_t sv_i, int scalar_is_left);
/* reductions: sum prod mean var stddev rms min max ptp kahan_sum max_index min_index argmax
 * argmin.  axis_mask bit i = reduce dimension i; 0 = reduce everything.  nan = the
 * method's `nan: true`. */
cb200_na_t* cb200_na_reduce(const char* op, cb200_na_t* a, uint32_t axis_mask, int keepdims, int nan);
int cb200_na_minmax(cb200_na_t* a, uint32_t axis_mask, int keepdims, int nan, cb200_na_t** out_min, cb200_na_t** out_max);
/* Bit#where (want_zeros 0) and the second half of where2 (want_zeros 1): ascending row-major positions of the
 * one / zero bits as Int32, or Int64 when the array has more than 2^32-1 elements (gen/tmpl_bit/where.c:97-130).
 * Reads the count back to size the result: synchronises. */
cb200_na_t* cb200_na_where(cb200_na_t* bits, int want_zeros);
/* cumsum / cumprod (narray/gen/tmpl/cum.c:41-70): axis < 0 runs over all elements in row-major order, else along
 * that axis; the result has the operand's shape and type.  nan: the NaN-skipping operator (float types). */
cb200_na_t* cb200_na_cum(const char* op, cb200_na_t* a, int axis, int nan);
/* bincount along the last axis (narray/gen/tmpl/bincount.c:176-240): counts as UInt32 (UInt64 when the length
 * exceeds 2^32-1), or sums of `weight` (SFloat stays SFloat, anything else is summed as DFloat); the length is
 * max+1 or `minlength` if larger; a negative element raises ArgumentError.  Reads the extremes back: synchronises. */
cb200_na_t* cb200_na_bincount(cb200_na_t* a, cb200_na_t* weight, int64_t minlength);
/* max_index / min_index / argmax / argmin together with the winning value, one pass; the index array is Int64.
 * Not a method of the reference: it exists for the sharded (multi-GPU) reductions. */
int cb200_na_arg_with_value(const char* op, cb200_na_t* a, uint32_t axis_mask, int nan, cb200_na_t** out_index, cb200_na_t** out_value);
/* The same with `index_base` added to every index (a shard's offset in the global array) and, when idx_out and
 * val_out are given, the results written into those contiguous device buffers (e.g. the two halves of a buffer
 * that a collective sends next); out_index / out_value may then be NULL. */
int cb200_na_arg_with_value_into(const char* op, cb200_na_t* a, uint32_t axis_mask, int nan, int64_t index_base, void* idx_out, void* val_out,
                                 cb200_na_t** out_index, cb200_na_t** out_value);
/* `a[idx, true]`-style selection along one axis (narray/index.c index arrays + the store through an index array,
 * gen/tmpl/store_from.c:82-89): positions from a 1-D Int32/Int64 device array, not range-checked; returns the copy. */
cb200_na_t* cb200_na_take(cb200_na_t* a, int axis, cb200_na_t* idx);
/* Bit#mask (gen/tmpl_bit/mask.c:95-140): the elements of `a` where `bits` (same shape) is one, row-major order, as a
 * 1-D array of a's type.  Reads the count back to size the result: synchronises. */
cb200_na_t* cb200_na_mask(cb200_na_t* bits, cb200_na_t* a);
/* count_true / count_false of a Bit array -> UInt64 */
cb200_na_t* cb200_na_count(cb200_na_t* a, uint32_t axis_mask, int keepdims, int want_false);
/* Bit o Bit: op = "and" | "or" | "xor" | "eq" with b, "copy" | "not" with b == NULL; operands broadcast like the value types. */
cb200_na_t* cb200_na_bit_op(const char* op, cb200_na_t* a, cb200_na_t* b);
/* Bit#all? / #any? over the axes of axis_mask (0 = all): a Bit array of the kept dims. */
cb200_na_t* cb200_na_bit_reduce(const char* op, cb200_na_t* a, uint32_t axis_mask, int keepdims);

/* `a.clip(min, max)`, reference: gen/tmpl/clip.c:218-276.  Each bound is absent (kind 0), a host numeric (kind 1:
 * the value in *_f for the float types, *_i for the integer types) or an array (kind 2).  OperationError when
 * min > max anywhere; ArgumentError when neither bound is given.  Writes into `a` when it is marked in-place. */
cb200_na_t* cb200_na_clip(cb200_na_t* a, int lo_kind, cb200_na_t* lo, double lo_f, int64_t lo_i,
                          int hi_kind, cb200_na_t* hi, double hi_f, int64_t hi_i);
/* `a.fill(v)` and `a.seq(beg, step)`, reference: gen/tmpl/fill.c:18-27, seq.c:21-117: write through `a`, which may
 * be any view; 0 on success */
int cb200_na_fill(cb200_na_t* a, double value_f, int64_t value_i);
int cb200_na_seq(cb200_na_t* a, double beg, double step);
/* `a.divmod(b)`, reference: gen/tmpl/binary2.c:58-95; `a.modf`, gen/tmpl/unary_ret2.c:33-44; `NMath.frexp(a)`,
 * gen/tmpl/frexp.c:36-48 (the exponents as an Int32 array).  Two results each; 0 on success. */
int cb200_na_divmod(cb200_na_t* a, cb200_na_t* b, cb200_na_t** out_quot, cb200_na_t** out_rem);
int cb200_na_modf(cb200_na_t* a, cb200_na_t** out_frac, cb200_na_t** out_whole);
int cb200_na_frexp(cb200_na_t* a, cb200_na_t** out_mantissa, cb200_na_t** out_exponent);
/* mulsum(a, b, axis...) = (a*b).sum(axis...) in one pass over the inputs */
cb200_na_t* cb200_na_mulsum(cb200_na_t* a, cb200_na_t* b, uint32_t axis_mask, int keepdims, int nan);
/* contiguous copy / cast (the reference's `dup`, `reshape` copy and `Type.cast`) */
cb200_na_t* cb200_na_cast(cb200_na_t* a, int dtype);
cb200_na_t* cb200_na_copy(cb200_na_t* a);

#ifdef __cplusplus
}
#endif
#endif /* CUMO_B200_HOST_H */
