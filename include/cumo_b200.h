/*
 * cumo_b200.h -- the C ABI of libcumo_b200: hand-written sm_100a kernels behind
 * the kernel-launch entry points of Cumo::NArray's data-parallel core.
 *
 * Every `cumo_..._kernel_launch` function declared here has the name, argument
 * list and meaning of the function of the same name that the reference's
 * generated type files declare on their host side and define in their `.cu`
 * half.  The comment above each group names the reference template that
 * declares it (paths are relative to the reference project root).  The host
 * code of the Ruby extension (ndloop, the generated `iter_*` functions) calls
 * these with descriptors that live on its stack; data pointers inside the
 * descriptors must be device-accessible.
 *
 * Conventions shared by all entry points (reference: ext/cumo/include/cumo/
 * template_kernel.h:83-90, ext/cumo/cuda/runtime.c:16-69):
 *   - return type is void; after each launch the function calls
 *     cumo_cuda_runtime_check_kernel_launch(), which the host program owns;
 *   - scratch memory is taken from cumo_cuda_runtime_malloc() and given back
 *     with cumo_cuda_runtime_free() before the function returns (stream-ordered
 *     reuse is safe because all work is issued on one stream);
 *   - kernels are launched asynchronously on the legacy default stream unless
 *     cb200_set_stream() chose another one for the calling thread;
 *   - data-dependent errors (integer division by zero, abs of the minimum
 *     integer) store 1 through the caller's `int*` flag, which must be
 *     device-writable (mapped pinned host memory in the reference), and skip
 *     the element.  Nothing ever traps.
 */
#ifndef CUMO_B200_H
#define CUMO_B200_H

#include <stddef.h>
#include <stdint.h>
#include <sys/types.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- descriptor layouts (ABI; reference: ext/cumo/include/cumo/indexer.h:16-68,
 *      ext/cumo/include/cumo/narray_kernel.h CUMO_NA_MAX_DIMENSION) ---- */
#ifndef CUMO_NA_MAX_DIMENSION
#define CUMO_NA_MAX_DIMENSION 12
#endif
#ifndef CUMO_BIT_DIGIT
#define CUMO_BIT_DIGIT unsigned int
#endif

#ifndef CUMO_INDEXER_H /* the reference's own header defines the same types */
typedef struct {
    unsigned char ndim;                      /* number of dimensions            */
    size_t total_size;                       /* number of elements              */
    size_t shape[CUMO_NA_MAX_DIMENSION];     /* extent of each dimension        */
    uint64_t index[CUMO_NA_MAX_DIMENSION];   /* scratch of the reference kernels; ignored here */
    uint64_t raw_index;                      /* idem                            */
} cumo_na_indexer_t;

typedef struct {
    char* ptr;                               /* first element (view offset applied) */
    ssize_t step[CUMO_NA_MAX_DIMENSION];     /* BYTE step per dimension; 0 = broadcast; may be negative */
} cumo_na_iarray_t;

typedef struct {
    CUMO_BIT_DIGIT* ptr;                     /* first 32-bit word of the Bit array */
    size_t pos;                              /* BIT position of the first element  */
    ssize_t step[CUMO_NA_MAX_DIMENSION];     /* BIT step per dimension             */
} cumo_na_bit_iarray_t;

/* A byte step or, when the low bit of the word is clear, a device array of byte offsets, one per position
 * along the dimension (reference: ext/cumo/include/cumo/narray_kernel.h:168-176, narray.h:329-330:
 * a step s is stored as (s << 1) | 1, an index array as its address). */
typedef union {
    ssize_t stride;
    size_t* index;
} cumo_stridx_t;

typedef struct {
    char* ptr;                               /* first element (view offset applied) */
    cumo_stridx_t stridx[CUMO_NA_MAX_DIMENSION];
} cumo_na_iarray_stridx_t;

typedef struct {
    CUMO_BIT_DIGIT* ptr;                     /* first 32-bit word of the Bit array */
    size_t pos;                              /* BIT position of the first element  */
    cumo_stridx_t stridx[CUMO_NA_MAX_DIMENSION];   /* BIT step ((s << 1) | 1) or array of bit offsets per dimension */
} cumo_na_bit_iarray_stridx_t;

typedef struct {
    cumo_na_iarray_t in;                     /* reduce dimensions are the LAST dims of `in` */
    cumo_na_iarray_t out;                    /* steps for the leading out_indexer.ndim dims */
    cumo_na_indexer_t in_indexer;
    cumo_na_indexer_t out_indexer;
} cumo_na_reduction_arg_t;
#endif

/* ---- callbacks owned by the host program (reference: template_kernel.h:83-90).
 * libcumo_b200 carries weak default definitions (a per-device caching pool over
 * cudaMalloc and an error latch read by cb200_last_error) so that it also
 * works standalone; inside cumo.so the extension's own strong definitions win. */
void  cumo_cuda_runtime_check_kernel_launch(void);
char* cumo_cuda_runtime_malloc(size_t size);
void  cumo_cuda_runtime_free(char* ptr);

/* ---- library-level helpers (no counterpart in the reference) ---- */
/* Stream used by the calling thread's launches; NULL = legacy default stream. */
void  cb200_set_stream(void* cuda_stream);
void* cb200_get_stream(void);
/* Error latch of the default check_kernel_launch: 0 = ok, else the cudaError_t
 * value; the message is valid until the next call on this thread.  Reading
 * clears the latch. */
int   cb200_last_error(const char** message);
/* Number of kernels this library has launched in this process. */
uint64_t cb200_launch_count(void);
/* Bytes held by / handed out from the default scratch pool on the current device. */
size_t cb200_pool_total_bytes(void);
size_t cb200_pool_used_bytes(void);
void   cb200_pool_free_all_blocks(void);
const char* cb200_version(void);

/* =====================================================================
 * Per-dtype entry points.  T is one of sfloat, dfloat, int32, int64 and
 * C the C element type (float, double, int32_t, int64_t).
 * ===================================================================== */

/* binary arithmetic, reference: gen/tmpl/binary.c:12-15, binary_kernel.cu:69-81.
 * z = x op y; `_s` carries a host numeric by value, on the left when
 * scalar_is_left != 0.  Integer div/mod by zero sets *divzero. */
#define CB200_DECL_BINARY(T, C, op) \
    void cumo_iter_##T##_##op##_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer, int* divzero);
#define CB200_DECL_BINARY_S(T, C, op) \
    CB200_DECL_BINARY(T, C, op) \
    void cumo_iter_##T##_##op##_s_kernel_launch(cumo_na_iarray_t* a1, C sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer, int* divzero, int scalar_is_left);

/* unary arithmetic, reference: gen/tmpl/unary.c:3, unary_kernel.cu:28-42.
 * Integer reciprocal of zero sets *divzero. */
#define CB200_DECL_UNARY(T, C, op) \
    void cumo_iter_##T##_##op##_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_indexer_t* indexer, int* divzero);

/* abs, reference: gen/tmpl/unary2.c:3, unary2_kernel.cu:26-38.  abs of the
 * minimum signed integer sets *intmin. */
#define CB200_DECL_ABS(T, C) \
    void cumo_iter_##T##_abs_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_indexer_t* indexer, int* intmin);

/* NMath one-argument functions, reference: gen/tmpl/unary_s.c:2, unary_s_kernel.cu:14-28 */
#define CB200_DECL_MATH(T, C, fn) \
    void cumo_iter_##T##_math_s_##fn##_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_indexer_t* indexer);

/* NMath two-argument functions, reference: gen/tmpl/binary_s.c:2-3, binary_s_kernel.cu:38-51 */
#define CB200_DECL_MATH2(T, C, fn) \
    void cumo_iter_##T##_math_s_##fn##_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_math_s_##fn##_s_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer, C sv, int scalar_is_left);

/* comparisons into a Bit array, reference: gen/tmpl/cond_binary.c:2-3, cond_binary_kernel.cu:41-53 */
#define CB200_DECL_COND(T, C, op) \
    void cumo_iter_##T##_##op##_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_bit_iarray_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_##op##_s_kernel_launch(cumo_na_iarray_t* a1, C sv, cumo_na_bit_iarray_t* a3, cumo_na_indexer_t* indexer, int scalar_is_left);

/* float classification into a Bit array, reference: gen/tmpl/cond_unary.c:2, cond_unary_kernel.cu:15-29 */
#define CB200_DECL_COND_UNARY(T, C, op) \
    void cumo_iter_##T##_##op##_kernel_launch(cumo_na_iarray_t* a1, cumo_na_bit_iarray_t* a2, cumo_na_indexer_t* indexer);

/* power, reference: gen/tmpl/pow.c:2-6, pow_kernel.cu:54-106.  The int32 forms
 * take an Int32 exponent (array or host numeric) and multiply repeatedly. */
#define CB200_DECL_POW(T, C) \
    void cumo_iter_##T##_pow_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_pow_int32_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_pow_s_kernel_launch(cumo_na_iarray_t* a1, C sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer, int scalar_is_left); \
    void cumo_iter_##T##_pow_int32_s_left_kernel_launch(C sv_base, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_pow_int32_s_kernel_launch(cumo_na_iarray_t* a1, int32_t sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer);

/* elementwise maximum/minimum, reference: gen/tmpl/ewcomp.c:19, ewcomp_kernel.cu:16-32 */
#define CB200_DECL_EWCOMP(T, C, op) \
    void cumo_##T##_##op##_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer);

/* clip, reference: gen/tmpl/clip.c:2-7, clip_kernel.cu:60-129.  x limited to [min, max]; `_min` / `_max` limit one
 * side only; `_s` carries host numerics.  With two arrays of bounds an element whose min > max sets *invalid and is
 * left unwritten; with two numerics the caller has compared them. */
#define CB200_DECL_CLIP(T, C) \
    void cumo_iter_##T##_clip_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_iarray_t* a4, cumo_na_indexer_t* indexer, int* invalid); \
    void cumo_iter_##T##_clip_s_kernel_launch(cumo_na_iarray_t* a1, C sv_min, C sv_max, cumo_na_iarray_t* a4, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_clip_min_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_clip_min_s_kernel_launch(cumo_na_iarray_t* a1, C sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_clip_max_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_clip_max_s_kernel_launch(cumo_na_iarray_t* a1, C sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer);

/* fill, reference: gen/tmpl/fill.c:2, fill_kernel.cu:13-29.  Every element of a1 takes val.
 * seq, reference: gen/tmpl/seq.c:19, seq_kernel.cu:37-53.  Element i (row-major over the indexer) takes
 * beg + step * (count + i); D is the reference's seq_data_t: the element type for the float types, double for the
 * integer types, whose value then goes through int64_t.
 * divmod, reference: gen/tmpl/binary2.c:2, binary2_kernel.cu:28-44.  a3 = a1 / a2 and a4 = a1 % a2 in one pass; an
 * integer zero divisor sets *divzero and leaves both elements unwritten. */
#define CB200_DECL_FILL_SEQ_DIVMOD(T, C, D) \
    void cumo_iter_##T##_fill_kernel_launch(cumo_na_iarray_t* a1, cumo_na_indexer_t* indexer, C val); \
    void cumo_iter_##T##_seq_kernel_launch(cumo_na_iarray_t* a1, cumo_na_indexer_t* indexer, D beg, D step, double count); \
    void cumo_iter_##T##_divmod_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_iarray_t* a4, cumo_na_indexer_t* indexer, int* divzero);

/* poly, reference: gen/tmpl/poly.c:2, poly_kernel.cu:22-44.  z = coef[0] + coef[1]*x + ... by Horner's rule; `coef` is a HOST
 * array of ncoef descriptors (a numeric coefficient arrives as an array whose steps are all 0); no coefficient: z = x.
 * eye, reference: gen/tmpl/eye.c:2, eye_kernel.cu:12-19.  The n0 x n1 matrix at ptr (byte steps s0, s1) gets `data` where
 * row + kofs == column and zero elsewhere. */
#define CB200_DECL_POLY_EYE(T, C) \
    void cumo_iter_##T##_poly_kernel_launch(cumo_na_iarray_t* x, cumo_na_iarray_t* coef, int ncoef, cumo_na_iarray_t* z, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_eye_stride_kernel_launch(char* ptr, ssize_t s0, ssize_t s1, ssize_t kofs, C data, uint64_t n0, uint64_t n1);

/* modf, reference: gen/tmpl/unary_ret2.c:2, unary_ret2_kernel.cu:16-31: a2 = fractional part, a3 = integral part.
 * frexp, reference: gen/tmpl/frexp.c:2, frexp_kernel.cu:15-31: a2 = mantissa, a3 = exponent (an Int32 array). */
#define CB200_DECL_MODF_FREXP(T) \
    void cumo_iter_##T##_modf_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_##T##_math_s_frexp_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* indexer);

/* value reductions, reference: gen/tmpl/accum.c:6-9, real_accum_kernel.cu:166-226,
 * float_accum_kernel.cu:155-206.  Integer sum/prod write int64_t. */
#define CB200_DECL_ACCUM(T, C, op) \
    void cumo_##T##_##op##_kernel_launch(cumo_na_reduction_arg_t* arg);

/* minmax, reference: gen/tmpl/minmax.c:2-5, real_accum_kernel.cu:191-194 */
#define CB200_DECL_MINMAX(T, C, sfx) \
    void cumo_##T##_minmax##sfx##_kernel_launch(cumo_na_reduction_arg_t* arg, cumo_na_iarray_t* out2);

/* index reductions, reference: gen/tmpl/accum_index.c:5 (max_index/min_index: flat
 * element offset from arg->in.ptr) and gen/tmpl/accum_arg.c:5 (argmax/argmin: index
 * along the reduced axes); accum_index_kernel.cu:121-144, accum_arg_kernel.cu:121-144.
 * The output element type is int32_t or int64_t as the name says. */
#define CB200_DECL_ACCUM_IDX(T, C, op) \
    void cumo_##T##_##op##_int32_kernel_launch(cumo_na_reduction_arg_t* arg); \
    void cumo_##T##_##op##_int64_kernel_launch(cumo_na_reduction_arg_t* arg);

/* Index reductions that also write the winning value (same descriptor as the entry above,
 * indices as int64_t; `values` has the layout of arg->out with the element type of the input).
 * `index_base` is added to every index (a shard's offset in the global array).
 * NOT in the reference: it is the per-GPU partial {value, index} of a sharded arg reduction,
 * produced in one pass over the data. */
#define CB200_DECL_ACCUM_IDX_VALUE(T, C, op) \
    void cb200_##T##_##op##_with_value_kernel_launch(cumo_na_reduction_arg_t* arg, cumo_na_iarray_t* values, int64_t index_base);

/* mulsum, reference: gen/tmpl/accum_binary.c:4-5, accum_binary_kernel.cu:69-92.
 * `_reduce_`: *p3 += sum_i x[i]*y[i];  plain: p3[i] += x[i]*y[i] (all steps in bytes). */
#define CB200_DECL_MULSUM(T, C, sfx) \
    void cumo_##T##_mulsum##sfx##_reduce_kernel_launch(char* p1, char* p2, char* p3, ssize_t s1, ssize_t s2, uint64_t n); \
    void cumo_##T##_mulsum##sfx##_kernel_launch(char* p1, char* p2, char* p3, ssize_t s1, ssize_t s2, ssize_t s3, uint64_t n);

/* mulsum over a whole loop in one launch: output k = (k_0 ..) gets sum over r of x*y ADDED to it, x at
 * p1 + sum k_i*keep_step1[i] + sum r_j*red_step1[j], y likewise with the *2 steps, the output at p3 + sum k_i*keep_step3[i]
 * (all byte steps; host arrays).  NOT in the reference, whose ndloop calls the two functions above once per innermost run
 * (gen/tmpl/accum_binary.c:9-46) -- one launch per element of the result of an integer `dot`. */
#define CB200_DECL_MULSUM_AXES(T, sfx) \
    void cb200_##T##_mulsum##sfx##_axes_kernel_launch(char* p1, char* p2, char* p3, int n_keep, const size_t* keep_shape, const ssize_t* keep_step1, \
        const ssize_t* keep_step2, const ssize_t* keep_step3, int n_red, const size_t* red_shape, const ssize_t* red_step1, const ssize_t* red_step2);
CB200_DECL_MULSUM_AXES(sfloat, ) CB200_DECL_MULSUM_AXES(dfloat, ) CB200_DECL_MULSUM_AXES(int32, ) CB200_DECL_MULSUM_AXES(int64, )
CB200_DECL_MULSUM_AXES(sfloat, _nan) CB200_DECL_MULSUM_AXES(dfloat, _nan)

/* store / cast from another element type (also the plain strided copy when the types
 * match), reference: gen/tmpl/store_from.c:2, store_from_kernel.cu:38-53.  NOTE the
 * argument order: a1 is the DESTINATION, a2 the source. */
#define CB200_DECL_STORE(T, F) \
    void cumo_iter_##T##_store_##F##_kernel_launch(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_indexer_t* indexer);

/* The same-type store for operands that may be addressed through index arrays (a view made by
 * `x[index_array, true]` or by Bit#mask), reference: gen/tmpl/store_from.c:5, store_from_kernel.cu:21-36. */
#define CB200_DECL_STORE_STRIDX(T) \
    void cumo_iter_##T##_store_##T##_stridx_kernel_launch(cumo_na_iarray_stridx_t* a1, cumo_na_iarray_stridx_t* a2, cumo_na_indexer_t* indexer);

/* one store per source class, as the reference instantiates them (gen/spec.rb:121-140) */
#define CB200_DECL_COMMON(T, C) \
    CB200_DECL_STORE(T, sfloat) CB200_DECL_STORE(T, dfloat) CB200_DECL_STORE(T, int32) CB200_DECL_STORE(T, int64) \
    CB200_DECL_STORE(T, int16) CB200_DECL_STORE(T, int8) CB200_DECL_STORE(T, uint64) CB200_DECL_STORE(T, uint32) \
    CB200_DECL_STORE(T, uint16) CB200_DECL_STORE(T, uint8) CB200_DECL_STORE_STRIDX(T) \
    CB200_DECL_BINARY_S(T, C, add) CB200_DECL_BINARY_S(T, C, sub) CB200_DECL_BINARY_S(T, C, mul) \
    CB200_DECL_BINARY_S(T, C, div) CB200_DECL_BINARY_S(T, C, mod) \
    CB200_DECL_UNARY(T, C, minus) CB200_DECL_UNARY(T, C, reciprocal) CB200_DECL_UNARY(T, C, sign) CB200_DECL_UNARY(T, C, square) \
    CB200_DECL_ABS(T, C) CB200_DECL_POW(T, C) \
    CB200_DECL_COND(T, C, eq) CB200_DECL_COND(T, C, ne) CB200_DECL_COND(T, C, gt) CB200_DECL_COND(T, C, ge) \
    CB200_DECL_COND(T, C, lt) CB200_DECL_COND(T, C, le) \
    CB200_DECL_EWCOMP(T, C, maximum) CB200_DECL_EWCOMP(T, C, minimum) \
    CB200_DECL_ACCUM(T, C, sum) CB200_DECL_ACCUM(T, C, prod) CB200_DECL_ACCUM(T, C, min) CB200_DECL_ACCUM(T, C, max) CB200_DECL_ACCUM(T, C, ptp) \
    CB200_DECL_MINMAX(T, C, ) \
    CB200_DECL_ACCUM_IDX(T, C, max_index) CB200_DECL_ACCUM_IDX(T, C, min_index) \
    CB200_DECL_ACCUM_IDX(T, C, argmax) CB200_DECL_ACCUM_IDX(T, C, argmin) \
    CB200_DECL_ACCUM_IDX_VALUE(T, C, max_index) CB200_DECL_ACCUM_IDX_VALUE(T, C, min_index) \
    CB200_DECL_ACCUM_IDX_VALUE(T, C, argmax) CB200_DECL_ACCUM_IDX_VALUE(T, C, argmin) \
    CB200_DECL_MULSUM(T, C, )

#define CB200_DECL_FLOAT(T, C) \
    CB200_DECL_COMMON(T, C) \
    CB200_DECL_BINARY_S(T, C, copysign) \
    CB200_DECL_UNARY(T, C, floor) CB200_DECL_UNARY(T, C, round) CB200_DECL_UNARY(T, C, ceil) CB200_DECL_UNARY(T, C, trunc) CB200_DECL_UNARY(T, C, rint) \
    CB200_DECL_COND(T, C, nearly_eq) \
    CB200_DECL_COND_UNARY(T, C, isnan) CB200_DECL_COND_UNARY(T, C, isinf) CB200_DECL_COND_UNARY(T, C, isposinf) \
    CB200_DECL_COND_UNARY(T, C, isneginf) CB200_DECL_COND_UNARY(T, C, isfinite) CB200_DECL_COND_UNARY(T, C, signbit) \
    CB200_DECL_MATH(T, C, sqrt) CB200_DECL_MATH(T, C, cbrt) CB200_DECL_MATH(T, C, log) CB200_DECL_MATH(T, C, log2) \
    CB200_DECL_MATH(T, C, log10) CB200_DECL_MATH(T, C, exp) CB200_DECL_MATH(T, C, exp2) CB200_DECL_MATH(T, C, exp10) \
    CB200_DECL_MATH(T, C, sin) CB200_DECL_MATH(T, C, cos) CB200_DECL_MATH(T, C, tan) CB200_DECL_MATH(T, C, asin) \
    CB200_DECL_MATH(T, C, acos) CB200_DECL_MATH(T, C, atan) CB200_DECL_MATH(T, C, sinh) CB200_DECL_MATH(T, C, cosh) \
    CB200_DECL_MATH(T, C, tanh) CB200_DECL_MATH(T, C, asinh) CB200_DECL_MATH(T, C, acosh) CB200_DECL_MATH(T, C, atanh) \
    CB200_DECL_MATH(T, C, sinc) CB200_DECL_MATH(T, C, erf) CB200_DECL_MATH(T, C, erfc) CB200_DECL_MATH(T, C, log1p) \
    CB200_DECL_MATH(T, C, expm1) \
    CB200_DECL_MATH2(T, C, atan2) CB200_DECL_MATH2(T, C, hypot) CB200_DECL_MATH2(T, C, ldexp) \
    CB200_DECL_EWCOMP(T, C, maximum_nan) CB200_DECL_EWCOMP(T, C, minimum_nan) \
    CB200_DECL_ACCUM(T, C, mean) CB200_DECL_ACCUM(T, C, var) CB200_DECL_ACCUM(T, C, stddev) CB200_DECL_ACCUM(T, C, rms) \
    CB200_DECL_ACCUM(T, C, sum_nan) CB200_DECL_ACCUM(T, C, prod_nan) CB200_DECL_ACCUM(T, C, min_nan) CB200_DECL_ACCUM(T, C, max_nan) \
    CB200_DECL_ACCUM(T, C, ptp_nan) CB200_DECL_ACCUM(T, C, mean_nan) CB200_DECL_ACCUM(T, C, var_nan) \
    CB200_DECL_ACCUM(T, C, stddev_nan) CB200_DECL_ACCUM(T, C, rms_nan) \
    CB200_DECL_MINMAX(T, C, _nan) \
    CB200_DECL_ACCUM_IDX(T, C, max_index_nan) CB200_DECL_ACCUM_IDX(T, C, min_index_nan) \
    CB200_DECL_ACCUM_IDX(T, C, argmax_nan) CB200_DECL_ACCUM_IDX(T, C, argmin_nan) \
    CB200_DECL_ACCUM_IDX_VALUE(T, C, max_index_nan) CB200_DECL_ACCUM_IDX_VALUE(T, C, min_index_nan) \
    CB200_DECL_ACCUM_IDX_VALUE(T, C, argmax_nan) CB200_DECL_ACCUM_IDX_VALUE(T, C, argmin_nan) \
    CB200_DECL_MULSUM(T, C, _nan)

#define CB200_DECL_INT(T, C) \
    CB200_DECL_COMMON(T, C) \
    CB200_DECL_BINARY_S(T, C, bit_and) CB200_DECL_BINARY_S(T, C, bit_or) CB200_DECL_BINARY_S(T, C, bit_xor) \
    CB200_DECL_BINARY_S(T, C, left_shift) CB200_DECL_BINARY_S(T, C, right_shift) \
    CB200_DECL_UNARY(T, C, bit_not)

CB200_DECL_FLOAT(sfloat, float)
CB200_DECL_FLOAT(dfloat, double)
CB200_DECL_INT(int32, int32_t)
CB200_DECL_INT(int64, int64_t)
CB200_DECL_CLIP(sfloat, float) CB200_DECL_CLIP(dfloat, double) CB200_DECL_CLIP(int32, int32_t) CB200_DECL_CLIP(int64, int64_t)
CB200_DECL_FILL_SEQ_DIVMOD(sfloat, float, float) CB200_DECL_FILL_SEQ_DIVMOD(dfloat, double, double)
CB200_DECL_FILL_SEQ_DIVMOD(int32, int32_t, double) CB200_DECL_FILL_SEQ_DIVMOD(int64, int64_t, double)
CB200_DECL_MODF_FREXP(sfloat) CB200_DECL_MODF_FREXP(dfloat)
CB200_DECL_POLY_EYE(sfloat, float) CB200_DECL_POLY_EYE(dfloat, double) CB200_DECL_POLY_EYE(int32, int32_t) CB200_DECL_POLY_EYE(int64, int64_t)

/* bincount along one run (integer types only), reference: gen/tmpl/bincount.c:18,70, bincount_kernel.cu:32-97.
 * The output run (n elements, byte step s2/s3) is cleared, then every element x of the input run (count elements
 * at p1, byte step s1, or byte offsets idx1[i] when idx1 is not NULL) adds 1 -- `_32`: uint32_t, `_64`: uint64_t
 * -- or its weight -- `_sf`: float, `_df`: double, weights at p2, byte step s2 -- to out[x].  An element outside
 * [0, n) sets *oor, leaves its value in *item and is skipped; both must be device-writable. */
#define CB200_DECL_BINCOUNT(T) \
    void cumo_iter_##T##_bincount_32_kernel_launch(char* p1, ssize_t s1, size_t* idx1, uint64_t count, char* p2, ssize_t s2, uint64_t n, int* oor, size_t* item); \
    void cumo_iter_##T##_bincount_64_kernel_launch(char* p1, ssize_t s1, size_t* idx1, uint64_t count, char* p2, ssize_t s2, uint64_t n, int* oor, size_t* item); \
    void cumo_iter_##T##_bincount_sf_kernel_launch(char* p1, ssize_t s1, char* p2, ssize_t s2, uint64_t count, char* p3, ssize_t s3, uint64_t n, int* oor, size_t* item); \
    void cumo_iter_##T##_bincount_df_kernel_launch(char* p1, ssize_t s1, char* p2, ssize_t s2, uint64_t count, char* p3, ssize_t s3, uint64_t n, int* oor, size_t* item);
CB200_DECL_BINCOUNT(int32)
CB200_DECL_BINCOUNT(int64)

/* Counting and sizing in one pass (unweighted).  NOT in the reference, whose method reads the run twice: a min/max reduction
 * that sizes the output (gen/tmpl/bincount.c:99-131), then the counting launch above.  The probe clears `hist`
 * (cb200_bincount_probe_bins() uint32_t counters, device memory), counts every element of the run with a value inside
 * [0, bins) and leaves the smallest and the largest value of ALL elements in extremes[0], extremes[1] (device memory).  A
 * caller that reads back 0 <= min and max < bins has the counts of the run in hist[0 .. max]; any other caller falls back
 * to the two passes. */
int cb200_bincount_probe_bins(void);
void cb200_int32_bincount_probe_kernel_launch(char* p1, ssize_t s1, uint64_t count, uint32_t* hist, long long* extremes);
void cb200_int64_bincount_probe_kernel_launch(char* p1, ssize_t s1, uint64_t count, uint32_t* hist, long long* extremes);

/* cumsum / cumprod along one run, reference: gen/tmpl/cum.c:3, cum_kernel.cu:56-80 (thrust::inclusive_scan there).
 * out[i] = x[0] op ... op x[i] for i < n; p1/p2 with byte steps s1/s2 of any sign.  `_nan` (float types): a NaN
 * accumulator is replaced by the next value, a NaN value is skipped (real_accum_kernel.h:12-26).  Returns the launch
 * status; the caller raises. */
#if defined(__CUDACC__) || defined(__DRIVER_TYPES_H__)
typedef cudaError_t cb200_cuda_status_t;
#else
typedef int cb200_cuda_status_t;          /* cudaError_t: an int-sized enum, 0 = cudaSuccess */
#endif
#define CB200_DECL_CUM(T, sfx) \
    cb200_cuda_status_t cumo_##T##_cumsum##sfx##_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n); \
    cb200_cuda_status_t cumo_##T##_cumprod##sfx##_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n);
CB200_DECL_CUM(sfloat, ) CB200_DECL_CUM(dfloat, ) CB200_DECL_CUM(int32, ) CB200_DECL_CUM(int64, )
CB200_DECL_CUM(sfloat, _nan) CB200_DECL_CUM(dfloat, _nan)

/* The same scans over MANY runs in one launch: run r (row-major over outer_shape) starts at p1 + sum k_i*outer_step1[i]
 * and writes from p2 + sum k_i*outer_step2[i]; s1, s2, n describe every run as above.  NOT in the reference, whose
 * ndloop calls the functions above once per run (gen/tmpl/cum.c:9-24): `cumsum(axis: 1)` of a 65536 x 2048 array is
 * 65536 calls.  The outer arrays are host arrays. */
#define CB200_DECL_CUM_RUNS(T, sfx) \
    cb200_cuda_status_t cb200_##T##_cumsum##sfx##_runs_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n, int n_outer, const size_t* outer_shape, const ssize_t* outer_step1, const ssize_t* outer_step2); \
    cb200_cuda_status_t cb200_##T##_cumprod##sfx##_runs_kernel_launch(char* p1, char* p2, ssize_t s1, ssize_t s2, uint64_t n, int n_outer, const size_t* outer_shape, const ssize_t* outer_step1, const ssize_t* outer_step2);
CB200_DECL_CUM_RUNS(sfloat, ) CB200_DECL_CUM_RUNS(dfloat, ) CB200_DECL_CUM_RUNS(int32, ) CB200_DECL_CUM_RUNS(int64, )
CB200_DECL_CUM_RUNS(sfloat, _nan) CB200_DECL_CUM_RUNS(dfloat, _nan)

/* Bit#where / where2, reference: gen/tmpl_bit/where.c:11-12, where_kernel.cu:83-110.  One call of
 * cumo_bit_where_scratch_new() per result (device memory from cumo_cuda_runtime_malloc, freed by the caller with
 * cumo_cuda_runtime_free), then one launch per run of the Bit array: element i of the run (bit p + i*s of `a`, or
 * p + idx[i]) that is one (invert: zero) appends `count + i` to `out` (elmsz 4: int32_t, 8: int64_t) at a cursor kept
 * in the scratch, so successive launches continue where the last one stopped. */
char* cumo_bit_where_scratch_new(void);
void cumo_bit_where_kernel_launch(CUMO_BIT_DIGIT* a, size_t p, ssize_t s, size_t* idx, uint64_t n, int invert, char* out,
                                  size_t elmsz, uint64_t count, char* scratch);

/* Bit#mask, reference: gen/tmpl_bit/mask.c:1, mask_kernel.cu:38-53.  The compaction of where, but a one at element
 * i of the run (bit p + i*s of `a`, or p + idx[i]) appends to `out` the BYTE position of element i of the masked
 * array: p2 + i*s2, or p2 + idx2[i].  `scratch` is a cumo_bit_where_scratch_new() block whose first cursor carries
 * the output position from one launch to the next. */
void cumo_bit_mask_kernel_launch(CUMO_BIT_DIGIT* a, size_t p, ssize_t s, size_t* idx, uint64_t n, size_t* out, size_t p2,
                                 ssize_t s2, size_t* idx2, char* scratch);

/* Single-precision matrix product on the tensor cores: C[M,N] = A[M,K] . Bt[N,K]^T, all row-major, leading
 * dimensions in elements.  Stands where the reference calls cublasSgemm for `a.dot(b)` on 2-D SFloat operands
 * (ext/cumo/narray/gen/tmpl/gemm.c:252-297); the reference has no kernel-launch entry of its own for it.
 * TF32 instructions with every operand split in two, fp32 accumulation: fp32-grade results.  K, lda, ldb must be
 * multiples of 4 and A, Bt 16-byte aligned.  Returns 0, or an error code with the reason in errbuf (1: shape or
 * alignment, nothing launched; 3/4: launch; 5: an in-kernel bounded wait ran out).  Synchronises the stream. */
int cb200_sgemm_nt_tc(int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* Bt, int64_t ldb,
                      float* C, int64_t ldc, char* errbuf, size_t errlen);

/* Rank-order folds of per-GPU partials (no counterpart in the reference, which has no multi-GPU code): the last
 * step of a row-sharded reduction.  The partials of all ranks lie `rank_stride` bytes apart (an all_gather's
 * output), n_out values per rank.
 *   sum: partials of the element type are added in float64 in rank order, divided by `divisor` unless it is 0
 *        (mean), rounded once to the element type;
 *   extreme: min (is_max == 0) or max of the per-rank answers with the single-GPU rules (nan_wins == 0: a NaN loses unless
 *        all are NaN; else a NaN wins);
 *   arg: {values[r][o], indices[r][o]} pairs are merged with the single-GPU kernels' own total order (NaN rule,
 *        better value, lower index), out_value may be NULL.  Indices are int64_t. */
void cb200_sfloat_rank_fold_sum_kernel_launch(const char* partials, int64_t rank_stride, int world, int64_t n_out, double divisor, char* out);
void cb200_dfloat_rank_fold_sum_kernel_launch(const char* partials, int64_t rank_stride, int world, int64_t n_out, double divisor, char* out);
#define CB200_DECL_FOLD_ARG(T) \
    void cb200_##T##_rank_fold_arg_kernel_launch(const char* indices, const char* values, int64_t rank_stride, int world, int64_t n_out, \
                                                 int is_max, int nan_wins, int64_t* out_index, char* out_value);
CB200_DECL_FOLD_ARG(sfloat) CB200_DECL_FOLD_ARG(dfloat) CB200_DECL_FOLD_ARG(int32) CB200_DECL_FOLD_ARG(int64)
#define CB200_DECL_FOLD_EXTREME(T) \
    void cb200_##T##_rank_fold_extreme_kernel_launch(const char* partials, int64_t rank_stride, int world, int64_t n_out, int is_max, \
                                                     int nan_wins, char* out);
CB200_DECL_FOLD_EXTREME(sfloat) CB200_DECL_FOLD_EXTREME(dfloat) CB200_DECL_FOLD_EXTREME(int32) CB200_DECL_FOLD_EXTREME(int64)

/* General matrix product with the argument list of cublas<T>gemmStridedBatched minus the handle (column-major:
 * C (m x n, ldc) = alpha * op(A) * op(B) + beta * C for `batch` entries `stride*` elements apart; transa/transb 0 = N,
 * 1 = T, 2 = C; alpha, beta host pointers).  Stands where the reference's host template calls cuBLAS for `dot`
 * (ext/cumo/narray/gen/tmpl/gemm.c:277-296); the reference has no launch function of its own for it.  Single precision
 * with alpha 1, beta 0 and K a multiple of 4 runs on the tensor cores (cb200_sgemm_nt_tc, an operand that is not
 * K-contiguous is copied transposed first); everything else, double precision included, on the CUDA cores.
 * Returns 0, 7 (invalid value) or 13 (execution failed), the cublasStatus_t codes. */
int cb200_sgemm_strided_batched(int transa, int transb, int m, int n, int k, const float* alpha, const float* A, int lda, long long strideA,
                                const float* B, int ldb, long long strideB, const float* beta, float* C, int ldc, long long strideC, int batch);
int cb200_dgemm_strided_batched(int transa, int transb, int m, int n, int k, const double* alpha, const double* A, int lda, long long strideA,
                                const double* B, int ldb, long long strideB, const double* beta, double* C, int ldc, long long strideC, int batch);

/* kahan_sum exists for the double-precision type only (reference: gen/spec.rb:321-323,
 * float_accum_kernel.cu:196-206). */
CB200_DECL_ACCUM(dfloat, double, kahan_sum)
CB200_DECL_ACCUM(dfloat, double, kahan_sum_nan)

/* Bit population counts, reference: gen/tmpl_bit/bit_count.c:4-7, bit_count_kernel.cu:48-78.
 * p1: bit position of the first element; a1: first word; s1: bit step; n: number of
 * bits looked at.  `stride`: *(uint64_t*)p2 += matches.  `stride_stride`:
 * *(uint64_t*)(p2 + i*s2) += 1 for each matching bit i.  The `index` forms read the
 * bit offsets from a device array of n size_t instead of using a step. */
#define CB200_DECL_BITCOUNT(name) \
    void cumo_iter_bit_##name##_index_kernel_launch(size_t p1, char* p2, CUMO_BIT_DIGIT* a1, size_t* idx1, uint64_t n); \
    void cumo_iter_bit_##name##_stride_kernel_launch(size_t p1, char* p2, CUMO_BIT_DIGIT* a1, ssize_t s1, uint64_t n); \
    void cumo_iter_bit_##name##_index_stride_kernel_launch(size_t p1, char* p2, CUMO_BIT_DIGIT* a1, size_t* idx1, ssize_t s2, uint64_t n); \
    void cumo_iter_bit_##name##_stride_stride_kernel_launch(size_t p1, char* p2, CUMO_BIT_DIGIT* a1, ssize_t s1, ssize_t s2, uint64_t n);
CB200_DECL_BITCOUNT(count_true)
CB200_DECL_BITCOUNT(count_false)

/* Fused k-means assignment step (no counterpart in the reference, whose benchmark builds it from
 * array operations and materialises the (N, K) distance matrix: bench/kmeans_bench.rb:108-126).
 * x: n points of d float32 (row-major, 16-byte aligned), c: k centroids of d float32.
 * labels[p] = argmin_k ( |c_k|^2 - 2 <x_p, c_k> ), lowest k on ties (the |x_p|^2 term is constant
 * per point and left out, as in the reference's formulation); min_dist (may be NULL) gets that
 * smallest value; counts (may be NULL) gets, ADDED to what it holds, the number of points per
 * cluster (zero it first; integer atomics, exact in any order).  d must be a multiple of 4 and the
 * centroid table must fit shared memory ((k rounded up to 128) * (d + 4) floats + 128 * (d + 4)
 * floats <= 200 KiB).  Returns 0, or non-zero with the reason in errbuf (may be NULL). */
int cb200_kmeans_assign_sfloat(const float* x, int64_t n, int d, const float* c, int k, int32_t* labels,
                               float* min_dist, unsigned long long* counts, char* errbuf, size_t errlen);

/* The same step with the contraction on the tcgen05 tensor cores (TF32 operands split into head and
 * tail, three products accumulated in fp32 in tensor memory: fp32-grade accuracy).  Same arguments
 * and results as cb200_kmeans_assign_sfloat; needs d a multiple of 32, k <= 256 and the centroid
 * table (2 * d * roundup(k,16) * 4 bytes) plus 96 KiB of point slots within 227 KiB of shared memory
 * (d = 64, k = 256 fits).  It reads back a status word, so it synchronises the stream; return 5 means
 * a bounded wait inside the kernel ran out and the outputs are not valid. */
int cb200_kmeans_assign_sfloat_tc(const float* x, int64_t n, int d, const float* c, int k, int32_t* labels,
                                  float* min_dist, unsigned long long* counts, char* errbuf, size_t errlen);

/* Integer `a / s` and `a % s` with a host scalar on the right multiply by a reciprocal that the host derives from the
 * scalar (cumo_iter_<T>_{div,mod}_s_kernel_launch choose that kernel themselves for flat arrays).  These two return the
 * derivation for a magnitude d >= 1 (host code, no GPU): q = (t + ((n - t) >> sh1)) >> sh2 with t = high word of m * n
 * equals n / d for every n up to 2^31 (u32) / 2^63 (u64). */
void cb200_invariant_divisor_u32(uint32_t d, uint32_t* m, int* sh1, int* sh2);
void cb200_invariant_divisor_u64(uint64_t d, uint64_t* m, int* sh1, int* sh2);

/* All-gather of a few KiB per GPU through peer memory: the exchange step of a row-sharded reduction (no counterpart in the
 * reference, which has no multi-GPU code).  One process per GPU on one box.  Each rank creates a buffer and hands its
 * 64-byte handle to the others (any host channel); each opens the others' handles; then, per reduction, every rank calls
 * cb200_peer_exchange_kernel_launch with the same sequence number (1, 2, 3, ... per set of buffers): a small kernel stores
 * the rank's partial into slot [rank] of every buffer, raises a flag at every peer and waits, bounded, for every peer's
 * flag.  Kernels queued behind it on the stream find all partials in local memory at
 *     bases[rank] + (seq & 1) * world * slot_bytes + r * slot_bytes,   r = 0 .. world-1
 * (the layout cb200_<T>_rank_fold_*_kernel_launch take, rank_stride = slot_bytes).  No kernel loads from peer memory.
 * `status` (device-writable int) receives 1 when a wait ran out after `spin_limit` polls (0 = the default, about ten
 * seconds): the gathered data is then not valid.  All return 0 or a cudaError_t value. */
size_t cb200_peer_buffer_bytes(size_t slot_bytes, int world);
int cb200_peer_buffer_create(size_t slot_bytes, int world, void** base_out, unsigned char* handle_out /* [64] */);
int cb200_peer_buffer_open(const unsigned char* handle /* [64] */, void** ptr_out);
int cb200_peer_buffer_close(void* ptr);
int cb200_peer_buffer_destroy(void* base);
int cb200_peer_exchange_kernel_launch(const void* src, size_t nbytes, void* const* bases, int world, int rank, size_t slot_bytes,
                                      unsigned long long seq, unsigned spin_limit, int* status);
/* The same exchange with the rank fold done by the same kernel, for the folds that work element by element: a CTA folds the
 * slice it exchanged as soon as its peers' flags for that slice are up.  op 0 = sum (float types; float64 accumulation in rank
 * order, `divisor` as in cb200_<T>_rank_fold_sum_kernel_launch), 1 = min, 2 = max (`nan_wins` as in the extreme fold);
 * dtype 0 sfloat, 1 dfloat, 2 int32, 3 int64; `src` holds this rank's n_out partials, `out` receives the n_out results. */
int cb200_peer_exchange_fold_kernel_launch(const void* src, int dtype, int op, int64_t n_out, double divisor, int nan_wins, void* out,
                                           void* const* bases, int world, int rank, size_t slot_bytes, unsigned long long seq,
                                           unsigned spin_limit, int* status);
/* ... and for index reductions: `src` holds this rank's n_out int64 global indices followed, `val_off` bytes in (a multiple
 * of 16), by the n_out winning values (what cb200_<T>_<op>_with_value_kernel_launch writes), both parts readable to the next
 * multiple of 16 bytes; `out_index` receives the indices merged with the single-GPU total order. */
int cb200_peer_exchange_arg_kernel_launch(const void* src, int dtype, int64_t n_out, size_t val_off, int is_max, int nan_wins, int64_t* out_index,
                                          void* const* bases, int world, int rank, size_t slot_bytes, unsigned long long seq,
                                          unsigned spin_limit, int* status);

/* Self-test of the bounded mbarrier wait the tcgen05 kernels use between their warp roles (no counterpart in the
 * reference): one CTA waits at most `spin_limit` polls on a barrier nothing arrives at.  Returns 5 when the wait gave
 * up by its limit -- the code cb200_sgemm_nt_tc / cb200_kmeans_assign_sfloat_tc return in that case -- 0 if the barrier
 * completed, 3/4 on launch problems.  The kernel always returns; the context stays usable. */
int cb200_selftest_bounded_wait(unsigned spin_limit, char* errbuf, size_t errlen);

/* Bit o Bit operations and the all? / any? reductions (reference: gen/tmpl_bit/binary.c:1-2, unary.c:1-2,
 * bit_reduce.c:1-3; kernels in binary_kernel.cu, unary_kernel.cu, bit_reduce_kernel.cu).  The `_contiguous` forms take, per
 * operand, the word that holds its first bit and that bit's position in the word (0..31), and n bits that lie end to end;
 * the general forms address every operand per dimension by a bit step or an index array.  For the reductions the output
 * bit(s) must hold the identity on entry (1 for all?, 0 for any?): `elementwise` folds run i of the input into output bit i,
 * `reduce` and `contiguous_reduce` fold n input bits into the one bit at p2. */
#define CB200_DECL_BIT_BINARY(op) \
    void cumo_iter_bit_##op##_kernel_launch(cumo_na_bit_iarray_stridx_t* a1, cumo_na_bit_iarray_stridx_t* a2, cumo_na_bit_iarray_stridx_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_bit_##op##_contiguous_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, CUMO_BIT_DIGIT* a2, size_t p2, CUMO_BIT_DIGIT* a3, size_t p3, uint64_t n);
#define CB200_DECL_BIT_UNARY(op) \
    void cumo_iter_bit_##op##_kernel_launch(cumo_na_bit_iarray_stridx_t* a1, cumo_na_bit_iarray_stridx_t* a3, cumo_na_indexer_t* indexer); \
    void cumo_iter_bit_##op##_contiguous_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, CUMO_BIT_DIGIT* a3, size_t p3, uint64_t n);
#define CB200_DECL_BIT_REDUCE(op) \
    void cumo_iter_bit_##op##_elementwise_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, ssize_t s1, size_t* idx1, CUMO_BIT_DIGIT* a2, size_t p2, ssize_t s2, size_t* idx2, uint64_t n); \
    void cumo_iter_bit_##op##_reduce_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, ssize_t s1, size_t* idx1, CUMO_BIT_DIGIT* a2, size_t p2, uint64_t n); \
    void cumo_iter_bit_##op##_contiguous_reduce_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, CUMO_BIT_DIGIT* a2, size_t p2, uint64_t n);
CB200_DECL_BIT_BINARY(and) CB200_DECL_BIT_BINARY(or) CB200_DECL_BIT_BINARY(xor) CB200_DECL_BIT_BINARY(eq)
CB200_DECL_BIT_UNARY(copy) CB200_DECL_BIT_UNARY(not)
CB200_DECL_BIT_REDUCE(all_p) CB200_DECL_BIT_REDUCE(any_p)

/* count_true / count_false along some axes, every output in one launch.  NOT in the reference, whose ndloop calls the
 * four functions above once per innermost run (gen/tmpl_bit/bit_count.c:9-36: one launch per row of a per-axis
 * count).  The bits of output k = (k_0 .. k_{n_keep-1}) are p1 + sum k_i*keep_bit_step[i] + sum r_j*red_bit_step[j]
 * over all r; the number of ones (zeros when want_false) among them is ADDED to the uint64_t at
 * out + sum k_i*keep_out_step[i], which the caller has filled with 0 as ndloop's `init` argument does.  The shape and
 * step arrays are host arrays. */
void cb200_bit_count_axes_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, int want_false,
                                        int n_keep, const size_t* keep_shape, const ssize_t* keep_bit_step, const ssize_t* keep_out_step,
                                        int n_red, const size_t* red_shape, const ssize_t* red_bit_step, char* out);

/* Conversions between Bit and value arrays, and Bit#fill.  Every operand is addressed per dimension by a step or an
 * index array (cumo_na_iarray_stridx_t: byte steps; cumo_na_bit_iarray_stridx_t: bit steps).
 * value <- Bit (0 or 1 in the element type), reference: gen/tmpl/store_bit.c:2, store_bit_kernel.cu:14-30.
 * Bit <- value (set where the value is not zero; a NaN sets it), one per source class as the reference instantiates
 * them (gen/spec.rb:125-139), reference: gen/tmpl_bit/store_from.c:2, store_from_kernel.cu:14-29.
 * Bit <- Bit, reference: gen/tmpl_bit/store_bit.c:1-2, store_bit_kernel.cu:22-46 (same argument lists as `copy`).
 * fill, reference: gen/tmpl_bit/fill.c:1-2, fill_kernel.cu:21-41: every addressed bit takes the low bit of y. */
#define CB200_DECL_STORE_BIT(T) \
    void cumo_iter_##T##_store_bit_kernel_launch(cumo_na_iarray_stridx_t* a1, cumo_na_bit_iarray_stridx_t* a2, cumo_na_indexer_t* indexer);
#define CB200_DECL_BIT_STORE(S) \
    void cumo_iter_bit_store_##S##_kernel_launch(cumo_na_bit_iarray_stridx_t* a1, cumo_na_iarray_stridx_t* a2, cumo_na_indexer_t* indexer);
CB200_DECL_STORE_BIT(sfloat) CB200_DECL_STORE_BIT(dfloat) CB200_DECL_STORE_BIT(int32) CB200_DECL_STORE_BIT(int64)
CB200_DECL_BIT_STORE(dfloat) CB200_DECL_BIT_STORE(sfloat) CB200_DECL_BIT_STORE(int64) CB200_DECL_BIT_STORE(int32)
CB200_DECL_BIT_STORE(int16) CB200_DECL_BIT_STORE(int8) CB200_DECL_BIT_STORE(uint64) CB200_DECL_BIT_STORE(uint32)
CB200_DECL_BIT_STORE(uint16) CB200_DECL_BIT_STORE(uint8)
CB200_DECL_BIT_UNARY(store_bit)
void cumo_iter_bit_fill_kernel_launch(cumo_na_bit_iarray_stridx_t* a3, CUMO_BIT_DIGIT y, cumo_na_indexer_t* indexer);
void cumo_iter_bit_fill_contiguous_kernel_launch(CUMO_BIT_DIGIT* a3, size_t p3, uint64_t n, CUMO_BIT_DIGIT y);

/* Elementwise operations on operands whose contiguous axes differ (`a + b.transpose`, `b.transpose.dup`, a cast of a
 * transposed view; reference: the strided branches of binary_kernel.cu:14-49, unary_kernel.cu:14-25, store_from_kernel.cu)
 * run, when every operand is 16-byte aligned, in a kernel whose input tiles are copied into shared memory by the tensor
 * memory accelerator several tiles ahead of the warps that use them.  Its waits are bounded; the launch functions return
 * void, so the outcome is kept in a status word:
 *   cb200_tile_pipeline_status(): 0 = no wait ran out on the current device since the last call, 1 = one did and that
 *     launch's output is not valid, 2 = the kernel found its shared memory misaligned and wrote nothing, -1 = the word
 *     could not be read.  Synchronises the device and clears the word.
 *   cb200_tile_pipeline_launches(): launches of that kernel in this process.
 * CB200_TILE_TMA in the environment: 0 sends such operands through the register-staged tile kernels, 1 through this
 * kernel whenever it can take them; unset, each goes where it measured faster (8-byte elements and planes up to
 * 256 MiB here). */
int cb200_tile_pipeline_status(void);
unsigned long long cb200_tile_pipeline_launches(void);

/* float32 `sum` that allocates nothing (no counterpart in the reference, whose reductions
 * always take scratch from cumo_cuda_runtime_malloc).  For callers that cannot reach an
 * allocator when they need the sum: a finalizer or other context in which the Ruby
 * extension's pool callback must not run the GC or raise, an embedder that handed out all
 * device memory at start-up, a loop that must not take the allocator's lock.  Same kernels
 * as cumo_sfloat_sum_kernel_launch, with the [output][segment] partial sums in a fixed 1 MiB
 * array inside the library image instead.  Its plan always cuts long rows into 32 KiB
 * segments, so its sums agree with the regular entry point's to fp32 rounding (<= 1e-5
 * relative to a float64 sum), not bit for bit.
 *   - accepts only reductions whose reduced axes form one contiguous run (a full sum of a
 *     contiguous array, sums along the last axes); needs outputs x segments <= 262144
 *     (a row is cut into 32 KiB segments, at most 8192 per row);
 *   - returns 0 on success; otherwise nothing was launched and `errbuf` (may be NULL)
 *     holds the reason: 1 layout not supported, 2 scratch too small for this shape,
 *     3 the scratch address could not be looked up, 4 the launch itself failed;
 *   - calls no cudaMalloc/cudaFree and no allocating library routine; launches on the
 *     stream cb200_set_stream chose and does not call cumo_cuda_runtime_check_kernel_launch;
 *   - all calls on a device share the array: calls whose kernels may overlap on the GPU
 *     race on it, so keep them on one stream; nothing in it needs clearing between calls;
 *   - the first call on each device, whatever its shape, looks up the array's address with
 *     that device current (cudaGetSymbolAddress): make that first call before any stream
 *     capture begins. */
int cb200_sfloat_sum_noalloc_kernel_launch(cumo_na_reduction_arg_t* arg, char* errbuf, size_t errlen);

#ifdef __cplusplus
}
#endif
#endif /* CUMO_B200_H */
