/*
 * TEST INFRASTRUCTURE -- CPU oracle for the libcumo_b200 parity tests and the
 * CPU-baseline leg of bench.py.  Nothing in the product may call into this file.
 *
 * It restates, as plain sequential C (OpenMP only across independent outputs /
 * rows), the host loops that the reference keeps for its CPU path and inherited
 * from Numo: elementwise loop shape and broadcasting
 * (ext/cumo/narray/gen/tmpl/binary.c:22-112, unary.c:9-74), per-type operation
 * macros (ext/cumo/include/cumo/types/float_macro.h:26-142, xint_macro.h:15-47,
 * int_macro.h:3-67), reductions (types/real_accum.h:25-441, float_macro.h:150-193),
 * Bit counting (ext/cumo/narray/gen/tmpl_bit/bit_count_cpu.c:4-67).  The per-type
 * bodies are in oracle_type.inc, which cites the lines each function follows.
 *
 * Pinning: tests/test_oracle_golden.py checks this oracle against the literal
 * expectations of the reference's own test suite (tests/golden/reference_cases.py
 * transcribes them with file:line).  The reference itself (a CRuby extension
 * generated from ERB templates) cannot be built or run here: no Ruby.
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp, no -ffast-math).
 */
#define _GNU_SOURCE
#include <math.h>
#include <float.h>
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { DT_SFLOAT = 0, DT_DFLOAT = 1, DT_INT32 = 2, DT_INT64 = 3 };
enum { KIND_BINARY = 0, KIND_UNARY = 1, KIND_COMPARE = 2 };

/* operation codes shared with oracle/cumo_oracle.py */
enum {
    OP_ADD = 0, OP_SUB, OP_MUL, OP_DIV, OP_MOD, OP_POW, OP_COPYSIGN, OP_ATAN2, OP_HYPOT, OP_LDEXP,
    OP_MAXIMUM, OP_MINIMUM, OP_MAXIMUM_NAN, OP_MINIMUM_NAN,
    OP_BIT_AND, OP_BIT_OR, OP_BIT_XOR, OP_LEFT_SHIFT, OP_RIGHT_SHIFT,
    OP_MINUS = 100, OP_RECIPROCAL, OP_SIGN, OP_SQUARE, OP_ABS, OP_FLOOR, OP_ROUND, OP_CEIL, OP_TRUNC, OP_RINT,
    OP_BIT_NOT,
    OP_SQRT, OP_CBRT, OP_LOG, OP_LOG2, OP_LOG10, OP_EXP, OP_EXP2, OP_EXP10, OP_SIN, OP_COS, OP_TAN,
    OP_ASIN, OP_ACOS, OP_ATAN, OP_SINH, OP_COSH, OP_TANH, OP_ASINH, OP_ACOSH, OP_ATANH, OP_SINC,
    OP_ERF, OP_ERFC, OP_LOG1P, OP_EXPM1,
    OP_EQ = 200, OP_NE, OP_GT, OP_GE, OP_LT, OP_LE, OP_NEARLY_EQ,
    OP_ISNAN, OP_ISINF, OP_ISPOSINF, OP_ISNEGINF, OP_ISFINITE, OP_SIGNBIT
};
enum {
    RED_SUM = 0, RED_PROD, RED_MEAN, RED_MIN, RED_MAX, RED_PTP, RED_MINMAX,
    RED_MIN_INDEX, RED_MAX_INDEX, RED_ARGMIN, RED_ARGMAX, RED_VAR, RED_STDDEV, RED_RMS, RED_KAHAN
};

/* clip / divmod / modf / frexp / seq (multi_flat in oracle_type.inc) */
enum { MULTI_CLIP = 0, MULTI_CLIP_MIN, MULTI_CLIP_MAX, MULTI_DIVMOD, MULTI_MODF, MULTI_FREXP, MULTI_SEQ };

#define TN sfloat
#define DT float
#define ACC float
#define IS_FP 1
#define EPS_V FLT_EPSILON
#include "oracle_type.inc"
#undef TN
#undef DT
#undef ACC
#undef IS_FP
#undef EPS_V

#define TN dfloat
#define DT double
#define ACC double
#define IS_FP 1
#define EPS_V DBL_EPSILON
#include "oracle_type.inc"
#undef TN
#undef DT
#undef ACC
#undef IS_FP
#undef EPS_V

#define TN int32
#define DT int32_t
#define UDT uint32_t
#define ACC int64_t
#define IS_FP 0
#define DATA_MIN_V INT32_MIN
#include "oracle_type.inc"
#undef TN
#undef DT
#undef UDT
#undef ACC
#undef IS_FP
#undef DATA_MIN_V

#define TN int64
#define DT int64_t
#define UDT uint64_t
#define ACC int64_t
#define IS_FP 0
#define DATA_MIN_V INT64_MIN
#include "oracle_type.inc"
#undef TN
#undef DT
#undef UDT
#undef ACC
#undef IS_FP
#undef DATA_MIN_V

/* ---- exported API ------------------------------------------------------------------------ */

/* kind: KIND_BINARY / KIND_UNARY / KIND_COMPARE.  Steps are in bytes (bits for the Bit
 * output of a comparison).  a == NULL or b == NULL: that operand is the scalar `sv`
 * (passed as double and as int64; the one matching the dtype is used). */
int oracle_elementwise(int dtype, int kind, int op, int ndim, const int64_t* shape,
                       const char* a, const int64_t* sa, const char* b, const int64_t* sb,
                       char* c, const int64_t* sc, double sv_f, int64_t sv_i, int* flag,
                       uint32_t* bits, uint64_t bitpos) {
    switch (dtype) {
    case DT_SFLOAT: return ew_loop_sfloat(kind, op, ndim, shape, a, sa, b, sb, c, sc, (float)sv_f, flag, bits, bitpos);
    case DT_DFLOAT: return ew_loop_dfloat(kind, op, ndim, shape, a, sa, b, sb, c, sc, sv_f, flag, bits, bitpos);
    case DT_INT32:  return ew_loop_int32(kind, op, ndim, shape, a, sa, b, sb, c, sc, (int32_t)sv_i, flag, bits, bitpos);
    case DT_INT64:  return ew_loop_int64(kind, op, ndim, shape, a, sa, b, sb, c, sc, sv_i, flag, bits, bitpos);
    }
    return -1;
}

int oracle_pow_int32(int dtype, int ndim, const int64_t* shape, const char* a, const int64_t* sa,
                     const char* b, const int64_t* sb, char* c, const int64_t* sc, double base_f,
                     int64_t base_i, int32_t sv_exp) {
    switch (dtype) {
    case DT_SFLOAT: pow_int32_loop_sfloat(ndim, shape, a, sa, b, sb, c, sc, (float)base_f, sv_exp); return 0;
    case DT_DFLOAT: pow_int32_loop_dfloat(ndim, shape, a, sa, b, sb, c, sc, base_f, sv_exp); return 0;
    case DT_INT32:  pow_int32_loop_int32(ndim, shape, a, sa, b, sb, c, sc, (int32_t)base_i, sv_exp); return 0;
    case DT_INT64:  pow_int32_loop_int64(ndim, shape, a, sa, b, sb, c, sc, base_i, sv_exp); return 0;
    }
    return -1;
}

/* clip / clip_min / clip_max / divmod / modf / frexp / seq over contiguous arrays of n elements (op: the MULTI_
 * codes of oracle_type.inc); operands an operation does not use are NULL. */
int oracle_multi(int dtype, int op, int64_t n, const void* x, const void* y, const void* z, void* o0, void* o1,
                 double beg, double step, double count, int* flag) {
    switch (dtype) {
    case DT_SFLOAT: return multi_flat_sfloat(op, n, x, y, z, o0, o1, beg, step, count, flag);
    case DT_DFLOAT: return multi_flat_dfloat(op, n, x, y, z, o0, o1, beg, step, count, flag);
    case DT_INT32:  return multi_flat_int32(op, n, x, y, z, o0, o1, beg, step, count, flag);
    case DT_INT64:  return multi_flat_int64(op, n, x, y, z, o0, o1, beg, step, count, flag);
    }
    return -1;
}

/* out dims (oshape, in_ostep, out_step[, out2_step]) and reduce dims (rshape, in_rstep),
 * all steps in bytes.  idx64 selects the output width of the index reductions. */
int oracle_reduce(int dtype, int op, int nan, int n_od, const int64_t* oshape, const int64_t* in_ostep,
                  const int64_t* out_step, const int64_t* out2_step, int n_rd, const int64_t* rshape,
                  const int64_t* in_rstep, const char* in, char* out, char* out2, int idx64) {
    switch (dtype) {
    case DT_SFLOAT: reduce_all_sfloat(op, nan, n_od, oshape, in_ostep, out_step, out2_step, n_rd, rshape, in_rstep, in, out, out2, idx64); return 0;
    case DT_DFLOAT: reduce_all_dfloat(op, nan, n_od, oshape, in_ostep, out_step, out2_step, n_rd, rshape, in_rstep, in, out, out2, idx64); return 0;
    case DT_INT32:  reduce_all_int32(op, 0, n_od, oshape, in_ostep, out_step, out2_step, n_rd, rshape, in_rstep, in, out, out2, idx64); return 0;
    case DT_INT64:  reduce_all_int64(op, 0, n_od, oshape, in_ostep, out_step, out2_step, n_rd, rshape, in_rstep, in, out, out2, idx64); return 0;
    }
    return -1;
}

int oracle_mulsum(int dtype, int nan, const char* p1, const char* p2, char* p3, int64_t s1, int64_t s2, int64_t s3, int64_t n) {
    switch (dtype) {
    case DT_SFLOAT: mulsum_sfloat(nan, p1, p2, p3, s1, s2, s3, n); return 0;
    case DT_DFLOAT: mulsum_dfloat(nan, p1, p2, p3, s1, s2, s3, n); return 0;
    case DT_INT32:  mulsum_int32(0, p1, p2, p3, s1, s2, s3, n); return 0;
    case DT_INT64:  mulsum_int64(0, p1, p2, p3, s1, s2, s3, n); return 0;
    }
    return -1;
}

/* Bits at pos + i*step, i < n, LSB-first in 32-bit words (narray.h:492-496).  The
 * contiguous case counts whole words the way bit_count_cpu.c:4-67 does. */
uint64_t oracle_bit_count(const uint32_t* words, uint64_t pos, int64_t step, uint64_t n, int want_false) {
    uint64_t c = 0;
    if (step == 1) {
        uint64_t i = 0;
        while (i < n && ((pos + i) & 31)) { c += (words[(pos + i) >> 5] >> ((pos + i) & 31)) & 1u; ++i; }
        for (; i + 32 <= n; i += 32) c += (uint64_t)__builtin_popcount(words[(pos + i) >> 5]);
        for (; i < n; ++i) c += (words[(pos + i) >> 5] >> ((pos + i) & 31)) & 1u;
    } else {
        for (uint64_t i = 0; i < n; ++i) {
            uint64_t b = pos + (uint64_t)((int64_t)i * step);
            c += (words[b >> 5] >> (b & 31)) & 1u;
        }
    }
    return want_false ? n - c : c;
}

/* float64 reference sum for tolerance checks: pairwise, so that its own error is
 * far below the 1e-12 the double-precision kernels are held to. */
static double pairwise_f64(const double* p, int64_t n) {
    if (n <= 64) { double s = 0; for (int64_t i = 0; i < n; ++i) s += p[i]; return s; }
    int64_t h = n / 2;
    return pairwise_f64(p, h) + pairwise_f64(p + h, n - h);
}
static double pairwise_f32(const float* p, int64_t n) {
    if (n <= 64) { double s = 0; for (int64_t i = 0; i < n; ++i) s += (double)p[i]; return s; }
    int64_t h = n / 2;
    return pairwise_f32(p, h) + pairwise_f32(p + h, n - h);
}
double oracle_sum_f64ref(int dtype, const char* p, int64_t n) {
    return dtype == DT_SFLOAT ? pairwise_f32((const float*)p, n) : pairwise_f64((const double*)p, n);
}

/* k-means assignment (the step of bench/kmeans_bench.rb:108-126: d = |c|^2 - 2 x.c, then the index
 * of the row minimum, lowest index on ties) evaluated in float64 from the float32 inputs, together
 * with the winning value and the runner-up's, so that a caller can tell a genuine disagreement from
 * a near-tie that float32 rounding may decide either way. */
void oracle_kmeans_assign(const float* x, int64_t n, int d, const float* c, int k, int32_t* labels,
                          double* best, double* second) {
    #pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < n; ++p) {
        double b = INFINITY, s = INFINITY;
        int32_t bk = 0;
        for (int kk = 0; kk < k; ++kk) {
            double dot = 0, cn = 0;
            for (int q = 0; q < d; ++q) {
                double cv = c[(int64_t)kk * d + q];
                dot += (double)x[p * d + q] * cv;
                cn += cv * cv;
            }
            double dist = cn - 2 * dot;
            if (dist < b) { s = b; b = dist; bk = kk; }
            else if (dist < s) s = dist;
        }
        labels[p] = bk;
        if (best) best[p] = b;
        if (second) second[p] = s;
    }
}

/* bincount along one run: the host loop the reference runs for small inputs is the same arithmetic as its
 * kernel (narray/gen/tmpl/bincount_kernel.cu:32-45 counts, :80-88 weighted): clear, then out[x] += 1 or w[i];
 * an item outside [0, n) is reported and skipped.  in64: items are int64_t (else int32_t).  kind: 0 uint32
 * counts, 1 uint64 counts, 2 float weights and sums, 3 double.  Steps in bytes.  Returns 1 when an item was out
 * of range (the last offender in *bad). */
int oracle_bincount(int in64, const char* p1, int64_t s1, int64_t count, int kind, const char* pw, int64_t sw,
                    char* out, int64_t so, int64_t n, int64_t* bad) {
    int oor = 0;
    for (int64_t b = 0; b < n; ++b) {
        if (kind == 0) *(uint32_t*)(out + b * so) = 0;
        else if (kind == 1) *(uint64_t*)(out + b * so) = 0;
        else if (kind == 2) *(float*)(out + b * so) = 0;
        else *(double*)(out + b * so) = 0;
    }
    for (int64_t i = 0; i < count; ++i) {
        int64_t x = in64 ? *(const int64_t*)(p1 + i * s1) : (int64_t)*(const int32_t*)(p1 + i * s1);
        if (x < 0 || x >= n) { oor = 1; if (bad) *bad = x; continue; }
        if (kind == 0) *(uint32_t*)(out + x * so) += 1u;
        else if (kind == 1) *(uint64_t*)(out + x * so) += 1ull;
        else if (kind == 2) *(float*)(out + x * so) += *(const float*)(pw + i * sw);
        else *(double*)(out + x * so) += *(const double*)(pw + i * sw);
    }
    return oor;
}

/* cumsum / cumprod along one run: the host loop of narray/gen/tmpl/cum.c:27-37 with the operators of
 * include/cumo/types/real_accum.h:9-24 (floats) and xint_macro.h:46-47 (integers, wrapping).  dtype: 0 float,
 * 1 double, 2 int32, 3 int64.  Steps in bytes. */
#define ORACLE_CUM_LOOP(T, ISF)                                                              \
    {                                                                                        \
        T x = *(const T*)p1;                                                                 \
        *(T*)p2 = x;                                                                         \
        for (int64_t i = 1; i < n; ++i) {                                                    \
            T y = *(const T*)(p1 + i * s1);                                                  \
            if (ISF && nan) {                                                                \
                if (x != x) x = y;                                                           \
                else if (y == y) x = prod ? (T)(x * y) : (T)(x + y);                         \
            } else x = prod ? (T)(x * y) : (T)(x + y);                                       \
            *(T*)(p2 + i * s2) = x;                                                          \
        }                                                                                    \
    }
int oracle_cum(int dtype, int prod, int nan, const char* p1, char* p2, int64_t s1, int64_t s2, int64_t n) {
    if (n <= 0) return 0;
    if (dtype == 0) ORACLE_CUM_LOOP(float, 1)
    else if (dtype == 1) ORACLE_CUM_LOOP(double, 1)
    else if (dtype == 2) { uint32_t x = *(const uint32_t*)p1; *(uint32_t*)p2 = x;      /* unsigned arithmetic: wraps like the device */
        for (int64_t i = 1; i < n; ++i) { uint32_t y = *(const uint32_t*)(p1 + i * s1); x = prod ? x * y : x + y; *(uint32_t*)(p2 + i * s2) = x; } }
    else if (dtype == 3) { uint64_t x = *(const uint64_t*)p1; *(uint64_t*)p2 = x;
        for (int64_t i = 1; i < n; ++i) { uint64_t y = *(const uint64_t*)(p1 + i * s1); x = prod ? x * y : x + y; *(uint64_t*)(p2 + i * s2) = x; } }
    else return 1;
    return 0;
}

/* Bit#where: the host loop of narray/gen/tmpl_bit/where.c:64-86 over elements given one per byte (0 / non-0),
 * in row-major order: the running element number of every one (invert: zero) bit.  Returns the hit count. */
int64_t oracle_where(const uint8_t* bits, int64_t n, int invert, int64_t* out) {
    int64_t hits = 0;
    for (int64_t count = 0; count < n; ++count) {
        int x = bits[count] != 0;
        if (invert) x = !x;
        if (x) out[hits++] = count;
    }
    return hits;
}

/* Reference value for the single-precision matrix product (the reference delegates it to cuBLAS,
 * narray/gen/tmpl/gemm.c:252-297, so there is no host loop to restate): C = A . Bt^T accumulated in double, plus
 * the sum of |a||b| per element, which bounds the rounding error of any fp32 summation order. */
void oracle_gemm_nt_f64(int64_t M, int64_t N, int64_t K, const float* A, const float* Bt, double* C, double* Cabs) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j) {
            double s = 0, sa = 0;
            for (int64_t k = 0; k < K; ++k) {
                double p = (double)A[i * K + k] * (double)Bt[j * K + k];
                s += p;
                sa += p < 0 ? -p : p;
            }
            C[i * N + j] = s;
            if (Cabs) Cabs[i * N + j] = sa;
        }
}

int oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void oracle_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n > 0 ? n : 1);
#else
    (void)n;
#endif
}
