// Definitions of the elementwise `cumo_iter_<T>_<op>_kernel_launch` entry points
// for one element type.  Included by abi_<type>_ew.cu after defining
//   CB_T      the type's name in symbols (sfloat, dfloat, int32, int64)
//   CB_C      its C type
//   CB_FLOAT  1 for the floating types
// Signatures are the reference's (see include/cumo_b200.h for the file:line of
// each declaration).  A host numeric operand (`sv`) always pairs with the array
// in a1; scalar_is_left says the numeric is the left operand, in which case the
// array becomes the kernel's second input.
#include "elementwise.cuh"
#include "divmod_scalar.cuh"
#include "multi.cuh"
#include "poly_eye.cuh"

using namespace cb200;

#define CB_CAT_(a, b) a##b
#define CB_CAT(a, b) CB_CAT_(a, b)
#define CB_SYM3_(t, name, sfx) cumo_iter_##t##_##name##sfx
#define CB_SYM3(t, name, sfx) CB_SYM3_(t, name, sfx)
#define CB_ITER(name, sfx) CB_SYM3(CB_T, name, sfx)
#define CB_SYM2_(t, name) cumo_##t##_##name##_kernel_launch
#define CB_SYM2(t, name) CB_SYM2_(t, name)
#define CB_PLAIN(name) CB_SYM2(CB_T, name)

#define DEF_BINARY(name, OP)                                                                           \
    extern "C" void CB_ITER(name, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2,           \
            cumo_na_iarray_t* a3, cumo_na_indexer_t* ix, int* divzero) {                                \
        launch_elementwise<op::OP<CB_C>>(a1, a2, a3, ix, CB_C(), CB_C(), 0, divzero);                   \
    }
#define DEF_BINARY_S(name, OP)                                                                         \
    DEF_BINARY(name, OP)                                                                               \
    extern "C" void CB_ITER(name, _s_kernel_launch)(cumo_na_iarray_t* a1, CB_C sv, cumo_na_iarray_t* a3, \
            cumo_na_indexer_t* ix, int* divzero, int scalar_is_left) {                                  \
        if (scalar_is_left) launch_elementwise<op::OP<CB_C>>(nullptr, a1, a3, ix, sv, CB_C(), 2, divzero); \
        else launch_elementwise<op::OP<CB_C>>(a1, nullptr, a3, ix, CB_C(), sv, 1, divzero);             \
    }
// integer division and remainder by a host scalar on the right: the divisor is turned into a multiplier on the host
#define DEF_BINARY_S_DIVMOD(name, OP, IS_MOD)                                                          \
    DEF_BINARY(name, OP)                                                                               \
    extern "C" void CB_ITER(name, _s_kernel_launch)(cumo_na_iarray_t* a1, CB_C sv, cumo_na_iarray_t* a3, \
            cumo_na_indexer_t* ix, int* divzero, int scalar_is_left) {                                  \
        if constexpr (std::is_integral<CB_C>::value) {                                                 \
            if (!scalar_is_left && launch_int_divmod_by_scalar<CB_C, IS_MOD>(a1, sv, a3, ix)) return;  \
        }                                                                                              \
        if (scalar_is_left) launch_elementwise<op::OP<CB_C>>(nullptr, a1, a3, ix, sv, CB_C(), 2, divzero); \
        else launch_elementwise<op::OP<CB_C>>(a1, nullptr, a3, ix, CB_C(), sv, 1, divzero);             \
    }
#define DEF_UNARY(name, OP)                                                                            \
    extern "C" void CB_ITER(name, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2,           \
            cumo_na_indexer_t* ix, int* flag) {                                                         \
        launch_elementwise<op::OP<CB_C>>(a1, nullptr, a2, ix, CB_C(), CB_C(), 0, flag);                 \
    }
#define DEF_MATH(name, OP)                                                                             \
    extern "C" void CB_ITER(math_s_##name, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2,  \
            cumo_na_indexer_t* ix) {                                                                    \
        launch_elementwise<op::OP<CB_C>>(a1, nullptr, a2, ix, CB_C(), CB_C(), 0, nullptr);              \
    }
#define DEF_MATH2(name, OP)                                                                            \
    extern "C" void CB_ITER(math_s_##name, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2,  \
            cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {                                              \
        launch_elementwise<op::OP<CB_C>>(a1, a2, a3, ix, CB_C(), CB_C(), 0, nullptr);                   \
    }                                                                                                  \
    extern "C" void CB_ITER(math_s_##name, _s_kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a3, \
            cumo_na_indexer_t* ix, CB_C sv, int scalar_is_left) {                                       \
        if (scalar_is_left) launch_elementwise<op::OP<CB_C>>(nullptr, a1, a3, ix, sv, CB_C(), 2, nullptr); \
        else launch_elementwise<op::OP<CB_C>>(a1, nullptr, a3, ix, CB_C(), sv, 1, nullptr);             \
    }
#define DEF_COND(name, OP)                                                                             \
    extern "C" void CB_ITER(name, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2,           \
            cumo_na_bit_iarray_t* a3, cumo_na_indexer_t* ix) {                                          \
        launch_compare<op::OP<CB_C>>(a1, a2, a3, ix, CB_C(), CB_C(), 0);                                \
    }                                                                                                  \
    extern "C" void CB_ITER(name, _s_kernel_launch)(cumo_na_iarray_t* a1, CB_C sv, cumo_na_bit_iarray_t* a3, \
            cumo_na_indexer_t* ix, int scalar_is_left) {                                                \
        if (scalar_is_left) launch_compare<op::OP<CB_C>>(nullptr, a1, a3, ix, sv, CB_C(), 2);           \
        else launch_compare<op::OP<CB_C>>(a1, nullptr, a3, ix, CB_C(), sv, 1);                          \
    }
#define DEF_COND_UNARY(name, OP)                                                                       \
    extern "C" void CB_ITER(name, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_bit_iarray_t* a2,       \
            cumo_na_indexer_t* ix) {                                                                    \
        launch_compare<op::OP<CB_C>>(a1, nullptr, a2, ix, CB_C(), CB_C(), 0);                           \
    }
#define DEF_EWCOMP(name, OP)                                                                           \
    extern "C" void CB_PLAIN(name)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3,    \
            cumo_na_indexer_t* ix) {                                                                    \
        launch_elementwise<op::OP<CB_C>>(a1, a2, a3, ix, CB_C(), CB_C(), 0, nullptr);                   \
    }

// store from another element type; a1 is the destination
#define DEF_STORE(from, FC)                                                                            \
    extern "C" void CB_ITER(store_##from, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2,   \
            cumo_na_indexer_t* ix) {                                                                    \
        launch_elementwise<op::Cast<CB_C, FC>>(a2, nullptr, a1, ix, FC(), FC(), 0, nullptr);            \
    }
DEF_STORE(sfloat, float)
DEF_STORE(dfloat, double)
DEF_STORE(int32, int32_t)
DEF_STORE(int64, int64_t)
// the reference instantiates the store template once per source class in every destination type
// (gen/spec.rb:121-140), so the narrow and unsigned integers are sources here too
DEF_STORE(int16, int16_t)
DEF_STORE(int8, int8_t)
DEF_STORE(uint64, uint64_t)
DEF_STORE(uint32, uint32_t)
DEF_STORE(uint16, uint16_t)
DEF_STORE(uint8, uint8_t)

DEF_BINARY_S(add, Add)
DEF_BINARY_S(sub, Sub)
DEF_BINARY_S(mul, Mul)
DEF_BINARY_S_DIVMOD(div, Div, false)
DEF_BINARY_S_DIVMOD(mod, Mod, true)
DEF_UNARY(minus, Minus)
DEF_UNARY(reciprocal, Reciprocal)
DEF_UNARY(sign, Sign)
DEF_UNARY(square, Square)
DEF_UNARY(abs, Abs)
DEF_COND(eq, Eq)
DEF_COND(ne, Ne)
DEF_COND(gt, Gt)
DEF_COND(ge, Ge)
DEF_COND(lt, Lt)
DEF_COND(le, Le)
DEF_EWCOMP(maximum, Maximum)
DEF_EWCOMP(minimum, Minimum)

// power: dtype exponent, and Int32 exponent by repeated multiplication
extern "C" void CB_ITER(pow, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    launch_elementwise<op::Pow<CB_C>>(a1, a2, a3, ix, CB_C(), CB_C(), 0, nullptr);
}
extern "C" void CB_ITER(pow, _s_kernel_launch)(cumo_na_iarray_t* a1, CB_C sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix, int scalar_is_left) {
    if (scalar_is_left) launch_elementwise<op::Pow<CB_C>>(nullptr, a1, a3, ix, sv, CB_C(), 2, nullptr);
    else launch_elementwise<op::Pow<CB_C>>(a1, nullptr, a3, ix, CB_C(), sv, 1, nullptr);
}
extern "C" void CB_ITER(pow_int32, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    launch_elementwise<op::PowInt32<CB_C>>(a1, a2, a3, ix, CB_C(), 0, 0, nullptr);
}
extern "C" void CB_ITER(pow_int32, _s_kernel_launch)(cumo_na_iarray_t* a1, int32_t sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    launch_elementwise<op::PowInt32<CB_C>>(a1, nullptr, a3, ix, CB_C(), sv, 1, nullptr);
}
extern "C" void CB_ITER(pow_int32, _s_left_kernel_launch)(CB_C sv_base, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    launch_elementwise<op::PowInt32<CB_C>>(nullptr, a2, a3, ix, sv_base, 0, 2, nullptr);
}

// clip: one bound through the two-input kernels, two numeric bounds as a one-input operation carrying both
// scalars, two arrays of bounds through the three-input kernel (which can refuse an empty range)
extern "C" void CB_ITER(clip_min, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    launch_elementwise<op::ClipLow<CB_C>>(a1, a2, a3, ix, CB_C(), CB_C(), 0, nullptr);
}
extern "C" void CB_ITER(clip_min_s, _kernel_launch)(cumo_na_iarray_t* a1, CB_C sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    launch_elementwise<op::ClipLow<CB_C>>(a1, nullptr, a3, ix, CB_C(), sv, 1, nullptr);
}
extern "C" void CB_ITER(clip_max, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    launch_elementwise<op::ClipHigh<CB_C>>(a1, a2, a3, ix, CB_C(), CB_C(), 0, nullptr);
}
extern "C" void CB_ITER(clip_max_s, _kernel_launch)(cumo_na_iarray_t* a1, CB_C sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    launch_elementwise<op::ClipHigh<CB_C>>(a1, nullptr, a3, ix, CB_C(), sv, 1, nullptr);
}
extern "C" void CB_ITER(clip_s, _kernel_launch)(cumo_na_iarray_t* a1, CB_C sv_min, CB_C sv_max, cumo_na_iarray_t* a4, cumo_na_indexer_t* ix) {
    launch_elementwise<op::ClipScalars<CB_C>>(a1, nullptr, a4, ix, sv_min, sv_max, 0, nullptr);
}
extern "C" void CB_ITER(clip, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_iarray_t* a4,
        cumo_na_indexer_t* ix, int* invalid) {
    const cumo_na_iarray_t* a[4] = {a1, a2, a3, a4};
    launch_multi<op::ClipArrays<CB_C>>(a, ix, op::NoParams(), invalid);
}
// fill: the store kernels with the value as their (repeated) input
extern "C" void CB_ITER(fill, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_indexer_t* ix, CB_C sv) {
    launch_elementwise<op::Cast<CB_C, CB_C>>(nullptr, nullptr, a1, ix, sv, CB_C(), 2, nullptr);
}
extern "C" void CB_ITER(seq, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_indexer_t* ix, op::SeqParams<CB_C>::Data beg,
        op::SeqParams<CB_C>::Data step, double count) {
    const cumo_na_iarray_t* a[1] = {a1};
    op::SeqParams<CB_C> prm;
    prm.beg = beg; prm.step = step; prm.count = count;
    launch_multi<op::Seq<CB_C>>(a, ix, prm, nullptr);
}
extern "C" void CB_ITER(poly, _kernel_launch)(cumo_na_iarray_t* x, cumo_na_iarray_t* coef, int ncoef, cumo_na_iarray_t* z, cumo_na_indexer_t* ix) {
    launch_poly<CB_C>(x, coef, ncoef, z, ix);
}
extern "C" void CB_ITER(eye, _stride_kernel_launch)(char* ptr, ssize_t s0, ssize_t s1, ssize_t kofs, CB_C data, uint64_t n0, uint64_t n1) {
    launch_eye<CB_C>(ptr, s0, s1, kofs, data, n0, n1);
}
extern "C" void CB_ITER(divmod, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_iarray_t* a4,
        cumo_na_indexer_t* ix, int* divzero) {
    const cumo_na_iarray_t* a[4] = {a1, a2, a3, a4};
    launch_multi<op::DivMod<CB_C>>(a, ix, op::NoParams(), divzero);
}

#if CB_FLOAT
extern "C" void CB_ITER(modf, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    const cumo_na_iarray_t* a[3] = {a1, a2, a3};
    launch_multi<op::Modf<CB_C>>(a, ix, op::NoParams(), nullptr);
}
extern "C" void CB_ITER(math_s_frexp, _kernel_launch)(cumo_na_iarray_t* a1, cumo_na_iarray_t* a2, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    const cumo_na_iarray_t* a[3] = {a1, a2, a3};
    launch_multi<op::Frexp<CB_C>>(a, ix, op::NoParams(), nullptr);
}
DEF_BINARY_S(copysign, CopySign)
DEF_UNARY(floor, Floor)
DEF_UNARY(round, Round)
DEF_UNARY(ceil, Ceil)
DEF_UNARY(trunc, Trunc)
DEF_UNARY(rint, Rint)
DEF_COND(nearly_eq, NearlyEq)
DEF_COND_UNARY(isnan, IsNan)
DEF_COND_UNARY(isinf, IsInf)
DEF_COND_UNARY(isposinf, IsPosInf)
DEF_COND_UNARY(isneginf, IsNegInf)
DEF_COND_UNARY(isfinite, IsFinite)
DEF_COND_UNARY(signbit, SignBit)
DEF_MATH(sqrt, Sqrt)
DEF_MATH(cbrt, Cbrt)
DEF_MATH(log, Log)
DEF_MATH(log2, Log2)
DEF_MATH(log10, Log10)
DEF_MATH(exp, Exp)
DEF_MATH(exp2, Exp2)
DEF_MATH(exp10, Exp10)
DEF_MATH(sin, Sin)
DEF_MATH(cos, Cos)
DEF_MATH(tan, Tan)
DEF_MATH(asin, Asin)
DEF_MATH(acos, Acos)
DEF_MATH(atan, Atan)
DEF_MATH(sinh, Sinh)
DEF_MATH(cosh, Cosh)
DEF_MATH(tanh, Tanh)
DEF_MATH(asinh, Asinh)
DEF_MATH(acosh, Acosh)
DEF_MATH(atanh, Atanh)
DEF_MATH(sinc, Sinc)
DEF_MATH(erf, Erf)
DEF_MATH(erfc, Erfc)
DEF_MATH(log1p, Log1p)
DEF_MATH(expm1, Expm1)
DEF_MATH2(atan2, Atan2)
DEF_MATH2(hypot, Hypot)
DEF_MATH2(ldexp, Ldexp)
DEF_EWCOMP(maximum_nan, MaximumNan)
DEF_EWCOMP(minimum_nan, MinimumNan)
#else
DEF_BINARY_S(bit_and, BitAnd)
DEF_BINARY_S(bit_or, BitOr)
DEF_BINARY_S(bit_xor, BitXor)
DEF_BINARY_S(left_shift, LeftShift)
DEF_BINARY_S(right_shift, RightShift)
DEF_UNARY(bit_not, BitNot)
#endif
