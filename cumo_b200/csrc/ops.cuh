// Elementwise operation functors.
//
// Semantics follow the device macros of the reference:
//   floats   ext/cumo/include/cumo/types/float_macro_kernel.h:29-149
//   integers ext/cumo/include/cumo/types/xint_macro_kernel.h:15-68, int_macro_kernel.h:4-49
//   NaN-aware maximum/minimum  ext/cumo/include/cumo/types/real_accum_kernel.h:27-69
// No fast-math: the reference is built without it, so the accurate CUDA libm
// functions are called through their C++ overloads.
//
// Every functor has
//   In1, In2, Out      element types of the operands and the result
//   arity              1 or 2
//   apply(x, y, z, flag) -> bool   computes z; returning false skips the store
//                                  (after raising *flag), as the reference's
//                                  cumo_check_intdivzero / cumo_check_intmin do.
#pragma once

#include <cuda_runtime.h>
#include <math.h>
#include <float.h>
#include <stdint.h>
#include <type_traits>
#include <limits>

namespace cb200 {
namespace op {

template <typename T> struct is_fp : std::is_floating_point<T> {};

#define CB200_BIN(NAME, EXPR)                                                          \
    template <typename T> struct NAME {                                                \
        using In1 = T; using In2 = T; using Out = T;                                   \
        static constexpr int arity = 2;                                                \
        __device__ __forceinline__ static bool apply(T x, T y, T& z, int*) {           \
            z = (EXPR); return true; }                                                 \
    };
#define CB200_UN(NAME, EXPR)                                                           \
    template <typename T> struct NAME {                                                \
        using In1 = T; using In2 = T; using Out = T;                                   \
        static constexpr int arity = 1;                                                \
        __device__ __forceinline__ static bool apply(T x, T, T& z, int*) {             \
            z = (EXPR); return true; }                                                 \
    };

CB200_BIN(Add, x + y)
CB200_BIN(Sub, x - y)
CB200_BIN(Mul, x * y)

// float: IEEE division; integer: C truncation, divisor 0 raises the flag and
// leaves the output element untouched (binary_kernel.cu:4-8).
template <typename T> struct Div {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, T y, T& z, int* flag) {
        if constexpr (is_fp<T>::value) { z = x / y; return true; }
        else {
            if (y == 0) { if (flag) *flag = 1; return false; }
            // the one overflowing quotient; the hardware sequence answers the minimum too
            if (y == (T)-1) { z = (T)(0 - (typename std::make_unsigned<T>::type)x); return true; }
            z = x / y; return true;
        }
    }
};
template <typename T> struct Mod {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, T y, T& z, int* flag) {
        if constexpr (is_fp<T>::value) { z = fmod(x, y); return true; }
        else {
            if (y == 0) { if (flag) *flag = 1; return false; }
            if (y == (T)-1) { z = 0; return true; }
            z = x % y; return true;
        }
    }
};

CB200_BIN(BitAnd, x & y)
CB200_BIN(BitOr, x | y)
CB200_BIN(BitXor, x ^ y)
CB200_BIN(LeftShift, x << y)
CB200_BIN(RightShift, x >> y)
CB200_BIN(CopySign, copysign(x, y))
CB200_BIN(Atan2, atan2(x, y))
CB200_BIN(Hypot, hypot(x, y))
CB200_BIN(Ldexp, ldexp(x, (int)y))

// pow(x, y) for floats; integer types multiply repeatedly (m_pow = pow_int).
template <typename T>
__device__ __forceinline__ T pow_int_dev(T x, int p) {
    if constexpr (is_fp<T>::value) {
        bool neg = p < 0;
        int q = neg ? -p : p;
        T r;
        switch (q) {
        case 0: r = 1; break;
        case 1: r = x; break;
        case 2: r = x * x; break;
        case 3: r = x * x * x; break;
        case 4: x = x * x; r = x * x; break;
        default:
            if (q > 64) { r = pow(x, (T)q); }
            else {
                r = 1;
                while (q) { if (q & 1) r *= x; x *= x; q >>= 1; }
            }
        }
        return neg ? 1 / r : r;
    } else {
        switch (p) {
        case 0: return 1;
        case 1: return x;
        case 2: return x * x;
        case 3: return x * x * x;
        }
        if (p < 0) return 0;
        T r = 1;
        while (p) { if (p & 1) r *= x; x *= x; p >>= 1; }
        return r;
    }
}
template <typename T> struct Pow {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, T y, T& z, int*) {
        if constexpr (is_fp<T>::value) z = pow(x, y); else z = pow_int_dev<T>(x, (int)y);
        return true;
    }
};
template <typename T> struct PowInt32 {
    using In1 = T; using In2 = int32_t; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, int32_t y, T& z, int*) { z = pow_int_dev<T>(x, y); return true; }
};

// elementwise maximum/minimum (ewcomp): the plain float form keeps the
// non-NaN operand, the _nan form propagates a NaN; integers compare directly.
template <typename T> struct Maximum {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, T y, T& z, int*) {
        if (x >= y) z = x;
        else if (is_fp<T>::value ? (y == y) : true) z = y;
        else z = x;
        return true;
    }
};
template <typename T> struct MaximumNan {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, T y, T& z, int*) {
        if (x >= y) z = x; else if (!(x == x)) z = x; else z = y;
        return true;
    }
};
template <typename T> struct Minimum {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, T y, T& z, int*) {
        if (x <= y) z = x;
        else if (is_fp<T>::value ? (y == y) : true) z = y;
        else z = x;
        return true;
    }
};
template <typename T> struct MinimumNan {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, T y, T& z, int*) {
        if (x <= y) z = x; else if (!(x == x)) z = x; else z = y;
        return true;
    }
};

// clip against one bound (clip_kernel.cu:24-42): a comparison with a NaN on either side is false, so the element
// passes through
template <typename T> struct ClipLow {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, T lo, T& z, int*) { z = x < lo ? lo : x; return true; }
};
template <typename T> struct ClipHigh {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool apply(T x, T hi, T& z, int*) { z = x > hi ? hi : x; return true; }
};
// clip against two host numerics (clip_kernel.cu:8-22 with use_scalar): the lower bound rides in the kernels' first
// scalar argument, the upper in the second; the caller has already refused lo > hi
template <typename T> struct ClipScalars {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 1;
    static constexpr bool two_scalars = true;
    __device__ __forceinline__ static bool apply2(T x, T lo, T hi, T& z) {
        if (x < lo) x = lo;
        if (x > hi) x = hi;
        z = x;
        return true;
    }
};

// store / cast between element types (m_from_real, m_from_int32, ... are plain C casts)
template <typename TO, typename TF> struct Cast {
    using In1 = TF; using In2 = TF; using Out = TO;
    static constexpr int arity = 1;
    __device__ __forceinline__ static bool apply(TF x, TF, TO& z, int*) { z = (TO)x; return true; }
};

// ---- unary ----
CB200_UN(Minus, -x)
CB200_UN(Square, x * x)
CB200_UN(BitNot, ~x)
CB200_UN(Floor, floor(x))
CB200_UN(Round, round(x))
CB200_UN(Ceil, ceil(x))
CB200_UN(Trunc, trunc(x))
CB200_UN(Rint, rint(x))

template <typename T> struct Reciprocal {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 1;
    __device__ __forceinline__ static bool apply(T x, T, T& z, int* flag) {
        if constexpr (is_fp<T>::value) { z = 1 / x; return true; }
        else {
            if (x == 0) { if (flag) *flag = 1; return false; }
            z = (x == 1) ? (T)1 : (x == -1 ? (T)-1 : (T)0);
            return true;
        }
    }
};
template <typename T> struct Sign {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 1;
    __device__ __forceinline__ static bool apply(T x, T, T& z, int*) {
        // a NaN fails all three comparisons and is passed through
        z = (x == 0) ? (T)0 : ((x > 0) ? (T)1 : ((x < 0) ? (T)-1 : x));
        return true;
    }
};
template <typename T> struct Abs {
    using In1 = T; using In2 = T; using Out = T;
    static constexpr int arity = 1;
    __device__ __forceinline__ static bool apply(T x, T, T& z, int* flag) {
        if constexpr (is_fp<T>::value) { z = fabs(x); return true; }
        else {
            if (x == std::numeric_limits<T>::min()) { if (flag) *flag = 1; return false; }
            z = x < 0 ? -x : x; return true;
        }
    }
};

CB200_UN(Sqrt, sqrt(x))
CB200_UN(Cbrt, cbrt(x))
CB200_UN(Log, log(x))
CB200_UN(Log2, log2(x))
CB200_UN(Log10, log10(x))
CB200_UN(Exp, exp(x))
CB200_UN(Exp2, exp2(x))
CB200_UN(Exp10, exp10(x))
CB200_UN(Sin, sin(x))
CB200_UN(Cos, cos(x))
CB200_UN(Tan, tan(x))
CB200_UN(Asin, asin(x))
CB200_UN(Acos, acos(x))
CB200_UN(Atan, atan(x))
CB200_UN(Sinh, sinh(x))
CB200_UN(Cosh, cosh(x))
CB200_UN(Tanh, tanh(x))
CB200_UN(Asinh, asinh(x))
CB200_UN(Acosh, acosh(x))
CB200_UN(Atanh, atanh(x))
CB200_UN(Sinc, sin(x) / x)   // the device macro has no x == 0 guard: 0/0 = NaN
CB200_UN(Erf, erf(x))
CB200_UN(Erfc, erfc(x))
CB200_UN(Log1p, log1p(x))
CB200_UN(Expm1, expm1(x))

// ---- comparisons (result is one bit) ----
#define CB200_CMP(NAME, EXPR)                                                          \
    template <typename T> struct NAME {                                                \
        using In1 = T; using In2 = T;                                                  \
        static constexpr int arity = 2;                                                \
        __device__ __forceinline__ static bool test(T x, T y) { return (EXPR); }       \
    };
#define CB200_CMP1(NAME, EXPR)                                                         \
    template <typename T> struct NAME {                                                \
        using In1 = T; using In2 = T;                                                  \
        static constexpr int arity = 1;                                                \
        __device__ __forceinline__ static bool test(T x, T) { return (EXPR); }         \
    };
CB200_CMP(Eq, x == y)
CB200_CMP(Ne, x != y)
CB200_CMP(Gt, x > y)
CB200_CMP(Ge, x >= y)
CB200_CMP(Lt, x < y)
CB200_CMP(Le, x <= y)
template <typename T> struct NearlyEq {
    using In1 = T; using In2 = T;
    static constexpr int arity = 2;
    __device__ __forceinline__ static bool test(T x, T y) {
        // |x-y| <= (|x|+|y|) * eps * 2   (types/sfloat_kernel.h, dfloat_kernel.h)
        const T eps = sizeof(T) == 4 ? (T)FLT_EPSILON : (T)DBL_EPSILON;
        return fabs(x - y) <= (fabs(x) + fabs(y)) * eps * 2;
    }
};
CB200_CMP1(IsNan, isnan(x))
CB200_CMP1(IsInf, isinf(x))
CB200_CMP1(IsPosInf, isinf(x) && !signbit(x))
CB200_CMP1(IsNegInf, isinf(x) && signbit(x))
CB200_CMP1(IsFinite, isfinite(x))
CB200_CMP1(SignBit, signbit(x))

#undef CB200_BIN
#undef CB200_UN
#undef CB200_CMP
#undef CB200_CMP1

}  // namespace op

// How the kernels of elementwise.cuh call an operation.  One that declares `two_scalars` takes both scalar arguments
// of the launch beside its array input; every other gets (x, y) as loaded or repeated.
template <typename Op, typename = void> struct takes_two_scalars : std::false_type {};
template <typename Op> struct takes_two_scalars<Op, std::void_t<decltype(Op::two_scalars)>> : std::true_type {};
template <typename Op, typename X, typename Y, typename Z>
__device__ __forceinline__ bool ew_apply(X x, Y y, typename Op::In1 sx, Z& z, int* flag) {
    if constexpr (takes_two_scalars<Op>::value) return Op::apply2(x, sx, y, z);
    else return Op::apply(x, y, z, flag);
}

}  // namespace cb200
