// Reduction functors.
//
// The rules (identities, NaN handling, tie breaking, output types) are those of
// the reference's functors:
//   sum/prod/min/max/ptp/minmax (+_nan)   gen/tmpl/real_accum_kernel.cu:11-157
//   mean/var/stddev/rms/kahan_sum (+_nan) gen/tmpl/float_accum_kernel.cu:15-146
//   max_index/min_index (+_nan)           gen/tmpl/accum_index_kernel.cu:15-113
//   argmax/argmin (+_nan)                 gen/tmpl/accum_arg_kernel.cu:15-113
// restated for an engine in which combine(a, b) merges two partial results, `a`
// covering earlier positions of the reduce axis than `b` wherever the engine can
// promise that, and in which every comparison-type functor is a total order with
// the element index as the last key, so that the answer does not depend on how
// the axis was cut into threads, CTAs or GPUs.
//
// Interface of a reducer R:
//   In, Acc                       element type, accumulator type (trivially copyable)
//   kIndexed                      map() wants the element's index
//   identity()                    neutral accumulator
//   map(v, idx)                   accumulator of one element
//   combine(a, b)                 merge
//   store(out, out2, acc)         MapOut and the store(s), out/out2 are byte pointers
#pragma once

#include "common.cuh"
#include <limits>
#include <type_traits>
#include <math.h>
#include <float.h>

namespace cb200 {
namespace red {

template <typename T> struct is_fp : std::is_floating_point<T> {};
template <typename T> __device__ __forceinline__ bool is_nan(T x) { return !(x == x); }

template <typename T> __host__ __device__ __forceinline__ T data_max() {
    if constexpr (sizeof(T) == 4 && is_fp<T>::value) return (T)FLT_MAX;
    else if constexpr (is_fp<T>::value) return (T)DBL_MAX;
    else return std::numeric_limits<T>::max();
}
template <typename T> __host__ __device__ __forceinline__ T data_min() {
    if constexpr (sizeof(T) == 4 && is_fp<T>::value) return (T)-FLT_MAX;
    else if constexpr (is_fp<T>::value) return (T)-DBL_MAX;
    else return std::numeric_limits<T>::min();
}
template <typename T> __device__ __forceinline__ T quiet_nan() {
    if constexpr (sizeof(T) == 4) return (T)nanf(""); else return (T)nan("");
}

// accumulator of sum/prod: the element type for floats, 64 bits for integers
template <typename T> struct WideOf { using type = typename std::conditional<is_fp<T>::value, T, int64_t>::type; };

// ---- sum / mean / prod -------------------------------------------------------
// mode 0: sum, 1: mean (divide by n, the reduce length cast to T), 2: prod
template <typename T, bool NAN_SKIP, bool PROD>
struct SumLike {
    using In = T;
    using Acc = typename WideOf<T>::type;
    static constexpr bool kIndexed = false;
    static constexpr bool kHasScan = false;
    int mean;
    T n;
    __device__ __forceinline__ Acc identity() const { return PROD ? (Acc)1 : (Acc)0; }
    __device__ __forceinline__ Acc map(T v, int64_t) const {
        if (NAN_SKIP && is_nan(v)) return identity();
        return (Acc)v;
    }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return PROD ? a * b : a + b; }
    __device__ __forceinline__ void store(char* out, char*, Acc a) const {
        if (mean) a = (Acc)(a / (Acc)n);
        *reinterpret_cast<Acc*>(out) = a;
    }
};

// mean_nan: divide by the count of non-NaN elements
template <typename T>
struct MeanNan {
    using In = T;
    struct Acc { T sum; T n; };
    static constexpr bool kIndexed = false;
    static constexpr bool kHasScan = false;
    __device__ __forceinline__ Acc identity() const { return {(T)0, (T)0}; }
    __device__ __forceinline__ Acc map(T v, int64_t) const { return is_nan(v) ? Acc{(T)0, (T)0} : Acc{v, (T)1}; }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return {a.sum + b.sum, a.n + b.n}; }
    __device__ __forceinline__ void store(char* out, char*, Acc a) const { *reinterpret_cast<T*>(out) = a.sum / a.n; }
};

// rms: sqrt(sum |x|^2 / n); the _nan form counts what it kept
template <typename T, bool NAN_SKIP>
struct Rms {
    using In = T;
    struct Acc { T sum; T n; };
    static constexpr bool kIndexed = false;
    static constexpr bool kHasScan = false;
    T n_all;
    __device__ __forceinline__ Acc identity() const { return {(T)0, (T)0}; }
    __device__ __forceinline__ Acc map(T v, int64_t) const {
        if (NAN_SKIP && is_nan(v)) return {(T)0, (T)0};
        T a = fabs(v);
        return {a * a, (T)1};
    }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return {a.sum + b.sum, a.n + b.n}; }
    __device__ __forceinline__ void store(char* out, char*, Acc a) const {
        *reinterpret_cast<T*>(out) = sqrt(a.sum / (NAN_SKIP ? a.n : n_all));
    }
};

// var / stddev: Chan's pairwise combination of (count, mean, M2)
template <typename T, bool NAN_SKIP>
struct Moments {
    using In = T;
    struct Acc { T n; T mean; T m2; };
    static constexpr bool kIndexed = false;
    static constexpr bool kHasScan = false;
    int take_sqrt;
    __device__ __forceinline__ Acc identity() const { return {(T)0, (T)0, (T)0}; }
    __device__ __forceinline__ Acc map(T v, int64_t) const {
        if (NAN_SKIP && is_nan(v)) return {(T)0, (T)0, (T)0};
        return {(T)1, v, (T)0};
    }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const {
        if (b.n == 0) return a;
        if (a.n == 0) return b;
        T n = a.n + b.n;
        T delta = b.mean - a.mean;
        Acc r;
        r.mean = a.mean + delta * (b.n / n);
        r.m2 = a.m2 + (b.m2 + delta * delta * a.n * b.n / n);
        r.n = n;
        return r;
    }
    __device__ __forceinline__ void store(char* out, char*, Acc a) const {
        T v;
        if (NAN_SKIP && a.n == 0) v = (T)0;
        else { v = a.m2 / (a.n - 1); if (take_sqrt) v = sqrt(v); }
        *reinterpret_cast<T*>(out) = v;
    }
};

// kahan_sum: Kahan-Babuska-Neumaier carried as (sum, compensation)
template <typename T, bool NAN_SKIP>
struct Kahan {
    using In = T;
    struct Acc { T sum; T comp; };
    static constexpr bool kIndexed = false;
    static constexpr bool kHasScan = false;
    __device__ __forceinline__ Acc identity() const { return {(T)0, (T)0}; }
    __device__ __forceinline__ Acc map(T v, int64_t) const {
        if (NAN_SKIP && is_nan(v)) return {(T)0, (T)0};
        return {v, (T)0};
    }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const {
        T t = a.sum + b.sum;
        T c = (fabs(a.sum) >= fabs(b.sum)) ? (a.sum - t) + b.sum : (b.sum - t) + a.sum;
        return {t, a.comp + (b.comp + c)};
    }
    __device__ __forceinline__ void store(char* out, char*, Acc a) const { *reinterpret_cast<T*>(out) = a.sum + a.comp; }
};

// ---- min / max ------------------------------------------------------------------
// Plain float form: identity NaN, a NaN loses to anything, so the answer is NaN
// only when every element is.  _nan form: a NaN wins and sticks; identities are
// the finite extremes DATA_MAX / DATA_MIN, exactly as the reference has them.
template <typename T, bool IS_MAX, bool NAN_WINS>
struct MinMax {
    using In = T;
    using Acc = T;
    static constexpr bool kIndexed = false;
    static constexpr bool kHasScan = false;
    __device__ __forceinline__ Acc identity() const {
        if constexpr (is_fp<T>::value && !NAN_WINS) return quiet_nan<T>();
        else return IS_MAX ? data_min<T>() : data_max<T>();
    }
    __device__ __forceinline__ Acc map(T v, int64_t) const { return v; }
    __device__ __forceinline__ static bool better(T b, T a) { return IS_MAX ? (a < b) : (b < a); }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const {
        if constexpr (!is_fp<T>::value) return better(b, a) ? b : a;
        else if constexpr (NAN_WINS) return (is_nan(b) || better(b, a)) ? b : a;
        else return (better(b, a) || is_nan(a)) ? b : a;
    }
    __device__ __forceinline__ void store(char* out, char*, Acc a) const { *reinterpret_cast<T*>(out) = a; }
};

// ptp (one output: max - min) and minmax (two outputs)
template <typename T, bool NAN_WINS, bool TWO_OUT>
struct MinAndMax {
    using In = T;
    struct Acc { T mn; T mx; };
    static constexpr bool kIndexed = false;
    static constexpr bool kHasScan = false;
    __device__ __forceinline__ Acc identity() const {
        if constexpr (TWO_OUT && is_fp<T>::value && !NAN_WINS) return {quiet_nan<T>(), quiet_nan<T>()};
        else return {data_max<T>(), data_min<T>()};
    }
    __device__ __forceinline__ Acc map(T v, int64_t) const { return {v, v}; }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const {
        if constexpr (!is_fp<T>::value) {
            return {b.mn < a.mn ? b.mn : a.mn, b.mx < a.mx ? a.mx : b.mx};
        } else if constexpr (NAN_WINS) {
            if (is_nan(b.mn) || b.mn < a.mn) a.mn = b.mn;
            if (is_nan(b.mx) || a.mx < b.mx) a.mx = b.mx;
            return a;
        } else if constexpr (TWO_OUT) {
            if (b.mn < a.mn || is_nan(a.mn)) a.mn = b.mn;
            if (a.mx < b.mx || is_nan(a.mx)) a.mx = b.mx;
            return a;
        } else {  // plain ptp: a NaN loses both comparisons
            if (b.mn < a.mn) a.mn = b.mn;
            if (a.mx < b.mx) a.mx = b.mx;
            return a;
        }
    }
    __device__ __forceinline__ void store(char* out, char* out2, Acc a) const {
        if constexpr (TWO_OUT) {
            *reinterpret_cast<T*>(out) = a.mn;
            *reinterpret_cast<T*>(out2) = a.mx;
        } else {
            T v;
            if (is_fp<T>::value && !NAN_WINS && a.mx < a.mn) v = quiet_nan<T>();  // every element was NaN
            else v = a.mx - a.mn;
            *reinterpret_cast<T*>(out) = v;
        }
    }
};

// ---- index reductions --------------------------------------------------------------
// Order: plain form -- a number beats a NaN, then the better value, then the lower
// index; _nan form -- a NaN beats a number, then the same.  The engine feeds either
// the position along the reduce axes (argmax/argmin) or the element's offset from
// the start of the input (max_index/min_index); `idx64` picks the output width.
template <typename T, bool IS_MAX, bool NAN_WINS>
struct ArgMinMax {
    using In = T;
    struct Acc { T value; int64_t index; };
    static constexpr bool kIndexed = true;
    static constexpr bool kHasScan = true;
    // 4-byte element types can fold a warp's accumulators with integer reduce instructions on an order-preserving key
    static constexpr bool kReduxFold = sizeof(T) == 4;
    // larger key = ranks better under combine()'s order; all values of the losing NaN class share key 0 (plain form:
    // NaN loses; NaN-wins form: NaN gets the top key), so among equal keys the lower index decides, as in combine()
    __device__ __forceinline__ uint32_t order_key(T v) const {
        uint32_t k;
        if constexpr (is_fp<T>::value) {
            const uint32_t b = __float_as_uint((float)v);
            if (v != v) return NAN_WINS ? 0xffffffffu : 0u;
            k = (b & 0x80000000u) ? ~b : (b | 0x80000000u);           // ascending with the float order; -0 < +0 here, see below
            if (v == 0) k = 0x80000000u;                               // both zeros compare equal: one key
        } else {
            k = (uint32_t)v ^ 0x80000000u;                             // ascending with the signed order
        }
        k = IS_MAX ? k : ~k;
        // keep clear of the keys reserved for the NaN class
        if constexpr (is_fp<T>::value) { if (k == 0u) k = 1u; if (k == 0xffffffffu) k = 0xfffffffeu; }
        return k;
    }
    int idx64;
    int64_t base = 0;          // added to every index written (a shard's offset in the global array)
    // A thread's private scan of a run visited in increasing index order.  A strict
    // comparison keeps the earlier of two equal elements, so no index is ever compared,
    // and the position is a 32-bit offset into the thread's segment.  The scan starts from
    // the identity value with position -1 and costs two compares and two selects per element;
    // if it ends with the position still negative, every element it saw ranks equal to the
    // identity (all NaN, all -inf, all INT_MIN ...), and the caller settles it on the first
    // position visited.  Same answers as folding combine(acc, map(v, idx)) over the run.
    struct Local { T value; int32_t pos; };
    __device__ __forceinline__ Local local_identity() const { return {identity().value, -1}; }
    __device__ __forceinline__ void local_scan(Local& l, T v, int32_t pos) const {
        bool take;
        if constexpr (!is_fp<T>::value) take = IS_MAX ? (l.value < v) : (v < l.value);
        else {
            // "not >=" is also true when either side is NaN
            const bool beats = IS_MAX ? !(l.value >= v) : !(l.value <= v);
            if constexpr (NAN_WINS) take = beats && (l.value == l.value);     // a NaN, once held, sticks
            else take = beats && (v == v);                                    // a NaN never replaces anything
        }
        if (take) { l.value = v; l.pos = pos; }
    }
    // two scans over disjoint sets of positions: the same total order as combine()
    __device__ __forceinline__ void local_merge(Local& a, const Local& b) const {
        if (b.pos < 0) return;
        if (a.pos < 0) { a = b; return; }
        const Acc m = combine(Acc{a.value, (int64_t)a.pos}, Acc{b.value, (int64_t)b.pos});
        a.value = m.value;
        a.pos = (int32_t)m.index;
    }
    __device__ __forceinline__ Acc identity() const {
        T v;
        if constexpr (!is_fp<T>::value) v = IS_MAX ? data_min<T>() : data_max<T>();
        else if constexpr (NAN_WINS) v = IS_MAX ? (T)-INFINITY : (T)INFINITY;
        else v = quiet_nan<T>();
        return {v, INT64_MAX};   // loses every tie; no real index reaches it
    }
    __device__ __forceinline__ Acc map(T v, int64_t idx) const { return {v, idx}; }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const {
        if constexpr (is_fp<T>::value) {
            bool an = is_nan(a.value), bn = is_nan(b.value);
            if (an || bn) {
                if constexpr (NAN_WINS) return (bn && (!an || b.index < a.index)) ? b : a;
                else return (an && (!bn || b.index < a.index)) ? b : a;
            }
        }
        bool better = IS_MAX ? (a.value < b.value) : (a.value > b.value);
        return (better || (a.value == b.value && b.index < a.index)) ? b : a;
    }
    // out2, when given, receives the winning value beside its index
    __device__ __forceinline__ void store(char* out, char* out2, Acc a) const {
        if (idx64) *reinterpret_cast<int64_t*>(out) = a.index + base;
        else *reinterpret_cast<int32_t*>(out) = (int32_t)(a.index + base);
        if (out2) *reinterpret_cast<T*>(out2) = a.value;
    }
};

}  // namespace red
}  // namespace cb200
