// Host layer above the kernel-launch ABI: NArray objects and an ndloop-style
// dispatcher.  See include/cumo_b200_host.h for what it mirrors in the reference.
//
// Everything here only prepares descriptors and calls the exported
// `cumo_..._kernel_launch` symbols by the names the reference's generated code
// uses; no arithmetic on array data happens on the host.
#include "../common.cuh"
#include "../../../include/cumo_b200_host.h"

#include <dlfcn.h>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace {

constexpr int kMaxD = CUMO_NA_MAX_DIMENSION;
const char* kTypeName[] = {"sfloat", "dfloat", "int32", "int64", "bit", "uint64", "uint32"};
const int kElemSize[] = {4, 8, 4, 8, 0, 8, 4};

thread_local std::string tl_class, tl_message;

struct Storage {
    char* ptr;
    size_t bytes;
    int refs;
    bool owned;
};

}  // namespace

struct cb200_na {
    int dtype;
    int ndim;
    int64_t shape[kMaxD];
    int64_t step[kMaxD];     // bytes; bits for CB200_BIT
    int64_t offset;          // same unit, from the start of the buffer
    Storage* st;
    bool inplace;
};

namespace {

std::mutex g_ref_mu;

void* fail(const char* klass, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    tl_class = klass;
    tl_message = buf;
    return nullptr;
}

bool cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    fail("CudaError", "%s: %s", what, cudaGetErrorString(e));
    return false;
}

// raise what the default launch check latched (a strong check supplied by a host
// program reports through its own channel and leaves the latch empty)
bool launch_ok() {
    const char* msg = nullptr;
    int e = cb200_last_error(&msg);
    if (e == 0) return true;
    fail("CudaError", "%s", msg);
    return false;
}

int64_t size_of(const cb200_na* a) {
    int64_t n = 1;
    for (int d = 0; d < a->ndim; ++d) n *= a->shape[d];
    return n;
}

size_t buffer_bytes(int dtype, int64_t n) {
    if (dtype == CB200_BIT) return (size_t)((n + 31) / 32) * 4;
    return (size_t)n * kElemSize[dtype];
}

void contiguous_steps(int dtype, int ndim, const int64_t* shape, int64_t* step) {
    int64_t s = dtype == CB200_BIT ? 1 : kElemSize[dtype];
    for (int d = ndim - 1; d >= 0; --d) { step[d] = s; s *= shape[d]; }
}

cb200_na* make(int dtype, int ndim, const int64_t* shape, bool zero) {
    if (dtype < 0 || dtype > CB200_UINT32) return (cb200_na*)fail("TypeError", "unknown dtype %d", dtype);
    if (ndim < 0 || ndim > kMaxD) return (cb200_na*)fail("ShapeError", "ndim %d out of range", ndim);
    cb200_na* a = new cb200_na();
    a->dtype = dtype;
    a->ndim = ndim;
    for (int d = 0; d < ndim; ++d) {
        if (shape[d] < 0) { delete a; return (cb200_na*)fail("ShapeError", "negative extent"); }
        a->shape[d] = shape[d];
    }
    contiguous_steps(dtype, ndim, a->shape, a->step);
    a->offset = 0;
    a->inplace = false;
    size_t bytes = buffer_bytes(dtype, size_of(a));
    char* p = cumo_cuda_runtime_malloc(bytes ? bytes : 4);
    if (!p) { delete a; launch_ok(); if (tl_message.empty()) fail("CudaError", "out of device memory"); return nullptr; }
    if (zero && bytes) {
        if (!cuda_ok(cudaMemsetAsync(p, 0, bytes, cb200::current_stream()), "cudaMemsetAsync")) {
            cumo_cuda_runtime_free(p); delete a; return nullptr;
        }
    }
    a->st = new Storage{p, bytes, 1, true};
    return a;
}

cb200_na* share(const cb200_na* src) {
    cb200_na* v = new cb200_na(*src);
    v->inplace = false;
    std::lock_guard<std::mutex> lk(g_ref_mu);
    ++v->st->refs;
    return v;
}

char* data_ptr(const cb200_na* a) {   // value types only
    return a->st->ptr + a->offset;
}

bool is_contiguous(const cb200_na* a) {
    int64_t s = a->dtype == CB200_BIT ? 1 : kElemSize[a->dtype];
    for (int d = a->ndim - 1; d >= 0; --d) {
        if (a->shape[d] != 1 && a->step[d] != s) return false;
        s *= a->shape[d];
    }
    return true;
}

// ---- symbol lookup ---------------------------------------------------------------------
void* lib_handle() {
    static void* h = [] {
        Dl_info info;
        if (dladdr((void*)&cb200_version, &info) && info.dli_fname) {
            void* hh = dlopen(info.dli_fname, RTLD_NOW | RTLD_NOLOAD);
            if (hh) return hh;
        }
        return dlopen(nullptr, RTLD_NOW);
    }();
    return h;
}

void* sym(const std::string& name) {
    void* f = dlsym(lib_handle(), name.c_str());
    if (!f) fail("NoMethodError", "libcumo_b200 has no entry point %s", name.c_str());
    return f;
}

// ---- the int* flag of integer div/mod/reciprocal/abs ------------------------------------
// One mapped pinned int per thread, as ext/cumo/cuda/runtime.c:22-47 allocates per call.
// (bincount's second word, the offending item, shares the allocation: a mapped allocation per call costs more than the
// kernels of a small call.)
struct Flag {
    int* host = nullptr;
    int* dev = nullptr;
    size_t* item_host = nullptr;
    size_t* item_dev = nullptr;
    bool ready() {
        if (host) return true;
        if (cudaHostAlloc((void**)&host, 16, cudaHostAllocMapped) != cudaSuccess) { host = nullptr; return false; }
        if (cudaHostGetDevicePointer((void**)&dev, host, 0) != cudaSuccess) { cudaFreeHost(host); host = nullptr; return false; }
        item_host = reinterpret_cast<size_t*>(reinterpret_cast<char*>(host) + 8);
        item_dev = reinterpret_cast<size_t*>(reinterpret_cast<char*>(dev) + 8);
        return true;
    }
};
thread_local Flag tl_flag;

// ---- descriptors ---------------------------------------------------------------------------
struct Loop {
    int ndim;
    int64_t shape[kMaxD];
};

// broadcast rule of ndloop_check_shape: extents are aligned at the last dimension, an
// extent of 1 repeats, anything else must match
bool broadcast(const cb200_na* a, const cb200_na* b, Loop* lp) {
    lp->ndim = a->ndim > b->ndim ? a->ndim : b->ndim;
    for (int i = 0; i < lp->ndim; ++i) {
        int da = i - (lp->ndim - a->ndim), db = i - (lp->ndim - b->ndim);
        int64_t na = da >= 0 ? a->shape[da] : 1, nb = db >= 0 ? b->shape[db] : 1;
        if (na != nb && na != 1 && nb != 1) {
            fail("ShapeError", "shape1[%d](=%lld) != shape2[%d](=%lld)", da, (long long)na, db, (long long)nb);
            return false;
        }
        lp->shape[i] = na == 1 ? nb : na;
    }
    return true;
}

void fill_indexer(cumo_na_indexer_t* ix, const Loop& lp) {
    memset(ix, 0, sizeof *ix);
    ix->ndim = (unsigned char)lp.ndim;
    ix->total_size = 1;
    for (int d = 0; d < lp.ndim; ++d) { ix->shape[d] = (size_t)lp.shape[d]; ix->total_size *= (size_t)lp.shape[d]; }
}

// operand steps against the loop shape: 0 where the operand's extent is 1 or missing
void fill_iarray(cumo_na_iarray_t* ia, const cb200_na* a, const Loop& lp) {
    memset(ia, 0, sizeof *ia);
    ia->ptr = data_ptr(a);
    for (int i = 0; i < lp.ndim; ++i) {
        int d = i - (lp.ndim - a->ndim);
        ia->step[i] = (d >= 0 && a->shape[d] != 1) ? (ssize_t)a->step[d] : 0;
    }
}

void fill_bit_iarray(cumo_na_bit_iarray_t* ia, const cb200_na* a, const Loop& lp) {
    memset(ia, 0, sizeof *ia);
    ia->ptr = reinterpret_cast<CUMO_BIT_DIGIT*>(a->st->ptr);
    ia->pos = (size_t)a->offset;
    for (int i = 0; i < lp.ndim; ++i) {
        int d = i - (lp.ndim - a->ndim);
        ia->step[i] = (d >= 0 && a->shape[d] != 1) ? (ssize_t)a->step[d] : 0;
    }
}

int upcast(int ta, int tb) {   // gen/def/{sfloat,dfloat,int32,int64}.rb
    if (ta == tb) return ta;
    if (ta == CB200_DFLOAT || tb == CB200_DFLOAT) return CB200_DFLOAT;
    if (ta == CB200_SFLOAT || tb == CB200_SFLOAT) return CB200_SFLOAT;
    return CB200_INT64;
}

bool is_value_type(int t) { return t >= CB200_SFLOAT && t <= CB200_INT64; }
bool is_float_type(int t) { return t == CB200_SFLOAT || t == CB200_DFLOAT; }

// Bit <-> value conversion: `SFloat.cast(mask)` runs the value type's store_bit (gen/tmpl/store_bit.c:14-27),
// `Bit.cast(values)` the Bit type's store_<source> (gen/tmpl_bit/store_from.c:14-27).  Both take operands addressed by
// step-or-index per dimension; a view reaches them with plain steps.
cb200_na* cast_bit(cb200_na* a, int dtype) {
    const bool to_bit = dtype == CB200_BIT;
    const cb200_na* val_src = to_bit ? a : nullptr;
    if (to_bit ? (a->dtype == CB200_BIT) : (a->dtype != CB200_BIT || !is_value_type(dtype)))
        return (cb200_na*)fail("TypeError", "cannot cast %s to %s", kTypeName[a->dtype], kTypeName[dtype]);
    cb200_na* out = make(dtype, a->ndim, a->shape, to_bit);
    if (!out) return nullptr;
    if (size_of(out) == 0) return out;
    const cb200_na* bits = to_bit ? out : a;
    const cb200_na* vals = to_bit ? val_src : out;
    cumo_na_indexer_t ix;
    cumo_na_iarray_stridx_t v;
    cumo_na_bit_iarray_stridx_t b;
    memset(&ix, 0, sizeof ix);
    memset(&v, 0, sizeof v);
    memset(&b, 0, sizeof b);
    ix.ndim = (unsigned char)a->ndim;
    ix.total_size = 1;
    v.ptr = data_ptr(vals);
    b.ptr = reinterpret_cast<CUMO_BIT_DIGIT*>(bits->st->ptr);
    b.pos = (size_t)bits->offset;
    for (int d = 0; d < a->ndim; ++d) {
        ix.shape[d] = (size_t)a->shape[d];
        ix.total_size *= (size_t)a->shape[d];
        v.stridx[d].stride = (ssize_t)((vals->step[d] << 1) | 1);        // a step, not an index array
        b.stridx[d].stride = (ssize_t)((bits->step[d] << 1) | 1);
    }
    bool ok;
    if (to_bit) {
        auto f = (void (*)(cumo_na_bit_iarray_stridx_t*, cumo_na_iarray_stridx_t*, cumo_na_indexer_t*))
            sym(std::string("cumo_iter_bit_store_") + kTypeName[a->dtype] + "_kernel_launch");
        ok = f != nullptr;
        if (ok) f(&b, &v, &ix);
    } else {
        auto f = (void (*)(cumo_na_iarray_stridx_t*, cumo_na_bit_iarray_stridx_t*, cumo_na_indexer_t*))
            sym(std::string("cumo_iter_") + kTypeName[dtype] + "_store_bit_kernel_launch");
        ok = f != nullptr;
        if (ok) f(&v, &b, &ix);
    }
    if (!ok || !launch_ok()) { cb200_na_release(out); return nullptr; }
    return out;
}

cb200_na* cast_to(cb200_na* a, int dtype) {
    if ((a->dtype == CB200_BIT) != (dtype == CB200_BIT)) return cast_bit(a, dtype);
    if (!is_value_type(a->dtype) || !is_value_type(dtype)) return (cb200_na*)fail("TypeError", "cannot cast %s to %s", kTypeName[a->dtype], kTypeName[dtype]);
    cb200_na* out = make(dtype, a->ndim, a->shape, false);
    if (!out) return nullptr;
    using Fn = void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*);
    Fn f = (Fn)sym(std::string("cumo_iter_") + kTypeName[dtype] + "_store_" + kTypeName[a->dtype] + "_kernel_launch");
    if (!f) { cb200_na_release(out); return nullptr; }
    Loop lp;
    lp.ndim = a->ndim;
    memcpy(lp.shape, a->shape, sizeof(int64_t) * a->ndim);
    cumo_na_indexer_t ix;
    cumo_na_iarray_t dst, src;
    fill_indexer(&ix, lp);
    fill_iarray(&dst, out, lp);
    fill_iarray(&src, a, lp);
    f(&dst, &src, &ix);
    if (!launch_ok()) { cb200_na_release(out); return nullptr; }
    return out;
}

// which family an operation name belongs to decides the symbol name and the signature
enum Family { F_BINARY_S, F_MATH2, F_EWCOMP, F_POW, F_NONE };
Family binary_family(const std::string& op, bool is_float) {
    static const char* with_s[] = {"add", "sub", "mul", "div", "mod"};
    for (auto s : with_s) if (op == s) return F_BINARY_S;
    if (is_float && op == "copysign") return F_BINARY_S;
    if (!is_float) for (auto s : {"bit_and", "bit_or", "bit_xor", "left_shift", "right_shift"}) if (op == s) return F_BINARY_S;
    if (is_float) for (auto s : {"atan2", "hypot", "ldexp"}) if (op == s) return F_MATH2;
    if (op == "maximum" || op == "minimum") return F_EWCOMP;
    if (is_float && (op == "maximum_nan" || op == "minimum_nan")) return F_EWCOMP;
    if (op == "pow") return F_POW;
    return F_NONE;
}

bool needs_flag(const std::string& op, int dtype) {
    if (op == "clip") return true;                 // an empty range, whatever the type (gen/tmpl/clip.c:47-53)
    if (is_float_type(dtype)) return false;
    return op == "div" || op == "mod" || op == "reciprocal" || op == "abs" || op == "divmod";
}

// run `launch(flag_ptr)`, then apply the flag protocol: synchronise and raise
template <typename L>
bool with_flag(const std::string& op, int dtype, L launch) {
    int* dev = nullptr;
    if (needs_flag(op, dtype)) {
        if (!tl_flag.ready()) { fail("CudaError", "cannot allocate the mapped error flag"); return false; }
        *tl_flag.host = 0;
        dev = tl_flag.dev;
    }
    launch(dev);
    if (!launch_ok()) return false;
    if (dev) {
        if (!cuda_ok(cudaStreamSynchronize(cb200::current_stream()), "cudaStreamSynchronize")) return false;
        if (*tl_flag.host) {
            if (op == "abs") fail("ValueError", "cannot convert the minimum integer");
            else if (op == "clip") fail("OperationError", "min is greater than max");
            else fail("ZeroDivisionError", "divided by 0");
            return false;
        }
    }
    return true;
}

// output of an elementwise method: the in-place operand when it was marked and fits
cb200_na* output_for(cb200_na* a, int dtype, const Loop& lp) {
    if (a && a->inplace && a->dtype == dtype && a->ndim == lp.ndim) {
        bool same = true;
        for (int d = 0; d < lp.ndim; ++d) if (a->shape[d] != lp.shape[d]) same = false;
        if (same) { a->inplace = false; return share(a); }
    }
    return make(dtype, lp.ndim, lp.shape, false);
}

template <typename C> C pick(double f, int64_t i);
template <> float pick<float>(double f, int64_t) { return (float)f; }
template <> double pick<double>(double f, int64_t) { return f; }
template <> int32_t pick<int32_t>(double, int64_t i) { return (int32_t)i; }
template <> int64_t pick<int64_t>(double, int64_t i) { return i; }

template <typename C>
bool call_binary_s(void* f, Family fam, cumo_na_iarray_t* a1, C sv, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix, int* flag, int left) {
    if (fam == F_BINARY_S) ((void (*)(cumo_na_iarray_t*, C, cumo_na_iarray_t*, cumo_na_indexer_t*, int*, int))f)(a1, sv, a3, ix, flag, left);
    else if (fam == F_MATH2) ((void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*, C, int))f)(a1, a3, ix, sv, left);
    else if (fam == F_POW) ((void (*)(cumo_na_iarray_t*, C, cumo_na_iarray_t*, cumo_na_indexer_t*, int))f)(a1, sv, a3, ix, left);
    else return false;
    return true;
}

template <typename C>
void call_compare_s(void* f, cumo_na_iarray_t* a1, C sv, cumo_na_bit_iarray_t* a3, cumo_na_indexer_t* ix, int left) {
    ((void (*)(cumo_na_iarray_t*, C, cumo_na_bit_iarray_t*, cumo_na_indexer_t*, int))f)(a1, sv, a3, ix, left);
}

std::string binary_symbol(const std::string& op, Family fam, int dtype, bool scalar) {
    std::string t = kTypeName[dtype];
    switch (fam) {
    case F_BINARY_S: return "cumo_iter_" + t + "_" + op + (scalar ? "_s_kernel_launch" : "_kernel_launch");
    case F_MATH2:    return "cumo_iter_" + t + "_math_s_" + op + (scalar ? "_s_kernel_launch" : "_kernel_launch");
    case F_POW:      return "cumo_iter_" + t + "_pow" + (scalar ? "_s_kernel_launch" : "_kernel_launch");
    case F_EWCOMP:   return "cumo_" + t + "_" + op + "_kernel_launch";
    default: return "";
    }
}

bool is_math_fn(const std::string& op) {
    static const char* names[] = {"sqrt", "cbrt", "log", "log2", "log10", "exp", "exp2", "exp10", "sin", "cos", "tan",
                                  "asin", "acos", "atan", "sinh", "cosh", "tanh", "asinh", "acosh", "atanh", "sinc",
                                  "erf", "erfc", "log1p", "expm1"};
    for (auto s : names) if (op == s) return true;
    return false;
}

// ---- reductions ----------------------------------------------------------------------------
struct ReducePlan {
    int n_keep, n_red;
    int keep[kMaxD], red[kMaxD];     // dimension numbers of `a`
    int64_t out_shape[kMaxD];        // extents of the kept dims
    int64_t keep_shape[kMaxD];       // result shape with keepdims
};

bool plan_reduce(const cb200_na* a, uint32_t mask, ReducePlan* rp) {
    if (a->ndim > 0 && (mask >> a->ndim) != 0) { fail("ArgumentError", "axis out of range"); return false; }
    if (mask == 0) mask = a->ndim >= 32 ? 0xffffffffu : ((1u << a->ndim) - 1u);
    rp->n_keep = rp->n_red = 0;
    for (int d = 0; d < a->ndim; ++d) {
        if (mask & (1u << d)) { rp->red[rp->n_red++] = d; rp->keep_shape[d] = 1; }
        else { rp->keep[rp->n_keep] = d; rp->out_shape[rp->n_keep++] = a->shape[d]; rp->keep_shape[d] = a->shape[d]; }
    }
    return true;
}

// cumo_na_make_reduction_arg (indexer.h:189-220) for `a` with the kept dims first
void fill_reduction_arg(cumo_na_reduction_arg_t* arg, const cb200_na* a, const ReducePlan& rp, const cb200_na* out) {
    memset(arg, 0, sizeof *arg);
    arg->in.ptr = data_ptr(a);
    arg->in_indexer.ndim = (unsigned char)a->ndim;
    arg->in_indexer.total_size = 1;
    int k = 0;
    for (int i = 0; i < rp.n_keep; ++i, ++k) {
        arg->in.step[k] = (ssize_t)a->step[rp.keep[i]];
        arg->in_indexer.shape[k] = (size_t)a->shape[rp.keep[i]];
    }
    for (int i = 0; i < rp.n_red; ++i, ++k) {
        arg->in.step[k] = (ssize_t)a->step[rp.red[i]];
        arg->in_indexer.shape[k] = (size_t)a->shape[rp.red[i]];
    }
    for (int d = 0; d < a->ndim; ++d) arg->in_indexer.total_size *= arg->in_indexer.shape[d];
    arg->out.ptr = data_ptr(out);
    arg->out_indexer.ndim = (unsigned char)rp.n_keep;
    arg->out_indexer.total_size = 1;
    for (int i = 0; i < rp.n_keep; ++i) {
        arg->out.step[i] = (ssize_t)out->step[i];
        arg->out_indexer.shape[i] = (size_t)rp.out_shape[i];
        arg->out_indexer.total_size *= (size_t)rp.out_shape[i];
    }
}

void apply_keepdims(cb200_na* out, const cb200_na* a, const ReducePlan& rp, int keepdims) {
    if (!keepdims) return;
    out->ndim = a->ndim;
    memcpy(out->shape, rp.keep_shape, sizeof(int64_t) * a->ndim);
    contiguous_steps(out->dtype, out->ndim, out->shape, out->step);
}

// Host loop over the outer dims of a non-indexer ndloop (ndloop.c:1574-1613): dims are
// ordered kept-first, neighbouring dims that every operand walks with one stride are
// merged, the innermost dim is handed to `body(n, offsets...)` and the rest iterate here.
struct StrideLoop {
    int nd;
    int64_t n[kMaxD];
    int64_t s[3][kMaxD];
};
void contract(StrideLoop* L, int nops) {
    int k = 0;
    for (int d = 0; d < L->nd; ++d) {
        if (L->n[d] == 1 && L->nd > 1) continue;
        bool merge = k > 0;
        for (int o = 0; o < nops && merge; ++o) if (L->s[o][k - 1] != L->s[o][d] * L->n[d]) merge = false;
        if (merge) {
            L->n[k - 1] *= L->n[d];
            for (int o = 0; o < nops; ++o) L->s[o][k - 1] = L->s[o][d];
        } else {
            L->n[k] = L->n[d];
            for (int o = 0; o < nops; ++o) L->s[o][k] = L->s[o][d];
            ++k;
        }
    }
    if (k == 0) { L->n[0] = 1; for (int o = 0; o < nops; ++o) L->s[o][0] = 0; k = 1; }
    L->nd = k;
}
template <typename Body>
void for_outer(const StrideLoop& L, int nops, Body body) {
    int64_t outer = 1;
    for (int d = 0; d < L.nd - 1; ++d) outer *= L.n[d];
    for (int64_t o = 0; o < outer; ++o) {
        int64_t off[3] = {0, 0, 0}, r = o;
        for (int d = L.nd - 2; d >= 0; --d) {
            int64_t i = r % L.n[d]; r /= L.n[d];
            for (int k = 0; k < nops; ++k) off[k] += i * L.s[k][d];
        }
        body(off);
    }
}

}  // namespace

// =============================================================================================
extern "C" {

const char* cb200_host_error(const char** klass) {
    if (klass) *klass = tl_class.c_str();
    return tl_message.c_str();
}

cb200_na_t* cb200_na_new(int dtype, int ndim, const int64_t* shape) { return make(dtype, ndim, shape, false); }
cb200_na_t* cb200_na_zeros(int dtype, int ndim, const int64_t* shape) { return make(dtype, ndim, shape, true); }

cb200_na_t* cb200_na_wrap(int dtype, int ndim, const int64_t* shape, const int64_t* step, void* device_ptr, int64_t offset) {
    if (dtype < 0 || dtype > CB200_UINT32) return (cb200_na*)fail("TypeError", "unknown dtype %d", dtype);
    if (ndim < 0 || ndim > kMaxD) return (cb200_na*)fail("ShapeError", "ndim %d out of range", ndim);
    cb200_na* a = new cb200_na();
    a->dtype = dtype;
    a->ndim = ndim;
    for (int d = 0; d < ndim; ++d) { a->shape[d] = shape[d]; a->step[d] = step[d]; }
    a->offset = offset;
    a->inplace = false;
    a->st = new Storage{(char*)device_ptr, 0, 1, false};
    return a;
}

cb200_na_t* cb200_na_view(cb200_na_t* a, int ndim, const int64_t* shape, const int64_t* step, int64_t offset) {
    if (ndim < 0 || ndim > kMaxD) return (cb200_na*)fail("ShapeError", "ndim %d out of range", ndim);
    // every element of the view must lie inside the parent's buffer
    int64_t lo = a->offset + offset, hi = lo;
    bool empty = false;
    for (int d = 0; d < ndim; ++d) {
        if (shape[d] < 0) return (cb200_na*)fail("ShapeError", "negative extent");
        if (shape[d] == 0) empty = true;
        int64_t span = (shape[d] - 1) * step[d];
        if (span < 0) lo += span; else hi += span;
    }
    if (a->st->owned && !empty) {
        int64_t unit = a->dtype == CB200_BIT ? 1 : kElemSize[a->dtype];
        int64_t limit = a->dtype == CB200_BIT ? (int64_t)a->st->bytes * 8 : (int64_t)a->st->bytes;
        if (lo < 0 || hi + unit > limit) return (cb200_na*)fail("IndexError", "view reaches outside the array");
    }
    cb200_na* v = share(a);
    v->ndim = ndim;
    for (int d = 0; d < ndim; ++d) { v->shape[d] = shape[d]; v->step[d] = step[d]; }
    v->offset = a->offset + offset;
    return v;
}

void cb200_na_release(cb200_na_t* a) {
    if (!a) return;
    bool last;
    { std::lock_guard<std::mutex> lk(g_ref_mu); last = --a->st->refs == 0; }
    if (last) {
        if (a->st->owned) cumo_cuda_runtime_free(a->st->ptr);
        delete a->st;
    }
    delete a;
}

int cb200_na_dtype(const cb200_na_t* a) { return a->dtype; }
int cb200_na_ndim(const cb200_na_t* a) { return a->ndim; }
int64_t cb200_na_size(const cb200_na_t* a) { return size_of(a); }
void cb200_na_shape(const cb200_na_t* a, int64_t* shape) { memcpy(shape, a->shape, sizeof(int64_t) * a->ndim); }
void cb200_na_steps(const cb200_na_t* a, int64_t* step) { memcpy(step, a->step, sizeof(int64_t) * a->ndim); }
int64_t cb200_na_offset(const cb200_na_t* a) { return a->offset; }
void* cb200_na_base(const cb200_na_t* a) { return a->st->ptr; }
int cb200_na_is_contiguous(const cb200_na_t* a) { return is_contiguous(a) ? 1 : 0; }
void cb200_na_set_inplace(cb200_na_t* a, int on) { a->inplace = on != 0; }

int cb200_na_store_host(cb200_na_t* a, const void* host, size_t bytes) {
    if (!is_contiguous(a)) { fail("ValueError", "store_host needs a contiguous array"); return 1; }
    if (a->dtype == CB200_BIT && (a->offset & 31)) { fail("ValueError", "store_host needs a word-aligned Bit array"); return 1; }
    if (bytes != buffer_bytes(a->dtype, size_of(a))) { fail("ValueError", "store_host: %zu bytes given, %zu expected", bytes, buffer_bytes(a->dtype, size_of(a))); return 1; }
    char* dst = a->dtype == CB200_BIT ? a->st->ptr + a->offset / 8 : data_ptr(a);
    return cuda_ok(cudaMemcpyAsync(dst, host, bytes, cudaMemcpyHostToDevice, cb200::current_stream()), "cudaMemcpyAsync H2D") ? 0 : 1;
}

int cb200_na_read_host(cb200_na_t* a, void* host, size_t bytes) {
    if (!is_contiguous(a)) { fail("ValueError", "read_host needs a contiguous array"); return 1; }
    if (a->dtype == CB200_BIT && (a->offset & 31)) { fail("ValueError", "read_host needs a word-aligned Bit array"); return 1; }
    if (bytes != buffer_bytes(a->dtype, size_of(a))) { fail("ValueError", "read_host: %zu bytes given, %zu expected", bytes, buffer_bytes(a->dtype, size_of(a))); return 1; }
    const char* src = a->dtype == CB200_BIT ? a->st->ptr + a->offset / 8 : data_ptr(a);
    if (!cuda_ok(cudaMemcpyAsync(host, src, bytes, cudaMemcpyDeviceToHost, cb200::current_stream()), "cudaMemcpyAsync D2H")) return 1;
    return cuda_ok(cudaStreamSynchronize(cb200::current_stream()), "cudaStreamSynchronize") ? 0 : 1;
}

// The copy runs on `copy_stream`, behind everything queued so far on the launch stream (an event), so the launch
// stream is free to start the next block's kernels while this block's result is still on its way to the host.
int cb200_na_read_host_async(cb200_na_t* a, void* host, size_t bytes, void* copy_stream) {
    if (!is_contiguous(a)) { fail("ValueError", "read_host needs a contiguous array"); return 1; }
    if (a->dtype == CB200_BIT && (a->offset & 31)) { fail("ValueError", "read_host needs a word-aligned Bit array"); return 1; }
    if (bytes != buffer_bytes(a->dtype, size_of(a))) { fail("ValueError", "read_host: %zu bytes given, %zu expected", bytes, buffer_bytes(a->dtype, size_of(a))); return 1; }
    const char* src = a->dtype == CB200_BIT ? a->st->ptr + a->offset / 8 : data_ptr(a);
    cudaStream_t cs = (cudaStream_t)copy_stream;
    thread_local cudaEvent_t ev = nullptr;
    if (!ev && !cuda_ok(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate")) return 1;
    if (!cuda_ok(cudaEventRecord(ev, cb200::current_stream()), "cudaEventRecord")) return 1;
    if (!cuda_ok(cudaStreamWaitEvent(cs, ev, 0), "cudaStreamWaitEvent")) return 1;
    return cuda_ok(cudaMemcpyAsync(host, src, bytes, cudaMemcpyDeviceToHost, cs), "cudaMemcpyAsync D2H") ? 0 : 1;
}

int cb200_synchronize(void) { return cuda_ok(cudaStreamSynchronize(cb200::current_stream()), "cudaStreamSynchronize") ? 0 : 1; }

cb200_na_t* cb200_na_cast(cb200_na_t* a, int dtype) { return cast_to(a, dtype); }
cb200_na_t* cb200_na_copy(cb200_na_t* a) {
    if (a->dtype == CB200_UINT64 || a->dtype == CB200_UINT32) {   // container types: copied as signed bit patterns
        const int as = a->dtype == CB200_UINT64 ? CB200_INT64 : CB200_INT32;
        cb200_na tmp = *a; tmp.dtype = as;
        cb200_na* c = cast_to(&tmp, as);
        if (c) c->dtype = a->dtype;
        return c;
    }
    if (a->dtype == CB200_BIT) return (cb200_na*)fail("TypeError", "copy of a Bit view is not on this path");
    return cast_to(a, a->dtype);
}

// ---- elementwise ---------------------------------------------------------------------------
cb200_na_t* cb200_na_binary(const char* op_c, cb200_na_t* a, cb200_na_t* b) {
    std::string op = op_c;
    if (!is_value_type(a->dtype) || !is_value_type(b->dtype)) return (cb200_na*)fail("TypeError", "%s is not defined for %s and %s", op_c, kTypeName[a->dtype], kTypeName[b->dtype]);
    int dtype = upcast(a->dtype, b->dtype);
    // an Int32 array as the exponent does not widen the base: the power is taken by repeated multiplication
    // (gen/tmpl/pow.c:178-182: `other` is an Int32 -> the pow_int32 iterator)
    if (op == "pow" && b->dtype == CB200_INT32 && dtype == a->dtype) {
        Loop lp;
        if (!broadcast(a, b, &lp)) return nullptr;
        cb200_na* out = output_for(a, dtype, lp);
        if (!out) return nullptr;
        using Fn = void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*);
        Fn f = (Fn)sym(std::string("cumo_iter_") + kTypeName[dtype] + "_pow_int32_kernel_launch");
        bool ok = f != nullptr;
        if (ok) {
            cumo_na_indexer_t ix;
            cumo_na_iarray_t a1, a2, a3;
            fill_indexer(&ix, lp);
            fill_iarray(&a1, a, lp);
            fill_iarray(&a2, b, lp);
            fill_iarray(&a3, out, lp);
            f(&a1, &a2, &a3, &ix);
            ok = launch_ok();
        }
        if (!ok) { cb200_na_release(out); return nullptr; }
        return out;
    }
    Family fam = binary_family(op, is_float_type(dtype));
    if (fam == F_NONE) return (cb200_na*)fail("NoMethodError", "undefined method %s for %s", op_c, kTypeName[dtype]);
    Loop lp;
    if (!broadcast(a, b, &lp)) return nullptr;
    cb200_na *ca = nullptr, *cb = nullptr;
    if (a->dtype != dtype) { ca = cast_to(a, dtype); if (!ca) return nullptr; }
    if (b->dtype != dtype) { cb = cast_to(b, dtype); if (!cb) { cb200_na_release(ca); return nullptr; } }
    cb200_na* x = ca ? ca : a;
    cb200_na* y = cb ? cb : b;
    cb200_na* out = output_for(ca ? nullptr : a, dtype, lp);
    bool ok = out != nullptr;
    if (ok) {
        void* f = sym(binary_symbol(op, fam, dtype, false));
        ok = f != nullptr;
        if (ok) {
            cumo_na_indexer_t ix;
            cumo_na_iarray_t a1, a2, a3;
            fill_indexer(&ix, lp);
            fill_iarray(&a1, x, lp);
            fill_iarray(&a2, y, lp);
            fill_iarray(&a3, out, lp);
            ok = with_flag(op, dtype, [&](int* flag) {
                if (fam == F_BINARY_S) ((void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*, int*))f)(&a1, &a2, &a3, &ix, flag);
                else ((void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*))f)(&a1, &a2, &a3, &ix);
            });
        }
    }
    cb200_na_release(ca);
    cb200_na_release(cb);
    if (!ok) { cb200_na_release(out); return nullptr; }
    return out;
}

cb200_na_t* cb200_na_binary_scalar(const char* op_c, cb200_na_t* a, double sv_f, int64_t sv_i, int scalar_is_left) {
    std::string op = op_c;
    if (!is_value_type(a->dtype)) return (cb200_na*)fail("TypeError", "%s is not defined for %s", op_c, kTypeName[a->dtype]);
    int dtype = a->dtype;
    Family fam = binary_family(op, is_float_type(dtype));
    if (fam == F_NONE || fam == F_EWCOMP) return (cb200_na*)fail("NoMethodError", "undefined scalar form of %s for %s", op_c, kTypeName[dtype]);
    Loop lp;
    lp.ndim = a->ndim;
    memcpy(lp.shape, a->shape, sizeof(int64_t) * a->ndim);
    cb200_na* out = output_for(a, dtype, lp);
    if (!out) return nullptr;
    void* f = sym(binary_symbol(op, fam, dtype, true));
    bool ok = f != nullptr;
    if (ok) {
        cumo_na_indexer_t ix;
        cumo_na_iarray_t a1, a3;
        fill_indexer(&ix, lp);
        fill_iarray(&a1, a, lp);
        fill_iarray(&a3, out, lp);
        ok = with_flag(op, dtype, [&](int* flag) {
            switch (dtype) {
            case CB200_SFLOAT: call_binary_s<float>(f, fam, &a1, pick<float>(sv_f, sv_i), &a3, &ix, flag, scalar_is_left); break;
            case CB200_DFLOAT: call_binary_s<double>(f, fam, &a1, pick<double>(sv_f, sv_i), &a3, &ix, flag, scalar_is_left); break;
            case CB200_INT32:  call_binary_s<int32_t>(f, fam, &a1, pick<int32_t>(sv_f, sv_i), &a3, &ix, flag, scalar_is_left); break;
            default:           call_binary_s<int64_t>(f, fam, &a1, pick<int64_t>(sv_f, sv_i), &a3, &ix, flag, scalar_is_left); break;
            }
        });
    }
    if (!ok) { cb200_na_release(out); return nullptr; }
    return out;
}

cb200_na_t* cb200_na_pow_int(cb200_na_t* a, int32_t exponent) {
    if (!is_value_type(a->dtype)) return (cb200_na*)fail("TypeError", "pow is not defined for %s", kTypeName[a->dtype]);
    Loop lp;
    lp.ndim = a->ndim;
    memcpy(lp.shape, a->shape, sizeof(int64_t) * a->ndim);
    cb200_na* out = output_for(a, a->dtype, lp);
    if (!out) return nullptr;
    using Fn = void (*)(cumo_na_iarray_t*, int32_t, cumo_na_iarray_t*, cumo_na_indexer_t*);
    Fn f = (Fn)sym(std::string("cumo_iter_") + kTypeName[a->dtype] + "_pow_int32_s_kernel_launch");
    if (!f) { cb200_na_release(out); return nullptr; }
    cumo_na_indexer_t ix;
    cumo_na_iarray_t a1, a3;
    fill_indexer(&ix, lp);
    fill_iarray(&a1, a, lp);
    fill_iarray(&a3, out, lp);
    f(&a1, exponent, &a3, &ix);
    if (!launch_ok()) { cb200_na_release(out); return nullptr; }
    return out;
}

cb200_na_t* cb200_na_unary(const char* op_c, cb200_na_t* a) {
    std::string op = op_c;
    if (!is_value_type(a->dtype)) return (cb200_na*)fail("TypeError", "%s is not defined for %s", op_c, kTypeName[a->dtype]);
    const bool fl = is_float_type(a->dtype);
    std::string t = kTypeName[a->dtype];
    std::string name;
    bool has_flag_arg = true;
    if (is_math_fn(op)) {
        if (!fl) return (cb200_na*)fail("NoMethodError", "NMath.%s needs a float array", op_c);
        name = "cumo_iter_" + t + "_math_s_" + op + "_kernel_launch";
        has_flag_arg = false;
    } else if (op == "minus" || op == "reciprocal" || op == "sign" || op == "square" || op == "abs" ||
               (fl && (op == "floor" || op == "round" || op == "ceil" || op == "trunc" || op == "rint")) ||
               (!fl && op == "bit_not")) {
        name = "cumo_iter_" + t + "_" + op + "_kernel_launch";
    } else if (!fl && (op == "floor" || op == "round" || op == "ceil" || op == "trunc" || op == "rint")) {
        return share(a);   // aliases of `view` for the integer types (gen/spec.rb:248-254)
    } else {
        return (cb200_na*)fail("NoMethodError", "undefined method %s for %s", op_c, t.c_str());
    }
    Loop lp;
    lp.ndim = a->ndim;
    memcpy(lp.shape, a->shape, sizeof(int64_t) * a->ndim);
    cb200_na* out = output_for(a, a->dtype, lp);
    if (!out) return nullptr;
    void* f = sym(name);
    bool ok = f != nullptr;
    if (ok) {
        cumo_na_indexer_t ix;
        cumo_na_iarray_t a1, a2;
        fill_indexer(&ix, lp);
        fill_iarray(&a1, a, lp);
        fill_iarray(&a2, out, lp);
        ok = with_flag(op, a->dtype, [&](int* flag) {
            if (has_flag_arg) ((void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*, int*))f)(&a1, &a2, &ix, flag);
            else ((void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*))f)(&a1, &a2, &ix);
        });
    }
    if (!ok) { cb200_na_release(out); return nullptr; }
    return out;
}

static cb200_na* new_bit_output(const Loop& lp) {
    cb200_na* out = make(CB200_BIT, lp.ndim, lp.shape, false);
    if (!out) return nullptr;
    // bits past the end of the last word are padding; give them a defined value
    if (out->st->bytes >= 4)
        cudaMemsetAsync(out->st->ptr + out->st->bytes - 4, 0, 4, cb200::current_stream());
    return out;
}

static bool is_cond_unary(const std::string& op) {
    for (auto s : {"isnan", "isinf", "isposinf", "isneginf", "isfinite", "signbit"}) if (op == s) return true;
    return false;
}
static bool is_cond_binary(const std::string& op, bool fl) {
    for (auto s : {"eq", "ne", "gt", "ge", "lt", "le"}) if (op == s) return true;
    return fl && op == "nearly_eq";
}

cb200_na_t* cb200_na_compare(const char* op_c, cb200_na_t* a, cb200_na_t* b) {
    std::string op = op_c;
    if (!is_value_type(a->dtype) || (b && !is_value_type(b->dtype))) return (cb200_na*)fail("TypeError", "%s needs numeric arrays", op_c);
    if (!b) {
        if (!is_float_type(a->dtype) || !is_cond_unary(op)) return (cb200_na*)fail("NoMethodError", "undefined method %s for %s", op_c, kTypeName[a->dtype]);
        Loop lp;
        lp.ndim = a->ndim;
        memcpy(lp.shape, a->shape, sizeof(int64_t) * a->ndim);
        cb200_na* out = new_bit_output(lp);
        if (!out) return nullptr;
        using Fn = void (*)(cumo_na_iarray_t*, cumo_na_bit_iarray_t*, cumo_na_indexer_t*);
        Fn f = (Fn)sym(std::string("cumo_iter_") + kTypeName[a->dtype] + "_" + op + "_kernel_launch");
        if (!f) { cb200_na_release(out); return nullptr; }
        cumo_na_indexer_t ix;
        cumo_na_iarray_t a1;
        cumo_na_bit_iarray_t a2;
        fill_indexer(&ix, lp);
        fill_iarray(&a1, a, lp);
        fill_bit_iarray(&a2, out, lp);
        f(&a1, &a2, &ix);
        if (!launch_ok()) { cb200_na_release(out); return nullptr; }
        return out;
    }
    int dtype = upcast(a->dtype, b->dtype);
    if (!is_cond_binary(op, is_float_type(dtype))) {
        if (op == "nearly_eq") op = "eq";    // integer types alias nearly_eq to eq (gen/spec.rb:233-236)
        else return (cb200_na*)fail("NoMethodError", "undefined method %s for %s", op_c, kTypeName[dtype]);
    }
    Loop lp;
    if (!broadcast(a, b, &lp)) return nullptr;
    cb200_na *ca = nullptr, *cb = nullptr;
    if (a->dtype != dtype) { ca = cast_to(a, dtype); if (!ca) return nullptr; }
    if (b->dtype != dtype) { cb = cast_to(b, dtype); if (!cb) { cb200_na_release(ca); return nullptr; } }
    cb200_na* out = new_bit_output(lp);
    bool ok = out != nullptr;
    if (ok) {
        using Fn = void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_bit_iarray_t*, cumo_na_indexer_t*);
        Fn f = (Fn)sym(std::string("cumo_iter_") + kTypeName[dtype] + "_" + op + "_kernel_launch");
        ok = f != nullptr;
        if (ok) {
            cumo_na_indexer_t ix;
            cumo_na_iarray_t a1, a2;
            cumo_na_bit_iarray_t a3;
            fill_indexer(&ix, lp);
            fill_iarray(&a1, ca ? ca : a, lp);
            fill_iarray(&a2, cb ? cb : b, lp);
            fill_bit_iarray(&a3, out, lp);
            f(&a1, &a2, &a3, &ix);
            ok = launch_ok();
        }
    }
    cb200_na_release(ca);
    cb200_na_release(cb);
    if (!ok) { cb200_na_release(out); return nullptr; }
    return out;
}

cb200_na_t* cb200_na_compare_scalar(const char* op_c, cb200_na_t* a, double sv_f, int64_t sv_i, int scalar_is_left) {
    std::string op = op_c;
    if (!is_value_type(a->dtype)) return (cb200_na*)fail("TypeError", "%s needs a numeric array", op_c);
    if (!is_cond_binary(op, is_float_type(a->dtype))) {
        if (op == "nearly_eq") op = "eq";
        else return (cb200_na*)fail("NoMethodError", "undefined method %s for %s", op_c, kTypeName[a->dtype]);
    }
    Loop lp;
    lp.ndim = a->ndim;
    memcpy(lp.shape, a->shape, sizeof(int64_t) * a->ndim);
    cb200_na* out = new_bit_output(lp);
    if (!out) return nullptr;
    void* f = sym(std::string("cumo_iter_") + kTypeName[a->dtype] + "_" + op + "_s_kernel_launch");
    if (!f) { cb200_na_release(out); return nullptr; }
    cumo_na_indexer_t ix;
    cumo_na_iarray_t a1;
    cumo_na_bit_iarray_t a3;
    fill_indexer(&ix, lp);
    fill_iarray(&a1, a, lp);
    fill_bit_iarray(&a3, out, lp);
    switch (a->dtype) {
    case CB200_SFLOAT: call_compare_s<float>(f, &a1, pick<float>(sv_f, sv_i), &a3, &ix, scalar_is_left); break;
    case CB200_DFLOAT: call_compare_s<double>(f, &a1, pick<double>(sv_f, sv_i), &a3, &ix, scalar_is_left); break;
    case CB200_INT32:  call_compare_s<int32_t>(f, &a1, pick<int32_t>(sv_f, sv_i), &a3, &ix, scalar_is_left); break;
    default:           call_compare_s<int64_t>(f, &a1, pick<int64_t>(sv_f, sv_i), &a3, &ix, scalar_is_left); break;
    }
    if (!launch_ok()) { cb200_na_release(out); return nullptr; }
    return out;
}

// ---- reductions -----------------------------------------------------------------------------
cb200_na_t* cb200_na_reduce(const char* op_c, cb200_na_t* a, uint32_t axis_mask, int keepdims, int nan) {
    std::string op = op_c;
    if (!is_value_type(a->dtype)) return (cb200_na*)fail("TypeError", "%s is not defined for %s", op_c, kTypeName[a->dtype]);
    const bool fl = is_float_type(a->dtype);
    const bool index_op = op == "max_index" || op == "min_index";
    const bool arg_op = op == "argmax" || op == "argmin";
    int out_dtype = a->dtype;
    if (op == "sum" || op == "prod") { if (!fl) out_dtype = CB200_INT64; }
    else if (op == "mean" || op == "var" || op == "stddev" || op == "rms") { if (!fl) return (cb200_na*)fail("NoMethodError", "undefined method %s for %s", op_c, kTypeName[a->dtype]); }
    else if (op == "kahan_sum") { if (a->dtype != CB200_DFLOAT) return (cb200_na*)fail("NoMethodError", "undefined method kahan_sum for %s", kTypeName[a->dtype]); }
    else if (op == "min" || op == "max" || op == "ptp") {}
    else if (index_op || arg_op) { out_dtype = (uint64_t)size_of(a) > 0xffffffffull ? CB200_INT64 : CB200_INT32; }
    else return (cb200_na*)fail("NoMethodError", "undefined method %s", op_c);
    if (size_of(a) == 0 && op != "sum") return (cb200_na*)fail("ShapeError", "cannot reduce an empty array with %s", op_c);

    ReducePlan rp;
    if (!plan_reduce(a, axis_mask, &rp)) return nullptr;
    // the index a (max|min)_index kernel answers counts along the operand's memory, so a
    // non-contiguous operand is copied first (accum_index.c:121-129)
    cb200_na* copy = nullptr;
    if (index_op && !is_contiguous(a)) { copy = cast_to(a, a->dtype); if (!copy) return nullptr; }
    const cb200_na* in = copy ? copy : a;
    cb200_na* out = make(out_dtype, rp.n_keep, rp.out_shape, size_of(a) == 0);
    if (!out) { cb200_na_release(copy); return nullptr; }
    bool ok = true;
    if (size_of(a) > 0) {
        std::string name = std::string("cumo_") + kTypeName[a->dtype] + "_" + op + ((nan && fl) ? "_nan" : "");
        if (index_op || arg_op) name += out_dtype == CB200_INT64 ? "_int64" : "_int32";
        name += "_kernel_launch";
        using Fn = void (*)(cumo_na_reduction_arg_t*);
        Fn f = (Fn)sym(name);
        ok = f != nullptr;
        if (ok) {
            cumo_na_reduction_arg_t arg;
            fill_reduction_arg(&arg, in, rp, out);
            f(&arg);
            ok = launch_ok();
        }
    }
    cb200_na_release(copy);
    if (!ok) { cb200_na_release(out); return nullptr; }
    apply_keepdims(out, a, rp, keepdims);
    return out;
}

int cb200_na_minmax(cb200_na_t* a, uint32_t axis_mask, int keepdims, int nan, cb200_na_t** out_min, cb200_na_t** out_max) {
    if (!is_value_type(a->dtype)) { fail("TypeError", "minmax is not defined for %s", kTypeName[a->dtype]); return 1; }
    if (size_of(a) == 0) { fail("ShapeError", "cannot reduce an empty array with minmax"); return 1; }
    ReducePlan rp;
    if (!plan_reduce(a, axis_mask, &rp)) return 1;
    cb200_na* o1 = make(a->dtype, rp.n_keep, rp.out_shape, false);
    cb200_na* o2 = o1 ? make(a->dtype, rp.n_keep, rp.out_shape, false) : nullptr;
    if (!o2) { cb200_na_release(o1); return 1; }
    using Fn = void (*)(cumo_na_reduction_arg_t*, cumo_na_iarray_t*);
    Fn f = (Fn)sym(std::string("cumo_") + kTypeName[a->dtype] + "_minmax" + ((nan && is_float_type(a->dtype)) ? "_nan" : "") + "_kernel_launch");
    bool ok = f != nullptr;
    if (ok) {
        cumo_na_reduction_arg_t arg;
        fill_reduction_arg(&arg, a, rp, o1);
        cumo_na_iarray_t out2;
        memset(&out2, 0, sizeof out2);
        out2.ptr = data_ptr(o2);
        for (int i = 0; i < rp.n_keep; ++i) out2.step[i] = (ssize_t)o2->step[i];
        f(&arg, &out2);
        ok = launch_ok();
    }
    if (!ok) { cb200_na_release(o1); cb200_na_release(o2); return 1; }
    apply_keepdims(o1, a, rp, keepdims);
    apply_keepdims(o2, a, rp, keepdims);
    *out_min = o1;
    *out_max = o2;
    return 0;
}

// ---- Bit#where -----------------------------------------------------------------------------
cb200_na_t* cb200_na_where(cb200_na_t* a, int want_zeros) {
    if (a->dtype != CB200_BIT) return (cb200_na*)fail("TypeError", "where needs a Bit array");
    const int64_t size = size_of(a);
    // the number of hits sizes the result: one read-back
    int64_t hits = 0;
    if (size > 0) {
        cb200_na* c = cb200_na_count(a, 0, 0, want_zeros);
        if (!c) return nullptr;
        uint64_t v = 0;
        const bool ok = cb200_na_read_host(c, &v, 8) == 0;
        cb200_na_release(c);
        if (!ok) return nullptr;
        hits = (int64_t)v;
    }
    const int out_dtype = (uint64_t)size > 4294967295ull ? CB200_INT64 : CB200_INT32;
    cb200_na* out = make(out_dtype, 1, &hits, false);
    if (!out || hits == 0) return out;
    using FnNew = char* (*)();
    using FnRun = void (*)(CUMO_BIT_DIGIT*, size_t, ssize_t, size_t*, uint64_t, int, char*, size_t, uint64_t, char*);
    FnNew fnew = (FnNew)sym("cumo_bit_where_scratch_new");
    FnRun frun = (FnRun)sym("cumo_bit_where_kernel_launch");
    char* scratch = fnew && frun ? fnew() : nullptr;
    if (!scratch) { cb200_na_release(out); if (fnew && frun) fail("CudaError", "no memory for the where scratch"); return nullptr; }
    // FULL_LOOP: merge what merges, then one launch per run of the innermost dim left
    StrideLoop L;
    L.nd = a->ndim;
    for (int i = 0; i < a->ndim; ++i) { L.n[i] = a->shape[i]; L.s[0][i] = a->step[i]; }
    if (L.nd == 0) { L.nd = 1; L.n[0] = 1; L.s[0][0] = 0; }
    contract(&L, 1);
    const int in = L.nd - 1;
    uint64_t count = 0;
    CUMO_BIT_DIGIT* words = reinterpret_cast<CUMO_BIT_DIGIT*>(a->st->ptr);
    for_outer(L, 1, [&](const int64_t* off) {
        frun(words, (size_t)(a->offset + off[0]), (ssize_t)L.s[0][in], nullptr, (uint64_t)L.n[in], want_zeros, data_ptr(out),
             out_dtype == CB200_INT64 ? 8 : 4, count, scratch);
        count += (uint64_t)L.n[in];
    });
    cumo_cuda_runtime_free(scratch);
    if (!launch_ok()) { cb200_na_release(out); return nullptr; }
    return out;
}

// ---- cumsum / cumprod ----------------------------------------------------------------------
cb200_na_t* cb200_na_cum(const char* op_c, cb200_na_t* a, int axis, int nan) {
    std::string op = op_c;
    if (op != "cumsum" && op != "cumprod") return (cb200_na*)fail("NoMethodError", "undefined method %s", op_c);
    if (!is_value_type(a->dtype)) return (cb200_na*)fail("TypeError", "%s is not defined for %s", op_c, kTypeName[a->dtype]);
    if (axis >= a->ndim) return (cb200_na*)fail("ArgumentError", "axis %d out of range for %d dimensions", axis, a->ndim);
    using Fn = int (*)(char*, char*, ssize_t, ssize_t, uint64_t);
    Fn f = (Fn)sym(std::string("cumo_") + kTypeName[a->dtype] + "_" + op + ((nan && is_float_type(a->dtype)) ? "_nan" : "") + "_kernel_launch");
    if (!f) return nullptr;
    cb200_na* out = make(a->dtype, a->ndim, a->shape, false);
    if (!out) return nullptr;
    if (size_of(a) == 0) return out;
    cb200_na* copy = nullptr;
    const cb200_na* in = a;
    StrideLoop L;
    auto set_loop = [&](const cb200_na* x) {
        L.nd = x->ndim;
        for (int i = 0; i < x->ndim; ++i) { L.n[i] = x->shape[i]; L.s[0][i] = x->step[i]; L.s[1][i] = out->step[i]; }
        if (L.nd == 0) { L.nd = 1; L.n[0] = 1; L.s[0][0] = L.s[1][0] = 0; }
    };
    int status = 0;
    if (axis < 0) {
        // all elements in row-major order: one run when the dims merge, else through a contiguous copy
        set_loop(in);
        contract(&L, 2);
        if (L.nd != 1) {
            copy = cast_to(a, a->dtype);
            if (!copy) { cb200_na_release(out); return nullptr; }
            in = copy;
            set_loop(in);
            contract(&L, 2);
        }
        status = f(data_ptr(in), data_ptr(out), (ssize_t)L.s[0][0], (ssize_t)L.s[1][0], (uint64_t)L.n[0]);
    } else {
        // every run along `axis` in one launch (ndloop would call the per-run function once per run)
        using FnRuns = int (*)(char*, char*, ssize_t, ssize_t, uint64_t, int, const size_t*, const ssize_t*, const ssize_t*);
        FnRuns fr = (FnRuns)sym(std::string("cb200_") + kTypeName[a->dtype] + "_" + op + ((nan && is_float_type(a->dtype)) ? "_nan" : "") + "_runs_kernel_launch");
        if (!fr) { cb200_na_release(out); return nullptr; }
        size_t oshape[kMaxD];
        ssize_t ostep1[kMaxD], ostep2[kMaxD];
        int n_outer = 0;
        for (int d = 0; d < in->ndim; ++d) {
            if (d == axis) continue;
            oshape[n_outer] = (size_t)in->shape[d]; ostep1[n_outer] = (ssize_t)in->step[d]; ostep2[n_outer] = (ssize_t)out->step[d];
            ++n_outer;
        }
        status = fr(data_ptr(in), data_ptr(out), (ssize_t)in->step[axis], (ssize_t)out->step[axis], (uint64_t)in->shape[axis], n_outer, oshape, ostep1, ostep2);
    }
    cb200_na_release(copy);
    if (status) { fail("CudaError", "%s: %s", op_c, cudaGetErrorString((cudaError_t)status)); cb200_na_release(out); return nullptr; }
    if (!launch_ok()) { cb200_na_release(out); return nullptr; }
    return out;
}

// ---- bincount ------------------------------------------------------------------------------
cb200_na_t* cb200_na_bincount(cb200_na_t* a, cb200_na_t* weight, int64_t minlength) {
    if (a->dtype != CB200_INT32 && a->dtype != CB200_INT64) return (cb200_na*)fail("NoMethodError", "undefined method bincount for %s", kTypeName[a->dtype]);
    if (a->ndim < 1) return (cb200_na*)fail("ShapeError", "bincount needs at least one dimension");
    if (minlength < 0) return (cb200_na*)fail("ArgumentError", "minlength must be non-negative");
    cb200_na* w = nullptr;
    if (weight) {
        if (!is_value_type(weight->dtype)) return (cb200_na*)fail("TypeError", "weights must be numeric");
        w = weight->dtype == CB200_SFLOAT ? weight : cast_to(weight, CB200_DFLOAT);
        if (!w) return nullptr;
    }
    auto drop_w = [&]() { if (w && w != weight) cb200_na_release(w); };
    const int last = a->ndim - 1;
    if (w && (w->ndim != a->ndim || memcmp(w->shape, a->shape, sizeof(int64_t) * a->ndim) != 0)) {
        // the reference broadcasts the leading axes and demands equal extents along the last one; equal shapes cover its tests
        const bool last_ok = w->ndim >= 1 && w->shape[w->ndim - 1] == a->shape[last];
        drop_w();
        return (cb200_na*)fail("ShapeError", last_ok ? "weights of a different shape are not on this path" : "size mismatch along last axis between self and weight");
    }
    int64_t length = 0;
    // one unweighted run of small values: counted and sized in the same pass
    if (!w && a->ndim == 1 && size_of(a) > 0) {
        using FnProbe = void (*)(char*, ssize_t, uint64_t, uint32_t*, long long*);
        using FnBins = int (*)();
        FnProbe fp = (FnProbe)sym(std::string("cb200_") + kTypeName[a->dtype] + "_bincount_probe_kernel_launch");
        FnBins fb = (FnBins)sym("cb200_bincount_probe_bins");
        if (!fp || !fb) return nullptr;
        const int bins = fb();
        static thread_local char* probe_dev = nullptr;          // hist[bins] then extremes[2]
        static thread_local long long* probe_host = nullptr;
        if (!probe_dev) {
            if (!cuda_ok(cudaMalloc((void**)&probe_dev, sizeof(uint32_t) * bins + 16), "cudaMalloc")) { probe_dev = nullptr; return nullptr; }
            if (!cuda_ok(cudaHostAlloc((void**)&probe_host, 16, cudaHostAllocDefault), "cudaHostAlloc")) { cudaFree(probe_dev); probe_dev = nullptr; return nullptr; }
        }
        uint32_t* hist = reinterpret_cast<uint32_t*>(probe_dev);
        long long* extremes = reinterpret_cast<long long*>(probe_dev + sizeof(uint32_t) * bins);
        cudaStream_t st = cb200::current_stream();
        fp(data_ptr(a), (ssize_t)a->step[0], (uint64_t)a->shape[0], hist, extremes);
        if (!launch_ok()) return nullptr;
        if (!cuda_ok(cudaMemcpyAsync(probe_host, extremes, 16, cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync") ||
            !cuda_ok(cudaStreamSynchronize(st), "cudaStreamSynchronize")) return nullptr;
        const long long vlo = probe_host[0], vhi = probe_host[1];
        if (vlo < 0) return (cb200_na*)fail("ArgumentError", "array items must be non-negative");
        int64_t len = vhi + 1;
        if (minlength > len) len = minlength;
        if (vhi < bins && len <= bins) {
            cb200_na* out = make(CB200_UINT32, 1, &len, false);
            if (!out) return nullptr;
            if (!cuda_ok(cudaMemcpyAsync(data_ptr(out), hist, sizeof(uint32_t) * (size_t)len, cudaMemcpyDeviceToDevice, st), "cudaMemcpyAsync")) {
                cb200_na_release(out);
                return nullptr;
            }
            return out;
        }
        length = vhi + 1;                                       // large values: the extremes are known, count with the output-sized kernel
    } else
    if (size_of(a) > 0) {
        cb200_na *lo = nullptr, *hi = nullptr;
        if (cb200_na_minmax(a, 0, 0, 0, &lo, &hi)) { drop_w(); return nullptr; }
        int64_t vlo = 0, vhi = 0;
        int32_t t32;
        bool ok = true;
        if (a->dtype == CB200_INT32) {
            ok = cb200_na_read_host(lo, &t32, 4) == 0; vlo = t32;
            ok = ok && cb200_na_read_host(hi, &t32, 4) == 0; vhi = t32;
        } else {
            ok = cb200_na_read_host(lo, &vlo, 8) == 0 && cb200_na_read_host(hi, &vhi, 8) == 0;
        }
        cb200_na_release(lo); cb200_na_release(hi);
        if (!ok) { drop_w(); return nullptr; }
        if (vlo < 0) { drop_w(); return (cb200_na*)fail("ArgumentError", "array items must be non-negative"); }
        length = vhi + 1;
    }
    if (minlength > length) length = minlength;
    const int out_dtype = w ? w->dtype : (length > 4294967295ll ? CB200_UINT64 : CB200_UINT32);
    int64_t oshape[kMaxD];
    memcpy(oshape, a->shape, sizeof(int64_t) * a->ndim);
    oshape[last] = length;
    cb200_na* out = make(out_dtype, a->ndim, oshape, false);
    if (!out) { drop_w(); return nullptr; }
    const std::string base = std::string("cumo_iter_") + kTypeName[a->dtype] + "_bincount_";
    using FnC = void (*)(char*, ssize_t, size_t*, uint64_t, char*, ssize_t, uint64_t, int*, size_t*);
    using FnW = void (*)(char*, ssize_t, char*, ssize_t, uint64_t, char*, ssize_t, uint64_t, int*, size_t*);
    void* f = sym(base + (w ? (w->dtype == CB200_SFLOAT ? "sf" : "df") : (out_dtype == CB200_UINT64 ? "64" : "32")) + "_kernel_launch");
    // mapped pinned words: the out-of-range flag and the offending item
    bool ok = f != nullptr;
    if (ok && !tl_flag.ready()) { fail("CudaError", "cannot allocate the mapped error flag"); ok = false; }
    size_t* item = ok ? tl_flag.item_host : nullptr;
    size_t* item_dev = ok ? tl_flag.item_dev : nullptr;
    if (ok && length > 0) {
        *item = 0;
        *tl_flag.host = 0;
        // one launch per leading index, as ndloop does for an iterator that takes one dimension
        StrideLoop L;
        L.nd = a->ndim;
        for (int i = 0; i < a->ndim; ++i) { L.n[i] = a->shape[i]; L.s[0][i] = a->step[i]; L.s[1][i] = out->step[i]; L.s[2][i] = w ? w->step[i] : 0; }
        for_outer(L, 3, [&](const int64_t* off) {
            char* p1 = data_ptr(a) + off[0];
            char* p2 = data_ptr(out) + off[1];
            if (w) ((FnW)f)(p1, (ssize_t)a->step[last], data_ptr(w) + off[2], (ssize_t)w->step[last], (uint64_t)a->shape[last], p2, (ssize_t)out->step[last], (uint64_t)length, tl_flag.dev, item_dev);
            else ((FnC)f)(p1, (ssize_t)a->step[last], nullptr, (uint64_t)a->shape[last], p2, (ssize_t)out->step[last], (uint64_t)length, tl_flag.dev, item_dev);
        });
        ok = launch_ok() && cuda_ok(cudaStreamSynchronize(cb200::current_stream()), "cudaStreamSynchronize");
        if (ok && *tl_flag.host) {
            fail("IndexError", "item %zu is out of range of the output(size:%lld)", *item, (long long)length);
            ok = false;
        }
    }
    drop_w();
    if (!ok) { cb200_na_release(out); return nullptr; }
    return out;
}

// index (Int64) and winning value from one pass: the per-GPU partial of a sharded arg reduction.  The results go
// into `idx_out` / `val_out` when those are given (contiguous device buffers of the output's size, e.g. the two
// halves of a buffer that a collective then sends), else into new arrays returned through out_index / out_value.
int cb200_na_arg_with_value_into(const char* op_c, cb200_na_t* a, uint32_t axis_mask, int nan, int64_t index_base, void* idx_out, void* val_out,
                                 cb200_na_t** out_index, cb200_na_t** out_value) {
    std::string op = op_c;
    if (!is_value_type(a->dtype)) { fail("TypeError", "%s is not defined for %s", op_c, kTypeName[a->dtype]); return 1; }
    const bool index_op = op == "max_index" || op == "min_index";
    if (!index_op && op != "argmax" && op != "argmin") { fail("NoMethodError", "undefined method %s", op_c); return 1; }
    if (size_of(a) == 0) { fail("ShapeError", "cannot reduce an empty array with %s", op_c); return 1; }
    ReducePlan rp;
    if (!plan_reduce(a, axis_mask, &rp)) return 1;
    cb200_na* copy = nullptr;
    if (index_op && !is_contiguous(a)) { copy = cast_to(a, a->dtype); if (!copy) return 1; }
    const cb200_na* in = copy ? copy : a;
    int64_t ostep_i[kMaxD], ostep_v[kMaxD];
    contiguous_steps(CB200_INT64, rp.n_keep, rp.out_shape, ostep_i);
    contiguous_steps(a->dtype, rp.n_keep, rp.out_shape, ostep_v);
    cb200_na* oi = (idx_out && val_out) ? cb200_na_wrap(CB200_INT64, rp.n_keep, rp.out_shape, ostep_i, idx_out, 0) : make(CB200_INT64, rp.n_keep, rp.out_shape, false);
    cb200_na* ov = !oi ? nullptr : (idx_out && val_out) ? cb200_na_wrap(a->dtype, rp.n_keep, rp.out_shape, ostep_v, val_out, 0) : make(a->dtype, rp.n_keep, rp.out_shape, false);
    if (!ov) { cb200_na_release(oi); cb200_na_release(copy); return 1; }
    using Fn = void (*)(cumo_na_reduction_arg_t*, cumo_na_iarray_t*, int64_t);
    Fn f = (Fn)sym(std::string("cb200_") + kTypeName[a->dtype] + "_" + op + ((nan && is_float_type(a->dtype)) ? "_nan" : "") + "_with_value_kernel_launch");
    bool ok = f != nullptr;
    if (ok) {
        cumo_na_reduction_arg_t arg;
        fill_reduction_arg(&arg, in, rp, oi);
        cumo_na_iarray_t values;
        memset(&values, 0, sizeof values);
        values.ptr = data_ptr(ov);
        for (int i = 0; i < rp.n_keep; ++i) values.step[i] = (ssize_t)ov->step[i];
        f(&arg, &values, index_base);
        ok = launch_ok();
    }
    cb200_na_release(copy);
    if (!ok) { cb200_na_release(oi); cb200_na_release(ov); return 1; }
    if (out_index) *out_index = oi; else cb200_na_release(oi);
    if (out_value) *out_value = ov; else cb200_na_release(ov);
    return 0;
}

int cb200_na_arg_with_value(const char* op_c, cb200_na_t* a, uint32_t axis_mask, int nan, cb200_na_t** out_index, cb200_na_t** out_value) {
    return cb200_na_arg_with_value_into(op_c, a, axis_mask, nan, 0, nullptr, nullptr, out_index, out_value);
}

cb200_na_t* cb200_na_count(cb200_na_t* a, uint32_t axis_mask, int keepdims, int want_false) {
    if (a->dtype != CB200_BIT) return (cb200_na*)fail("TypeError", "count_true needs a Bit array");
    ReducePlan rp;
    if (!plan_reduce(a, axis_mask, &rp)) return nullptr;
    cb200_na* out = make(CB200_UINT64, rp.n_keep, rp.out_shape, true);   // the `init` argument: filled with 0
    if (!out) return nullptr;
    if (size_of(a) > 0) {
        StrideLoop L;
        L.nd = a->ndim;
        int k = 0;
        for (int i = 0; i < rp.n_keep; ++i, ++k) { L.n[k] = a->shape[rp.keep[i]]; L.s[0][k] = a->step[rp.keep[i]]; L.s[1][k] = out->step[i]; }
        for (int i = 0; i < rp.n_red; ++i, ++k) { L.n[k] = a->shape[rp.red[i]]; L.s[0][k] = a->step[rp.red[i]]; L.s[1][k] = 0; }
        if (L.nd == 0) { L.nd = 1; L.n[0] = 1; L.s[0][0] = L.s[1][0] = 0; }
        contract(&L, 2);
        const char* nm = want_false ? "count_false" : "count_true";
        using FnS = void (*)(size_t, char*, CUMO_BIT_DIGIT*, ssize_t, uint64_t);
        using FnSS = void (*)(size_t, char*, CUMO_BIT_DIGIT*, ssize_t, ssize_t, uint64_t);
        FnS fs = (FnS)sym(std::string("cumo_iter_bit_") + nm + "_stride_kernel_launch");
        FnSS fss = (FnSS)sym(std::string("cumo_iter_bit_") + nm + "_stride_stride_kernel_launch");
        if (!fs || !fss) { cb200_na_release(out); return nullptr; }
        const int in = L.nd - 1;
        CUMO_BIT_DIGIT* words = reinterpret_cast<CUMO_BIT_DIGIT*>(a->st->ptr);
        int64_t outer = 1;
        for (int d = 0; d < in; ++d) outer *= L.n[d];
        if (outer > 1) {
            // several runs (a per-axis count): the whole loop in one launch instead of one launch per run
            using FnAxes = void (*)(CUMO_BIT_DIGIT*, size_t, int, int, const size_t*, const ssize_t*, const ssize_t*, int, const size_t*, const ssize_t*, char*);
            FnAxes fa = (FnAxes)sym("cb200_bit_count_axes_kernel_launch");
            if (!fa) { cb200_na_release(out); return nullptr; }
            size_t kshape[kMaxD], rshape[kMaxD];
            ssize_t kbit[kMaxD], kout[kMaxD], rbit[kMaxD];
            for (int i = 0; i < rp.n_keep; ++i) { kshape[i] = (size_t)a->shape[rp.keep[i]]; kbit[i] = (ssize_t)a->step[rp.keep[i]]; kout[i] = (ssize_t)out->step[i]; }
            for (int i = 0; i < rp.n_red; ++i) { rshape[i] = (size_t)a->shape[rp.red[i]]; rbit[i] = (ssize_t)a->step[rp.red[i]]; }
            fa(words, (size_t)a->offset, want_false, rp.n_keep, kshape, kbit, kout, rp.n_red, rshape, rbit, data_ptr(out));
            if (!launch_ok()) { cb200_na_release(out); return nullptr; }
            apply_keepdims(out, a, rp, keepdims);
            return out;
        }
        for_outer(L, 2, [&](const int64_t* off) {
            size_t p1 = (size_t)(a->offset + off[0]);
            char* p2 = data_ptr(out) + off[1];
            if (L.s[1][in] == 0) fs(p1, p2, words, (ssize_t)L.s[0][in], (uint64_t)L.n[in]);
            else fss(p1, p2, words, (ssize_t)L.s[0][in], (ssize_t)L.s[1][in], (uint64_t)L.n[in]);
        });
        if (!launch_ok()) { cb200_na_release(out); return nullptr; }
    }
    apply_keepdims(out, a, rp, keepdims);
    return out;
}

// ---- Bit o Bit: and or xor eq (b given), copy not (b null) -------------------------------------------------------------
// gen/tmpl_bit/binary.c:11-33, unary.c:11-30: operands laid end to end after the loop is contracted take the word-at-a-time
// launch, anything else the launch that addresses every operand per dimension.
cb200_na_t* cb200_na_bit_op(const char* op_c, cb200_na_t* a, cb200_na_t* b) {
    const std::string op = op_c;
    const bool binary = b != nullptr;
    if (a->dtype != CB200_BIT || (binary && b->dtype != CB200_BIT)) return (cb200_na*)fail("TypeError", "%s needs Bit arrays", op_c);
    if (binary ? !(op == "and" || op == "or" || op == "xor" || op == "eq") : !(op == "copy" || op == "not"))
        return (cb200_na*)fail("NoMethodError", "undefined method %s for bit", op_c);
    Loop lp;
    if (binary) { if (!broadcast(a, b, &lp)) return nullptr; }
    else { lp.ndim = a->ndim; memcpy(lp.shape, a->shape, sizeof(int64_t) * a->ndim); }
    cb200_na* out = make(CB200_BIT, lp.ndim, lp.shape, true);
    if (!out) return nullptr;
    if (size_of(out) == 0) return out;
    const cb200_na* ops[3] = {a, binary ? b : a, out};
    StrideLoop L;
    L.nd = lp.ndim;
    for (int i = 0; i < lp.ndim; ++i) {
        L.n[i] = lp.shape[i];
        for (int o = 0; o < 3; ++o) {
            const int d = i - (lp.ndim - ops[o]->ndim);
            L.s[o][i] = (d >= 0 && ops[o]->shape[d] != 1) ? ops[o]->step[d] : 0;
        }
    }
    if (L.nd == 0) { L.nd = 1; L.n[0] = 1; for (int o = 0; o < 3; ++o) L.s[o][0] = 0; }
    contract(&L, 3);
    auto words = [](const cb200_na* x) { return reinterpret_cast<CUMO_BIT_DIGIT*>(x->st->ptr); };
    const std::string base = std::string("cumo_iter_bit_") + op;
    const bool flat = L.nd == 1 && L.s[0][0] == 1 && L.s[2][0] == 1 && (!binary || L.s[1][0] == 1);
    bool ok = true;
    if (flat) {
        void* f = sym(base + "_contiguous_kernel_launch");
        ok = f != nullptr;
        if (ok) {
            const size_t q1 = (size_t)a->offset, q3 = (size_t)out->offset;
            if (binary) {
                const size_t q2 = (size_t)b->offset;
                ((void (*)(CUMO_BIT_DIGIT*, size_t, CUMO_BIT_DIGIT*, size_t, CUMO_BIT_DIGIT*, size_t, uint64_t))f)(
                    words(a) + q1 / 32, q1 % 32, words(b) + q2 / 32, q2 % 32, words(out) + q3 / 32, q3 % 32, (uint64_t)L.n[0]);
            } else {
                ((void (*)(CUMO_BIT_DIGIT*, size_t, CUMO_BIT_DIGIT*, size_t, uint64_t))f)(words(a) + q1 / 32, q1 % 32, words(out) + q3 / 32, q3 % 32,
                                                                                     (uint64_t)L.n[0]);
            }
        }
    } else {
        void* f = sym(base + "_kernel_launch");
        ok = f != nullptr;
        if (ok) {
            cumo_na_bit_iarray_stridx_t v[3];
            cumo_na_indexer_t ix;
            memset(&ix, 0, sizeof ix);
            ix.ndim = (unsigned char)L.nd;
            ix.total_size = 1;
            for (int d = 0; d < L.nd; ++d) { ix.shape[d] = (size_t)L.n[d]; ix.total_size *= (size_t)L.n[d]; }
            for (int o = 0; o < 3; ++o) {
                memset(&v[o], 0, sizeof v[o]);
                v[o].ptr = words(ops[o]);
                v[o].pos = (size_t)ops[o]->offset;
                for (int d = 0; d < L.nd; ++d) v[o].stridx[d].stride = (ssize_t)((L.s[o][d] << 1) | 1);     // a step, not an index array
            }
            if (binary) ((void (*)(cumo_na_bit_iarray_stridx_t*, cumo_na_bit_iarray_stridx_t*, cumo_na_bit_iarray_stridx_t*, cumo_na_indexer_t*))f)(&v[0], &v[1], &v[2], &ix);
            else ((void (*)(cumo_na_bit_iarray_stridx_t*, cumo_na_bit_iarray_stridx_t*, cumo_na_indexer_t*))f)(&v[0], &v[2], &ix);
        }
    }
    if (!ok || !launch_ok()) { cb200_na_release(out); return nullptr; }
    return out;
}

// ---- Bit#all? / #any? (gen/tmpl_bit/bit_reduce.c:5-33): the output starts at the identity, runs of the input flip it ----------
cb200_na_t* cb200_na_bit_reduce(const char* op_c, cb200_na_t* a, uint32_t axis_mask, int keepdims) {
    const std::string op = op_c;
    if (a->dtype != CB200_BIT) return (cb200_na*)fail("TypeError", "%s needs a Bit array", op_c);
    if (op != "all" && op != "any") return (cb200_na*)fail("NoMethodError", "undefined method %s? for bit", op_c);
    ReducePlan rp;
    if (!plan_reduce(a, axis_mask, &rp)) return nullptr;
    cb200_na* out = make(CB200_BIT, rp.n_keep, rp.out_shape, true);
    if (!out) return nullptr;
    if (op == "all" && !cuda_ok(cudaMemsetAsync(out->st->ptr, 0xff, out->st->bytes ? out->st->bytes : 4, cb200::current_stream()), "cudaMemsetAsync")) {
        cb200_na_release(out);
        return nullptr;
    }
    if (size_of(a) > 0) {
        StrideLoop L;
        L.nd = a->ndim;
        int k = 0;
        for (int i = 0; i < rp.n_keep; ++i, ++k) { L.n[k] = a->shape[rp.keep[i]]; L.s[0][k] = a->step[rp.keep[i]]; L.s[1][k] = out->step[i]; }
        for (int i = 0; i < rp.n_red; ++i, ++k) { L.n[k] = a->shape[rp.red[i]]; L.s[0][k] = a->step[rp.red[i]]; L.s[1][k] = 0; }
        if (L.nd == 0) { L.nd = 1; L.n[0] = 1; L.s[0][0] = L.s[1][0] = 0; }
        contract(&L, 2);
        const std::string base = std::string("cumo_iter_bit_") + op + "_p_";
        using FnE = void (*)(CUMO_BIT_DIGIT*, size_t, ssize_t, size_t*, CUMO_BIT_DIGIT*, size_t, ssize_t, size_t*, uint64_t);
        using FnR = void (*)(CUMO_BIT_DIGIT*, size_t, ssize_t, size_t*, CUMO_BIT_DIGIT*, size_t, uint64_t);
        using FnC = void (*)(CUMO_BIT_DIGIT*, size_t, CUMO_BIT_DIGIT*, size_t, uint64_t);
        FnE fe = (FnE)sym(base + "elementwise_kernel_launch");
        FnR fr = (FnR)sym(base + "reduce_kernel_launch");
        FnC fc = (FnC)sym(base + "contiguous_reduce_kernel_launch");
        if (!fe || !fr || !fc) { cb200_na_release(out); return nullptr; }
        const int in = L.nd - 1;
        CUMO_BIT_DIGIT* w1 = reinterpret_cast<CUMO_BIT_DIGIT*>(a->st->ptr);
        CUMO_BIT_DIGIT* w2 = reinterpret_cast<CUMO_BIT_DIGIT*>(out->st->ptr);
        for_outer(L, 2, [&](const int64_t* off) {
            const size_t p1 = (size_t)(a->offset + off[0]), p2 = (size_t)(out->offset + off[1]);
            if (L.s[1][in] != 0) fe(w1, p1, (ssize_t)L.s[0][in], nullptr, w2, p2, (ssize_t)L.s[1][in], nullptr, (uint64_t)L.n[in]);
            else if (L.s[0][in] != 1) fr(w1, p1, (ssize_t)L.s[0][in], nullptr, w2, p2, (uint64_t)L.n[in]);
            else fc(w1, p1, w2, p2, (uint64_t)L.n[in]);
        });
        if (!launch_ok()) { cb200_na_release(out); return nullptr; }
    }
    apply_keepdims(out, a, rp, keepdims);
    return out;
}

// ---- clip, fill, seq, divmod, modf, frexp ----------------------------------------------------------
extern "C++" {
namespace {

Loop loop_of(const cb200_na* a) {
    Loop lp;
    lp.ndim = a->ndim;
    memcpy(lp.shape, a->shape, sizeof(int64_t) * a->ndim);
    return lp;
}

template <typename C>
void call_fill(void* f, cumo_na_iarray_t* a1, cumo_na_indexer_t* ix, double vf, int64_t vi) {
    ((void (*)(cumo_na_iarray_t*, cumo_na_indexer_t*, C))f)(a1, ix, pick<C>(vf, vi));
}

bool fill_with(cb200_na* a, double vf, int64_t vi) {
    void* f = sym(std::string("cumo_iter_") + kTypeName[a->dtype] + "_fill_kernel_launch");
    if (!f) return false;
    Loop lp = loop_of(a);
    cumo_na_indexer_t ix;
    cumo_na_iarray_t a1;
    fill_indexer(&ix, lp);
    fill_iarray(&a1, a, lp);
    switch (a->dtype) {
    case CB200_SFLOAT: call_fill<float>(f, &a1, &ix, vf, vi); break;
    case CB200_DFLOAT: call_fill<double>(f, &a1, &ix, vf, vi); break;
    case CB200_INT32:  call_fill<int32_t>(f, &a1, &ix, vf, vi); break;
    default:           call_fill<int64_t>(f, &a1, &ix, vf, vi); break;
    }
    return launch_ok();
}

// a bound of clip as an array of the clipped array's type: the array itself, a converted copy, or one element
// holding the numeric (the reference casts a numeric against an array bound the same way, ndloop.c's cast of ain {cT,0})
cb200_na* bound_array(cb200_na* arr, int kind, double vf, int64_t vi, int dtype) {
    if (kind == 2) return arr->dtype == dtype ? share(arr) : cast_to(arr, dtype);
    const int64_t one = 1;
    cb200_na* b = make(dtype, 1, &one, false);
    if (b && !fill_with(b, vf, vi)) { cb200_na_release(b); b = nullptr; }
    return b;
}

template <typename C>
void call_clip_s(void* f, cumo_na_iarray_t* a1, double lf, int64_t li, double hf, int64_t hi, cumo_na_iarray_t* a4, cumo_na_indexer_t* ix) {
    ((void (*)(cumo_na_iarray_t*, C, C, cumo_na_iarray_t*, cumo_na_indexer_t*))f)(a1, pick<C>(lf, li), pick<C>(hf, hi), a4, ix);
}
template <typename C>
void call_clip_one_s(void* f, cumo_na_iarray_t* a1, double vf, int64_t vi, cumo_na_iarray_t* a3, cumo_na_indexer_t* ix) {
    ((void (*)(cumo_na_iarray_t*, C, cumo_na_iarray_t*, cumo_na_indexer_t*))f)(a1, pick<C>(vf, vi), a3, ix);
}
template <typename C> bool empty_range(double lf, int64_t li, double hf, int64_t hi) { return pick<C>(lf, li) > pick<C>(hf, hi); }

}  // namespace
}  // extern "C++"

// `a.clip(min, max)` (gen/tmpl/clip.c:218-276).  A bound is absent (kind 0), a host numeric (1) or an array (2).
// Two numerics are compared here and go by value; one numeric with no other bound goes by value too; every other
// combination runs the array forms, a numeric becoming a one-element array that is repeated.
cb200_na_t* cb200_na_clip(cb200_na_t* a, int lo_kind, cb200_na_t* lo, double lo_f, int64_t lo_i,
                          int hi_kind, cb200_na_t* hi, double hi_f, int64_t hi_i) {
    if (!is_value_type(a->dtype)) return (cb200_na*)fail("TypeError", "clip is not defined for %s", kTypeName[a->dtype]);
    if (lo_kind == 0 && hi_kind == 0) return (cb200_na*)fail("ArgumentError", "min and max are not given");
    const int dtype = a->dtype;
    const std::string t = kTypeName[dtype];
    if (lo_kind != 2 && hi_kind != 2) {
        Loop lp = loop_of(a);
        if (lo_kind == 1 && hi_kind == 1) {
            bool empty;
            switch (dtype) {
            case CB200_SFLOAT: empty = empty_range<float>(lo_f, lo_i, hi_f, hi_i); break;
            case CB200_DFLOAT: empty = empty_range<double>(lo_f, lo_i, hi_f, hi_i); break;
            case CB200_INT32:  empty = empty_range<int32_t>(lo_f, lo_i, hi_f, hi_i); break;
            default:           empty = empty_range<int64_t>(lo_f, lo_i, hi_f, hi_i); break;
            }
            if (empty) return (cb200_na*)fail("OperationError", "min is greater than max");
        }
        void* f = sym("cumo_iter_" + t + (lo_kind && hi_kind ? "_clip_s" : lo_kind ? "_clip_min_s" : "_clip_max_s") + "_kernel_launch");
        if (!f) return nullptr;
        cb200_na* out = output_for(a, dtype, lp);
        if (!out) return nullptr;
        cumo_na_indexer_t ix;
        cumo_na_iarray_t a1, a4;
        fill_indexer(&ix, lp);
        fill_iarray(&a1, a, lp);
        fill_iarray(&a4, out, lp);
        const double vf = lo_kind ? lo_f : hi_f;
        const int64_t vi = lo_kind ? lo_i : hi_i;
        if (lo_kind && hi_kind) {
            switch (dtype) {
            case CB200_SFLOAT: call_clip_s<float>(f, &a1, lo_f, lo_i, hi_f, hi_i, &a4, &ix); break;
            case CB200_DFLOAT: call_clip_s<double>(f, &a1, lo_f, lo_i, hi_f, hi_i, &a4, &ix); break;
            case CB200_INT32:  call_clip_s<int32_t>(f, &a1, lo_f, lo_i, hi_f, hi_i, &a4, &ix); break;
            default:           call_clip_s<int64_t>(f, &a1, lo_f, lo_i, hi_f, hi_i, &a4, &ix); break;
            }
        } else {
            switch (dtype) {
            case CB200_SFLOAT: call_clip_one_s<float>(f, &a1, vf, vi, &a4, &ix); break;
            case CB200_DFLOAT: call_clip_one_s<double>(f, &a1, vf, vi, &a4, &ix); break;
            case CB200_INT32:  call_clip_one_s<int32_t>(f, &a1, vf, vi, &a4, &ix); break;
            default:           call_clip_one_s<int64_t>(f, &a1, vf, vi, &a4, &ix); break;
            }
        }
        if (!launch_ok()) { cb200_na_release(out); return nullptr; }
        return out;
    }
    cb200_na* bl = lo_kind ? bound_array(lo, lo_kind, lo_f, lo_i, dtype) : nullptr;
    cb200_na* bh = hi_kind ? bound_array(hi, hi_kind, hi_f, hi_i, dtype) : nullptr;
    cb200_na* out = nullptr;
    bool ok = (!lo_kind || bl) && (!hi_kind || bh);
    Loop lp, l2;
    if (ok) ok = broadcast(a, bl ? bl : bh, &lp);
    if (ok && bl && bh) {
        // the loop shape of three operands: fold the third into the shape of the first two
        cb200_na tmp = *a;
        tmp.ndim = lp.ndim;
        memcpy(tmp.shape, lp.shape, sizeof(int64_t) * lp.ndim);
        ok = broadcast(&tmp, bh, &l2);
        if (ok) lp = l2;
    }
    if (ok) { out = output_for(a, dtype, lp); ok = out != nullptr; }
    if (ok) {
        void* f = sym("cumo_iter_" + t + (bl && bh ? "_clip" : bl ? "_clip_min" : "_clip_max") + "_kernel_launch");
        ok = f != nullptr;
        if (ok) {
            cumo_na_indexer_t ix;
            cumo_na_iarray_t a1, a2, a3, a4;
            fill_indexer(&ix, lp);
            fill_iarray(&a1, a, lp);
            fill_iarray(&a4, out, lp);
            if (bl && bh) {
                fill_iarray(&a2, bl, lp);
                fill_iarray(&a3, bh, lp);
                ok = with_flag("clip", dtype, [&](int* flag) {
                    ((void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*, int*))f)(&a1, &a2, &a3, &a4, &ix, flag);
                });
            } else {
                fill_iarray(&a2, bl ? bl : bh, lp);
                ((void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*))f)(&a1, &a2, &a4, &ix);
                ok = launch_ok();
            }
        }
    }
    cb200_na_release(bl);
    cb200_na_release(bh);
    if (!ok) { cb200_na_release(out); return nullptr; }
    return out;
}

// `a.fill(value)` (gen/tmpl/fill.c:18-27): through any view; 0 on success
int cb200_na_fill(cb200_na_t* a, double value_f, int64_t value_i) {
    if (a->dtype == CB200_BIT) {                 // Bit#fill (gen/tmpl_bit/fill.c:16-49): the low bit of the value
        if (size_of(a) == 0) return 0;
        auto f = (void (*)(cumo_na_bit_iarray_stridx_t*, CUMO_BIT_DIGIT, cumo_na_indexer_t*))sym("cumo_iter_bit_fill_kernel_launch");
        if (!f) return -1;
        cumo_na_indexer_t ix;
        cumo_na_bit_iarray_stridx_t b;
        memset(&ix, 0, sizeof ix);
        memset(&b, 0, sizeof b);
        ix.ndim = (unsigned char)a->ndim;
        ix.total_size = 1;
        b.ptr = reinterpret_cast<CUMO_BIT_DIGIT*>(a->st->ptr);
        b.pos = (size_t)a->offset;
        for (int d = 0; d < a->ndim; ++d) {
            ix.shape[d] = (size_t)a->shape[d];
            ix.total_size *= (size_t)a->shape[d];
            b.stridx[d].stride = (ssize_t)((a->step[d] << 1) | 1);
        }
        f(&b, (CUMO_BIT_DIGIT)((value_f != 0.0 || value_i != 0) ? 1u : 0u), &ix);
        return launch_ok() ? 0 : -1;
    }
    if (!is_value_type(a->dtype)) { fail("TypeError", "fill is not defined for %s", kTypeName[a->dtype]); return -1; }
    return fill_with(a, value_f, value_i) ? 0 : -1;
}

// `a.seq(beg, step)` (gen/tmpl/seq.c:21-117): element i in row-major order takes beg + i*step
int cb200_na_seq(cb200_na_t* a, double beg, double step) {
    if (!is_value_type(a->dtype)) { fail("TypeError", "seq is not defined for %s", kTypeName[a->dtype]); return -1; }
    void* f = sym(std::string("cumo_iter_") + kTypeName[a->dtype] + "_seq_kernel_launch");
    if (!f) return -1;
    Loop lp = loop_of(a);
    cumo_na_indexer_t ix;
    cumo_na_iarray_t a1;
    fill_indexer(&ix, lp);
    fill_iarray(&a1, a, lp);
    if (a->dtype == CB200_SFLOAT) ((void (*)(cumo_na_iarray_t*, cumo_na_indexer_t*, float, float, double))f)(&a1, &ix, (float)beg, (float)step, 0.0);
    else ((void (*)(cumo_na_iarray_t*, cumo_na_indexer_t*, double, double, double))f)(&a1, &ix, beg, step, 0.0);
    return launch_ok() ? 0 : -1;
}

// `a.divmod(b)` (gen/tmpl/binary2.c:58-95): both results of the broadcast pair, in the upcast type
int cb200_na_divmod(cb200_na_t* a, cb200_na_t* b, cb200_na_t** out_quot, cb200_na_t** out_rem) {
    *out_quot = *out_rem = nullptr;
    if (!is_value_type(a->dtype) || !is_value_type(b->dtype)) { fail("TypeError", "divmod is not defined for %s and %s", kTypeName[a->dtype], kTypeName[b->dtype]); return -1; }
    const int dtype = upcast(a->dtype, b->dtype);
    Loop lp;
    if (!broadcast(a, b, &lp)) return -1;
    cb200_na *ca = nullptr, *cb = nullptr;
    if (a->dtype != dtype) { ca = cast_to(a, dtype); if (!ca) return -1; }
    if (b->dtype != dtype) { cb = cast_to(b, dtype); if (!cb) { cb200_na_release(ca); return -1; } }
    cb200_na* q = make(dtype, lp.ndim, lp.shape, false);
    cb200_na* r = make(dtype, lp.ndim, lp.shape, false);
    void* f = sym(std::string("cumo_iter_") + kTypeName[dtype] + "_divmod_kernel_launch");
    bool ok = q && r && f;
    if (ok) {
        cumo_na_indexer_t ix;
        cumo_na_iarray_t a1, a2, a3, a4;
        fill_indexer(&ix, lp);
        fill_iarray(&a1, ca ? ca : a, lp);
        fill_iarray(&a2, cb ? cb : b, lp);
        fill_iarray(&a3, q, lp);
        fill_iarray(&a4, r, lp);
        ok = with_flag("divmod", dtype, [&](int* flag) {
            ((void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*, int*))f)(&a1, &a2, &a3, &a4, &ix, flag);
        });
    }
    cb200_na_release(ca);
    cb200_na_release(cb);
    if (!ok) { cb200_na_release(q); cb200_na_release(r); return -1; }
    *out_quot = q;
    *out_rem = r;
    return 0;
}

// `a.modf` (gen/tmpl/unary_ret2.c:33-44) and `NMath.frexp(a)` (gen/tmpl/frexp.c:36-48): float arrays only;
// the second result of frexp is an Int32 array
static int two_results(cb200_na_t* a, const char* what, const std::string& symbol, int second_dtype, cb200_na_t** out1, cb200_na_t** out2) {
    *out1 = *out2 = nullptr;
    if (!is_float_type(a->dtype)) { fail("NoMethodError", "%s needs a float array", what); return -1; }
    Loop lp = loop_of(a);
    cb200_na* r1 = make(a->dtype, lp.ndim, lp.shape, false);
    cb200_na* r2 = make(second_dtype, lp.ndim, lp.shape, false);
    void* f = sym(symbol);
    bool ok = r1 && r2 && f;
    if (ok) {
        cumo_na_indexer_t ix;
        cumo_na_iarray_t a1, a2, a3;
        fill_indexer(&ix, lp);
        fill_iarray(&a1, a, lp);
        fill_iarray(&a2, r1, lp);
        fill_iarray(&a3, r2, lp);
        ((void (*)(cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_iarray_t*, cumo_na_indexer_t*))f)(&a1, &a2, &a3, &ix);
        ok = launch_ok();
    }
    if (!ok) { cb200_na_release(r1); cb200_na_release(r2); return -1; }
    *out1 = r1;
    *out2 = r2;
    return 0;
}

int cb200_na_modf(cb200_na_t* a, cb200_na_t** out_frac, cb200_na_t** out_whole) {
    return two_results(a, "modf", std::string("cumo_iter_") + kTypeName[a->dtype] + "_modf_kernel_launch", a->dtype, out_frac, out_whole);
}

int cb200_na_frexp(cb200_na_t* a, cb200_na_t** out_mantissa, cb200_na_t** out_exponent) {
    return two_results(a, "frexp", std::string("cumo_iter_") + kTypeName[a->dtype] + "_math_s_frexp_kernel_launch", CB200_INT32, out_mantissa, out_exponent);
}

cb200_na_t* cb200_na_mulsum(cb200_na_t* a, cb200_na_t* b, uint32_t axis_mask, int keepdims, int nan) {
    if (!is_value_type(a->dtype) || !is_value_type(b->dtype)) return (cb200_na*)fail("TypeError", "mulsum needs numeric arrays");
    int dtype = upcast(a->dtype, b->dtype);
    Loop lp;
    if (!broadcast(a, b, &lp)) return nullptr;
    cb200_na *ca = nullptr, *cb = nullptr;
    if (a->dtype != dtype) { ca = cast_to(a, dtype); if (!ca) return nullptr; }
    if (b->dtype != dtype) { cb = cast_to(b, dtype); if (!cb) { cb200_na_release(ca); return nullptr; } }
    const cb200_na* x = ca ? ca : a;
    const cb200_na* y = cb ? cb : b;
    // reduce plan over the broadcast loop shape
    cb200_na shape_only;
    shape_only.ndim = lp.ndim;
    memcpy(shape_only.shape, lp.shape, sizeof(int64_t) * lp.ndim);
    ReducePlan rp;
    cb200_na* out = nullptr;
    bool ok = plan_reduce(&shape_only, axis_mask, &rp);
    if (ok) { out = make(dtype, rp.n_keep, rp.out_shape, true); ok = out != nullptr; }
    if (ok) {
        cumo_na_iarray_t sx, sy;
        fill_iarray(&sx, x, lp);
        fill_iarray(&sy, y, lp);
        StrideLoop L;
        L.nd = lp.ndim;
        int k = 0;
        for (int i = 0; i < rp.n_keep; ++i, ++k) { L.n[k] = lp.shape[rp.keep[i]]; L.s[0][k] = sx.step[rp.keep[i]]; L.s[1][k] = sy.step[rp.keep[i]]; L.s[2][k] = out->step[i]; }
        for (int i = 0; i < rp.n_red; ++i, ++k) { L.n[k] = lp.shape[rp.red[i]]; L.s[0][k] = sx.step[rp.red[i]]; L.s[1][k] = sy.step[rp.red[i]]; L.s[2][k] = 0; }
        if (L.nd == 0) { L.nd = 1; L.n[0] = 1; L.s[0][0] = L.s[1][0] = L.s[2][0] = 0; }
        contract(&L, 3);
        std::string base = std::string("cumo_") + kTypeName[dtype] + "_mulsum" + ((nan && is_float_type(dtype)) ? "_nan" : "");
        using FnR = void (*)(char*, char*, char*, ssize_t, ssize_t, uint64_t);
        using FnE = void (*)(char*, char*, char*, ssize_t, ssize_t, ssize_t, uint64_t);
        FnR fr = (FnR)sym(base + "_reduce_kernel_launch");
        FnE fe = (FnE)sym(base + "_kernel_launch");
        ok = fr && fe;
        int64_t outer_runs = 1;
        for (int d = 0; d + 1 < L.nd; ++d) outer_runs *= L.n[d];
        if (ok && outer_runs >= 64) {
            // many runs: the whole loop in one launch instead of one launch per run
            using FnAxes = void (*)(char*, char*, char*, int, const size_t*, const ssize_t*, const ssize_t*, const ssize_t*, int, const size_t*, const ssize_t*, const ssize_t*);
            FnAxes fa = (FnAxes)sym(std::string("cb200_") + kTypeName[dtype] + "_mulsum" + ((nan && is_float_type(dtype)) ? "_nan" : "") + "_axes_kernel_launch");
            ok = fa != nullptr;
            if (ok) {
                size_t kshape[kMaxD], rshape[kMaxD];
                ssize_t k1[kMaxD], k2[kMaxD], k3[kMaxD], r1[kMaxD], r2[kMaxD];
                for (int i = 0; i < rp.n_keep; ++i) { kshape[i] = (size_t)lp.shape[rp.keep[i]]; k1[i] = sx.step[rp.keep[i]]; k2[i] = sy.step[rp.keep[i]]; k3[i] = (ssize_t)out->step[i]; }
                for (int i = 0; i < rp.n_red; ++i) { rshape[i] = (size_t)lp.shape[rp.red[i]]; r1[i] = sx.step[rp.red[i]]; r2[i] = sy.step[rp.red[i]]; }
                fa(sx.ptr, sy.ptr, data_ptr(out), rp.n_keep, kshape, k1, k2, k3, rp.n_red, rshape, r1, r2);
                ok = launch_ok();
            }
        } else if (ok) {
            const int in = L.nd - 1;
            for_outer(L, 3, [&](const int64_t* off) {
                char* p1 = sx.ptr + off[0];
                char* p2 = sy.ptr + off[1];
                char* p3 = data_ptr(out) + off[2];
                if (L.s[2][in] == 0) fr(p1, p2, p3, (ssize_t)L.s[0][in], (ssize_t)L.s[1][in], (uint64_t)L.n[in]);
                else fe(p1, p2, p3, (ssize_t)L.s[0][in], (ssize_t)L.s[1][in], (ssize_t)L.s[2][in], (uint64_t)L.n[in]);
            });
            ok = launch_ok();
        }
    }
    cb200_na_release(ca);
    cb200_na_release(cb);
    if (!ok) { cb200_na_release(out); return nullptr; }
    apply_keepdims(out, &shape_only, rp, keepdims);
    return out;
}

// ---- index-array gather and Bit#mask --------------------------------------------------------------
// Both end in the same-type store through an index array (cumo_iter_T_store_T_stridx_kernel_launch), which is how the
// reference materialises a view that carries an index array (gen/tmpl/store_from.c:82-89).  The result here is the
// contiguous copy; the reference hands back the view and copies when the view is next used.
static bool stridx_copy(const cb200_na* dst, char* src_ptr, int dtype, int ndim, const int64_t* shape, const int64_t* src_step,
                        int indexed_dim, size_t* index) {
    using Fn = void (*)(cumo_na_iarray_stridx_t*, cumo_na_iarray_stridx_t*, cumo_na_indexer_t*);
    Fn f = (Fn)sym(std::string("cumo_iter_") + kTypeName[dtype] + "_store_" + kTypeName[dtype] + "_stridx_kernel_launch");
    if (!f) return false;
    cumo_na_iarray_stridx_t d, s2;
    cumo_na_indexer_t ix;
    memset(&d, 0, sizeof d); memset(&s2, 0, sizeof s2); memset(&ix, 0, sizeof ix);
    d.ptr = data_ptr(dst);
    s2.ptr = src_ptr;
    ix.ndim = (unsigned char)ndim;
    ix.total_size = 1;
    for (int i = 0; i < ndim; ++i) {
        ix.shape[i] = (size_t)shape[i];
        ix.total_size *= (size_t)shape[i];
        d.stridx[i].stride = (ssize_t)((dst->step[i] << 1) | 1);
        if (i == indexed_dim) s2.stridx[i].index = index;
        else s2.stridx[i].stride = (ssize_t)((src_step[i] << 1) | 1);
    }
    f(&d, &s2, &ix);
    return launch_ok();
}

cb200_na_t* cb200_na_take(cb200_na_t* a, int axis, cb200_na_t* idx) {
    if (!is_value_type(a->dtype)) return (cb200_na*)fail("TypeError", "take needs a numeric array");
    if (idx->dtype != CB200_INT32 && idx->dtype != CB200_INT64) return (cb200_na*)fail("TypeError", "the index array must be Int32 or Int64");
    if (axis < 0) axis += a->ndim;
    if (axis < 0 || axis >= a->ndim || idx->ndim != 1) return (cb200_na*)fail("IndexError", "take: axis %d of a %d-d array, %d-d index", axis, a->ndim, idx->ndim);
    // byte offsets = positions * step of the axis, computed by the library's own kernels
    cb200_na* wide = cast_to(idx, CB200_INT64);
    if (!wide) return nullptr;
    cb200_na* off = cb200_na_binary_scalar("mul", wide, 0.0, a->step[axis], 0);
    cb200_na_release(wide);
    if (!off) return nullptr;
    int64_t shape[kMaxD];
    for (int i = 0; i < a->ndim; ++i) shape[i] = a->shape[i];
    shape[axis] = idx->shape[0];
    cb200_na* out = make(a->dtype, a->ndim, shape, false);
    bool ok = out != nullptr;
    if (ok && size_of(out) > 0) ok = stridx_copy(out, data_ptr(a), a->dtype, a->ndim, shape, a->step, axis, reinterpret_cast<size_t*>(data_ptr(off)));
    cb200_na_release(off);
    if (!ok) { cb200_na_release(out); return nullptr; }
    return out;
}

cb200_na_t* cb200_na_mask(cb200_na_t* bits, cb200_na_t* a) {
    if (bits->dtype != CB200_BIT) return (cb200_na*)fail("TypeError", "mask needs a Bit array");
    if (!is_value_type(a->dtype)) return (cb200_na*)fail("TypeError", "mask needs a numeric array to select from");
    if (bits->ndim != a->ndim) return (cb200_na*)fail("ShapeError", "mask and masked arrays must have the same shape");
    for (int i = 0; i < a->ndim; ++i)
        if (bits->shape[i] != a->shape[i]) return (cb200_na*)fail("ShapeError", "mask and masked arrays must have the same shape");
    int64_t hits = 0;
    if (size_of(bits) > 0) {                       // the count sizes the result: one read-back, as in the reference (mask.c:122)
        cb200_na* c = cb200_na_count(bits, 0, 0, 0);
        if (!c) return nullptr;
        uint64_t v = 0;
        const bool ok = cb200_na_read_host(c, &v, 8) == 0;
        cb200_na_release(c);
        if (!ok) return nullptr;
        hits = (int64_t)v;
    }
    cb200_na* out = make(a->dtype, 1, &hits, false);
    if (!out || hits == 0) return out;
    cb200_na* pos = make(CB200_INT64, 1, &hits, false);           // byte positions of the kept elements (size_t)
    if (!pos) { cb200_na_release(out); return nullptr; }
    using FnNew = char* (*)();
    using FnRun = void (*)(CUMO_BIT_DIGIT*, size_t, ssize_t, size_t*, uint64_t, size_t*, size_t, ssize_t, size_t*, char*);
    FnNew fnew = (FnNew)sym("cumo_bit_where_scratch_new");
    FnRun frun = (FnRun)sym("cumo_bit_mask_kernel_launch");
    char* scratch = fnew && frun ? fnew() : nullptr;
    if (!scratch) { cb200_na_release(out); cb200_na_release(pos); if (fnew && frun) fail("CudaError", "no memory for the mask scratch"); return nullptr; }
    StrideLoop L;
    L.nd = a->ndim;
    for (int i = 0; i < a->ndim; ++i) { L.n[i] = a->shape[i]; L.s[0][i] = bits->step[i]; L.s[1][i] = a->step[i]; }
    if (L.nd == 0) { L.nd = 1; L.n[0] = 1; L.s[0][0] = L.s[1][0] = 0; }
    contract(&L, 2);
    const int in = L.nd - 1;
    CUMO_BIT_DIGIT* words = reinterpret_cast<CUMO_BIT_DIGIT*>(bits->st->ptr);
    for_outer(L, 2, [&](const int64_t* off) {
        frun(words, (size_t)(bits->offset + off[0]), (ssize_t)L.s[0][in], nullptr, (uint64_t)L.n[in], reinterpret_cast<size_t*>(data_ptr(pos)),
             (size_t)(a->offset + off[1]), (ssize_t)L.s[1][in], nullptr, scratch);
    });
    cumo_cuda_runtime_free(scratch);
    bool ok = launch_ok();
    const int64_t no_step = 0;
    if (ok) ok = stridx_copy(out, a->st->ptr, a->dtype, 1, &hits, &no_step, 0, reinterpret_cast<size_t*>(data_ptr(pos)));
    cb200_na_release(pos);
    if (!ok) { cb200_na_release(out); return nullptr; }
    return out;
}

}  // extern "C"
