// General matrix product on the CUDA cores, with the argument list of cublas<T>gemmStridedBatched minus the handle.
//
// The reference computes `dot` on float matrices with that cuBLAS call from its HOST template
// (ext/cumo/narray/gen/tmpl/gemm.c:252-297: column-major bookkeeping, transpose flags from the operands' layouts,
// alpha/beta, a batch count); it has no kernel-launch function for it.  cb200_sgemm_strided_batched /
// cb200_dgemm_strided_batched take exactly those arguments, so the one place to bind them is that call.
//   * single precision, one product per batch entry with alpha = 1, beta = 0 and K, lda, ldb multiples of 4:
//     the tcgen05 kernel (cb200_sgemm_nt_tc: split-TF32, fp32-grade results); it wants both operands contiguous
//     along K, so the operand that is not gets a transposed copy through the shared-memory tile kernel first;
//   * everything else (double precision -- there is no fp64 tensor-core path here --, alpha/beta, odd sizes):
//     gemm_cc_kernel below, a 128 x 128 x 16 shared-memory tile with an 8 x 8 register tile per thread, FMA in the
//     element type.  Double precision is bound by the FP64 FMA rate.
// Column-major throughout, like cuBLAS: C (m x n, leading dimension ldc) = alpha * op(A) * op(B) + beta * C.
#include "elementwise.cuh"

#include <cstdio>

extern "C" int cb200_sgemm_nt_tc(int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* Bt, int64_t ldb,
                                 float* C, int64_t ldc, char* errbuf, size_t errlen);

namespace cb200 {

constexpr int kGcM = 128, kGcN = 128, kGcK = 16, kGcPad = 4;

template <typename T>
struct GemmCc {
    int m, n, k;
    T alpha, beta;
    const T* A; int64_t a_i, a_k, a_batch;      // element (i, kk) of op(A) at A[i * a_i + kk * a_k]
    const T* B; int64_t b_k, b_j, b_batch;      // element (kk, j) of op(B) at B[kk * b_k + j * b_j]
    T* C; int64_t ldc, c_batch;
    int tiles_m, tiles_n;
};

template <typename T>
__global__ void __launch_bounds__(kBlock)
gemm_cc_kernel(const GemmCc<T> g) {
    __shared__ T As[kGcK][kGcM + kGcPad];
    __shared__ T Bs[kGcK][kGcN + kGcPad];
    const int tile = blockIdx.x;
    const int tm = tile % g.tiles_m, tn = tile / g.tiles_m;
    const int batch = blockIdx.y;
    const T* A = g.A + (int64_t)batch * g.a_batch;
    const T* B = g.B + (int64_t)batch * g.b_batch;
    T* C = g.C + (int64_t)batch * g.c_batch;
    const int i0 = tm * kGcM, j0 = tn * kGcN;
    // 16 x 16 threads, 8 x 8 outputs each: rows ti, ti + 16, ... (neighbouring lanes read neighbouring elements of the A
    // tile: no bank conflicts, and their stores to a column of C are consecutive), columns tj * 8 .. tj * 8 + 7 (a warp
    // holds two values of tj: its reads of the B tile are broadcasts)
    const int ti = threadIdx.x % 16, tj = threadIdx.x / 16;
    T acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = T(0);
    // lanes run along whichever axis of each operand is contiguous in memory
    const bool a_along_i = g.a_i == 1 || g.a_k != 1;
    const bool b_along_j = g.b_j == 1 || g.b_k != 1;
    constexpr int PER = kGcM * kGcK / kBlock;                         // 8 elements per thread and operand
    T ra[PER], rb[PER];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int f = e * kBlock + threadIdx.x;
            const int ii = a_along_i ? f % kGcM : f / kGcK, ka = a_along_i ? f / kGcM : f % kGcK;
            ra[e] = (i0 + ii < g.m && k0 + ka < g.k) ? A[(int64_t)(i0 + ii) * g.a_i + (int64_t)(k0 + ka) * g.a_k] : T(0);
            const int jj = b_along_j ? f % kGcN : f / kGcK, kb = b_along_j ? f / kGcN : f % kGcK;
            rb[e] = (j0 + jj < g.n && k0 + kb < g.k) ? B[(int64_t)(k0 + kb) * g.b_k + (int64_t)(j0 + jj) * g.b_j] : T(0);
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < g.k; k0 += kGcK) {
        __syncthreads();                                             // the previous block's tiles are no longer read
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int f = e * kBlock + threadIdx.x;
            const int ii = a_along_i ? f % kGcM : f / kGcK, ka = a_along_i ? f / kGcM : f % kGcK;
            As[ka][ii] = ra[e];
            const int jj = b_along_j ? f % kGcN : f / kGcK, kb = b_along_j ? f / kGcN : f % kGcK;
            Bs[kb][jj] = rb[e];
        }
        __syncthreads();
        if (k0 + kGcK < g.k) fetch(k0 + kGcK);                       // the next block's loads fly while this one is multiplied
#pragma unroll
        for (int kk = 0; kk < kGcK; ++kk) {
            T a[8], b[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) { a[x] = As[kk][ti + 16 * x]; b[x] = Bs[kk][tj * 8 + x]; }
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int y = 0; y < 8; ++y) acc[x][y] = a[x] * b[y] + acc[x][y];
        }
    }
#pragma unroll
    for (int y = 0; y < 8; ++y) {
        const int j = j0 + tj * 8 + y;
        if (j >= g.n) continue;
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            const int i = i0 + ti + 16 * x;
            if (i >= g.m) continue;
            T* c = C + (int64_t)j * g.ldc + i;
            // beta == 0 must not read C (it may hold NaN or be uninitialised), as in BLAS
            *c = g.beta == T(0) ? g.alpha * acc[x][y] : g.alpha * acc[x][y] + g.beta * *c;
        }
    }
}

template <typename T>
static int gemm_cc(int transa, int transb, int m, int n, int k, T alpha, const T* A, int lda, long long strideA, const T* B, int ldb,
                   long long strideB, T beta, T* C, int ldc, long long strideC, int batch) {
    GemmCc<T> g;
    g.m = m; g.n = n; g.k = k; g.alpha = alpha; g.beta = beta;
    g.A = A; g.a_i = transa ? lda : 1; g.a_k = transa ? 1 : lda; g.a_batch = strideA;
    g.B = B; g.b_k = transb ? ldb : 1; g.b_j = transb ? 1 : ldb; g.b_batch = strideB;
    g.C = C; g.ldc = ldc; g.c_batch = strideC;
    g.tiles_m = (m + kGcM - 1) / kGcM;
    g.tiles_n = (n + kGcN - 1) / kGcN;
    dim3 grid((unsigned)(g.tiles_m * g.tiles_n), (unsigned)batch);
    gemm_cc_kernel<T><<<grid, kBlock, 0, current_stream()>>>(g);
    count_launch();
    cumo_cuda_runtime_check_kernel_launch();
    return 0;
}

static bool bad_shape(int transa, int transb, int m, int n, int k, int lda, int ldb, int ldc, int batch) {
    if (m < 0 || n < 0 || k < 0 || batch < 0) return true;
    if (transa < 0 || transa > 2 || transb < 0 || transb > 2) return true;
    if (lda < (transa ? k : m) || ldb < (transb ? n : k) || ldc < m) return true;
    return lda < 1 || ldb < 1 || ldc < 1;
}

}  // namespace cb200

using namespace cb200;

// Return values follow cublasStatus_t: 0 success, 7 (CUBLAS_STATUS_INVALID_VALUE) for a bad argument, 13
// (CUBLAS_STATUS_EXECUTION_FAILED) when the tensor-core path reported a failure.  transa/transb: 0 = N, 1 = T, 2 = C
// (same as T for real types).  alpha and beta are host pointers.
extern "C" int cb200_dgemm_strided_batched(int transa, int transb, int m, int n, int k, const double* alpha, const double* A, int lda,
                                           long long strideA, const double* B, int ldb, long long strideB, const double* beta, double* C,
                                           int ldc, long long strideC, int batch) {
    if (!alpha || !beta || bad_shape(transa, transb, m, n, k, lda, ldb, ldc, batch)) return 7;
    if (m == 0 || n == 0 || batch == 0) return 0;
    return gemm_cc<double>(transa != 0, transb != 0, m, n, k, *alpha, A, lda, strideA, B, ldb, strideB, *beta, C, ldc, strideC, batch);
}

extern "C" int cb200_sgemm_strided_batched(int transa, int transb, int m, int n, int k, const float* alpha, const float* A, int lda,
                                           long long strideA, const float* B, int ldb, long long strideB, const float* beta, float* C,
                                           int ldc, long long strideC, int batch) {
    if (!alpha || !beta || bad_shape(transa, transb, m, n, k, lda, ldb, ldc, batch)) return 7;
    if (m == 0 || n == 0 || batch == 0) return 0;
    const bool ta = transa != 0, tb = transb != 0;
    // Tensor-core path.  In row-major words (what cb200_sgemm_nt_tc speaks) the column-major C (m x n) is the n x m matrix
    // C' with leading dimension ldc, and C' = B' . A' with A' = op(A)^T, B' = op(B)^T.  The kernel wants both of its
    // operands contiguous along k: its first operand rows = columns j of op(B), i.e. op(B) column-major with b_k == 1
    // (transb == N), its second operand rows = rows i of op(A) with a_k == 1 (transa == T).
    const bool big = (long long)m * n * k >= (1ll << 24) && k % 4 == 0;
    if (big && *alpha == 1.0f && *beta == 0.0f && k >= 32) {
        char err[160];
        int rc = 0;
        for (int b = 0; b < batch && rc == 0; ++b) {
            const float* Ab = A + (long long)b * strideA;
            const float* Bb = B + (long long)b * strideB;
            float* Cb = C + (long long)b * strideC;
            const float* first = Bb;   int64_t ld_first = ldb;     // n rows of k
            const float* second = Ab;  int64_t ld_second = lda;    // m rows of k
            char* tmp1 = nullptr;
            char* tmp2 = nullptr;
            auto transposed_copy = [&](const float* src, int rows, int cols, int ld) -> char* {
                // src: column-major (rows x cols, leading dimension ld) -> a contiguous copy of its transpose, i.e. the
                // same matrix stored with `rows` contiguous per ... cols: out[r][c] (row-major rows x cols) = src[c * ld + r]
                char* out = cumo_cuda_runtime_malloc((size_t)rows * cols * sizeof(float));
                if (!out) return nullptr;
                cumo_na_iarray_t s, d;
                cumo_na_indexer_t ix;
                memset(&s, 0, sizeof s); memset(&d, 0, sizeof d); memset(&ix, 0, sizeof ix);
                ix.ndim = 2; ix.shape[0] = (size_t)rows; ix.shape[1] = (size_t)cols; ix.total_size = (size_t)rows * cols;
                s.ptr = (char*)src; s.step[0] = 4; s.step[1] = (ssize_t)ld * 4;
                d.ptr = out; d.step[0] = (ssize_t)cols * 4; d.step[1] = 4;
                launch_elementwise<op::Cast<float, float>>(&s, nullptr, &d, &ix, 0.0f, 0.0f, 0, nullptr);
                return out;
            };
            if (tb) {            // op(B) = B^T: B is n x k column-major, a row j of k is strided -> copy to n rows of k
                tmp1 = transposed_copy(Bb, n, k, ldb);
                if (!tmp1) { rc = 13; break; }
                first = reinterpret_cast<const float*>(tmp1); ld_first = k;
            }
            if (!ta) {           // op(A) = A: m x k column-major, a row i of k is strided -> copy to m rows of k
                tmp2 = transposed_copy(Ab, m, k, lda);
                if (!tmp2) { cumo_cuda_runtime_free(tmp1); rc = 13; break; }
                second = reinterpret_cast<const float*>(tmp2); ld_second = k;
            }
            const bool ok = ld_first % 4 == 0 && ld_second % 4 == 0 && aligned16(first) && aligned16(second);
            int e = ok ? cb200_sgemm_nt_tc(n, m, k, first, ld_first, second, ld_second, Cb, ldc, err, sizeof err) : 1;
            cumo_cuda_runtime_free(tmp1);
            cumo_cuda_runtime_free(tmp2);
            if (e == 1) {        // a shape the tensor-core kernel does not take after all: the CUDA-core kernel for this entry
                gemm_cc<float>(ta, tb, m, n, k, 1.0f, Ab, lda, 0, Bb, ldb, 0, 0.0f, Cb, ldc, 0, 1);
            } else if (e != 0) {
                rc = 13;
            }
        }
        return rc;
    }
    return gemm_cc<float>(ta, tb, m, n, k, *alpha, A, lda, strideA, B, ldb, strideB, *beta, C, ldc, strideC, batch);
}
