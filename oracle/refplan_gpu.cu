// BENCH INFRASTRUCTURE, not product code: the reference's EXECUTION PLAN for a handful of hot-path
// kernels, restated in new code so that bench.py can time "how the reference lays this work out"
// on the same GPU as the library.  The reference itself cannot be built here (its kernels are
// generated from ERB templates by Ruby).  Nothing in cumo_b200/ links or loads this file.
//
// What is restated (reference file:line of the plan, not of any code reused):
//   elementwise   one element per thread, 128-thread blocks, grid = n/128 + 1, grid-stride loop
//                 (include/cumo/template_kernel.h:58-81); 1-D arrays address by raw_index*step
//                 (include/cumo/indexer.h:259-263), 2-D arrays split the flat index with 64-bit
//                 div/mod per element (indexer.h:239-248)
//   reductions    512-thread blocks; the reduce axis gets all 512 threads when it is the contiguous
//                 one, 16 reduce lanes x 32 outputs per block when the OUT axis is contiguous
//                 (include/cumo/reduce_kernel.h:143-150); scalar loads, shared-memory tree
//                 (:194-245); when fewer than 256 blocks would run the reduce extent is split into
//                 chunks, up to 1024, and a second launch combines them (:386-393, :413-438);
//                 index reductions are never split (:400-404)
//   compare->Bit  one thread per element, one atomicOr / atomicAnd per element
//                 (include/cumo/template_kernel.h:26-35)
//   count_true    one thread per bit, one atomicAdd per set bit (narray/gen/tmpl_bit/bit_count_kernel.cu)
// The restatement is favourable to the reference where the two differ: its 2-D indexer is forced
// into local memory (reduce_kernel.h:41-48 measures that), this one keeps the split in registers.
#include <cstdint>
#include <cuda_runtime.h>

namespace {

constexpr int kBlock = 128;
constexpr int kRedBlock = 512;

inline unsigned grid_for(size_t n) {
    size_t g = n / kBlock + 1;
    const size_t cap = 4294967295ul / kBlock;
    return (unsigned)(g > cap ? cap : g);
}

template <int OP> __device__ __forceinline__ float apply(float x, float y) {
    return OP == 0 ? x + y : OP == 1 ? x * y : OP == 2 ? expf(x) : 0.f;
}

template <int OP>
__global__ void ew1(const char* a, const char* b, char* o, size_t n, int64_t sa, int64_t sb, int64_t so) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)blockDim.x * gridDim.x) {
        const float x = *(const float*)(a + i * sa);
        const float y = b ? *(const float*)(b + i * sb) : 0.f;
        *(float*)(o + i * so) = apply<OP>(x, y);
    }
}

template <int OP>
__global__ void ew2(const char* a, const char* b, char* o, size_t n, uint64_t n1, int64_t sa0, int64_t sa1,
                    int64_t sb0, int64_t sb1, int64_t so0, int64_t so1) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)blockDim.x * gridDim.x) {
        const uint64_t i1 = i % n1, i0 = i / n1;              // the per-element 64-bit split
        const float x = *(const float*)(a + i0 * sa0 + i1 * sa1);
        const float y = *(const float*)(b + i0 * sb0 + i1 * sb1);
        *(float*)(o + i0 * so0 + i1 * so1) = apply<OP>(x, y);
    }
}

__global__ void ew1_scalar_mul(const float* a, float s, float* o, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)blockDim.x * gridDim.x) o[i] = a[i] * s;
}
__global__ void ew1_scalar_mul_i32(const int* a, int s, int* o, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)blockDim.x * gridDim.x) o[i] = a[i] * s;
}

// reduce axis contiguous: all 512 threads of a block stride along it; grid = (outputs, chunks)
template <bool ARG>
__global__ void red_rows(const float* in, int64_t n_red, int64_t chunk, float* out_v, int64_t* out_i, int n_split) {
    __shared__ float sv[kRedBlock];
    __shared__ int64_t si[kRedBlock];
    const int64_t o = blockIdx.x, s = blockIdx.y;
    const int64_t begin = s * chunk, end = begin + chunk < n_red ? begin + chunk : n_red;
    const float* row = in + o * n_red;
    float v = ARG ? -INFINITY : 0.f;
    int64_t idx = INT64_MAX;
    for (int64_t i = begin + threadIdx.x; i < end; i += kRedBlock) {
        const float x = row[i];
        if (ARG) { if (x > v || (x == v && i < idx)) { v = x; idx = i; } } else v += x;
    }
    sv[threadIdx.x] = v; si[threadIdx.x] = idx;
    __syncthreads();
    for (int d = kRedBlock / 2; d > 0; d >>= 1) {
        if (threadIdx.x < d) {
            if (ARG) {
                const float y = sv[threadIdx.x + d]; const int64_t j = si[threadIdx.x + d];
                if (y > sv[threadIdx.x] || (y == sv[threadIdx.x] && j < si[threadIdx.x])) { sv[threadIdx.x] = y; si[threadIdx.x] = j; }
            } else sv[threadIdx.x] += sv[threadIdx.x + d];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (ARG) out_i[o * n_split + s] = si[0] + (n_split == 1 ? o * n_red : 0);
        else out_v[o * n_split + s] = sv[0];
    }
}

// out axis contiguous: 32 outputs x 16 reduce lanes per block; grid = (column blocks, chunks)
__global__ void red_cols(const float* in, int64_t rows, int64_t cols, int64_t chunk, float* out, int n_split) {
    __shared__ float sv[16][33];
    const int c = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int64_t col = (int64_t)blockIdx.x * 32 + c, s = blockIdx.y;
    const int64_t begin = s * chunk, end = begin + chunk < rows ? begin + chunk : rows;
    float v = 0.f;
    if (col < cols)
        for (int64_t i = begin + r; i < end; i += 16) v += in[i * cols + col];
    sv[r][c] = v;
    __syncthreads();
    if (r == 0 && col < cols) {
        for (int k = 1; k < 16; ++k) v += sv[k][c];
        out[col * n_split + s] = v;
    }
}

__global__ void combine(const float* partial, int64_t n_out, int n_split, float* out) {
    __shared__ float sv[kRedBlock];
    const int64_t o = blockIdx.x;
    float v = 0.f;
    for (int i = threadIdx.x; i < n_split; i += kRedBlock) v += partial[o * n_split + i];
    sv[threadIdx.x] = v;
    __syncthreads();
    for (int d = kRedBlock / 2; d > 0; d >>= 1) { if (threadIdx.x < d) sv[threadIdx.x] += sv[threadIdx.x + d]; __syncthreads(); }
    if (threadIdx.x == 0) out[o] = sv[0];
}

__global__ void gt_bits(const int* a, int s, uint32_t* bits, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)blockDim.x * gridDim.x) {
        if (a[i] > s) atomicOr(bits + (i >> 5), 1u << (i & 31));
        else atomicAnd(bits + (i >> 5), ~(1u << (i & 31)));
    }
}

__global__ void count_bits(const uint32_t* bits, size_t n, unsigned long long* out) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)blockDim.x * gridDim.x)
        if ((bits[i >> 5] >> (i & 31)) & 1u) atomicAdd(out, 1ull);
}

int split_count(int64_t reduce_total, int64_t out_blocks) {      // reduce_kernel.h:386-393 (min chunk: one block's worth)
    if (out_blocks >= 256) return 1;
    if (reduce_total < 2 * kRedBlock) return 1;
    int64_t want = (256 + out_blocks - 1) / out_blocks, fits = reduce_total / kRedBlock;
    int64_t n = want < fits ? want : fits;
    if (n > 1024) n = 1024;
    return n < 2 ? 1 : (int)n;
}

}  // namespace

// op: 0 add, 1 mul, 2 exp (b ignored).  Steps in bytes; n0 == 1 takes the 1-D form.
extern "C" void refplan_ew_f32(int op, const void* a, const void* b, void* o, uint64_t n0, uint64_t n1, int64_t sa0, int64_t sa1,
                               int64_t sb0, int64_t sb1, int64_t so0, int64_t so1) {
    const size_t n = (size_t)n0 * n1;
    const unsigned g = grid_for(n);
    const char *pa = (const char*)a, *pb = (const char*)b;
    char* po = (char*)o;
    if (n0 == 1) {
        if (op == 0) ew1<0><<<g, kBlock>>>(pa, pb, po, n, sa1, sb1, so1);
        else if (op == 1) ew1<1><<<g, kBlock>>>(pa, pb, po, n, sa1, sb1, so1);
        else ew1<2><<<g, kBlock>>>(pa, nullptr, po, n, sa1, 0, so1);
    } else {
        if (op == 0) ew2<0><<<g, kBlock>>>(pa, pb, po, n, n1, sa0, sa1, sb0, sb1, so0, so1);
        else ew2<1><<<g, kBlock>>>(pa, pb, po, n, n1, sa0, sa1, sb0, sb1, so0, so1);
    }
}
extern "C" void refplan_mul_scalar_f32(const float* a, float s, float* o, uint64_t n) { ew1_scalar_mul<<<grid_for(n), kBlock>>>(a, s, o, n); }
extern "C" void refplan_mul_scalar_i32(const int* a, int s, int* o, uint64_t n) { ew1_scalar_mul_i32<<<grid_for(n), kBlock>>>(a, s, o, n); }

// sum over the contiguous axis of (n_out, n_red); scratch must hold n_out * 1024 floats
extern "C" void refplan_sum_rows_f32(const float* in, int64_t n_out, int64_t n_red, float* out, float* scratch) {
    const int ns = split_count(n_red, n_out);
    const int64_t chunk = (n_red + ns - 1) / ns;
    red_rows<false><<<dim3((unsigned)n_out, ns), kRedBlock>>>(in, n_red, chunk, ns == 1 ? out : scratch, nullptr, ns);
    if (ns > 1) combine<<<(unsigned)n_out, kRedBlock>>>(scratch, n_out, ns, out);
}
// max_index over the contiguous axis of (n_out, n_red), flat element offsets, never split
extern "C" void refplan_max_index_rows_f32(const float* in, int64_t n_out, int64_t n_red, int64_t* out) {
    red_rows<true><<<dim3((unsigned)n_out, 1), kRedBlock>>>(in, n_red, n_red, nullptr, out, 1);
}
// sum over axis 0 of a row-major (rows, cols); scratch must hold cols * 1024 floats
extern "C" void refplan_sum_cols_f32(const float* in, int64_t rows, int64_t cols, float* out, float* scratch) {
    const int64_t blocks = (cols + 31) / 32;
    const int ns = split_count(rows, blocks);
    const int64_t chunk = (rows + ns - 1) / ns;
    red_cols<<<dim3((unsigned)blocks, ns), kRedBlock>>>(in, rows, cols, chunk, ns == 1 ? out : scratch, ns);
    if (ns > 1) combine<<<(unsigned)cols, kRedBlock>>>(scratch, cols, ns, out);
}
extern "C" void refplan_gt_scalar_i32(const int* a, int s, uint32_t* bits, uint64_t n) { gt_bits<<<grid_for(n), kBlock>>>(a, s, bits, n); }
extern "C" void refplan_count_true(const uint32_t* bits, uint64_t n, unsigned long long* out) {
    cudaMemsetAsync(out, 0, sizeof(unsigned long long));
    count_bits<<<grid_for(n), kBlock>>>(bits, n, out);
}
