// count_true / count_false along some axes of a Bit array, every output in ONE launch.
//
// The reference reaches a per-axis count through ndloop, which calls its iterator once per innermost run
// (narray/gen/tmpl_bit/bit_count.c:9-36): `mask.count_true(axis: 1)` of a (65536, 2048) mask is 65536 launches of a
// kernel that looks at 2048 bits.  This entry point takes the whole loop instead -- the kept dimensions with the bit
// step of the input and the byte step of the UInt64 output, the counted dimensions with their bit steps -- and adds
// to every output the number of ones (or zeros) among its bits.  Not in the reference; its caller would be the
// function that today hands the loop to ndloop (bit_count.c:52-72).
//
// Plan:
//   * ROWS: the innermost counted dimension is a run of consecutive bits (bit step 1) of at least two words.  A warp
//     per output: lanes take the words of each run in turn, the end words under masks, __popc, one shuffle fold.
//   * COLUMNS: anything else (typically the counted axis is an outer one: `count_true(axis: 0)`).  A thread per
//     output walking the counted elements one bit at a time; consecutive threads are consecutive outputs, so when the
//     innermost kept dimension is contiguous a warp reads one word per step and every lane picks its own bit.
//     With too few outputs to fill the GPU the counted range is cut into slices that add to the output atomically
//     (integer adds commute: exact in any order).
// Otherwise each output has exactly one writer and the sum is a plain add into the caller's zero-filled array.
#include "common.cuh"

namespace cb200 {
namespace {

struct CountAxes {
    int n_keep, n_red;
    int64_t outputs;                      // product of the kept extents
    int64_t reduced;                      // product of the counted extents
    int64_t kshape[kMaxDim], kbit[kMaxDim], kout[kMaxDim];
    int64_t rshape[kMaxDim], rbit[kMaxDim];
};

__device__ __forceinline__ void output_of(const CountAxes& c, int64_t o, int64_t* bit, int64_t* out) {
    int64_t b = 0, q = 0, r = o;
    for (int d = c.n_keep - 1; d >= 0; --d) {
        const int64_t n = c.kshape[d];
        const int64_t k = d > 0 ? r % n : r;
        r = d > 0 ? r / n : 0;
        b += k * c.kbit[d];
        q += k * c.kout[d];
    }
    *bit = b;
    *out = q;
}

// ones among bits [first, first + n) of `words`, the lanes of one warp sharing the words
__device__ __forceinline__ unsigned long long run_ones(const uint32_t* __restrict__ words, uint64_t first, uint64_t n, int lane) {
    const uint64_t w0 = first >> 5, w1 = (first + n - 1) >> 5;
    const uint32_t head = 0xffffffffu << (first & 31);
    const uint32_t last_bits = (uint32_t)((first + n) & 31);
    const uint32_t tail = last_bits ? (0xffffffffu >> (32 - last_bits)) : 0xffffffffu;
    unsigned long long acc = 0;
    for (uint64_t w = w0 + lane; w <= w1; w += 32) {
        uint32_t x = words[w];
        if (w == w0) x &= head;
        if (w == w1) x &= tail;
        acc += __popc(x);
    }
    return acc;
}

__global__ void __launch_bounds__(kBlock)
bit_count_rows_kernel(const CountAxes c, const uint32_t* __restrict__ words, uint64_t pos, int want_false, char* out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * kBlock + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * kBlock) >> 5;
    const int last = c.n_red - 1;
    const int64_t run = c.rshape[last];
    const int64_t runs = c.reduced / run;
    for (int64_t o = warp; o < c.outputs; o += n_warps) {
        int64_t bit, q;
        output_of(c, o, &bit, &q);
        unsigned long long acc = 0;
        for (int64_t j = 0; j < runs; ++j) {
            int64_t b = bit, r = j;
            for (int d = last - 1; d >= 0; --d) {
                const int64_t n = c.rshape[d];
                const int64_t k = d > 0 ? r % n : r;
                r = d > 0 ? r / n : 0;
                b += k * c.rbit[d];
            }
            acc += run_ones(words, pos + (uint64_t)b, (uint64_t)run, lane);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
        if (lane == 0) {
            unsigned long long* dst = reinterpret_cast<unsigned long long*>(out + q);
            *dst += want_false ? (unsigned long long)c.reduced - acc : acc;
        }
    }
}

// gridDim.y slices of the counted range share an output when there are too few outputs to fill the GPU; their integer
// atomic adds commute, so the count is exact in any order.
__global__ void __launch_bounds__(kBlock)
bit_count_columns_kernel(const CountAxes c, const uint32_t* __restrict__ words, uint64_t pos, int want_false, char* out) {
    const int64_t per = (c.reduced + gridDim.y - 1) / gridDim.y;
    const int64_t j0 = (int64_t)blockIdx.y * per;
    const int64_t j1 = j0 + per < c.reduced ? j0 + per : c.reduced;
    if (j0 >= j1) return;
    for (int64_t o = (int64_t)blockIdx.x * kBlock + threadIdx.x; o < c.outputs; o += (int64_t)gridDim.x * kBlock) {
        int64_t bit, q;
        output_of(c, o, &bit, &q);
        unsigned long long acc = 0;
        if (c.n_red == 1) {
            const int64_t step = c.rbit[0];
            uint64_t b = pos + (uint64_t)(bit + j0 * step);
            for (int64_t j = j0; j < j1; ++j, b += (uint64_t)step) acc += (words[b >> 5] >> (b & 31)) & 1u;
        } else {
            for (int64_t j = j0; j < j1; ++j) {
                int64_t b = bit, r = j;
                for (int d = c.n_red - 1; d >= 0; --d) {
                    const int64_t n = c.rshape[d];
                    const int64_t k = d > 0 ? r % n : r;
                    r = d > 0 ? r / n : 0;
                    b += k * c.rbit[d];
                }
                const uint64_t a = pos + (uint64_t)b;
                acc += (words[a >> 5] >> (a & 31)) & 1u;
            }
        }
        unsigned long long* dst = reinterpret_cast<unsigned long long*>(out + q);
        const unsigned long long add = want_false ? (unsigned long long)(j1 - j0) - acc : acc;
        if (gridDim.y == 1) *dst += add;
        else if (add) atomicAdd(dst, add);
    }
}

}  // namespace
}  // namespace cb200

using namespace cb200;

extern "C" void cb200_bit_count_axes_kernel_launch(CUMO_BIT_DIGIT* a1, size_t p1, int want_false,
                                                   int n_keep, const size_t* keep_shape, const ssize_t* keep_bit_step, const ssize_t* keep_out_step,
                                                   int n_red, const size_t* red_shape, const ssize_t* red_bit_step, char* out) {
    CB200_TRACE_LAUNCH();
    if (n_keep < 0 || n_red < 0 || n_keep > kMaxDim || n_red > kMaxDim) return;
    CountAxes c;
    c.n_keep = n_keep;
    c.n_red = n_red;
    c.outputs = 1;
    c.reduced = 1;
    for (int d = 0; d < kMaxDim; ++d) { c.kshape[d] = c.rshape[d] = 1; c.kbit[d] = c.kout[d] = c.rbit[d] = 0; }
    for (int d = 0; d < n_keep; ++d) {
        c.kshape[d] = (int64_t)keep_shape[d]; c.kbit[d] = (int64_t)keep_bit_step[d]; c.kout[d] = (int64_t)keep_out_step[d];
        c.outputs *= c.kshape[d];
    }
    for (int d = 0; d < n_red; ++d) { c.rshape[d] = (int64_t)red_shape[d]; c.rbit[d] = (int64_t)red_bit_step[d]; c.reduced *= c.rshape[d]; }
    if (c.outputs <= 0) return;
    if (n_red == 0) { c.n_red = 1; }                       // nothing counted away: every output looks at its own bit
    cudaStream_t st = current_stream();
    const bool rows = c.reduced > 0 && c.rbit[c.n_red - 1] == 1 && c.rshape[c.n_red - 1] >= 64;
    if (c.reduced == 0) {
        // empty counted extent: the counts are zero, the outputs stay as they are
    } else if (rows) {
        const int64_t ctas = (c.outputs + kBlock / 32 - 1) / (kBlock / 32);
        bit_count_rows_kernel<<<grid_for(ctas, 16), kBlock, 0, st>>>(c, a1, (uint64_t)p1, want_false, out);
        count_launch();
    } else {
        const unsigned gx = grid_for((c.outputs + kBlock - 1) / kBlock, 16);
        int64_t slices = ((int64_t)sm_count() * 8 + gx - 1) / gx;              // enough CTAs to fill the GPU ...
        if (slices > c.reduced / 64) slices = c.reduced / 64;                  // ... of at least 64 counted elements each
        if (slices < 1) slices = 1;
        if (slices > 65535) slices = 65535;
        bit_count_columns_kernel<<<dim3(gx, (unsigned)slices), kBlock, 0, st>>>(c, a1, (uint64_t)p1, want_false, out);
        count_launch();
    }
    cumo_cuda_runtime_check_kernel_launch();
}
