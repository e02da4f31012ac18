// Bit#where / where2 / mask: the positions of the one (or, inverted, zero) bits of a run, ascending.
//
// Entry points and protocol are the reference's (narray/gen/tmpl_bit/where.c:11-12 declares
// them, where_kernel.cu:83-110 defines them): the host allocates `scratch` once per call with
// cumo_bit_where_scratch_new(), then launches once per run of the array; a cursor inside the
// scratch (one for ones, one for zeros) carries the output position from one launch to the next
// on the device, so nothing is read back.  Position i of a run is reported as `count + i`.
//
// Plan: a "chunk" is 32 consecutive elements of the run gathered into one word (two loads and a
// funnel shift when the run is contiguous, 32 single-bit loads otherwise).  A tile is 256 threads
// x 4 consecutive chunks.  (1) every CTA counts the hits of its tiles, (2) one CTA turns the
// counts into output positions and advances the cursor, (3) every CTA gathers its chunks again,
// scans its threads' counts, lays the hits of 8192 elements out in shared memory and writes them
// as one run of consecutive stores.  The reference caps the grid at 1024
// blocks; here it grows with the run up to 65536 CTAs.
#include "common.cuh"

namespace cb200 {

constexpr int kWhereChunksPerThread = 4;
constexpr int kWhereTileChunks = kBlock * kWhereChunksPerThread;        // 1024 chunks = 32768 elements
constexpr int kWhereMaxCtas = 65536;

struct WhereRun {
    const uint32_t* words;
    uint64_t p;            // bit position of element 0
    int64_t s;             // bit step
    const size_t* idx;     // or bit offsets
    uint64_t n;            // elements
    uint64_t n_chunks;
    int contiguous;
    int invert;
};

// elements [32c, 32c+32) of the run as a word, zero past the end
__device__ __forceinline__ uint32_t where_chunk(const WhereRun& r, uint64_t c) {
    const uint64_t e0 = c * 32;
    if (e0 >= r.n) return 0;
    uint32_t z;
    if (r.contiguous) {
        const uint64_t b = r.p + e0;
        const uint64_t w = b >> 5;
        const uint32_t sh = (uint32_t)(b & 31);
        const uint32_t lo = r.words[w];
        // the second word exists only if the chunk really reaches into it
        const uint64_t last_bit = r.p + (e0 + 32 <= r.n ? e0 + 31 : r.n - 1);
        const uint32_t hi = (sh != 0 && (last_bit >> 5) > w) ? r.words[w + 1] : 0u;
        z = __funnelshift_r(lo, hi, sh);
    } else {
        z = 0;
        const uint32_t m = r.n - e0 < 32 ? (uint32_t)(r.n - e0) : 32u;
        for (uint32_t k = 0; k < m; ++k) {
            const uint64_t b = r.idx ? r.p + r.idx[e0 + k] : r.p + (uint64_t)((int64_t)(e0 + k) * r.s);
            z |= ((r.words[b >> 5] >> (b & 31)) & 1u) << k;
        }
    }
    if (r.invert) z = ~z;
    if (r.n - e0 < 32) z &= (1u << (uint32_t)(r.n - e0)) - 1u;
    return z;
}

// exclusive scan of one count per thread over the CTA, thread order; *total = the CTA's sum
__device__ __forceinline__ uint32_t block_exscan(uint32_t v, uint32_t* total, uint32_t* smem /* [warps + 1] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
    }
    if (lane == 31) smem[warp] = inc;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t acc = 0;
        for (int w = 0; w < kWarpsPerBlock; ++w) { const uint32_t t = smem[w]; smem[w] = acc; acc += t; }
        smem[kWarpsPerBlock] = acc;
    }
    __syncthreads();
    const uint32_t pre = smem[warp] + inc - v;
    *total = smem[kWarpsPerBlock];
    __syncthreads();
    return pre;
}

__global__ void __launch_bounds__(kBlock)
where_count_kernel(const WhereRun r, uint64_t tiles_per_cta, uint64_t n_tiles, unsigned long long* cta_sums) {
    const uint64_t t_begin = blockIdx.x * tiles_per_cta;
    uint64_t t_end = t_begin + tiles_per_cta; if (t_end > n_tiles) t_end = n_tiles;
    uint32_t cnt = 0;                          // per thread at most tiles_per_cta * 128: the host keeps that below 2^32
    for (uint64_t t = t_begin; t < t_end; ++t) {
        const uint64_t c0 = t * kWhereTileChunks + (uint64_t)threadIdx.x * kWhereChunksPerThread;
#pragma unroll
        for (int j = 0; j < kWhereChunksPerThread; ++j) cnt += __popc(where_chunk(r, c0 + j));
    }
    // 64-bit CTA total
    unsigned long long v = cnt;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_down_sync(0xffffffffu, v, d);
    __shared__ unsigned long long wsum[kWarpsPerBlock];
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long acc = 0;
        for (int w = 0; w < kWarpsPerBlock; ++w) acc += wsum[w];
        cta_sums[blockIdx.x] = acc;
    }
}

// cta_sums -> exclusive output positions (cursor included); cursor += everything
__global__ void __launch_bounds__(1024)
where_scan_kernel(unsigned long long* cta_sums, uint32_t n_ctas, unsigned long long* running) {
    __shared__ unsigned long long wsum[33];
    __shared__ unsigned long long carry_s;
    if (threadIdx.x == 0) carry_s = *running;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t base = 0; base < n_ctas; base += 1024) {
        const uint32_t i = base + threadIdx.x;
        const unsigned long long v = i < n_ctas ? cta_sums[i] : 0ull;
        unsigned long long inc = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned long long o = __shfl_up_sync(0xffffffffu, inc, d);
            if (lane >= d) inc += o;
        }
        if (lane == 31) wsum[warp] = inc;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long acc = 0;
            for (int w = 0; w < 32; ++w) { const unsigned long long t = wsum[w]; wsum[w] = acc; acc += t; }
            wsum[32] = acc;
        }
        __syncthreads();
        const unsigned long long carry = carry_s;
        if (i < n_ctas) cta_sums[i] = carry + wsum[warp] + inc - v;
        __syncthreads();
        if (threadIdx.x == 0) carry_s = carry + wsum[32];
        __syncthreads();
    }
    if (threadIdx.x == 0) *running = carry_s;
}

// What a hit at element e of the run appends: where -- its position `count + e`; mask -- the byte position
// of element e of the masked array, p2 + e * s2 or p2 + idx2[e] (mask_kernel.cu:6-36 of the reference).
struct WhereEmit {
    uint64_t count;
    __device__ __forceinline__ uint64_t operator()(uint64_t e) const { return count + e; }
};
struct MaskEmit {
    uint64_t p2;
    int64_t s2;
    const size_t* idx2;
    __device__ __forceinline__ uint64_t operator()(uint64_t e) const {
        return idx2 ? p2 + idx2[e] : (uint64_t)((int64_t)p2 + (int64_t)e * s2);
    }
};

template <typename TI, typename Emit>
__global__ void __launch_bounds__(kBlock)
where_scatter_kernel(const WhereRun r, uint64_t tiles_per_cta, uint64_t n_tiles, const unsigned long long* __restrict__ cta_pos,
                     TI* out, const Emit emit) {
    __shared__ uint32_t smem[kWarpsPerBlock + 1];
    // the hits of one sub-tile (kBlock chunks = 8192 elements), as element numbers relative to the sub-tile, in order;
    // slot j of the sub-tile's hits sits at rel[pad + j], pad = the output position of hit 0 modulo 4, so that groups of
    // four slots are groups of four output elements that start on a 16-byte boundary
    __shared__ __align__(8) uint16_t rel[kBlock * 32 + 4];
    constexpr int G = 4;                                   // slots per thread and step of the copy-out
    constexpr int VO = 16 / (int)sizeof(TI);               // output elements per 16-byte store
    const uint64_t t_begin = blockIdx.x * tiles_per_cta;
    uint64_t t_end = t_begin + tiles_per_cta; if (t_end > n_tiles) t_end = n_tiles;
    unsigned long long off = cta_pos[blockIdx.x];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sh = (lane & 7) * 4;                         // this lane's four bits of a word
    const uint32_t below = (1u << sh) - 1u;
    const bool out_aligned = (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
    for (uint64_t t = t_begin; t < t_end; ++t) {
        for (int sub = 0; sub < kWhereChunksPerThread; ++sub) {
            const uint64_t cbase = t * kWhereTileChunks + (uint64_t)sub * kBlock;      // first chunk of the sub-tile
            const uint32_t z = where_chunk(r, cbase + threadIdx.x);
            uint32_t total;
            const uint32_t pad = (uint32_t)(off & (G - 1));
            const uint32_t pre = block_exscan((uint32_t)__popc(z), &total, smem) + pad;
            // Expansion into shared memory, four words of the warp at a time: a lane takes four bits of one word and
            // notes its set bits from the word's offset plus the set bits below its own.
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int wi = it * 4 + (lane >> 3);
                const uint32_t w = __shfl_sync(0xffffffffu, z, wi);
                uint32_t o = __shfl_sync(0xffffffffu, pre, wi) + (uint32_t)__popc(w & below);
                const uint32_t nib = (w >> sh) & 15u;
                const uint32_t id = (uint32_t)((warp * 32 + wi) * 32 + sh);
                if (nib & 1u) rel[o++] = (uint16_t)id;
                if (nib & 2u) rel[o++] = (uint16_t)(id + 1);
                if (nib & 4u) rel[o++] = (uint16_t)(id + 2);
                if (nib & 8u) rel[o] = (uint16_t)(id + 3);
            }
            __syncthreads();
            // The sub-tile's positions leave as one run of consecutive 16-byte stores: whole lines except at the two ends.
            // (Writing each word's few positions straight to global memory made L2 fetch every partly written sector.)
            const uint64_t ebase = cbase * 32;
            TI* const o0 = out + (off - pad);               // output element of slot 0: a multiple of four elements
            const uint32_t end = pad + total;
            for (uint32_t g = threadIdx.x * G; g < end; g += kBlock * G) {
                const uint2 four = *reinterpret_cast<const uint2*>(&rel[g]);
                const uint32_t e0 = four.x & 0xffffu, e1 = four.x >> 16, e2 = four.y & 0xffffu, e3 = four.y >> 16;
                if (g >= pad && g + G <= end && out_aligned) {
                    TI v[G] = {(TI)emit(ebase + e0), (TI)emit(ebase + e1), (TI)emit(ebase + e2), (TI)emit(ebase + e3)};
#pragma unroll
                    for (int k = 0; k < G; k += VO) *reinterpret_cast<int4*>(o0 + g + k) = *reinterpret_cast<const int4*>(&v[k]);
                } else {
                    const uint32_t e[G] = {e0, e1, e2, e3};
#pragma unroll
                    for (int k = 0; k < G; ++k)
                        if (g + k >= pad && g + k < end) o0[g + k] = (TI)emit(ebase + e[k]);
                }
            }
            off += total;
            // the barriers inside the next block_exscan keep `rel` from being rewritten before everyone has read it
        }
    }
}

}  // namespace cb200

using namespace cb200;

// scratch: [cursor for ones][cursor for zeros][per-CTA sums x kWhereMaxCtas], cursors cleared
extern "C" char* cumo_bit_where_scratch_new(void) {
    char* scratch = cumo_cuda_runtime_malloc((2 + (size_t)kWhereMaxCtas) * sizeof(unsigned long long));
    if (scratch) cudaMemsetAsync(scratch, 0, 2 * sizeof(unsigned long long), current_stream());
    cumo_cuda_runtime_check_kernel_launch();
    return scratch;
}

extern "C" void cumo_bit_where_kernel_launch(CUMO_BIT_DIGIT* a, size_t p, ssize_t s, size_t* idx, uint64_t n, int invert, char* out,
                                             size_t elmsz, uint64_t count, char* scratch) {
    if (n == 0 || !scratch) return;
    WhereRun r;
    r.words = a; r.p = p; r.s = s; r.idx = idx; r.n = n;
    r.n_chunks = (n + 31) / 32;
    r.contiguous = idx == nullptr && s == 1;
    r.invert = invert;
    const uint64_t n_tiles = (r.n_chunks + kWhereTileChunks - 1) / kWhereTileChunks;
    uint64_t tiles_per_cta = (n_tiles + kWhereMaxCtas - 1) / kWhereMaxCtas;
    if (tiles_per_cta < 1) tiles_per_cta = 1;
    const uint32_t n_ctas = (uint32_t)((n_tiles + tiles_per_cta - 1) / tiles_per_cta);
    unsigned long long* running = reinterpret_cast<unsigned long long*>(scratch) + (invert ? 1 : 0);
    unsigned long long* cta_sums = reinterpret_cast<unsigned long long*>(scratch) + 2;
    cudaStream_t st = current_stream();
    where_count_kernel<<<n_ctas, kBlock, 0, st>>>(r, tiles_per_cta, n_tiles, cta_sums);
    where_scan_kernel<<<1, 1024, 0, st>>>(cta_sums, n_ctas, running);
    const WhereEmit emit{count};
    if (elmsz == 8) where_scatter_kernel<int64_t><<<n_ctas, kBlock, 0, st>>>(r, tiles_per_cta, n_tiles, cta_sums, reinterpret_cast<int64_t*>(out), emit);
    else            where_scatter_kernel<int32_t><<<n_ctas, kBlock, 0, st>>>(r, tiles_per_cta, n_tiles, cta_sums, reinterpret_cast<int32_t*>(out), emit);
    count_launch(3);
    cumo_cuda_runtime_check_kernel_launch();
}

// Bit#mask (narray/gen/tmpl_bit/mask.c:1 declares it, mask_kernel.cu:38-53 defines it): the same compaction, but a
// set bit at element i of the run appends the BYTE position of element i of the masked array -- p2 + i * s2, or
// p2 + idx2[i] when that array is itself addressed through an index array -- as a size_t.  The host then wraps
// `out` as the index array of a 1-D view of the masked array.  Same scratch and cursor protocol as where.
extern "C" void cumo_bit_mask_kernel_launch(CUMO_BIT_DIGIT* a, size_t p, ssize_t s, size_t* idx, uint64_t n, size_t* out, size_t p2,
                                            ssize_t s2, size_t* idx2, char* scratch) {
    if (n == 0 || !scratch) return;
    WhereRun r;
    r.words = a; r.p = p; r.s = s; r.idx = idx; r.n = n;
    r.n_chunks = (n + 31) / 32;
    r.contiguous = idx == nullptr && s == 1;
    r.invert = 0;
    const uint64_t n_tiles = (r.n_chunks + kWhereTileChunks - 1) / kWhereTileChunks;
    uint64_t tiles_per_cta = (n_tiles + kWhereMaxCtas - 1) / kWhereMaxCtas;
    if (tiles_per_cta < 1) tiles_per_cta = 1;
    const uint32_t n_ctas = (uint32_t)((n_tiles + tiles_per_cta - 1) / tiles_per_cta);
    unsigned long long* running = reinterpret_cast<unsigned long long*>(scratch);
    unsigned long long* cta_sums = reinterpret_cast<unsigned long long*>(scratch) + 2;
    cudaStream_t st = current_stream();
    where_count_kernel<<<n_ctas, kBlock, 0, st>>>(r, tiles_per_cta, n_tiles, cta_sums);
    where_scan_kernel<<<1, 1024, 0, st>>>(cta_sums, n_ctas, running);
    const MaskEmit emit{(uint64_t)p2, (int64_t)s2, idx2};
    where_scatter_kernel<unsigned long long><<<n_ctas, kBlock, 0, st>>>(r, tiles_per_cta, n_tiles, cta_sums, reinterpret_cast<unsigned long long*>(out), emit);
    count_launch(3);
    cumo_cuda_runtime_check_kernel_launch();
}
