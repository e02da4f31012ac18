// Single-precision matrix product on the 5th-generation tensor cores (tcgen05, sm_100a):
//     C[M, N] = A[M, K] . Bt[N, K]^T          (all row-major; K is the contiguous axis of both inputs)
//
// This is the contraction the reference hands to cublasSgemm for `a.dot(b)` on 2-D SFloat operands
// (ext/cumo/narray/gen/tmpl/gemm.c:252-297).  It is computed with TF32 tensor-core instructions at
// fp32-grade accuracy by splitting every operand into a TF32 head and tail and accumulating three
// products per term (see kmeans_tc.cu, which uses the same scheme); accumulators are fp32 in tensor
// memory, for at most 512 elements of K at a time: the tensor cores add into the accumulator with
// truncation, a bias that grows with the length of the chain (measured: 1e-2 absolute on sums of
// magnitude 300 at K = 4096), so after every 16 K-blocks the epilogue takes the partial product over
// into C with ordinary rounded fp32 additions and the MMAs start a fresh accumulator.
// Bt is the second operand with its axes swapped: the caller passes `b` itself when it is
// already laid out that way (a weight matrix stored [out, in]) or a transposed copy otherwise.
//
// One persistent CTA per SM owns 128 x 256 tiles of C, 13 warps:
//   warp 0        allocates tensor memory and issues every tcgen05.mma (one thread)
//   warps 1..8    producers: per K-block of 32 they copy 128 rows of A and 256 rows of Bt from global
//                 memory into a 128-byte-swizzled, K-major stage in shared memory (ring of 2), splitting
//                 hi/lo on the way, with the next K-block already loaded into registers
//   warps 9..12   epilogue: tcgen05.ld of the finished 128 x 256 accumulator (one row of C per thread),
//                 stores to C
// Two accumulators (all 512 columns of tensor memory) let the epilogue of one tile overlap the MMAs of
// the next.  Every hand-over is an mbarrier with a bounded wait; on expiry the kernel raises an error
// word, drains what it issued, frees tensor memory and returns.
#include "common.cuh"
#include "tc_common.cuh"

#include <cstdio>
#include <mutex>

namespace cb200 {

constexpr int kGemmM = 128, kGemmN = 256, kGemmKB = 32;
constexpr int kGemmStages = 2;
constexpr int kGemmChunkBlocks = 16;                             // K-blocks accumulated in tensor memory before C takes them over
constexpr int kGemmStageBytes = 2 * (kGemmM + kGemmN) * 128;     // hi + lo of A and Bt rows: 96 KiB
constexpr int kGemmProducers = 256;                              // threads
constexpr int kGemmLoads = (kGemmM + kGemmN) * 8 / kGemmProducers;   // 16-byte chunks per producer thread per K-block: 12

// stage layout: A hi [128 x 128B] | A lo | Bt hi [256 x 128B] | Bt lo
__global__ void __launch_bounds__(416, 1)
sgemm_nt_tc_kernel(const float* __restrict__ A, int64_t lda, const float* __restrict__ Bt, int64_t ldb, float* __restrict__ C, int64_t ldc,
                   int64_t M, int64_t N, int64_t K, int64_t tiles_m, int64_t n_tiles, int* __restrict__ error_word) {
    extern __shared__ __align__(1024) char smem_raw[];
    char* base = smem_raw;
    if ((smem_u32(base) & 1023u) != 0) {          // the swizzled blocks need 1024-byte alignment; uniform exit before any barrier
        if (threadIdx.x == 0) atomicExch(error_word, 2);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + kGemmStages * kGemmStageBytes);
    uint64_t* slot_full = bars;               // [2] producers -> MMA, 256 arrivals
    uint64_t* slot_empty = bars + 2;          // [2] MMA -> producers, tcgen05.commit
    uint64_t* acc_full = bars + 4;            // [2] MMA -> epilogue, tcgen05.commit
    uint64_t* acc_empty = bars + 6;           // [2] epilogue -> MMA, 128 arrivals
    uint64_t* drain = bars + 8;               // [1] MMA -> itself: everything issued has finished
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < kGemmStages; ++i) { mbar_init(slot_full + i, kGemmProducers); mbar_init(slot_empty + i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(acc_full + i, 1); mbar_init(acc_empty + i, 128); }
        mbar_init(drain, 1);
        abort_flag[0] = 0;
        abort_flag[1] = 0;                    // never set: the drain wait polls it as its "someone gave up" word
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t KB = (uint32_t)((K + kGemmKB - 1) / kGemmKB);
    const int64_t my_tiles = n_tiles > blockIdx.x ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // tile t of this CTA -> (row block, column block); row blocks vary fastest so that CTAs running
    // together share the same 256 rows of Bt.  (Numbering the tiles in bands of 16 row blocks, which cuts the
    // DRAM reads of A from once per column block to about once, measured 12 % slower at 8192^3: the kernel is
    // bound by shared-memory traffic, not by DRAM.)
    auto tile_of = [&](int64_t t, int64_t* m0, int64_t* n0) {
        const int64_t g = (int64_t)blockIdx.x + t * gridDim.x;
        const int64_t tn = g / tiles_m;
        *m0 = (g - tn * tiles_m) * kGemmM;
        *n0 = tn * kGemmN;
    };

    if (warp == 0) {
        // ---- MMA issuer ---------------------------------------------------------------------
        if (lane == 0) {
            // M = 128, N = 256, TF32 x TF32 -> F32, both operands K-major
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kGemmN >> 3) << 17) | ((uint32_t)(kGemmM >> 4) << 24);
            uint32_t it = 0;                      // K-blocks consumed so far
            uint32_t item = 0;                    // (tile, K-chunk) pairs issued so far: each gets an accumulator of its own
            bool ok = true;
            for (int64_t t = 0; t < my_tiles && ok; ++t) {
                for (uint32_t kb0 = 0; kb0 < KB && ok; kb0 += kGemmChunkBlocks, ++item) {
                    const uint32_t acc = item & 1u;
                    if (!mbar_wait(acc_empty + acc, ((item >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t d_tmem = tmem_base + acc * 256u;
                    const uint32_t kb1 = kb0 + kGemmChunkBlocks < KB ? kb0 + kGemmChunkBlocks : KB;
                    for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
                        const uint32_t slot = it % kGemmStages;
                        if (!mbar_wait(slot_full + slot, (it / kGemmStages) & 1u, abort_flag)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t a_hi = smem_u32(base + slot * kGemmStageBytes);
                        const uint32_t a_lo = a_hi + kGemmM * 128u;
                        const uint32_t b_hi = a_lo + kGemmM * 128u;
                        const uint32_t b_lo = b_hi + kGemmN * 128u;
#pragma unroll
                        for (int term = 0; term < 3; ++term) {
                            const uint32_t a_addr = term == 1 ? a_lo : a_hi;
                            const uint32_t b_addr = term == 2 ? b_lo : b_hi;
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) {          // 8 TF32 (32 bytes) of K per instruction
                                const uint64_t da = umma_desc(a_addr + ks * 32u), db = umma_desc(b_addr + ks * 32u);
                                const uint32_t accumulate = ((kb - kb0) | (uint32_t)term | (uint32_t)ks) != 0;
                                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                             "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                                             ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
                            }
                        }
                        // the stage is free again once these MMAs have read it
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(slot_empty + slot)) : "memory");
                    }
                    if (!ok) break;
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(acc_full + acc)) : "memory");
                }
            }
            // whatever happened above, let the MMAs already issued finish before tensor memory is freed (bounded, like every wait)
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(drain)) : "memory");
            mbar_wait(drain, 0u, abort_flag + 1);
        }
        __syncwarp();
    } else if (warp <= 8) {
        // ---- producers: 256 threads, 8 lanes per 128-byte row -----------------------------------
        const int pt = tid - 32;                   // 0..255
        const uint32_t ch = pt & 7;                // 16-byte chunk of the row
        const int r0 = pt >> 3;                    // rows r0, r0+32, ...: 0..127 are A's, 128..383 are Bt's
        const uint32_t total = (uint32_t)(my_tiles * KB);
        float4 cur[kGemmLoads], nxt[kGemmLoads];
        auto fetch = [&](uint32_t it, float4 (&v)[kGemmLoads]) {
            const uint32_t t = it / KB, kb = it - t * KB;
            int64_t m0, n0;
            tile_of((int64_t)t, &m0, &n0);
            const int64_t kcol = (int64_t)kb * kGemmKB + ch * 4;
#pragma unroll
            for (int i = 0; i < kGemmLoads; ++i) {
                const int row = r0 + i * 32;
                v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (kcol < K) {
                    if (row < kGemmM) { if (m0 + row < M) v[i] = __ldg(reinterpret_cast<const float4*>(A + (m0 + row) * lda + kcol)); }
                    else { const int rb = row - kGemmM; if (n0 + rb < N) v[i] = __ldg(reinterpret_cast<const float4*>(Bt + (n0 + rb) * ldb + kcol)); }
                }
            }
        };
        uint32_t it = 0;
        if (it < total) fetch(it, cur);
        for (; it < total; ++it) {
            if (it + 1 < total) fetch(it + 1, nxt);               // in flight while this block waits for its stage
            const uint32_t slot = it % kGemmStages;
            if (!mbar_wait(slot_empty + slot, ((it / kGemmStages) & 1u) ^ 1u, abort_flag)) break;
            char* a_hi = base + slot * kGemmStageBytes;
            char* a_lo = a_hi + kGemmM * 128;
            char* b_hi = a_lo + kGemmM * 128;
            char* b_lo = b_hi + kGemmN * 128;
#pragma unroll
            for (int i = 0; i < kGemmLoads; ++i) {
                const int row = r0 + i * 32;
                if (row < kGemmM) split_store(a_hi, a_lo, swz((uint32_t)row, ch), cur[i]);
                else split_store(b_hi, b_lo, swz((uint32_t)(row - kGemmM), ch), cur[i]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(slot_full + slot);
#pragma unroll
            for (int i = 0; i < kGemmLoads; ++i) cur[i] = nxt[i];
        }
    } else {
        // ---- epilogue: one row of C (one tensor-memory lane) per thread ------------------------
        const uint32_t quarter = (uint32_t)(warp & 3);             // the lanes this warp may read
        const int row = (int)quarter * 32 + lane;
        uint32_t item = 0;
        bool ok = true;
        for (int64_t t = 0; t < my_tiles && ok; ++t) {
            int64_t m0, n0;
            tile_of(t, &m0, &n0);
            float* crow = C + (m0 + row) * ldc + n0;
            const bool row_ok = m0 + row < M;
            const bool vec_ok = ((reinterpret_cast<uintptr_t>(crow) & 15) == 0);
            for (uint32_t kb0 = 0; kb0 < KB; kb0 += kGemmChunkBlocks, ++item) {
                const uint32_t acc = item & 1u;
                // tcgen05.ld is warp-collective: the warp leaves together or not at all
                if (!__all_sync(0xffffffffu, mbar_wait(acc_full + acc, (item >> 1) & 1u, abort_flag))) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + acc * 256u + ((quarter * 32u) << 16);
                const bool add = kb0 > 0;             // later K-chunks are added to what C already holds, rounded to nearest
                uint32_t ra[16], rb[16];
                // what C holds so far for 16 columns, requested a step ahead so that the round trip overlaps the step before
                float4 oa[4], ob[4];
                auto fetch16 = [&](int c0, float4 (&o)[4]) {
                    if (!(add && row_ok && vec_ok && n0 + c0 + 16 <= N)) return;
#pragma unroll
                    for (int q = 0; q < 4; ++q) o[q] = *(reinterpret_cast<const float4*>(crow + c0) + q);
                };
                auto put16 = [&](int c0, const uint32_t (&r)[16], const float4 (&o)[4]) {
                    if (!row_ok) return;
                    if (vec_ok && n0 + c0 + 16 <= N) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                            if (add) { v.x += o[q].x; v.y += o[q].y; v.z += o[q].z; v.w += o[q].w; }
                            *(reinterpret_cast<float4*>(crow + c0) + q) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (n0 + c0 + j < N) crow[c0 + j] = add ? crow[c0 + j] + __uint_as_float(r[j]) : __uint_as_float(r[j]);
                    }
                };
                constexpr int n_chunks = kGemmN / 16;
                fetch16(0, oa);
                tmem_ld16(taddr, ra);
                tmem_ld_wait(ra);
#pragma unroll 1
                for (int chn = 0; chn < n_chunks; chn += 2) {
                    tmem_ld16(taddr + (uint32_t)(chn + 1) * 16u, rb);
                    fetch16((chn + 1) * 16, ob);
                    put16(chn * 16, ra, oa);
                    tmem_ld_wait(rb);
                    if (chn + 2 < n_chunks) { tmem_ld16(taddr + (uint32_t)(chn + 2) * 16u, ra); fetch16((chn + 2) * 16, oa); }
                    put16((chn + 1) * 16, rb, ob);
                    if (chn + 2 < n_chunks) tmem_ld_wait(ra);
                }
                // the accumulator may be overwritten now
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(acc_empty + acc);
            }
        }
    }

    // ---- wind-down: everyone meets here, also after a bounded wait ran out ----------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
    if ((abort_flag[0] | abort_flag[1]) && tid == 0) atomicExch(error_word, 1);
}

// status word of the kernel's bounded waits, one per device that loads the library (host code sees only a handle)
static __device__ int g_sgemm_nt_tc_error_word;

}  // namespace cb200

// C[M, N] = A[M, K] . Bt[N, K]^T, float32, row-major with leading dimensions in elements.
// Needs K, lda and ldb multiples of 4 and A, Bt 16-byte aligned (rows are read as 16-byte packets).
// error: 0 ok, 1 shape or alignment not supported (nothing launched), 3/4 launch problems, 5 a bounded wait
// inside the kernel ran out (results are not valid).  Reads an error word back: synchronises the stream.
extern "C" int cb200_sgemm_nt_tc(int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* Bt, int64_t ldb,
                                 float* C, int64_t ldc, char* errbuf, size_t errlen) {
    using namespace cb200;
    char local[8];
    if (!errbuf || errlen == 0) { errbuf = local; errlen = sizeof local; }
    errbuf[0] = 0;
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 4 != 0 || lda % 4 != 0 || ldb % 4 != 0 || lda < K || ldb < K || ldc < N || !aligned16(A) || !aligned16(Bt) ||
        (reinterpret_cast<uintptr_t>(C) & 3) != 0) {
        snprintf(errbuf, errlen, "sgemm_nt_tc: needs K, lda, ldb multiples of 4 (K=%lld lda=%lld ldb=%lld) and 16-byte aligned A, Bt",
                 (long long)K, (long long)lda, (long long)ldb);
        return 1;
    }
    const size_t smem = (size_t)kGemmStages * kGemmStageBytes + 9 * 8 + 16;
    // one call at a time per process: the error word is per device, and the call ends with a read-back anyway
    static std::mutex call_mutex;
    std::lock_guard<std::mutex> lock(call_mutex);
    struct PerDevice { bool ready; int* error_word; };
    static PerDevice dev_state[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!dev_state[dev].ready) {
        cudaError_t e = cudaFuncSetAttribute(sgemm_nt_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) { snprintf(errbuf, errlen, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return 3; }
        // the word lives in the library image: no allocator callback (which, inside the Ruby extension, may
        // raise with a longjmp) is ever called while call_mutex is held
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&dev_state[dev].error_word), g_sgemm_nt_tc_error_word);
        if (e != cudaSuccess || !dev_state[dev].error_word) { snprintf(errbuf, errlen, "sgemm_nt_tc: cudaGetSymbolAddress: %s", cudaGetErrorString(e)); return 3; }
        dev_state[dev].ready = true;
    }
    cudaStream_t st = current_stream();
    cudaMemsetAsync(dev_state[dev].error_word, 0, sizeof(int), st);
    const int64_t tiles_m = (M + kGemmM - 1) / kGemmM, tiles_n = (N + kGemmN - 1) / kGemmN;
    const int64_t n_tiles = tiles_m * tiles_n;
    const unsigned grid = grid_for(n_tiles, 1);
    sgemm_nt_tc_kernel<<<grid, 416, smem, st>>>(A, lda, Bt, ldb, C, ldc, M, N, K, tiles_m, n_tiles, dev_state[dev].error_word);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { snprintf(errbuf, errlen, "sgemm_nt_tc launch: %s", cudaGetErrorString(e)); return 4; }
    int word = 0;
    e = cudaMemcpyAsync(&word, dev_state[dev].error_word, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { snprintf(errbuf, errlen, "sgemm_nt_tc: %s", cudaGetErrorString(e)); return 4; }
    if (word) { snprintf(errbuf, errlen, "sgemm_nt_tc: a bounded wait inside the kernel ran out; results are not valid"); return 5; }
    return 0;
}
