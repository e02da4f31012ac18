// k-means assignment step on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// Same contract as kmeans.cu (labels = argmin_k(|c_k|^2 - 2 <x, c_k>), lowest k on ties,
// counts per cluster); the contraction <x, c_k> is done by tcgen05.mma with TF32 operands and
// fp32 accumulators in tensor memory.  To keep fp32-grade accuracy every operand is split into
// a TF32 head and a tail (x = x_hi + x_lo exactly in fp32; the head is exactly a TF32 number, the
// tail's 13 significant bits are cut to 11 by the tensor core, an error of 2^-22 relative to x)
// and three products are accumulated: x_hi.c_hi + x_lo.c_hi + x_hi.c_lo (the dropped x_lo.c_lo
// term is also ~2^-22 relative).  This is the contraction the reference hands to cuBLAS (bench/kmeans_bench.rb:110),
// fused with the |c|^2 add and the row argmin so that the (N, K) matrix only ever exists as one
// 128 x K tile in tensor memory.
//
// One persistent CTA per SM, 13 warps:
//   warp 0        allocates tensor memory, issues every tcgen05.mma (one thread)
//   warps 1..8    producers, two groups of 128 threads that take alternate K-blocks: copy a block of
//                 128 points x 32 features from global memory into a 128-byte-swizzled, K-major
//                 shared-memory slot (ring of 3), splitting hi/lo on the way; each group holds its
//                 next block in registers while it waits for a slot, so two blocks are always in flight
//   warps 9..12   epilogue: tcgen05.ld the 128 x K accumulator tile (one point per thread, 16 columns
//                 at a time, the next load issued before the current one is scanned), add |c_k|^2,
//                 keep the first minimum in four independent chains, write label / distance, count clusters
// The centroid table (hi and lo, swizzled, K-major) stays in shared memory for the whole kernel.
// Two accumulator tiles (2 x 256 columns = all of tensor memory) let the epilogue of one tile
// overlap the MMAs of the next.  Shared-memory slots and accumulators are handed over through
// mbarriers; every wait is bounded and, on expiry, raises an error word that the host reads.
#include "common.cuh"
#include "tc_common.cuh"

#include <cstdio>
#include <mutex>

namespace cb200 {

constexpr int kTcPoints = 128;           // M: points per tile
constexpr int kTcKBlock = 32;            // fp32 features per 128-byte swizzle row
constexpr int kTcSlots = 3;              // ring of K-block slots for the points
constexpr int kTcSlotBytes = 2 * kTcPoints * 128;   // hi + lo
// dynamic shared memory (1024-byte aligned):
//   B hi [KB][N][128B] | B lo [KB][N][128B] | A slots [3][hi 128x128B | lo 128x128B] | cnorm[N] | hist[N] | barriers | tmem slot | abort
__global__ void __launch_bounds__(416, 1)
kmeans_assign_tc_kernel(const float* __restrict__ x, int64_t n, int d, const float* __restrict__ c, int k, int n_pad,
                        int32_t* __restrict__ labels, float* __restrict__ min_dist, unsigned long long* __restrict__ counts,
                        int64_t n_tiles, int* __restrict__ error_word) {
    extern __shared__ __align__(1024) char smem_raw[];
    char* base = smem_raw;
    if ((smem_u32(base) & 1023u) != 0) {          // the swizzled blocks need 1024-byte alignment; uniform exit before any barrier
        if (threadIdx.x == 0) atomicExch(error_word, 2);
        return;
    }
    const int KB = d / kTcKBlock;
    const uint32_t b_block = (uint32_t)n_pad * 128u;                 // one K-block of the centroid table
    char* b_hi = base;
    char* b_lo = b_hi + (size_t)KB * b_block;
    char* a_slots = b_lo + (size_t)KB * b_block;
    float* cnorm = reinterpret_cast<float*>(a_slots + kTcSlots * kTcSlotBytes);
    unsigned* hist = reinterpret_cast<unsigned*>(cnorm + n_pad);
    uint64_t* bars = reinterpret_cast<uint64_t*>(hist + n_pad);
    uint64_t* slot_full = bars;               // [3] producers -> MMA, 128 arrivals (one group fills a slot)
    uint64_t* slot_empty = bars + 3;          // [3] MMA -> producers, tcgen05.commit
    uint64_t* acc_full = bars + 6;            // [2] MMA -> epilogue, tcgen05.commit
    uint64_t* acc_empty = bars + 8;           // [2] epilogue -> MMA, 128 arrivals
    uint64_t* drain = bars + 10;              // [1] MMA -> itself: everything issued has finished (used when giving up)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- set-up by everyone: centroid table (hi/lo, swizzled), its norms, barriers --------------
    for (int i = tid; i < n_pad * (d / 4); i += blockDim.x) {
        const int kk = i / (d / 4), q = i - kk * (d / 4);          // q-th float4 of centroid kk
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kk < k) v = *reinterpret_cast<const float4*>(c + (size_t)kk * d + q * 4);
        const int kb = q >> 3, ch = q & 7;
        split_store(b_hi + (size_t)kb * b_block, b_lo + (size_t)kb * b_block, swz(kk, ch), v);
    }
    for (int kk = tid; kk < n_pad; kk += blockDim.x) {
        float s = INFINITY;                                        // padding centroids can never win
        if (kk < k) { s = 0.f; for (int q = 0; q < d; ++q) { const float v = c[(size_t)kk * d + q]; s = fmaf(v, v, s); } }
        cnorm[kk] = s;
        hist[kk] = 0;
    }
    if (tid == 0) {
        for (int i = 0; i < 3; ++i) { mbar_init(slot_full + i, 128); mbar_init(slot_empty + i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(acc_full + i, 1); mbar_init(acc_empty + i, 128); }
        mbar_init(drain, 1);
        abort_flag[0] = 0;
        abort_flag[1] = 0;                    // never set: the drain wait below polls it as its "someone gave up" word
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the table was written by ordinary stores
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int64_t my_tiles = n_tiles > blockIdx.x ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (warp == 0) {
        // ---- MMA issuer ---------------------------------------------------------------------
        if (lane == 0) {
            // M = 128, N = n_pad, TF32 x TF32 -> F32, both operands K-major
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n_pad >> 3) << 17) | ((uint32_t)(kTcPoints >> 4) << 24);
            uint32_t it = 0;                      // K-blocks consumed so far
            for (int64_t t = 0; t < my_tiles; ++t) {
                const uint32_t acc = (uint32_t)(t & 1);
                if (!mbar_wait(acc_empty + acc, ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + acc * 256u;
                bool ok = true;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const uint32_t slot = it % kTcSlots;
                    if (!mbar_wait(slot_full + slot, (it / kTcSlots) & 1u, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_hi = smem_u32(a_slots + slot * kTcSlotBytes);
                    const uint32_t a_lo = a_hi + kTcPoints * 128u;
                    const uint32_t bh = smem_u32(b_hi + (size_t)kb * b_block), bl = smem_u32(b_lo + (size_t)kb * b_block);
#pragma unroll
                    for (int term = 0; term < 3; ++term) {
                        const uint32_t a_addr = term == 1 ? a_lo : a_hi;
                        const uint32_t b_addr = term == 2 ? bl : bh;
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {          // 8 TF32 (32 bytes) of K per instruction
                            const uint64_t da = umma_desc(a_addr + ks * 32u), db = umma_desc(b_addr + ks * 32u);
                            const uint32_t accumulate = (kb | term | ks) != 0;
                            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                         "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                                         ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
                        }
                    }
                    // the slot is free again once these MMAs have read it
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(slot_empty + slot)) : "memory");
                }
                if (!ok) break;
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(acc_full + acc)) : "memory");
            }
            // whatever happened above, let the MMAs already issued finish before tensor memory is freed (bounded, like every wait)
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(drain)) : "memory");
            mbar_wait(drain, 0u, abort_flag + 1);
        }
        __syncwarp();
    } else if (warp <= 8) {
        // ---- producers: two groups of 128 threads, 8 lanes per point row ---------------------
        const int pt = (tid - 32) & 127;
        const uint32_t group = (uint32_t)(tid - 32) >> 7;      // 0 or 1: K-blocks group, group + 2, ... are mine
        const uint32_t ch = pt & 7;                // 16-byte chunk of the 128-byte row
        const int r0 = pt >> 3;                    // first of my rows; I take rows r0, r0+16, ...
        const uint32_t total = (uint32_t)(my_tiles * KB);
        float4 cur[8], nxt[8];
        auto fetch = [&](uint32_t it, float4 (&v)[8]) {
            const uint32_t t = it / (uint32_t)KB, kb = it - t * (uint32_t)KB;
            const int64_t p0 = ((int64_t)blockIdx.x + (int64_t)t * gridDim.x) * kTcPoints;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int64_t p = p0 + r0 + i * 16;
                v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (p < n) v[i] = __ldcs(reinterpret_cast<const float4*>(x + (size_t)p * d + kb * kTcKBlock + ch * 4));
            }
        };
        uint32_t it = group;
        if (it < total) fetch(it, cur);
        for (; it < total; it += 2) {
            if (it + 2 < total) fetch(it + 2, nxt);            // in flight while this block waits for its slot
            const uint32_t slot = it % kTcSlots;
            if (!mbar_wait(slot_empty + slot, ((it / kTcSlots) & 1u) ^ 1u, abort_flag)) break;
            char* hi = a_slots + slot * kTcSlotBytes;
            char* lo = hi + kTcPoints * 128;
#pragma unroll
            for (int i = 0; i < 8; ++i) split_store(hi, lo, swz((uint32_t)(r0 + i * 16), ch), cur[i]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(slot_full + slot);
#pragma unroll
            for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
        }
    } else {
        // ---- epilogue: one point (one tensor-memory lane) per thread ---------------------------
        const uint32_t quarter = (uint32_t)(warp & 3);             // the lanes this warp may read
        const int row = (int)quarter * 32 + lane;
        const int n_chunks = n_pad >> 4;
        for (int64_t t = 0; t < my_tiles; ++t) {
            const uint32_t acc = (uint32_t)(t & 1);
            // tcgen05.ld is warp-collective: the warp leaves together or not at all
            if (!__all_sync(0xffffffffu, mbar_wait(acc_full + acc, (uint32_t)(t >> 1) & 1u, abort_flag))) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + acc * 256u + ((quarter * 32u) << 16);
            // chain q sees columns q, q+4, q+8, ... in rising order; a strict compare keeps the earliest
            float best[4] = {INFINITY, INFINITY, INFINITY, INFINITY};
            int best_k[4] = {0, 0, 0, 0};
            auto scan16 = [&](int c0, const uint32_t (&r)[16]) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float dist = fmaf(-2.f, __uint_as_float(r[j]), cnorm[c0 + j]);
                    if (dist < best[j & 3]) { best[j & 3] = dist; best_k[j & 3] = c0 + j; }
                }
            };
            uint32_t ra[16], rb[16];
            tmem_ld16(taddr, ra);
            tmem_ld_wait(ra);
            for (int chn = 0; chn < n_chunks; chn += 2) {
                const bool more1 = chn + 1 < n_chunks, more2 = chn + 2 < n_chunks;      // warp-uniform
                if (more1) tmem_ld16(taddr + (uint32_t)(chn + 1) * 16u, rb);
                scan16(chn * 16, ra);
                if (more1) {
                    tmem_ld_wait(rb);
                    if (more2) tmem_ld16(taddr + (uint32_t)(chn + 2) * 16u, ra);
                    scan16((chn + 1) * 16, rb);
                    if (more2) tmem_ld_wait(ra);
                }
            }
            // the accumulator tile may be overwritten now
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(acc_empty + acc);
            float bv = best[0];
            int bk = best_k[0];
#pragma unroll
            for (int q = 1; q < 4; ++q)
                if (best[q] < bv || (best[q] == bv && best_k[q] < bk)) { bv = best[q]; bk = best_k[q]; }
            const int64_t p = ((int64_t)blockIdx.x + t * gridDim.x) * kTcPoints + row;
            if (p < n) {
                labels[p] = bk;
                if (min_dist) min_dist[p] = bv;
                atomicAdd(&hist[bk], 1u);
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
    if (abort_flag[0] | abort_flag[1]) {
        if (tid == 0) atomicExch(error_word, 1);
        return;
    }
    if (counts)
        for (int kk = tid; kk < k; kk += blockDim.x)
            if (hist[kk]) atomicAdd(counts + kk, (unsigned long long)hist[kk]);
}

static size_t tc_smem_bytes(int d, int n_pad) {
    const size_t KB = d / kTcKBlock;
    return 2 * KB * (size_t)n_pad * 128 + (size_t)kTcSlots * kTcSlotBytes + 2 * (size_t)n_pad * 4 + 11 * 8 + 16;
}

// status word of the kernel's bounded waits, one per device that loads the library (host code sees only a handle)
static __device__ int g_kmeans_assign_tc_error_word;

}  // namespace cb200

// The tensor-core form.  Shapes: d a multiple of 32, k <= 256, and the table must fit shared memory
// (d = 64 with k <= 256 does).  error: 0 ok, 1/2 shape not supported (nothing launched), 3/4 launch problems,
// 5 a bounded wait inside the kernel ran out (results are not valid).  This last check synchronises the
// stream, since the word is written by the kernel.
extern "C" int cb200_kmeans_assign_sfloat_tc(const float* x, int64_t n, int d, const float* c, int k, int32_t* labels,
                                             float* min_dist, unsigned long long* counts, char* errbuf, size_t errlen) {
    using namespace cb200;
    char local[8];
    if (!errbuf || errlen == 0) { errbuf = local; errlen = sizeof local; }
    errbuf[0] = 0;
    if (n <= 0) return 0;
    if (d < 32 || d % 32 != 0 || k < 1 || k > 256) {
        snprintf(errbuf, errlen, "kmeans_assign_tc: needs D a multiple of 32 and 1 <= K <= 256 (D=%d, K=%d)", d, k);
        return 1;
    }
    if (!aligned16(x) || !aligned16(c)) { snprintf(errbuf, errlen, "kmeans_assign_tc: x and c must be 16-byte aligned"); return 1; }
    const int n_pad = (k + 15) / 16 * 16;
    const size_t smem = tc_smem_bytes(d, n_pad);
    if (smem > 227 * 1024) {
        snprintf(errbuf, errlen, "kmeans_assign_tc: K=%d x D=%d needs %zu bytes of shared memory (limit %d)", k, d, smem, 227 * 1024);
        return 2;
    }
    // one call at a time per process: the error word is per device, and the call ends with a read-back anyway
    static std::mutex call_mutex;
    std::lock_guard<std::mutex> lock(call_mutex);
    struct PerDevice { bool ready; int* error_word; };
    static PerDevice dev_state[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!dev_state[dev].ready) {
        cudaError_t e = cudaFuncSetAttribute(kmeans_assign_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) { snprintf(errbuf, errlen, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return 3; }
        // the word lives in the library image: no allocator callback (which, inside the Ruby extension, may
        // raise with a longjmp) is ever called while call_mutex is held
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&dev_state[dev].error_word), g_kmeans_assign_tc_error_word);
        if (e != cudaSuccess || !dev_state[dev].error_word) { snprintf(errbuf, errlen, "kmeans_assign_tc: cudaGetSymbolAddress: %s", cudaGetErrorString(e)); return 3; }
        dev_state[dev].ready = true;
    }
    cudaStream_t st = current_stream();
    cudaMemsetAsync(dev_state[dev].error_word, 0, sizeof(int), st);
    const int64_t n_tiles = (n + kTcPoints - 1) / kTcPoints;
    const unsigned grid = grid_for(n_tiles, 1);
    kmeans_assign_tc_kernel<<<grid, 416, smem, st>>>(x, n, d, c, k, n_pad, labels, min_dist, counts, n_tiles, dev_state[dev].error_word);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { snprintf(errbuf, errlen, "kmeans_assign_tc launch: %s", cudaGetErrorString(e)); return 4; }
    int word = 0;
    e = cudaMemcpyAsync(&word, dev_state[dev].error_word, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { snprintf(errbuf, errlen, "kmeans_assign_tc: %s", cudaGetErrorString(e)); return 4; }
    if (word) { snprintf(errbuf, errlen, "kmeans_assign_tc: a bounded wait inside the kernel ran out; results are not valid"); return 5; }
    return 0;
}
