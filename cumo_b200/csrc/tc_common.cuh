// Pieces shared by the tcgen05 kernels (sm_100a): mbarrier helpers with bounded waits, the shared-memory
// matrix descriptor for K-major operands in the 128-byte swizzle, the hi/lo TF32 split, tensor-memory loads.
#pragma once

#include "common.cuh"

namespace cb200 {

constexpr uint32_t kSpinLimit = 1u << 22;      // polls of ~50 ns each: a fraction of a second at most

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// bounded wait: false when the limit ran out or another role already gave up
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t limit = kSpinLimit) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < limit; ++spin) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (spin > 16) __nanosleep(32);
        if ((spin & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups of 1024 bytes
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);            // start address
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused with this swizzle)
    d |= (uint64_t)(1024u >> 4) << 32;                   // stride byte offset: one 8-row group
    d |= (uint64_t)1 << 46;                              // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                              // 128-byte swizzle
    return d;
}

// byte offset of 16-byte chunk `c` of row `r` inside a swizzled block
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

__device__ __forceinline__ void split_store(char* hi_block, char* lo_block, uint32_t off, float4 v) {
    float4 h, l;
    h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = v.x - h.x;
    h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = v.y - h.y;
    h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = v.z - h.z;
    h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = v.w - h.w;
    *reinterpret_cast<float4*>(hi_block + off) = h;
    *reinterpret_cast<float4*>(lo_block + off) = l;
}

// 16 consecutive columns of this warp's 32 tensor-memory lanes, one lane per thread (asynchronous)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
// waits for every tcgen05.ld this thread has issued; the registers pass through it so that no use can move above
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :: "memory");
}

}  // namespace cb200
