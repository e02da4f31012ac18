// All-gather of a few KiB per GPU through peer memory: the exchange step of a row-sharded reduction.
//
// After the local reduction every rank holds a partial of a few bytes to a few tens of KiB per output set, and every
// rank needs everyone's.  A library all-gather of that size costs its fixed latency (10-20 us at 4-8 ranks: several
// times the data's flight time over NVLink); here one small kernel per rank does it:
//
//   1. every CTA takes a slice of this rank's partial and stores it, 16 bytes per thread, into slot [rank] of EVERY
//      rank's exchange buffer (plain stores into peer memory that the host opened with the CUDA IPC calls);
//   2. a system-scope fence, then one thread per peer stores the call's sequence number into that peer's flag
//      [rank][cta];
//   3. one thread per peer polls this GPU's OWN flag [peer][cta] until it shows the sequence number (bounded: after
//      `spin_limit` polls it writes 1 to the status word and the kernel returns), a fence, and the kernel ends: the fold
//      kernel queued behind it on the stream reads the gathered partials from local memory.
//
// No kernel ever loads from a peer's memory, nothing is multicast, and the CTAs of one launch do not wait for each other.
// Two alternating slots make reuse safe without a second handshake: a rank writes slot s of call k + 2 only after it
// has seen every peer's flag of call k + 1, which a peer sets from a kernel that is stream-ordered behind its own fold of
// call k.  The ranks' kernels wait for one another, so each rank must run on a GPU of its own (one process per GPU).
//
// Buffer of one rank:  data[2][world][slot_bytes] | flags[2][world][kPeerMaxCtas] (64-bit sequence numbers)
#include <cstdint>
#include <cstring>

#include "common.cuh"

namespace cb200 {

constexpr int kPeerMaxCtas = 16;
constexpr int kPeerMaxWorld = 32;
constexpr size_t kPeerSliceBytes = 4096;           // per CTA at least this much, so small partials take one CTA

struct PeerBases { char* base[kPeerMaxWorld]; };

__device__ __forceinline__ size_t peer_flag_offset(size_t slot_bytes, int world, int slot, int rank, int cta) {
    return 2 * (size_t)world * slot_bytes + (((size_t)slot * world + rank) * kPeerMaxCtas + cta) * sizeof(unsigned long long);
}

__global__ void __launch_bounds__(kBlock)
peer_exchange_kernel(const char* __restrict__ src, size_t nbytes, const PeerBases peers, int world, int rank, size_t slot_bytes,
                     unsigned long long seq, unsigned spin_limit, int* status) {
    pdl_trigger();                      // the fold queued behind may become resident; it waits for this grid to finish
    pdl_wait();                         // this grid itself is launched as a dependent of the local reduction's last kernel
    const int slot = (int)(seq & 1ull);
    const size_t packets = (nbytes + 15) / 16;                                   // the source is padded to whole packets by the host
    const size_t per_cta = (packets + gridDim.x - 1) / gridDim.x;
    const size_t p_begin = (size_t)blockIdx.x * per_cta;
    size_t p_end = p_begin + per_cta; if (p_end > packets) p_end = packets;
    const size_t mine = p_end > p_begin ? p_end - p_begin : 0;
    // 1. my slice into everyone's slot [rank]
    const size_t dst_off = ((size_t)slot * world + rank) * slot_bytes;
    for (size_t i = threadIdx.x; i < mine * world; i += kBlock) {
        const int p = (int)(i / mine);
        const size_t k = p_begin + (i - (size_t)p * mine);
        const int4 v = *reinterpret_cast<const int4*>(src + k * 16);
        *reinterpret_cast<int4*>(peers.base[p] + dst_off + k * 16) = v;
    }
    __threadfence_system();
    __syncthreads();
    // 2. tell every peer, 3. wait for every peer
    if (threadIdx.x < world) {
        const int p = threadIdx.x;
        volatile unsigned long long* there = reinterpret_cast<volatile unsigned long long*>(peers.base[p] + peer_flag_offset(slot_bytes, world, slot, rank, blockIdx.x));
        *there = seq;
        volatile unsigned long long* here = reinterpret_cast<volatile unsigned long long*>(peers.base[rank] + peer_flag_offset(slot_bytes, world, slot, p, blockIdx.x));
        bool seen = false;
        for (unsigned spin = 0; spin < spin_limit; ++spin) {
            if (*here >= seq) { seen = true; break; }
            if (spin > 64) __nanosleep(200);
        }
        if (!seen) atomicExch(status, 1);
        __threadfence_system();
    }
    __syncthreads();
}

}  // namespace cb200

using namespace cb200;

extern "C" {

// Bytes of one rank's exchange buffer for `world` ranks and slots of `slot_bytes` (a multiple of 16).
size_t cb200_peer_buffer_bytes(size_t slot_bytes, int world) {
    return 2 * (size_t)world * slot_bytes + 2 * (size_t)world * kPeerMaxCtas * sizeof(unsigned long long);
}

// Allocates this rank's buffer on the current device (cleared) and exports it: `handle_out` receives the 64 bytes
// that another process on the same box passes to cb200_peer_buffer_open.  0 on success, else a cudaError_t.
int cb200_peer_buffer_create(size_t slot_bytes, int world, void** base_out, unsigned char* handle_out) {
    if (!base_out || !handle_out || world < 1 || world > kPeerMaxWorld || slot_bytes == 0 || slot_bytes % 16 != 0) return (int)cudaErrorInvalidValue;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, cb200_peer_buffer_bytes(slot_bytes, world));
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(p, 0, cb200_peer_buffer_bytes(slot_bytes, world));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); cudaGetLastError(); return (int)e; }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    memcpy(handle_out, &h, 64);
    *base_out = p;
    return 0;
}

// Maps another rank's buffer into this process (peer access is enabled on the way).
int cb200_peer_buffer_open(const unsigned char* handle, void** ptr_out) {
    if (!handle || !ptr_out) return (int)cudaErrorInvalidValue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    const cudaError_t e = cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) cudaGetLastError();
    return (int)e;
}
int cb200_peer_buffer_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
int cb200_peer_buffer_destroy(void* base) { return (int)cudaFree(base); }

// One exchange: `src` (nbytes <= slot_bytes, readable up to the next multiple of 16) goes to slot [rank] of every buffer
// in `bases` (host array of `world` device pointers, bases[rank] this rank's own); returns when queued.  The gathered
// partials of call `seq` are at bases[rank] + (seq & 1) * world * slot_bytes, `slot_bytes` apart, valid for kernels
// queued behind this one on the same stream.  `seq` counts the calls on these buffers from 1 and must be the same on
// every rank.  `status`: device-writable int that receives 1 when a wait ran out (the gathered data is then not valid).
// Returns 0, or a cudaError_t when the arguments are refused or the launch failed.
int cb200_peer_exchange_kernel_launch(const void* src, size_t nbytes, void* const* bases, int world, int rank, size_t slot_bytes,
                                      unsigned long long seq, unsigned spin_limit, int* status) {
    if (!src || !bases || !status || world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world || nbytes == 0 || nbytes > slot_bytes ||
        slot_bytes % 16 != 0 || seq == 0 || (reinterpret_cast<uintptr_t>(src) & 15) != 0)
        return (int)cudaErrorInvalidValue;
    PeerBases pb;
    for (int p = 0; p < kPeerMaxWorld; ++p) pb.base[p] = p < world ? static_cast<char*>(bases[p]) : nullptr;
    size_t ctas = (nbytes + kPeerSliceBytes - 1) / kPeerSliceBytes;
    if (ctas > (size_t)kPeerMaxCtas) ctas = kPeerMaxCtas;
    launch_dependent(peer_exchange_kernel, (unsigned)ctas, kBlock, current_stream(), static_cast<const char*>(src), nbytes, pb, world, rank, slot_bytes, seq,
                     spin_limit ? spin_limit : (1u << 25), status);
    count_launch();
    return (int)cudaGetLastError();
}

}  // extern "C"
