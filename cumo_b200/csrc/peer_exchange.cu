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

#include "reducers.cuh"

namespace cb200 {

constexpr int kPeerMaxCtas = 16;
constexpr int kPeerMaxWorld = 32;
constexpr size_t kPeerSliceBytes = 4096;           // per CTA at least this much, so small partials take one CTA

struct PeerBases { char* base[kPeerMaxWorld]; };

__device__ __forceinline__ size_t peer_flag_offset(size_t slot_bytes, int world, int slot, int rank, int cta) {
    return 2 * (size_t)world * slot_bytes + (((size_t)slot * world + rank) * kPeerMaxCtas + cta) * sizeof(unsigned long long);
}

// Steps 1-3 for this CTA's slice [p_begin, p_end) of 16-byte packets; false when a wait ran out.
__device__ __forceinline__ bool exchange_slice(const char* __restrict__ src, size_t p_begin, size_t p_end, const PeerBases& peers, int world, int rank,
                                               size_t slot_bytes, unsigned long long seq, unsigned spin_limit, int* status) {
    __shared__ int gave_up;
    const int slot = (int)(seq & 1ull);
    const size_t mine = p_end > p_begin ? p_end - p_begin : 0;
    if (threadIdx.x == 0) gave_up = 0;
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
        if (!seen) { atomicExch(status, 1); gave_up = 1; }
        __threadfence_system();
    }
    __syncthreads();
    return gave_up == 0;
}

// Steps 2 and 3 alone (the data of this CTA's slice has been stored and fenced): raise my flag at every peer, wait for theirs.
__device__ __forceinline__ bool signal_and_wait(const PeerBases& peers, int world, int rank, size_t slot_bytes, unsigned long long seq,
                                                unsigned spin_limit, int* status) {
    __shared__ int gave_up2;
    const int slot = (int)(seq & 1ull);
    if (threadIdx.x == 0) gave_up2 = 0;
    __threadfence_system();
    __syncthreads();
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
        if (!seen) { atomicExch(status, 1); gave_up2 = 1; }
        __threadfence_system();
    }
    __syncthreads();
    return gave_up2 == 0;
}

__device__ __forceinline__ void slice_of(size_t nbytes, size_t& p_begin, size_t& p_end) {
    const size_t packets = (nbytes + 15) / 16;                                   // the source is padded to whole packets by the host
    const size_t per_cta = (packets + gridDim.x - 1) / gridDim.x;
    p_begin = (size_t)blockIdx.x * per_cta;
    p_end = p_begin + per_cta;
    if (p_end > packets) p_end = packets;
}

__global__ void __launch_bounds__(kBlock)
peer_exchange_kernel(const char* __restrict__ src, size_t nbytes, const PeerBases peers, int world, int rank, size_t slot_bytes,
                     unsigned long long seq, unsigned spin_limit, int* status) {
    pdl_trigger();                      // the fold queued behind may become resident; it waits for this grid to finish
    pdl_wait();                         // this grid itself is launched as a dependent of the local reduction's last kernel
    size_t p_begin, p_end;
    slice_of(nbytes, p_begin, p_end);
    exchange_slice(src, p_begin, p_end, peers, world, rank, slot_bytes, seq, spin_limit, status);
}

// The exchange and the rank fold in one kernel, for folds that work element by element (sums, min, max): a CTA folds the
// slice it exchanged as soon as its own peers' flags are up -- one launch and one launch gap less per reduction.
// MODE 0: sum in float64 in rank order, divided by `divisor` unless 0, rounded once.  MODE 1: min / max with the
// single-GPU functor's NaN rules.
template <typename T, int MODE, bool IS_MAX, bool NAN_WINS>
__global__ void __launch_bounds__(kBlock)
peer_exchange_fold_kernel(const char* __restrict__ src, size_t nbytes, const PeerBases peers, int world, int rank, size_t slot_bytes,
                          unsigned long long seq, unsigned spin_limit, int* status, int64_t n_out, double divisor, T* out) {
    pdl_trigger();
    pdl_wait();
    size_t p_begin, p_end;
    slice_of(nbytes, p_begin, p_end);
    if (!exchange_slice(src, p_begin, p_end, peers, world, rank, slot_bytes, seq, spin_limit, status)) return;
    constexpr int V = 16 / (int)sizeof(T);
    const char* mine = peers.base[rank] + (size_t)(seq & 1ull) * world * slot_bytes;
    const int64_t o_begin = (int64_t)p_begin * V;
    int64_t o_end = (int64_t)p_end * V;
    if (o_end > n_out) o_end = n_out;
    using R = red::MinMax<T, IS_MAX, NAN_WINS>;
    const R r{};
    for (int64_t o = o_begin + threadIdx.x; o < o_end; o += kBlock) {
        if (MODE == 0) {
            double acc = 0.0;
            for (int k = 0; k < world; ++k) acc += (double)__ldcg(reinterpret_cast<const T*>(mine + (size_t)k * slot_bytes) + o);
            if (divisor != 0.0) acc /= divisor;
            out[o] = (T)acc;
        } else {
            T acc = __ldcg(reinterpret_cast<const T*>(mine) + o);
            for (int k = 1; k < world; ++k) acc = r.combine(acc, __ldcg(reinterpret_cast<const T*>(mine + (size_t)k * slot_bytes) + o));
            out[o] = acc;
        }
    }
}

// Index reductions: a rank's partial is {int64 global index, value} per output, indices first, the values starting
// `val_off` bytes into the buffer (a multiple of 16).  A CTA takes a run of outputs, stores their indices and their values
// into every rank's slot, and once its peers' flags are up merges the `world` candidates of each of those outputs with the
// single-GPU functor's total order (NaN rule, better value, lower index).
template <typename T, bool IS_MAX, bool NAN_WINS>
__global__ void __launch_bounds__(kBlock)
peer_exchange_arg_kernel(const char* __restrict__ src, int64_t n_out, size_t val_off, const PeerBases peers, int world, int rank, size_t slot_bytes,
                         unsigned long long seq, unsigned spin_limit, int* status, int64_t* out_index) {
    pdl_trigger();
    pdl_wait();
    constexpr int64_t G = 16 / (int64_t)sizeof(T);                 // outputs per 16 bytes of values (and per 16 * 8 / sizeof(T) bytes of indices)
    int64_t per_cta = (n_out + gridDim.x - 1) / gridDim.x;
    per_cta = (per_cta + G - 1) / G * G;
    const int64_t o_begin = (int64_t)blockIdx.x * per_cta;
    int64_t o_end = o_begin + per_cta;
    const int64_t padded = (n_out + G - 1) / G * G;                 // the host pads both parts of the buffer to whole packets
    if (o_end > padded) o_end = padded;
    const int64_t mine = o_end > o_begin ? o_end - o_begin : 0;
    const int slot = (int)(seq & 1ull);
    const size_t dst_off = ((size_t)slot * world + rank) * slot_bytes;
    const int64_t idx_packets = mine * 8 / 16, val_packets = mine * (int64_t)sizeof(T) / 16;
    const int64_t per_peer = idx_packets + val_packets;
    for (int64_t i = threadIdx.x; i < per_peer * world; i += kBlock) {
        const int p = (int)(i / per_peer);
        const int64_t k = i - (int64_t)p * per_peer;
        const size_t off = k < idx_packets ? (size_t)o_begin * 8 + (size_t)k * 16 : val_off + (size_t)o_begin * sizeof(T) + (size_t)(k - idx_packets) * 16;
        const int4 v = *reinterpret_cast<const int4*>(src + off);
        *reinterpret_cast<int4*>(peers.base[p] + dst_off + off) = v;
    }
    if (!signal_and_wait(peers, world, rank, slot_bytes, seq, spin_limit, status)) return;
    using R = red::ArgMinMax<T, IS_MAX, NAN_WINS>;
    const R r{1};
    const char* base = peers.base[rank] + (size_t)slot * world * slot_bytes;
    const int64_t stop = o_end < n_out ? o_end : n_out;
    for (int64_t o = o_begin + threadIdx.x; o < stop; o += kBlock) {
        typename R::Acc acc = r.identity();
        for (int k = 0; k < world; ++k) {
            typename R::Acc b;
            b.index = __ldcg(reinterpret_cast<const long long*>(base + (size_t)k * slot_bytes) + o);
            b.value = __ldcg(reinterpret_cast<const T*>(base + (size_t)k * slot_bytes + val_off) + o);
            acc = r.combine(acc, b);
        }
        out_index[o] = acc.index;
    }
}

template <typename T>
static void launch_exchange_arg(const char* s, int64_t n_out, size_t val_off, const PeerBases& pb, int world, int rank, size_t slot_bytes,
                                unsigned long long seq, unsigned limit, int* status, int is_max, int nan_wins, int64_t* out, unsigned ctas, cudaStream_t st) {
    constexpr bool fp = red::is_fp<T>::value;
    auto go = [&](auto kernel) { launch_dependent(kernel, ctas, kBlock, st, s, n_out, val_off, pb, world, rank, slot_bytes, seq, limit, status, out); };
    if (is_max) {
        if (nan_wins && fp) go(peer_exchange_arg_kernel<T, true, fp>); else go(peer_exchange_arg_kernel<T, true, false>);
    } else {
        if (nan_wins && fp) go(peer_exchange_arg_kernel<T, false, fp>); else go(peer_exchange_arg_kernel<T, false, false>);
    }
}

template <typename T>
static void launch_exchange_fold(const char* s, size_t nbytes, const PeerBases& pb, int world, int rank, size_t slot_bytes, unsigned long long seq,
                                 unsigned limit, int* status, int64_t n_out, double divisor, int op, int nan_wins, void* out, unsigned ctas,
                                 cudaStream_t st) {
    T* o = static_cast<T*>(out);
    constexpr bool fp = red::is_fp<T>::value;
    auto go = [&](auto kernel) { launch_dependent(kernel, ctas, kBlock, st, s, nbytes, pb, world, rank, slot_bytes, seq, limit, status, n_out, divisor, o); };
    if (op == 0) {
        if constexpr (fp) go(peer_exchange_fold_kernel<T, 0, false, false>);
    } else if (op == 2) {
        if (nan_wins && fp) go(peer_exchange_fold_kernel<T, 1, true, fp>); else go(peer_exchange_fold_kernel<T, 1, true, false>);
    } else {
        if (nan_wins && fp) go(peer_exchange_fold_kernel<T, 1, false, fp>); else go(peer_exchange_fold_kernel<T, 1, false, false>);
    }
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

// The same exchange with the rank fold done by the same kernel: `op` 0 = sum (float types; `divisor` as in
// cb200_<T>_rank_fold_sum_kernel_launch), 1 = min, 2 = max (`nan_wins` as in the extreme fold); `dtype` 0 sfloat, 1 dfloat,
// 2 int32, 3 int64 (min / max only for the integer types); `src` holds n_out elements, `out` receives n_out.
int cb200_peer_exchange_fold_kernel_launch(const void* src, int dtype, int op, int64_t n_out, double divisor, int nan_wins, void* out,
                                           void* const* bases, int world, int rank, size_t slot_bytes, unsigned long long seq,
                                           unsigned spin_limit, int* status) {
    static const size_t es_of[4] = {4, 8, 4, 8};
    if (dtype < 0 || dtype > 3 || op < 0 || op > 2 || n_out <= 0 || !out || (op == 0 && dtype > 1)) return (int)cudaErrorInvalidValue;
    const size_t nbytes = (size_t)n_out * es_of[dtype];
    if (!src || !bases || !status || world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world || nbytes > slot_bytes ||
        slot_bytes % 16 != 0 || seq == 0 || (reinterpret_cast<uintptr_t>(src) & 15) != 0)
        return (int)cudaErrorInvalidValue;
    PeerBases pb;
    for (int p = 0; p < kPeerMaxWorld; ++p) pb.base[p] = p < world ? static_cast<char*>(bases[p]) : nullptr;
    size_t ctas = (nbytes + kPeerSliceBytes - 1) / kPeerSliceBytes;
    if (ctas > (size_t)kPeerMaxCtas) ctas = kPeerMaxCtas;
    const unsigned limit = spin_limit ? spin_limit : (1u << 25);
    const char* s = static_cast<const char*>(src);
    cudaStream_t st = current_stream();
    switch (dtype) {
    case 0: launch_exchange_fold<float>(s, nbytes, pb, world, rank, slot_bytes, seq, limit, status, n_out, divisor, op, nan_wins, out, (unsigned)ctas, st); break;
    case 1: launch_exchange_fold<double>(s, nbytes, pb, world, rank, slot_bytes, seq, limit, status, n_out, divisor, op, nan_wins, out, (unsigned)ctas, st); break;
    case 2: launch_exchange_fold<int32_t>(s, nbytes, pb, world, rank, slot_bytes, seq, limit, status, n_out, divisor, op, nan_wins, out, (unsigned)ctas, st); break;
    default: launch_exchange_fold<int64_t>(s, nbytes, pb, world, rank, slot_bytes, seq, limit, status, n_out, divisor, op, nan_wins, out, (unsigned)ctas, st); break;
    }
    count_launch();
    return (int)cudaGetLastError();
}

// The exchange and the merge of an index reduction's partials in one kernel.  `src`: this rank's buffer, n_out int64 global
// indices followed, `val_off` bytes in (a multiple of 16, >= 8 * n_out), by the n_out winning values of type `dtype`; both parts
// readable up to the next multiple of 16 bytes.  `out_index` receives the n_out merged indices.
int cb200_peer_exchange_arg_kernel_launch(const void* src, int dtype, int64_t n_out, size_t val_off, int is_max, int nan_wins, int64_t* out_index,
                                          void* const* bases, int world, int rank, size_t slot_bytes, unsigned long long seq,
                                          unsigned spin_limit, int* status) {
    static const size_t es_of[4] = {4, 8, 4, 8};
    if (dtype < 0 || dtype > 3 || n_out <= 0 || !out_index || val_off % 16 != 0 || val_off < (size_t)n_out * 8) return (int)cudaErrorInvalidValue;
    const size_t es = es_of[dtype];
    const size_t nbytes = val_off + ((size_t)n_out * es + 15) / 16 * 16;
    if (!src || !bases || !status || world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world || nbytes > slot_bytes ||
        slot_bytes % 16 != 0 || seq == 0 || (reinterpret_cast<uintptr_t>(src) & 15) != 0)
        return (int)cudaErrorInvalidValue;
    PeerBases pb;
    for (int p = 0; p < kPeerMaxWorld; ++p) pb.base[p] = p < world ? static_cast<char*>(bases[p]) : nullptr;
    size_t ctas = (nbytes + kPeerSliceBytes - 1) / kPeerSliceBytes;
    if (ctas > (size_t)kPeerMaxCtas) ctas = kPeerMaxCtas;
    const unsigned limit = spin_limit ? spin_limit : (1u << 25);
    const char* s = static_cast<const char*>(src);
    cudaStream_t st = current_stream();
    switch (dtype) {
    case 0: launch_exchange_arg<float>(s, n_out, val_off, pb, world, rank, slot_bytes, seq, limit, status, is_max, nan_wins, out_index, (unsigned)ctas, st); break;
    case 1: launch_exchange_arg<double>(s, n_out, val_off, pb, world, rank, slot_bytes, seq, limit, status, is_max, nan_wins, out_index, (unsigned)ctas, st); break;
    case 2: launch_exchange_arg<int32_t>(s, n_out, val_off, pb, world, rank, slot_bytes, seq, limit, status, is_max, nan_wins, out_index, (unsigned)ctas, st); break;
    default: launch_exchange_arg<int64_t>(s, n_out, val_off, pb, world, rank, slot_bytes, seq, limit, status, is_max, nan_wins, out_index, (unsigned)ctas, st); break;
    }
    count_launch();
    return (int)cudaGetLastError();
}

}  // extern "C"
