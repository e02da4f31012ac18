// TILE kernel fed by the tensor memory accelerator (sm_100a): operands whose contiguous axes differ.
//
// Same plane as the tile kernels of elementwise.cuh -- out[r][c] = op(x[r][c], y[r][c]), the output contiguous along c,
// at least one input contiguous along r -- but every input tile is brought into shared memory by one elected thread
// with `cp.async.bulk.tensor` (this GPU's memory only, a plain one-CTA copy) through a ring of stages guarded by
// mbarriers, several tiles ahead of the warps that consume them.  The loads therefore cost neither registers nor
// issue slots, and the bytes in flight per SM no longer depend on the occupancy of the consumer warps, which is
// what bounded the register-staged form (46 % of the warp slots, stalls on the loads and on the CTA barrier).
//
// Shared-memory layout of one input tile (kTmaTileC = 64 elements of c by TR = 256 / sizeof(T) elements of r, 16 KiB):
//   transposed input (contiguous along r): boxes of [V][64 / V][128 bytes of r], V = elements per 16 bytes, in the
//     128-byte swizzle.  The tensor map splits c into (c / V, c % V) and puts c % V outermost, so that the row of
//     shared memory that holds column c is (c % V) * (64 / V) + c / V: the threads of a quarter warp, which take
//     neighbouring packets of c, read rows whose low three bits differ, and the swizzle sends their 16-byte reads to
//     different banks.  A thread reads V packets (V consecutive columns, the same V rows), transposes the V x V block
//     in registers and stores V packets of the output.
//   row-like input (contiguous along c): one box [TR][64 elements], no swizzle; read with the same lane map.
// Out-of-range parts of edge tiles are filled with zeros by the copy engine and never used.
//
// Every wait is bounded: a role that gives up raises the CTA's abort flag, the others leave at their next poll, the
// kernel writes 1 into the library's status word (cb200_tile_pipeline_status) and returns.
#pragma once

#include <cuda.h>          // CUtensorMap and its enums; the encoder itself is looked up through the runtime

#include "ops.cuh"
#include "tc_common.cuh"

namespace cb200 {

// The plane of a tile kernel (the register-staged forms live in elementwise.cuh) and the dims around it.
struct TilePlan {
    int n_outer;                              // dims besides the plane
    int64_t oshape[kMaxDim];
    int64_t ostep[3][kMaxDim];                // [0],[1] inputs, [2] output
    int64_t R, C;                             // extents of the plane: r = the transposed inputs' contiguous axis, c = the output's
    int64_t rstep[3], cstep[3];               // byte steps along r and c per operand
    int64_t tiles_r, tiles_c, n_tiles;
};

constexpr int kTmaConsumers = kBlock;                   // 8 warps that compute and store
constexpr int kTmaThreads = kTmaConsumers + 32;         // + the warp whose first lane issues the copies
constexpr int kTmaMaxStages = 6;

// defined in tile_tma.cu
using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encoder();                 // null when the driver has none
int* tile_status_word();                                // device address on the current device, null on failure
int tile_tma_stages(int n_inputs);                      // ring depth (environment override for measurements)
int tile_tma_mode();                                    // 0 never, 1 always, 2 where it measured faster
bool tile_tma_raise_smem_limit(const void* kernel);     // once per (kernel, device)
void note_tile_tma_launch();                            // counts launches (cb200_tile_pipeline_launches)

struct TmaTileArgs {
    int64_t R, C;
    int64_t tiles_r, tiles_c, n_tiles;
    int64_t out_rstep;                                  // bytes
    int n_outer;
    int64_t oshape[2];
    int64_t out_ostep[2];
    int bmul[2][2];                                     // [input][outer dim]: 0 when the input repeats along that dim
    int stages;
    int have;                                           // bit 0: input 1 is an array, bit 1: input 2
};

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// one box of a 5-d tensor map of this GPU's memory into this CTA's shared memory; completion is counted on `bar`
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x0, int x1, int x2, int x3, int x4) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                 ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x0), "r"(x1), "r"(x2), "r"(x3), "r"(x4) : "memory");
}

// Tile number -> (batch, tile row, tile column), columns fastest.  The host keeps every count below 2^31: 32-bit splits.
// (Numbering the tiles in strips, so that those in flight cover a compact block of source and output, changed nothing.)
__device__ __forceinline__ void tile_coords(const TmaTileArgs& t, uint32_t tile, uint32_t& batch, uint32_t& tr, uint32_t& tc) {
    const uint32_t rest = tile / (uint32_t)t.tiles_c;
    tc = tile - rest * (uint32_t)t.tiles_c;
    batch = rest / (uint32_t)t.tiles_r;
    tr = rest - batch * (uint32_t)t.tiles_r;
}

template <typename Op, bool T1, bool T2, int TC, int TR>
__global__ void __launch_bounds__(kTmaThreads)
ew_tile_tma_kernel(const TmaTileArgs t, const __grid_constant__ CUtensorMap map1, const __grid_constant__ CUtensorMap map2, char* a3,
                   typename Op::In1 sx, typename Op::In2 sy, int* flag, int* status_word) {
    using X = typename Op::In1;
    using Y = typename Op::In2;
    using TO = typename Op::Out;
    static_assert(sizeof(X) == sizeof(TO) && sizeof(Y) == sizeof(TO), "one element size");
    constexpr int ES = sizeof(TO);
    constexpr int V = 16 / ES;
    constexpr uint32_t kSlot = TC * TR * ES;               // one input tile
    constexpr int NPC = TC / V;                            // packets along c
    constexpr int NQ = TR / V;                             // 16-byte chunks along r
    constexpr int NBOX = NQ / 8;                           // 128-byte boxes along r of a transposed input
    constexpr int BOX_R = 128 / ES;
    static_assert(NPC % 8 == 0 && NQ % 8 == 0, "lane map");

    extern __shared__ __align__(1024) char smem_raw[];
    const bool have1 = t.have & 1, have2 = (t.have & 2) && Op::arity == 2;
    const int n_in = (have1 ? 1 : 0) + (have2 ? 1 : 0);
    const uint32_t stage_bytes = (uint32_t)n_in * kSlot;
    const uint32_t slot2 = have1 ? kSlot : 0;      // where input 2 sits inside a stage
    if ((smem_u32(smem_raw) & 1023u) != 0) {               // the swizzle pattern is a function of the address: uniform exit before any barrier
        if (threadIdx.x == 0) atomicExch(status_word, 2);
        return;
    }
    const int S = t.stages;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)S * stage_bytes);
    uint64_t* empty = full + kTmaMaxStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kTmaMaxStages);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kTmaConsumers / 32); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kTmaConsumers / 32) {
        // ---- the copy role ----
        if (lane == 0) {
            uint32_t it = 0;
            for (int64_t tile = blockIdx.x; tile < t.n_tiles; tile += gridDim.x, ++it) {
                const uint32_t s = it % (uint32_t)S, k = it / (uint32_t)S;
                if (k > 0 && !mbar_wait(&empty[s], (k - 1) & 1, abort_flag)) break;
                uint32_t batch, tr, tc;
                tile_coords(t, (uint32_t)tile, batch, tr, tc);
                int b0 = 0, b1 = 0;
                if (t.n_outer == 1) b0 = (int)batch;
                else if (t.n_outer == 2) { b0 = (int)(batch / (uint32_t)t.oshape[1]); b1 = (int)(batch - (uint32_t)b0 * (uint32_t)t.oshape[1]); }
                const int r0 = (int)(tr * TR), c0 = (int)(tc * TC);
                const uint32_t base = smem_u32(smem_raw) + s * stage_bytes;
                mbar_expect_tx(&full[s], stage_bytes);
                if (have1) {
                    if (T1) {
#pragma unroll
                        for (int h = 0; h < NBOX; ++h)
                            tma_load_5d(base + h * (128 * TC), &map1, &full[s], r0 + h * BOX_R, c0 / V, 0, b0 * t.bmul[0][0], b1 * t.bmul[0][1]);
                    } else {
                        tma_load_5d(base, &map1, &full[s], c0, r0, b0 * t.bmul[0][0], b1 * t.bmul[0][1], 0);
                    }
                }
                if (have2) {
                    if (T2) {
#pragma unroll
                        for (int h = 0; h < NBOX; ++h)
                            tma_load_5d(base + slot2 + h * (128 * TC), &map2, &full[s], r0 + h * BOX_R, c0 / V, 0, b0 * t.bmul[1][0], b1 * t.bmul[1][1]);
                    } else {
                        tma_load_5d(base + slot2, &map2, &full[s], c0, r0, b0 * t.bmul[1][0], b1 * t.bmul[1][1], 0);
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ---- the compute-and-store role ----
        uint32_t it = 0;
        for (int64_t tile = blockIdx.x; tile < t.n_tiles; tile += gridDim.x, ++it) {
            const uint32_t s = it % (uint32_t)S, k = it / (uint32_t)S;
            uint32_t batch, tr, tc;
            tile_coords(t, (uint32_t)tile, batch, tr, tc);
            int64_t out_off = 0;
            if (t.n_outer == 1) out_off = (int64_t)batch * t.out_ostep[0];
            else if (t.n_outer == 2) {
                const uint32_t i0 = batch / (uint32_t)t.oshape[1], i1 = batch - i0 * (uint32_t)t.oshape[1];
                out_off = (int64_t)i0 * t.out_ostep[0] + (int64_t)i1 * t.out_ostep[1];
            }
            const int64_t r0 = (int64_t)tr * TR, c0 = (int64_t)tc * TC;
            if (!mbar_wait(&full[s], k & 1, abort_flag)) break;
            const char* st1 = smem_raw + (size_t)s * stage_bytes;
            const char* st2 = st1 + slot2;
#pragma unroll
            for (int b = tid; b < NPC * NQ; b += kTmaConsumers) {
                const int pc = b % NPC, Q = b / NPC;
                const bool ok = c0 + pc * V < t.C && r0 + Q * V < t.R;     // extents are whole packets: a V x V block is in or out
                Pack<X> x[V];
                Pack<Y> y[V];
#pragma unroll
                for (int i = 0; i < V; ++i) {
#pragma unroll
                    for (int e = 0; e < V; ++e) { x[i].v[e] = sx; y[i].v[e] = sy; }
                }
                if (ok) {
                    // transposed: packet e is column c = pc * V + e, rows Q * V .. Q * V + V - 1
                    const uint32_t t_off = (uint32_t)(Q / 8) * (128 * TC) + (uint32_t)pc * 128u + ((uint32_t)((Q & 7) ^ (pc & 7)) << 4);
                    // row-like: packet i is row Q * V + i, columns pc * V .. pc * V + V - 1
                    const uint32_t r_off = (uint32_t)(Q * V) * (TC * ES) + (uint32_t)pc * 16u;
                    if (have1) {
                        if (T1) {
#pragma unroll
                            for (int e = 0; e < V; ++e) {
                                const Pack<X> p = *reinterpret_cast<const Pack<X>*>(st1 + t_off + e * (NPC * 128));
#pragma unroll
                                for (int i = 0; i < V; ++i) x[i].v[e] = p.v[i];
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < V; ++i) x[i] = *reinterpret_cast<const Pack<X>*>(st1 + r_off + i * (TC * ES));
                        }
                    }
                    if (have2) {
                        if (T2) {
#pragma unroll
                            for (int e = 0; e < V; ++e) {
                                const Pack<Y> p = *reinterpret_cast<const Pack<Y>*>(st2 + t_off + e * (NPC * 128));
#pragma unroll
                                for (int i = 0; i < V; ++i) y[i].v[e] = p.v[i];
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < V; ++i) y[i] = *reinterpret_cast<const Pack<Y>*>(st2 + r_off + i * (TC * ES));
                        }
                    }
                    char* w = a3 + out_off + (r0 + Q * V) * t.out_rstep + (c0 + pc * V) * ES;
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        Pack<TO> z;
                        unsigned keep = 0;
#pragma unroll
                        for (int e = 0; e < V; ++e) {
                            TO zv = TO();
                            if (ew_apply<Op>(x[i].v[e], y[i].v[e], sx, zv, flag)) keep |= 1u << e;
                            z.v[e] = zv;
                        }
                        char* q = w + i * t.out_rstep;
                        if (keep == (1u << V) - 1u) st_pack<TO>(q, z);
                        else {
#pragma unroll
                            for (int e = 0; e < V; ++e)
                                if (keep & (1u << e)) st_one<TO>(q + e * ES, z.v[e]);
                        }
                    }
                }
            }
            // the stores above took their operands from the stage: every read of it by this warp has completed
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
    }
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicExch(status_word, 1);
}

// One tensor map per input over the plane (and up to two batch dims).  False when the driver refuses the geometry.
inline bool encode_tile_map(CUtensorMap* m, const char* base, int es, int TC, int TR, bool transposed, int64_t R, int64_t C, int64_t rstep, int64_t cstep,
                            int n_outer, const int64_t* oshape, const int64_t* ostep, int* bmul) {
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return false;
    const int V = 16 / es;
    cuuint64_t dim[5] = {1, 1, 1, 1, 1};
    cuuint64_t stride[4] = {16, 16, 16, 16};           // bytes, of dims 1..4
    cuuint32_t box[5] = {1, 1, 1, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    int nb;
    if (transposed) {
        dim[0] = (cuuint64_t)R;                  box[0] = 128 / es;
        dim[1] = (cuuint64_t)(C / V);            box[1] = TC / V;   stride[0] = (cuuint64_t)(cstep * V);
        dim[2] = (cuuint64_t)V;                  box[2] = V;               stride[1] = (cuuint64_t)cstep;
        nb = 3;
    } else {
        dim[0] = (cuuint64_t)C;                  box[0] = TC;
        dim[1] = (cuuint64_t)R;                  box[1] = TR;              stride[0] = (cuuint64_t)rstep;
        nb = 2;
    }
    cuuint64_t last = stride[nb - 2];
    for (int d = 0; d < 2; ++d) {
        bmul[d] = 0;
        if (d < n_outer && ostep[d] != 0) {
            dim[nb + d] = (cuuint64_t)oshape[d];
            stride[nb + d - 1] = (cuuint64_t)ostep[d];
            last = stride[nb + d - 1];
            bmul[d] = 1;
        } else {
            stride[nb + d - 1] = last;                  // an extent of 1: the step is never applied
        }
    }
    if (!transposed) stride[3] = last;
    for (int d = 0; d < 4; ++d) if (stride[d] % 16 != 0 || stride[d] >= (1ULL << 40) || stride[d] == 0) return false;
    for (int d = 0; d < 5; ++d) if (dim[d] == 0 || dim[d] > (1ULL << 32)) return false;
    const CUresult rc = enc(m, es == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT64, 5, const_cast<char*>(base), dim, stride,
                            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, transposed ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

// Launches the copy-engine form of the tile plan when every array input can be described to it; false otherwise (the
// register-staged tile kernels take the plan).
template <typename Op, int TC, int TR>
bool launch_tiled_tma_shape(const TilePlan& p, const bool* tr, const char* p1, const char* p2, char* p3, bool have1, bool have2,
                            typename Op::In1 sx, typename Op::In2 sy, int* flag, cudaStream_t st) {
    constexpr int ES = sizeof(typename Op::Out);
    constexpr int V = 16 / ES;
    constexpr size_t kSlot = (size_t)TC * TR * ES;
    if (p.n_outer > 2) return false;
    if (p.R % V != 0 || p.C % V != 0 || p.R >= (1LL << 31) || p.C >= (1LL << 31)) return false;
    if (!aligned16(p3) || !mult16(p.rstep[2]) || p.cstep[2] != ES) return false;
    const bool have[2] = {have1, have2 && Op::arity == 2};
    const char* bases[2] = {p1, p2};
    TmaTileArgs t;
    CUtensorMap maps[2];
    memset(maps, 0, sizeof maps);
    t.R = p.R; t.C = p.C;
    t.n_outer = p.n_outer;
    int64_t batch = 1;
    for (int d = 0; d < 2; ++d) {
        t.oshape[d] = d < p.n_outer ? p.oshape[d] : 1;
        t.out_ostep[d] = d < p.n_outer ? p.ostep[2][d] : 0;
        if (t.oshape[d] >= (1LL << 31)) return false;
        batch *= t.oshape[d];
        t.bmul[0][d] = t.bmul[1][d] = 0;
    }
    int n_in = 0;
    for (int a = 0; a < 2; ++a) {
        if (!have[a]) continue;
        ++n_in;
        if (!aligned16(bases[a])) return false;
        if (tr[a]) { if (p.rstep[a] != ES || p.cstep[a] <= 0) return false; }
        else if (p.cstep[a] != ES || p.rstep[a] <= 0) return false;            // repeated rows or columns: not a dense box
        int64_t os[2] = {0, 0};
        for (int d = 0; d < p.n_outer; ++d) { os[d] = p.ostep[a][d]; if (os[d] < 0) return false; }
        if (!encode_tile_map(&maps[a], bases[a], ES, TC, TR, tr[a], p.R, p.C, p.rstep[a], p.cstep[a], p.n_outer, t.oshape, os, t.bmul[a])) return false;
    }
    if (n_in == 0) return false;
    int* status = tile_status_word();
    if (!status) return false;
    t.tiles_r = (p.R + TR - 1) / TR;
    t.tiles_c = (p.C + TC - 1) / TC;
    t.n_tiles = t.tiles_r * t.tiles_c * batch;
    if (t.n_tiles >= (1LL << 31)) return false;
    t.out_rstep = p.rstep[2];
    t.stages = tile_tma_stages(n_in);
    while (t.stages > 2 && (size_t)t.stages * n_in * kSlot > 190u * 1024u) --t.stages;
    if ((size_t)t.stages * n_in * kSlot > 190u * 1024u) return false;
    t.have = (have[0] ? 1 : 0) | (have[1] ? 2 : 0);
    const size_t smem = (size_t)t.stages * n_in * kSlot + 2 * kTmaMaxStages * sizeof(uint64_t) + 16;
    const int per_sm = (int)((220u * 1024u) / (smem + 1024));
    const unsigned grid = grid_for(t.n_tiles, per_sm < 1 ? 1 : (per_sm > 6 ? 6 : per_sm));
    auto go = [&](auto kernel) {
        if (!tile_tma_raise_smem_limit(reinterpret_cast<const void*>(kernel))) return false;
        kernel<<<grid, kTmaThreads, smem, st>>>(t, maps[0], maps[1], p3, sx, sy, flag, status);
        note_tile_tma_launch();
        return true;
    };
    if constexpr (Op::arity == 1) {
        return go(ew_tile_tma_kernel<Op, true, false, TC, TR>);
    } else {
        if (tr[0] && tr[1]) return go(ew_tile_tma_kernel<Op, true, true, TC, TR>);
        if (tr[0]) return go(ew_tile_tma_kernel<Op, true, false, TC, TR>);
        return go(ew_tile_tma_kernel<Op, false, true, TC, TR>);
    }
}

template <typename Op>
bool launch_tiled_tma(const TilePlan& p, const bool* tr, const char* p1, const char* p2, char* p3, bool have1, bool have2,
                      typename Op::In1 sx, typename Op::In2 sy, int* flag, cudaStream_t st) {
    constexpr int ES = sizeof(typename Op::Out);
    const int mode = tile_tma_mode();
    if (mode == 0) return false;
    if (mode == 2 && ES == 4) {
        // Measured on B200 (16384^2 and 4096^2 planes): with 8-byte elements this form is never slower and 1.5x faster for
        // a binary operation; with 4-byte elements it wins up to a few hundred MiB (5.7 against 4.9 TB/s for a 64 MiB
        // transposed copy) and the register-staged form is 3 to 6 % ahead beyond.
        int64_t batch = 1;
        for (int d = 0; d < p.n_outer; ++d) batch *= p.oshape[d];
        if (p.R * p.C * batch * ES > (256LL << 20)) return false;
    }
    return launch_tiled_tma_shape<Op, 64, 256 / ES>(p, tr, p1, p2, p3, have1, have2, sx, sy, flag, st);
}

}  // namespace cb200
