// K2: dequant-fused GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), many activation rows.
//
//   y[t, r] = sum_k x[t, k] * dequant(W)[r, k]          f16 operands, fp32 accumulation in TMEM
//
// Stands in for mlx-native's kernel_mul_mm_<q>_f32 / hf2q_mul_mm_tensor_v2 that hf2q reaches
// through quantized_matmul_ggml with m > 8 (MM_ROUTING_THRESHOLD; src/serve/forward_mlx.rs:9800,
// src/inference/models/qwen35/gpu_ffn.rs:1457-1538, src/serve/forward_prefill_batched.rs:1114-1122).
// The reference's kernel dequantises the weight tile to half and keeps activations as float
// (docs/ADR-011-phase3-wave-p3a-mm-qmatmul-verification.md:66-69); here both operands are f16
// (a bf16 weight tile would miss the 1e-3 accuracy gate, f16 measures ~2e-4).
//
// One CTA computes a tile of 128 weight rows x NT activation rows (tokens):
//
//   warp 8 (one lane)   TMA producer.  Per 256-element K-block: one 2-D tensor copy of the RAW block
//                       bytes of 128 weight rows (box 128 x <=272 B, no swizzle) and four 2-D copies
//                       of the f16 activations (box NT x 64 elements, 128-byte swizzle) into
//                       shared-memory rings; completion on mbarriers.
//   warps 0-7           dequantisers, two per weight row (one per half K-block).  A thread reads its row's raw bytes from
//                       shared memory (16-byte vectors, conflict-free pitch), unpacks 256 codes,
//                       applies d*scale (and -dmin*min) in f16x2 and writes the A operand straight
//                       into TENSOR MEMORY with tcgen05.st (row = TMEM lane), double-buffered.
//                       No cross-lane traffic, no shared-memory round trip for the dequantised tile.
//   warp 9 (one lane)   MMA issuer.  tcgen05.mma.kind::f16, M = 128, N = NT, K = 16, A from TMEM,
//                       B (activations, K-major, 128B-swizzled) from shared memory, D in TMEM;
//                       tcgen05.commit releases the activation stages and the A buffers.
//   warps 0-7 again     epilogue: tcgen05.ld the fp32 accumulators, coalesced stores of y.
//
// TMEM: 512 columns = D (<= 256) + 2 x 128 (two A buffers of one K-block each).
// Every mbarrier wait is bounded; a wait that gives up sets the status word and all roles drain to
// the final barrier, where TMEM is freed.  No cluster launch, no multicast.
#include <cuda.h>

#include <cstdlib>

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace hf2q {

using namespace tc;

namespace {

constexpr int TILE_N = 128;      // weight rows per CTA (MMA M)
constexpr int KB = 256;          // K elements per block step
constexpr int XK = 64;           // K elements per activation stage (128 bytes of f16)
// Tiles of <= 64 tokens, and the 128-token tiles of the expert-routed product (short K, many tiles), run two CTAs
// per SM (one CTA's fixed latencies and its epilogue hide behind the other's work): one A buffer instead of two,
// 256 TMEM columns instead of 512, and buffers sized so that two CTAs fit the SM's shared memory.
constexpr bool two_ctas_of(int nt, bool grouped) { return nt <= 64 || (grouped && nt == 128); }
constexpr int raw_stages_of(uint32_t type, int nt, bool grouped) {
    return (type == HF2Q_TYPE_Q8_0 || nt >= 256 || two_ctas_of(nt, grouped)) ? 2 : 3;
}
constexpr int a_bufs_of(int nt, bool grouped) { return two_ctas_of(nt, grouped) ? 1 : 2; }
constexpr uint32_t tmem_cols_of(int nt, bool grouped) { return two_ctas_of(nt, grouped) ? 256u : 512u; }
// activation stages: one stage is NT rows x 64 elements; keep ~128 KB of them in flight so that the
// copies for the next K-blocks are issued long before the MMA warp needs them
constexpr int x_stages_of(uint32_t type, int nt, bool grouped) {
    return nt >= 256 ? (type == HF2Q_TYPE_Q8_0 ? 4 : 5) : (grouped && nt == 128) ? 3 : 8;
}
constexpr int DEQ_GROUPS = 2;                        // groups of 4 dequantiser warps; group g takes quarters g*2, g*2+1
constexpr int QPG = 4 / DEQ_GROUPS;                  // quarters (64 elements) of a K-block per group
constexpr int DEQ_WARPS = 4 * DEQ_GROUPS;
constexpr int GEMM_THREADS = (DEQ_WARPS + 2) * 32;

// One token tile of the grouped (expert-routed) product: rows [start, start+count) of the
// expert-sorted activation panel belong to expert `expert`.
struct GroupTile { uint32_t expert, start, count, pad; };

struct GParams {
    float* y;
    uint32_t m, n, k;
    uint32_t ldy;           // floats between consecutive activation rows of y (n, or the full width when y is a column block)
    // grouped mode (mul_mat_id): tile table, its length, and the routed-row index of every sorted row
    const GroupTile* tiles;
    const uint32_t* n_tiles;
    const uint32_t* perm;
    // epilogue options: y += residual (same layout as y); DUAL kernels store silu(gate) * up, either as f32 into y
    // or, for the expert-routed form, as f16 into act16[sorted row][n] (the down product's activation panel)
    const float* residual;
    __half* act16;
    // expert-routed product only: instead of storing row perm[tok] of y, add route_w[perm[tok]] * value to row
    // perm[tok] / top_k of reduce_out (the weighted sum over the top-k slots; floating-point atomics, so the
    // rounding depends on the arrival order)
    const float* route_w;
    float* reduce_out;
    uint32_t top_k;
    uint32_t tiles_per_cta; // weight-row tiles (of 128 rows) one CTA walks, re-using its barriers, TMEM and token tile
    uint32_t boxw;          // bytes per weight row in one raw stage
    uint32_t blk_bytes;     // bytes of one 256-element K-block of a row
    uint32_t* status;
};

// Thread r dequantises quarters [Q0, Q0 + QPG) of its row's K-block into TMEM columns taddr + 32*q.
template <uint32_t TYPE, int Q0>
__device__ __forceinline__ void dequant_quarters(const uint8_t* row, uint32_t off, uint32_t taddr) {
    with_row_block<TYPE>(off, [&](auto rb) {
        rb.load(row, off);
#pragma unroll
        for (int qd = Q0; qd < Q0 + QPG; ++qd) {
            uint32_t out[32];
            rb.quarter(qd, out);
            tmem_st32(taddr + 32 * qd, out);
        }
    });
}
template <uint32_t TYPE>
__device__ __forceinline__ void dequant_dispatch(uint32_t grp, const uint8_t* row, uint32_t off, uint32_t taddr) {
    if constexpr (DEQ_GROUPS == 1) {
        dequant_quarters<TYPE, 0>(row, off, taddr);
    } else if constexpr (DEQ_GROUPS == 2) {
        if (grp == 0) dequant_quarters<TYPE, 0>(row, off, taddr);
        else dequant_quarters<TYPE, 2>(row, off, taddr);
    } else {
        switch (grp) {
            case 0: dequant_quarters<TYPE, 0>(row, off, taddr); break;
            case 1: dequant_quarters<TYPE, 1>(row, off, taddr); break;
            case 2: dequant_quarters<TYPE, 2>(row, off, taddr); break;
            default: dequant_quarters<TYPE, 3>(row, off, taddr); break;
        }
    }
}


// ---------------------------------------------------------------- the kernel
// DUAL: a tile is 64 output rows of a GATE matrix and the same 64 rows of an UP matrix -- two 64-row boxes per
// raw stage from two tensor maps.  The dequantiser thread of tensor-memory lane 32q + l reads gate row 16q + l
// (l < 16) or up row 16q + l - 16, so each warp holds both halves of 16 outputs; the MMA loop does not know.
// The epilogue pairs lane l with lane l + 16 by one shuffle per value and stores silu(gate) * up: the
// SwiGLU of build_dense_ffn_layer_gpu_q / build_moe_ffn_layer_gpu_q (gpu_ffn.rs:896-935, 2606-2760) without
// the two f32 round trips and the dispatch_silu_mul in between.
template <uint32_t TYPE, int NT, bool GROUPED, bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS, (two_ctas_of(NT, GROUPED) ? 2 : 1))
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
               const __grid_constant__ CUtensorMap tmap_x, const GParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    constexpr uint32_t X_STAGE = NT * 128;                       // NT rows x 64 f16, 128B-swizzled
    constexpr int X_STAGES = x_stages_of(TYPE, NT, GROUPED);
    uint8_t* xs = smem;                                          // X_STAGES x X_STAGE (1024-aligned)
    constexpr int RAW_STAGES = raw_stages_of(TYPE, NT, GROUPED);
    constexpr uint32_t TILE_ROWS = DUAL ? 64 : TILE_N;           // output rows of one tile
    uint8_t* raw = xs + X_STAGES * X_STAGE;                      // RAW_STAGES x 128 x boxw
    const uint32_t raw_stage = TILE_N * p.boxw;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw + RAW_STAGES * raw_stage);
    uint64_t* raw_full = bars;                  // [RAW_STAGES]
    uint64_t* raw_empty = raw_full + RAW_STAGES;
    uint64_t* x_full = raw_empty + RAW_STAGES;  // [X_STAGES]
    uint64_t* x_empty = x_full + X_STAGES;
    constexpr int A_BUFS = a_bufs_of(NT, GROUPED);
    constexpr uint32_t TMEM_COLS = tmem_cols_of(NT, GROUPED);
    uint64_t* a_full = x_empty + X_STAGES;      // [A_BUFS][DEQ_GROUPS]: each group's half (128 K elements) of an A buffer
    uint64_t* a_empty = a_full + 4;
    uint64_t* d_full = a_empty + 4;             // [1]
    uint64_t* d_empty = d_full + 1;             // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // this CTA's weight-row tiles: [tile0, tile0 + ntile)
    const uint32_t n_row_tiles = (p.n + TILE_ROWS - 1) / TILE_ROWS;
    const uint32_t tile0 = blockIdx.x * p.tiles_per_cta;
    const uint32_t ntile = min(p.tiles_per_cta, n_row_tiles - tile0);
    uint32_t tok0 = blockIdx.y * NT, tok_end = p.m, expert = 0;
    if constexpr (GROUPED) {
        if (blockIdx.y >= *p.n_tiles) return;              // the grid is sized for the worst case
        const GroupTile gt = p.tiles[blockIdx.y];
        tok0 = gt.start; tok_end = gt.start + gt.count; expert = gt.expert;
    }
    const uint32_t nkb = p.k / KB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RAW_STAGES; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], DEQ_WARPS); }
        for (int s = 0; s < X_STAGES; ++s) { mbar_init(&x_full[s], 1); mbar_init(&x_empty[s], 1); }
        for (int s = 0; s < 4; ++s) { mbar_init(&a_full[s], DEQ_WARPS / DEQ_GROUPS); mbar_init(&a_empty[s], 1); }
        mbar_init(d_full, 1);
        mbar_init(d_empty, DEQ_WARPS);
        mbar_fence_init();
    }
    if (warp == DEQ_WARPS + 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_d = tmem_base;                 // columns [0, NT)
    const uint32_t tmem_a = tmem_base + (A_BUFS == 1 ? 128 : 256);     // A_BUFS buffers of 128 columns

    if (warp == DEQ_WARPS) {
        // ------------------------------ TMA producer: lane 0 streams the weight stages, lane 1 the activation stages
        // (two independent rings: a full activation ring must not hold back the next weight stage)
        if (lane == 0) {
            bool ok = true;
            for (uint32_t tl = 0, gk = 0; tl < ntile && ok; ++tl) {           // gk: K-block count over all tiles
                const uint32_t row0 = (tile0 + tl) * TILE_ROWS;
                for (uint32_t kb = 0; kb < nkb && ok; ++kb, ++gk) {
                    const uint32_t rs = gk % RAW_STAGES;
                    if (gk >= RAW_STAGES) ok = mbar_wait_bounded(&raw_empty[rs], ((gk / RAW_STAGES) - 1) & 1, p.status);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&raw_full[rs], raw_stage);
                    const uint32_t byte0 = (kb * p.blk_bytes) & ~15u;       // 16-byte aligned start of the box
                    if constexpr (GROUPED)
                        tma_3d(raw + rs * raw_stage, &tmap_w, static_cast<int>(byte0 >> 1), static_cast<int>(row0), static_cast<int>(expert), &raw_full[rs]);
                    else
                        tma_2d(raw + rs * raw_stage, &tmap_w, static_cast<int>(byte0 >> 1), static_cast<int>(row0), &raw_full[rs]);
                    if constexpr (DUAL) {                                   // the up rows: second half of the stage (both boxes hold 64 rows)
                        uint8_t* dst2 = raw + rs * raw_stage + 64 * p.boxw;
                        if constexpr (GROUPED)
                            tma_3d(dst2, &tmap_w2, static_cast<int>(byte0 >> 1), static_cast<int>(row0), static_cast<int>(expert), &raw_full[rs]);
                        else
                            tma_2d(dst2, &tmap_w2, static_cast<int>(byte0 >> 1), static_cast<int>(row0), &raw_full[rs]);
                    }
                }
            }
        } else if (lane == 1) {
            bool ok = true;
            const uint32_t nx = ntile * nkb * (KB / XK);
            for (uint32_t xi = 0; xi < nx && ok; ++xi) {
                const uint32_t st = xi % X_STAGES, kx = xi % (nkb * (KB / XK));      // K position inside the current tile
                if (xi >= X_STAGES) ok = mbar_wait_bounded(&x_empty[st], ((xi / X_STAGES) - 1) & 1, p.status);
                if (!ok) break;
                mbar_arrive_expect_tx(&x_full[st], X_STAGE);
                tma_2d(xs + st * X_STAGE, &tmap_x, static_cast<int>(kx * XK), static_cast<int>(tok0), &x_full[st]);
            }
        }
    } else if (warp == DEQ_WARPS + 1) {
        // ------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor: D f32, A/B f16, both K-major, M = 128, N = the tile's token count rounded up to 16
            // (an expert's tile is rarely full: the MMAs skip the token columns nobody reads)
            const uint32_t n_mma = max(16u, (min(static_cast<uint32_t>(NT), tok_end - tok0) + 15u) & ~15u);
            const uint32_t IDESC = (1u << 4) | ((n_mma >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
            bool ok = true;
            for (uint32_t tl = 0, gk = 0; tl < ntile && ok; ++tl) {
                // the previous tile's accumulators must have been read before they are overwritten
                if (tl) ok = mbar_wait_bounded(d_empty, (tl - 1) & 1, p.status);
                for (uint32_t kb = 0; kb < nkb && ok; ++kb, ++gk) {
                    const uint32_t ab = gk % A_BUFS;
                    for (uint32_t j = 0; j < KB / XK && ok; ++j) {
                        // quarters 0, 1 come from dequantiser group 0, quarters 2, 3 from group 1
                        if ((j & (QPG - 1)) == 0) {
                            ok = mbar_wait_bounded(&a_full[ab * DEQ_GROUPS + j / QPG], (gk / A_BUFS) & 1, p.status);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        const uint32_t xi = gk * (KB / XK) + j, st = xi % X_STAGES;
                        ok = mbar_wait_bounded(&x_full[st], (xi / X_STAGES) & 1, p.status);
                        if (!ok) break;
                        tc_fence_after();
                        const uint64_t bdesc = smem_desc_sw128(smem_u32(xs + st * X_STAGE));
#pragma unroll
                        for (uint32_t kk = 0; kk < XK / 16; ++kk) {
                            // A: 8 columns (16 f16) per K step; B: +32 bytes inside the swizzled row
                            umma_ts(tmem_d, tmem_a + ab * 128 + (j * (XK / 16) + kk) * 8, bdesc + 2 * kk, IDESC,
                                    (kb | j | kk) != 0 ? 1u : 0u);
                        }
                        tc_commit(&x_empty[st]);       // activation stage free once these MMAs retire,
                        if ((j & (QPG - 1)) == QPG - 1) tc_commit(&a_empty[ab * DEQ_GROUPS + j / QPG]);   // and the group's half of A
                    }
                }
                if (ok) tc_commit(d_full);
            }
        }
    } else {
        // ------------------------------ dequantisers (thread = weight row), then epilogue
        const uint32_t quad = warp & 3, grp = static_cast<uint32_t>(warp) >> 2;
        const uint32_t r = quad * 32 + lane;               // weight row of the tile == TMEM lane
        const uint32_t lane_addr = (quad * 32u) << 16;
        // row of the raw stage this thread dequantises (DUAL: gate box rows 0..63, up box rows 64..127)
        const uint32_t src_row = DUAL ? ((lane < 16 ? 0u : 64u) + 16 * quad + (lane & 15)) : r;
        const int n_cols = static_cast<int>(min(static_cast<uint32_t>(NT), tok_end - tok0));   // token columns in use
        bool ok = true;
        for (uint32_t tl = 0, gk = 0; tl < ntile && ok; ++tl) {
            const uint32_t row0 = (tile0 + tl) * TILE_ROWS;
            for (uint32_t kb = 0; kb < nkb; ++kb, ++gk) {
                const uint32_t rs = gk % RAW_STAGES, ab = gk % A_BUFS;
                if (ok) ok = mbar_wait_bounded(&raw_full[rs], (gk / RAW_STAGES) & 1, p.status);
                if (ok && gk >= A_BUFS) ok = mbar_wait_bounded(&a_empty[ab * DEQ_GROUPS + grp], ((gk / A_BUFS) - 1) & 1, p.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t off = (kb * p.blk_bytes) & 15u;
                dequant_dispatch<TYPE>(grp, raw + rs * raw_stage + src_row * p.boxw, off, tmem_a + ab * 128 + lane_addr);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { mbar_arrive(&a_full[ab * DEQ_GROUPS + grp]); mbar_arrive(&raw_empty[rs]); }
            }
            // epilogue of this tile
            if (ok) ok = mbar_wait_bounded(d_full, tl & 1, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if constexpr (DUAL) {
                // lanes 0..15 of this warp hold gate rows, lanes 16..31 the up rows of the same 16 outputs.  Of each
                // pair of tokens the lower lane finishes the even one and the upper lane the odd one: one exchange
                // per pair, every lane busy.
                const uint32_t row = row0 + 16 * quad + (lane & 15);
                const bool upper = lane >= 16;
                bool clipped = false;
#pragma unroll 1
                for (int c0 = 32 * static_cast<int>(grp); c0 < n_cols; c0 += 32 * DEQ_GROUPS) {
                    uint32_t v[32];
                    tmem_ld32(tmem_d + lane_addr + c0, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float other = __shfl_xor_sync(0xffffffffu, __uint_as_float(upper ? v[j] : v[j + 1]), 16);
                        const float g = upper ? other : __uint_as_float(v[j]);
                        const float u = upper ? __uint_as_float(v[j + 1]) : other;
                        const uint32_t tok = tok0 + c0 + j + (upper ? 1 : 0);
                        if (row < p.n && tok < tok_end) {
                            const float act = g / (1.0f + expf(-g)) * u;
                            if (GROUPED && p.act16) {          // same clipping rule as the f32 -> f16 conversion of any activation panel
                                clipped |= fabsf(act) > 65504.0f;
                                p.act16[static_cast<size_t>(tok) * p.n + row] = __float2half_rn(fminf(fmaxf(act, -65504.0f), 65504.0f));
                            } else {
                                p.y[static_cast<size_t>(GROUPED ? p.perm[tok] : tok) * p.ldy + row] = act;
                            }
                        }
                    }
                }
                if (clipped) atomicOr(p.status, STATUS_X_CLIPPED);
            } else {
            const uint32_t row = row0 + r;
#pragma unroll 1
            for (int c0 = 32 * static_cast<int>(grp); c0 < n_cols; c0 += 32 * DEQ_GROUPS) {   // the groups share the columns
                uint32_t v[32];
                tmem_ld32(tmem_d + lane_addr + c0, v);
                tmem_wait_ld();
                if (row < p.n) {
                    if (p.residual) {
                        // y may be the residual itself: issue all loads before the first store
                        float res[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t tok = tok0 + c0 + j;
                            res[j] = tok < tok_end ? __ldcg(p.residual + static_cast<size_t>(GROUPED ? p.perm[tok] : tok) * p.ldy + row) : 0.f;
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + res[j]);
                    }
                    if (GROUPED && p.reduce_out) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t tok = tok0 + c0 + j;
                            if (tok < tok_end) {
                                const uint32_t dst = p.perm[tok];
                                atomicAdd(p.reduce_out + static_cast<size_t>(dst / p.top_k) * p.ldy + row, p.route_w[dst] * __uint_as_float(v[j]));
                            }
                        }
                    } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t tok = tok0 + c0 + j;
                        if (tok < tok_end) {
                            const uint32_t dst = GROUPED ? p.perm[tok] : tok;      // scatter back to routed-row order
                            p.y[static_cast<size_t>(dst) * p.ldy + row] = __uint_as_float(v[j]);
                        }
                    }
                    }
                }
            }
            }
            // this warp is done reading the accumulators: the next tile's MMAs may overwrite them
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(d_empty);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == DEQ_WARPS + 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---------------------------------------------------------------- activations -> f16 panel
__global__ void __launch_bounds__(256) x_to_f16_kernel(const void* __restrict__ x, uint32_t x_bf16, __half* __restrict__ out,
                                                       uint64_t n_elems, uint32_t* status) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    bool clipped = false;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_elems; i += stride) {
        float v = x_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(x)[i]) : static_cast<const float*>(x)[i];
        clipped |= fabsf(v) > 65504.0f;
        v = fminf(fmaxf(v, -65504.0f), 65504.0f);
        out[i] = __float2half_rn(v);
    }
    if (clipped) atomicOr(status, STATUS_X_CLIPPED);
}

// The same conversion for activations stored [n_heads][m][head_dim] (the layout flash attention writes; the
// reference's O projection reads it through quantized_matmul_mm_tensor_perm021, forward_prefill_batched.rs:2218-2258):
// logical (t, c) is physical (h = c / head_dim, t, f = c % head_dim).  8 elements per thread.
__global__ void __launch_bounds__(256) x_perm021_to_f16_kernel(const void* __restrict__ x, uint32_t x_bf16, __half* __restrict__ out,
                                                               uint32_t m, uint32_t k, uint32_t head_dim, uint32_t* status) {
    const uint64_t n8 = static_cast<uint64_t>(m) * k / 8, stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    bool clipped = false;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const uint64_t e = i * 8;
        const uint32_t t = static_cast<uint32_t>(e / k), c = static_cast<uint32_t>(e % k), h = c / head_dim, f = c % head_dim;
        const uint64_t src = (static_cast<uint64_t>(h) * m + t) * head_dim + f;
        float v[8];
        if (x_bf16) {
            const uint4 r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + src));
            const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[2 * j] = __uint_as_float(rr[j] << 16); v[2 * j + 1] = __uint_as_float(rr[j] & 0xffff0000u); }
        } else {
            const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(x) + src));
            const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(x) + src + 4));
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            clipped |= (fabsf(v[2 * j]) > 65504.0f) | (fabsf(v[2 * j + 1]) > 65504.0f);
            const __half2 hh = __floats2half2_rn(fminf(fmaxf(v[2 * j], -65504.0f), 65504.0f), fminf(fmaxf(v[2 * j + 1], -65504.0f), 65504.0f));
            o[j] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        *reinterpret_cast<uint4*>(out + e) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (clipped) atomicOr(status, STATUS_X_CLIPPED);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

uint32_t boxw_of(uint32_t type) { return tc_boxw(type); }

template <uint32_t TYPE, int NT, bool GROUPED, bool DUAL = false>
cudaError_t launch_gemm_t(const CUtensorMap& tw, const CUtensorMap& tw2, const CUtensorMap& tx, const GParams& p, uint32_t grid_y, cudaStream_t st) {
    auto kern = gemm_tc_kernel<TYPE, NT, GROUPED, DUAL>;
    const size_t raw_stages = raw_stages_of(TYPE, NT, GROUPED);
    const size_t smem = 1024 + static_cast<size_t>(x_stages_of(TYPE, NT, GROUPED)) * NT * 128 + raw_stages * TILE_N * p.boxw + 512;
    static PerDeviceFlag attr;
    if (const cudaError_t e = ensure_max_dynamic_smem(kern, 227 * 1024, attr); e != cudaSuccess) return e;
    const uint32_t tile_rows = DUAL ? 64 : TILE_N;
    const uint32_t row_tiles = (p.n + tile_rows - 1) / tile_rows;
    const dim3 grid((row_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta, grid_y);
    kern<<<grid, GEMM_THREADS, smem, st>>>(tw, tw2, tx, p);
    return cudaGetLastError();
}

template <uint32_t TYPE>
cudaError_t launch_gemm_nt(const CUtensorMap& tw, const CUtensorMap& tx, const GParams& p, uint32_t nt, cudaStream_t st) {
    const uint32_t gy = (p.m + nt - 1) / nt;
    switch (nt) {
        case 32: return launch_gemm_t<TYPE, 32, false>(tw, tw, tx, p, gy, st);
        case 64: return launch_gemm_t<TYPE, 64, false>(tw, tw, tx, p, gy, st);
        case 128: return launch_gemm_t<TYPE, 128, false>(tw, tw, tx, p, gy, st);
        default: return launch_gemm_t<TYPE, 256, false>(tw, tw, tx, p, gy, st);
    }
}

// the SwiGLU pair
template <uint32_t TYPE, bool GROUPED>
cudaError_t launch_gemm_dual_nt(const CUtensorMap& tg, const CUtensorMap& tu, const CUtensorMap& tx, const GParams& p, uint32_t nt, uint32_t gy,
                                cudaStream_t st) {
    switch (nt) {
        case 32: return launch_gemm_t<TYPE, 32, GROUPED, true>(tg, tu, tx, p, gy, st);
        case 64: return launch_gemm_t<TYPE, 64, GROUPED, true>(tg, tu, tx, p, gy, st);
        case 128: return launch_gemm_t<TYPE, 128, GROUPED, true>(tg, tu, tx, p, gy, st);
        default: return launch_gemm_t<TYPE, 256, GROUPED, true>(tg, tu, tx, p, gy, st);
    }
}

}  // namespace


bool gemm_tc_supported(uint32_t type, const void* w, uint32_t n, uint32_t k) {
    (void)n;
    const BlockGeom g = block_geom(type);
    const uint64_t row_bytes = static_cast<uint64_t>(k) / g.elems * g.bytes;
    return encode_fn() != nullptr && k % KB == 0 && row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0;
}

uint64_t gemm_tc_workspace_bytes(uint32_t m, uint32_t k) {
    return (static_cast<uint64_t>(m) * k * 2 + 255) & ~static_cast<uint64_t>(255);
}

// Tokens per CTA tile for m activation rows over `tiles_n` weight-row tiles: the widest tile whose
// CTA count still fills the SMs evenly (wide tiles amortise the dequantisation best).
uint32_t gemm_tc_token_tile(uint32_t m, uint32_t tiles_n, int sms) {
    if (m <= 32) return 32;
    if (m <= 64) return 64;
    uint32_t best = 128;
    double best_score = -1.0;
    for (uint32_t nt : {256u, 128u, 64u}) {
        if (nt / 2 >= m) continue;
        const uint32_t ctas = tiles_n * ((m + nt - 1) / nt);
        const uint32_t waves = (ctas + sms - 1) / sms;
        const double fill = static_cast<double>(ctas) / (static_cast<double>(waves) * sms);
        const double score = fill * (nt == 256 ? 1.0 : nt == 128 ? 0.78 : 0.55);   // measured relative tile efficiency
        if (score > best_score) { best_score = score; best = nt; }
    }
    return best;
}

namespace {
// w_up != nullptr: the SwiGLU pair (w = gate); residual != nullptr: y = product + residual
cudaError_t gemm_tc_dense(uint32_t type, const void* w, const void* w_up, const void* x, uint32_t x_dtype, float* y, uint32_t m, uint32_t n,
                          uint32_t k, void* workspace, uint32_t* status, int sm_count, cudaStream_t st, int* launches,
                          uint32_t ldy, bool x_ready, const float* residual, uint32_t perm_head_dim = 0) {
    const bool dual = w_up != nullptr;
    const BlockGeom g = block_geom(type);
    const uint64_t row_bytes = static_cast<uint64_t>(k) / g.elems * g.bytes;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;

    // 1. activations -> f16 [m][k] in the workspace
    __half* xh = static_cast<__half*>(workspace);
    const uint64_t nx = static_cast<uint64_t>(m) * k;
    if (!x_ready) {       // (a caller that runs several products on the same activations converts them once)
        uint64_t want = (nx + 255) / 256;
        const uint64_t cap = static_cast<uint64_t>(sm_count) * 16;
        if (perm_head_dim) {
            want = (nx / 8 + 255) / 256;
            x_perm021_to_f16_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, st>>>(x, x_dtype == HF2Q_DT_BF16, xh, m, k, perm_head_dim, status);
        } else {
            x_to_f16_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, st>>>(x, x_dtype == HF2Q_DT_BF16, xh, nx, status);
        }
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    // 2. tensor maps
    GParams p{};
    p.y = y; p.m = m; p.n = n; p.k = k;
    p.ldy = ldy ? ldy : n;
    p.residual = residual;
    p.tiles_per_cta = 1;
    p.boxw = boxw_of(type);
    p.blk_bytes = KB / g.elems * g.bytes;
    p.status = status;
    const uint32_t tile_rows = dual ? 64 : TILE_N;
    const uint32_t nt = gemm_tc_token_tile(m, (n + tile_rows - 1) / tile_rows, sm_count);
    alignas(64) CUtensorMap tw, tw2, tx;
    for (int which = 0; which < (dual ? 2 : 1); ++which) {
        // weights: [n rows][row_bytes] viewed as u16, box = boxw bytes x 128 (pair: 64) rows, no swizzle
        cuuint64_t dims[2] = {row_bytes / 2, n};
        cuuint64_t strides[1] = {row_bytes};
        cuuint32_t box[2] = {p.boxw / 2, tile_rows};
        cuuint32_t es[2] = {1, 1};
        CUresult r = enc(which ? &tw2 : &tw, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(which ? w_up : w), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    {
        // activations: [m][k] f16, box = 64 elements x nt rows, 128-byte swizzle
        cuuint64_t dims[2] = {k, m};
        cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
        cuuint32_t box[2] = {XK, nt};
        cuuint32_t es[2] = {1, 1};
        CUresult r = enc(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xh, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    if (launches) *launches = x_ready ? 1 : 2;
    if (dual) {
        const uint32_t gy = (m + nt - 1) / nt;
        switch (type) {
            case HF2Q_TYPE_Q4_0: return launch_gemm_dual_nt<HF2Q_TYPE_Q4_0, false>(tw, tw2, tx, p, nt, gy, st);
            case HF2Q_TYPE_Q8_0: return launch_gemm_dual_nt<HF2Q_TYPE_Q8_0, false>(tw, tw2, tx, p, nt, gy, st);
            case HF2Q_TYPE_Q4_K: return launch_gemm_dual_nt<HF2Q_TYPE_Q4_K, false>(tw, tw2, tx, p, nt, gy, st);
            case HF2Q_TYPE_Q5_K: return launch_gemm_dual_nt<HF2Q_TYPE_Q5_K, false>(tw, tw2, tx, p, nt, gy, st);
            case HF2Q_TYPE_Q6_K: return launch_gemm_dual_nt<HF2Q_TYPE_Q6_K, false>(tw, tw2, tx, p, nt, gy, st);
            default: return cudaErrorNotSupported;
        }
    }
    switch (type) {
        case HF2Q_TYPE_Q4_0: return launch_gemm_nt<HF2Q_TYPE_Q4_0>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q8_0: return launch_gemm_nt<HF2Q_TYPE_Q8_0>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q4_K: return launch_gemm_nt<HF2Q_TYPE_Q4_K>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q5_K: return launch_gemm_nt<HF2Q_TYPE_Q5_K>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q6_K: return launch_gemm_nt<HF2Q_TYPE_Q6_K>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q4_1: return launch_gemm_nt<HF2Q_TYPE_Q4_1>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q5_0: return launch_gemm_nt<HF2Q_TYPE_Q5_0>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q5_1: return launch_gemm_nt<HF2Q_TYPE_Q5_1>(tw, tx, p, nt, st);
        case HF2Q_TYPE_IQ4_NL: return launch_gemm_nt<HF2Q_TYPE_IQ4_NL>(tw, tx, p, nt, st);
        case HF2Q_TYPE_MLX_AFFINE4_GS32: return launch_gemm_nt<HF2Q_TYPE_MLX_AFFINE4_GS32>(tw, tx, p, nt, st);
        default: return cudaErrorInvalidValue;
    }
}
}  // namespace

cudaError_t launch_gemm_tc(uint32_t type, const void* w, const void* x, uint32_t x_dtype, float* y, uint32_t m, uint32_t n,
                           uint32_t k, void* workspace, uint32_t* status, int sm_count, cudaStream_t st, int* launches,
                           uint32_t ldy, bool x_ready, const float* residual, uint32_t perm_head_dim) {
    return gemm_tc_dense(type, w, nullptr, x, x_dtype, y, m, n, k, workspace, status, sm_count, st, launches, ldy, x_ready, residual, perm_head_dim);
}

// the five formats hf2q's quantizer writes for FFN tensors; the 32-element fallback formats keep the unfused sequence
bool gemm_tc_swiglu_supported(uint32_t type) {
    return type == HF2Q_TYPE_Q4_0 || type == HF2Q_TYPE_Q8_0 || type == HF2Q_TYPE_Q4_K || type == HF2Q_TYPE_Q5_K || type == HF2Q_TYPE_Q6_K;
}

cudaError_t launch_gemm_tc_swiglu(uint32_t type, const void* w_gate, const void* w_up, const void* x, uint32_t x_dtype, float* y,
                                  uint32_t m, uint32_t n, uint32_t k, void* workspace, uint32_t* status, int sm_count,
                                  cudaStream_t st, int* launches, bool x_ready) {
    return gemm_tc_dense(type, w_gate, w_up, x, x_dtype, y, m, n, k, workspace, status, sm_count, st, launches, n, x_ready, nullptr);
}


bool gemm_tc_grouped_supported(uint32_t type, const void* w, uint64_t expert_stride, uint32_t n_experts, uint32_t k) {
    return gemm_tc_supported(type, w, 0, k) && expert_stride % 16 == 0 && n_experts <= 2048;
}

template <uint32_t TYPE>
cudaError_t launch_grouped_nt(const CUtensorMap& tw, const CUtensorMap& tx, const GParams& p, uint32_t nt, uint32_t gy, cudaStream_t st) {
    switch (nt) {
        case 32: return launch_gemm_t<TYPE, 32, true>(tw, tw, tx, p, gy, st);
        case 64: return launch_gemm_t<TYPE, 64, true>(tw, tw, tx, p, gy, st);
        case 128: return launch_gemm_t<TYPE, 128, true>(tw, tw, tx, p, gy, st);
        default: return launch_gemm_t<TYPE, 256, true>(tw, tw, tx, p, gy, st);
    }
}

// One launch over (weight-row tile, token tile of one expert).  The grid is sized for the largest
// possible number of token tiles; CTAs past the actual count (read from the scratch header) exit.
// w_up != nullptr: the SwiGLU pair (w_stacked = gate); act16 != nullptr: its result
// goes to act16[sorted row][n] as f16 instead of y.  x_panel overrides the gathered activation panel of the
// scratch (the down product reads the act16 panel of the pair launch).
cudaError_t launch_gemm_tc_grouped(uint32_t type, const void* w_stacked, uint64_t expert_stride, uint32_t n_experts, uint32_t rows,
                                   float* y, uint32_t n, uint32_t k, uint32_t nt, void* scratch, const MoeScratch& lay,
                                   uint32_t* status, cudaStream_t st, const void* w_up, const void* x_panel, void* act16,
                                   const float* route_w, float* reduce_out, uint32_t top_k) {
    const bool dual = w_up != nullptr;
    const uint32_t tile_rows = dual ? 64 : TILE_N;
    const BlockGeom g = block_geom(type);
    const uint64_t row_bytes = static_cast<uint64_t>(k) / g.elems * g.bytes;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    uint8_t* base = static_cast<uint8_t*>(scratch);
    GParams p{};
    p.y = y; p.m = rows; p.n = n; p.k = k;
    p.ldy = n;
    {
        // One CTA walks several weight-row tiles of its (expert, token tile): barriers, tensor memory and the
        // first copies' latency are paid once.  Keep about two CTAs per resident slot (2 per SM) in the grid.
        static const int forced = [] { const char* v = getenv("HF2Q_CUDA_MOE_TPC"); return v && *v ? atoi(v) : 0; }();   // tuning aid
        const uint32_t row_tiles = (n + tile_rows - 1) / tile_rows, token_tiles = rows / nt + n_experts / 2;
        uint32_t tpc = static_cast<uint32_t>(static_cast<uint64_t>(row_tiles) * token_tiles / (4 * 148 * 2));
        if (forced > 0) tpc = static_cast<uint32_t>(forced);
        p.tiles_per_cta = tpc < 1 ? 1 : tpc > 8 ? 8 : tpc;
        if (p.tiles_per_cta > row_tiles) p.tiles_per_cta = row_tiles;
    }
    p.tiles = reinterpret_cast<const GroupTile*>(base + lay.tiles_off);
    p.n_tiles = reinterpret_cast<const uint32_t*>(base);
    p.perm = reinterpret_cast<const uint32_t*>(base + lay.perm_off);
    p.act16 = static_cast<__half*>(act16);
    p.route_w = route_w; p.reduce_out = reduce_out; p.top_k = top_k ? top_k : 1;
    p.boxw = boxw_of(type);
    p.blk_bytes = KB / g.elems * g.bytes;
    p.status = status;
    alignas(64) CUtensorMap tw, tw2, tx;
    for (int which = 0; which < (dual ? 2 : 1); ++which) {
        // stacked experts: [E][n rows][row_bytes] viewed as u16; box = boxw bytes x 128 (pair: 64) rows x 1 expert
        cuuint64_t dims[3] = {row_bytes / 2, n, n_experts};
        cuuint64_t strides[2] = {row_bytes, expert_stride};
        cuuint32_t box[3] = {p.boxw / 2, tile_rows, 1};
        cuuint32_t es[3] = {1, 1, 1};
        CUresult r = enc(which ? &tw2 : &tw, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(which ? w_up : w_stacked), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    {
        cuuint64_t dims[2] = {k, rows};
        cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
        cuuint32_t box[2] = {XK, nt};
        cuuint32_t es[2] = {1, 1};
        void* xp = x_panel ? const_cast<void*>(x_panel) : static_cast<void*>(base + lay.xg_off);
        CUresult r = enc(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xp, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    const uint32_t gy = rows / nt + n_experts;           // >= sum over experts of ceil(count / nt)
    if (dual) {
        switch (type) {
            case HF2Q_TYPE_Q4_0: return launch_gemm_dual_nt<HF2Q_TYPE_Q4_0, true>(tw, tw2, tx, p, nt, gy, st);
            case HF2Q_TYPE_Q8_0: return launch_gemm_dual_nt<HF2Q_TYPE_Q8_0, true>(tw, tw2, tx, p, nt, gy, st);
            case HF2Q_TYPE_Q4_K: return launch_gemm_dual_nt<HF2Q_TYPE_Q4_K, true>(tw, tw2, tx, p, nt, gy, st);
            case HF2Q_TYPE_Q5_K: return launch_gemm_dual_nt<HF2Q_TYPE_Q5_K, true>(tw, tw2, tx, p, nt, gy, st);
            case HF2Q_TYPE_Q6_K: return launch_gemm_dual_nt<HF2Q_TYPE_Q6_K, true>(tw, tw2, tx, p, nt, gy, st);
            default: return cudaErrorNotSupported;
        }
    }
    switch (type) {
        case HF2Q_TYPE_Q4_0: return launch_grouped_nt<HF2Q_TYPE_Q4_0>(tw, tx, p, nt, gy, st);
        case HF2Q_TYPE_Q8_0: return launch_grouped_nt<HF2Q_TYPE_Q8_0>(tw, tx, p, nt, gy, st);
        case HF2Q_TYPE_Q4_K: return launch_grouped_nt<HF2Q_TYPE_Q4_K>(tw, tx, p, nt, gy, st);
        case HF2Q_TYPE_Q5_K: return launch_grouped_nt<HF2Q_TYPE_Q5_K>(tw, tx, p, nt, gy, st);
        case HF2Q_TYPE_Q6_K: return launch_grouped_nt<HF2Q_TYPE_Q6_K>(tw, tx, p, nt, gy, st);
        case HF2Q_TYPE_Q4_1: return launch_grouped_nt<HF2Q_TYPE_Q4_1>(tw, tx, p, nt, gy, st);
        case HF2Q_TYPE_Q5_0: return launch_grouped_nt<HF2Q_TYPE_Q5_0>(tw, tx, p, nt, gy, st);
        case HF2Q_TYPE_Q5_1: return launch_grouped_nt<HF2Q_TYPE_Q5_1>(tw, tx, p, nt, gy, st);
        case HF2Q_TYPE_IQ4_NL: return launch_grouped_nt<HF2Q_TYPE_IQ4_NL>(tw, tx, p, nt, gy, st);
        case HF2Q_TYPE_MLX_AFFINE4_GS32: return launch_grouped_nt<HF2Q_TYPE_MLX_AFFINE4_GS32>(tw, tx, p, nt, gy, st);
        default: return cudaErrorInvalidValue;
    }
}

// ---------------------------------------------------------------- allocation-free variant
// Scratch for hf2q_cuda_qmatmul_static: the f16 copy of the activations lives in this fixed
// array instead of a caller workspace.  Every GPU that loads the library holds these 8 MiB until
// the process exits.  In host code `g_static_x16` is only a handle for the runtime, not a device
// address; the address a kernel can use comes from cudaGetSymbolAddress, per device.
constexpr uint64_t STATIC_SCRATCH_BYTES = 8ull << 20;
static __device__ __align__(256) unsigned char g_static_x16[STATIC_SCRATCH_BYTES];

uint64_t gemm_tc_static_scratch_bytes() { return STATIC_SCRATCH_BYTES; }

// Device address of the scratch array on `device` (which must be the current device).  The first
// call per device asks the runtime; later calls return the cached pointer.
cudaError_t gemm_tc_static_scratch(int device, void** out) {
    constexpr int MAX_DEV = 64;
    static std::mutex mu;
    static void* cached[MAX_DEV] = {nullptr};
    if (device < 0 || device >= MAX_DEV) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[device]) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_x16);
        if (e != cudaSuccess) return e;
        cached[device] = ptr;
    }
    *out = cached[device];
    return cudaSuccess;
}

}  // namespace hf2q
