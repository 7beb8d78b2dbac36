// K1 / K3 (main variant): dequant-fused mat-vec for 1..8 activation rows, dense and expert-routed.
//
//   y[t, r] = sum_k x[t, k] * dequant(W)[r, k]
//
// Stands in for mlx-native's kernel_mul_mv_<q>_f32 / kernel_mul_mv_id_<q>_f32 that hf2q reaches
// through quantized_matmul_ggml (m <= 8; src/inference/models/qwen35/gpu_ffn.rs:1236-1306,
// src/serve/forward_mlx.rs:9960-9968) and quantized_matmul_id_ggml (few rows; gpu_ffn.rs:188-206,
// forward_mlx.rs:5285-5292).
//
// Why it looks the way it does.  At 6.5 TB/s a B200 SM receives ~25 weight bytes per clock, i.e.
// 30 (Q6_K) to 44 (Q4_K) weight elements, but issues only 128 lane-instructions per clock: about
// 3-4 instructions per element, for all activation rows together.  One FMA per element and row
// already breaks that budget at 4 rows, so the multiply-accumulate goes through the warp-level
// m16n8k16 MMA (16 weight rows x 16 elements x 8 activation columns per instruction) and the
// CUDA cores only unpack bits:
//
//   * a persistent CTA (one per SM) owns groups of 16 weight rows; a producer warp streams their
//     RAW block bytes into a shared-memory ring with 1-D bulk copies (cp.async.bulk + mbarrier),
//     2048 elements per row and stage, so 18/34/210-byte blocks are readable at any 2-byte offset;
//   * consumer warps work in teams of 8, one team per ring stage, one warp per 256-element block
//     of the stage for all 16 rows: lane (g, t) unpacks rows g and g+8, four elements at a time,
//     into the A fragment.  The integer codes are fed as f16 SUBNORMALS (code * 2^-24): a single
//     PRMT turns two packed bytes into an f16x2 operand, with no int->float conversion and no
//     offset to subtract;
//   * scales stay out of the per-element path: Q4_K/Q5_K apply d*scale (f32, exact) to the sum of
//     each 32-element sub-block's two MMA steps; Q6_K applies d*scale to each 16-element MMA
//     result; Q4_0/Q8_0 apply d per block.  Offsets (the -dmin*m of Q4_K/Q5_K, the -32/-8/-128
//     code biases) become one small extra MMA (or FMA) per block against per-sub-block sums of x
//     that every CTA computes once;
//   * activations live in shared memory as f16 (bf16 input: exact in range; f32 input: split
//     into hi + lo halves on two MMA columns, ~2^-22 relative); rows too long for that are
//     handled in k-phases (see the kernel);
//   * a reducer warp combines the consumer warps' partial sums in a fixed order: no atomics,
//     bit-reproducible.
//
// Measured on B200: the per-block unpack + 9 MMAs of a Q6_K half block issue ~205 instructions
// per warp, and the legacy warp-level MMA holds its pipe for ~32 cycles per instruction and SM
// sub-partition, which caps this design at ~28 weight elements per clock and SM, i.e. about the
// HBM rate for Q6_K.
//
// Needs 16-byte aligned rows and k a multiple of 256; other shapes take the fp32 kernel in
// k1_gemv.cu.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>
#include <unordered_map>
#include <vector>

#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace hf2q {

namespace {

constexpr int ROWS = 16;               // weight rows per stage = rows of one MMA tile
constexpr uint32_t PRE_STAGES = 3;     // ring stages requested before the previous kernel has completed
constexpr int TEAM = 8;                // consumer warps per stage: one per 256-element block
constexpr int MAX_TEAMS = 3;
constexpr int SLICE_ELEMS = 2048;
constexpr int MAX_STAGES = 8;

struct MParams {
    const uint8_t* w;
    const uint8_t* w2;     // second expert tensor of a routed pair (or nullptr): slots >= pair_slots use it and y2
    const void* x;
    float* y;
    float* y2;
    uint32_t pair_slots;
    const uint32_t* ids;
    uint64_t expert_stride;
    uint32_t x_bf16;
    uint32_t m;            // activation rows of this launch (bf16: <= 8, f32: <= 4)
    uint32_t nslots;       // MMA columns in use: m (bf16) or 2m (f32 hi/lo split)
    uint32_t n, k;
    uint32_t top_k, n_experts;
    uint32_t row_bytes, slice_bytes, pitch, nslices, ngroups, stages;
    uint32_t xpitch;       // bytes between activation rows in shared memory
    uint32_t phase_base, phase_rem;   // k-phases: the first phase_rem have phase_base + 1 slices, the rest phase_base
    uint32_t last_nblk;        // 256-element blocks in the last slice of a row
    uint32_t w_evict_first;    // != 0: weight copies carry the L2 evict-first policy
    uint32_t swiglu;           // != 0 (EXT): w = gate, w2 = up; a CTA's row groups alternate gate, up and y = silu(gate) * up
    const float* residual;     // != nullptr: y = residual + product (may alias y)
    uint32_t use_tmap;         // != 0: a stage (16 rows x one slice) arrives with ONE 2-D tensor copy (dense launches)
    uint32_t dense_stage;      // != 0: a row is one slice and rows sit back to back in the stage, one bulk copy per stage
    uint32_t sub_groups;       // short rows (<= 4 blocks): a stage holds this many 16-row groups, one warp per (group, block)
    // fused all-gather (row-sharded weights over several GPUs); g_nranks == 0: plain store to y
    float* g_y[8];
    uint32_t* g_flag[8];
    uint32_t g_peer_ctas[8];   // CTAs of the same product on every rank (their arrivals at this rank)
    uint32_t g_nranks, g_rank, g_ntotal, g_col0, g_wait;
    long long wait_limit;      // clock ticks a wait for other ranks may take before it gives up
    // split-k (EXT): k is cut into `split` parts of one 2048-element slice each, part = blockIdx.y; every
    // part writes its partial sums to y + part * m * n (a scratch buffer) and a second kernel adds the parts
    const float* norm_w;       // != nullptr: x is RMS-normalised with this weight (and norm_eps) while the panel is built
    float norm_eps;
    uint32_t split, k_last;    // parts (0 = off); elements of the last part
    uint32_t kx;               // elements between activation rows of x in global memory (k of the whole product)
    uint32_t* status;
};


// The one CTA-wide barrier (id 0).  The producer warp arrives and carries on, the other warps
// wait.  Every participant names the thread count: a barrier whose participants disagree on the
// count (as the count-less form would once the producer warp has exited) is an error; and the warp
// must be converged, which the producer's per-lane copy loops do not guarantee by themselves.
template <int NTHREADS>
__device__ __forceinline__ void cta_arrive_n() {
    __syncwarp();
    asm volatile("bar.arrive 0, %0;" ::"n"(NTHREADS) : "memory");
}
template <int NTHREADS>
__device__ __forceinline__ void cta_sync_n() {
    asm volatile("bar.sync 0, %0;" ::"n"(NTHREADS) : "memory");
}

// m16n8k16, f16 inputs, f32 accumulate.  Lane (g = lane/4, t = lane%4) holds A for rows g (a0, a2)
// and g+8 (a1, a3) at k-columns {2t, 2t+1} (a0, a1) and {2t+8, 2t+9} (a2, a3); B for column g at
// the same k positions; C/D rows g (c[0], c[1]) and g+8 (c[2], c[3]) at columns 2t, 2t+1.
__device__ __forceinline__ void mma_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_new(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// bytes (b0,b1) / (b2,b3) of w as two f16 subnormals each: value = byte * 2^-24
__device__ __forceinline__ uint32_t sub01(uint32_t w) { return __byte_perm(w, 0u, 0x4140u); }
__device__ __forceinline__ uint32_t sub23(uint32_t w) { return __byte_perm(w, 0u, 0x4342u); }
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint2 ld_x4(const uint8_t* xrow, uint32_t e) {
    return *reinterpret_cast<const uint2*>(xrow + 2 * e);
}
constexpr float TWO24 = 16777216.0f;

// Bounded wait until source rank `src` has delivered everything the products launched here so far
// expect from it: arrival counter flag[src] against the expected count flag[8 + src] (written by
// earlier kernels of this stream, which have completed).  The acquire load orders the reads of the
// gathered columns after it.  Gives up after `limit` clock ticks and records that in *status.
__device__ __forceinline__ void gather_wait_source(const uint32_t* flag, uint32_t src, long long limit, uint32_t* status) {
    const uint32_t want = *reinterpret_cast<const volatile uint32_t*>(flag + 8 + src);
    const long long t0 = clock64();
    for (;;) {
        uint32_t got;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(flag + src) : "memory");
        if (static_cast<int32_t>(got - want) >= 0) break;
        if (clock64() - t0 > limit) { atomicOr(status, STATUS_WAIT_TIMEOUT); break; }
        __nanosleep(50);
    }
}

// ---- Q4_K / Q5_K: half a block (128 elements = chunks 2*half, 2*half+1 = sub-blocks 4*half..+3) of
// rows g and g+8.  A chunk is 32 bytes whose low nibbles are sub-block 2c and whose high nibbles are
// sub-block 2c+1.  Lane t takes words t and t+4 of each chunk, so an MMA step (sub-block, j) covers
// the 16 consecutive elements 16j..16j+15 of ONE sub-block (lane t: 16j+4t..+3): the four lanes read
// 32 consecutive bytes of activations, and the sub-block's scale is applied to the sum of its two
// steps in f32 instead of to every code.  Lane t decodes the scale and min of sub-block 4*half+t for
// both rows and hands the scales to the other lanes through the warp's scratch.
template <bool Q5>
__device__ __forceinline__ void half_k45(const uint8_t* blk0, const uint8_t* blk1, int half, uint32_t e0,
                                         const uint8_t* xrow, const uint8_t* sxblk, float* scrw, int g, int t, float (&f)[4]) {
    constexpr int QS = Q5 ? 48 : 16;
    const int sb = 4 * half + t;
    const uint4 h0 = *reinterpret_cast<const uint4*>(blk0), h1 = *reinterpret_cast<const uint4*>(blk1);
    uint32_t sc0, m0, sc1, m1;
    scale_min_k4(sb, h0.y, h0.z, h0.w, sc0, m0);
    scale_min_k4(sb, h1.y, h1.z, h1.w, sc1, m1);
    // codes enter the MMA as f16 subnormals code * 2^-24; Q4_K takes the high nibbles (odd sub-blocks)
    // where they are, i.e. as 16 * code.  d * 2^k * scale is exact in f32.
    const float unit = (!Q5 && (t & 1)) ? 1048576.0f : TWO24;
    const float s0 = f16_bits_to_f32(h0.x & 0xffffu) * unit * static_cast<float>(sc0);
    const float s1 = f16_bits_to_f32(h1.x & 0xffffu) * unit * static_cast<float>(sc1);
    __syncwarp();                                                        // previous reads of scratch done
    *reinterpret_cast<float2*>(scrw + 2 * (8 * t + g)) = make_float2(s0, s1);
    __syncwarp();
    // -dmin * sum_j m_j * Sx_j over the half's four sub-blocks: lane t carries m of ITS sub-block as
    // the integer subnormal on k-column 2t (against the hi part of Sx) and 2t+8 (lo part); the
    // neighbouring columns are zero on the A side.  The panel stores, per block, hi[8] then lo[8] (f16).
    float mn[4];
    mma_new(mn, m0, m1, m0, m1, ld_u16(sxblk + 2 * sb), ld_u16(sxblk + 16 + 2 * sb));
    const float dm0 = f16_bits_to_f32(h0.x >> 16) * TWO24, dm1 = f16_bits_to_f32(h1.x >> 16) * TWO24;
    const uint8_t* q0 = blk0 + QS + 64 * half + 4 * t;
    const uint8_t* q1 = blk1 + QS + 64 * half + 4 * t;
    uint32_t gv0[2] = {0u, 0u}, gv1[2] = {0u, 0u};
    if constexpr (Q5) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            gv0[j] = *reinterpret_cast<const uint32_t*>(blk0 + 16 + 16 * j + 4 * t);
            gv1[j] = *reinterpret_cast<const uint32_t*>(blk1 + 16 + 16 * j + 4 * t);
        }
    }
    const float* sread = scrw + 2 * g;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint32_t w0[2], w1[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            w0[j] = *reinterpret_cast<const uint32_t*>(q0 + 32 * c + 16 * j);
            w1[j] = *reinterpret_cast<const uint32_t*>(q1 + 32 * c + 16 * j);
        }
#pragma unroll
        for (int nib = 0; nib < 2; ++nib) {
            float acc[4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t c0, c1;
                if (nib == 0) {
                    c0 = w0[j] & 0x0F0F0F0Fu;
                    c1 = w1[j] & 0x0F0F0F0Fu;
                } else if constexpr (Q5) {
                    c0 = (w0[j] >> 4) & 0x0F0F0F0Fu;
                    c1 = (w1[j] >> 4) & 0x0F0F0F0Fu;
                } else {
                    c0 = w0[j] & 0xF0F0F0F0u;
                    c1 = w1[j] & 0xF0F0F0F0u;
                }
                if constexpr (Q5) {
                    const int bit = 2 * (2 * half + c) + nib;
                    c0 |= ((gv0[j] >> bit) & 0x01010101u) << 4;
                    c1 |= ((gv1[j] >> bit) & 0x01010101u) << 4;
                }
                const uint2 xv = ld_x4(xrow, e0 + 128 * half + 64 * c + 32 * nib + 16 * j + 4 * t);
                if (j == 0) mma_new(acc, sub01(c0), sub01(c1), sub23(c0), sub23(c1), xv.x, xv.y);
                else mma_acc(acc, sub01(c0), sub01(c1), sub23(c0), sub23(c1), xv.x, xv.y);
            }
            const float2 sc = *reinterpret_cast<const float2*>(sread + 16 * (2 * c + nib));
            f[0] += sc.x * acc[0];
            f[1] += sc.x * acc[1];
            f[2] += sc.y * acc[2];
            f[3] += sc.y * acc[3];
        }
    }
    f[0] -= dm0 * mn[0];
    f[1] -= dm0 * mn[1];
    f[2] -= dm1 * mn[2];
    f[3] -= dm1 * mn[3];
}

// ---- Q6_K: half n (128 elements, sub-blocks 8n..8n+7) of one block of rows g and g+8; every MMA
// step is one 16-element sub-block, so d*scale is applied to each step's result.  ALIGNED: the
// block starts on a 4-byte boundary (even block index), so 32-bit fields load in one instruction.
template <bool ALIGNED>
__device__ __forceinline__ uint32_t ld_w(const uint8_t* p) {
    if constexpr (ALIGNED) return *reinterpret_cast<const uint32_t*>(p);
    else return ld_u32_a2(p);
}
// converts this lane's two scales (sub-blocks 8n+2t, 8n+2t+1) of one row, publishes d*2^24*scale
// to the row's scratch line and returns the exact f16x2 scales for the bias MMA
__device__ __forceinline__ uint32_t q6_scales(const uint8_t* blk, int n, int t, float* scr_row, float& d) {
    const uint32_t packed = ld_u16(blk + 192 + 8 * n + 2 * t) ^ 0x8080u;
    const __half2 off = __half2half2(__ushort_as_half(0x6480));          // 1152 = 1024 + 128
    uint32_t h01 = __byte_perm(packed, 0x64646464u, 0x4140u);
    __half2 s01 = __hsub2(*reinterpret_cast<__half2*>(&h01), off);       // exact signed ints
    d = f16_bits_to_f32(ld_u16(blk + 208));
    const float d24 = d * TWO24;
    *reinterpret_cast<float2*>(scr_row + 2 * t) = make_float2(__low2float(s01) * d24, __high2float(s01) * d24);
    return *reinterpret_cast<uint32_t*>(&s01);
}
template <bool ALIGNED>
__device__ __forceinline__ void q6_codes(const uint8_t* blk, int n, int h, int t, uint32_t (&q)[4]) {
    const uint32_t qa = ld_w<ALIGNED>(blk + 64 * n + 16 * h + 4 * t);
    const uint32_t qb = ld_w<ALIGNED>(blk + 64 * n + 32 + 16 * h + 4 * t);
    const uint32_t qh = ld_w<ALIGNED>(blk + 128 + 32 * n + 16 * h + 4 * t);
    q[0] = (qa & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u);
    q[1] = (qb & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u);
    q[2] = ((qa >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u);
    q[3] = ((qb >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u);
}
template <bool ALIGNED>
__device__ __forceinline__ void half_q6k(const uint8_t* blk0, const uint8_t* blk1, int n, uint32_t e0,
                                         const uint8_t* xrow, const uint8_t* sxblk, float* scr0, float* scr1,
                                         int t, float (&f)[4]) {
    float d0, d1;
    __syncwarp();                                                        // previous reads of scratch done
    const uint32_t sa0 = q6_scales(blk0, n, t, scr0, d0);
    const uint32_t sa1 = q6_scales(blk1, n, t, scr1, d1);
    __syncwarp();
    float sc0[8], sc1[8];
    {
        const float4 a = *reinterpret_cast<const float4*>(scr0), b = *reinterpret_cast<const float4*>(scr0 + 4);
        sc0[0] = a.x; sc0[1] = a.y; sc0[2] = a.z; sc0[3] = a.w; sc0[4] = b.x; sc0[5] = b.y; sc0[6] = b.z; sc0[7] = b.w;
        const float4 c = *reinterpret_cast<const float4*>(scr1), e = *reinterpret_cast<const float4*>(scr1 + 4);
        sc1[0] = c.x; sc1[1] = c.y; sc1[2] = c.z; sc1[3] = c.w; sc1[4] = e.x; sc1[5] = e.y; sc1[6] = e.z; sc1[7] = e.w;
    }
    // bias: sum_s sc_s * Sx_s (hi on k-columns 2t,2t+1; lo on 2t+8,2t+9), later scaled by -32 d.
    // The panel stores, per block, hi[16] then lo[16] (f16).
    float bias[4];
    mma_new(bias, sa0, sa1, sa0, sa1, *reinterpret_cast<const uint32_t*>(sxblk + 16 * n + 4 * t),
            *reinterpret_cast<const uint32_t*>(sxblk + 32 + 16 * n + 4 * t));
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t q0[4], q1[4];
        q6_codes<ALIGNED>(blk0, n, h, t, q0);
        q6_codes<ALIGNED>(blk1, n, h, t, q1);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint2 xv = ld_x4(xrow, e0 + 128 * n + 32 * k + 16 * h + 4 * t);
            float c[4];
            mma_new(c, sub01(q0[k]), sub01(q1[k]), sub23(q0[k]), sub23(q1[k]), xv.x, xv.y);
            f[0] += sc0[2 * k + h] * c[0];
            f[1] += sc0[2 * k + h] * c[1];
            f[2] += sc1[2 * k + h] * c[2];
            f[3] += sc1[2 * k + h] * c[3];
        }
    }
    f[0] -= 32.0f * d0 * bias[0];
    f[1] -= 32.0f * d0 * bias[1];
    f[2] -= 32.0f * d1 * bias[2];
    f[3] -= 32.0f * d1 * bias[3];
}

// ---- Q4_0 / Q8_0: four 32-element blocks of rows g and g+8; two MMA steps per block ----
template <bool Q8>
__device__ __forceinline__ void legacy_codes(const uint8_t* blk, int t, uint32_t& w0, uint32_t& w1) {
    if constexpr (Q8) {
        w0 = ld_u32_a2(blk + 2 + 8 * t) ^ 0x80808080u;      // code + 128, elements 8t..8t+3
        w1 = ld_u32_a2(blk + 6 + 8 * t) ^ 0x80808080u;      // elements 8t+4..8t+7
    } else {
        const uint32_t w = ld_u32_a2(blk + 2 + 4 * t);
        w0 = w & 0x0F0F0F0Fu;                                // elements 4t..4t+3
        w1 = (w >> 4) & 0x0F0F0F0Fu;                         // elements 16+4t..
    }
}
template <bool Q8>
__device__ __forceinline__ void half_legacy(const uint8_t* p0, const uint8_t* p1, uint32_t e0,
                                            const uint8_t* xrow, const float* sxf, int t, float (&f)[4]) {
    constexpr int BB = Q8 ? 34 : 18;
    constexpr float BIAS = Q8 ? 128.0f : 8.0f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const uint8_t* blk0 = p0 + b * BB;
        const uint8_t* blk1 = p1 + b * BB;
        const uint32_t e = e0 + 32 * b;
        const float d0 = f16_bits_to_f32(ld_u16(blk0)), d1 = f16_bits_to_f32(ld_u16(blk1));
        uint32_t u0, u1, v0, v1;
        legacy_codes<Q8>(blk0, t, u0, u1);
        legacy_codes<Q8>(blk1, t, v0, v1);
        const uint32_t ea = Q8 ? e + 8 * t : e + 4 * t, eb = Q8 ? ea + 4 : ea + 16;
        const uint2 xa = ld_x4(xrow, ea), xb = ld_x4(xrow, eb);
        float c[4];
        mma_new(c, sub01(u0), sub01(v0), sub23(u0), sub23(v0), xa.x, xa.y);
        mma_acc(c, sub01(u1), sub01(v1), sub23(u1), sub23(v1), xb.x, xb.y);
        const float2 sx = *reinterpret_cast<const float2*>(sxf + (e >> 5) * 8 + 2 * t);
        f[0] += d0 * (TWO24 * c[0] - BIAS * sx.x);
        f[1] += d0 * (TWO24 * c[1] - BIAS * sx.y);
        f[2] += d1 * (TWO24 * c[2] - BIAS * sx.x);
        f[3] += d1 * (TWO24 * c[3] - BIAS * sx.y);
    }
}

// Builds the f16 activation panel of elements [k0, k0 + klen) and its sub-block sums; called by
// all CTH consumer threads.  A thread converts 8 consecutive elements (one 16-byte store) of up
// to U columns per round; lanes holding the same sub-block combine their sums by shuffle (a warp's
// 32 threads cover 256 consecutive elements).  f32 input yields two columns per activation row:
// hi = f16(x) and lo = f16(x - hi).  Values beyond the f16 range are clamped and flagged.
// INPLACE (bf16 input, used by the k-phase variant, whose main loop leaves no registers for loads in
// flight): the raw rows are bulk-copied into the panel's own place and converted there.
template <uint32_t TYPE, int CTH, int U, bool INPLACE, bool NORM>
__device__ __forceinline__ void build_panel(const void* x, bool x_bf16, uint32_t nslots, uint32_t k, uint32_t xpitch,
                                         uint32_t* status, uint8_t* xh, uint8_t* sxp, uint32_t sx_slot_bytes,
                                         uint32_t xrow_idx, uint32_t k0, uint32_t klen, uint64_t* xbar, uint32_t xparity,
                                         const float* norm_w, float norm_eps, float* nscratch) {
    constexpr bool K45 = TYPE == HF2Q_TYPE_Q4_K || TYPE == HF2Q_TYPE_Q5_K;
    constexpr bool LEG = TYPE == HF2Q_TYPE_Q4_0 || TYPE == HF2Q_TYPE_Q8_0;
    constexpr uint32_t SXB = K45 ? 32 : 64;
    constexpr uint32_t SUB = LEG ? 32 : (K45 ? 32 : 16);      // elements per sub-block sum
    constexpr uint32_t PER = 256 / SUB;
    const uint32_t ctid = threadIdx.x, lane = threadIdx.x & 31;
    const uint32_t k8 = klen >> 3;
    uint32_t clipped = 0;
    const __half2 lim = __half2half2(__ushort_as_half(0x7BFF));          // 65504
    // f16x2 from two floats, clamped to the finite range; flags a change; adds the values to acc
    auto pack = [&](float a, float b, float& acc) -> __half2 {
        const __half2 raw = __floats2half2_rn(a, b);
        const __half2 h = __hmin2(__hmax2(raw, __hneg2(lim)), lim);
        clipped |= *reinterpret_cast<const uint32_t*>(&raw) ^ *reinterpret_cast<const uint32_t*>(&h);
        const float2 f = __half22float2(h);
        acc += f.x + f.y;
        return h;
    };
    auto store = [&](uint32_t s, uint32_t pos, const __half2 (&h)[4], float acc) {
        *reinterpret_cast<uint4*>(xh + s * xpitch + 16 * pos) =
            make_uint4(*reinterpret_cast<const uint32_t*>(&h[0]), *reinterpret_cast<const uint32_t*>(&h[1]),
                       *reinterpret_cast<const uint32_t*>(&h[2]), *reinterpret_cast<const uint32_t*>(&h[3]));
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        if constexpr (SUB == 32) acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if ((lane & (SUB / 8 - 1)) == 0) {
            const uint32_t j = (8 * pos) / SUB;
            if constexpr (LEG) {
                reinterpret_cast<float*>(sxp)[j * 8 + s] = acc;
            } else {
                const __half hi = __float2half_rn(acc);
                const __half lo = __float2half_rn(acc - __half2float(hi));
                __half* dst = reinterpret_cast<__half*>(sxp + s * sx_slot_bytes + (j / PER) * SXB);
                dst[j % PER] = hi;
                dst[PER + j % PER] = lo;
            }
        }
    };
    // bf16 -> f16 is exact inside the f16 normal range, so the sub-block sums are taken from the f32
    // values; out-of-range values are clamped, and noticed through a running maximum of |raw f16|
    __half2 seen = __float2half2_rn(0.f);
    auto convert_bf16 = [&](const uint4& r, uint32_t s, uint32_t pos) {
        const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
        __half2 h[4];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = __uint_as_float(rr[j] << 16), b = __uint_as_float(rr[j] & 0xffff0000u);
            const __half2 raw = __floats2half2_rn(a, b);
            seen = __hmax2(seen, __habs2(raw));
            h[j] = __hmin2(__hmax2(raw, __hneg2(lim)), lim);
            acc += a + b;
        }
        store(s, pos, h, acc);
    };
    // k8 is a multiple of 32, so a warp is either wholly inside or wholly outside the loops.
    // bf16 input: SU columns x PU positions are loaded before any is converted.
    auto bf16_rounds = [&](auto su_c, auto pu_c) {
        constexpr int SU = decltype(su_c)::value, PU = decltype(pu_c)::value;
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(x) + static_cast<size_t>(xrow_idx) * k + k0;
        asm volatile("griddepcontrol.wait;" ::: "memory");               // x may be an earlier kernel's output
        for (uint32_t pos0 = ctid; pos0 < k8; pos0 += PU * CTH) {
            for (uint32_t s0 = 0; s0 < nslots; s0 += SU) {
                uint4 ra[SU * PU];
#pragma unroll
                for (int a = 0; a < SU; ++a)
#pragma unroll
                    for (int b = 0; b < PU; ++b)
                        if (s0 + a < nslots && pos0 + b * CTH < k8)
                            ra[a * PU + b] = __ldcg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(s0 + a) * k + 8 * (pos0 + b * CTH)));
#pragma unroll
                for (int a = 0; a < SU; ++a)
#pragma unroll
                    for (int b = 0; b < PU; ++b)
                        if (s0 + a < nslots && pos0 + b * CTH < k8) convert_bf16(ra[a * PU + b], s0 + a, pos0 + b * CTH);
            }
        }
    };
    if (x_bf16 && INPLACE) {
        // bf16 and f16 are both two bytes: the raw rows are bulk-copied into the panel's own place
        // (one asynchronous copy per column, all in flight at once) and converted there
        asm volatile("griddepcontrol.wait;" ::: "memory");               // x may be an earlier kernel's output
        if (ctid < nslots) {
            if (ctid == 0) mbar_arrive_expect_tx(xbar, nslots * klen * 2);
            __syncwarp(__activemask());
            // x may have been written by other GPUs' plain stores that this CTA only ordered through an
            // acquire load and a barrier: make the asynchronous copy below observe them as well
            asm volatile("fence.proxy.async;" ::: "memory");
            bulk_g2s(xh + ctid * xpitch, static_cast<const __nv_bfloat16*>(x) + (static_cast<size_t>(xrow_idx) + ctid) * k + k0, klen * 2, xbar);
        }
        if (!mbar_wait_bounded(xbar, xparity, status)) return;
        for (uint32_t pos = ctid; pos < k8; pos += CTH)
            for (uint32_t sl = 0; sl < nslots; ++sl) {
                convert_bf16(*reinterpret_cast<const uint4*>(xh + sl * xpitch + 16 * pos), sl, pos);
            }
    } else if (x_bf16) {
        if constexpr (U >= 8) {
            if (k8 <= CTH) bf16_rounds(std::integral_constant<int, 8>{}, std::integral_constant<int, 1>{});
            else if (NORM && nslots > 2) bf16_rounds(std::integral_constant<int, 4>{}, std::integral_constant<int, 2>{});
            else bf16_rounds(std::integral_constant<int, 2>{}, std::integral_constant<int, 4>{});       // (the plain variants carry one long-row form only)
        } else {
            bf16_rounds(std::integral_constant<int, U>{}, std::integral_constant<int, 1>{});
        }
    } else if (NORM && norm_w) {
        // f32 input with the RMSNorm in front of the product fused in (rms_norm_rows, forward_cpu.rs:36-48:
        // x * rsqrt(mean(x^2) + eps) * weight).  The whole row is resident (k <= 8 * CTH, one chunk of eight
        // elements per thread and activation row, at most four rows): sums of squares per row across the
        // consumer threads, then scale, split into hi + lo halves and store as below.
        asm volatile("griddepcontrol.wait;" ::: "memory");               // x may be an earlier kernel's output
        const uint32_t ntok = nslots >> 1, pos = ctid;
        const bool have = pos < k8;
        float v[4][8], ss[4] = {0.f, 0.f, 0.f, 0.f};
        const float* src = static_cast<const float*>(x) + static_cast<size_t>(xrow_idx) * k + 8 * pos;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            if (static_cast<uint32_t>(t) < ntok && have) {
                const float4* q = reinterpret_cast<const float4*>(src + static_cast<size_t>(t) * k);
                const float4 a = __ldcg(q), b = __ldcg(q + 1);
                v[t][0] = a.x; v[t][1] = a.y; v[t][2] = a.z; v[t][3] = a.w; v[t][4] = b.x; v[t][5] = b.y; v[t][6] = b.z; v[t][7] = b.w;
#pragma unroll
                for (int j = 0; j < 8; ++j) ss[t] += v[t][j] * v[t][j];
            }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t)
            for (int o = 16; o > 0; o >>= 1) ss[t] += __shfl_xor_sync(0xffffffffu, ss[t], o);
        if (lane == 0)
#pragma unroll
            for (int t = 0; t < 4; ++t) nscratch[(ctid >> 5) * 4 + t] = ss[t];
        asm volatile("bar.sync 1, %0;" ::"n"(CTH));
        float inv[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            float tot = 0.f;
            for (int w = 0; w < CTH / 32; ++w) tot += nscratch[w * 4 + t];
            inv[t] = 1.0f / sqrtf(tot / static_cast<float>(klen) + norm_eps);
        }
        if (have) {                                                      // (k8 is a multiple of 32: whole warps)
            const float4 wa = __ldg(reinterpret_cast<const float4*>(norm_w + 8 * pos)), wb = __ldg(reinterpret_cast<const float4*>(norm_w + 8 * pos) + 1);
            const float w8[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
            for (uint32_t t = 0; t < ntok; ++t) {
                __half2 hi[4], lo[4];
                float acc_hi = 0.f, acc_lo = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float ra = v[t][2 * j] * inv[t] * w8[2 * j], rb = v[t][2 * j + 1] * inv[t] * w8[2 * j + 1];
                    const float a = fminf(fmaxf(ra, -65504.0f), 65504.0f), b = fminf(fmaxf(rb, -65504.0f), 65504.0f);
                    clipped |= static_cast<uint32_t>(!(a == ra)) | static_cast<uint32_t>(!(b == rb));
                    hi[j] = pack(a, b, acc_hi);
                    const float2 f = __half22float2(hi[j]);
                    lo[j] = pack(a - f.x, b - f.y, acc_lo);
                }
                store(2 * t, pos, hi, acc_hi);
                store(2 * t + 1, pos, lo, acc_lo);
            }
        }
    } else {
    asm volatile("griddepcontrol.wait;" ::: "memory");                   // x may be an earlier kernel's output
    for (uint32_t pos = ctid; pos < k8; pos += CTH) {
        {
            constexpr int UT = U > 4 ? 4 : (U > 1 ? U / 2 : 1);      // activation rows per round (two float4 each)
            const float* src = static_cast<const float*>(x) + static_cast<size_t>(xrow_idx) * k + k0 + 8 * pos;
            const uint32_t ntok = nslots >> 1;
            for (uint32_t t0 = 0; t0 < ntok; t0 += UT) {
                float4 ra[UT], rb[UT];
#pragma unroll
                for (int u = 0; u < UT; ++u)
                    if (t0 + u < ntok) {
                        const float4* q = reinterpret_cast<const float4*>(src + static_cast<size_t>(t0 + u) * k);
                        ra[u] = __ldcg(q);
                        rb[u] = __ldcg(q + 1);
                    }
#pragma unroll
                for (int u = 0; u < UT; ++u) {
                    if (t0 + u >= ntok) break;
                    const float v[8] = {ra[u].x, ra[u].y, ra[u].z, ra[u].w, rb[u].x, rb[u].y, rb[u].z, rb[u].w};
                    __half2 hi[4], lo[4];
                    float acc_hi = 0.f, acc_lo = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float a = fminf(fmaxf(v[2 * j], -65504.0f), 65504.0f);
                        const float b = fminf(fmaxf(v[2 * j + 1], -65504.0f), 65504.0f);
                        clipped |= static_cast<uint32_t>(a != v[2 * j]) | static_cast<uint32_t>(b != v[2 * j + 1]);
                        hi[j] = pack(a, b, acc_hi);
                        const float2 f = __half22float2(hi[j]);
                        lo[j] = pack(a - f.x, b - f.y, acc_lo);
                    }
                    store(2 * (t0 + u), pos, hi, acc_hi);
                    store(2 * (t0 + u) + 1, pos, lo, acc_lo);
                }
            }
        }
    }
    }
    // (a NaN in `seen` fails the comparison as well)
    if (!(__hle(__low2half(seen), __low2half(lim)) && __hle(__high2half(seen), __low2half(lim)))) clipped = 1;
    if (clipped) atomicOr(status, STATUS_X_CLIPPED);
}

// Warp roles.  Consumer warps form NTEAMS teams of TEAM = 8; ring stage i belongs to team
// i % NTEAMS, whose eight warps each take one 256-element block of the stage for all 16 rows.  So
// NTEAMS stages are being unpacked at any time while the producer warp refills the others.  A
// reducer warp adds the consumers' partial sums of a finished row group (fixed order: bit-
// reproducible) and stores them; the hand-over goes through two mbarrier pairs, so consumers never
// stop at a CTA-wide barrier inside the main loop.
//
// Long rows: the f16 activation panel of all columns must sit in shared memory next to the ring.
// When it does not fit, k is cut into PHASES of whole slices.  The CTA walks all its row groups
// once per phase with only that phase's activations resident, and the reducer adds the phase's
// sums to what the previous phase stored (same thread, same address: ordered, no atomics).  Every
// weight byte is still read exactly once.
// PHASED = false compiles the single-phase case without the phase loop (fewer live registers in
// the main loop); SUBG = false compiles out the stacked row groups of short rows; EXT = false the
// fused all-gather and the routed pair.
template <uint32_t TYPE, int NTEAMS, bool PHASED, bool SUBG, bool EXT>
__global__ void __launch_bounds__((NTEAMS * TEAM + 2) * 32, 1) gemv_mma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                                                                               const MParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool K45 = TYPE == HF2Q_TYPE_Q4_K || TYPE == HF2Q_TYPE_Q5_K;
    constexpr bool Q6 = TYPE == HF2Q_TYPE_Q6_K;
    constexpr bool LEG = TYPE == HF2Q_TYPE_Q4_0 || TYPE == HF2Q_TYPE_Q8_0;
    constexpr BlockGeom G = block_geom(TYPE);
    constexpr int CW = NTEAMS * TEAM;          // consumer warps
    constexpr int CTH = CW * 32;
    // bytes of x-sum panel per 256 elements and column: K45 8 x (hi,lo) f16, Q6 16 x (hi,lo) f16;
    // Q4_0/Q8_0 keep f32 sums for all 8 columns per 32-element block
    constexpr uint32_t SXB = K45 ? 32 : 64;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* red_full = empty + MAX_STAGES;
    uint64_t* red_empty = red_full + 2;
    uint64_t* xbar = red_empty + 2;                    // completion of the activation rows' bulk copies
    uint8_t* ring = smem + 256;
    const uint32_t stages = p.stages, pitch = p.pitch, nslices = p.nslices;
    const uint32_t spp = p.phase_base + (p.phase_rem ? 1u : 0u);              // slices of the longest phase
    // SUBG: a row is one short slice and a stage holds p.sub_groups groups of 16 rows
    const uint32_t nsub = SUBG ? p.sub_groups : 1u, stage_rows = ROWS * nsub;
    const uint32_t stage_bytes = stage_rows * pitch;
    float* red = reinterpret_cast<float*>(ring + stages * stage_bytes);          // [2][CW][16][8]
    float* scr = red + 2 * CW * 128;                                            // [CW][16][8]
    uint8_t* xh = reinterpret_cast<uint8_t*>(scr + CW * 16 * 8);                 // [nslots][xpitch]
    uint8_t* sxp = xh + p.nslots * p.xpitch;
    const uint32_t kphase = min(spp * SLICE_ELEMS, (EXT && p.split) ? static_cast<uint32_t>(SLICE_ELEMS) : p.k);   // elements of k resident at a time
    const uint32_t sx_slot_bytes = (kphase >> 8) * SXB + 16;                    // K45 / Q6 panels; +16: columns 4 banks apart

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t slot = blockIdx.y;
    // split-k: this CTA works on slice `part` of every row of its groups; to the loops below that is a
    // product with one-slice rows whose copies start `part` slices into the row
    const uint32_t part = (EXT && p.split) ? blockIdx.y : 0u;
    if (EXT && p.split) slot = 0;
    const uint32_t kloc = (EXT && p.split) ? (part + 1 == p.split ? p.k_last : static_cast<uint32_t>(SLICE_ELEMS)) : p.k;
    const void* xbase = (EXT && p.split) ? static_cast<const void*>(static_cast<const uint8_t*>(p.x) + static_cast<size_t>(part) * SLICE_ELEMS * (p.x_bf16 ? 2u : 4u))
                                         : p.x;
    const uint8_t* wbase = p.w;
    float* ybase = p.y;
    const uint8_t* wbase2 = EXT ? p.w2 : nullptr;     // fused SwiGLU: the up tensor (of the same expert)
    if (EXT && p.w2 && slot >= p.pair_slots) { slot -= p.pair_slots; wbase = p.w2; ybase = p.y2; }
    uint32_t xrow_idx = 0;
    bool slot_ok = true;
    if (p.ids) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t e = p.ids[slot];
        slot_ok = e < p.n_experts;
        if (!slot_ok && threadIdx.x == 0) atomicOr(p.status, STATUS_BAD_EXPERT_ID);
        wbase += static_cast<uint64_t>(slot_ok ? e : 0) * p.expert_stride;
        if (EXT && p.w2) wbase2 += static_cast<uint64_t>(slot_ok ? e : 0) * p.expert_stride;
        xrow_idx = slot / p.top_k;
    }
    float* yout = ybase + ((EXT && p.split) ? static_cast<size_t>(part) * p.m * p.n : static_cast<size_t>(slot) * p.n);
    // row groups of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
    const uint32_t own = blockIdx.x < p.ngroups ? (p.ngroups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // fused SwiGLU: every row group is walked twice in a row, first in the gate matrix, then in the up matrix
    const bool sw = EXT && p.swiglu;
    const uint32_t gcta = sw ? 2 * own : own;

    // Programmatic dependent launch: let the next kernel of the stream start its own prologue as soon
    // as SMs free up, and do not touch anything an earlier kernel may still be writing (activations,
    // expert ids, outputs) before that kernel has completed.  Weight bytes are immutable, so the
    // producer of a dense launch starts streaming without waiting.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Start-up: the producer warp initialises the ring's barriers itself and issues the first copies
    // at once; the reducer warp initialises the hand-over barriers; the consumers build the
    // activation panel.  One CTA-wide barrier then publishes all of that to everyone.
    if (warp == CW) {
        // ---------------- producer warp: lane r copies row r of each stage ----------------
        if (lane == 0) {
            for (uint32_t i = 0; i < stages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], TEAM); }
            mbar_fence_init();
        }
        __syncwarp();
        bool synced = false;
        if (slot_ok) {
            // weight bytes are read once per launch: first in line for eviction, so that streaming them
            // leaves activations and outputs (which the next launches re-read) in L2
            const uint64_t wpolicy = p.w_evict_first ? l2_policy_evict_first() : l2_policy_evict_normal();
            uint32_t it = 0, st = 0, ph = 1;      // ring slot and the parity of its previous use
            for (uint32_t s0 = 0, pi = 0; s0 < nslices; ++pi) {
                const uint32_t s1 = s0 + p.phase_base + (pi < p.phase_rem ? 1u : 0u);
                for (uint32_t gi = 0; gi < gcta; ++gi) {
                    const uint32_t rg = blockIdx.x + (sw ? gi >> 1 : gi) * gridDim.x;
                    const bool second = sw && (gi & 1u);
                    const uint8_t* wsrc = second ? wbase2 : wbase;
                    const CUtensorMap* tmap = second ? &tmap_w2 : &tmap_w;
                    const uint32_t row0 = rg * stage_rows;
                    const uint32_t nrows = min(stage_rows, p.n - row0);
                    for (uint32_t s = s0; s < s1; ++s, ++it, st = (st + 1 == stages ? 0 : st + 1), ph ^= (st == 0)) {
                        // The copies of the first stage are on their way: tell the other warps that the
                        // ring's barriers exist, WITHOUT waiting for them -- the consumers may sit in
                        // their dependency wait for microseconds, which is when the ring should fill.
                        if (it == 1) { cta_arrive_n<(NTEAMS * TEAM + 2) * 32>(); synced = true; }
                        // Ahead of the previous kernel's completion only PRE_STAGES stages are requested:
                        // enough for both teams to start at once, while a whole ring per CTA, requested
                        // by the CTAs that start last, was measured to delay the completion itself (and
                        // with it every CTA's activation panel) by ~1.4 us on long launches.  The wait also
                        // means that the bounded waits below only ever measure this kernel's own consumers.
                        if (it == PRE_STAGES) asm volatile("griddepcontrol.wait;" ::: "memory");
                        if (it >= stages) {
                            bool alive = mbar_wait_bounded(&empty[st], ph, p.status);
                            alive = __all_sync(0xffffffffu, alive);
                            if (!alive) return;
                        }
                        const uint32_t off = (s + part) * p.slice_bytes;
                        const uint32_t bytes = min(p.slice_bytes, p.row_bytes - off);
                        if (p.use_tmap) {
                            // one tensor copy for the whole stage: the copy engine spends ~15 cycles per copy
                            // descriptor, which 16 per-row copies per stage made 15 % of the streaming time.
                            // Rows past n and bytes past the row end are zero-filled and count as transferred.
                            if (lane == 0) {
                                mbar_arrive_expect_tx(&full[st], stage_bytes);
                                asm volatile(
                                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
                                    ::"r"(smem_u32(ring + st * stage_bytes)), "l"(reinterpret_cast<uint64_t>(tmap)),
                                      "r"(static_cast<int>((s + part) * (p.slice_bytes >> 3))), "r"(static_cast<int>(row0)), "r"(smem_u32(&full[st])),
                                      "l"(wpolicy)
                                    : "memory");
                            }
                            continue;
                        }
                        if (lane == 0) mbar_arrive_expect_tx(&full[st], nrows * bytes);
                        __syncwarp();
                        if (p.dense_stage) {
                            // whole rows, contiguous in memory and in the stage: one copy
                            if (lane == 0)
                                bulk_g2s_hint(ring + st * stage_bytes, wsrc + static_cast<uint64_t>(row0) * p.row_bytes, nrows * bytes, &full[st], wpolicy);
                        } else {
                            for (uint32_t rr = lane; rr < nrows; rr += 32)
                                bulk_g2s_hint(ring + st * stage_bytes + rr * pitch,
                                              wsrc + static_cast<uint64_t>(row0 + rr) * p.row_bytes + off, bytes, &full[st], wpolicy);
                        }
                    }
                }
                s0 = s1;
            }
        }
        if (!synced) cta_arrive_n<(NTEAMS * TEAM + 2) * 32>();
        return;
    }
    if (warp == CW + 1) {
        // ---------------- reducer warp: lane sums outputs 4*lane .. 4*lane+3 of the [16 rows][8 columns]
        // tile (row lane/2, columns 4*(lane%2)..+3) over the teams that worked on the group, in team order
        const uint32_t nteams = nslices < NTEAMS ? nslices : NTEAMS;      // every phase has at least NTEAMS slices
        if (lane == 0) {                                                  // unless the whole row has fewer
            for (int i = 0; i < 2; ++i) { mbar_init(&red_full[i], nteams * TEAM); mbar_init(&red_empty[i], 1); }
            mbar_fence_init();
        }
        cta_sync_n<(NTEAMS * TEAM + 2) * 32>();
        if (!slot_ok) return;
        asm volatile("griddepcontrol.wait;" ::: "memory");                // before the first store to y
        uint32_t fl = 0, first = 0;                   // flush counter; team of the group's first stage
        float gate[4] = {0.f, 0.f, 0.f, 0.f};         // fused SwiGLU: the gate sums wait here for the up sums
        for (uint32_t s0 = 0, pi = 0; s0 < nslices; ++pi) {
            const uint32_t nsp = p.phase_base + (pi < p.phase_rem ? 1u : 0u);
            for (uint32_t gi = 0; gi < gcta; ++gi, ++fl, first = (first + nsp) % NTEAMS) {
                const uint32_t rg = blockIdx.x + (sw ? gi >> 1 : gi) * gridDim.x;
                const bool second = sw && (gi & 1u);
                const uint32_t rs = fl & 1;
                if (!mbar_wait_bounded(&red_full[rs], (fl >> 1) & 1, p.status)) return;
                // partial sums sit at [team][block of the stage]; a sub-group's blocks are adjacent
                const uint32_t nb = nsub > 1 ? p.last_nblk : static_cast<uint32_t>(TEAM);
                for (uint32_t sg = 0; sg < nsub; ++sg) {
                    float v[4] = {0.f, 0.f, 0.f, 0.f};
                    for (uint32_t i = 0, tm = first; i < nteams; ++i, tm = (tm + 1 == NTEAMS ? 0 : tm + 1)) {
                        const float4* rbuf = reinterpret_cast<const float4*>(red + (rs * CW + tm * TEAM + sg * nb) * 128) + lane;
                        if (nsub == 1) {
#pragma unroll
                            for (int w = 0; w < TEAM; ++w) {
                                const float4 a = rbuf[w * 32];
                                v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
                            }
                        } else {
                            for (uint32_t w = 0; w < nb; ++w) {
                                const float4 a = rbuf[w * 32];
                                v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
                            }
                        }
                    }
                    if (sg + 1 == nsub) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&red_empty[rs]);
                    }
                    const uint32_t row = rg * stage_rows + sg * ROWS + (lane >> 1);
                    if (!p.x_bf16) {                                         // (hi, lo) column pairs
                        v[0] += v[1];
                        v[1] = v[2] + v[3];
                    }
                    const uint32_t ncol = p.x_bf16 ? 4u : 2u, tok0 = (lane & 1u) * ncol;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t tok = tok0 + j;
                        const float out = v[j];
                        if (static_cast<uint32_t>(j) < ncol && row < p.n && tok < p.m) {
                            if (EXT && sw) {
                                if (!second) gate[j] = out;
                                else yout[static_cast<size_t>(tok) * p.n + row] = gate[j] / (1.0f + expf(-gate[j])) * out;
                            } else if (!EXT || p.g_nranks == 0) {
                                float* dst = yout + static_cast<size_t>(tok) * p.n + row;
                                float o = out;
                                if (s0 == 0 && p.residual) o += p.residual[static_cast<size_t>(slot) * p.n + static_cast<size_t>(tok) * p.n + row];
                                *dst = s0 ? *dst + o : o;
                            } else {
                                // the own buffer accumulates the phases; the last phase's total goes to every rank
                                const size_t off = static_cast<size_t>(tok) * p.g_ntotal + p.g_col0 + row;
                                float* own = p.g_y[p.g_rank] + off;
                                const float total = s0 ? *own + out : out;
                                *own = total;
                                if (s0 + nsp == nslices)
                                    for (uint32_t r = 0; r < p.g_nranks; ++r)
                                        if (r != p.g_rank) p.g_y[r][off] = total;
                            }
                        }
                    }
                }
            }
            s0 += nsp;
        }
        if (EXT && p.g_nranks > 1) {
            // Tell the other ranks that this CTA's part of the columns has landed.  Rank r's counter
            // block holds one arrival counter per SOURCE rank (words 0..7) and, next to it, how many
            // arrivals the products launched HERE so far stand for from each source (words 8..15):
            // a source's columns of every earlier product are complete once its counter has caught up,
            // whatever the other sources have delivered and however many CTAs each rank's shard needs.
            __syncwarp();
            if (lane == 0) {
                if (blockIdx.x == 0 && blockIdx.y == 0)
                    for (uint32_t r = 0; r < p.g_nranks; ++r)
                        if (r != p.g_rank) atomicAdd(p.g_flag[p.g_rank] + 8 + r, p.g_peer_ctas[r]);
                // Release at system scope: the adds become visible after this warp's stores (the warp
                // barrier above makes it cover all lanes' stores).  ONE fence and then relaxed adds, so
                // that the wait for the stores' acknowledgement is paid once and not once per peer.
                asm volatile("fence.acq_rel.sys;" ::: "memory");
                for (uint32_t r = 0; r < p.g_nranks; ++r)
                    if (r != p.g_rank)
                        asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(p.g_flag[r] + p.g_rank) : "memory");
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int ctid = threadIdx.x;
    // Ahead of the dependency wait: ask for the activations' lines (and their address translation).
    // A prefetch returns no data, so it may run while the previous kernel is still writing them.
    if (!p.ids && !(EXT && p.split)) {
        const uint32_t xbytes = p.k * (p.x_bf16 ? 2u : 4u), m_rows = p.x_bf16 ? p.nslots : p.nslots >> 1;
        for (uint32_t off = static_cast<uint32_t>(ctid) * 128u; off < m_rows * xbytes; off += CTH * 128u)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const uint8_t*>(p.x) + off));
    }
    // (the consumers' dependency wait sits inside build_panel, directly in front of the first load of
    // the activations: everything up to there is set-up that does not touch what an earlier kernel writes)
    if constexpr (PHASED) {
        if (ctid == 0) { mbar_init(xbar, 1); mbar_fence_init(); }
        asm volatile("bar.sync 1, %0;" ::"n"(CTH));
    }
    if (!slot_ok) {
        asm volatile("griddepcontrol.wait;" ::: "memory");                // before writing y
        cta_sync_n<(NTEAMS * TEAM + 2) * 32>();
        for (uint32_t r = ctid; r < p.n; r += CTH) yout[r] = 0.f;
        return;
    }

    // Lane (g, t): weight rows g and g+8, MMA column g.  Columns beyond nslots alias column 0: a
    // column of the product depends only on its own column of B, and those outputs are never stored.
    const int g = lane >> 2, t = lane & 3;
    const uint32_t col = static_cast<uint32_t>(g) < p.nslots ? g : 0;
    const uint8_t* xrow = xh + col * p.xpitch;
    const uint8_t* sxslot = sxp + col * sx_slot_bytes;
    float* scr0 = scr + (warp * 16 + g) * 8;
    float* scr1 = scr0 + 64;
    (void)scr0; (void)scr1; (void)sxslot;
    const uint32_t team = static_cast<uint32_t>(warp) / TEAM;
    const uint8_t* ring_g = ring + g * pitch;                            // this lane's first row in slot 0
    float* red_t = red + team * (TEAM * 128) + g * 8 + 2 * t;              // + block * 128: this team's partial sums
    const uint32_t last_slice = nslices - 1, last_nblk = (EXT && p.split) ? kloc >> 8 : p.last_nblk;
    uint32_t blk = static_cast<uint32_t>(warp) % TEAM;                   // block of the stage this warp takes; rotates
    uint32_t fl_base = 0;                                                // flushes of earlier phases

    for (uint32_t s0 = 0, pi = 0, nsp = 0; s0 < (PHASED ? nslices : 1u); s0 += nsp, ++pi, fl_base += gcta) {
        nsp = PHASED ? p.phase_base + (pi < p.phase_rem ? 1u : 0u) : nslices;     // slices of this phase
        if (PHASED && s0) asm volatile("bar.sync 1, %0;" ::"n"(CTH));    // everyone is done with the previous panel
        const uint32_t k0 = s0 * SLICE_ELEMS;
        if (EXT && s0 == 0 && p.g_wait) {
            // the activations are another product's gathered output: wait until every rank's part of
            // it has arrived here (bounded; the peers' kernels run on other GPUs)
            asm volatile("griddepcontrol.wait;" ::: "memory");            // the counters belong to earlier kernels too
            if (static_cast<uint32_t>(ctid) < p.g_nranks && static_cast<uint32_t>(ctid) != p.g_rank)
                gather_wait_source(p.g_flag[p.g_rank], ctid, p.wait_limit, p.status);
            asm volatile("bar.sync 1, %0;" ::"n"(CTH));
        }
        build_panel<TYPE, CTH, (PHASED ? 2 : 8), PHASED, EXT>(xbase, p.x_bf16 != 0, p.nslots, p.kx, p.xpitch, p.status, xh, sxp, sx_slot_bytes, xrow_idx, k0,
                               min(nsp * SLICE_ELEMS, kloc - k0), xbar, pi & 1u, p.norm_w, p.norm_eps, scr);
        if (s0 == 0) cta_sync_n<(NTEAMS * TEAM + 2) * 32>();             // panel + all barrier initialisations
        else asm volatile("bar.sync 1, %0;" ::"n"(CTH));

        // Stages of this phase are numbered it0 .. it0 + gcta * nsp - 1 (group-major); this team
        // owns those with index = team (mod NTEAMS); stage i sits in ring slot i % stages.  (No
        // divisions in the common cases: their latency sits between the panel barrier and the
        // first block.)
        const uint32_t it0 = gcta * s0;
        const uint32_t rel = (team + NTEAMS - it0 % NTEAMS) % NTEAMS;    // first own stage, relative to it0
        uint32_t grp, s, st, ph, step_s, step_g;
        if constexpr (NTEAMS == 2) {                                     // rel is 0 or 1
            const bool one = nsp == 1;
            grp = one ? rel : 0u;
            s = one ? 0u : rel;
        } else {
            grp = rel / nsp; s = rel - grp * nsp;
        }
        step_s = NTEAMS % nsp; step_g = NTEAMS / nsp;
        if constexpr (PHASED) {
            st = (it0 + rel) % stages; ph = ((it0 + rel) / stages) & 1u;
        } else {                                                         // it0 = 0 and rel < NTEAMS <= 2 * stages
            const bool wrap = rel >= stages;
            st = wrap ? rel - stages : rel;
            ph = wrap ? 1u : 0u;
        }
        float f[4] = {0.f, 0.f, 0.f, 0.f};
        while (grp < gcta) {
            if (!mbar_wait_bounded(&full[st], ph, p.status)) return;
            // the block a warp takes rotates, so that the slower unaligned (odd) Q6_K blocks and the
            // idle turns of a short last slice spread evenly over the team
            blk = (blk + 1) & (TEAM - 1);
            // short rows: the stage holds nsub groups of 16 rows and `blk` counts (group, block) pairs
            const uint32_t sgi = nsub > 1 ? blk / last_nblk : 0u, bb = nsub > 1 ? blk - sgi * last_nblk : blk;
            const uint32_t nblk = nsub > 1 ? nsub * last_nblk : (s0 + s == last_slice ? last_nblk : static_cast<uint32_t>(TEAM));
            if (blk < nblk) {
                const uint8_t* r0 = ring_g + st * stage_bytes + sgi * (ROWS * pitch);
                const uint8_t* r1 = r0 + 8 * pitch;
                const uint32_t e0 = s * SLICE_ELEMS + 256 * bb;           // element index inside the panel
                if constexpr (K45) {
                    const uint8_t* b0 = r0 + bb * G.bytes;
                    const uint8_t* b1 = r1 + bb * G.bytes;
                    const uint8_t* sx = sxslot + (e0 >> 8) * SXB;
                    half_k45<TYPE == HF2Q_TYPE_Q5_K>(b0, b1, 0, e0, xrow, sx, scr0 - 8 * g, g, t, f);
                    half_k45<TYPE == HF2Q_TYPE_Q5_K>(b0, b1, 1, e0, xrow, sx, scr0 - 8 * g, g, t, f);
                } else if constexpr (Q6) {
                    const uint8_t* b0 = r0 + bb * 210;
                    const uint8_t* b1 = r1 + bb * 210;
                    const uint8_t* sx = sxslot + (e0 >> 8) * SXB;
                    // (the two halves run as a loop: half the code, which the instruction cache likes)
                    if (bb & 1) {
#pragma unroll 1
                        for (int nh = 0; nh < 2; ++nh) half_q6k<false>(b0, b1, nh, e0, xrow, sx, scr0, scr1, t, f);
                    } else {
#pragma unroll 1
                        for (int nh = 0; nh < 2; ++nh) half_q6k<true>(b0, b1, nh, e0, xrow, sx, scr0, scr1, t, f);
                    }
                } else {
#pragma unroll
                    for (uint32_t h = 0; h < 2; ++h)
                        half_legacy<TYPE == HF2Q_TYPE_Q8_0>(r0 + (2 * bb + h) * 4 * G.bytes, r1 + (2 * bb + h) * 4 * G.bytes,
                                                            e0 + 128 * h, xrow, reinterpret_cast<const float*>(sxp), t, f);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
            st += NTEAMS;
            if (st >= stages) { st -= stages; ph ^= 1u; }
            s += step_s;
            uint32_t dg = step_g;
            if (s >= nsp) { s -= nsp; ++dg; }
            if (dg) {
                // that was this team's last stage of the group: hand the partial sums to the reducer
                const uint32_t fl = fl_base + grp, rs = fl & 1;
                if (fl >= 2 && !mbar_wait_bounded(&red_empty[rs], ((fl >> 1) - 1) & 1, p.status)) return;
                float* rb = red_t + rs * (CW * 128) + blk * 128;
                *reinterpret_cast<float2*>(rb) = make_float2(f[0], f[1]);
                *reinterpret_cast<float2*>(rb + 64) = make_float2(f[2], f[3]);
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_full[rs]);
                f[0] = f[1] = f[2] = f[3] = 0.f;
                grp += dg;
            }
        }
    }
}

// shared memory that does not depend on the ring depth; kphase = elements of k resident at a time
size_t smem_base_bytes(uint32_t type, uint32_t kphase, uint32_t nslots, int teams) {
    const bool k45 = type == HF2Q_TYPE_Q4_K || type == HF2Q_TYPE_Q5_K;
    const bool leg = type == HF2Q_TYPE_Q4_0 || type == HF2Q_TYPE_Q8_0;
    const size_t cw = static_cast<size_t>(teams) * TEAM;
    const size_t fixed = 256 + (2 * cw * 128 + cw * 16 * 8) * 4;
    const size_t xbytes = static_cast<size_t>(nslots) * (2 * static_cast<size_t>(kphase) + 32);
    const size_t sxbytes = leg ? static_cast<size_t>(kphase / 32) * 8 * 4
                               : static_cast<size_t>(nslots) * ((kphase / 256) * (k45 ? 32 : 64) + 16);
    return fixed + xbytes + sxbytes;
}
// Bytes between rows of a stage: the slice plus 0 or 16 bytes of padding such that consecutive
// rows start 4 banks apart (pitch / 4 = 4 mod 8): lanes (g, t) reading word t of rows g = 0..7 then
// touch 32 different banks.
uint32_t row_pitch(uint32_t slice_bytes) {
    for (uint32_t pad = 0; pad <= 48; pad += 16)
        if (((slice_bytes + pad) / 4) % 8 == 4) return slice_bytes + pad;
    return slice_bytes + 16;
}
// Rows of at most four 256-element blocks would leave most of a team idle (one warp per block), so a
// stage then holds several 16-row groups: 8, 4 or 2 for 1, 2 or 3..4 blocks.
uint32_t sub_groups_of(uint32_t k) {
    const uint32_t nblk = k >> 8;
    return nblk == 1 ? 8u : nblk == 2 ? 4u : nblk <= 4 ? 2u : 1u;
}
// A row that fits one slice can be staged without padding -- the rows of a stage are then one
// contiguous range of memory and arrive with a single bulk copy instead of one per row -- unless that
// pitch puts rows 0 or 16 banks apart (8- and 4-way conflicts on every weight load).
bool dense_stage_ok(uint32_t row_bytes, uint32_t k) {
    const uint32_t words = row_bytes / 4;
    return k <= SLICE_ELEMS && words % 16 != 0;
}
size_t stage_bytes_of(uint32_t type, uint32_t k) {
    const BlockGeom g = block_geom(type);
    uint32_t slice = SLICE_ELEMS / g.elems * g.bytes;
    const uint32_t row = k / g.elems * g.bytes;
    if (slice > row) slice = row;
    const uint32_t pitch = dense_stage_ok(row, k) ? row : row_pitch(slice);
    return static_cast<size_t>(ROWS) * sub_groups_of(k) * pitch;
}

int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

// How k is cut into phases and how deep the ring is, for `teams` consumer teams.
struct Plan {
    uint32_t phase_base = 0, phase_rem = 0, stages = 0;
    size_t smem = 0;
};
// Fewest phases (of nslices / phases slices, the first nslices % phases one longer, none shorter
// than `teams` unless the row is) whose activation panel leaves room for a ring of teams + 2
// stages: each team holds one stage while two are in flight (measured: fewer phases beat a deeper
// ring).  Failing that, teams + 1.
Plan make_plan_uncached(uint32_t type, uint32_t k, uint32_t nslots, int teams, size_t limit) {
    const uint32_t nslices = (k + SLICE_ELEMS - 1) / SLICE_ELEMS;
    const size_t stage = stage_bytes_of(type, k);
    static const uint32_t first_spare = static_cast<uint32_t>(env_int("HF2Q_CUDA_MMA_SPARE", 2));   // tuning aid
    for (uint32_t spare = first_spare; spare >= 1; --spare) {
        for (uint32_t phases = 1; phases <= nslices; ++phases) {
            const uint32_t base = nslices / phases, rem = nslices % phases;
            if (phases > 1 && base < static_cast<uint32_t>(teams)) break;
            const uint32_t longest = base + (rem ? 1 : 0);
            const uint32_t kphase = longest * SLICE_ELEMS < k ? longest * SLICE_ELEMS : k;
            const size_t fixed = smem_base_bytes(type, kphase, nslots, teams);
            if (fixed >= limit) continue;
            size_t s = (limit - fixed) / stage;
            if (s > MAX_STAGES) s = MAX_STAGES;
            if (s >= static_cast<size_t>(teams) + spare) {
                Plan pl;
                pl.phase_base = base;
                pl.phase_rem = rem;
                pl.stages = static_cast<uint32_t>(s);
                pl.smem = fixed + s * stage;
                return pl;
            }
        }
    }
    return Plan{};
}

// The plan depends on five small numbers and is asked for several times per launch: remember it.
Plan make_plan(uint32_t type, uint32_t k, uint32_t nslots, int teams, size_t limit) {
    struct Entry { uint32_t type, k, nslots; int teams; size_t limit; Plan plan; };
    static std::mutex mu;
    static std::vector<Entry> cache;
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry& e : cache)
        if (e.type == type && e.k == k && e.nslots == nslots && e.teams == teams && e.limit == limit) return e.plan;
    const Plan pl = make_plan_uncached(type, k, nslots, teams, limit);
    if (cache.size() >= 256) cache.clear();
    cache.push_back(Entry{type, k, nslots, teams, limit, pl});
    return pl;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// Tensor map over a dense weight matrix viewed as 8-byte elements: box = one stage (16 rows x the
// padded slice).  False if the shape does not fit a box (inner extent > 256 elements: Q8_0).
bool make_stage_map(CUtensorMap* map, const MParams& p, const uint8_t* w) {
    EncodeTiledFn enc = encode_fn();
    if (!enc || p.ids || p.sub_groups > 1 || p.dense_stage || p.pitch % 8 || p.pitch / 8 > 256 || p.slice_bytes % 16 || p.row_bytes % 16) return false;
    static const bool off = [] { const char* v = getenv("HF2Q_CUDA_MMA_TMAP"); return v && v[0] == '0'; }();      // tuning aid
    if (off) return false;
    // Encoding takes about a microsecond of host time and weights stay where they are: remember the
    // maps by (address, geometry).  A map holds nothing but those, so a stale entry cannot be wrong.
    struct Entry { const uint8_t* w; uint32_t row_bytes, n, pitch; CUtensorMap map; };
    static std::mutex mu;
    static std::unordered_map<uint64_t, Entry> cache;
    const uint64_t hkey = reinterpret_cast<uint64_t>(w) ^ (static_cast<uint64_t>(p.n) << 40) ^ (static_cast<uint64_t>(p.pitch) << 52);
    {
        std::lock_guard<std::mutex> lock(mu);
        const auto it = cache.find(hkey);
        if (it != cache.end() && it->second.w == w && it->second.row_bytes == p.row_bytes && it->second.n == p.n && it->second.pitch == p.pitch) {
            *map = it->second.map;
            return true;
        }
    }
    cuuint64_t dims[2] = {p.row_bytes / 8, p.n};
    cuuint64_t strides[1] = {p.row_bytes};
    cuuint32_t box[2] = {p.pitch / 8, ROWS};
    cuuint32_t es[2] = {1, 1};
    if (enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(w), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() >= 8192) cache.clear();
    cache[hkey] = Entry{w, p.row_bytes, p.n, p.pitch, *map};
    return true;
}

template <uint32_t TYPE, int NTEAMS, bool PHASED, bool SUBG, bool EXT>
cudaError_t launch_mma_tt(MParams p, uint32_t slots, const Plan& pl, const DeviceInfo& dev, cudaStream_t st) {
    auto kern = gemv_mma_kernel<TYPE, NTEAMS, PHASED, SUBG, EXT>;
    static PerDeviceFlag smem_attr;
    if (const cudaError_t e = ensure_max_dynamic_smem(kern, dev.max_smem_optin, smem_attr); e != cudaSuccess) return e;
    p.stages = pl.stages;
    p.phase_base = pl.phase_base;
    p.phase_rem = pl.phase_rem;
    const uint32_t longest = pl.phase_base + (pl.phase_rem ? 1 : 0);
    const uint32_t kphase = longest * SLICE_ELEMS < p.k ? longest * SLICE_ELEMS : p.k;
    p.xpitch = 2 * kphase + 32;                   // activation rows land 8 banks apart
    uint32_t gx = (static_cast<uint32_t>(dev.sm_count) + slots - 1) / slots;      // one CTA per SM
    if (p.split) gx = static_cast<uint32_t>(dev.sm_count) / slots;                // split-k: all parts of a group run at the same time
    if (gx > p.ngroups) gx = p.ngroups;
    if (gx < 1) gx = 1;
    static const int pdl = env_int("HF2Q_CUDA_PDL", 1);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(gx, slots);
    cfg.blockDim = dim3((NTEAMS * TEAM + 2) * 32);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    alignas(64) CUtensorMap tmap, tmap2;
    memset(&tmap, 0, sizeof tmap);
    memset(&tmap2, 0, sizeof tmap2);
    static const bool evict_first = env_int("HF2Q_CUDA_MMA_EVICT_FIRST", 1) != 0;      // tuning aid
    p.w_evict_first = evict_first ? 1u : 0u;
    p.use_tmap = make_stage_map(&tmap, p, p.w) && (!p.swiglu || make_stage_map(&tmap2, p, p.w2)) ? 1u : 0u;
    return cudaLaunchKernelEx(&cfg, kern, tmap, tmap2, p);
}

// Adds the split-k parts: y[i] = sum over parts of scratch[part][i] (+ residual[i]), parts in index order.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ scratch, uint32_t parts, uint64_t count,
                                                            const float* __restrict__ residual, float* __restrict__ y) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");                    // the parts are the previous kernel's output
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        float v = __ldcg(scratch + i);
        for (uint32_t pt = 1; pt < parts; ++pt) v += __ldcg(scratch + pt * count + i);
        if (residual) v += residual[i];
        y[i] = v;
    }
}

cudaError_t launch_splitk_reduce(const float* scratch, uint32_t parts, uint64_t count, const float* residual, float* y, const DeviceInfo& dev,
                                 cudaStream_t st) {
    static const int pdl = env_int("HF2Q_CUDA_PDL", 1);
    cudaLaunchConfig_t cfg{};
    const uint64_t want = (count + 255) / 256, cap = static_cast<uint64_t>(dev.sm_count) * 4;
    cfg.gridDim = dim3(static_cast<unsigned>(want < cap ? want : cap));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, scratch, parts, count, residual, y);
}

template <uint32_t TYPE>
cudaError_t launch_mma_t(MParams p, uint32_t slots, const DeviceInfo& dev, cudaStream_t st, const GemvArgs& a) {
    const size_t limit = static_cast<size_t>(dev.max_smem_optin);
    // two teams: a third (26 warps, 72 registers) measured no faster
    const Plan pl = make_plan(TYPE, p.k, p.nslots, 2, limit);
    if (!pl.stages) return cudaErrorInvalidConfiguration;
    const bool phased = pl.phase_base != p.nslices;
    if (phased && p.swiglu) return cudaErrorInvalidConfiguration;       // the gate sums cannot wait across phases
    // the fused RMSNorm needs the whole f32 row in one panel, one chunk of eight elements per consumer thread
    if (p.norm_w && (phased || p.x_bf16 || p.ids || p.k > 8u * 2 * TEAM * 32 || p.nslots > 8)) return cudaErrorInvalidConfiguration;
    const bool ext = p.g_nranks != 0 || p.w2 != nullptr || p.norm_w != nullptr;      // (the fused RMSNorm is compiled into the EXT variants only)
    if (p.sub_groups > 1)                                                                          // one short slice per row
        return ext ? launch_mma_tt<TYPE, 2, false, true, true>(p, slots, pl, dev, st) : launch_mma_tt<TYPE, 2, false, true, false>(p, slots, pl, dev, st);
    if (phased) {
        // Rows too long for the activation panel.  Preferred: split k over the CTAs -- every CTA keeps ONE
        // slice of the activations and streams that slice of all its row groups, the parts meet in a
        // scratch buffer and a small second kernel adds them in part order (deterministic).  Needs the
        // context's scratch, a dense plain product and at least as many SMs as parts; otherwise the CTA
        // walks its groups once per k-phase (below).
        static const bool split_on = env_int("HF2Q_CUDA_MMA_SPLITK", 1) != 0;                      // tuning aid
        const uint32_t parts = p.nslices;
        const uint64_t count = static_cast<uint64_t>(p.m) * p.n;
        if (split_on && !ext && !p.ids && slots == 1 && a.splitk_scratch && parts * count * 4 <= a.splitk_bytes &&
            parts <= static_cast<uint32_t>(dev.sm_count)) {
            MParams q = p;
            q.split = parts;
            q.k_last = p.k - (parts - 1) * SLICE_ELEMS;
            q.k = SLICE_ELEMS;
            q.nslices = 1;
            q.last_nblk = SLICE_ELEMS >> 8;
            q.y = a.splitk_scratch;
            q.residual = nullptr;
            const Plan pl1 = make_plan(TYPE, SLICE_ELEMS, p.nslots, 2, limit);
            if (pl1.stages && pl1.phase_base == 1) {
                cudaError_t e = launch_mma_tt<TYPE, 2, false, false, true>(q, parts, pl1, dev, st);
                if (e != cudaSuccess) return e;
                if (a.n_launches) *a.n_launches = 2;
                return launch_splitk_reduce(a.splitk_scratch, parts, count, p.residual, p.y, dev, st);
            }
        }
        return ext ? launch_mma_tt<TYPE, 2, true, false, true>(p, slots, pl, dev, st) : launch_mma_tt<TYPE, 2, true, false, false>(p, slots, pl, dev, st);
    }
    return ext ? launch_mma_tt<TYPE, 2, false, false, true>(p, slots, pl, dev, st) : launch_mma_tt<TYPE, 2, false, false, false>(p, slots, pl, dev, st);
}

}  // namespace


namespace {
__global__ void gather_wait_kernel(const uint32_t* flag, uint32_t n_ranks, uint32_t rank, long long limit, uint32_t* status) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x < n_ranks && threadIdx.x != rank) gather_wait_source(flag, threadIdx.x, limit, status);
}
}  // namespace

cudaError_t launch_gather_wait(const uint32_t* flag, uint32_t n_ranks, uint32_t rank, long long limit, uint32_t* status, cudaStream_t st) {
    gather_wait_kernel<<<1, 32, 0, st>>>(flag, n_ranks, rank, limit, status);
    return cudaGetLastError();
}

namespace {
// x[i] += sum over the n_parts parts r (in order: the same bits on every rank) of parts[r * stride + i], after the
// columns of every rank have arrived here.  The gathered buffer holds one full-length PARTIAL product per rank
// (a product whose contraction dimension is sharded): this is the all-reduce of a column-sharded projection,
// built from the all-gather in the producing product's epilogue and a local sum.
__global__ void __launch_bounds__(256) gather_sum_kernel(const uint32_t* flag, uint32_t n_ranks, uint32_t rank, long long limit, uint32_t* status,
                                                         const float* __restrict__ parts, uint32_t stride, uint32_t n_parts, float* __restrict__ x,
                                                         uint32_t n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the next kernel may start its own prologue
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x < n_ranks && threadIdx.x != rank) gather_wait_source(flag, threadIdx.x, limit, status);
    __syncthreads();
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float acc = x[i];
    for (uint32_t r = 0; r < n_parts; ++r) acc += __ldcg(parts + static_cast<size_t>(r) * stride + i);
    x[i] = acc;
}
// dst[r][0 .. width) = src[r * pitch + 0 .. width) for r < m, after the columns of every rank have arrived here: the
// gathered rows of the most recent product leave the group's buffer in one launch (the sharded host-buffer batch
// copies them out behind the kernels).
__global__ void __launch_bounds__(256) gather_take_kernel(const uint32_t* flag, uint32_t n_ranks, uint32_t rank, long long limit, uint32_t* status,
                                                          const float* __restrict__ src, uint32_t pitch, uint32_t width, uint32_t m,
                                                          float* __restrict__ dst, uint32_t vec4) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the next kernel may start its own prologue
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x < n_ranks && threadIdx.x != rank) gather_wait_source(flag, threadIdx.x, limit, status);
    __syncthreads();
    const uint32_t stride = gridDim.x * 256;
    if (vec4) {
        const uint32_t w4 = width / 4, total = m * w4;
        for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
            const uint32_t r = i / w4, c = i - r * w4;
            reinterpret_cast<float4*>(dst)[i] = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(r) * pitch) + c);
        }
    } else {
        const uint32_t total = m * width;
        for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
            const uint32_t r = i / width, c = i - r * width;
            dst[i] = __ldcg(src + static_cast<size_t>(r) * pitch + c);
        }
    }
}
}  // namespace

namespace {
// The exchange of the fused all-gather without a product: src[0 .. n) goes to columns [col0, col0 + n) of row 0 of
// every rank's buffer, and the peers' arrival counters are bumped exactly as the mat-vec's epilogue does it (one
// fence, then one relaxed add per peer and CTA; CTA 0 books the arrivals this rank expects from every source).
// For results that the gathering mat-vec cannot produce itself (unaligned rows run on the fp32 kernel).
constexpr uint32_t GCOPY_PER_CTA = 1024;
struct GatherCopyParams {
    float* y[8];
    uint32_t* flag[8];
    uint32_t peer_ctas[8];
    uint32_t n_ranks, rank, col0, n;
};
__global__ void __launch_bounds__(256) gather_copy_kernel(const float* __restrict__ src, const GatherCopyParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the next kernel may start its own prologue
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t i = blockIdx.x * GCOPY_PER_CTA + threadIdx.x; i < min((blockIdx.x + 1) * GCOPY_PER_CTA, p.n); i += 256) {
        const float v = src[i];
        for (uint32_t r = 0; r < p.n_ranks; ++r) p.y[r][p.col0 + i] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0 && p.n_ranks > 1) {
        if (blockIdx.x == 0)
            for (uint32_t r = 0; r < p.n_ranks; ++r)
                if (r != p.rank) atomicAdd(p.flag[p.rank] + 8 + r, p.peer_ctas[r]);
        asm volatile("fence.acq_rel.sys;" ::: "memory");
        for (uint32_t r = 0; r < p.n_ranks; ++r)
            if (r != p.rank) asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(p.flag[r] + p.rank) : "memory");
    }
}
}  // namespace

cudaError_t launch_gather_copy(const float* src, const GatherArgs& g, uint32_t n, const uint32_t* n_each, cudaStream_t st) {
    GatherCopyParams p{};
    for (uint32_t r = 0; r < g.n_ranks; ++r) {
        p.y[r] = g.y_all[r];
        p.flag[r] = g.flags[r];
        p.peer_ctas[r] = (n_each[r] + GCOPY_PER_CTA - 1) / GCOPY_PER_CTA;
    }
    p.n_ranks = g.n_ranks; p.rank = g.rank; p.col0 = g.col0; p.n = n;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((n + GCOPY_PER_CTA - 1) / GCOPY_PER_CTA);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gather_copy_kernel, src, p);
}

cudaError_t launch_gather_sum(const uint32_t* flag, uint32_t n_ranks, uint32_t rank, long long limit, uint32_t* status, const float* parts,
                              uint32_t stride, uint32_t n_parts, float* x, uint32_t n, cudaStream_t st) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((n + 255) / 256);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gather_sum_kernel, flag, n_ranks, rank, limit, status, parts, stride, n_parts, x, n);
}

cudaError_t launch_gather_take(const uint32_t* flag, uint32_t n_ranks, uint32_t rank, long long limit, uint32_t* status, const float* src,
                               uint32_t pitch, uint32_t width, uint32_t m, float* dst, int sm_count, cudaStream_t st) {
    const bool vec4 = width % 4 == 0 && pitch % 4 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
    const uint64_t items = static_cast<uint64_t>(m) * width / (vec4 ? 4 : 1);
    const uint64_t want = (items + 255) / 256, cap = static_cast<uint64_t>(sm_count) * 4;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(want < 1 ? 1 : want < cap ? want : cap));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gather_take_kernel, flag, n_ranks, rank, limit, status, src, pitch, width, m, dst, vec4 ? 1u : 0u);
}

uint32_t gemv_mma_grid_x(uint32_t n, uint32_t k, const DeviceInfo& dev) {
    const uint32_t rows = ROWS * sub_groups_of(k);
    const uint32_t ngroups = (n + rows - 1) / rows;
    const uint32_t gx = static_cast<uint32_t>(dev.sm_count) < ngroups ? static_cast<uint32_t>(dev.sm_count) : ngroups;
    return gx < 1 ? 1 : gx;
}

bool gemv_mma_supported(const GemvArgs& a) {
    const BlockGeom g = block_geom(a.type);
    const uint64_t row_bytes = static_cast<uint64_t>(a.k) / g.elems * g.bytes;
    // (the four 32-element fall-back formats take the CUDA-core kernel: no warp-MMA unpack routine exists for them)
    return !type_is_fallback32(a.type) && a.k % 256 == 0 && row_bytes % 16 == 0 && a.expert_stride % 16 == 0 &&
           reinterpret_cast<uintptr_t>(a.w) % 16 == 0 && reinterpret_cast<uintptr_t>(a.x) % 16 == 0;
}

// Activation rows one launch can take: 8 MMA columns (bf16: one per row, f32: two per row), capped
// by what fits in shared memory next to a ring of at least 4 stages.
uint32_t gemv_mma_max_rows(uint32_t type, uint32_t k, uint32_t x_dtype, const DeviceInfo& dev) {
    const uint32_t per_row = x_dtype == HF2Q_DT_BF16 ? 1 : 2;
    uint32_t rows = 8 / per_row;
    if (type_is_fallback32(type)) return 0;
    while (rows > 0 && !make_plan(type, k, rows * per_row, 2, static_cast<size_t>(dev.max_smem_optin)).stages) --rows;
    return rows;
}

// whether a launch can take m f32 activation rows with the RMSNorm fused into its panel build
bool gemv_mma_norm_ok(uint32_t type, uint32_t k, uint32_t m, const DeviceInfo& dev) {
    if (m == 0 || m > 4 || k % 256 || k > 8u * 2 * TEAM * 32 || type_is_fallback32(type)) return false;
    const Plan pl = make_plan(type, k, 2 * m, 2, static_cast<size_t>(dev.max_smem_optin));
    return pl.stages && pl.phase_base == (k + SLICE_ELEMS - 1) / SLICE_ELEMS;
}

bool gemv_mma_swiglu_ok(uint32_t type, uint32_t k, uint32_t m, uint32_t x_dtype, const DeviceInfo& dev) {
    const uint32_t nslots = x_dtype == HF2Q_DT_BF16 ? m : 2 * m;
    if (m == 0 || nslots > 8 || k % 256 || sub_groups_of(k) > 1 || type_is_fallback32(type)) return false;
    const Plan pl = make_plan(type, k, nslots, 2, static_cast<size_t>(dev.max_smem_optin));
    return pl.stages && pl.phase_base == (k + SLICE_ELEMS - 1) / SLICE_ELEMS;
}

// One launch: bf16 activations, m <= 8; f32 activations, m <= 4 (hi/lo split on two columns).
cudaError_t launch_gemv_mma(const GemvArgs& a, const DeviceInfo& dev, cudaStream_t st) {
    const BlockGeom g = block_geom(a.type);
    MParams p{};
    p.w = static_cast<const uint8_t*>(a.w);
    p.w2 = static_cast<const uint8_t*>(a.w2);
    p.y2 = a.y2;
    p.pair_slots = a.swiglu ? 0xffffffffu : a.slots;
    p.swiglu = a.swiglu ? 1u : 0u;
    p.residual = a.residual;
    p.norm_w = a.norm_weight;
    p.norm_eps = a.norm_eps;
    p.x = a.x;
    p.y = a.y;
    p.ids = a.ids;
    p.expert_stride = a.expert_stride;
    p.x_bf16 = a.x_dtype == HF2Q_DT_BF16;
    p.m = a.m;
    p.nslots = p.x_bf16 ? a.m : 2 * a.m;
    if (p.nslots > 8) return cudaErrorInvalidValue;
    p.n = a.n;
    p.k = a.k;
    p.kx = a.k;
    p.top_k = a.top_k ? a.top_k : 1;
    p.n_experts = a.n_experts;
    p.row_bytes = a.k / g.elems * g.bytes;
    p.slice_bytes = SLICE_ELEMS / g.elems * g.bytes;
    if (p.slice_bytes > p.row_bytes) p.slice_bytes = p.row_bytes;
    p.dense_stage = dense_stage_ok(p.row_bytes, a.k) ? 1u : 0u;
    p.pitch = p.dense_stage ? p.row_bytes : row_pitch(p.slice_bytes);
    p.nslices = (a.k + SLICE_ELEMS - 1) / SLICE_ELEMS;
    p.sub_groups = sub_groups_of(a.k);
    p.ngroups = (a.n + ROWS * p.sub_groups - 1) / (ROWS * p.sub_groups);
    p.last_nblk = (a.k - (p.nslices - 1) * SLICE_ELEMS) >> 8;
    p.status = a.status;
    if (a.gather) {
        const GatherArgs& g = *a.gather;
        if (a.ids || g.n_ranks < 1 || g.n_ranks > 8 || g.rank >= g.n_ranks) return cudaErrorInvalidValue;
        for (uint32_t r = 0; r < g.n_ranks; ++r) { p.g_y[r] = g.y_all[r]; p.g_flag[r] = g.flags[r]; p.g_peer_ctas[r] = g.peer_ctas[r]; }
        p.g_nranks = g.n_ranks; p.g_rank = g.rank; p.g_ntotal = g.n_total; p.g_col0 = g.col0;
        p.g_wait = g.wait_expected;
        p.wait_limit = g.wait_limit;
    }
    if (a.swiglu && (!a.w2 || a.gather || a.residual || p.sub_groups > 1)) return cudaErrorInvalidValue;
    const uint32_t slots = a.w2 && !a.swiglu ? 2 * a.slots : a.slots;
    switch (a.type) {
        case HF2Q_TYPE_Q4_0: return launch_mma_t<HF2Q_TYPE_Q4_0>(p, slots, dev, st, a);
        case HF2Q_TYPE_Q8_0: return launch_mma_t<HF2Q_TYPE_Q8_0>(p, slots, dev, st, a);
        case HF2Q_TYPE_Q4_K: return launch_mma_t<HF2Q_TYPE_Q4_K>(p, slots, dev, st, a);
        case HF2Q_TYPE_Q5_K: return launch_mma_t<HF2Q_TYPE_Q5_K>(p, slots, dev, st, a);
        case HF2Q_TYPE_Q6_K: return launch_mma_t<HF2Q_TYPE_Q6_K>(p, slots, dev, st, a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace hf2q
