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
// m16n8k16 MMA (8 weight rows x 16 elements x 8 activation columns per instruction) and the
// CUDA cores only unpack bits:
//
//   * a persistent CTA owns groups of 8 weight rows; a producer warp streams their RAW block
//     bytes into a shared-memory ring with 1-D bulk copies (cp.async.bulk + mbarrier), 2048
//     elements per row and stage, so 18/34/210-byte blocks are readable at any 2-byte offset;
//   * each of 8 consumer warps takes one 256-element chunk of the stage for all 8 rows: lane
//     (g, t) unpacks row g, four elements at a time, into the A fragment.  The integer codes are
//     fed as f16 SUBNORMALS (code * 2^-24): a single PRMT turns two packed bytes into an f16x2
//     operand, with no int->float conversion and no offset to subtract;
//   * scales stay out of the per-element path: Q4_K/Q5_K multiply the codes by the 6-bit
//     sub-block scale in f16 (code*scale < 2048, exact) and apply d once per block; Q6_K applies
//     d*scale to each 16-element MMA result; Q4_0/Q8_0 apply d per block.  Offsets (the -dmin*m
//     of Q4_K/Q5_K, the -32/-8/-128 code biases) become one small extra MMA (or FMA) per block
//     against per-sub-block sums of x that every CTA computes once;
//   * activations live in shared memory as f16 (bf16 input: exact in range; f32 input: split
//     into hi + lo halves on two MMA columns, ~2^-22 relative);
//   * partial sums of the 8 warps are combined through shared memory in a fixed order: no
//     atomics, bit-reproducible.
//
// Needs 16-byte aligned rows and k a multiple of 256; other shapes take the fp32 kernel in
// k1_gemv.cu.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace hf2q {

namespace {

constexpr int ROWS = 16;               // weight rows per stage = rows of one MMA tile
constexpr int CWARPS = 16;             // consumer warps; each takes 128 elements x 16 rows per stage
constexpr int CT = CWARPS * 32;
constexpr int THREADS = CT + 32;
constexpr int SLICE_ELEMS = 2048;
constexpr int MAX_STAGES = 8;

struct MParams {
    const uint8_t* w;
    const void* x;
    float* y;
    const uint32_t* ids;
    uint64_t expert_stride;
    uint32_t x_bf16;
    uint32_t m;            // activation rows of this launch (bf16: <= 8, f32: <= 4)
    uint32_t nslots;       // MMA columns in use: m (bf16) or 2m (f32 hi/lo split)
    uint32_t n, k;
    uint32_t top_k, n_experts;
    uint32_t row_bytes, slice_bytes, pitch, nslices, ngroups, stages;
    uint32_t xpitch;       // bytes between activation rows in shared memory
    uint32_t* status;
};

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

// ---- Q4_K / Q5_K: half a block (128 elements = chunks 2*half, 2*half+1) of rows g and g+8.
// Lane t owns 16 bytes of qs per row: chunk c = 2*half + (t>>1), bytes 16*(t&1)..+15, i.e. 16
// elements of sub-block 2c (low nibbles) and 16 of sub-block 2c+1 (high nibbles).
template <bool Q5>
struct K45Row {
    uint32_t qv[4], gv[4], s1, s2, am;
    float d, dm;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, int hb) {
        constexpr int QS = Q5 ? 48 : 16;
        const uint4 hd = *reinterpret_cast<const uint4*>(blk);
        const uint4 qa = *reinterpret_cast<const uint4*>(blk + QS + 32 * c + 16 * hb);
        qv[0] = qa.x; qv[1] = qa.y; qv[2] = qa.z; qv[3] = qa.w;
        if constexpr (Q5) {
            const uint4 ga = *reinterpret_cast<const uint4*>(blk + 16 + 16 * hb);
            gv[0] = ga.x; gv[1] = ga.y; gv[2] = ga.z; gv[3] = ga.w;
        }
        uint32_t sc1, m1, sc2, m2;
        scale_min_k4(2 * c, hd.y, hd.z, hd.w, sc1, m1);
        scale_min_k4(2 * c + 1, hd.y, hd.z, hd.w, sc2, m2);
        // scale * 2^10 as f16x2 (<= 64512): code*2^-24 * scale*2^10 = code*scale*2^-14, exact
        const __half2 s1h = __half2half2(__uint2half_rn(sc1 << 10));
        const __half2 s2h = __half2half2(__uint2half_rn(sc2 << 10));
        s1 = *reinterpret_cast<const uint32_t*>(&s1h);
        s2 = *reinterpret_cast<const uint32_t*>(&s2h);
        am = hb ? 0u : (m1 | (m2 << 16));
        d = f16_bits_to_f32(hd.x & 0xffffu) * 16384.0f;
        dm = f16_bits_to_f32(hd.x >> 16) * TWO24;
    }
    __device__ __forceinline__ void codes(int i, int c, uint32_t& lo, uint32_t& hi) const {
        lo = qv[i] & 0x0F0F0F0Fu;
        hi = (qv[i] >> 4) & 0x0F0F0F0Fu;
        if constexpr (Q5) {
            lo |= ((gv[i] >> (2 * c)) & 0x01010101u) << 4;
            hi |= ((gv[i] >> (2 * c + 1)) & 0x01010101u) << 4;
        }
    }
};

template <bool Q5>
__device__ __forceinline__ void half_k45(const uint8_t* blk0, const uint8_t* blk1, int half, uint32_t e0,
                                         const uint8_t* xrow, const uint8_t* sxblk, int t, float (&f)[4]) {
    const int c = 2 * half + (t >> 1), hb = t & 1;
    K45Row<Q5> r0, r1;
    r0.load(blk0, c, hb);
    r1.load(blk1, c, hb);
    const uint32_t eb = e0 + 64 * c + 16 * hb;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t lo0, hi0, lo1, hi1;
        r0.codes(i, c, lo0, hi0);
        r1.codes(i, c, lo1, hi1);
        const uint2 xl = ld_x4(xrow, eb + 4 * i);
        mma_acc(acc, hmul2_bits(sub01(lo0), r0.s1), hmul2_bits(sub01(lo1), r1.s1),
                hmul2_bits(sub23(lo0), r0.s1), hmul2_bits(sub23(lo1), r1.s1), xl.x, xl.y);
        const uint2 xh = ld_x4(xrow, eb + 32 + 4 * i);
        mma_acc(acc, hmul2_bits(sub01(hi0), r0.s2), hmul2_bits(sub01(hi1), r1.s2),
                hmul2_bits(sub23(hi0), r0.s2), hmul2_bits(sub23(hi1), r1.s2), xh.x, xh.y);
    }
    // -dmin * sum_j m_j * Sx_j over this half's four sub-blocks: lanes with (t&1)==0 carry
    // (m_2c, m_2c+1) against Sx_hi on k-columns (2t, 2t+1) and against Sx_lo on (2t+8, 2t+9);
    // odd lanes carry zeros.  The panel stores, per block, hi[8] then lo[8] (f16).
    const uint32_t bs0 = *reinterpret_cast<const uint32_t*>(sxblk + 4 * c);
    const uint32_t bs1 = *reinterpret_cast<const uint32_t*>(sxblk + 16 + 4 * c);
    float mn[4];
    mma_new(mn, r0.am, r1.am, r0.am, r1.am, bs0, bs1);
    f[0] += r0.d * acc[0] - r0.dm * mn[0];
    f[1] += r0.d * acc[1] - r0.dm * mn[1];
    f[2] += r1.d * acc[2] - r1.dm * mn[2];
    f[3] += r1.d * acc[3] - r1.dm * mn[3];
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

template <uint32_t TYPE>
__global__ void __launch_bounds__(THREADS) gemv_mma_kernel(const MParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool K45 = TYPE == HF2Q_TYPE_Q4_K || TYPE == HF2Q_TYPE_Q5_K;
    constexpr bool Q6 = TYPE == HF2Q_TYPE_Q6_K;
    constexpr bool LEG = TYPE == HF2Q_TYPE_Q4_0 || TYPE == HF2Q_TYPE_Q8_0;
    constexpr BlockGeom G = block_geom(TYPE);
    // bytes of x-sum panel per 256 elements and column: K45 8 x (hi,lo) f16, Q6 16 x (hi,lo) f16;
    // Q4_0/Q8_0 keep f32 sums for all 8 columns per 32-element block
    constexpr uint32_t SXB = K45 ? 32 : 64;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + MAX_STAGES;
    uint8_t* ring = smem + 128;
    const uint32_t stage_bytes = ROWS * p.pitch;
    float* red = reinterpret_cast<float*>(ring + p.stages * stage_bytes);        // [CWARPS][16][8]
    float* scr = red + CWARPS * 128;                                            // [CWARPS][16][8]
    uint8_t* xh = reinterpret_cast<uint8_t*>(scr + CWARPS * 16 * 8);             // [nslots][xpitch]
    uint8_t* sxp = xh + p.nslots * p.xpitch;
    const uint32_t nblk_total = p.k >> 8;
    const uint32_t sx_slot_bytes = nblk_total * SXB;                            // K45 / Q6 panels

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t slot = blockIdx.y;
    const uint8_t* wbase = p.w;
    uint32_t xrow_idx = 0;
    bool slot_ok = true;
    if (p.ids) {
        const uint32_t e = p.ids[slot];
        slot_ok = e < p.n_experts;
        if (!slot_ok && threadIdx.x == 0) atomicOr(p.status, STATUS_BAD_EXPERT_ID);
        wbase += static_cast<uint64_t>(slot_ok ? e : 0) * p.expert_stride;
        xrow_idx = slot / p.top_k;
    }
    float* yout = p.y + static_cast<size_t>(slot) * p.n;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CWARPS); }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == CWARPS) {
        // ---------------- producer warp: lane r copies row r of each stage ----------------
        if (slot_ok) {
            uint32_t it = 0, st = 0, ph = 1;      // ring slot and the parity of its previous use
            bool alive = true;
            for (uint32_t rg = blockIdx.x; rg < p.ngroups && alive; rg += gridDim.x) {
                const uint32_t row0 = rg * ROWS;
                const uint32_t nrows = min(static_cast<uint32_t>(ROWS), p.n - row0);
                for (uint32_t s = 0; s < p.nslices; ++s, ++it, st = (st + 1 == p.stages ? 0 : st + 1), ph ^= (st == 0)) {
                    if (it >= p.stages) {
                        alive = mbar_wait_bounded(&empty[st], ph, p.status);
                        alive = __all_sync(0xffffffffu, alive);
                        if (!alive) break;
                    }
                    const uint32_t off = s * p.slice_bytes;
                    const uint32_t bytes = min(p.slice_bytes, p.row_bytes - off);
                    if (lane == 0) mbar_arrive_expect_tx(&full[st], nrows * bytes);
                    __syncwarp();
                    if (static_cast<uint32_t>(lane) < nrows)
                        bulk_g2s(ring + st * stage_bytes + lane * p.pitch,
                                 wbase + static_cast<uint64_t>(row0 + lane) * p.row_bytes + off, bytes, &full[st]);
                }
            }
        }
        return;
    }

    // ---------------- consumers: build the f16 activation panel and its sub-block sums ------------
    const int ctid = threadIdx.x;
    {
        // 8 elements per item; four items per thread and pass so that four independent loads are
        // in flight before the first conversion
        const uint32_t k8 = p.k >> 3, total = p.nslots * k8;
        bool clipped = false;
        for (uint32_t base = ctid; base < total; base += 4 * CT) {
            uint4 ra[4], rb[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t idx = base + u * CT;
                ra[u] = make_uint4(0, 0, 0, 0); rb[u] = ra[u];
                if (idx < total) {
                    const uint32_t s = idx / k8, e = (idx - s * k8) * 8;
                    if (p.x_bf16) {
                        ra[u] = __ldg(reinterpret_cast<const uint4*>(
                            static_cast<const __nv_bfloat16*>(p.x) + (static_cast<size_t>(xrow_idx) + s) * p.k + e));
                    } else {
                        const float* src = static_cast<const float*>(p.x) + (static_cast<size_t>(xrow_idx) + (s >> 1)) * p.k + e;
                        ra[u] = __ldg(reinterpret_cast<const uint4*>(src));
                        rb[u] = __ldg(reinterpret_cast<const uint4*>(src + 4));
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t idx = base + u * CT;
                if (idx >= total) continue;
                const uint32_t s = idx / k8, e = (idx - s * k8) * 8;
                float v[8];
                if (p.x_bf16) {
                    const uint32_t rr[4] = {ra[u].x, ra[u].y, ra[u].z, ra[u].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        v[2 * j] = __uint_as_float(rr[j] << 16);
                        v[2 * j + 1] = __uint_as_float(rr[j] & 0xffff0000u);
                    }
                } else {
                    v[0] = __uint_as_float(ra[u].x); v[1] = __uint_as_float(ra[u].y); v[2] = __uint_as_float(ra[u].z); v[3] = __uint_as_float(ra[u].w);
                    v[4] = __uint_as_float(rb[u].x); v[5] = __uint_as_float(rb[u].y); v[6] = __uint_as_float(rb[u].z); v[7] = __uint_as_float(rb[u].w);
                }
                uint32_t out[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float a = v[2 * j], b = v[2 * j + 1];
                    clipped |= (fabsf(a) > 65504.0f) | (fabsf(b) > 65504.0f);
                    a = fminf(fmaxf(a, -65504.0f), 65504.0f);
                    b = fminf(fmaxf(b, -65504.0f), 65504.0f);
                    __half ha = __float2half_rn(a), hb = __float2half_rn(b);
                    if (!p.x_bf16 && (s & 1)) {          // lo part of the f32 split
                        ha = __float2half_rn(a - __half2float(ha));
                        hb = __float2half_rn(b - __half2float(hb));
                    }
                    out[j] = static_cast<uint32_t>(__half_as_ushort(ha)) | (static_cast<uint32_t>(__half_as_ushort(hb)) << 16);
                }
                *reinterpret_cast<uint4*>(xh + s * p.xpitch + 2 * e) = make_uint4(out[0], out[1], out[2], out[3]);
            }
        }
        if (clipped) atomicOr(p.status, STATUS_X_CLIPPED);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CT));
    if constexpr (LEG) {
        float* sxf = reinterpret_cast<float*>(sxp);
        const uint32_t nb = p.k >> 5;
        for (uint32_t idx = ctid; idx < nb * 8; idx += CT) {
            const uint32_t b = idx >> 3, s = idx & 7;
            float acc = 0.f;
            if (s < p.nslots) {
                const uint4* src = reinterpret_cast<const uint4*>(xh + s * p.xpitch + 64 * b);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 r = src[j];
                    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&rr[q]));
                        acc += f.x + f.y;
                    }
                }
            }
            sxf[idx] = acc;
        }
    } else {
        constexpr uint32_t SUB = K45 ? 32 : 16;            // elements per sub-block sum
        constexpr uint32_t PER = 256 / SUB;                // sums per block: 8 or 16
        const uint32_t nsub = p.k / SUB;
        for (uint32_t idx = ctid; idx < p.nslots * nsub; idx += CT) {
            const uint32_t s = idx / nsub, j = idx - s * nsub;
            const uint4* src = reinterpret_cast<const uint4*>(xh + s * p.xpitch + 2 * SUB * j);
            float acc = 0.f;
#pragma unroll
            for (uint32_t v = 0; v < SUB / 8; ++v) {
                const uint4 r = src[v];
                const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&rr[q]));
                    acc += f.x + f.y;
                }
            }
            const __half hi = __float2half_rn(acc);
            const __half lo = __float2half_rn(acc - __half2float(hi));
            __half* dst = reinterpret_cast<__half*>(sxp + s * sx_slot_bytes + (j / PER) * SXB);
            dst[j % PER] = hi;
            dst[PER + j % PER] = lo;
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CT));
    if (!slot_ok) {
        for (uint32_t r = ctid; r < p.n; r += CT) yout[r] = 0.f;
        return;
    }

    // Lane (g, t): weight row g, MMA column g.  Columns beyond nslots alias column 0: a column of
    // the product depends only on its own column of B, and those outputs are never stored.
    const int g = lane >> 2, t = lane & 3;
    const uint32_t col = static_cast<uint32_t>(g) < p.nslots ? g : 0;
    const uint8_t* xrow = xh + col * p.xpitch;
    const uint8_t* sxslot = sxp + col * sx_slot_bytes;
    float* scr0 = scr + (warp * 16 + g) * 8;
    float* scr1 = scr0 + 64;
    (void)scr0; (void)scr1; (void)sxslot;

    uint32_t it = 0, grp = 0, st = 0, ph = 0;     // ring slot and the parity of its current use
    bool alive = true;
    for (uint32_t rg = blockIdx.x; rg < p.ngroups; rg += gridDim.x, ++grp) {
        float f[4] = {0.f, 0.f, 0.f, 0.f};
        for (uint32_t s = 0; s < p.nslices; ++s, ++it, st = (st + 1 == p.stages ? 0 : st + 1), ph ^= (st == 0)) {
            // a wait that gives up marks the warp dead; it keeps walking the loops (skipping waits
            // and work) so the named barriers below are still reached by all consumers
            if (alive && !mbar_wait_bounded(&full[st], ph, p.status)) alive = false;
            const uint32_t kbase = s * SLICE_ELEMS;
            const uint32_t nhalf = min(static_cast<uint32_t>(SLICE_ELEMS), p.k - kbase) >> 7;
            // which 128-element piece this warp takes rotates with the stage, so that idle warps
            // (short slices) and the slower unaligned Q6_K blocks spread evenly over the warps
            const uint32_t hb = (static_cast<uint32_t>(warp) + it) & (CWARPS - 1);
            if (alive && hb < nhalf) {
                const uint8_t* r0 = ring + st * stage_bytes + g * p.pitch;
                const uint8_t* r1 = r0 + 8 * p.pitch;
                const uint32_t b = hb >> 1, half = hb & 1;
                const uint32_t e0 = kbase + 256 * b;
                if constexpr (K45) {
                    half_k45<TYPE == HF2Q_TYPE_Q5_K>(r0 + b * G.bytes, r1 + b * G.bytes, half, e0, xrow,
                                                     sxslot + (e0 >> 8) * SXB, t, f);
                } else if constexpr (Q6) {
                    if (b & 1) half_q6k<false>(r0 + b * 210, r1 + b * 210, half, e0, xrow, sxslot + (e0 >> 8) * SXB, scr0, scr1, t, f);
                    else half_q6k<true>(r0 + b * 210, r1 + b * 210, half, e0, xrow, sxslot + (e0 >> 8) * SXB, scr0, scr1, t, f);
                } else {
                    half_legacy<TYPE == HF2Q_TYPE_Q8_0>(r0 + hb * 4 * G.bytes, r1 + hb * 4 * G.bytes, kbase + 128 * hb, xrow,
                                                        reinterpret_cast<const float*>(sxp), t, f);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        }
        // combine the warps' partial sums in a fixed order
        float* rbuf = red;
        if (grp) asm volatile("bar.sync 1, %0;" ::"n"(CT));      // the previous group's readers are done
        *reinterpret_cast<float2*>(rbuf + warp * 128 + g * 8 + 2 * t) = make_float2(f[0], f[1]);
        *reinterpret_cast<float2*>(rbuf + warp * 128 + (g + 8) * 8 + 2 * t) = make_float2(f[2], f[3]);
        asm volatile("bar.sync 1, %0;" ::"n"(CT));
        if (ctid < 128) {
            const uint32_t r = ctid >> 3, c = ctid & 7;
            const uint32_t row = rg * ROWS + r;
            float v = 0.f;
            if (p.x_bf16) {
#pragma unroll
                for (int w = 0; w < CWARPS; ++w) v += rbuf[w * 128 + r * 8 + c];
                if (row < p.n && c < p.m) yout[static_cast<size_t>(c) * p.n + row] = v;
            } else if (c < 4) {
#pragma unroll
                for (int w = 0; w < CWARPS; ++w) v += rbuf[w * 128 + r * 8 + 2 * c] + rbuf[w * 128 + r * 8 + 2 * c + 1];
                if (row < p.n && c < p.m) yout[static_cast<size_t>(c) * p.n + row] = v;
            }
        }
    }
}

// shared memory that does not depend on the ring depth
size_t smem_base_bytes(uint32_t type, uint32_t k, uint32_t nslots) {
    const bool k45 = type == HF2Q_TYPE_Q4_K || type == HF2Q_TYPE_Q5_K;
    const bool leg = type == HF2Q_TYPE_Q4_0 || type == HF2Q_TYPE_Q8_0;
    const size_t fixed = 128 + (CWARPS * 128 + CWARPS * 16 * 8) * 4;
    const size_t xbytes = static_cast<size_t>(nslots) * (2 * static_cast<size_t>(k) + 32);
    const size_t sxbytes = leg ? static_cast<size_t>(k / 32) * 8 * 4
                               : static_cast<size_t>(nslots) * (k / 256) * (k45 ? 32 : 64);
    return fixed + xbytes + sxbytes;
}
size_t stage_bytes_of(uint32_t type, uint32_t k) {
    const BlockGeom g = block_geom(type);
    uint32_t slice = SLICE_ELEMS / g.elems * g.bytes;
    const uint32_t row = k / g.elems * g.bytes;
    if (slice > row) slice = row;
    return static_cast<size_t>(ROWS) * (slice + 16);
}

template <uint32_t TYPE>
cudaError_t launch_mma_t(MParams p, uint32_t slots, const DeviceInfo& dev, cudaStream_t st) {
    auto kern = gemv_mma_kernel<TYPE>;
    const size_t stage = static_cast<size_t>(ROWS) * p.pitch;
    const size_t limit = static_cast<size_t>(dev.max_smem_optin);
    const size_t base = smem_base_bytes(TYPE, p.k, p.nslots);
    if (base + 2 * stage > limit) return cudaErrorInvalidConfiguration;
    // two CTAs per SM (twice the warps to hide latency) when each can still have a ring of >= 3
    // stages, else one CTA with as deep a ring as fits (up to 8 stages): bytes in flight per SM are
    // what hides HBM latency
    const size_t half = limit / 2 - 1024;
    uint32_t stages = 0;
    for (uint32_t s = 4; s >= 3; --s)
        if (base + s * stage <= half) { stages = s; break; }
    if (!stages) {
        stages = MAX_STAGES;
        while (stages > 2 && base + stages * stage > limit) --stages;
    }
    p.stages = stages;
    const size_t smem = base + stages * stage;

    static std::mutex mu;
    static bool attr_set = false;
    static size_t cached_smem = ~static_cast<size_t>(0);
    static int cached_per_sm = 1;
    int per_sm;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dev.max_smem_optin);
            if (e != cudaSuccess) return e;
            attr_set = true;
        }
        if (cached_smem != smem) {
            int q = 1;
            cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kern, THREADS, smem);
            if (e != cudaSuccess) return e;
            cached_per_sm = q < 1 ? 1 : q;
            cached_smem = smem;
        }
        per_sm = cached_per_sm;
    }
    const uint32_t want = static_cast<uint32_t>(dev.sm_count) * per_sm;
    uint32_t gx = (want + slots - 1) / slots;
    if (gx > p.ngroups) gx = p.ngroups;
    if (gx < 1) gx = 1;
    kern<<<dim3(gx, slots), THREADS, smem, st>>>(p);
    return cudaGetLastError();
}

}  // namespace

bool gemv_mma_supported(const GemvArgs& a) {
    const BlockGeom g = block_geom(a.type);
    const uint64_t row_bytes = static_cast<uint64_t>(a.k) / g.elems * g.bytes;
    return a.k % 256 == 0 && row_bytes % 16 == 0 && a.expert_stride % 16 == 0 &&
           reinterpret_cast<uintptr_t>(a.w) % 16 == 0 && reinterpret_cast<uintptr_t>(a.x) % 16 == 0;
}

// Activation rows one launch can take: 8 MMA columns (bf16: one per row, f32: two per row), capped
// by what fits in shared memory next to a ring of at least 3 stages.
uint32_t gemv_mma_max_rows(uint32_t type, uint32_t k, uint32_t x_dtype, const DeviceInfo& dev) {
    const uint32_t per_row = x_dtype == HF2Q_DT_BF16 ? 1 : 2;
    uint32_t rows = 8 / per_row;
    while (rows > 0 && smem_base_bytes(type, k, rows * per_row) + 3 * stage_bytes_of(type, k) >
                           static_cast<size_t>(dev.max_smem_optin))
        --rows;
    return rows;
}

// One launch: bf16 activations, m <= 8; f32 activations, m <= 4 (hi/lo split on two columns).
cudaError_t launch_gemv_mma(const GemvArgs& a, const DeviceInfo& dev, cudaStream_t st) {
    const BlockGeom g = block_geom(a.type);
    MParams p{};
    p.w = static_cast<const uint8_t*>(a.w);
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
    p.top_k = a.top_k ? a.top_k : 1;
    p.n_experts = a.n_experts;
    p.row_bytes = a.k / g.elems * g.bytes;
    p.slice_bytes = SLICE_ELEMS / g.elems * g.bytes;
    if (p.slice_bytes > p.row_bytes) p.slice_bytes = p.row_bytes;
    p.pitch = p.slice_bytes + 16;                 // rows land 4 banks apart
    p.nslices = (a.k + SLICE_ELEMS - 1) / SLICE_ELEMS;
    p.ngroups = (a.n + ROWS - 1) / ROWS;
    p.xpitch = 2 * a.k + 32;                      // activation rows land 8 banks apart
    p.status = a.status;
    switch (a.type) {
        case HF2Q_TYPE_Q4_0: return launch_mma_t<HF2Q_TYPE_Q4_0>(p, a.slots, dev, st);
        case HF2Q_TYPE_Q8_0: return launch_mma_t<HF2Q_TYPE_Q8_0>(p, a.slots, dev, st);
        case HF2Q_TYPE_Q4_K: return launch_mma_t<HF2Q_TYPE_Q4_K>(p, a.slots, dev, st);
        case HF2Q_TYPE_Q5_K: return launch_mma_t<HF2Q_TYPE_Q5_K>(p, a.slots, dev, st);
        case HF2Q_TYPE_Q6_K: return launch_mma_t<HF2Q_TYPE_Q6_K>(p, a.slots, dev, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace hf2q
