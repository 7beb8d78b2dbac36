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
//   warp 4 (one lane)   TMA producer.  Per 256-element K-block: one 2-D tensor copy of the RAW block
//                       bytes of 128 weight rows (box 128 x <=272 B, no swizzle) and four 2-D copies
//                       of the f16 activations (box NT x 64 elements, 128-byte swizzle) into
//                       shared-memory rings; completion on mbarriers.
//   warps 0-3           dequantisers.  Thread r owns weight row r: it reads its own raw bytes from
//                       shared memory (16-byte vectors, conflict-free pitch), unpacks 256 codes,
//                       applies d*scale (and -dmin*min) in f16x2 and writes the A operand straight
//                       into TENSOR MEMORY with tcgen05.st (row = TMEM lane), double-buffered.
//                       No cross-lane traffic, no shared-memory round trip for the dequantised tile.
//   warp 5 (one lane)   MMA issuer.  tcgen05.mma.kind::f16, M = 128, N = NT, K = 16, A from TMEM,
//                       B (activations, K-major, 128B-swizzled) from shared memory, D in TMEM;
//                       tcgen05.commit releases the activation stages and the A buffers.
//   warps 0-3 again     epilogue: tcgen05.ld the fp32 accumulators, coalesced stores of y.
//
// TMEM: 512 columns = D (<= 256) + 2 x 128 (two A buffers of one K-block each).
// Every mbarrier wait is bounded; a wait that gives up sets the status word and all roles drain to
// the final barrier, where TMEM is freed.  No cluster launch, no multicast.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace hf2q {

namespace {

constexpr int TILE_N = 128;      // weight rows per CTA (MMA M)
constexpr int KB = 256;          // K elements per block step
constexpr int XK = 64;           // K elements per activation stage (128 bytes of f16)
constexpr int raw_stages_of(uint32_t type) { return type == HF2Q_TYPE_Q8_0 ? 2 : 3; }   // 272-byte rows: 2 stages fit
constexpr int X_STAGES = 4;
constexpr int GEMM_THREADS = 192;

struct GParams {
    float* y;
    uint32_t m, n, k;
    uint32_t boxw;          // bytes per weight row in one raw stage
    uint32_t blk_bytes;     // bytes of one 256-element K-block of a row
    uint32_t* status;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void tma_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem_d] (+)= A[tmem_a] * B[smem desc]; M = 128, K = 16, f16 inputs, f32 accumulate
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte swizzled shared-memory operand: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(1) << 16) |
           (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) |
           (static_cast<uint64_t>(2) << 61);
}

// ---------------------------------------------------------------- per-row dequantisers
// Each produces the 64 f16 values of quarter `qd` (elements 64qd .. 64qd+63 of a 256-element
// K-block, in natural order) packed two per register.

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
// two packed bytes -> (1024 + b) as f16x2, then minus `bias` (>= 1024), exact
__device__ __forceinline__ __half2 codes01(uint32_t w, __half2 bias) {
    uint32_t h = __byte_perm(w, 0x64646464u, 0x4140u);
    return __hsub2(*reinterpret_cast<__half2*>(&h), bias);
}
__device__ __forceinline__ __half2 codes23(uint32_t w, __half2 bias) {
    uint32_t h = __byte_perm(w, 0x64646464u, 0x4342u);
    return __hsub2(*reinterpret_cast<__half2*>(&h), bias);
}

// Q4_K / Q5_K.  P: the block's 36 / 44 words.  Quarter qd = chunk c: low nibbles are sub-block 2c,
// high nibbles sub-block 2c+1;  w = f16(d*sc) * q - f16(dmin*m).
template <bool Q5>
__device__ __forceinline__ void dq_k45(const uint32_t* P, int c, uint32_t (&out)[32]) {
    constexpr int QW = Q5 ? 12 : 4;         // first qs word
    const float d = f16_bits_to_f32(P[0] & 0xffffu), dmin = f16_bits_to_f32(P[0] >> 16);
    uint32_t sc1, m1, sc2, m2;
    scale_min_k4(2 * c, P[1], P[2], P[3], sc1, m1);
    scale_min_k4(2 * c + 1, P[1], P[2], P[3], sc2, m2);
    const __half2 S1 = __float2half2_rn(d * static_cast<float>(sc1)), M1 = __float2half2_rn(-dmin * static_cast<float>(m1));
    const __half2 S2 = __float2half2_rn(d * static_cast<float>(sc2)), M2 = __float2half2_rn(-dmin * static_cast<float>(m2));
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t w = P[QW + 8 * c + i];
        uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
        if constexpr (Q5) {
            const uint32_t g = P[4 + i];
            lo |= ((g >> (2 * c)) & 0x01010101u) << 4;
            hi |= ((g >> (2 * c + 1)) & 0x01010101u) << 4;
        }
        out[2 * i] = h2_bits(__hfma2(codes01(lo, k1024), S1, M1));
        out[2 * i + 1] = h2_bits(__hfma2(codes23(lo, k1024), S1, M1));
        out[16 + 2 * i] = h2_bits(__hfma2(codes01(hi, k1024), S2, M2));
        out[16 + 2 * i + 1] = h2_bits(__hfma2(codes23(hi, k1024), S2, M2));
    }
}

// Q6_K.  W(j): logical 32-bit word j of the 210-byte block.  Quarter qd: half n = qd>>1, k in
// {2*(qd&1), 2*(qd&1)+1}; element 128n + 32k + l comes from ql/qh as in the quantizer's packing.
template <typename WordFn>
__device__ __forceinline__ void dq_q6k(WordFn W, int qd, uint32_t (&out)[32]) {
    const int n = qd >> 1, kp = qd & 1;
    const float d = f16_bits_to_f32(W(52) & 0xffffu);
    const uint32_t scw = W(48 + 2 * n + kp);             // scales 8n+4kp .. 8n+4kp+3
    const __half2 k1056 = __half2half2(__ushort_as_half(0x6420));   // 1024 + 32
    __half2 S[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float s = static_cast<float>(static_cast<int8_t>((scw >> (8 * j)) & 0xffu));
        S[j] = __float2half2_rn(d * s);                  // sub-block 8n + 4kp + j = 8n + 2k + (l/16)
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t qa = W(16 * n + i), qb = W(16 * n + 8 + i), qh = W(32 + 8 * n + i);
        uint32_t q0, q1;
        if (kp == 0) {
            q0 = (qa & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u);
            q1 = (qb & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u);
        } else {
            q0 = ((qa >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u);
            q1 = ((qb >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u);
        }
        const int h = i >> 2;                            // l / 16
        out[2 * i] = h2_bits(__hmul2(codes01(q0, k1056), S[h]));
        out[2 * i + 1] = h2_bits(__hmul2(codes23(q0, k1056), S[h]));
        out[16 + 2 * i] = h2_bits(__hmul2(codes01(q1, k1056), S[2 + h]));
        out[16 + 2 * i + 1] = h2_bits(__hmul2(codes23(q1, k1056), S[2 + h]));
    }
}

// Q4_0 / Q8_0: eight 32-element blocks per K-block; element-wise decode (correct, not tuned).
template <uint32_t TYPE>
__device__ __forceinline__ void dq_legacy(const uint8_t* row, int qd, uint32_t (&out)[32]) {
    constexpr BlockGeom G = block_geom(TYPE);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        const uint8_t* blk = row + (2 * qd + b) * G.bytes;
#pragma unroll
        for (int e = 0; e < 32; e += 2)
            out[16 * b + e / 2] = pack_h2(dequant_elem<TYPE>(blk, e), dequant_elem<TYPE>(blk, e + 1));
    }
}

template <uint32_t TYPE, int OFF>
__device__ __forceinline__ void dequant_row_to_tmem(const uint8_t* row, uint32_t taddr) {
    if constexpr (TYPE == HF2Q_TYPE_Q4_K || TYPE == HF2Q_TYPE_Q5_K) {
        constexpr int NW = TYPE == HF2Q_TYPE_Q4_K ? 36 : 44;
        uint32_t P[NW];
#pragma unroll
        for (int u = 0; u < NW / 4; ++u) {
            const uint4 v = reinterpret_cast<const uint4*>(row)[u];
            P[4 * u] = v.x; P[4 * u + 1] = v.y; P[4 * u + 2] = v.z; P[4 * u + 3] = v.w;
        }
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            uint32_t out[32];
            dq_k45<TYPE == HF2Q_TYPE_Q5_K>(P, qd, out);
            tmem_st32(taddr + 32 * qd, out);
        }
    } else if constexpr (TYPE == HF2Q_TYPE_Q6_K) {
        uint32_t P[60];
#pragma unroll
        for (int u = 0; u < 15; ++u) {
            const uint4 v = reinterpret_cast<const uint4*>(row)[u];
            P[4 * u] = v.x; P[4 * u + 1] = v.y; P[4 * u + 2] = v.z; P[4 * u + 3] = v.w;
        }
        auto W = [&](int j) -> uint32_t {
            if constexpr (OFF % 4 == 0) return P[j + OFF / 4];
            else return __funnelshift_r(P[j + OFF / 4], P[j + OFF / 4 + 1], 16);
        };
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            uint32_t out[32];
            dq_q6k(W, qd, out);
            tmem_st32(taddr + 32 * qd, out);
        }
    } else {
#pragma unroll 1
        for (int qd = 0; qd < 4; ++qd) {
            uint32_t out[32];
            dq_legacy<TYPE>(row, qd, out);
            tmem_st32(taddr + 32 * qd, out);
        }
    }
}

template <uint32_t TYPE>
__device__ __forceinline__ void dequant_dispatch(const uint8_t* row, uint32_t off, uint32_t taddr) {
    if constexpr (TYPE == HF2Q_TYPE_Q6_K) {
        switch (off) {   // byte offset of the block inside its 16-byte aligned box; warp-uniform
            case 0: dequant_row_to_tmem<TYPE, 0>(row, taddr); break;
            case 2: dequant_row_to_tmem<TYPE, 2>(row, taddr); break;
            case 4: dequant_row_to_tmem<TYPE, 4>(row, taddr); break;
            case 6: dequant_row_to_tmem<TYPE, 6>(row, taddr); break;
            case 8: dequant_row_to_tmem<TYPE, 8>(row, taddr); break;
            case 10: dequant_row_to_tmem<TYPE, 10>(row, taddr); break;
            case 12: dequant_row_to_tmem<TYPE, 12>(row, taddr); break;
            default: dequant_row_to_tmem<TYPE, 14>(row, taddr); break;
        }
    } else {
        dequant_row_to_tmem<TYPE, 0>(row, taddr);
    }
}

// ---------------------------------------------------------------- the kernel
template <uint32_t TYPE, int NT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const GParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    constexpr uint32_t X_STAGE = NT * 128;                       // NT rows x 64 f16, 128B-swizzled
    uint8_t* xs = smem;                                          // X_STAGES x X_STAGE (1024-aligned)
    constexpr int RAW_STAGES = raw_stages_of(TYPE);
    uint8_t* raw = xs + X_STAGES * X_STAGE;                      // RAW_STAGES x 128 x boxw
    const uint32_t raw_stage = TILE_N * p.boxw;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw + RAW_STAGES * raw_stage);
    uint64_t* raw_full = bars;                  // [RAW_STAGES]
    uint64_t* raw_empty = raw_full + RAW_STAGES;
    uint64_t* x_full = raw_empty + RAW_STAGES;  // [X_STAGES]
    uint64_t* x_empty = x_full + X_STAGES;
    uint64_t* a_full = x_empty + X_STAGES;      // [2]
    uint64_t* a_empty = a_full + 2;
    uint64_t* d_full = a_empty + 2;             // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row0 = blockIdx.x * TILE_N, tok0 = blockIdx.y * NT;
    const uint32_t nkb = p.k / KB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RAW_STAGES; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], 4); }
        for (int s = 0; s < X_STAGES; ++s) { mbar_init(&x_full[s], 1); mbar_init(&x_empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&a_full[s], 4); mbar_init(&a_empty[s], 1); }
        mbar_init(d_full, 1);
        mbar_fence_init();
    }
    if (warp == 5) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_d = tmem_base;                 // columns [0, NT)
    const uint32_t tmem_a = tmem_base + 256;           // two buffers of 128 columns

    if (warp == 4) {
        // ------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
                const uint32_t rs = kb % RAW_STAGES;
                if (kb >= RAW_STAGES) ok = mbar_wait_bounded(&raw_empty[rs], ((kb / RAW_STAGES) - 1) & 1, p.status);
                if (!ok) break;
                mbar_arrive_expect_tx(&raw_full[rs], raw_stage);
                const uint32_t byte0 = (kb * p.blk_bytes) & ~15u;       // 16-byte aligned start of the box
                tma_2d(raw + rs * raw_stage, &tmap_w, static_cast<int>(byte0 >> 1), static_cast<int>(row0), &raw_full[rs]);
                for (uint32_t j = 0; j < KB / XK && ok; ++j) {
                    const uint32_t xi = kb * (KB / XK) + j, st = xi % X_STAGES;
                    if (xi >= X_STAGES) ok = mbar_wait_bounded(&x_empty[st], ((xi / X_STAGES) - 1) & 1, p.status);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&x_full[st], X_STAGE);
                    tma_2d(xs + st * X_STAGE, &tmap_x, static_cast<int>(kb * KB + j * XK), static_cast<int>(tok0), &x_full[st]);
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor: D f32, A/B f16, both K-major, N = NT, M = 128
            constexpr uint32_t IDESC = (1u << 4) | (static_cast<uint32_t>(NT >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
                const uint32_t ab = kb & 1;
                ok = mbar_wait_bounded(&a_full[ab], (kb >> 1) & 1, p.status);
                if (!ok) break;
                tc_fence_after();
                for (uint32_t j = 0; j < KB / XK && ok; ++j) {
                    const uint32_t xi = kb * (KB / XK) + j, st = xi % X_STAGES;
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
                    tc_commit(&x_empty[st]);       // activation stage free once these MMAs retire
                }
                if (ok) tc_commit(&a_empty[ab]);
            }
            if (ok) tc_commit(d_full);
        }
    } else {
        // ------------------------------ dequantisers (thread = weight row), then epilogue
        const uint32_t r = threadIdx.x;                    // 0..127 == TMEM lane
        const uint32_t lane_addr = (static_cast<uint32_t>(warp) * 32u) << 16;
        bool ok = true;
        for (uint32_t kb = 0; kb < nkb; ++kb) {
            const uint32_t rs = kb % RAW_STAGES, ab = kb & 1;
            if (ok) ok = mbar_wait_bounded(&raw_full[rs], (kb / RAW_STAGES) & 1, p.status);
            if (ok && kb >= 2) ok = mbar_wait_bounded(&a_empty[ab], ((kb >> 1) - 1) & 1, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t off = (kb * p.blk_bytes) & 15u;
            dequant_dispatch<TYPE>(raw + rs * raw_stage + r * p.boxw, off, tmem_a + ab * 128 + lane_addr);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&a_full[ab]); mbar_arrive(&raw_empty[rs]); }
        }
        // epilogue
        if (ok) ok = mbar_wait_bounded(d_full, 0, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            const uint32_t row = row0 + r;
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_d + lane_addr + c0, v);
                tmem_wait_ld();
                if (row < p.n) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t tok = tok0 + c0 + j;
                        if (tok < p.m) p.y[static_cast<size_t>(tok) * p.n + row] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
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

uint32_t boxw_of(uint32_t type) {
    switch (type) {
        case HF2Q_TYPE_Q4_K: return 144;
        case HF2Q_TYPE_Q5_K: return 176;
        case HF2Q_TYPE_Q6_K: return 240;     // 210 bytes at an offset of 0..14, pitch 15 x 16 bytes
        case HF2Q_TYPE_Q4_0: return 144;     // 8 blocks
        case HF2Q_TYPE_Q8_0: return 272;     // 8 blocks
        default: return 0;
    }
}

template <uint32_t TYPE, int NT>
cudaError_t launch_gemm_t(const CUtensorMap& tw, const CUtensorMap& tx, const GParams& p, cudaStream_t st) {
    auto kern = gemm_tc_kernel<TYPE, NT>;
    const size_t smem = 1024 + static_cast<size_t>(X_STAGES) * NT * 128 + static_cast<size_t>(raw_stages_of(TYPE)) * TILE_N * p.boxw + 256;
    static std::mutex mu;
    static bool attr_set = false;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return e;
            attr_set = true;
        }
    }
    const dim3 grid((p.n + TILE_N - 1) / TILE_N, (p.m + NT - 1) / NT);
    kern<<<grid, GEMM_THREADS, smem, st>>>(tw, tx, p);
    return cudaGetLastError();
}

template <uint32_t TYPE>
cudaError_t launch_gemm_nt(const CUtensorMap& tw, const CUtensorMap& tx, const GParams& p, uint32_t nt, cudaStream_t st) {
    switch (nt) {
        case 32: return launch_gemm_t<TYPE, 32>(tw, tx, p, st);
        case 64: return launch_gemm_t<TYPE, 64>(tw, tx, p, st);
        case 128: return launch_gemm_t<TYPE, 128>(tw, tx, p, st);
        default: return launch_gemm_t<TYPE, 256>(tw, tx, p, st);
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

// Tokens per CTA tile for m activation rows.
uint32_t gemm_tc_token_tile(uint32_t m) { return m > 128 ? 256 : m > 64 ? 128 : m > 32 ? 64 : 32; }

cudaError_t launch_gemm_tc(uint32_t type, const void* w, const void* x, uint32_t x_dtype, float* y, uint32_t m, uint32_t n,
                           uint32_t k, void* workspace, uint32_t* status, int sm_count, cudaStream_t st, int* launches) {
    const BlockGeom g = block_geom(type);
    const uint64_t row_bytes = static_cast<uint64_t>(k) / g.elems * g.bytes;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;

    // 1. activations -> f16 [m][k] in the workspace
    __half* xh = static_cast<__half*>(workspace);
    const uint64_t nx = static_cast<uint64_t>(m) * k;
    {
        uint64_t want = (nx + 255) / 256;
        const uint64_t cap = static_cast<uint64_t>(sm_count) * 16;
        x_to_f16_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, st>>>(x, x_dtype == HF2Q_DT_BF16, xh, nx, status);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    // 2. tensor maps
    GParams p{};
    p.y = y; p.m = m; p.n = n; p.k = k;
    p.boxw = boxw_of(type);
    p.blk_bytes = KB / g.elems * g.bytes;
    p.status = status;
    const uint32_t nt = gemm_tc_token_tile(m);
    alignas(64) CUtensorMap tw, tx;
    {
        // weights: [n rows][row_bytes] viewed as u16, box = boxw bytes x 128 rows, no swizzle
        cuuint64_t dims[2] = {row_bytes / 2, n};
        cuuint64_t strides[1] = {row_bytes};
        cuuint32_t box[2] = {p.boxw / 2, TILE_N};
        cuuint32_t es[2] = {1, 1};
        CUresult r = enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(w), dims, strides, box, es,
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
    if (launches) *launches = 2;
    switch (type) {
        case HF2Q_TYPE_Q4_0: return launch_gemm_nt<HF2Q_TYPE_Q4_0>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q8_0: return launch_gemm_nt<HF2Q_TYPE_Q8_0>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q4_K: return launch_gemm_nt<HF2Q_TYPE_Q4_K>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q5_K: return launch_gemm_nt<HF2Q_TYPE_Q5_K>(tw, tx, p, nt, st);
        case HF2Q_TYPE_Q6_K: return launch_gemm_nt<HF2Q_TYPE_Q6_K>(tw, tx, p, nt, st);
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
