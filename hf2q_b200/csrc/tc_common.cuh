// Device helpers of the tcgen05 kernels (k2_gemm_tc.cu): PTX wrappers for
// TMA tensor copies, tensor-memory allocation / load / store, tcgen05.mma issue and commit, and the
// per-row block dequantisers that produce f16x2 registers in natural element order.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace hf2q {
namespace tc {

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void tma_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
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
// high nibbles sub-block 2c+1;  w = d*sc*q - dmin*m, rounded to f16.
template <bool Q5>
__device__ __forceinline__ void dq_k45(const uint32_t* P, int c, uint32_t (&out)[32]) {
    constexpr int QW = Q5 ? 12 : 4;         // first qs word
    const float d = f16_bits_to_f32(P[0] & 0xffffu), dmin = f16_bits_to_f32(P[0] >> 16);
    uint32_t sc1, m1, sc2, m2;
    scale_min_k4(2 * c, P[1], P[2], P[3], sc1, m1);
    scale_min_k4(2 * c + 1, P[1], P[2], P[3], sc2, m2);
    // w = d*sc*q - dmin*m is a difference of two terms several times larger than w, so rounding
    // d*sc and dmin*m to f16 separately would cost accuracy.  Re-centre instead:
    //   w = (q - q0) * S + r,   S = f16(d*sc),  q0 = round(dmin*m / S),  r = f16(q0*S - dmin*m)
    // (q - q0) is an exact small integer, |r| <= S/2, and only S carries a relative error.
    // The scale itself is carried as S + L (f16 hi + lo parts of d*sc), so the only rounding that
    // is left is the final one to f16:  w = (q-q0)*S + ((q-q0)*L + r).
    auto centre = [&](uint32_t sc, uint32_t mn, __half2& S, __half2& L, __half2& R, __half2& B) {
        const float s_full = d * static_cast<float>(sc), mf = dmin * static_cast<float>(mn);
        const __half s_h = __float2half_rn(s_full);
        const float s_f = __half2float(s_h);
        float q0 = s_full != 0.f ? rintf(__fdividef(mf, s_full)) : 0.f;
        q0 = fminf(fmaxf(q0, 0.f), 960.f);                                   // keeps 1024 + q0 exact in f16
        S = __half2half2(s_h);
        L = __float2half2_rn(s_full - s_f);
        R = __float2half2_rn(fmaf(q0, s_full, -mf));
        B = __float2half2_rn(1024.0f + q0);
    };
    __half2 S1, L1, M1, B1, S2, L2, M2, B2;
    centre(sc1, m1, S1, L1, M1, B1);
    centre(sc2, m2, S2, L2, M2, B2);
    auto value = [](__half2 q, __half2 S, __half2 L, __half2 R) { return h2_bits(__hfma2(q, S, __hfma2(q, L, R))); };
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t w = P[QW + 8 * c + i];
        uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
        if constexpr (Q5) {
            const uint32_t g = P[4 + i];
            lo |= ((g >> (2 * c)) & 0x01010101u) << 4;
            hi |= ((g >> (2 * c + 1)) & 0x01010101u) << 4;
        }
        out[2 * i] = value(codes01(lo, B1), S1, L1, M1);
        out[2 * i + 1] = value(codes23(lo, B1), S1, L1, M1);
        out[16 + 2 * i] = value(codes01(hi, B2), S2, L2, M2);
        out[16 + 2 * i + 1] = value(codes23(hi, B2), S2, L2, M2);
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
    __half2 S[4], L[4];                                  // d*scale as f16 hi + lo parts
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float s = d * static_cast<float>(static_cast<int8_t>((scw >> (8 * j)) & 0xffu));
        const __half sh = __float2half_rn(s);            // sub-block 8n + 4kp + j = 8n + 2k + (l/16)
        S[j] = __half2half2(sh);
        L[j] = __float2half2_rn(s - __half2float(sh));
    }
    auto value = [](__half2 q, __half2 Sh, __half2 Lo) { return h2_bits(__hfma2(q, Sh, __hmul2(q, Lo))); };
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
        out[2 * i] = value(codes01(q0, k1056), S[h], L[h]);
        out[2 * i + 1] = value(codes23(q0, k1056), S[h], L[h]);
        out[16 + 2 * i] = value(codes01(q1, k1056), S[2 + h], L[2 + h]);
        out[16 + 2 * i + 1] = value(codes23(q1, k1056), S[2 + h], L[2 + h]);
    }
}

// Q4_0 / Q8_0 / Q4_1 / Q5_0 / Q5_1 / IQ4_NL: eight 32-element blocks per K-block; element-wise decode (correct, not tuned).
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


// One 256-element K-block of one weight row, held by the thread that owns the row.  load() pulls
// the raw bytes out of shared memory (16-byte vectors), quarter() yields elements 64qd..64qd+63 as
// 32 f16x2 registers.  OFF is the byte offset of the block inside its 16-byte aligned box (only
// Q6_K blocks, 210 bytes, ever sit at a non-zero offset).  IN_REGS: the stage may be released
// right after load().
template <uint32_t TYPE, int ODD>
struct RowBlock {
    static constexpr bool IN_REGS = TYPE == HF2Q_TYPE_Q4_K || TYPE == HF2Q_TYPE_Q5_K || TYPE == HF2Q_TYPE_Q6_K;
    static constexpr int NW = TYPE == HF2Q_TYPE_Q4_K ? 36 : TYPE == HF2Q_TYPE_Q5_K ? 44 : TYPE == HF2Q_TYPE_Q6_K ? 56 : 1;
    uint32_t P[NW];
    const uint8_t* row;
    // off: byte offset of the block inside its 16-byte aligned box (Q6_K only; warp-uniform).
    // The word part of the offset (off/4 = 0..3) is removed with two conditional register shifts,
    // so one code path serves all eight offsets; ODD says whether 2 more bytes remain.
    __device__ __forceinline__ void load(const uint8_t* r, uint32_t off) {
        row = r;
        if constexpr (TYPE == HF2Q_TYPE_Q6_K) {
            uint32_t T[60];
#pragma unroll
            for (int u = 0; u < 15; ++u) {
                const uint4 v = reinterpret_cast<const uint4*>(r)[u];
                T[4 * u] = v.x; T[4 * u + 1] = v.y; T[4 * u + 2] = v.z; T[4 * u + 3] = v.w;
            }
            const bool s1 = (off >> 2) & 1u, s2 = (off >> 3) & 1u;
#pragma unroll
            for (int j = 0; j < 59; ++j) T[j] = s1 ? T[j + 1] : T[j];
#pragma unroll
            for (int j = 0; j < 57; ++j) T[j] = s2 ? T[j + 2] : T[j];
#pragma unroll
            for (int j = 0; j < NW; ++j) P[j] = T[j];
        } else if constexpr (IN_REGS) {
#pragma unroll
            for (int u = 0; u < NW / 4; ++u) {
                const uint4 v = reinterpret_cast<const uint4*>(r)[u];
                P[4 * u] = v.x; P[4 * u + 1] = v.y; P[4 * u + 2] = v.z; P[4 * u + 3] = v.w;
            }
        }
    }
    __device__ __forceinline__ void quarter(int qd, uint32_t (&out)[32]) const {
        if constexpr (TYPE == HF2Q_TYPE_Q4_K) dq_k45<false>(P, qd, out);
        else if constexpr (TYPE == HF2Q_TYPE_Q5_K) dq_k45<true>(P, qd, out);
        else if constexpr (TYPE == HF2Q_TYPE_Q6_K) {
            auto W = [&](int j) -> uint32_t {
                if constexpr (ODD == 0) return P[j];
                else return __funnelshift_r(P[j], P[j + 1], 16);
            };
            dq_q6k(W, qd, out);
        } else dq_legacy<TYPE>(row, qd, out);
    }
};

// Calls f(RowBlock<TYPE, odd>{}) for the parity of `off` (warp-uniform).
template <uint32_t TYPE, typename F>
__device__ __forceinline__ void with_row_block(uint32_t off, F&& f) {
    if constexpr (TYPE == HF2Q_TYPE_Q6_K) {
        if (off & 2u) f(RowBlock<TYPE, 1>{});
        else f(RowBlock<TYPE, 0>{});
    } else {
        f(RowBlock<TYPE, 0>{});
    }
}

// bytes per weight row of one 256-element K-block as staged in shared memory (the tensor-map box)
__host__ __device__ constexpr uint32_t tc_boxw(uint32_t type) {
    return type == HF2Q_TYPE_Q4_K ? 144u : type == HF2Q_TYPE_Q5_K ? 176u
         : type == HF2Q_TYPE_Q6_K ? 240u   // 210 bytes at an offset of 0..14; pitch of 15 x 16 bytes
         : type == HF2Q_TYPE_Q4_0 ? 144u : type == HF2Q_TYPE_Q8_0 ? 272u
         : type == HF2Q_TYPE_Q4_1 ? 160u : type == HF2Q_TYPE_Q5_0 ? 176u : type == HF2Q_TYPE_Q5_1 ? 192u
         : type == HF2Q_TYPE_IQ4_NL ? 144u : type == HF2Q_TYPE_MLX_AFFINE4_GS32 ? 192u : 0u;
}

}  // namespace tc
}  // namespace hf2q
