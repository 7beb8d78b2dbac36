// Shared device/host helpers for the GGUF block formats on the quantized-matmul path.
//
// Block layouts and the dequantisation formulas are the inverse of hf2q's quantizers' re-encode
// step (src/quantize/ggml_quants/q4_0.rs:47-64, q8_0.rs:59-67, q4_k.rs:183-215 + 329-337,
// q5_k.rs:100-158, q6_k.rs:96-143); sizes follow ggml_type.rs:60-133.  The four 32-element fall-back
// formats (q4_1.rs, q5_0.rs, q5_1.rs, iq4_nl.rs) dequantise to the value their quantizers' error
// terms assign to a code: d*q + m, (q - 16)*d and d*kvalues[q].
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hf2q_cuda.h"

namespace hf2q {

constexpr int QK_K = 256;

// Device status word bits (read back by hf2q_cuda_check_status).
enum : uint32_t {
    STATUS_WAIT_TIMEOUT = 1u,   // a bounded mbarrier wait gave up
    STATUS_BAD_EXPERT_ID = 2u,  // ids[] held a value >= n_experts
    STATUS_X_CLIPPED = 4u,      // an activation exceeded the f16 range (65504) and was clipped
};

struct BlockGeom { uint32_t elems, bytes; };

__host__ __device__ constexpr bool type_supported(uint32_t t) {
    return t == HF2Q_TYPE_Q4_0 || t == HF2Q_TYPE_Q8_0 || t == HF2Q_TYPE_Q4_K ||
           t == HF2Q_TYPE_Q5_K || t == HF2Q_TYPE_Q6_K || t == HF2Q_TYPE_Q4_1 || t == HF2Q_TYPE_Q5_0 ||
           t == HF2Q_TYPE_Q5_1 || t == HF2Q_TYPE_IQ4_NL || t == HF2Q_TYPE_MLX_AFFINE4_GS32;
}
// the 32-element formats hf2q's quantizer falls back to (standard_policy.rs:128-192), and the mlx-affine container:
// all of them run on the generic element-wise consumers
__host__ __device__ constexpr bool type_is_fallback32(uint32_t t) {
    return t == HF2Q_TYPE_Q4_1 || t == HF2Q_TYPE_Q5_0 || t == HF2Q_TYPE_Q5_1 || t == HF2Q_TYPE_IQ4_NL || t == HF2Q_TYPE_MLX_AFFINE4_GS32;
}
__host__ __device__ constexpr BlockGeom block_geom(uint32_t t) {
    return t == HF2Q_TYPE_Q4_0 ? BlockGeom{32, 18}
         : t == HF2Q_TYPE_Q8_0 ? BlockGeom{32, 34}
         : t == HF2Q_TYPE_Q4_K ? BlockGeom{256, 144}
         : t == HF2Q_TYPE_Q5_K ? BlockGeom{256, 176}
         : t == HF2Q_TYPE_Q6_K ? BlockGeom{256, 210}
         : t == HF2Q_TYPE_Q4_1 ? BlockGeom{32, 20}
         : t == HF2Q_TYPE_Q5_0 ? BlockGeom{32, 22}
         : t == HF2Q_TYPE_Q5_1 ? BlockGeom{32, 24}
         : t == HF2Q_TYPE_IQ4_NL ? BlockGeom{32, 18}
         : t == HF2Q_TYPE_MLX_AFFINE4_GS32 ? BlockGeom{32, 24}
                               : BlockGeom{0, 0};
}

// ---- unaligned little-endian field access (blocks are only 2-byte aligned in general) --------
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) {
    return *reinterpret_cast<const uint16_t*>(p);
}
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) {   // p is 2-byte aligned
    return ld_u16(p) | (ld_u16(p + 2) << 16);
}
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

// 6-bit scale / min of sub-block j from the 12 packed bytes held as three little-endian words
// s0 = bytes 0..3, s1 = bytes 4..7, s2 = bytes 8..11 (get_scale_min_k4, q4_k.rs:329-337).
__device__ __forceinline__ void scale_min_k4(int j, uint32_t s0, uint32_t s1, uint32_t s2,
                                             uint32_t& sc, uint32_t& mn) {
    if (j < 4) {
        sc = (s0 >> (8 * j)) & 63u;
        mn = (s1 >> (8 * j)) & 63u;
    } else {
        const int sh = 8 * (j - 4);
        const uint32_t b2 = (s2 >> sh) & 0xffu;
        sc = (b2 & 0xFu) | ((((s0 >> sh) & 0xffu) >> 6) << 4);
        mn = (b2 >> 4) | ((((s1 >> sh) & 0xffu) >> 6) << 4);
    }
}

// The IQ4_NL codebook (iq4_nl.rs KVALUES_IQ4NL) as four packed words of signed bytes.
__device__ __forceinline__ int iq4nl_value(uint32_t code) {
    // -127 -104 -83 -65 | -49 -35 -22 -10 | 1 13 25 38 | 53 69 89 113   (little-endian bytes)
    const uint32_t w = code < 8 ? (code < 4 ? 0xBFAD9881u : 0xF6EADDCFu) : (code < 12 ? 0x26190D01u : 0x71594535u);
    return static_cast<int>(static_cast<int8_t>((w >> (8 * (code & 3u))) & 0xffu));
}

// Value of element e (0 <= e < block elems) of one block, in f32, bit-exact with the oracle:
// every product below is exact in f32 (11-bit f16 significand x 6..8-bit scale x <= 6-bit code),
// and the single subtraction of Q4_K/Q5_K rounds the same exact value with or without FMA
// contraction.  Byte-granular loads: works for any 2-byte aligned block.
template <uint32_t TYPE>
__device__ __forceinline__ float dequant_elem(const uint8_t* __restrict__ b, int e) {
    if constexpr (TYPE == HF2Q_TYPE_Q4_0) {
        const float d = f16_bits_to_f32(ld_u16(b));
        const uint32_t q = b[2 + (e & 15)];
        const int v = static_cast<int>(e < 16 ? (q & 15u) : (q >> 4)) - 8;
        return static_cast<float>(v) * d;
    } else if constexpr (TYPE == HF2Q_TYPE_Q8_0) {
        const float d = f16_bits_to_f32(ld_u16(b));
        return static_cast<float>(static_cast<int8_t>(b[2 + e])) * d;
    } else if constexpr (TYPE == HF2Q_TYPE_Q4_1) {
        const float d = f16_bits_to_f32(ld_u16(b)), m = f16_bits_to_f32(ld_u16(b + 2));
        const uint32_t q = b[4 + (e & 15)];
        return __fadd_rn(__fmul_rn(d, static_cast<float>(e < 16 ? (q & 15u) : (q >> 4))), m);
    } else if constexpr (TYPE == HF2Q_TYPE_Q5_0 || TYPE == HF2Q_TYPE_Q5_1) {
        constexpr int O = TYPE == HF2Q_TYPE_Q5_0 ? 2 : 4;            // qh follows d (and m)
        const float d = f16_bits_to_f32(ld_u16(b));
        const uint32_t qh = ld_u32_a2(b + O);
        const uint32_t v = b[O + 4 + (e & 15)];
        const uint32_t q = (e < 16 ? (v & 15u) : (v >> 4)) | (((qh >> e) & 1u) << 4);
        if constexpr (TYPE == HF2Q_TYPE_Q5_0) return static_cast<float>(static_cast<int>(q) - 16) * d;
        else return __fadd_rn(__fmul_rn(d, static_cast<float>(q)), f16_bits_to_f32(ld_u16(b + 2)));
    } else if constexpr (TYPE == HF2Q_TYPE_IQ4_NL) {
        const float d = f16_bits_to_f32(ld_u16(b));
        const uint32_t v = b[2 + (e & 15)];
        return d * static_cast<float>(iq4nl_value(e < 16 ? (v & 15u) : (v >> 4)));
    } else if constexpr (TYPE == HF2Q_TYPE_MLX_AFFINE4_GS32) {
        // f32 scale, f32 bias, codes in element order (element e = nibble e): scale * code + bias, two roundings
        const float sc = __uint_as_float(ld_u32_a2(b)), bias = __uint_as_float(ld_u32_a2(b + 4));
        const uint32_t q = (b[8 + (e >> 1)] >> (4 * (e & 1))) & 15u;
        return __fadd_rn(__fmul_rn(sc, static_cast<float>(q)), bias);
    } else if constexpr (TYPE == HF2Q_TYPE_Q4_K || TYPE == HF2Q_TYPE_Q5_K) {
        const float d = f16_bits_to_f32(ld_u16(b));
        const float dmin = f16_bits_to_f32(ld_u16(b + 2));
        const uint32_t s0 = ld_u32_a2(b + 4), s1 = ld_u32_a2(b + 8), s2 = ld_u32_a2(b + 12);
        const int c = e >> 6, hi = (e >> 5) & 1, l = e & 31;
        uint32_t sc, mn;
        scale_min_k4(2 * c + hi, s0, s1, s2, sc, mn);
        uint32_t q;
        if constexpr (TYPE == HF2Q_TYPE_Q4_K) {
            const uint32_t v = b[16 + 32 * c + l];
            q = hi ? (v >> 4) : (v & 15u);
        } else {
            const uint32_t v = b[48 + 32 * c + l];
            const uint32_t h = (b[16 + l] >> (2 * c + hi)) & 1u;
            q = (hi ? (v >> 4) : (v & 15u)) + 16u * h;
        }
        const float d1 = d * static_cast<float>(sc);
        const float m1 = dmin * static_cast<float>(mn);
        return d1 * static_cast<float>(q) - m1;
    } else {   // Q6_K
        const int n = e >> 7, k = (e >> 5) & 3, l = e & 31;
        const uint32_t qlb = b[64 * n + l + 32 * (k & 1)];
        const uint32_t lo = (k < 2) ? (qlb & 15u) : (qlb >> 4);
        const uint32_t hi = (b[128 + 32 * n + l] >> (2 * k)) & 3u;
        const int q = static_cast<int>(lo | (hi << 4)) - 32;
        const float sc = static_cast<float>(static_cast<int8_t>(b[192 + (e >> 4)]));
        const float d = f16_bits_to_f32(ld_u16(b + 208));
        return (d * sc) * static_cast<float>(q);
    }
}

// Byte k (0..3) of a packed word as an exact float: PRMT drops the byte into the low mantissa
// byte of 2^23, the subtraction removes 2^23 (+ bias) exactly.
template <int BIAS>
__device__ __forceinline__ float byte_to_float(uint32_t w, int k) {
    const uint32_t bits = __byte_perm(w, 0x4B000000u, 0x7650u + static_cast<uint32_t>(k));
    return __uint_as_float(bits) - (8388608.0f + static_cast<float>(BIAS));
}

// ---- mbarrier / bulk-copy PTX (sm_90+; used here for sm_100a only) ----------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Same probe, but the hardware may park the thread for up to `ns` nanoseconds while the phase is
// incomplete (it resumes at once when the phase completes): far fewer polling instructions.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^31 clock ticks (about a second), records it in *status and
// returns false so the caller can leave its loop with the context intact.  The first probe is
// checked before the clock is read at all; later probes let the hardware park the thread.
template <uint32_t SLEEP_NS>
__device__ __forceinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, uint32_t* status) {
    const long long t0 = clock64();
    for (uint32_t n = 1;; ++n) {
        if (mbar_try_wait_parked(bar, parity, 2000u)) return true;
        if constexpr (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if ((n & 15u) == 0 && clock64() - t0 > (1ll << 31)) {
            if (status) atomicOr(status, STATUS_WAIT_TIMEOUT);
            return false;
        }
    }
}
template <uint32_t SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t* status) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow<SLEEP_NS>(bar, parity, status);
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
// dst, src and bytes must be multiples of 16.  The copy targets this CTA only.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// The same copy with an L2 eviction policy (from l2_policy_evict_first): bytes that are read once
// should not push re-used data (activations, outputs) out of L2.
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_normal() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

}  // namespace hf2q
