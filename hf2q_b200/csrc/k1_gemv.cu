// K1 / K3: dequant-fused mat-vec for 1..8 activation rows, dense and expert-routed.
//
//   y[t, r] = sum_k x[t, k] * dequant(W)[r, k]          (fp32 multiply-add, fp32 accumulate)
//
// Stands in for mlx-native's kernel_mul_mv_<q>_f32 / kernel_mul_mv_id_<q>_f32 that hf2q reaches
// through quantized_matmul_ggml (m <= 8; src/inference/models/qwen35/gpu_ffn.rs:1236-1306,
// src/serve/forward_mlx.rs:9960-9968) and quantized_matmul_id_ggml (few rows; gpu_ffn.rs:188-206,
// forward_mlx.rs:5285-5292).  It is HBM-bound, so it uses no tensor cores:
//
//   * a persistent CTA per SM slot owns groups of 8 weight rows (one row per consumer warp);
//   * a producer warp streams the RAW block bytes of those rows into a 4-deep shared-memory ring
//     with 1-D bulk copies (cp.async.bulk, completion on an mbarrier), 2048 elements per row and
//     stage, so 18/34/210-byte blocks can be read at any 2-byte offset without repacking;
//   * consumers unpack nibbles / 5- and 6-bit codes in registers as whole 32-bit words, turn
//     bytes into floats with a PRMT into the mantissa of 2^23, and apply the block and sub-block
//     scales once per group of codes, not per element;
//   * the activation rows are converted to f32 once per CTA and kept in shared memory together
//     with their 16-element partial sums (the `- dmin*m` term of Q4_K/Q5_K needs only those);
//   * each row's partial sums are reduced with warp shuffles; no atomics, deterministic.
//
// Rows whose byte length is not a multiple of 16 (e.g. Q6_K with k = 512, Q4_0 with k = 32)
// cannot be bulk-copied and take the simple warp-per-row kernel at the end of this file.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace hf2q {

namespace {

constexpr int ROWS = 8;            // consumer warps == weight rows per stage
constexpr int STAGES = 4;
constexpr int SLICE_ELEMS = 2048;  // elements of one row per stage (multiple of every block size)
constexpr int THREADS = (ROWS + 1) * 32;

struct KParams {
    const uint8_t* w;
    const void* x;
    float* y;
    const uint32_t* ids;
    uint64_t expert_stride;
    uint32_t x_bf16;       // 1: x is bf16, 0: f32
    uint32_t m;            // live activation rows (<= M)
    uint32_t n, k;
    uint32_t top_k, n_experts;
    uint32_t row_bytes;    // bytes of one weight row
    uint32_t slice_bytes;  // bytes of a full 2048-element slice
    uint32_t nslices;
    uint32_t ngroups;      // ceil(n / ROWS)
    uint32_t* status;
};

// ---- activation access --------------------------------------------------------------------
template <bool XSMEM>
struct XAcc {
    const float* xs;     // [M][k] f32 in shared memory (XSMEM)
    const void* xg;      // global base of this slot's first activation row
    uint32_t k, x_bf16, m;
    __device__ __forceinline__ float4 ld4(int t, uint32_t e) const {
        if constexpr (XSMEM) {
            return *reinterpret_cast<const float4*>(xs + static_cast<size_t>(t) * k + e);
        } else {
            const uint32_t tt = static_cast<uint32_t>(t) < m ? t : m - 1;   // padded rows alias
            if (x_bf16) {
                const uint2 r = __ldg(reinterpret_cast<const uint2*>(
                    static_cast<const __nv_bfloat16*>(xg) + static_cast<size_t>(tt) * k + e));
                return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                                   __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
            }
            return __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(xg) +
                                                         static_cast<size_t>(tt) * k + e));
        }
    }
};

__device__ __forceinline__ float dot4(uint32_t w, float4 x) {
    return byte_to_float<0>(w, 0) * x.x + byte_to_float<0>(w, 1) * x.y +
           byte_to_float<0>(w, 2) * x.z + byte_to_float<0>(w, 3) * x.w;
}
template <int BIAS>
__device__ __forceinline__ float dot4b(uint32_t w, float4 x) {
    return byte_to_float<BIAS>(w, 0) * x.x + byte_to_float<BIAS>(w, 1) * x.y +
           byte_to_float<BIAS>(w, 2) * x.z + byte_to_float<BIAS>(w, 3) * x.w;
}

// ---- per-format slice consumers -------------------------------------------------------------
// sb: this warp's row slice in shared memory (16-byte aligned), nblk blocks, first element kbase.
// xsum: [M][k/16] partial sums of x (Q4_K / Q5_K only).

template <uint32_t TYPE, int M, bool XSMEM>
__device__ __forceinline__ void consume_k45(const uint8_t* sb, int nblk, uint32_t kbase,
                                            const XAcc<XSMEM>& xa, const float* xsum,
                                            float (&acc)[M], int lane) {
    constexpr int BB = TYPE == HF2Q_TYPE_Q4_K ? 144 : 176;
    constexpr int QS = TYPE == HF2Q_TYPE_Q4_K ? 16 : 48;
    const int nunits = nblk * 8;                // (block, chunk c of 64, half h of 16 bytes)
    for (int u = lane; u < nunits; u += 32) {
        const int b = u >> 3, c = (u >> 1) & 3, h = u & 1;
        const uint8_t* blk = sb + b * BB;
        const uint4 hd = *reinterpret_cast<const uint4*>(blk);
        const uint4 q = *reinterpret_cast<const uint4*>(blk + QS + 32 * c + 16 * h);
        uint4 lo, hi;
        lo.x = q.x & 0x0F0F0F0Fu; hi.x = (q.x >> 4) & 0x0F0F0F0Fu;
        lo.y = q.y & 0x0F0F0F0Fu; hi.y = (q.y >> 4) & 0x0F0F0F0Fu;
        lo.z = q.z & 0x0F0F0F0Fu; hi.z = (q.z >> 4) & 0x0F0F0F0Fu;
        lo.w = q.w & 0x0F0F0F0Fu; hi.w = (q.w >> 4) & 0x0F0F0F0Fu;
        if constexpr (TYPE == HF2Q_TYPE_Q5_K) {
            const uint4 g = *reinterpret_cast<const uint4*>(blk + 16 + 16 * h);
            const int s1 = 2 * c, s2 = 2 * c + 1;
            lo.x |= ((g.x >> s1) & 0x01010101u) << 4; hi.x |= ((g.x >> s2) & 0x01010101u) << 4;
            lo.y |= ((g.y >> s1) & 0x01010101u) << 4; hi.y |= ((g.y >> s2) & 0x01010101u) << 4;
            lo.z |= ((g.z >> s1) & 0x01010101u) << 4; hi.z |= ((g.z >> s2) & 0x01010101u) << 4;
            lo.w |= ((g.w >> s1) & 0x01010101u) << 4; hi.w |= ((g.w >> s2) & 0x01010101u) << 4;
        }
        const float d = f16_bits_to_f32(hd.x & 0xffffu);
        const float dmin = f16_bits_to_f32(hd.x >> 16);
        uint32_t sc1, m1, sc2, m2;
        scale_min_k4(2 * c, hd.y, hd.z, hd.w, sc1, m1);
        scale_min_k4(2 * c + 1, hd.y, hd.z, hd.w, sc2, m2);
        const float d1 = d * static_cast<float>(sc1), d2 = d * static_cast<float>(sc2);
        const float mm1 = dmin * static_cast<float>(m1), mm2 = dmin * static_cast<float>(m2);
        const uint32_t e0 = kbase + b * 256 + 64 * c + 16 * h;
#pragma unroll
        for (int t = 0; t < M; ++t) {
            float sl = dot4(lo.x, xa.ld4(t, e0)) + dot4(lo.y, xa.ld4(t, e0 + 4)) +
                       dot4(lo.z, xa.ld4(t, e0 + 8)) + dot4(lo.w, xa.ld4(t, e0 + 12));
            float sh = dot4(hi.x, xa.ld4(t, e0 + 32)) + dot4(hi.y, xa.ld4(t, e0 + 36)) +
                       dot4(hi.z, xa.ld4(t, e0 + 40)) + dot4(hi.w, xa.ld4(t, e0 + 44));
            const float* xs16 = xsum + static_cast<size_t>(t) * (xa.k >> 4) + (e0 >> 4);
            acc[t] += d1 * sl + d2 * sh - (mm1 * xs16[0] + mm2 * xs16[2]);
        }
    }
}

template <int M, bool XSMEM>
__device__ __forceinline__ void consume_q6k(const uint8_t* sb, int nblk, uint32_t kbase,
                                            const XAcc<XSMEM>& xa, float (&acc)[M], int lane) {
    const int nunits = nblk * 16;               // (block, half n of 128, run i of 4 lanes l)
    for (int u = lane; u < nunits; u += 32) {
        const int b = u >> 4, n = (u >> 3) & 1, i = u & 7;
        const uint8_t* blk = sb + b * 210;      // 2-byte aligned
        const uint32_t qa = ld_u32_a2(blk + 64 * n + 4 * i);
        const uint32_t qb = ld_u32_a2(blk + 64 * n + 32 + 4 * i);
        const uint32_t qh = ld_u32_a2(blk + 128 + 32 * n + 4 * i);
        const uint8_t* scp = blk + 192 + 8 * n + (i >> 2);
        const float d = f16_bits_to_f32(ld_u16(blk + 208));
        const float s0 = d * static_cast<float>(static_cast<int8_t>(scp[0]));
        const float s1 = d * static_cast<float>(static_cast<int8_t>(scp[2]));
        const float s2 = d * static_cast<float>(static_cast<int8_t>(scp[4]));
        const float s3 = d * static_cast<float>(static_cast<int8_t>(scp[6]));
        const uint32_t q0 = (qa & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u);
        const uint32_t q1 = (qb & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u);
        const uint32_t q2 = ((qa >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u);
        const uint32_t q3 = ((qb >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u);
        const uint32_t e0 = kbase + b * 256 + 128 * n + 4 * i;
#pragma unroll
        for (int t = 0; t < M; ++t) {
            acc[t] += s0 * dot4b<32>(q0, xa.ld4(t, e0)) + s1 * dot4b<32>(q1, xa.ld4(t, e0 + 32)) +
                      s2 * dot4b<32>(q2, xa.ld4(t, e0 + 64)) + s3 * dot4b<32>(q3, xa.ld4(t, e0 + 96));
        }
    }
}

template <int M, bool XSMEM>
__device__ __forceinline__ void consume_q4_0(const uint8_t* sb, int nblk, uint32_t kbase,
                                             const XAcc<XSMEM>& xa, float (&acc)[M], int lane) {
    for (int u = lane; u < nblk; u += 32) {
        const uint8_t* blk = sb + u * 18;
        const float d = f16_bits_to_f32(ld_u16(blk));
        uint32_t q[4];
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) q[wi] = ld_u32_a2(blk + 2 + 4 * wi);
        const uint32_t e0 = kbase + u * 32;
#pragma unroll
        for (int t = 0; t < M; ++t) {
            float s = 0.f;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                s += dot4b<8>(q[wi] & 0x0F0F0F0Fu, xa.ld4(t, e0 + 4 * wi));
                s += dot4b<8>((q[wi] >> 4) & 0x0F0F0F0Fu, xa.ld4(t, e0 + 16 + 4 * wi));
            }
            acc[t] += d * s;
        }
    }
}

template <int M, bool XSMEM>
__device__ __forceinline__ void consume_q8_0(const uint8_t* sb, int nblk, uint32_t kbase,
                                             const XAcc<XSMEM>& xa, float (&acc)[M], int lane) {
    for (int u = lane; u < nblk; u += 32) {
        const uint8_t* blk = sb + u * 34;
        const float d = f16_bits_to_f32(ld_u16(blk));
        uint32_t q[8];
#pragma unroll
        for (int wi = 0; wi < 8; ++wi) q[wi] = ld_u32_a2(blk + 2 + 4 * wi) ^ 0x80808080u;
        const uint32_t e0 = kbase + u * 32;
#pragma unroll
        for (int t = 0; t < M; ++t) {
            float s = 0.f;
#pragma unroll
            for (int wi = 0; wi < 8; ++wi) s += dot4b<128>(q[wi], xa.ld4(t, e0 + 4 * wi));
            acc[t] += d * s;
        }
    }
}

// Q4_1 / Q5_0 / Q5_1 / IQ4_NL (the quantizer's fall-back formats for rows that are not a multiple
// of 256 long): one 32-element block per lane and turn, every element decoded by the shared
// dequant_elem, so this path and the stand-alone dequantiser cannot drift apart.  These tensors are
// rare and small; the path is correct and streams, it is not tuned.
template <uint32_t TYPE, int M, bool XSMEM>
__device__ __forceinline__ void consume_block32(const uint8_t* sb, int nblk, uint32_t kbase,
                                                const XAcc<XSMEM>& xa, float (&acc)[M], int lane) {
    constexpr BlockGeom G = block_geom(TYPE);
    for (int u = lane; u < nblk; u += 32) {
        const uint8_t* blk = sb + u * G.bytes;
        const uint32_t e0 = kbase + u * 32;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float w0 = dequant_elem<TYPE>(blk, 4 * j), w1 = dequant_elem<TYPE>(blk, 4 * j + 1);
            const float w2 = dequant_elem<TYPE>(blk, 4 * j + 2), w3 = dequant_elem<TYPE>(blk, 4 * j + 3);
#pragma unroll
            for (int t = 0; t < M; ++t) {
                const float4 x = xa.ld4(t, e0 + 4 * j);
                acc[t] += (w0 * x.x + w1 * x.y) + (w2 * x.z + w3 * x.w);
            }
        }
    }
}

// ---- the streaming kernel ---------------------------------------------------------------------
template <uint32_t TYPE, int M, bool XSMEM>
__global__ void __launch_bounds__(THREADS) gemv_stream_kernel(const KParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr BlockGeom G = block_geom(TYPE);
    constexpr bool NEED_XSUM = TYPE == HF2Q_TYPE_Q4_K || TYPE == HF2Q_TYPE_Q5_K;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + STAGES;
    uint8_t* stage_base = smem + 128;
    const uint32_t stage_bytes = ROWS * p.slice_bytes;
    float* xs = reinterpret_cast<float*>(stage_base + STAGES * stage_bytes);
    float* xsum = xs + (XSMEM ? static_cast<size_t>(M) * p.k : 0);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t slot = blockIdx.y;

    // routed call: this slot's expert matrix and activation row
    const uint8_t* wbase = p.w;
    uint32_t xrow = 0;
    bool slot_ok = true;
    if (p.ids) {
        const uint32_t e = p.ids[slot];
        slot_ok = e < p.n_experts;
        if (!slot_ok && threadIdx.x == 0) atomicOr(p.status, STATUS_BAD_EXPERT_ID);
        wbase += static_cast<uint64_t>(slot_ok ? e : 0) * p.expert_stride;
        xrow = slot / p.top_k;
    }
    const size_t xoff = static_cast<size_t>(xrow) * p.k;
    const void* xg = p.x_bf16 ? static_cast<const void*>(static_cast<const __nv_bfloat16*>(p.x) + xoff)
                              : static_cast<const void*>(static_cast<const float*>(p.x) + xoff);
    float* yout = p.y + static_cast<size_t>(slot) * p.n;     // dense: slot == 0

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], ROWS); }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == ROWS) {
        // ---------------- producer warp: lane r copies row r of each stage ----------------
        if (slot_ok) {
            uint32_t it = 0;
            bool alive = true;
            for (uint32_t rg = blockIdx.x; rg < p.ngroups && alive; rg += gridDim.x) {
                const uint32_t row0 = rg * ROWS;
                const uint32_t nrows = min(static_cast<uint32_t>(ROWS), p.n - row0);
                for (uint32_t s = 0; s < p.nslices; ++s, ++it) {
                    const uint32_t st = it % STAGES;
                    if (it >= STAGES) {
                        alive = mbar_wait_bounded(&empty[st], ((it / STAGES) - 1) & 1, p.status);
                        alive = __all_sync(0xffffffffu, alive);
                        if (!alive) break;
                    }
                    const uint32_t off = s * p.slice_bytes;
                    const uint32_t bytes = min(p.slice_bytes, p.row_bytes - off);
                    if (lane == 0) mbar_arrive_expect_tx(&full[st], nrows * bytes);
                    __syncwarp();
                    if (static_cast<uint32_t>(lane) < nrows)
                        bulk_g2s(stage_base + st * stage_bytes + lane * p.slice_bytes,
                                 wbase + static_cast<uint64_t>(row0 + lane) * p.row_bytes + off, bytes,
                                 &full[st]);
                }
            }
        }
        return;
    }

    // ---------------- consumers: stage the activations while the first copies fly ----------
    const int ctid = threadIdx.x;                 // 0 .. ROWS*32-1
    constexpr int CT = ROWS * 32;
    if constexpr (XSMEM) {
        for (uint32_t i = ctid; i < static_cast<uint32_t>(M) * p.k; i += CT) {
            const uint32_t t = i / p.k;
            float v = 0.f;
            if (t < p.m)
                v = p.x_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(xg)[i])
                             : static_cast<const float*>(xg)[i];
            xs[i] = v;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CT));
    }
    XAcc<XSMEM> xa{xs, xg, p.k, p.x_bf16, p.m};
    if constexpr (NEED_XSUM) {
        const uint32_t ng = p.k >> 4;
        for (uint32_t i = ctid; i < static_cast<uint32_t>(M) * ng; i += CT) {
            const uint32_t t = i / ng, g = i % ng;
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 v = xa.ld4(t, 16 * g + 4 * j);
                s += (v.x + v.y) + (v.z + v.w);
            }
            xsum[i] = (t < p.m) ? s : 0.f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CT));
    }
    if (!slot_ok) {
        for (uint32_t r = ctid; r < p.n; r += CT) yout[r] = 0.f;
        return;
    }

    uint32_t it = 0;
    for (uint32_t rg = blockIdx.x; rg < p.ngroups; rg += gridDim.x) {
        const uint32_t row = rg * ROWS + warp;
        const bool valid = row < p.n;
        float acc[M];
#pragma unroll
        for (int t = 0; t < M; ++t) acc[t] = 0.f;
        for (uint32_t s = 0; s < p.nslices; ++s, ++it) {
            const uint32_t st = it % STAGES;
            if (!mbar_wait_bounded(&full[st], (it / STAGES) & 1, p.status)) return;
            if (valid) {
                const uint8_t* sb = stage_base + st * stage_bytes + warp * p.slice_bytes;
                const uint32_t kbase = s * SLICE_ELEMS;
                const int nblk = static_cast<int>(min(static_cast<uint32_t>(SLICE_ELEMS), p.k - kbase) / G.elems);
                if constexpr (TYPE == HF2Q_TYPE_Q4_K || TYPE == HF2Q_TYPE_Q5_K)
                    consume_k45<TYPE, M, XSMEM>(sb, nblk, kbase, xa, xsum, acc, lane);
                else if constexpr (TYPE == HF2Q_TYPE_Q6_K)
                    consume_q6k<M, XSMEM>(sb, nblk, kbase, xa, acc, lane);
                else if constexpr (TYPE == HF2Q_TYPE_Q4_0)
                    consume_q4_0<M, XSMEM>(sb, nblk, kbase, xa, acc, lane);
                else if constexpr (TYPE == HF2Q_TYPE_Q8_0)
                    consume_q8_0<M, XSMEM>(sb, nblk, kbase, xa, acc, lane);
                else
                    consume_block32<TYPE, M, XSMEM>(sb, nblk, kbase, xa, acc, lane);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        }
#pragma unroll
        for (int t = 0; t < M; ++t) {
            float v = acc[t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && valid && static_cast<uint32_t>(t) < p.m)
                yout[static_cast<size_t>(t) * p.n + row] = v;
        }
    }
}

// ---- fallback: any 2-byte aligned layout, one warp per output row -------------------------------
template <uint32_t TYPE>
__global__ void __launch_bounds__(256) gemv_simple_kernel(const KParams p) {
    constexpr BlockGeom G = block_geom(TYPE);
    const int lane = threadIdx.x & 31;
    const uint32_t slot = blockIdx.y;
    const uint8_t* wbase = p.w;
    uint32_t xrow = 0;
    bool slot_ok = true;
    if (p.ids) {
        const uint32_t e = p.ids[slot];
        slot_ok = e < p.n_experts;
        if (!slot_ok && threadIdx.x == 0) atomicOr(p.status, STATUS_BAD_EXPERT_ID);
        wbase += static_cast<uint64_t>(slot_ok ? e : 0) * p.expert_stride;
        xrow = slot / p.top_k;
    }
    float* yout = p.y + static_cast<size_t>(slot) * p.n;
    const uint32_t warps = gridDim.x * (blockDim.x >> 5);
    for (uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < p.n; row += warps) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (slot_ok) {
            const uint8_t* wr = wbase + static_cast<uint64_t>(row) * p.row_bytes;
            for (uint32_t e = lane; e < p.k; e += 32) {
                const float wv = dequant_elem<TYPE>(wr + (e / G.elems) * G.bytes, static_cast<int>(e % G.elems));
                for (uint32_t t = 0; t < p.m; ++t) {
                    const size_t xi = (static_cast<size_t>(xrow) + t) * p.k + e;
                    const float xv = p.x_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.x)[xi])
                                              : static_cast<const float*>(p.x)[xi];
                    acc[t] += wv * xv;
                }
            }
        }
        for (uint32_t t = 0; t < p.m; ++t) {
            float v = acc[t];
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) yout[static_cast<size_t>(t) * p.n + row] = v;
        }
    }
}

template <uint32_t TYPE, int M, bool XSMEM>
cudaError_t launch_stream(const KParams& p, uint32_t slots, size_t smem, const DeviceInfo& dev,
                          cudaStream_t st) {
    auto kern = gemv_stream_kernel<TYPE, M, XSMEM>;
    // The opt-in shared-memory limit is raised once per kernel and device; the occupancy answer is
    // cached per device for the last shared-memory size, so the steady-state launch path makes no
    // other runtime call.
    static PerDeviceFlag attr;
    if (const cudaError_t e = ensure_max_dynamic_smem(kern, dev.max_smem_optin, attr); e != cudaSuccess) return e;
    static std::mutex mu;
    static size_t cached_smem[MAX_DEVICES];
    static int cached_per_sm[MAX_DEVICES];
    static bool cached[MAX_DEVICES] = {};
    int per_sm, cur = 0;
    if (const cudaError_t e = cudaGetDevice(&cur); e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!cached[cur] || cached_smem[cur] != smem) {
            int q = 1;
            cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kern, THREADS, smem);
            if (e != cudaSuccess) return e;
            cached_per_sm[cur] = q < 1 ? 1 : q;
            cached_smem[cur] = smem;
            cached[cur] = true;
        }
        per_sm = cached_per_sm[cur];
    }
    uint32_t want = static_cast<uint32_t>(dev.sm_count) * per_sm;
    uint32_t gx = (want + slots - 1) / slots;
    if (gx > p.ngroups) gx = p.ngroups;
    if (gx < 1) gx = 1;
    kern<<<dim3(gx, slots), THREADS, smem, st>>>(p);
    return cudaGetLastError();
}

template <uint32_t TYPE, int M>
cudaError_t launch_stream_m(const KParams& p, uint32_t slots, const DeviceInfo& dev, cudaStream_t st) {
    constexpr bool NEED_XSUM = TYPE == HF2Q_TYPE_Q4_K || TYPE == HF2Q_TYPE_Q5_K;
    const size_t ring = 128 + static_cast<size_t>(STAGES) * ROWS * p.slice_bytes;
    const size_t xsum = NEED_XSUM ? static_cast<size_t>(M) * (p.k / 16) * 4 : 0;
    const size_t xs = static_cast<size_t>(M) * p.k * 4;
    const size_t limit = static_cast<size_t>(dev.max_smem_optin) - 1024;
    if (ring + xs + xsum <= limit) return launch_stream<TYPE, M, true>(p, slots, ring + xs + xsum, dev, st);
    if (ring + xsum <= limit) return launch_stream<TYPE, M, false>(p, slots, ring + xsum, dev, st);
    return cudaErrorInvalidConfiguration;
}

template <uint32_t TYPE>
cudaError_t launch_type(const KParams& p, uint32_t slots, bool can_stream, const DeviceInfo& dev,
                        cudaStream_t st) {
    if (can_stream) {
        cudaError_t e;
        if (p.m == 1) e = launch_stream_m<TYPE, 1>(p, slots, dev, st);
        else if (p.m == 2) e = launch_stream_m<TYPE, 2>(p, slots, dev, st);
        else if (p.m <= 4) e = launch_stream_m<TYPE, 4>(p, slots, dev, st);
        else e = launch_stream_m<TYPE, 8>(p, slots, dev, st);
        if (e != cudaErrorInvalidConfiguration) return e;
        (void)cudaGetLastError();
    }
    const uint32_t want = static_cast<uint32_t>(dev.sm_count) * 8;
    uint32_t gx = (p.n + 7) / 8;
    if (gx > want) gx = want;
    gemv_simple_kernel<TYPE><<<dim3(gx, slots), 256, 0, st>>>(p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemv(const GemvArgs& a, const DeviceInfo& dev, cudaStream_t st, int* launches) {
    const BlockGeom g = block_geom(a.type);
    KParams p{};
    p.w = static_cast<const uint8_t*>(a.w);
    p.x = a.x;
    p.y = a.y;
    p.ids = a.ids;
    p.expert_stride = a.expert_stride;
    p.x_bf16 = a.x_dtype == HF2Q_DT_BF16;
    p.m = a.m;
    p.n = a.n;
    p.k = a.k;
    p.top_k = a.top_k ? a.top_k : 1;
    p.n_experts = a.n_experts;
    p.row_bytes = a.k / g.elems * g.bytes;
    p.slice_bytes = SLICE_ELEMS / g.elems * g.bytes;
    if (p.slice_bytes > p.row_bytes) p.slice_bytes = p.row_bytes;
    p.nslices = (a.k + SLICE_ELEMS - 1) / SLICE_ELEMS;
    p.ngroups = (a.n + ROWS - 1) / ROWS;
    p.status = a.status;
    // bulk copies need 16-byte aligned sources and sizes; activations are read as 16-byte vectors
    const bool can_stream = (reinterpret_cast<uintptr_t>(a.w) % 16 == 0) && (p.row_bytes % 16 == 0) &&
                            (a.expert_stride % 16 == 0) && (a.k % 16 == 0) &&
                            (reinterpret_cast<uintptr_t>(a.x) % 16 == 0);
    if (launches) *launches = 1;
    switch (a.type) {
        case HF2Q_TYPE_Q4_0: return launch_type<HF2Q_TYPE_Q4_0>(p, a.slots, can_stream, dev, st);
        case HF2Q_TYPE_Q8_0: return launch_type<HF2Q_TYPE_Q8_0>(p, a.slots, can_stream, dev, st);
        case HF2Q_TYPE_Q4_K: return launch_type<HF2Q_TYPE_Q4_K>(p, a.slots, can_stream, dev, st);
        case HF2Q_TYPE_Q5_K: return launch_type<HF2Q_TYPE_Q5_K>(p, a.slots, can_stream, dev, st);
        case HF2Q_TYPE_Q6_K: return launch_type<HF2Q_TYPE_Q6_K>(p, a.slots, can_stream, dev, st);
        case HF2Q_TYPE_Q4_1: return launch_type<HF2Q_TYPE_Q4_1>(p, a.slots, can_stream, dev, st);
        case HF2Q_TYPE_Q5_0: return launch_type<HF2Q_TYPE_Q5_0>(p, a.slots, can_stream, dev, st);
        case HF2Q_TYPE_Q5_1: return launch_type<HF2Q_TYPE_Q5_1>(p, a.slots, can_stream, dev, st);
        case HF2Q_TYPE_IQ4_NL: return launch_type<HF2Q_TYPE_IQ4_NL>(p, a.slots, can_stream, dev, st);
        case HF2Q_TYPE_MLX_AFFINE4_GS32: return launch_type<HF2Q_TYPE_MLX_AFFINE4_GS32>(p, a.slots, can_stream, dev, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace hf2q
