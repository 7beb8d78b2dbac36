// The kernels that sit between the quantized products in a decoder forward pass: embedding row
// look-up, RMSNorm (with the residual add), rotary position embedding fused with the append to an
// 8-bit KV cache, attention over that cache (decode: split over the context; prefill: tiled), and
// the greedy arg-max.  Together with the products they make the forward of
// Qwen35Model::forward_gpu_greedy (src/inference/models/qwen35/forward_gpu.rs:4140) on Llama-shaped
// layers; the arithmetic follows the reference's scalar specs: rms_norm_rows
// (src/inference/models/qwen35/forward_cpu.rs:36-48), residual_add (:51-56), the causal softmax
// attention of gated_full_attention_cpu_ref (full_attn.rs:219-360, without its output gate and with
// the plain rotary embedding of the Llama architecture), embed_tokens / apply_output_head
// (io_heads.rs).
//
// KV cache.  The reference keeps K and V as one byte per element plus one f32 norm per (head,
// position) (TqFullAttnKvBuffers, kv_cache.rs:1982-2012); its byte is an index into a 256-entry
// Lloyd-Max codebook that lives in the external mlx-native crate.  That codebook is not available,
// so the byte here is a signed 8-bit integer and the f32 per (head, position) is the scale
// amax / 127: same layout, same bytes per position, a linear code instead of the codebook.
//   k_codes, v_codes : int8  [n_kv_heads][max_seq][head_dim]
//   k_scale, v_scale : float [n_kv_heads][max_seq]
#include <math_constants.h>

#include "common.cuh"
#include "kernels.h"

namespace hf2q {
namespace {

// ------------------------------------------------------------------ embedding rows
template <uint32_t TYPE>
__global__ void __launch_bounds__(256) get_rows_kernel(const uint8_t* __restrict__ w, uint64_t row_bytes, uint32_t n_rows,
                                                       uint32_t k, const uint32_t* __restrict__ ids, float* __restrict__ out,
                                                       uint32_t* status) {
    constexpr BlockGeom G = block_geom(TYPE);
    const uint32_t t = blockIdx.x;
    uint32_t id = ids[t];
    if (id >= n_rows) {                                   // out of range: zero row, flagged
        if (threadIdx.x == 0) atomicOr(status, STATUS_BAD_EXPERT_ID);
        for (uint32_t e = threadIdx.x; e < k; e += 256) out[static_cast<size_t>(t) * k + e] = 0.f;
        return;
    }
    const uint8_t* row = w + static_cast<uint64_t>(id) * row_bytes;
    for (uint32_t e = threadIdx.x; e < k; e += 256)
        out[static_cast<size_t>(t) * k + e] = dequant_elem<TYPE>(row + (e / G.elems) * G.bytes, static_cast<int>(e % G.elems));
}

// ------------------------------------------------------------------ RMSNorm (+ residual add)
// x[t,:] += delta[t,:] (if delta), then out[t,:] = x[t,:] * rsqrt(mean(x^2) + eps) * weight[:]
// (forward_cpu.rs:36-48: sum of squares in f32, sequential per row there, tree-reduced here).
template <typename OUT>
__global__ void __launch_bounds__(1024) rms_norm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                        const float* __restrict__ weight, float eps, OUT* __restrict__ out,
                                                        uint32_t h) {
    __shared__ float part[32];
    float* row = x + static_cast<size_t>(blockIdx.x) * h;
    const float* drow = delta ? delta + static_cast<size_t>(blockIdx.x) * h : nullptr;
    OUT* orow = out + static_cast<size_t>(blockIdx.x) * h;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < h; i += blockDim.x) {
        float v = row[i];
        if (drow) { v += drow[i]; row[i] = v; }
        ss += v * v;
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) part[0] = 1.0f / sqrtf(v / static_cast<float>(h) + eps);
    }
    __syncthreads();
    const float inv = part[0];
    for (uint32_t i = threadIdx.x; i < h; i += blockDim.x) {
        const float v = row[i] * inv * weight[i];
        if constexpr (sizeof(OUT) == 4) orow[i] = v;
        else orow[i] = __float2bfloat16_rn(v);
    }
}

// ------------------------------------------------------------------ rotary embedding + KV append
// qkv: [m][(n_q + 2 n_kv) * hd] f32 (fused QKV product).  Token t sits at position *pos + t.
// One warp per (token, head).  q heads are rotated in place and scaled by `q_scale` (1/sqrt(hd), so
// the attention kernels need no multiply); k heads are rotated, then k and v heads are quantized
// to int8 with one scale per (head, position) and stored in the cache.  Pairs are (2i, 2i+1) with
// angle pos * theta^(-2i/hd) -- the rotary form of the Llama architecture.
__global__ void __launch_bounds__(256) rope_kv_append_kernel(float* __restrict__ qkv, uint32_t m, uint32_t n_q, uint32_t n_kv,
                                                             uint32_t hd, const uint32_t* __restrict__ pos_dev, float theta,
                                                             float q_scale, int8_t* __restrict__ k_codes, float* __restrict__ k_scale,
                                                             int8_t* __restrict__ v_codes, float* __restrict__ v_scale,
                                                             uint32_t max_seq, uint32_t* status) {
    const uint32_t heads = n_q + 2 * n_kv;
    const uint32_t wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (wid >= m * heads) return;
    const uint32_t t = wid / heads, hidx = wid % heads;
    const uint32_t pos = *pos_dev + t;
    float* v = qkv + static_cast<size_t>(t) * heads * hd + static_cast<size_t>(hidx) * hd;
    const bool is_q = hidx < n_q, is_k = !is_q && hidx < n_q + n_kv;
    // hd <= 256: each lane owns up to 4 consecutive pairs
    float vals[8];
    const uint32_t per = hd / 32;                        // elements per lane (hd = 64, 128 or 256)
    float amax = 0.f;
    for (uint32_t j = 0; j < per; j += 2) {
        const uint32_t e = lane * per + j;
        float a = v[e], b = v[e + 1];
        if (is_q || is_k) {
            const float freq = powf(theta, -static_cast<float>(e) / static_cast<float>(hd));
            float sn, cs;
            sincosf(static_cast<float>(pos) * freq, &sn, &cs);
            const float ra = a * cs - b * sn, rb = a * sn + b * cs;
            a = ra; b = rb;
        }
        if (is_q) { a *= q_scale; b *= q_scale; v[e] = a; v[e + 1] = b; }
        vals[j] = a; vals[j + 1] = b;
        amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
    }
    if (is_q) return;
    if (pos >= max_seq) { if (lane == 0) atomicOr(status, STATUS_BAD_EXPERT_ID); return; }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax / 127.0f, inv = amax > 0.f ? 127.0f / amax : 0.f;
    const uint32_t kvh = is_k ? hidx - n_q : hidx - n_q - n_kv;
    int8_t* codes = (is_k ? k_codes : v_codes) + (static_cast<size_t>(kvh) * max_seq + pos) * hd;
    for (uint32_t j = 0; j < per; ++j) codes[lane * per + j] = static_cast<int8_t>(__float2int_rn(vals[j] * inv));
    if (lane == 0) (is_k ? k_scale : v_scale)[static_cast<size_t>(kvh) * max_seq + pos] = scale;
}

// ------------------------------------------------------------------ decode attention, split over the context
// grid (n_kv_heads, n_splits); one CTA handles the G = n_q / n_kv query heads of its KV head over
// positions [lo, hi) of the n_ctx = *pos + 1 cached positions.  hd == 128, G <= 8.
// Scores: a warp takes 32 positions at a time, lane = position: the lane walks its K row (128 int8)
// against the G query vectors in shared memory.  Values: lane = 4 dims; the warp walks the 32
// positions with their probabilities from shared memory.  Each CTA leaves (max, sum, acc[G][128]) of
// its range in scratch; attn_combine_kernel merges the splits.
constexpr int ATT_WARPS = 8;
constexpr int ATT_HD = 128;
constexpr int ATT_MAXG = 8;
constexpr int ATT_PART = 4 + ATT_HD;     // floats of one partial result: max, sum, two pad words, 128 accumulators (16-byte aligned)

// D (16x8, f32) += A (16x16, f16, row-major) * B (16x8, f16, column-major); c[0..1] = row lane/4, columns 2 (lane%4) + {0,1}
__device__ __forceinline__ void mma_m16n8k16_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float4 s8x4_to_float4(uint32_t w) {
    return make_float4(byte_to_float<128>(w ^ 0x80808080u, 0), byte_to_float<128>(w ^ 0x80808080u, 1),
                       byte_to_float<128>(w ^ 0x80808080u, 2), byte_to_float<128>(w ^ 0x80808080u, 3));
}

template <int G>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_decode_kernel(const float* __restrict__ q, uint32_t q_stride_heads,
                                                                     const int8_t* __restrict__ k_codes, const float* __restrict__ k_scale,
                                                                     const int8_t* __restrict__ v_codes, const float* __restrict__ v_scale,
                                                                     uint32_t max_seq, const uint32_t* __restrict__ pos_dev,
                                                                     float* __restrict__ part /* [n_kv][splits][G][2 + 128] */) {
    __shared__ __align__(16) float qs[G][ATT_HD];
    __shared__ float ps[ATT_WARPS][G][32];
    __shared__ float red_m[ATT_WARPS][G], red_l[ATT_WARPS][G];
    __shared__ __align__(16) float red_acc[ATT_WARPS][G][ATT_HD];
    (void)q_stride_heads;
    const uint32_t kvh = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y;
    const uint32_t n_ctx = *pos_dev + 1;
    const uint32_t chunk = (n_ctx + nsplit - 1) / nsplit;
    const uint32_t lo = min(split * chunk, n_ctx), hi = min(lo + chunk, n_ctx);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t i = threadIdx.x; i < G * ATT_HD; i += ATT_WARPS * 32)
        qs[i / ATT_HD][i % ATT_HD] = q[(static_cast<size_t>(kvh) * G + i / ATT_HD) * ATT_HD + i % ATT_HD];
    __syncthreads();
    const int8_t* kc = k_codes + static_cast<size_t>(kvh) * max_seq * ATT_HD;
    const int8_t* vc = v_codes + static_cast<size_t>(kvh) * max_seq * ATT_HD;
    const float* ksc = k_scale + static_cast<size_t>(kvh) * max_seq;
    const float* vsc = v_scale + static_cast<size_t>(kvh) * max_seq;

    float mx[G], l[G], acc[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) { mx[g] = -CUDART_INF_F; l[g] = 0.f; acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f; }

    for (uint32_t p0 = lo + warp * 32; p0 < hi; p0 += ATT_WARPS * 32) {
        const uint32_t p = p0 + lane;
        const bool live = p < hi;
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = 0.f;
        if (live) {
            const uint4* kr = reinterpret_cast<const uint4*>(kc + static_cast<size_t>(p) * ATT_HD);
#pragma unroll
            for (int c = 0; c < ATT_HD / 16; ++c) {
                const uint4 kv = __ldcs(kr + c);
                const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 kf = s8x4_to_float4(kw[j]);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float4 qv = *reinterpret_cast<const float4*>(&qs[g][16 * c + 4 * j]);
                        s[g] += kf.x * qv.x + kf.y * qv.y + kf.z * qv.z + kf.w * qv.w;
                    }
                }
            }
            const float sc = ksc[p];
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] *= sc;
        }
        // online softmax over this batch of 32 positions; the V scale is folded into the probability
        const float vs = live ? vsc[p] : 0.f;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float bm = live ? s[g] : -CUDART_INF_F;
            for (int o = 16; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
            const float nm = fmaxf(mx[g], bm);
            const float corr = __expf(mx[g] - nm);             // exp(-inf) = 0 on the first batch
            const float pr = live ? __expf(s[g] - nm) : 0.f;
            float bs = pr;
            for (int o = 16; o > 0; o >>= 1) bs += __shfl_xor_sync(0xffffffffu, bs, o);
            l[g] = l[g] * corr + bs;
            mx[g] = nm;
            acc[g][0] *= corr; acc[g][1] *= corr; acc[g][2] *= corr; acc[g][3] *= corr;
            ps[warp][g][lane] = pr * vs;
        }
        __syncwarp();
        const uint32_t cnt = min(32u, hi - p0);
        for (uint32_t i = 0; i < cnt; ++i) {
            const uint32_t vw = __ldcs(reinterpret_cast<const uint32_t*>(vc + static_cast<size_t>(p0 + i) * ATT_HD) + lane);
            const float4 vf = s8x4_to_float4(vw);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float pw = ps[warp][g][i];
                acc[g][0] += pw * vf.x; acc[g][1] += pw * vf.y; acc[g][2] += pw * vf.z; acc[g][3] += pw * vf.w;
            }
        }
        __syncwarp();
    }
    // merge the warps of this CTA
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) { red_m[warp][g] = mx[g]; red_l[warp][g] = l[g]; }
        *reinterpret_cast<float4*>(&red_acc[warp][g][4 * lane]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < G * ATT_HD; i += ATT_WARPS * 32) {
        const int g = i / ATT_HD, d = i % ATT_HD;
        float m_all = -CUDART_INF_F;
        for (int w = 0; w < ATT_WARPS; ++w) m_all = fmaxf(m_all, red_m[w][g]);
        float l_all = 0.f, a = 0.f;
        for (int w = 0; w < ATT_WARPS; ++w) {
            const float c = red_m[w][g] == -CUDART_INF_F ? 0.f : __expf(red_m[w][g] - m_all);
            l_all += red_l[w][g] * c;
            a += red_acc[w][g][d] * c;
        }
        float* dst = part + ((static_cast<size_t>(kvh) * nsplit + split) * G + g) * ATT_PART;
        if (d == 0) { dst[0] = m_all; dst[1] = l_all; }
        dst[4 + d] = a;
    }
}

// ---- the same, as ONE launch per layer: rotary embedding of the query, append of the new position's K
// and V, the split attention, and the merge of the splits.
//   * every CTA rotates and scales the G query heads of its KV head itself (512 values);
//   * the CTA whose range holds the new position (*pos) rotates and quantizes that position's K and V
//     from the fused QKV row, writes them to the cache and then reads them like any other position;
//   * every CTA leaves its (max, sum, acc) in scratch, bumps a per-KV-head counter, and the CTA that
//     arrives last merges all splits of that head and resets the counter (no atomics on data, fixed
//     merge order: bit-reproducible).
// qkv: one fused QKV row, f32 [(n_q + 2 n_kv) * 128]; the query part is NOT modified.
template <int G, typename OUT>
__global__ void __launch_bounds__(ATT_WARPS * 32, 2) attn_decode_fused_kernel(const float* __restrict__ qkv, uint32_t n_q, uint32_t n_kv,
                                                                           float theta, float q_scale,
                                                                           int8_t* __restrict__ k_codes, float* __restrict__ k_scale,
                                                                           int8_t* __restrict__ v_codes, float* __restrict__ v_scale,
                                                                           uint32_t max_seq, const uint32_t* __restrict__ pos_dev,
                                                                           float* __restrict__ part, uint32_t* __restrict__ counters,
                                                                           OUT* __restrict__ out, uint32_t* status) {
    __shared__ __align__(16) float qs[G][ATT_HD];
    __shared__ float ps[ATT_WARPS][G][32];
    __shared__ float red_m[ATT_WARPS][G], red_l[ATT_WARPS][G];
    __shared__ __align__(16) float red_acc[ATT_WARPS][G][ATT_HD + 4];     // rows padded by 16 bytes: the accumulator fragments of the eight row groups land in different banks
    __shared__ uint32_t is_last;
    const uint32_t kvh = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y;
    // programmatic dependent launch: the next kernel of the stream (the O product) may start its own
    // prologue now; this kernel touches nothing an earlier kernel writes before that kernel has completed
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // everything that does not depend on the position is requested before the position itself is read:
    // the query pairs of this thread and (warps 0 and 1) the new row's K / V values
    constexpr int QPAIRS = (G * ATT_HD / 2 + ATT_WARPS * 32 - 1) / (ATT_WARPS * 32);
    float2 qraw[QPAIRS];
#pragma unroll
    for (int u = 0; u < QPAIRS; ++u) {
        const uint32_t i = threadIdx.x + u * ATT_WARPS * 32;
        qraw[u] = i < G * ATT_HD / 2
                      ? *reinterpret_cast<const float2*>(qkv + (static_cast<size_t>(kvh) * G + i / (ATT_HD / 2)) * ATT_HD + 2 * (i % (ATT_HD / 2)))
                      : make_float2(0.f, 0.f);
    }
    float4 newrow = make_float4(0.f, 0.f, 0.f, 0.f);
    if (warp < 2) newrow = *reinterpret_cast<const float4*>(qkv + (static_cast<size_t>(n_q) + (warp == 0 ? 0u : n_kv) + kvh) * ATT_HD + 4 * lane);
    const uint32_t pos = *pos_dev;
    if (pos >= max_seq) { if (threadIdx.x == 0 && split == 0) atomicOr(status, STATUS_BAD_EXPERT_ID); return; }
    const uint32_t n_ctx = pos + 1;
    const uint32_t chunk = (n_ctx + nsplit - 1) / nsplit;
    const uint32_t lo = min(split * chunk, n_ctx), hi = min(lo + chunk, n_ctx);
    int8_t* kc = k_codes + static_cast<size_t>(kvh) * max_seq * ATT_HD;
    int8_t* vc = v_codes + static_cast<size_t>(kvh) * max_seq * ATT_HD;
    float* ksc = k_scale + static_cast<size_t>(kvh) * max_seq;
    float* vsc = v_scale + static_cast<size_t>(kvh) * max_seq;
    // rotated, scaled query heads: thread -> (head g, pair i)
#pragma unroll
    for (int u = 0; u < QPAIRS; ++u) {
        const uint32_t i = threadIdx.x + u * ATT_WARPS * 32;
        if (i < G * ATT_HD / 2) {
            const uint32_t g = i / (ATT_HD / 2), pr = i % (ATT_HD / 2);
            const float freq = powf(theta, -static_cast<float>(2 * pr) / static_cast<float>(ATT_HD));      // as in rope_kv_append_kernel
            float sn, cs;
            sincosf(static_cast<float>(pos) * freq, &sn, &cs);
            qs[g][2 * pr] = (qraw[u].x * cs - qraw[u].y * sn) * q_scale;
            qs[g][2 * pr + 1] = (qraw[u].x * sn + qraw[u].y * cs) * q_scale;
        }
    }
    if (pos >= lo && pos < hi && warp < 2) {
        // the new position: warp 0 -> K (rotated), warp 1 -> V; lane owns 4 consecutive elements
        const bool is_k = warp == 0;
        float v4[4] = {newrow.x, newrow.y, newrow.z, newrow.w};
        if (is_k) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const float freq = powf(theta, -static_cast<float>(4 * lane + j) / static_cast<float>(ATT_HD));
                float sn, cs;
                sincosf(static_cast<float>(pos) * freq, &sn, &cs);
                const float a = v4[j], b = v4[j + 1];
                v4[j] = a * cs - b * sn;
                v4[j + 1] = a * sn + b * cs;
            }
        }
        float amax = fmaxf(fmaxf(fabsf(v4[0]), fabsf(v4[1])), fmaxf(fabsf(v4[2]), fabsf(v4[3])));
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float inv = amax > 0.f ? 127.0f / amax : 0.f;
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) w |= (static_cast<uint32_t>(__float2int_rn(v4[j] * inv)) & 0xffu) << (8 * j);
        reinterpret_cast<uint32_t*>((is_k ? kc : vc) + static_cast<size_t>(pos) * ATT_HD)[lane] = w;
        if (lane == 0) (is_k ? ksc : vsc)[pos] = amax / 127.0f;
    }
    __syncthreads();            // qs ready; the new position's codes are visible to this CTA

    // ---- scores and weighted values on the tensor cores (mma.sync m16n8k16, f16 operands, f32 accumulators).
    // M = query heads of this KV head (rows gid < G; the rest of the 16 rows are zero), a warp step = 16 positions.
    //   scores:  A = Q (f16), B = K^T with the 8-bit codes as the integers 1024 + (code + 128) in f16 (exact);
    //            the offset 1152 * sum(q) is taken off afterwards.  The contraction order over the 128 dims is
    //            free, so lane (gid, t) takes bytes [32t, 32t + 32) of row gid: two 16-byte loads, no shuffles.
    //   values:  A = P * vscale (f16, straight from the score accumulators: same fragment layout), B = V with the
    //            codes as f16 SUBNORMALS (code + 128) * 2^-24 (exact); pairs of positions are gathered byte-wise
    //            from two rows; the offset 128 * sum(P * vscale) is taken off at the end.
    const uint32_t gid = lane >> 2, t = lane & 3;
    uint32_t qa0[8], qa2[8];
    float qsum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        qa0[j] = qa2[j] = 0u;
        if (gid < static_cast<uint32_t>(G)) {
            const float4 q4 = *reinterpret_cast<const float4*>(&qs[gid][32 * t + 4 * j]);
            const __half2 lo2 = __floats2half2_rn(q4.x, q4.y), hi2 = __floats2half2_rn(q4.z, q4.w);
            qa0[j] = *reinterpret_cast<const uint32_t*>(&lo2);
            qa2[j] = *reinterpret_cast<const uint32_t*>(&hi2);
            qsum += (__low2float(lo2) + __high2float(lo2)) + (__low2float(hi2) + __high2float(hi2));
        }
    }
    qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
    qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
    const float qfix = 1152.0f * qsum;

    float mx = -CUDART_INF_F, l = 0.f, lfix = 0.f;       // of head gid (the four lanes of a row group agree)
    float o0[16], o1[16];                                 // out[gid][32t + j], out[gid][32t + 16 + j]
#pragma unroll
    for (int j = 0; j < 16; ++j) o0[j] = o1[j] = 0.f;
    for (uint32_t p0 = lo + warp * 16; p0 < hi; p0 += ATT_WARPS * 16) {
        // K: rows p0 + gid and p0 + 8 + gid, bytes [32t, 32t + 32); V: rows p0 + 2t, +1, +8, +9, bytes [16 gid, 16 gid + 16).
        // Rows past the end are clamped to the last one; their probabilities are forced to zero.
        const uint32_t last = hi - 1;
        uint4 kq[2][2], vq[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const uint4* kr = reinterpret_cast<const uint4*>(kc + static_cast<size_t>(min(p0 + 8 * nt + gid, last)) * ATT_HD + 32 * t);
            kq[nt][0] = kr[0];
            kq[nt][1] = kr[1];
        }
        const uint32_t pc[4] = {p0 + 2 * t, p0 + 2 * t + 1, p0 + 2 * t + 8, p0 + 2 * t + 9};   // this lane's score / probability columns
        float kscl[4], vscl[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            vq[i] = *reinterpret_cast<const uint4*>(vc + static_cast<size_t>(min(pc[i], last)) * ATT_HD + 16 * gid);
            kscl[i] = ksc[min(pc[i], last)];
            vscl[i] = vsc[min(pc[i], last)];
        }
        float sc[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t kw[8] = {kq[nt][0].x, kq[nt][0].y, kq[nt][0].z, kq[nt][0].w, kq[nt][1].x, kq[nt][1].y, kq[nt][1].z, kq[nt][1].w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t x = kw[j] ^ 0x80808080u;
                const uint32_t b0 = __byte_perm(x, 0x64646464u, 0x4140u), b1 = __byte_perm(x, 0x64646464u, 0x4342u);
                mma_m16n8k16_f16(c, qa0[j], 0u, qa2[j], 0u, b0, b1);
            }
            sc[2 * nt] = pc[2 * nt] < hi ? (c[0] - qfix) * kscl[2 * nt] : -CUDART_INF_F;
            sc[2 * nt + 1] = pc[2 * nt + 1] < hi ? (c[1] - qfix) * kscl[2 * nt + 1] : -CUDART_INF_F;
        }
        float bm = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));          // finite: position p0 < hi is one of the sixteen
        const float nm = fmaxf(mx, bm);
        const float corr = __expf(mx - nm);
        float pr[4], wf[4];
        uint32_t pa[2];
#pragma unroll
        for (int i = 0; i < 4; ++i) pr[i] = __expf(sc[i] - nm);       // exp(-inf) = 0 for the clamped columns
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const __half2 w2 = __floats2half2_rn(pr[2 * h] * vscl[2 * h] * 256.0f, pr[2 * h + 1] * vscl[2 * h + 1] * 256.0f);
            pa[h] = *reinterpret_cast<const uint32_t*>(&w2);
            wf[2 * h] = __low2float(w2);
            wf[2 * h + 1] = __high2float(w2);
        }
        float bs = (pr[0] + pr[1]) + (pr[2] + pr[3]), bw = (wf[0] + wf[1]) + (wf[2] + wf[3]);
        bs += __shfl_xor_sync(0xffffffffu, bs, 1);
        bw += __shfl_xor_sync(0xffffffffu, bw, 1);
        bs += __shfl_xor_sync(0xffffffffu, bs, 2);
        bw += __shfl_xor_sync(0xffffffffu, bw, 2);
        l = l * corr + bs;
        lfix = lfix * corr + bw;
        mx = nm;
#pragma unroll
        for (int j = 0; j < 16; ++j) { o0[j] *= corr; o1[j] *= corr; }
        // V operand: word c of the lane's 16 bytes = dims 16 gid + 4c .. + 3 = column gid of the tiles 4c .. 4c + 3
        const uint32_t va[4] = {vq[0].x ^ 0x80808080u, vq[0].y ^ 0x80808080u, vq[0].z ^ 0x80808080u, vq[0].w ^ 0x80808080u};
        const uint32_t vb[4] = {vq[1].x ^ 0x80808080u, vq[1].y ^ 0x80808080u, vq[1].z ^ 0x80808080u, vq[1].w ^ 0x80808080u};
        const uint32_t vc8[4] = {vq[2].x ^ 0x80808080u, vq[2].y ^ 0x80808080u, vq[2].z ^ 0x80808080u, vq[2].w ^ 0x80808080u};
        const uint32_t vd[4] = {vq[3].x ^ 0x80808080u, vq[3].y ^ 0x80808080u, vq[3].z ^ 0x80808080u, vq[3].w ^ 0x80808080u};
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
            // [A.b0 A.b1 B.b0 B.b1] and [A.b2 A.b3 B.b2 B.b3] of the row pairs (2t, 2t+1) and (2t+8, 2t+9)
            const uint32_t lo01 = __byte_perm(va[c4], vb[c4], 0x5410u), hi01 = __byte_perm(va[c4], vb[c4], 0x7632u);
            const uint32_t lo89 = __byte_perm(vc8[c4], vd[c4], 0x5410u), hi89 = __byte_perm(vc8[c4], vd[c4], 0x7632u);
            const uint32_t b0[4] = {lo01 & 0x00FF00FFu, __byte_perm(lo01, 0u, 0x4341u), hi01 & 0x00FF00FFu, __byte_perm(hi01, 0u, 0x4341u)};
            const uint32_t b1[4] = {lo89 & 0x00FF00FFu, __byte_perm(lo89, 0u, 0x4341u), hi89 & 0x00FF00FFu, __byte_perm(hi89, 0u, 0x4341u)};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float d[4] = {o0[4 * c4 + i], o1[4 * c4 + i], 0.f, 0.f};
                mma_m16n8k16_f16(d, pa[0], 0u, pa[1], 0u, b0[i], b1[i]);
                o0[4 * c4 + i] = d[0];
                o1[4 * c4 + i] = d[1];
            }
        }
    }
    // accumulators hold sum(P vscale 2^8 * (code + 128) 2^-24): back to sum(P vscale code)
    if (gid < static_cast<uint32_t>(G)) {
        const float off = 128.0f * lfix * (1.0f / 256.0f);
        if (t == 0) { red_m[warp][gid] = mx; red_l[warp][gid] = l; }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            red_acc[warp][gid][32 * t + j] = o0[j] * 65536.0f - off;
            red_acc[warp][gid][32 * t + 16 + j] = o1[j] * 65536.0f - off;
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < G * ATT_HD; i += ATT_WARPS * 32) {
        const int g = i / ATT_HD, d = i % ATT_HD;
        float m_all = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) m_all = fmaxf(m_all, red_m[w][g]);
        float l_all = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) {
            const float c = red_m[w][g] == -CUDART_INF_F ? 0.f : __expf(red_m[w][g] - m_all);
            l_all += red_l[w][g] * c;
            a += red_acc[w][g][d] * c;
        }
        float* dst = part + ((static_cast<size_t>(kvh) * nsplit + split) * G + g) * ATT_PART;
        if (d == 0) { dst[0] = m_all; dst[1] = l_all; }
        dst[4 + d] = a;
    }
    // the CTA that completes this KV head merges its splits
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t old = atomicAdd(&counters[kvh], 1u);
        is_last = old == nsplit - 1 ? 1u : 0u;
        if (is_last) counters[kvh] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // Merge of the splits: (1) every split's (max, sum) into shared memory; (2) warp g turns those of head g into
    // the weights exp(max_s - max) and the normaliser; (3) warp w adds the partial results of splits w, w + 8, ...
    // (16-byte loads, all in flight), the eight sums are added in warp order: a fixed order, bit-reproducible.
    float* sm_m = &ps[0][0][0];                          // [nsplit][G] (nsplit <= 64: fits the probability scratch)
    float* sm_c = &qs[0][0];                             // [nsplit][G] weights (G * 128 floats), normaliser per head in red_m[0][g]
    const float* pbase = part + static_cast<size_t>(kvh) * nsplit * G * ATT_PART;
    for (uint32_t i = threadIdx.x; i < nsplit * G; i += ATT_WARPS * 32) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(pbase + static_cast<size_t>(i) * ATT_PART));
        sm_m[i] = ml.x;
        sm_c[i] = ml.y;                                  // the sums for now
    }
    __syncthreads();
    if (warp < G) {
        const uint32_t g = warp;
        const uint32_t s0 = lane, s1 = lane + 32;
        const float m0 = s0 < nsplit ? sm_m[s0 * G + g] : -CUDART_INF_F, m1 = s1 < nsplit ? sm_m[s1 * G + g] : -CUDART_INF_F;
        float m_all = fmaxf(m0, m1);
        for (int o = 16; o > 0; o >>= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
        const float c0 = m0 == -CUDART_INF_F ? 0.f : __expf(m0 - m_all), c1 = m1 == -CUDART_INF_F ? 0.f : __expf(m1 - m_all);
        float l_all = (s0 < nsplit ? sm_c[s0 * G + g] * c0 : 0.f) + (s1 < nsplit ? sm_c[s1 * G + g] * c1 : 0.f);
        for (int o = 16; o > 0; o >>= 1) l_all += __shfl_xor_sync(0xffffffffu, l_all, o);
        if (s0 < nsplit) sm_c[s0 * G + g] = c0;
        if (s1 < nsplit) sm_c[s1 * G + g] = c1;
        if (lane == 0) red_m[0][g] = l_all;
    }
    __syncthreads();
    {
        // lane: float4 column `lane` of each of the G heads
        float4 a4[G];
#pragma unroll
        for (int g = 0; g < G; ++g) a4[g] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (uint32_t sp = warp; sp < nsplit; sp += ATT_WARPS) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(pbase + (static_cast<size_t>(sp) * G + g) * ATT_PART + 4) + lane);
                const float c = sm_c[sp * G + g];
                a4[g].x += v.x * c; a4[g].y += v.y * c; a4[g].z += v.z * c; a4[g].w += v.w * c;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) *reinterpret_cast<float4*>(&red_acc[warp][g][4 * lane]) = a4[g];
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < G * ATT_HD; i += ATT_WARPS * 32) {
        const uint32_t g = i / ATT_HD, d = i % ATT_HD;
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) a += red_acc[w][g][d];
        const float l_all = red_m[0][g];
        const float v = l_all > 0.f ? a / l_all : 0.f;
        const size_t o = (static_cast<size_t>(kvh) * G + g) * ATT_HD + d;
        if constexpr (sizeof(OUT) == 4) out[o] = v;
        else out[o] = __float2bfloat16_rn(v);
    }
}

// out[head][d] = sum over splits, renormalised.  grid = n_q heads, block = 128.
template <typename OUT>
__global__ void __launch_bounds__(ATT_HD) attn_combine_kernel(const float* __restrict__ part, uint32_t nsplit, uint32_t G,
                                                              OUT* __restrict__ out) {
    const uint32_t head = blockIdx.x, kvh = head / G, g = head % G, d = threadIdx.x;
    float m_all = -CUDART_INF_F;
    for (uint32_t s = 0; s < nsplit; ++s) m_all = fmaxf(m_all, part[((static_cast<size_t>(kvh) * nsplit + s) * G + g) * ATT_PART]);
    float l_all = 0.f, a = 0.f;
    for (uint32_t s = 0; s < nsplit; ++s) {
        const float* src = part + ((static_cast<size_t>(kvh) * nsplit + s) * G + g) * ATT_PART;
        const float c = src[0] == -CUDART_INF_F ? 0.f : __expf(src[0] - m_all);
        l_all += src[1] * c;
        a += src[4 + d] * c;
    }
    const float v = l_all > 0.f ? a / l_all : 0.f;
    if constexpr (sizeof(OUT) == 4) out[static_cast<size_t>(head) * ATT_HD + d] = v;
    else out[static_cast<size_t>(head) * ATT_HD + d] = __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------ prefill attention (causal, tensor cores)
// grid (ceil(m / tokens per CTA), n_kv_heads), 4 warps per CTA.  A warp owns 16 rows = 16 / G query tokens x the
// G heads of its KV head (row r: token r / G, head r % G) and walks the cached positions [0, pos0 + token] in
// steps of 16 with the decode kernel's two products (mma.sync m16n8k16: K codes as the exact f16 integers
// 1024 + (code + 128), V codes as f16 subnormals gathered byte-wise from pairs of rows, P * vscale straight
// from the score accumulators), here with all 16 rows of the A operand in use.  The K / V rows of a KV head are
// shared by the warps and CTAs of that head through L2 (1 MB per head at 8192 positions).  Heavy tiles (late
// tokens) are scheduled first.  q is read rotated and scaled (rope_kv_append_kernel ran before).
constexpr int PF_WARPS = 4;

template <int G, typename OUT>
__global__ void __launch_bounds__(PF_WARPS * 32) attn_prefill_kernel(const float* __restrict__ qkv, uint32_t row_stride, uint32_t m,
                                                                     const int8_t* __restrict__ k_codes, const float* __restrict__ k_scale,
                                                                     const int8_t* __restrict__ v_codes, const float* __restrict__ v_scale,
                                                                     uint32_t max_seq, uint32_t pos0, OUT* __restrict__ out,
                                                                     uint32_t out_stride) {
    constexpr uint32_t TPW = 16 / G;                        // tokens per warp
    const uint32_t kvh = blockIdx.y, tile = gridDim.x - 1 - blockIdx.x;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, t = lane & 3;
    const uint32_t wtok0 = (tile * PF_WARPS + warp) * TPW;
    if (wtok0 >= m) return;
    const int8_t* kc = k_codes + static_cast<size_t>(kvh) * max_seq * ATT_HD;
    const int8_t* vc = v_codes + static_cast<size_t>(kvh) * max_seq * ATT_HD;
    const float* ksc = k_scale + static_cast<size_t>(kvh) * max_seq;
    const float* vsc = v_scale + static_cast<size_t>(kvh) * max_seq;
    const uint32_t wlast = pos0 + min(wtok0 + TPW, m) - 1;  // last position any row of this warp sees
    // this lane's two rows: gid and gid + 8
    uint32_t rtok[2], rlast[2];
    uint32_t qa[4][8];                                      // A fragments of the 8 k-steps: [a0 a1 a2 a3][j]
    float qfix[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t r = gid + 8 * h;
        rtok[h] = wtok0 + r / G;
        const bool live = rtok[h] < m;
        rlast[h] = live ? pos0 + rtok[h] : wlast;           // (rows past the end compute on zeros and are not stored)
        const float* q = qkv + static_cast<size_t>(live ? rtok[h] : 0) * row_stride + (static_cast<size_t>(kvh) * G + r % G) * ATT_HD + 32 * t;
        float qsum = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 q4 = live ? __ldg(reinterpret_cast<const float4*>(q) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            const __half2 lo2 = __floats2half2_rn(q4.x, q4.y), hi2 = __floats2half2_rn(q4.z, q4.w);
            qa[h][j] = *reinterpret_cast<const uint32_t*>(&lo2);
            qa[2 + h][j] = *reinterpret_cast<const uint32_t*>(&hi2);
            qsum += (__low2float(lo2) + __high2float(lo2)) + (__low2float(hi2) + __high2float(hi2));
        }
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
        qfix[h] = 1152.0f * qsum;
    }
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f}, lfix[2] = {0.f, 0.f};
    float o[16][4];                                         // [tile j]: rows gid (0,1) and gid + 8 (2,3), dims 32t + j and 32t + 16 + j
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    for (uint32_t p0 = 0; p0 <= wlast; p0 += 16) {
        uint4 kq[2][2], vq[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const uint4* kr = reinterpret_cast<const uint4*>(kc + static_cast<size_t>(min(p0 + 8 * nt + gid, wlast)) * ATT_HD + 32 * t);
            kq[nt][0] = kr[0];
            kq[nt][1] = kr[1];
        }
        const uint32_t pc[4] = {p0 + 2 * t, p0 + 2 * t + 1, p0 + 2 * t + 8, p0 + 2 * t + 9};
        float kscl[4], vscl[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            vq[i] = *reinterpret_cast<const uint4*>(vc + static_cast<size_t>(min(pc[i], wlast)) * ATT_HD + 16 * gid);
            kscl[i] = ksc[min(pc[i], wlast)];
            vscl[i] = vsc[min(pc[i], wlast)];
        }
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t kw[8] = {kq[nt][0].x, kq[nt][0].y, kq[nt][0].z, kq[nt][0].w, kq[nt][1].x, kq[nt][1].y, kq[nt][1].z, kq[nt][1].w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t x = kw[j] ^ 0x80808080u;
                mma_m16n8k16_f16(c, qa[0][j], qa[1][j], qa[2][j], qa[3][j], __byte_perm(x, 0x64646464u, 0x4140u), __byte_perm(x, 0x64646464u, 0x4342u));
            }
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    sc[h][2 * nt + i] = pc[2 * nt + i] <= rlast[h] ? (c[2 * h + i] - qfix[h]) * kscl[2 * nt + i] : -CUDART_INF_F;
        }
        uint32_t pa[4];                                     // a0 (row gid, tile 0), a1 (row gid + 8, tile 0), a2, a3 (tile 1)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float bm = fmaxf(fmaxf(sc[h][0], sc[h][1]), fmaxf(sc[h][2], sc[h][3]));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
            const float nm = fmaxf(mx[h], bm);              // finite from the first step on: position 0 is visible to every row
            const float corr = __expf(mx[h] - nm);
            float pr[4], wsum = 0.f, psum = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) pr[i] = __expf(sc[h][i] - nm);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const __half2 w2 = __floats2half2_rn(pr[2 * nt] * vscl[2 * nt] * 256.0f, pr[2 * nt + 1] * vscl[2 * nt + 1] * 256.0f);
                pa[2 * nt + h] = *reinterpret_cast<const uint32_t*>(&w2);
                wsum += __low2float(w2) + __high2float(w2);
                psum += pr[2 * nt] + pr[2 * nt + 1];
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            wsum += __shfl_xor_sync(0xffffffffu, wsum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            wsum += __shfl_xor_sync(0xffffffffu, wsum, 2);
            l[h] = l[h] * corr + psum;
            lfix[h] = lfix[h] * corr + wsum;
            mx[h] = nm;
#pragma unroll
            for (int j = 0; j < 16; ++j) { o[j][2 * h] *= corr; o[j][2 * h + 1] *= corr; }
        }
        const uint32_t va[4] = {vq[0].x ^ 0x80808080u, vq[0].y ^ 0x80808080u, vq[0].z ^ 0x80808080u, vq[0].w ^ 0x80808080u};
        const uint32_t vb[4] = {vq[1].x ^ 0x80808080u, vq[1].y ^ 0x80808080u, vq[1].z ^ 0x80808080u, vq[1].w ^ 0x80808080u};
        const uint32_t vc8[4] = {vq[2].x ^ 0x80808080u, vq[2].y ^ 0x80808080u, vq[2].z ^ 0x80808080u, vq[2].w ^ 0x80808080u};
        const uint32_t vd[4] = {vq[3].x ^ 0x80808080u, vq[3].y ^ 0x80808080u, vq[3].z ^ 0x80808080u, vq[3].w ^ 0x80808080u};
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
            const uint32_t lo01 = __byte_perm(va[c4], vb[c4], 0x5410u), hi01 = __byte_perm(va[c4], vb[c4], 0x7632u);
            const uint32_t lo89 = __byte_perm(vc8[c4], vd[c4], 0x5410u), hi89 = __byte_perm(vc8[c4], vd[c4], 0x7632u);
            const uint32_t b0[4] = {lo01 & 0x00FF00FFu, __byte_perm(lo01, 0u, 0x4341u), hi01 & 0x00FF00FFu, __byte_perm(hi01, 0u, 0x4341u)};
            const uint32_t b1[4] = {lo89 & 0x00FF00FFu, __byte_perm(lo89, 0u, 0x4341u), hi89 & 0x00FF00FFu, __byte_perm(hi89, 0u, 0x4341u)};
#pragma unroll
            for (int i = 0; i < 4; ++i) mma_m16n8k16_f16(o[4 * c4 + i], pa[0], pa[1], pa[2], pa[3], b0[i], b1[i]);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (rtok[h] >= m) continue;
        const uint32_t r = gid + 8 * h;
        const float inv = l[h] > 0.f ? 1.0f / l[h] : 0.f, off = 128.0f * lfix[h] * (1.0f / 256.0f);
        OUT* dst = out + static_cast<size_t>(rtok[h]) * out_stride + (static_cast<size_t>(kvh) * G + r % G) * ATT_HD + 32 * t;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float v0 = (o[j][2 * h] * 65536.0f - off) * inv, v1 = (o[j][2 * h + 1] * 65536.0f - off) * inv;
            if constexpr (sizeof(OUT) == 4) { dst[j] = v0; dst[16 + j] = v1; }
            else { dst[j] = __float2bfloat16_rn(v0); dst[16 + j] = __float2bfloat16_rn(v1); }
        }
    }
}

// ------------------------------------------------------------------ greedy arg-max (+ position advance)
// The index of the largest logit (the lowest index on ties, NaN never wins) goes to *out_id; if
// pos != nullptr the position counter is advanced by one -- the decode loop's hand-over to the next
// step, so that a captured step can be replayed without the host.  ARGMAX_CTAS CTAs scan a slice
// each and leave (value, index) in scratch; the CTA that arrives last picks the winner.
constexpr int ARGMAX_CTAS = 64;

__device__ __forceinline__ void argmax_take(float& best, uint32_t& idx, float ov, uint32_t oi) {
    if (oi != 0xffffffffu && (idx == 0xffffffffu || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
}
__device__ __forceinline__ void argmax_block(float& best, uint32_t& idx, float* bv, uint32_t* bi) {
    for (int o = 16; o > 0; o >>= 1) argmax_take(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < (blockDim.x >> 5) ? bv[threadIdx.x] : -CUDART_INF_F;
        idx = threadIdx.x < (blockDim.x >> 5) ? bi[threadIdx.x] : 0xffffffffu;
        for (int o = 16; o > 0; o >>= 1) argmax_take(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    }
}

// scratch: [0] arrival counter, then ARGMAX_CTAS (value, index) pairs
__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, uint32_t n, uint32_t* __restrict__ out_id,
                                                     uint32_t* __restrict__ pos, uint32_t* __restrict__ scratch) {
    __shared__ float bv[8];
    __shared__ uint32_t bi[8];
    __shared__ uint32_t is_last;
    float best = -CUDART_INF_F;
    uint32_t idx = 0xffffffffu;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = logits[i];
        if (v > best || (idx == 0xffffffffu && v == v)) { best = v; idx = i; }
    }
    argmax_block(best, idx, bv, bi);
    if (threadIdx.x == 0) {
        scratch[2 + 2 * blockIdx.x] = __float_as_uint(best);
        scratch[3 + 2 * blockIdx.x] = idx;
        __threadfence();
        const uint32_t old = atomicAdd(&scratch[0], 1u);
        is_last = old == gridDim.x - 1 ? 1u : 0u;
        if (is_last) scratch[0] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    best = -CUDART_INF_F;
    idx = 0xffffffffu;
    if (threadIdx.x < gridDim.x) {
        best = __uint_as_float(__ldcg(&scratch[2 + 2 * threadIdx.x]));
        idx = __ldcg(&scratch[3 + 2 * threadIdx.x]);
    }
    __syncthreads();
    argmax_block(best, idx, bv, bi);
    if (threadIdx.x == 0) {
        *out_id = idx == 0xffffffffu ? 0u : idx;
        if (pos) *pos += 1;
    }
}

__global__ void __launch_bounds__(256) add_kernel(float* __restrict__ x, const float* __restrict__ d, uint64_t n) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) x[i] += d[i];
}

}  // namespace

cudaError_t launch_get_rows(uint32_t type, const void* w, uint64_t row_bytes, uint32_t n_rows, uint32_t k, const uint32_t* ids,
                            uint32_t m, float* out, uint32_t* status, cudaStream_t st) {
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    switch (type) {
#define HF2Q_CASE(T) case T: get_rows_kernel<T><<<m, 256, 0, st>>>(wb, row_bytes, n_rows, k, ids, out, status); break;
        HF2Q_CASE(HF2Q_TYPE_Q4_0) HF2Q_CASE(HF2Q_TYPE_Q8_0) HF2Q_CASE(HF2Q_TYPE_Q4_K) HF2Q_CASE(HF2Q_TYPE_Q5_K) HF2Q_CASE(HF2Q_TYPE_Q6_K)
        HF2Q_CASE(HF2Q_TYPE_Q4_1) HF2Q_CASE(HF2Q_TYPE_Q5_0) HF2Q_CASE(HF2Q_TYPE_Q5_1) HF2Q_CASE(HF2Q_TYPE_IQ4_NL)
        HF2Q_CASE(HF2Q_TYPE_MLX_AFFINE4_GS32)
#undef HF2Q_CASE
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_rms_norm(float* x, const float* delta, const float* weight, float eps, void* out, uint32_t out_dtype, uint32_t m,
                            uint32_t h, cudaStream_t st) {
    const unsigned threads = h >= 4096 ? 1024 : h >= 1024 ? 512 : 256;
    if (out_dtype == HF2Q_DT_F32) rms_norm_kernel<float><<<m, threads, 0, st>>>(x, delta, weight, eps, static_cast<float*>(out), h);
    else if (out_dtype == HF2Q_DT_BF16) rms_norm_kernel<__nv_bfloat16><<<m, threads, 0, st>>>(x, delta, weight, eps, static_cast<__nv_bfloat16*>(out), h);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_rope_kv_append(float* qkv, uint32_t m, uint32_t n_q, uint32_t n_kv, uint32_t hd, const uint32_t* pos, float theta,
                                  const KvCacheView& kv, uint32_t* status, cudaStream_t st) {
    const uint32_t warps = m * (n_q + 2 * n_kv);
    rope_kv_append_kernel<<<(warps + 7) / 8, 256, 0, st>>>(qkv, m, n_q, n_kv, hd, pos, theta, 1.0f / sqrtf(static_cast<float>(hd)),
                                                            kv.k_codes, kv.k_scale, kv.v_codes, kv.v_scale, kv.max_seq, status);
    return cudaGetLastError();
}

size_t attn_decode_scratch_bytes(uint32_t n_kv, uint32_t group, uint32_t n_splits) {
    // 256 bytes of per-KV-head completion counters (the fused form), then the splits' partial results
    return 256 + static_cast<size_t>(n_kv) * n_splits * group * ATT_PART * sizeof(float);
}

cudaError_t launch_attn_decode(const float* q, uint32_t n_q, uint32_t n_kv, uint32_t hd, const KvCacheView& kv, const uint32_t* pos,
                               void* out, uint32_t out_dtype, float* scratch, uint32_t n_splits, cudaStream_t st) {
    if (hd != ATT_HD || n_kv == 0 || n_q % n_kv || n_q / n_kv > ATT_MAXG) return cudaErrorInvalidValue;
    const uint32_t G = n_q / n_kv;
    const dim3 grid(n_kv, n_splits);
    switch (G) {
#define HF2Q_CASE(GG) case GG: attn_decode_kernel<GG><<<grid, ATT_WARPS * 32, 0, st>>>(q, n_q, kv.k_codes, kv.k_scale, kv.v_codes, kv.v_scale, kv.max_seq, pos, scratch + 64); break;
        HF2Q_CASE(1) HF2Q_CASE(2) HF2Q_CASE(4) HF2Q_CASE(8)
#undef HF2Q_CASE
        default: return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (out_dtype == HF2Q_DT_F32) attn_combine_kernel<float><<<n_q, ATT_HD, 0, st>>>(scratch + 64, n_splits, G, static_cast<float*>(out));
    else if (out_dtype == HF2Q_DT_BF16) attn_combine_kernel<__nv_bfloat16><<<n_q, ATT_HD, 0, st>>>(scratch + 64, n_splits, G, static_cast<__nv_bfloat16*>(out));
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_attn_decode_fused(const float* qkv, uint32_t n_q, uint32_t n_kv, uint32_t hd, float theta, const KvCacheView& kv,
                                     const uint32_t* pos, void* out, uint32_t out_dtype, float* scratch, uint32_t n_splits, uint32_t* status,
                                     cudaStream_t st) {
    if (hd != ATT_HD || n_kv == 0 || n_q % n_kv || n_q / n_kv > ATT_MAXG) return cudaErrorInvalidValue;
    const uint32_t G = n_q / n_kv;
    const dim3 grid(n_kv, n_splits);
    // scratch: [n_kv] counters (256 bytes reserved), then the partial results
    uint32_t* counters = reinterpret_cast<uint32_t*>(scratch);
    float* part = scratch + 64;
    const float qs = 1.0f / sqrtf(static_cast<float>(hd));
    const bool f32 = out_dtype == HF2Q_DT_F32;
    if (!f32 && out_dtype != HF2Q_DT_BF16) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(ATT_WARPS * 32);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    switch (G) {
#define HF2Q_CASE(GG) case GG: \
        if (f32) return cudaLaunchKernelEx(&cfg, attn_decode_fused_kernel<GG, float>, qkv, n_q, n_kv, theta, qs, kv.k_codes, kv.k_scale, kv.v_codes, kv.v_scale, kv.max_seq, pos, part, counters, static_cast<float*>(out), status); \
        return cudaLaunchKernelEx(&cfg, attn_decode_fused_kernel<GG, __nv_bfloat16>, qkv, n_q, n_kv, theta, qs, kv.k_codes, kv.k_scale, kv.v_codes, kv.v_scale, kv.max_seq, pos, part, counters, static_cast<__nv_bfloat16*>(out), status);
        HF2Q_CASE(1) HF2Q_CASE(2) HF2Q_CASE(4) HF2Q_CASE(8)
#undef HF2Q_CASE
        default: return cudaErrorInvalidValue;
    }
}

template <int G, typename OUT>
static cudaError_t launch_prefill_g(const float* qkv, uint32_t row_stride, uint32_t m, const KvCacheView& kv, uint32_t n_kv, uint32_t pos0,
                                    OUT* out, uint32_t out_stride, cudaStream_t st) {
    constexpr uint32_t TOK = PF_WARPS * (16 / G);           // query tokens per CTA
    const dim3 grid((m + TOK - 1) / TOK, n_kv);
    attn_prefill_kernel<G, OUT><<<grid, PF_WARPS * 32, 0, st>>>(qkv, row_stride, m, kv.k_codes, kv.k_scale, kv.v_codes, kv.v_scale, kv.max_seq, pos0,
                                                                out, out_stride);
    return cudaGetLastError();
}

cudaError_t launch_attn_prefill(const float* qkv, uint32_t row_stride, uint32_t m, uint32_t n_q, uint32_t n_kv, uint32_t hd,
                                const KvCacheView& kv, uint32_t pos0, void* out, uint32_t out_dtype, uint32_t out_stride, cudaStream_t st) {
    if (hd != ATT_HD || n_kv == 0 || n_q % n_kv) return cudaErrorInvalidValue;
    const uint32_t G = n_q / n_kv;
    const bool f32 = out_dtype == HF2Q_DT_F32;
    if (!f32 && out_dtype != HF2Q_DT_BF16) return cudaErrorInvalidValue;
    switch (G) {
#define HF2Q_CASE(GG) case GG: return f32 ? launch_prefill_g<GG, float>(qkv, row_stride, m, kv, n_kv, pos0, static_cast<float*>(out), out_stride, st) \
                                          : launch_prefill_g<GG, __nv_bfloat16>(qkv, row_stride, m, kv, n_kv, pos0, static_cast<__nv_bfloat16*>(out), out_stride, st);
        HF2Q_CASE(1) HF2Q_CASE(2) HF2Q_CASE(4) HF2Q_CASE(8)
#undef HF2Q_CASE
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_argmax(const float* logits, uint32_t n, uint32_t* out_id, uint32_t* pos, uint32_t* scratch, cudaStream_t st) {
    argmax_kernel<<<ARGMAX_CTAS, 256, 0, st>>>(logits, n, out_id, pos, scratch);
    return cudaGetLastError();
}

cudaError_t launch_add(float* x, const float* d, uint64_t n, int sm_count, cudaStream_t st) {
    const uint64_t want = (n + 255) / 256, cap = static_cast<uint64_t>(sm_count) * 16;
    add_kernel<<<static_cast<unsigned>(want < cap ? (want ? want : 1) : cap), 256, 0, st>>>(x, d, n);
    return cudaGetLastError();
}

}  // namespace hf2q
