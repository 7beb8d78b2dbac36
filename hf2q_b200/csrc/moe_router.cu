// Router helper for the expert-routed product: softmax over the experts, top-k by probability,
// renormalise.  Semantics of hf2q's softmax_topk_renorm_cpu
// (src/inference/models/qwen35/gpu_ffn.rs:1879-1924), which its GPU path reaches through
// dispatch_moe_softmax_topk (gpu_ffn.rs:2551): descending probability, equal probabilities keep
// the lower expert index first (the reference sorts stably), weights = p / sum(selected p), with
// the same 1e-20 guards.  One warp per token; probabilities live in shared memory.
#include <math_constants.h>

#include "common.cuh"
#include "kernels.h"

namespace hf2q {

namespace {
constexpr int WARPS = 4;

__global__ void __launch_bounds__(WARPS * 32) softmax_topk_kernel(const float* __restrict__ logits,
                                                                  uint32_t* __restrict__ ids,
                                                                  float* __restrict__ weights,
                                                                  uint32_t n_tokens, uint32_t n_experts,
                                                                  uint32_t top_k) {
    extern __shared__ float probs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t t = blockIdx.x * WARPS + warp;
    if (t >= n_tokens) return;
    float* probs = probs_all + static_cast<size_t>(warp) * n_experts;
    const float* row = logits + static_cast<size_t>(t) * n_experts;

    float mx = -CUDART_INF_F;
    for (uint32_t e = lane; e < n_experts; e += 32) mx = fmaxf(mx, row[e]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float denom = 0.f;
    for (uint32_t e = lane; e < n_experts; e += 32) {
        const float v = expf(row[e] - mx);
        probs[e] = v;
        denom += v;
    }
    for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    const float inv_d = denom > 1e-20f ? 1.0f / denom : 1.0f;
    for (uint32_t e = lane; e < n_experts; e += 32) probs[e] *= inv_d;
    __syncwarp();

    // Selection is total: a NaN probability (a NaN logit, or a row whose logits are all -inf) ranks
    // below every number and among NaNs the lower index wins, so every round finds a candidate
    // (top_k <= n_experts) and no index is ever out of range.  Taken entries are marked -2 in
    // shared memory; the ranking key of a NaN is -1, so the two cannot be confused.  The reported
    // weight is the probability itself (a NaN stays a NaN, as IEEE arithmetic gives the reference).
    float sum_sel = 0.f;
    float my_w = 0.f;          // lane s keeps the s-th selected probability (top_k <= 32 per pass)
    uint32_t my_id = 0;
    for (uint32_t s = 0; s < top_k; ++s) {
        float best = -1.5f;    // keys are >= -1; taken entries (-2) never qualify
        uint32_t bi = 0xffffffffu;
        for (uint32_t e = lane; e < n_experts; e += 32) {
            const float v = probs[e];
            const float key = v != v ? -1.0f : v;
            if (key > best) { best = key; bi = e; }  // strided scan keeps the lowest index on ties
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        float val = 0.f;
        if (bi < n_experts) {                        // always true for top_k <= n_experts; guards the store
            val = probs[bi];
            __syncwarp();
            if (lane == 0) probs[bi] = -2.0f;
        } else {
            bi = 0;
        }
        __syncwarp();
        sum_sel += val;
        if ((s & 31u) == static_cast<uint32_t>(lane)) { my_w = val; my_id = bi; }
        if ((s & 31u) == 31u || s + 1 == top_k) {
            // flush this pass of up to 32 selections; weights are scaled after the loop
            const uint32_t base = s & ~31u;
            if (base + lane <= s) {
                ids[static_cast<size_t>(t) * top_k + base + lane] = my_id;
                weights[static_cast<size_t>(t) * top_k + base + lane] = my_w;
            }
        }
    }
    __syncwarp();
    const float inv_sum = sum_sel > 1e-20f ? 1.0f / sum_sel : 1.0f / static_cast<float>(top_k);
    for (uint32_t s = lane; s < top_k; s += 32) weights[static_cast<size_t>(t) * top_k + s] *= inv_sum;
}
}  // namespace

cudaError_t launch_softmax_topk(const float* logits, uint32_t* ids, float* weights, uint32_t n_tokens,
                                uint32_t n_experts, uint32_t top_k, cudaStream_t st) {
    const size_t smem = static_cast<size_t>(WARPS) * n_experts * sizeof(float);
    if (smem > 48 * 1024) return cudaErrorInvalidValue;
    const unsigned grid = (n_tokens + WARPS - 1) / WARPS;
    softmax_topk_kernel<<<grid, WARPS * 32, smem, st>>>(logits, ids, weights, n_tokens, n_experts, top_k);
    return cudaGetLastError();
}

}  // namespace hf2q
