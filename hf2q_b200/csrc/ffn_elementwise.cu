// Element-wise glue of the FFN builders that sit directly on the quantized products:
// SwiGLU (silu(gate) * up) and the MoE combine (weighted sum over the top-k slots, plus the
// sigmoid-gated shared expert and the residual).  Semantics follow hf2q's scalar references
// dense_swiglu_cpu_ref (src/inference/models/qwen35/ffn.rs:91-112) and moe_ffn_cpu_ref
// (ffn.rs:179-336); the reference's GPU builders dispatch dispatch_silu_mul /
// dispatch_moe_weighted_reduce for the same steps (gpu_ffn.rs:1086-1351, 2313-2802).
#include "common.cuh"
#include "kernels.h"

namespace hf2q {
namespace {

__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }     // ffn.rs:24-26

__global__ void __launch_bounds__(256) silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                       float* __restrict__ out, uint64_t n4) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 g = reinterpret_cast<const float4*>(gate)[i], u = reinterpret_cast<const float4*>(up)[i];
        reinterpret_cast<float4*>(out)[i] = make_float4(silu(g.x) * u.x, silu(g.y) * u.y, silu(g.z) * u.z, silu(g.w) * u.w);
    }
}
__global__ void __launch_bounds__(256) silu_mul_tail_kernel(const float* gate, const float* up, float* out, uint64_t from, uint64_t n) {
    const uint64_t i = from + blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = silu(gate[i]) * up[i];
}

// out[t, :] = sum_s w[t*k+s] * y[t*k+s, :]  (+ sigmoid(gate_logit[t]) * shared[t, :])  (+ residual[t, :])
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ w,
                                                          const float* __restrict__ shared, const float* __restrict__ gate_logit,
                                                          const float* __restrict__ residual, float* __restrict__ out,
                                                          uint32_t n_tokens, uint32_t top_k, uint32_t h) {
    const uint32_t t = blockIdx.y;
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_tokens || c >= h) return;
    float acc = 0.f;
    for (uint32_t s = 0; s < top_k; ++s)
        acc += w[t * top_k + s] * y[(static_cast<size_t>(t) * top_k + s) * h + c];      // slot order, as the reference sums
    if (shared) {
        const float gv = gate_logit ? 1.0f / (1.0f + expf(-gate_logit[t])) : 1.0f;      // ffn.rs:28-30
        acc += gv * shared[static_cast<size_t>(t) * h + c];
    }
    if (residual) acc += residual[static_cast<size_t>(t) * h + c];
    out[static_cast<size_t>(t) * h + c] = acc;
}

// out[t] = sum_i v[i] * x[t, i]   (the shared expert's gate logit, a [1, h] f32 matrix)
__global__ void __launch_bounds__(256) rowdot_kernel(const float* __restrict__ x, const float* __restrict__ v, float* __restrict__ out,
                                                     uint32_t n_tokens, uint32_t h) {
    __shared__ float part[8];
    const uint32_t t = blockIdx.x;
    float acc = 0.f;
    for (uint32_t i = threadIdx.x; i < h; i += 256) acc += v[i] * x[static_cast<size_t>(t) * h + i];
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int i = 0; i < 8; ++i) s += part[i];
        out[t] = s;
    }
    (void)n_tokens;
}

// Router logits of an MoE layer: out[t, e] = sum_h x[t, h] * w[e, h], all f32 (the router is a small
// dense f32 matrix in the reference as well: phase 1 of the six-phase graph at gpu_ffn.rs:2347-2359).
// Classic shared-memory tiling: a CTA computes 64 tokens x 64 experts, 4 x 4 outputs per thread.
constexpr int RT = 64, RKT = 16;
__global__ void __launch_bounds__(256) router_logits_kernel(const void* __restrict__ x, uint32_t x_bf16, const float* __restrict__ w,
                                                            float* __restrict__ out, uint32_t n_tokens, uint32_t n_experts, uint32_t h) {
    __shared__ float xs[RKT][RT + 4], ws[RKT][RT + 4];
    const uint32_t t0 = blockIdx.y * RT, e0 = blockIdx.x * RT;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // outputs: tokens 4ty..4ty+3, experts 4tx..4tx+3
    float acc[4][4] = {};
    for (uint32_t k0 = 0; k0 < h; k0 += RKT) {
        for (int i = threadIdx.x; i < RT * RKT; i += 256) {
            const int r = i / RKT, c = i % RKT;
            const uint32_t t = t0 + r, e = e0 + r, kk = k0 + c;
            float xv = 0.f;
            if (t < n_tokens && kk < h)
                xv = x_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(x)[static_cast<size_t>(t) * h + kk])
                            : static_cast<const float*>(x)[static_cast<size_t>(t) * h + kk];
            xs[c][r] = xv;
            ws[c][r] = (e < n_experts && kk < h) ? w[static_cast<size_t>(e) * h + kk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < RKT; ++c) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[c][4 * ty]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[c][4 * tx]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t t = t0 + 4 * ty + i, e = e0 + 4 * tx + j;
            if (t < n_tokens && e < n_experts) out[static_cast<size_t>(t) * n_experts + e] = acc[i][j];
        }
}

}  // namespace

cudaError_t launch_router_logits(const void* x, uint32_t x_bf16, const float* w, float* out, uint32_t n_tokens, uint32_t n_experts,
                                 uint32_t h, cudaStream_t st) {
    const dim3 grid((n_experts + RT - 1) / RT, (n_tokens + RT - 1) / RT);
    router_logits_kernel<<<grid, 256, 0, st>>>(x, x_bf16, w, out, n_tokens, n_experts, h);
    return cudaGetLastError();
}

cudaError_t launch_silu_mul(const float* gate, const float* up, float* out, uint64_t n, int sm_count, cudaStream_t st) {
    const bool vec = (reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
    const uint64_t n4 = vec ? n / 4 : 0;
    if (n4) {
        const uint64_t want = (n4 + 255) / 256, cap = static_cast<uint64_t>(sm_count) * 16;
        silu_mul_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, st>>>(gate, up, out, n4);
    }
    const uint64_t done = n4 * 4;
    if (done < n) silu_mul_tail_kernel<<<static_cast<unsigned>((n - done + 255) / 256), 256, 0, st>>>(gate, up, out, done, n);
    return cudaGetLastError();
}

cudaError_t launch_moe_combine(const float* y, const float* w, const float* shared, const float* gate_logit, const float* residual,
                               float* out, uint32_t n_tokens, uint32_t top_k, uint32_t h, cudaStream_t st) {
    const dim3 grid((h + 255) / 256, n_tokens);
    moe_combine_kernel<<<grid, 256, 0, st>>>(y, w, shared, gate_logit, residual, out, n_tokens, top_k, h);
    return cudaGetLastError();
}

cudaError_t launch_rowdot(const float* x, const float* v, float* out, uint32_t n_tokens, uint32_t h, cudaStream_t st) {
    rowdot_kernel<<<n_tokens, 256, 0, st>>>(x, v, out, n_tokens, h);
    return cudaGetLastError();
}

}  // namespace hf2q
