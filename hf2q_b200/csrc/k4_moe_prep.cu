// K4 preparation: device-side grouping of routed rows by expert for the grouped tensor-core
// product (mul_mat_id with many rows).
//
// Stands in for mlx-native's kernel_mul_mm_id_map0 stage that hf2q reaches through
// quantized_matmul_id_ggml_pooled (src/inference/models/qwen35/gpu_ffn.rs:188-206; the scratch it
// fills is IdMmScratch, decode_pool.rs:205-214): ids[n_tokens*top_k] -> per-expert row lists.
// Here one counting sort produces (a) perm[]: routed-row indices grouped by expert, (b) a table of
// token tiles (expert, first sorted row, row count) that the grouped GEMM walks with ONE launch,
// and then the activation rows are gathered into that order as f16.
#include <cstdlib>
#include "common.cuh"
#include "kernels.h"

namespace hf2q {

namespace {

constexpr int SORT_THREADS = 1024;

// Single CTA: histogram, exclusive scans, scatter.  Shared memory: 4 arrays of (E+1) u32 + 66 words of scan scratch.
// The ids are read 16 per thread and step with all loads in flight (the kernel is one CTA deep in load latency
// otherwise), the two scans over the experts are block-wide shuffle scans.
__device__ __forceinline__ void load_ids16(const uint32_t* __restrict__ ids, uint32_t r0, uint32_t rows, bool vec, uint32_t (&e)[16]) {
    if (vec && r0 + 16 <= rows) {
        const uint4* p = reinterpret_cast<const uint4*>(ids + r0);
        const uint4 a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2), d = __ldg(p + 3);
        e[0] = a.x; e[1] = a.y; e[2] = a.z; e[3] = a.w; e[4] = b.x; e[5] = b.y; e[6] = b.z; e[7] = b.w;
        e[8] = c.x; e[9] = c.y; e[10] = c.z; e[11] = c.w; e[12] = d.x; e[13] = d.y; e[14] = d.z; e[15] = d.w;
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) e[j] = r0 + j < rows ? __ldg(ids + r0 + j) : 0xffffffffu;
    }
}

__global__ void __launch_bounds__(SORT_THREADS) moe_sort_kernel(const uint32_t* __restrict__ ids, uint32_t rows, uint32_t n_experts,
                                                                uint32_t nt, uint32_t* __restrict__ header, uint4* __restrict__ tiles,
                                                                uint32_t* __restrict__ perm, float* __restrict__ y, float* __restrict__ y2,
                                                                uint32_t n, uint32_t* status) {
    extern __shared__ uint32_t sm[];
    uint32_t* cnt = sm;                       // [E]
    uint32_t* off = cnt + n_experts;          // [E+1] first sorted row of each expert
    uint32_t* toff = off + n_experts + 1;     // [E+1] first tile of each expert
    uint32_t* cur = toff + n_experts + 1;     // [E]
    uint32_t* wsum = cur + n_experts;         // [32] + [32] warp totals of the two scans, [2] running totals
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool vec = reinterpret_cast<uintptr_t>(ids) % 16 == 0;
    for (uint32_t e = tid; e < n_experts; e += SORT_THREADS) cnt[e] = 0;
    if (tid < 2) wsum[64 + tid] = 0;
    __syncthreads();
    bool bad = false;
    for (uint32_t r0 = tid * 16; r0 < rows; r0 += SORT_THREADS * 16) {
        uint32_t e[16];
        load_ids16(ids, r0, rows, vec, e);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (e[j] < n_experts) atomicAdd(&cnt[e[j]], 1u);
            else bad |= r0 + j < rows;
        }
    }
    if (bad) atomicOr(status, STATUS_BAD_EXPERT_ID);
    __syncthreads();
    // exclusive scans of the row counts and of the tile counts over the experts
    for (uint32_t base = 0; base < n_experts; base += SORT_THREADS) {
        const uint32_t e = base + tid;
        const uint32_t c = e < n_experts ? cnt[e] : 0u, t = (c + nt - 1) / nt;
        uint32_t ic = c, it = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t uc = __shfl_up_sync(0xffffffffu, ic, d), ut = __shfl_up_sync(0xffffffffu, it, d);
            if (lane >= static_cast<uint32_t>(d)) { ic += uc; it += ut; }
        }
        if (lane == 31) { wsum[warp] = ic; wsum[32 + warp] = it; }
        __syncthreads();
        if (warp == 0) {
            uint32_t wc = wsum[lane], wt = wsum[32 + lane];
            const uint32_t tc = wc, tt = wt;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t uc = __shfl_up_sync(0xffffffffu, wc, d), ut = __shfl_up_sync(0xffffffffu, wt, d);
                if (lane >= static_cast<uint32_t>(d)) { wc += uc; wt += ut; }
            }
            wsum[lane] = wc - tc;             // exclusive prefix of the warp totals
            wsum[32 + lane] = wt - tt;
            if (lane == 31) { wsum[66] = wc; wsum[67] = wt; }          // totals of this pass
        }
        __syncthreads();
        if (e < n_experts) {
            off[e] = wsum[64] + wsum[warp] + ic - c;
            toff[e] = wsum[65] + wsum[32 + warp] + it - t;
        }
        __syncthreads();
        if (tid == 0) { wsum[64] += wsum[66]; wsum[65] += wsum[67]; }
        __syncthreads();
    }
    if (tid == 0) {
        off[n_experts] = wsum[64]; toff[n_experts] = wsum[65];
        header[0] = wsum[65];       // number of token tiles
        header[1] = wsum[64];       // number of sorted (valid) rows
    }
    for (uint32_t e = tid; e < n_experts; e += SORT_THREADS) {
        cur[e] = off[e];
        const uint32_t c = cnt[e];
        for (uint32_t j = 0, t = toff[e]; j * nt < c; ++j, ++t)
            tiles[t] = make_uint4(e, off[e] + j * nt, min(nt, c - j * nt), 0u);
    }
    __syncthreads();
    for (uint32_t r0 = tid * 16; r0 < rows; r0 += SORT_THREADS * 16) {
        uint32_t e[16];
        load_ids16(ids, r0, rows, vec, e);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t r = r0 + j;
            if (e[j] < n_experts) {
                perm[atomicAdd(&cur[e[j]], 1u)] = r;
            } else if (r < rows && y) {
                for (uint32_t c = 0; c < n; ++c) {                                       // rejected row: defined output
                    y[static_cast<size_t>(r) * n + c] = 0.f;
                    if (y2) y2[static_cast<size_t>(r) * n + c] = 0.f;
                }
            }
        }
    }
}

// One CTA per sorted row: copy the routed row's activations (token = routed row / top_k) as f16.
__global__ void __launch_bounds__(256) moe_gather_kernel(const void* __restrict__ x, uint32_t x_bf16, uint32_t top_k, uint32_t k,
                                                         const uint32_t* __restrict__ header, const uint32_t* __restrict__ perm,
                                                         __half* __restrict__ xg, uint32_t* status) {
    const uint32_t n_sorted = header[1];
    bool clipped = false;
    for (uint32_t pos = blockIdx.x; pos < n_sorted; pos += gridDim.x) {
        const uint32_t tok = perm[pos] / top_k;
        __half* dst = xg + static_cast<size_t>(pos) * k;
        for (uint32_t e = threadIdx.x * 8; e < k; e += 256 * 8) {
            float v[8];
            if (x_bf16) {
                const uint4 r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + static_cast<size_t>(tok) * k + e));
                const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[2 * j] = __uint_as_float(rr[j] << 16);
                    v[2 * j + 1] = __uint_as_float(rr[j] & 0xffff0000u);
                }
            } else {
                const float* src = static_cast<const float*>(x) + static_cast<size_t>(tok) * k + e;
                const float4 a = __ldg(reinterpret_cast<const float4*>(src)), b = __ldg(reinterpret_cast<const float4*>(src + 4));
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            }
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float a = v[2 * j], b = v[2 * j + 1];
                clipped |= (fabsf(a) > 65504.0f) | (fabsf(b) > 65504.0f);
                a = fminf(fmaxf(a, -65504.0f), 65504.0f);
                b = fminf(fmaxf(b, -65504.0f), 65504.0f);
                const __half2 h = __floats2half2_rn(a, b);
                o[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(dst + e) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    if (clipped) atomicOr(status, STATUS_X_CLIPPED);
}

}  // namespace

// tokens per tile of the grouped product for `rows` routed rows over `n_experts` experts
uint32_t moe_token_tile(uint32_t rows, uint32_t n_experts) {
    static const int forced = [] { const char* v = getenv("HF2Q_CUDA_MOE_NT"); return v && *v ? atoi(v) : 0; }();   // tuning aid
    if (forced == 32 || forced == 64 || forced == 128 || forced == 256) return static_cast<uint32_t>(forced);
    const uint32_t avg = rows / (n_experts ? n_experts : 1);
    // (128-token tiles run two CTAs per SM like the smaller ones, and a tile that holds all rows of its expert
    // dequantises that expert's weights once)
    return avg <= 20 ? 32 : avg <= 40 ? 64 : avg <= 192 ? 128 : 256;
}

MoeScratch moe_scratch_layout(uint32_t n_experts, uint32_t rows, uint32_t k) {
    MoeScratch s{};
    s.max_tiles = rows / 32 + n_experts + 1;          // bound for the smallest tile (32 rows)
    uint64_t o = 256;                                 // header
    s.tiles_off = o;  o += static_cast<uint64_t>(s.max_tiles) * 16;  o = (o + 255) & ~255ull;
    s.perm_off = o;   o += static_cast<uint64_t>(rows) * 4;          o = (o + 255) & ~255ull;
    s.xg_off = o;     o += static_cast<uint64_t>(rows) * k * 2;      o = (o + 255) & ~255ull;
    s.total = o;
    return s;
}

cudaError_t launch_moe_prep(const uint32_t* ids, uint32_t rows, uint32_t n_experts, uint32_t top_k, uint32_t nt, const void* x,
                            uint32_t x_dtype, uint32_t k, float* y, float* y2, uint32_t n, void* scratch, const MoeScratch& lay,
                            uint32_t* status, int sm_count, cudaStream_t st) {
    uint8_t* base = static_cast<uint8_t*>(scratch);
    uint32_t* header = reinterpret_cast<uint32_t*>(base);
    uint4* tiles = reinterpret_cast<uint4*>(base + lay.tiles_off);
    uint32_t* perm = reinterpret_cast<uint32_t*>(base + lay.perm_off);
    __half* xg = reinterpret_cast<__half*>(base + lay.xg_off);
    const size_t smem = (4 * static_cast<size_t>(n_experts) + 2 + 68) * 4;
    moe_sort_kernel<<<1, SORT_THREADS, smem, st>>>(ids, rows, n_experts, nt, header, tiles, perm, y, y2, n, status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const unsigned grid = rows < static_cast<uint32_t>(sm_count) * 8 ? rows : static_cast<uint32_t>(sm_count) * 8;
    moe_gather_kernel<<<grid, 256, 0, st>>>(x, x_dtype == HF2Q_DT_BF16, top_k, k, header, perm, xg, status);
    return cudaGetLastError();
}

}  // namespace hf2q
