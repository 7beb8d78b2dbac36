// K0: standalone block dequantisation, W[n,k] blocks -> dense [n,k] (f32 bit-exact, or f16/bf16
// rounded to nearest even).  One thread per output element so stores coalesce; the block header
// re-reads hit L1.  Stands in for mlx-native's dequant-to-f16 kernel that hf2q reaches through
// dequant_to_f16::materialize_f16_shadow (src/serve/forward_mlx.rs:9440) and for the CPU
// GgufFile::load_tensor_f32 its loaders use.
#include "common.cuh"
#include "kernels.h"

namespace hf2q {

template <typename T> __device__ __forceinline__ T cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half cvt_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

template <uint32_t TYPE, typename OUT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ w,
                                                      OUT* __restrict__ out, uint64_t n_elems) {
    constexpr BlockGeom G = block_geom(TYPE);
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_elems;
         i += stride) {
        const uint64_t blk = i / G.elems;
        const int e = static_cast<int>(i % G.elems);
        out[i] = cvt_out<OUT>(dequant_elem<TYPE>(w + blk * G.bytes, e));
    }
}

template <uint32_t TYPE>
static cudaError_t launch_dequant_t(const void* w, void* out, uint32_t out_dtype, uint64_t n_elems,
                                    int sm_count, cudaStream_t st) {
    const uint64_t want = (n_elems + 255) / 256;
    const uint64_t cap = static_cast<uint64_t>(sm_count) * 32;
    const unsigned grid = static_cast<unsigned>(want < cap ? (want ? want : 1) : cap);
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    switch (out_dtype) {
        case HF2Q_DT_F32:
            dequant_kernel<TYPE, float><<<grid, 256, 0, st>>>(wb, static_cast<float*>(out), n_elems);
            break;
        case HF2Q_DT_F16:
            dequant_kernel<TYPE, __half><<<grid, 256, 0, st>>>(wb, static_cast<__half*>(out), n_elems);
            break;
        case HF2Q_DT_BF16:
            dequant_kernel<TYPE, __nv_bfloat16>
                <<<grid, 256, 0, st>>>(wb, static_cast<__nv_bfloat16*>(out), n_elems);
            break;
        default:
            return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_dequant(uint32_t type, const void* w, void* out, uint32_t out_dtype,
                           uint64_t n_elems, int sm_count, cudaStream_t st) {
    switch (type) {
        case HF2Q_TYPE_Q4_0: return launch_dequant_t<HF2Q_TYPE_Q4_0>(w, out, out_dtype, n_elems, sm_count, st);
        case HF2Q_TYPE_Q8_0: return launch_dequant_t<HF2Q_TYPE_Q8_0>(w, out, out_dtype, n_elems, sm_count, st);
        case HF2Q_TYPE_Q4_K: return launch_dequant_t<HF2Q_TYPE_Q4_K>(w, out, out_dtype, n_elems, sm_count, st);
        case HF2Q_TYPE_Q5_K: return launch_dequant_t<HF2Q_TYPE_Q5_K>(w, out, out_dtype, n_elems, sm_count, st);
        case HF2Q_TYPE_Q6_K: return launch_dequant_t<HF2Q_TYPE_Q6_K>(w, out, out_dtype, n_elems, sm_count, st);
        case HF2Q_TYPE_Q4_1: return launch_dequant_t<HF2Q_TYPE_Q4_1>(w, out, out_dtype, n_elems, sm_count, st);
        case HF2Q_TYPE_Q5_0: return launch_dequant_t<HF2Q_TYPE_Q5_0>(w, out, out_dtype, n_elems, sm_count, st);
        case HF2Q_TYPE_Q5_1: return launch_dequant_t<HF2Q_TYPE_Q5_1>(w, out, out_dtype, n_elems, sm_count, st);
        case HF2Q_TYPE_IQ4_NL: return launch_dequant_t<HF2Q_TYPE_IQ4_NL>(w, out, out_dtype, n_elems, sm_count, st);
        case HF2Q_TYPE_MLX_AFFINE4_GS32: return launch_dequant_t<HF2Q_TYPE_MLX_AFFINE4_GS32>(w, out, out_dtype, n_elems, sm_count, st);
        default: return cudaErrorInvalidValue;
    }
}

// mlx-affine arrays -> the library's 24-byte blocks (f32 scale, f32 bias, 16 code bytes): one thread per group of
// 32 elements.  The four u32 words of a group hold its 32 nibbles already in element order (mlx packs element i
// of a word into bits 4 (i % 8) ..), so the code bytes are copied as they are.
__global__ void __launch_bounds__(256) affine_pack_kernel(const uint32_t* __restrict__ codes, const float* __restrict__ scales,
                                                          const float* __restrict__ biases, uint64_t n_groups, uint8_t* __restrict__ out) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t g = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < n_groups; g += stride) {
        const uint4 c = __ldg(reinterpret_cast<const uint4*>(codes) + g);
        uint32_t* dst = reinterpret_cast<uint32_t*>(out + g * 24);          // 24 g is a multiple of 8
        dst[0] = __float_as_uint(__ldg(scales + g));
        dst[1] = __float_as_uint(__ldg(biases + g));
        dst[2] = c.x; dst[3] = c.y; dst[4] = c.z; dst[5] = c.w;
    }
}

cudaError_t launch_affine_pack(const uint32_t* codes, const float* scales, const float* biases, uint64_t n_groups, void* out, int sm_count,
                               cudaStream_t st) {
    uint64_t want = (n_groups + 255) / 256;
    const uint64_t cap = static_cast<uint64_t>(sm_count) * 16;
    affine_pack_kernel<<<static_cast<unsigned>(want < cap ? (want ? want : 1) : cap), 256, 0, st>>>(codes, scales, biases, n_groups,
                                                                                                    static_cast<uint8_t*>(out));
    return cudaGetLastError();
}

}  // namespace hf2q
