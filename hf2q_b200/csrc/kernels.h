// Host-side launch interface between the C ABI (api.cu) and the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

struct hf2q_ctx;

namespace hf2q {

// the context's device status word (api.cu), for the translation units that launch kernels outside api.cu
uint32_t* ctx_status_word(hf2q_ctx* ctx);
int32_t ctx_fail(hf2q_ctx* ctx, int32_t code, const char* msg);      // sets the context's last-error text, returns code

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the CURRENT device only, and one
// process may hold contexts on several GPUs: the opt-in is remembered per device, not per process.
constexpr int MAX_DEVICES = 64;
struct PerDeviceFlag {
    std::mutex mu;
    bool set[MAX_DEVICES] = {};
};
template <typename Kernel>
inline cudaError_t ensure_max_dynamic_smem(Kernel kern, int bytes, PerDeviceFlag& flag) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(flag.mu);
    if (!flag.set[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        flag.set[dev] = true;
    }
    return cudaSuccess;
}

// K0 (k0_dequant.cu)
cudaError_t launch_dequant(uint32_t type, const void* w, void* out, uint32_t out_dtype,
                           uint64_t n_elems, int sm_count, cudaStream_t st);

// K1 / K3 (k1_gemv.cu): y[slot*?..] = x . dequant(W)^T for 1..8 activation rows.
// Dense call: ids == nullptr, top_k == 1, slots == 1, m = activation rows (1..8).
// Routed call (mul_mv_id): ids != nullptr, one slot per routed output row, m == 1 per slot;
// slot r reads x row r / top_k and the expert matrix at w + ids[r] * expert_stride.
// Row-sharded product whose all-gather is part of the kernel: every rank's output buffer
// [m][n_total] and arrival counter, as mapped into this process (peer memory for the other ranks).
struct GatherArgs {
    float* y_all[8];
    uint32_t* flags[8];
    uint32_t n_ranks, rank, n_total, col0;   // this rank's rows are columns [col0, col0 + n) of the full output
    uint32_t wait_expected;                  // != 0: wait for the previous products' columns from all ranks before reading x
    uint32_t peer_ctas[8];                   // CTAs rank r launches for this product (gemv_mma_grid_x of its shard)
    long long wait_limit;                    // clock ticks a wait for other ranks may take
};
struct GemvArgs {
    const void* w;
    const void* x;
    float* y;
    const uint32_t* ids;
    uint64_t expert_stride;
    uint32_t x_dtype;
    uint32_t type;
    uint32_t m, n, k;
    uint32_t slots, top_k, n_experts;
    uint32_t* status;
    const GatherArgs* gather = nullptr;      // dense mat-vec only
    // routed pair (two stacked expert tensors of the same geometry, same x and ids): slots [slots, 2*slots)
    // read w2 and write y2; nullptr = single product
    const void* w2 = nullptr;
    float* y2 = nullptr;
    // dense fused SwiGLU: w = gate, w2 = up (same geometry), y = silu(x gate^T) * (x up^T) in one launch
    bool swiglu = false;
    // y = residual + product (dense and routed mat-vec; may alias y); nullptr = plain product
    const float* residual = nullptr;
    // RMSNorm fused in front of the product: x is normalised with this f32 [k] weight while the
    // activation panel is built (f32 x, m <= 4, the whole row resident); nullptr = none
    const float* norm_weight = nullptr;
    float norm_eps = 0.f;
    // scratch for the split-k form of long rows (the context's; nullptr = k-phases instead), and where to
    // report that a call took two launches
    float* splitk_scratch = nullptr;
    uint64_t splitk_bytes = 0;
    int* n_launches = nullptr;
};
struct DeviceInfo {
    int sm_count;
    int max_smem_optin;
};
cudaError_t launch_gemv(const GemvArgs& a, const DeviceInfo& dev, cudaStream_t st, int* launches);

// Tensor-core (warp MMA) variant of the same product (k1_gemv_mma.cu).  One launch handles up to
// gemv_mma_max_rows() activation rows; needs 16-byte aligned rows and k % 256 == 0.
bool gemv_mma_supported(const GemvArgs& a);
uint32_t gemv_mma_max_rows(uint32_t type, uint32_t k, uint32_t x_dtype, const DeviceInfo& dev);
cudaError_t launch_gemv_mma(const GemvArgs& a, const DeviceInfo& dev, cudaStream_t st);
bool gemv_mma_norm_ok(uint32_t type, uint32_t k, uint32_t m, const DeviceInfo& dev);
// whether one launch can take m activation rows with the SwiGLU epilogue (all of k resident, k > 1024)
bool gemv_mma_swiglu_ok(uint32_t type, uint32_t k, uint32_t m, uint32_t x_dtype, const DeviceInfo& dev);
// CTAs along x that launch_gemv_mma uses for a dense product of n rows (one per SM, at most one per row group)
uint32_t gemv_mma_grid_x(uint32_t n, uint32_t k, const DeviceInfo& dev);
// bounded wait (one warp) until every other rank's arrival counter flag[r] has caught up with the expected
// count flag[8 + r]; a timeout (after `limit` clock ticks) sets STATUS_WAIT_TIMEOUT
cudaError_t launch_gather_wait(const uint32_t* flag, uint32_t n_ranks, uint32_t rank, long long limit, uint32_t* status, cudaStream_t st);
// src[0 .. n) -> columns [col0, col0 + n) of row 0 of every rank's buffer + the arrival signalling of the fused gather
cudaError_t launch_gather_copy(const float* src, const GatherArgs& g, uint32_t n, const uint32_t* n_each, cudaStream_t st);
// waits like launch_gather_wait, then x[i] += sum_{r < n_parts} parts[r * stride + i], i < n (in order)
cudaError_t launch_gather_take(const uint32_t* flag, uint32_t n_ranks, uint32_t rank, long long limit, uint32_t* status, const float* src,
                               uint32_t pitch, uint32_t width, uint32_t m, float* dst, int sm_count, cudaStream_t st);
cudaError_t launch_gather_sum(const uint32_t* flag, uint32_t n_ranks, uint32_t rank, long long limit, uint32_t* status, const float* parts,
                              uint32_t stride, uint32_t n_parts, float* x, uint32_t n, cudaStream_t st);

// mlx-affine arrays (u32 codes [groups][4], f32 scales, f32 biases) -> 24-byte blocks (k0_dequant.cu)
cudaError_t launch_affine_pack(const uint32_t* codes, const float* scales, const float* biases, uint64_t n_groups, void* out, int sm_count,
                               cudaStream_t st);

// K2 (k2_gemm_tc.cu): tcgen05 GEMM for many activation rows.  Needs k % 256 == 0, 16-byte aligned
// rows and a workspace of gemm_tc_workspace_bytes(m, k) for the f16 copy of the activations.
bool gemm_tc_supported(uint32_t type, const void* w, uint32_t n, uint32_t k);
uint64_t gemm_tc_workspace_bytes(uint32_t m, uint32_t k);
// ldy: floats between activation rows of y (0 = n); x_ready: the workspace already holds the f16 copy of x;
// perm_head_dim != 0: x is stored [k / head_dim][m][head_dim] (attention output, heads outermost)
cudaError_t launch_gemm_tc(uint32_t type, const void* w, const void* x, uint32_t x_dtype, float* y, uint32_t m, uint32_t n,
                           uint32_t k, void* workspace, uint32_t* status, int sm_count, cudaStream_t st, int* launches,
                           uint32_t ldy = 0, bool x_ready = false, const float* residual = nullptr, uint32_t perm_head_dim = 0);
// y[m][n] = silu(x . gate^T) * (x . up^T) in one launch (the five main formats)
bool gemm_tc_swiglu_supported(uint32_t type);
cudaError_t launch_gemm_tc_swiglu(uint32_t type, const void* w_gate, const void* w_up, const void* x, uint32_t x_dtype, float* y,
                                  uint32_t m, uint32_t n, uint32_t k, void* workspace, uint32_t* status, int sm_count,
                                  cudaStream_t st, int* launches, bool x_ready = false);

// K4: grouped expert-routed product.  moe_scratch_layout() carves the caller's scratch into header
// (tile count, sorted-row count), tile table, permutation and the f16 activation panel;
// launch_moe_prep() sorts routed rows by expert and gathers their activations (k4_moe_prep.cu);
// launch_gemm_tc_grouped() is the one grouped tensor-core launch (k2_gemm_tc.cu).
struct MoeScratch {
    uint64_t tiles_off, perm_off, xg_off, total;
    uint32_t max_tiles;
};
uint32_t moe_token_tile(uint32_t rows, uint32_t n_experts);
MoeScratch moe_scratch_layout(uint32_t n_experts, uint32_t rows, uint32_t k);
cudaError_t launch_moe_prep(const uint32_t* ids, uint32_t rows, uint32_t n_experts, uint32_t top_k, uint32_t nt, const void* x,
                            uint32_t x_dtype, uint32_t k, float* y, float* y2, uint32_t n, void* scratch, const MoeScratch& lay,
                            uint32_t* status, int sm_count, cudaStream_t st);   // y2: second output of a pair call or nullptr
bool gemm_tc_grouped_supported(uint32_t type, const void* w, uint64_t expert_stride, uint32_t n_experts, uint32_t k);
cudaError_t launch_gemm_tc_grouped(uint32_t type, const void* w_stacked, uint64_t expert_stride, uint32_t n_experts, uint32_t rows,
                                   float* y, uint32_t n, uint32_t k, uint32_t nt, void* scratch, const MoeScratch& lay,
                                   uint32_t* status, cudaStream_t st, const void* w_up = nullptr, const void* x_panel = nullptr,
                                   void* act16 = nullptr, const float* route_w = nullptr, float* reduce_out = nullptr, uint32_t top_k = 0);

// Fixed scratch of the allocation-free GEMM entry (lives in k2_gemm_tc.cu).
uint64_t gemm_tc_static_scratch_bytes();
cudaError_t gemm_tc_static_scratch(int device, void** out);

// softmax -> top-k -> renormalise (moe_router.cu)
cudaError_t launch_softmax_topk(const float* logits, uint32_t* ids, float* weights,
                                uint32_t n_tokens, uint32_t n_experts, uint32_t top_k,
                                cudaStream_t st);


// ---- the glue of a full decoder forward (decoder_ops.cu) ----
// 8-bit KV cache of one layer: int8 codes [n_kv_heads][max_seq][head_dim] and one f32 scale per
// (head, position), for K and for V.
struct KvCacheView {
    int8_t* k_codes;
    float* k_scale;
    int8_t* v_codes;
    float* v_scale;
    uint32_t max_seq;
};
cudaError_t launch_get_rows(uint32_t type, const void* w, uint64_t row_bytes, uint32_t n_rows, uint32_t k, const uint32_t* ids,
                            uint32_t m, float* out, uint32_t* status, cudaStream_t st);
cudaError_t launch_rms_norm(float* x, const float* delta, const float* weight, float eps, void* out, uint32_t out_dtype, uint32_t m,
                            uint32_t h, cudaStream_t st);
cudaError_t launch_rope_kv_append(float* qkv, uint32_t m, uint32_t n_q, uint32_t n_kv, uint32_t hd, const uint32_t* pos, float theta,
                                  const KvCacheView& kv, uint32_t* status, cudaStream_t st);
size_t attn_decode_scratch_bytes(uint32_t n_kv, uint32_t group, uint32_t n_splits);
cudaError_t launch_attn_decode(const float* q, uint32_t n_q, uint32_t n_kv, uint32_t hd, const KvCacheView& kv, const uint32_t* pos,
                               void* out, uint32_t out_dtype, float* scratch, uint32_t n_splits, cudaStream_t st);
cudaError_t launch_attn_prefill(const float* qkv, uint32_t row_stride, uint32_t m, uint32_t n_q, uint32_t n_kv, uint32_t hd,
                                const KvCacheView& kv, uint32_t pos0, void* out, uint32_t out_dtype, uint32_t out_stride, cudaStream_t st);
// scratch: 1 + 2 * 64 + 1 zero-initialised words owned by the caller (the context), one arg-max at a time
cudaError_t launch_argmax(const float* logits, uint32_t n, uint32_t* out_id, uint32_t* pos, uint32_t* scratch, cudaStream_t st);
// rotary embedding of the query, append of the new position, split attention and merge in one launch;
// scratch as for launch_attn_decode (its first 256 bytes are completion counters and must start zeroed)
cudaError_t launch_attn_decode_fused(const float* qkv, uint32_t n_q, uint32_t n_kv, uint32_t hd, float theta, const KvCacheView& kv,
                                     const uint32_t* pos, void* out, uint32_t out_dtype, float* scratch, uint32_t n_splits, uint32_t* status,
                                     cudaStream_t st);
cudaError_t launch_add(float* x, const float* d, uint64_t n, int sm_count, cudaStream_t st);

// element-wise glue of the FFN builders (ffn_elementwise.cu)
cudaError_t launch_silu_mul(const float* gate, const float* up, float* out, uint64_t n, int sm_count, cudaStream_t st);
cudaError_t launch_moe_combine(const float* y, const float* w, const float* shared, const float* gate_logit, const float* residual,
                               float* out, uint32_t n_tokens, uint32_t top_k, uint32_t h, cudaStream_t st);
cudaError_t launch_router_logits(const void* x, uint32_t x_bf16, const float* w, float* out, uint32_t n_tokens, uint32_t n_experts,
                                 uint32_t h, cudaStream_t st);
cudaError_t launch_rowdot(const float* x, const float* v, float* out, uint32_t n_tokens, uint32_t h, cudaStream_t st);

}  // namespace hf2q
