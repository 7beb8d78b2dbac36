/*
 * hf2q_cuda.h -- C ABI of the B200 (sm_100a) backend for hf2q's quantized-weight matmul path.
 *
 * Every entry point is plain C: pointers, sizes and integer tags only.  The functions are the ones
 * a `hf2q-cuda-sys` FFI crate would bind in place of the calls hf2q makes today into the external
 * mlx-native crate; each declaration cites the hf2q call site or type it stands in for (paths are
 * relative to the hf2q source tree).
 *
 * Conventions kept from the reference's op surface
 *   - enqueue, do not execute: compute calls launch on the caller's stream and return; they never
 *     synchronise and never allocate (gpu_ffn.rs:1044-1049, 2300-2311; scratch is passed in, as
 *     with IdMmScratch, decode_pool.rs:181-228).  The *_host convenience calls are the exception
 *     and say so.
 *   - buffers are caller-owned; outputs must be pre-sized (gpu_ffn.rs:757-763).
 *   - unsupported types and malformed shapes are errors, never a silent fallback
 *     (forward_mlx.rs:9647-9651; weight_loader.rs:1059-1079).
 *   - a context is bound to one device and may be used from one thread at a time; the library
 *     keeps no other mutable global state (decode_pool.rs:51-76, serve/gpu.rs:38-39).
 *
 * `stream` arguments are `cudaStream_t` passed as `void*` (NULL = the legacy default stream).
 */
#ifndef HF2Q_CUDA_H
#define HF2Q_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define HF2Q_API __attribute__((visibility("default")))
#else
#define HF2Q_API
#endif

typedef struct hf2q_ctx hf2q_ctx;

/* Status codes (the reference returns Result<(), MlxError>: InvalidArgument, CommandBufferError,
 * IoError -- gpu_ffn.rs:160, 207). */
enum {
    HF2Q_OK = 0,
    HF2Q_ERR_INVALID_ARGUMENT = 1, /* null pointer, zero or mismatched shape, misaligned buffer   */
    HF2Q_ERR_UNSUPPORTED_TYPE = 2, /* type outside the block formats listed below                  */
    HF2Q_ERR_CUDA = 3,             /* a CUDA runtime call failed; see hf2q_cuda_last_error        */
    HF2Q_ERR_WORKSPACE = 4,        /* workspace / scratch missing or too small                    */
    HF2Q_ERR_TIMEOUT = 5,          /* a bounded device-side wait gave up (status word non-zero)   */
    HF2Q_ERR_OUT_OF_MEMORY = 6,
    HF2Q_ERR_NO_DEVICE = 7
};

/* GGUF numeric type ids (src/quantize/ggml_quants/ggml_type.rs:18-45).  Q4_0 .. Q6_K are the formats
 * of the quantized-weight matmul path proper; Q4_1, Q5_0, Q5_1 and IQ4_NL are what hf2q's quantizer
 * falls back to for tensors whose row length is not a multiple of 256
 * (tensor_type_fallback, src/quantize/ggml_quants/standard_policy.rs:128-192).  Every entry point
 * takes all nine; the four fall-back formats run on the CUDA-core mat-vec (m <= 8) and on the
 * tensor-core GEMM, but not on the fused epilogue variants, which answer "not supported". */
enum {
    HF2Q_TYPE_Q4_0 = 2,
    HF2Q_TYPE_Q4_1 = 3,
    HF2Q_TYPE_Q5_0 = 6,
    HF2Q_TYPE_Q5_1 = 7,
    HF2Q_TYPE_Q8_0 = 8,
    HF2Q_TYPE_Q4_K = 12,
    HF2Q_TYPE_Q5_K = 13,
    HF2Q_TYPE_Q6_K = 14,
    HF2Q_TYPE_IQ4_NL = 20,
    /* Not a GGML id: mlx-affine 4-bit weights with groups of 32 (MlxAffineExtra, src/serve/forward_mlx.rs:340-360;
     * w = scale * code + bias), in this library's own 24-byte block: f32 scale, f32 bias, 16 bytes of codes with
     * element i in nibble i (low nibble first) -- what hf2q_cuda_affine_pack writes from the three mlx arrays. */
    HF2Q_TYPE_MLX_AFFINE4_GS32 = 1000
};

/* Element types of activations and of dequantised output. */
enum { HF2Q_DT_F32 = 0, HF2Q_DT_F16 = 1, HF2Q_DT_BF16 = 2 };

/* ---- context ------------------------------------------------------------------------------ */

/* GpuContext::new (src/serve/gpu.rs:19-38): binds a device, queries its SM count and shared-memory
 * limits, allocates the 4-byte device status word the bounded waits report through. */
HF2Q_API int32_t hf2q_cuda_ctx_create(int32_t device, hf2q_ctx** out);
HF2Q_API int32_t hf2q_cuda_ctx_destroy(hf2q_ctx* ctx);

/* MlxError's Display (gpu_ffn.rs:160): static text for a status code. */
HF2Q_API const char* hf2q_cuda_strerror(int32_t status);
/* Detail of the last failure on this context (shape that was rejected, CUDA error string). */
HF2Q_API const char* hf2q_cuda_last_error(const hf2q_ctx* ctx);
/* Reads and clears the device status word (synchronises `stream`); HF2Q_ERR_TIMEOUT if a kernel
 * recorded that a bounded wait ran out.  Stands where the reference learns of a failed command
 * buffer at commit_and_wait (gpu_ffn.rs:1036-1040). */
HF2Q_API int32_t hf2q_cuda_check_status(hf2q_ctx* ctx, void* stream);

/* ---- geometry ----------------------------------------------------------------------------- */

/* GgmlType::block_size / type_size (ggml_type.rs:60-127). */
HF2Q_API int32_t hf2q_cuda_block_geometry(uint32_t ggml_type, uint32_t* block_elems,
                                          uint32_t* block_bytes);
/* GgmlType::row_size (ggml_type.rs:131-133): bytes of one row of k elements. */
HF2Q_API int32_t hf2q_cuda_row_bytes(uint32_t ggml_type, uint64_t k, uint64_t* out);
/* ggml_type_stride (gpu_ffn.rs:400-412): bytes of one expert's [rows, cols] slice. */
HF2Q_API int32_t hf2q_cuda_expert_stride(uint32_t ggml_type, uint64_t rows, uint64_t cols,
                                         uint64_t* out);

/* ---- weight residency --------------------------------------------------------------------- */

/* GgufFile::load_tensor as used by load_tensor_with_residency (weight_loader.rs:147-159) and
 * load_gguf_qweight (forward_mlx.rs:9356-9386): copies the raw GGUF block bytes to the device
 * UNCHANGED.  Allocates (load time, not launch path); synchronous.  Free with hf2q_cuda_free. */
HF2Q_API int32_t hf2q_cuda_upload_blocks(hf2q_ctx* ctx, const void* host_bytes, uint64_t nbytes,
                                         void** dev_out);
HF2Q_API int32_t hf2q_cuda_free(hf2q_ctx* ctx, void* dev_ptr);

/* ---- K0: standalone dequantisation -------------------------------------------------------- */

/* dequant_to_f16::materialize_f16_shadow (forward_mlx.rs:9440) and GgufFile::load_tensor_f32
 * (gpu_full_attn.rs upload helpers): W[n,k] blocks -> dense [n,k] of out_dtype.  F32 output is
 * bit-exact with the inverse of the quantizers' re-encode step. */
HF2Q_API int32_t hf2q_cuda_dequantize(hf2q_ctx* ctx, void* stream, const void* w,
                                      uint32_t ggml_type, uint64_t n, uint64_t k, void* out,
                                      uint32_t out_dtype);

/* ---- a4: dense quantized matmul ----------------------------------------------------------- */

/* quantized_matmul_ggml(enc, registry, device, input, weight, &mut out,
 *                       &GgmlQuantizedMatmulParams{m,n,k,ggml_type})
 * (gpu_ffn.rs:1236-1306, gpu_full_attn.rs:848-855, gpu_delta_net.rs:399-407,
 *  forward_mlx.rs:9960-9968):  y[m,n] = x[m,k] . dequant(W[n,k])^T, fp32 accumulation.
 * x is row-major [m,k] of x_dtype (F32 or BF16), y is row-major f32 [m,n], w is the raw block
 * bytes of W.  m <= 8 takes the mat-vec kernel (the reference's MM_ROUTING_THRESHOLD,
 * forward_mlx.rs:9800); larger m takes the tensor-core kernel, which needs the workspace reported
 * by hf2q_cuda_qmatmul_workspace_bytes (0 for m <= 8). */
HF2Q_API int32_t hf2q_cuda_qmatmul(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                   const void* w, float* y, uint32_t m, uint32_t n, uint32_t k,
                                   uint32_t ggml_type, void* workspace, uint64_t workspace_bytes);
HF2Q_API int32_t hf2q_cuda_qmatmul_workspace_bytes(uint32_t m, uint32_t n, uint32_t k,
                                                   uint32_t ggml_type, uint32_t x_dtype,
                                                   uint64_t* out);

/* No counterpart in the reference.  The same product as hf2q_cuda_qmatmul through the tensor-core
 * GEMM, for callers that cannot hand the library a workspace because they cannot allocate device
 * memory at all: code that runs after the host application has handed the device to its own
 * arena or pools (hf2q keeps such arenas for its FFN buffers), plugin or FFI glue
 * that sees only the tensors of one op, and latency-critical loops where a cudaMalloc would stall
 * every stream of the device.  The f16 copy of the activations that the GEMM needs is kept in a
 * fixed array inside the library image instead: 8 MiB per GPU, held from library load to process
 * exit, so m * k must not exceed hf2q_cuda_qmatmul_static_max_elements() (4 194 304; e.g. 512
 * rows of k = 8192); larger products fail with HF2Q_ERR_WORKSPACE and a message saying so.
 * The call allocates nothing (no cudaMalloc / cudaFree, no allocating library routine) and is
 * enqueued on `stream` like the others.  Needs k % 256 == 0 and 16-byte aligned weight rows.
 * The FIRST call on each device looks the array's device address up (cudaGetSymbolAddress, with
 * that device current) and caches it; make that first call before any stream capture begins.
 * All calls on a device share the one array and it keeps the previous call's contents (every
 * element a call reads is written by that call first, so nothing needs clearing); two calls whose
 * kernels can overlap on the GPU -- different streams, or graph branches -- race on it and must be
 * ordered by the caller. */
HF2Q_API int32_t hf2q_cuda_qmatmul_static(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                          const void* w, float* y, uint32_t m, uint32_t n, uint32_t k,
                                          uint32_t ggml_type);
HF2Q_API uint64_t hf2q_cuda_qmatmul_static_max_elements(void);

/* Dense SwiGLU FFN fusions for 1..8 activation rows.  The reference's dense builder
 * (build_dense_ffn_layer_gpu_q, src/inference/models/qwen35/gpu_ffn.rs:896-960) issues the gate and
 * up products, dispatch_silu_mul, the down product and, with `add_residual`, an elementwise_add;
 * here that is two launches:
 *   hf2q_cuda_qmatmul_swiglu: y[m][n] = silu(x * Wgate^T) .* (x * Wup^T), silu(v) = v / (1 + exp(-v));
 *     every CTA walks a row group first in the gate and then in the up tensor (same geometry, both
 *     raw-block uploads) and its reducer applies the activation, so neither product is ever stored.
 *     One launch only: hf2q_cuda_qmatmul_swiglu_supported() returns 1 when (m, k, type, x_dtype) fits
 *     (k % 256 == 0, k > 1024, 16-byte aligned rows, all m activation rows resident: bf16 m <= 8,
 *     f32 m <= 4, smaller for very long rows); otherwise the call fails with
 *     HF2Q_ERR_INVALID_ARGUMENT and the caller issues the three separate ops.
 *   hf2q_cuda_qmatmul_add: y = residual + x * W^T (residual [m][n] f32, may be y itself); mat-vec
 *     path only (k % 256 == 0, 16-byte aligned rows: hf2q_cuda_qmatmul_add_supported() returns 1),
 *     any m (8 rows per launch); other shapes fail with HF2Q_ERR_INVALID_ARGUMENT. */
HF2Q_API int32_t hf2q_cuda_qmatmul_swiglu_supported(hf2q_ctx* ctx, uint32_t m, uint32_t n, uint32_t k,
                                                    uint32_t ggml_type, uint32_t x_dtype);
HF2Q_API int32_t hf2q_cuda_qmatmul_swiglu(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                          const void* w_gate, const void* w_up, float* y, uint32_t m,
                                          uint32_t n, uint32_t k, uint32_t ggml_type);
HF2Q_API int32_t hf2q_cuda_qmatmul_add_supported(hf2q_ctx* ctx, uint32_t n, uint32_t k, uint32_t ggml_type,
                                                 uint32_t x_dtype);
HF2Q_API int32_t hf2q_cuda_qmatmul_add(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                       const void* w, const float* residual, float* y, uint32_t m,
                                       uint32_t n, uint32_t k, uint32_t ggml_type);

/* hf2q_cuda_qmatmul for activations stored heads-outermost: x is [k / head_dim][m][head_dim] (what flash
 * attention writes), logical element (t, c) at ((c / head_dim) * m + t) * head_dim + c % head_dim.  Replaces
 * mlx_native::quantized_matmul_mm_tensor_perm021 (params {m, n, k, head_dim, ggml_type}; call site
 * src/serve/forward_prefill_batched.rs:2218-2258, the O projection of the batched prefill).  The permute is
 * folded into the f16 staging of the activations, as the reference folds it into its B-stage; any m runs on
 * the tensor-core GEMM.  head_dim % 8 == 0, x 16-byte aligned, workspace as for hf2q_cuda_qmatmul with m > 8
 * (gemm: m * k * 2 bytes, rounded up to 256). */
HF2Q_API int32_t hf2q_cuda_qmatmul_perm021(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                           const void* w, float* y, uint32_t m, uint32_t n, uint32_t k,
                                           uint32_t head_dim, uint32_t ggml_type, void* workspace,
                                           uint64_t workspace_bytes);

/* The two fusions above for ANY number of activation rows (prefill): up to 8 rows they are the calls above;
 * beyond that the tensor-core GEMM computes the gate and the up tile side by side in tensor memory and
 * stores silu(gate) * up (five main formats), or adds the residual in its epilogue (any format; residual
 * may be y itself).  Workspace as for hf2q_cuda_qmatmul (hf2q_cuda_qmatmul_workspace_bytes(m, n, k, ...)).
 * Replace the reference's gate, up, silu_mul / down, add sequences of build_dense_ffn_layer_gpu_q_into
 * (src/inference/models/qwen35/gpu_ffn.rs:1150-1330) when m > 8.  *_supported() returns 1 when the
 * shape takes the fused form; otherwise the calls fail with HF2Q_ERR_INVALID_ARGUMENT. */
HF2Q_API int32_t hf2q_cuda_qmatmul_swiglu_ws_supported(hf2q_ctx* ctx, uint32_t m, uint32_t n, uint32_t k,
                                                       uint32_t ggml_type, uint32_t x_dtype);
HF2Q_API int32_t hf2q_cuda_qmatmul_swiglu_ws(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                             const void* w_gate, const void* w_up, float* y, uint32_t m,
                                             uint32_t n, uint32_t k, uint32_t ggml_type, void* workspace,
                                             uint64_t workspace_bytes);
HF2Q_API int32_t hf2q_cuda_qmatmul_add_ws_supported(hf2q_ctx* ctx, uint32_t m, uint32_t n, uint32_t k,
                                                    uint32_t ggml_type, uint32_t x_dtype);
HF2Q_API int32_t hf2q_cuda_qmatmul_add_ws(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                          const void* w, const float* residual, float* y, uint32_t m,
                                          uint32_t n, uint32_t k, uint32_t ggml_type, void* workspace,
                                          uint64_t workspace_bytes);

/* mlx-affine (DWQ) weights: `codes` u32 [n][k / 8] (element i of a word in bits 4 (i % 8) .., mlx/ops.cpp
 * packing as MlxQWeight::from_mlx_affine_linear writes it, forward_mlx.rs:425-470), `scales` / `biases` f32
 * [n][k / 32].  Interleaves them, once, at load time, into HF2Q_TYPE_MLX_AFFINE4_GS32 blocks (k / 32 * 24 bytes
 * per row, at `out_blocks`); from then on the weight goes through every entry of this header like any block
 * format -- the replacement for dispatch_qmm_affine_t_packed_simd4_b4 in dispatch_qmatmul's affine branch
 * (forward_mlx.rs:9749-9790) is hf2q_cuda_qmatmul with that type.  bits = 4 and group_size = 32 only, as in
 * the reference. */
HF2Q_API int32_t hf2q_cuda_affine_pack(hf2q_ctx* ctx, void* stream, const uint32_t* codes, const float* scales,
                                       const float* biases, uint32_t n, uint32_t k, uint32_t bits,
                                       uint32_t group_size, void* out_blocks);

/* Same product for callers that hold HOST buffers: copies x in, runs, copies y out, waits.
 * Uses staging buffers the context grows on first use.  Stands for the reference's
 * `apply_linear_projection_f32` + download pattern in its tests (gpu_ffn.rs:3209-3275). */
HF2Q_API int32_t hf2q_cuda_qmatmul_host(hf2q_ctx* ctx, const void* x_host, uint32_t x_dtype,
                                        const void* w_dev, float* y_host, uint32_t m, uint32_t n,
                                        uint32_t k, uint32_t ggml_type);
/* The same call without the wait: work is queued on the context's own streams (copy-in + kernel
 * on one, copy-out on another, so the copy-out of one call overlaps the next kernel) and y_host is
 * valid after hf2q_cuda_host_sync.  x_host and y_host must stay alive until then; pinned memory
 * keeps the copies asynchronous.  Mirrors the reference's "append to the encoder, commit_and_wait
 * once" use of its ops (gpu_ffn.rs:1044-1049, 2300-2311). */
HF2Q_API int32_t hf2q_cuda_qmatmul_host_async(hf2q_ctx* ctx, const void* x_host, uint32_t x_dtype,
                                        const void* w_dev, float* y_host, uint32_t m, uint32_t n,
                                        uint32_t k, uint32_t ggml_type);
/* Many host-buffer products queued by ONE call (a decode step's products, a benchmark pass): copies-in on one
 * stream, the kernels back to back on a second (consecutive mat-vecs overlap as they do for device callers),
 * copies-out on a third; results are valid after hf2q_cuda_host_sync.  Buffers as for
 * hf2q_cuda_qmatmul_host_async (pinned memory for real overlap; alive until the sync).  The products are
 * independent: no item may read another item's output.  A batch that arrives a second time unchanged (same
 * pointers, shapes and types -- a decode loop) is captured into a CUDA graph and replayed from then on: the
 * host buffers are read and written at every call as before, the call itself costs one graph launch
 * (HF2Q_HOST_BATCH_GRAPH=0 in the environment keeps the plain enqueueing).  A batch is recognised by its
 * pointers, shapes and types alone: host buffers that were freed and allocated again at the same addresses
 * must be of the same kind (pinned or pageable) as when the batch was first seen. */
typedef struct hf2q_host_product {
    const void* x_host;   /* [m][k], x_dtype */
    const void* w_dev;    /* device blocks, as for hf2q_cuda_qmatmul */
    float* y_host;        /* [m][n] */
    uint32_t m, n, k, ggml_type, x_dtype, reserved;
} hf2q_host_product;
HF2Q_API int32_t hf2q_cuda_qmatmul_host_batch(hf2q_ctx* ctx, const hf2q_host_product* items, uint32_t n_items);

HF2Q_API int32_t hf2q_cuda_host_sync(hf2q_ctx* ctx);

/* ---- a6: expert-routed quantized matmul --------------------------------------------------- */

/* quantized_matmul_id_ggml_pooled(enc, registry, device, input, weight, ids, out,
 *     &mut IdMmScratch, &GgmlQuantizedMatmulIdParams{n_tokens, top_k, n, k, n_experts,
 *     expert_stride, ggml_type})   (gpu_ffn.rs:188-206, 2606-2618, 2728-2736;
 *  forward_mlx.rs:5285-5292, 5367-5374; forward_prefill_batched.rs:2692-2707, 2805-2820):
 *   y[t*top_k+s, :] = x[t, :] . dequant(W_e)^T,  e = ids[t*top_k+s],
 *   W_e = w_stacked + e*expert_stride (raw blocks of an [n,k] matrix).
 * x is [n_tokens,k] of x_dtype, ids is u32 [n_tokens*top_k] token-major, y is f32
 * [n_tokens*top_k, n].  An id >= n_experts makes that output row zero and sets the status word.
 * Few rows take the per-row mat-vec; many rows take the grouped tensor-core kernel, which sorts
 * rows by expert on the device inside `scratch` (>= hf2q_cuda_qmatmul_id_scratch_bytes). */
HF2Q_API int32_t hf2q_cuda_qmatmul_id(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                      const void* w_stacked, const uint32_t* ids, float* y,
                                      uint32_t n_tokens, uint32_t top_k, uint32_t n, uint32_t k,
                                      uint32_t n_experts, uint64_t expert_stride,
                                      uint32_t ggml_type, void* scratch, uint64_t scratch_bytes);
/* IdMmScratch::alloc(device, n_experts, max_n_tokens) (decode_pool.rs:205-214). */
/* The same product for TWO stacked expert tensors of identical geometry that share x and ids: the
 * gate and up projections of build_moe_ffn_layer_gpu_q_into (gpu_ffn.rs:2606-2618 builds both with one
 * parameter block).  Few routed rows: one launch serves both tensors; many: the sort by expert and
 * the activation gather are done once for both grouped products.  Same scratch as hf2q_cuda_qmatmul_id. */
HF2Q_API int32_t hf2q_cuda_qmatmul_id_pair(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                           const void* w_a, const void* w_b, const uint32_t* ids,
                                           float* y_a, float* y_b, uint32_t n_tokens, uint32_t top_k,
                                           uint32_t n, uint32_t k, uint32_t n_experts, uint64_t expert_stride,
                                           uint32_t ggml_type, void* scratch, uint64_t scratch_bytes);

/* Gate and up of an MoE layer with the SwiGLU in the epilogue, for few routed rows (n_tokens * top_k
 * <= 32, the mat-vec path): y[row][n] = silu(x_tok * Wgate[e]^T) .* (x_tok * Wup[e]^T), e = ids[row].
 * Replaces the two quantized_matmul_id_ggml_pooled calls and the dispatch_silu_mul between them
 * (src/inference/models/qwen35/gpu_ffn.rs:2606-2760) with one launch; hf2q_cuda_qmatmul_id_swiglu_supported
 * returns 1 when the shape fits (k % 256 == 0, k > 1024, 16-byte aligned rows and expert stride),
 * otherwise the call fails with HF2Q_ERR_INVALID_ARGUMENT and the caller uses hf2q_cuda_qmatmul_id_pair
 * + hf2q_cuda_silu_mul.  Rows whose expert index is out of range are zero-filled and flagged. */
HF2Q_API int32_t hf2q_cuda_qmatmul_id_swiglu_supported(hf2q_ctx* ctx, uint32_t n_tokens, uint32_t top_k,
                                                       uint32_t n, uint32_t k, uint32_t ggml_type,
                                                       uint32_t x_dtype);
HF2Q_API int32_t hf2q_cuda_qmatmul_id_swiglu(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                             const void* w_gate, const void* w_up, const uint32_t* ids,
                                             float* y, uint32_t n_tokens, uint32_t top_k, uint32_t n,
                                             uint32_t k, uint32_t n_experts, uint64_t expert_stride,
                                             uint32_t ggml_type);
HF2Q_API int32_t hf2q_cuda_qmatmul_id_scratch_bytes(uint32_t n_experts, uint32_t max_rows,
                                                    uint32_t k, uint32_t x_dtype, uint64_t* out);

/* The routed experts of one MoE layer for MANY routed rows (n_tokens * top_k > 32), four launches:
 *   sort by expert + gather of x as f16;  gate and up tiles side by side with silu(gate) * up stored as
 *   the f16 activation panel in expert-sorted order;  the down product reading that panel, rows
 *   scattered back:  y[n_tokens * top_k][hidden] f32, row r = routed slot r (feed hf2q_cuda_moe_combine).
 * Replaces quantized_matmul_id (gate), (up), dispatch_silu_mul, quantized_matmul_id (down) of
 * build_moe_ffn_layer_gpu_q_into (src/inference/models/qwen35/gpu_ffn.rs:2606-2760).  The activation
 * between the two products is f16, as it is for every tensor-core product of this library.
 * Rows whose expert id is >= n_experts give zero rows and set the bad-expert status bit.
 * w_gate / w_up: n_experts stacked [ffn][hidden] matrices `stride_gate_up` bytes apart (one of the five main
 * formats); w_down: stacked [hidden][ffn], `stride_down` apart.  hidden % 256 == 0, ffn % 256 == 0 and
 * 16-byte aligned rows; hf2q_cuda_moe_experts_supported() returns 1 when the call will run, otherwise use
 * hf2q_cuda_qmatmul_id_swiglu / _pair + hf2q_cuda_qmatmul_id.  scratch: 256-byte aligned,
 * hf2q_cuda_moe_experts_scratch_bytes(). */
HF2Q_API int32_t hf2q_cuda_moe_experts_scratch_bytes(uint32_t n_experts, uint32_t max_rows, uint32_t hidden,
                                                     uint32_t ffn, uint64_t* out);
HF2Q_API int32_t hf2q_cuda_moe_experts_supported(hf2q_ctx* ctx, uint32_t n_tokens, uint32_t top_k, uint32_t hidden,
                                                 uint32_t ffn, uint32_t n_experts, uint32_t type_gate_up,
                                                 uint32_t type_down);
HF2Q_API int32_t hf2q_cuda_moe_experts(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                       const void* w_gate, const void* w_up, const void* w_down,
                                       const uint32_t* ids, float* y, uint32_t n_tokens, uint32_t top_k,
                                       uint32_t hidden, uint32_t ffn, uint32_t n_experts,
                                       uint64_t stride_gate_up, uint32_t type_gate_up, uint64_t stride_down,
                                       uint32_t type_down, void* scratch, uint64_t scratch_bytes);
/* The same four launches with the weighted sum over the top-k slots (dispatch_moe_weighted_reduce,
 * gpu_ffn.rs:2347-2359 phase F) folded into the down product's epilogue: every slot's row, scaled by
 * weights[slot], is ADDED to row slot / top_k of out[n_tokens][hidden] with floating-point atomics.  The caller
 * initialises `out` first (zeros, or shared expert + residual: hf2q_cuda_moe_combine with top_k = 0 writes
 * exactly that).  Saves the [n_tokens * top_k][hidden] f32 round trip and the combine pass; the price is that
 * the rounding of each sum depends on the order in which the experts' tiles finish, so results can differ
 * in the last bits from run to run -- which is why this is a separate, opt-in entry. */
HF2Q_API int32_t hf2q_cuda_moe_experts_reduce(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                              const void* w_gate, const void* w_up, const void* w_down,
                                              const uint32_t* ids, const float* weights, float* out,
                                              uint32_t n_tokens, uint32_t top_k, uint32_t hidden, uint32_t ffn,
                                              uint32_t n_experts, uint64_t stride_gate_up, uint32_t type_gate_up,
                                              uint64_t stride_down, uint32_t type_down, void* scratch,
                                              uint64_t scratch_bytes);


/* dispatch_moe_softmax_topk (gpu_ffn.rs:2551), semantics of softmax_topk_renorm_cpu
 * (gpu_ffn.rs:1879-1924): logits f32 [n_tokens, n_experts] -> ids u32 [n_tokens*top_k] (descending
 * probability, ties to the lower index) and renormalised weights f32 [n_tokens*top_k]. */
HF2Q_API int32_t hf2q_cuda_moe_softmax_topk(hf2q_ctx* ctx, void* stream, const float* logits,
                                            uint32_t* ids, float* weights, uint32_t n_tokens,
                                            uint32_t n_experts, uint32_t top_k);

/* One weight matrix whose ROW RANGES use different block formats -- the Q4_K_M mix keeps the V rows
 * of a fused QKV tensor in Q6_K while the Q and K rows are Q4_K (use_more_bits / attn_v rule,
 * src/quantize/ggml_quants/standard_policy.rs:563-567; per-tensor types in the unfused layout,
 * :646-658).  The reference issues one quantized_matmul_ggml per tensor (gpu_full_attn.rs:848-855,
 * 941-950); here the ranges are given as segments in row order, each with its own raw-block buffer,
 * and the call computes y[m][n] with n = sum of the segments' rows: the activations are converted
 * once and every range writes its own columns of y.  Every segment must fit the kernel that m
 * selects (16-byte aligned weight rows, k % 256 == 0); workspace as for hf2q_cuda_qmatmul. */
typedef struct hf2q_row_segment {
    const void* w;           /* raw blocks of this range's rows, [rows][k / block * block_bytes] */
    uint32_t rows;
    uint32_t ggml_type;
} hf2q_row_segment;
HF2Q_API int32_t hf2q_cuda_qmatmul_segments(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                            const hf2q_row_segment* segs, uint32_t n_segs, float* y,
                                            uint32_t m, uint32_t k, void* workspace, uint64_t workspace_bytes);

/* ---- e: row-sharded mat-vec with the all-gather in its epilogue ------------------------------- *
 * The reference runs on one device and has no collective; this is the multi-GPU form of
 * quantized_matmul_ggml for weights sharded by output rows (one process per GPU).  Every rank owns
 * full-width output buffers [m][n_total] and a 256-byte counter block, allocated with
 * hf2q_cuda_ipc_alloc (zero-filled) and opened by the other ranks with hf2q_cuda_ipc_open (CUDA IPC;
 * needs peer access, i.e. NVLink or PCIe P2P between the GPUs).  hf2q_cuda_qmatmul_gather computes
 * this rank's n rows of the product and stores them into columns [col0, col0 + n) of EVERY rank's
 * buffer (plain stores to peer memory from the kernel's epilogue).  Every CTA then adds 1 to word
 * `rank` of every other rank's counter block (one arrival counter per SOURCE rank, words 0..7), and
 * the launch adds, for every source r, the number of CTAs rank r's shard takes (derived from
 * n_rows[r]) to word 8 + r of the own block (the expected counts).  All ranks issue the same sequence
 * of calls, so a rank holds source r's columns of every product launched so far once word r has
 * caught up with word 8 + r -- independently of what the other sources have delivered and of
 * uneven shards.  A consumer waits for that either inside the next product (wait_previous != 0:
 * the kernel prefetches weights, then waits before it reads x) or with hf2q_cuda_gather_wait.
 * Both waits are bounded (hf2q_cuda_set_wait_limit; about a second by default; a timeout is
 * reported by hf2q_cuda_check_status and leaves the context usable) and depend on device-side
 * counters only, so a captured CUDA graph of such calls can be replayed.
 *
 * Buffers and ordering.  A product must not store into a buffer that some rank may still be
 * reading.  A decode chain (x of product i+1 = gathered output of product i) therefore alternates
 * between TWO output buffers and passes wait_previous != 0 on every product after the first: rank q
 * starts storing product i+1 only after it has seen product i complete on every rank, and a rank
 * signals completion only after all its CTAs have read their activations, so nobody still reads
 * the buffer of product i-1 that product i+1 overwrites.  A product launched with
 * wait_previous == 0 is only ordered by the caller (e.g. a host barrier before it).
 * m <= 8 and the shapes of the tensor-core mat-vec only (16-byte aligned weight rows,
 * k % 256 == 0); one launch per call. */
typedef struct hf2q_gather {
    void* y_all[8];          /* float [m][n_total] of rank 0..n_ranks-1 as mapped in this process */
    void* flags[8];          /* 256-byte counter block of rank 0..n_ranks-1 */
    uint32_t n_ranks, rank;
    uint32_t n_total, col0;
    uint32_t wait_previous;  /* != 0: wait for all ranks' earlier products before reading x */
    uint32_t n_rows[8];      /* rows of rank r's shard of this product (n_rows[rank] == n; the sum must fit n_total) */
} hf2q_gather;
HF2Q_API int32_t hf2q_cuda_ipc_alloc(hf2q_ctx* ctx, uint64_t bytes, void** dev, uint8_t* handle64);
HF2Q_API int32_t hf2q_cuda_ipc_open(hf2q_ctx* ctx, const uint8_t* handle64, void** dev);
HF2Q_API int32_t hf2q_cuda_ipc_close(hf2q_ctx* ctx, void* dev);
HF2Q_API int32_t hf2q_cuda_qmatmul_gather(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                          const void* w, const hf2q_gather* g, uint32_t m, uint32_t n,
                                          uint32_t k, uint32_t ggml_type);
/* Queues a one-warp kernel that waits (bounded) until every other rank's arrivals at this rank have
 * caught up with the products launched here so far; only flags[], n_ranks and rank of g are read. */
HF2Q_API int32_t hf2q_cuda_gather_wait(hf2q_ctx* ctx, void* stream, const hf2q_gather* g);
/* Whether hf2q_cuda_qmatmul_gather takes this product (it runs on the warp-MMA mat-vec only: 16-byte aligned
 * weight rows, k % 256 == 0, one of the five main formats, m within one launch).  When it does not, run the product
 * with hf2q_cuda_qmatmul into a local buffer and distribute it with hf2q_cuda_gather_copy: the exchange of
 * the fused gather without a product -- src[0 .. n) goes to columns [col0, col0 + n) of row 0 of every rank's buffer
 * and the arrival counters are bumped the same way (n_rows[r] = the length rank r copies in the same step). */
HF2Q_API int32_t hf2q_cuda_gather_supported(hf2q_ctx* ctx, const void* w, uint32_t m, uint32_t n, uint32_t k,
                                            uint32_t ggml_type, uint32_t x_dtype);
HF2Q_API int32_t hf2q_cuda_gather_copy(hf2q_ctx* ctx, void* stream, const hf2q_gather* g, const float* src, uint32_t n);

/* The all-reduce of a projection whose CONTRACTION dimension is sharded (the O and down projections of a
 * tensor-parallel decoder: every rank multiplies its columns of the weight with its slice of the activations):
 * each rank runs hf2q_cuda_qmatmul_gather with m = 1, n = the full output length, col0 = rank * n,
 * n_rows[r] = n and n_total >= n_ranks * n, so that the gathered row holds one partial product per rank; this
 * call then waits (bounded, like hf2q_cuda_gather_wait) until every rank's columns have arrived in `g`'s buffer
 * of THIS rank and adds n_parts = n_ranks partials to x in rank order:  x[i] += sum_{r < n_parts} y[r * n + i].
 * Same bits on every rank.  n_parts = 1 adds a gathered full-length result (a row-sharded projection). */
HF2Q_API int32_t hf2q_cuda_gather_sum(hf2q_ctx* ctx, void* stream, const hf2q_gather* g, float* x, uint32_t n,
                                      uint32_t n_parts);
/* hf2q_cuda_qmatmul_host_batch for row-sharded weights: every rank calls it with the same list of products (its own
 * shard in w_dev, n = rows of one shard, equal on all ranks; the same activations in x_host).  Product i runs
 * through hf2q_cuda_qmatmul_gather with wait_previous set, columns [rank * n, (rank + 1) * n), into buffer
 * (first_buf + i) & 1 of the group: g->y_all[] names every rank's buffer 0, its buffer 1 lies buf_stride bytes behind
 * it; pass the parity the group's previous product left off at, the next call continues with first_buf + n_items.
 * A rank whose item has y_host != NULL receives the gathered [m][n_ranks * n] rows there (the rows leave the gather
 * buffer on the kernel stream before that rank's next product, so the two-buffer rule above holds with the copies
 * to the host running behind); y_host == NULL on the ranks that do not need the result on the host.  Copies-in,
 * kernels and copies-out run on the context's three streams as in hf2q_cuda_qmatmul_host_batch; results are valid
 * after hf2q_cuda_host_sync.  The serving shape of a tensor-parallel decode step: hf2q's single-device
 * "append ops, commit_and_wait once" (gpu_ffn.rs:1044-1049) with every weight split by rows over the GPUs. */
HF2Q_API int32_t hf2q_cuda_qmatmul_gather_host_batch(hf2q_ctx* ctx, const hf2q_gather* g, uint64_t buf_stride, uint32_t first_buf,
                                                     const hf2q_host_product* items, uint32_t n_items);

/* Upper bound, in GPU clock ticks, of the device-side waits for other GPUs (the fused gather's
 * arrival counters).  A context setting: set once after creation, never on the launch path.  The
 * default 2^31 ticks is about a second.  After a timeout the waiting kernel records it (reported as
 * HF2Q_ERR_TIMEOUT by hf2q_cuda_check_status), carries on with whatever data is there and returns. */
HF2Q_API int32_t hf2q_cuda_set_wait_limit(hf2q_ctx* ctx, uint64_t clock_ticks);

/* ---- e: the general multi-GPU forms over NCCL ---------------------------------------------------- *
 * One process per GPU.  NCCL is looked up at run time (libnccl.so.2, the copy the host framework has
 * loaded if there is one).  hf2q_cuda_comm_unique_id is called on one rank, its 128 bytes reach the
 * others by the application's own means (a file, MPI, torch.distributed), and every rank then calls
 * hf2q_cuda_comm_create.  No counterpart in the reference, which is single-device. */
typedef struct hf2q_comm hf2q_comm;
HF2Q_API int32_t hf2q_cuda_comm_unique_id(uint8_t* id128);
HF2Q_API int32_t hf2q_cuda_comm_create(int32_t device, const uint8_t* id128, int32_t rank, int32_t world, hf2q_comm** out);
HF2Q_API int32_t hf2q_cuda_comm_destroy(hf2q_comm* comm);
HF2Q_API const char* hf2q_cuda_comm_last_error(const hf2q_comm* comm);
/* quantized_matmul_ggml for weights sharded by output rows, any m: this rank's n_local rows (the same
 * count on every rank), ncclAllGather of the column blocks, unpacked on the device into
 * y_full[m][world * n_local] with rank r's columns at [r * n_local, (r + 1) * n_local). */
HF2Q_API int32_t hf2q_cuda_qmatmul_rowshard_workspace_bytes(uint32_t m, uint32_t n_local, uint32_t k, uint32_t ggml_type,
                                                            uint32_t x_dtype, uint32_t world, uint64_t* out);
HF2Q_API int32_t hf2q_cuda_qmatmul_rowshard(hf2q_ctx* ctx, hf2q_comm* comm, void* stream, const void* x, uint32_t x_dtype,
                                            const void* w_shard, float* y_full, uint32_t m, uint32_t n_local, uint32_t k,
                                            uint32_t ggml_type, void* workspace, uint64_t workspace_bytes);
/* quantized_matmul_id_ggml_pooled with the experts split in contiguous ranges of n_experts / world over
 * the ranks: x_rows[rows][k] holds one activation row per routed row of THIS rank, ids[rows] their
 * global expert indices, w_local this rank's stacked experts; y[rows][n] comes back in the caller's row
 * order.  Routed rows travel to the owner of their expert and the results travel back (two all-to-alls
 * made of ncclSend / ncclRecv groups, packed and unpacked by device kernels).  cap_recv bounds the rows
 * that may ARRIVE at this rank (at most the sum of all ranks' rows); the scratch is sized from it.  The
 * call reads the per-rank row counts back to the host: it synchronises the stream once. */
HF2Q_API int32_t hf2q_cuda_qmatmul_id_ep_scratch_bytes(uint32_t rows, uint32_t cap_recv, uint32_t world, uint32_t n, uint32_t k,
                                                       uint32_t n_experts, uint32_t x_dtype, uint64_t* out);
HF2Q_API int32_t hf2q_cuda_qmatmul_id_ep(hf2q_ctx* ctx, hf2q_comm* comm, void* stream, const void* x_rows, uint32_t x_dtype,
                                         const uint32_t* ids, const void* w_local, float* y, uint32_t rows, uint32_t cap_recv,
                                         uint32_t n, uint32_t k, uint32_t n_experts, uint64_t expert_stride, uint32_t ggml_type,
                                         void* scratch, uint64_t scratch_bytes);

/* The expert part of build_moe_ffn_layer_gpu_q_into (gpu_ffn.rs:2313-2802, phases B-E) expert-parallel:
 * every routed row travels ONCE to the owner of its expert, which runs gate, up, SwiGLU and down on it,
 * and the [hidden] result travels back: y[rows][hidden] = down_e(silu(gate_e x) * (up_e x)), e = ids[row].
 * The weighted sum over the top-k slots stays with the caller (hf2q_cuda_moe_combine). */
HF2Q_API int32_t hf2q_cuda_moe_experts_ep_scratch_bytes(uint32_t rows, uint32_t cap_recv, uint32_t world, uint32_t hidden,
                                                        uint32_t inter, uint32_t n_experts, uint32_t x_dtype, uint64_t* out);
HF2Q_API int32_t hf2q_cuda_moe_experts_ep(hf2q_ctx* ctx, hf2q_comm* comm, void* stream, const void* x_rows, uint32_t x_dtype,
                                          const uint32_t* ids, const void* w_gate_local, const void* w_up_local,
                                          const void* w_down_local, float* y, uint32_t rows, uint32_t cap_recv,
                                          uint32_t hidden, uint32_t inter, uint32_t n_experts, uint64_t stride_gate_up,
                                          uint64_t stride_down, uint32_t type_gate_up, uint32_t type_down, void* scratch,
                                          uint64_t scratch_bytes);

/* ---- a8: element-wise glue of the FFN builders ---------------------------------------------- */

/* dispatch_silu_mul as used by build_dense_ffn_layer_gpu_q_into (gpu_ffn.rs:1086-1351), semantics
 * of dense_swiglu_cpu_ref (ffn.rs:91-112): out[i] = silu(gate[i]) * up[i], silu(x) = x / (1 + e^-x). */
HF2Q_API int32_t hf2q_cuda_silu_mul(hf2q_ctx* ctx, void* stream, const float* gate, const float* up,
                                    float* out, uint64_t n);
/* dispatch_moe_weighted_reduce + shared-expert gate + residual add of
 * build_moe_ffn_layer_gpu_q_into (gpu_ffn.rs:2313-2802), semantics of moe_ffn_cpu_ref
 * (ffn.rs:179-336): out[t,:] = sum_s weights[t*top_k+s] * y[t*top_k+s,:]
 *                             + sigmoid(shared_gate_logit[t]) * shared[t,:]   (if shared != NULL;
 *                               gate 1 if shared_gate_logit == NULL)
 * top_k == 0 (y, weights may be NULL): only the shared-expert and residual terms (zeros without them).
 *                             + residual[t,:]                                 (if residual != NULL). */
HF2Q_API int32_t hf2q_cuda_moe_combine(hf2q_ctx* ctx, void* stream, const float* y, const float* weights,
                                       const float* shared, const float* shared_gate_logit,
                                       const float* residual, float* out, uint32_t n_tokens,
                                       uint32_t top_k, uint32_t hidden);
/* Router logits of build_moe_ffn_layer_gpu_q_into (phase 1 of the graph at gpu_ffn.rs:2347-2359;
 * moe_ffn_cpu_ref ffn.rs:203-214): logits[t, e] = sum_h x[t, h] * router[e, h], router f32
 * [n_experts, hidden], x f32 or bf16. */
HF2Q_API int32_t hf2q_cuda_router_logits(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                         const float* router, float* logits, uint32_t n_tokens,
                                         uint32_t n_experts, uint32_t hidden);
/* The shared expert's gate logit, a [1, hidden] f32 matrix applied per token (ffn.rs:298-304):
 * out[t] = sum_i v[i] * x[t,i]. */
HF2Q_API int32_t hf2q_cuda_rowdot(hf2q_ctx* ctx, void* stream, const float* x, const float* v, float* out,
                                  uint32_t n_tokens, uint32_t hidden);

/* ---- the two FFN builders as single calls ------------------------------------------------------ *
 * build_dense_ffn_layer_gpu_q_into (src/inference/models/qwen35/gpu_ffn.rs:1086-1351) and
 * build_moe_ffn_layer_gpu_q_into (gpu_ffn.rs:2313-2802) composed from the entries above on the caller's
 * stream; every intermediate lives in the ONE scratch buffer the caller passes (the reference pools them
 * per thread, decode_pool.rs:181-228).  Fused kernels are used where the shape takes them; otherwise, or
 * with HF2Q_FFN_NO_FUSION in `flags`, the reference's own op sequence runs -- same values either way.
 *   dense:  y[m][hidden] = down . (silu(gate . x) * (up . x)) (+ residual, which may be y itself)
 *   moe:    router logits -> softmax/top-k/renorm -> routed experts -> weighted sum over the slots
 *           + sigmoid(shared_gate_logit . x) * shared expert + residual   (moe_ffn_cpu_ref, ffn.rs:179-336)
 * scratch: 256-byte aligned, hf2q_cuda_dense_ffn_scratch_bytes / hf2q_cuda_moe_ffn_scratch_bytes. */
#define HF2Q_FFN_NO_FUSION 1u
#define HF2Q_FFN_ATOMIC_COMBINE 2u   /* moe: weighted reduce inside the down product (hf2q_cuda_moe_experts_reduce) */
HF2Q_API int32_t hf2q_cuda_dense_ffn_scratch_bytes(uint32_t m, uint32_t hidden, uint32_t ffn, uint64_t* out);
HF2Q_API int32_t hf2q_cuda_dense_ffn(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                     const void* w_gate, uint32_t type_gate, const void* w_up, uint32_t type_up,
                                     const void* w_down, uint32_t type_down, const float* residual, float* y,
                                     uint32_t m, uint32_t hidden, uint32_t ffn, void* scratch,
                                     uint64_t scratch_bytes, uint32_t flags);
/* MoeFfnWeightsGpuQ (gpu_ffn.rs:362-398) as plain pointers. */
typedef struct hf2q_moe_ffn_weights {
    const float* router;            /* f32 [n_experts][hidden] */
    const void* expert_gate;        /* n_experts stacked [ffn][hidden], stride_gate_up bytes apart */
    const void* expert_up;
    const void* expert_down;        /* n_experts stacked [hidden][ffn], stride_down bytes apart */
    uint64_t stride_gate_up, stride_down;
    uint32_t type_gate_up, type_down;
    uint32_t n_experts, top_k, ffn; /* ffn = moe_intermediate_size */
    uint32_t shared_ffn;            /* intermediate size of the shared expert (ignored without one) */
    const void* shared_gate;        /* shared expert (all three or none) */
    const void* shared_up;
    const void* shared_down;
    uint32_t shared_type_gate, shared_type_up, shared_type_down, reserved;
    const float* shared_gate_logit; /* f32 [hidden] or NULL (gate = 1); needs f32 activations */
} hf2q_moe_ffn_weights;
HF2Q_API int32_t hf2q_cuda_moe_ffn_scratch_bytes(const hf2q_moe_ffn_weights* w, uint32_t n_tokens, uint32_t hidden,
                                                 uint64_t* out);
HF2Q_API int32_t hf2q_cuda_moe_ffn(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                   const hf2q_moe_ffn_weights* w, const float* residual, float* y,
                                   uint32_t n_tokens, uint32_t hidden, void* scratch, uint64_t scratch_bytes,
                                   uint32_t flags);

/* ---- f-3: the glue of a full decoder forward ---------------------------------------------------- *
 * What sits between the quantized products in forward_gpu_greedy
 * (src/inference/models/qwen35/forward_gpu.rs:4140) on Llama-shaped layers.  Arithmetic after the
 * reference's scalar specs: rms_norm_rows and residual_add (forward_cpu.rs:36-56), causal softmax
 * attention (full_attn.rs:219-360, without the output gate, with the plain rotary embedding of the
 * Llama architecture: pairs (2i, 2i+1), angle pos * theta^(-2i/head_dim)), embed_tokens /
 * apply_output_head (io_heads.rs).
 *
 * KV cache of one layer, laid out like TqFullAttnKvBuffers (kv_cache.rs:1982-2012): one byte per
 * element, [n_kv_heads][max_seq][head_dim], plus one f32 per (head, position).  The reference's
 * byte indexes a 256-entry codebook that lives in the external mlx-native crate; here it is a
 * signed 8-bit integer and the f32 is the scale amax / 127 (a stand-in with the same footprint). */
typedef struct hf2q_kv_cache {
    void* k_codes;           /* int8 [n_kv_heads][max_seq][head_dim] */
    void* k_scale;           /* f32  [n_kv_heads][max_seq] */
    void* v_codes;
    void* v_scale;
    uint32_t n_kv_heads, head_dim, max_seq;
} hf2q_kv_cache;
HF2Q_API int32_t hf2q_cuda_kv_cache_bytes(uint32_t n_kv_heads, uint32_t head_dim, uint32_t max_seq,
                                          uint64_t* codes_bytes, uint64_t* scale_bytes);
/* embed_tokens: out[t,:] = dequant(W[ids[t],:]), W any of the block formats, [n_rows][k]. */
HF2Q_API int32_t hf2q_cuda_get_rows(hf2q_ctx* ctx, void* stream, const void* w, uint32_t ggml_type,
                                    uint32_t n_rows, uint32_t k, const uint32_t* ids, uint32_t m, float* out);
/* x[t,:] += delta[t,:] (delta may be NULL), then out[t,:] = x[t,:] / sqrt(mean(x^2) + eps) * weight. */
HF2Q_API int32_t hf2q_cuda_rms_norm(hf2q_ctx* ctx, void* stream, float* x, const float* delta,
                                    const float* weight, float eps, void* out, uint32_t out_dtype,
                                    uint32_t m, uint32_t h);
/* qkv: the fused QKV product, f32 [m][(n_q_heads + 2 n_kv_heads) * head_dim].  Token t is at
 * position *pos + t (pos: device memory, so a captured decode step can be replayed).  Query heads
 * are rotated in place and scaled by 1/sqrt(head_dim); key heads are rotated; key and value heads
 * are quantized and stored at their positions of the cache. */
HF2Q_API int32_t hf2q_cuda_rope_kv_append(hf2q_ctx* ctx, void* stream, float* qkv, uint32_t m,
                                          uint32_t n_q_heads, float theta, const uint32_t* pos,
                                          const hf2q_kv_cache* kv);
/* One query token at position *pos against cache positions 0..*pos: out[n_q_heads][head_dim].
 * q: the rotated, scaled query heads (the first n_q_heads * head_dim floats of a qkv row). */
HF2Q_API int32_t hf2q_cuda_attn_decode_scratch_bytes(hf2q_ctx* ctx, uint32_t n_q_heads,
                                                     uint32_t n_kv_heads, uint64_t* out);
HF2Q_API int32_t hf2q_cuda_attn_decode(hf2q_ctx* ctx, void* stream, const float* q, uint32_t n_q_heads,
                                       const hf2q_kv_cache* kv, const uint32_t* pos, void* out,
                                       uint32_t out_dtype, void* scratch, uint64_t scratch_bytes);
/* RMSNorm fused in front of a product (decode: 1..4 f32 activation rows, k <= 4096): the kernel
 * normalises x -- x / sqrt(mean(x^2) + eps) * norm_weight, rms_norm_rows of forward_cpu.rs:36-48 --
 * while it converts the activations for its tensor-core operand, so the norm costs no launch and
 * no round trip through memory.  x itself is not modified.  hf2q_cuda_norm_supported tells whether
 * a (m, k, type) fits; otherwise call hf2q_cuda_rms_norm and the plain product. */
HF2Q_API int32_t hf2q_cuda_norm_supported(hf2q_ctx* ctx, uint32_t m, uint32_t k, uint32_t ggml_type);
HF2Q_API int32_t hf2q_cuda_norm_qmatmul_segments(hf2q_ctx* ctx, void* stream, const float* x,
                                                 const float* norm_weight, float eps,
                                                 const hf2q_row_segment* segs, uint32_t n_segs, float* y,
                                                 uint32_t m, uint32_t k);
HF2Q_API int32_t hf2q_cuda_norm_qmatmul_swiglu(hf2q_ctx* ctx, void* stream, const float* x,
                                               const float* norm_weight, float eps, const void* w_gate,
                                               const void* w_up, float* y, uint32_t m, uint32_t n,
                                               uint32_t k, uint32_t ggml_type);
/* The decode step's attention as ONE launch: hf2q_cuda_rope_kv_append (m = 1) and
 * hf2q_cuda_attn_decode together.  qkv is one fused QKV row and is not modified; the new position's
 * K and V go to the cache.  The first 256 bytes of scratch are completion counters: zero them once
 * when the buffer is allocated (every call leaves them zero). */
HF2Q_API int32_t hf2q_cuda_attn_decode_fused(hf2q_ctx* ctx, void* stream, const float* qkv, uint32_t n_q_heads,
                                             float theta, const hf2q_kv_cache* kv, const uint32_t* pos,
                                             void* out, uint32_t out_dtype, void* scratch, uint64_t scratch_bytes);
/* m query tokens at positions pos0 .. pos0 + m - 1 (already appended), causal:
 * out[m][n_q_heads * head_dim].  qkv as for hf2q_cuda_rope_kv_append (after it). */
HF2Q_API int32_t hf2q_cuda_attn_prefill(hf2q_ctx* ctx, void* stream, const float* qkv, uint32_t m,
                                        uint32_t n_q_heads, const hf2q_kv_cache* kv, uint32_t pos0,
                                        void* out, uint32_t out_dtype);
/* Greedy sampling: *out_id = index of the largest logit (lowest index on ties); if pos != NULL,
 * *pos += 1 afterwards, which hands a captured decode step over to its next replay. */
HF2Q_API int32_t hf2q_cuda_argmax(hf2q_ctx* ctx, void* stream, const float* logits, uint32_t n,
                                  uint32_t* out_id, uint32_t* pos);
/* residual_add: x[i] += delta[i]. */
HF2Q_API int32_t hf2q_cuda_add(hf2q_ctx* ctx, void* stream, float* x, const float* delta, uint64_t n);

/* ---- introspection ------------------------------------------------------------------------ */

/* Number of kernels this library has launched through `ctx` since creation (the reference keeps
 * dispatch counters for the same purpose, forward_mlx.rs:3346). */
HF2Q_API uint64_t hf2q_cuda_launch_count(const hf2q_ctx* ctx);
HF2Q_API int32_t hf2q_cuda_sm_count(const hf2q_ctx* ctx);
HF2Q_API const char* hf2q_cuda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HF2Q_CUDA_H */
