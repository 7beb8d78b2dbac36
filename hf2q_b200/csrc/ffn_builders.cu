// The two FFN builders of hf2q's qwen35 models as C entries: build_dense_ffn_layer_gpu_q_into
// (src/inference/models/qwen35/gpu_ffn.rs:1086-1351) and build_moe_ffn_layer_gpu_q_into
// (gpu_ffn.rs:2313-2802; six-phase graph at :2347-2359), composed from this library's own entries on the
// caller's stream.  Host code only: every launch goes through the entries of include/hf2q_cuda.h, so shapes
// that a fused kernel does not take fall back to the reference's own sequence of ops inside the same call.
// All intermediates live in ONE caller-supplied scratch buffer (the reference pools them per thread,
// decode_pool.rs:181-228); nothing is allocated on the op path.
#include <cstdint>

#include "../../include/hf2q_cuda.h"

namespace hf2q {
int32_t ctx_fail(hf2q_ctx* ctx, int32_t code, const char* msg);      // api.cu: sets the context's last-error text, returns code
}
using hf2q::ctx_fail;

namespace {

constexpr uint64_t align256(uint64_t v) { return (v + 255) & ~static_cast<uint64_t>(255); }

struct DenseLayout {
    uint64_t act, up, tmp, ws, total;
};

DenseLayout dense_layout(uint32_t m, uint32_t hidden, uint32_t ffn) {
    DenseLayout L{};
    uint64_t o = 0;
    L.act = o; o += align256(static_cast<uint64_t>(m) * ffn * 4);
    L.up = o;  o += align256(static_cast<uint64_t>(m) * ffn * 4);
    L.tmp = o; o += align256(static_cast<uint64_t>(m) * hidden * 4);      // the down product when y doubles as the residual (unfused form)
    L.ws = o;
    if (m > 8) {     // f16 copy of the activations of the larger product
        const uint64_t kmax = hidden > ffn ? hidden : ffn;
        o += align256(static_cast<uint64_t>(m) * kmax * 2);
    }
    L.total = o;
    return L;
}

int32_t dense_ffn(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w_gate, uint32_t type_gate, const void* w_up,
                  uint32_t type_up, const void* w_down, uint32_t type_down, const float* residual, float* y, uint32_t m, uint32_t hidden,
                  uint32_t ffn, uint8_t* sb, uint32_t flags) {
    const DenseLayout L = dense_layout(m, hidden, ffn);
    float* act = reinterpret_cast<float*>(sb + L.act);
    float* up = reinterpret_cast<float*>(sb + L.up);
    void* ws = m > 8 ? sb + L.ws : nullptr;
    const uint64_t ws_bytes = L.total - L.ws;
    const bool fuse = !(flags & HF2Q_FFN_NO_FUSION);
    int32_t rc;
    if (fuse && type_gate == type_up && hf2q_cuda_qmatmul_swiglu_ws_supported(ctx, m, ffn, hidden, type_gate, x_dtype)) {
        rc = hf2q_cuda_qmatmul_swiglu_ws(ctx, stream, x, x_dtype, w_gate, w_up, act, m, ffn, hidden, type_gate, ws, ws_bytes);
        if (rc) return rc;
    } else {
        rc = hf2q_cuda_qmatmul(ctx, stream, x, x_dtype, w_gate, act, m, ffn, hidden, type_gate, ws, ws_bytes);
        if (!rc) rc = hf2q_cuda_qmatmul(ctx, stream, x, x_dtype, w_up, up, m, ffn, hidden, type_up, ws, ws_bytes);
        if (!rc) rc = hf2q_cuda_silu_mul(ctx, stream, act, up, act, static_cast<uint64_t>(m) * ffn);
        if (rc) return rc;
    }
    if (residual && fuse && hf2q_cuda_qmatmul_add_ws_supported(ctx, m, hidden, ffn, type_down, HF2Q_DT_F32))
        return hf2q_cuda_qmatmul_add_ws(ctx, stream, act, HF2Q_DT_F32, w_down, residual, y, m, hidden, ffn, type_down, ws, ws_bytes);
    if (residual == y) {                       // in place on the residual stream: the product must not overwrite it first
        float* tmp = reinterpret_cast<float*>(sb + L.tmp);
        rc = hf2q_cuda_qmatmul(ctx, stream, act, HF2Q_DT_F32, w_down, tmp, m, hidden, ffn, type_down, ws, ws_bytes);
        if (!rc) rc = hf2q_cuda_add(ctx, stream, y, tmp, static_cast<uint64_t>(m) * hidden);
        return rc;
    }
    rc = hf2q_cuda_qmatmul(ctx, stream, act, HF2Q_DT_F32, w_down, y, m, hidden, ffn, type_down, ws, ws_bytes);
    if (!rc && residual) rc = hf2q_cuda_add(ctx, stream, y, residual, static_cast<uint64_t>(m) * hidden);
    return rc;
}

struct MoeLayout {
    uint64_t logits, ids, wts, d, g, u, shared_y, gate_logit, inner, dense, total;
};

MoeLayout moe_layout(const hf2q_moe_ffn_weights* w, uint32_t T, uint32_t hidden) {
    MoeLayout L{};
    const uint64_t rows = static_cast<uint64_t>(T) * w->top_k;
    uint64_t o = 0;
    L.logits = o;     o += align256(static_cast<uint64_t>(T) * w->n_experts * 4);
    L.ids = o;        o += align256(rows * 4);
    L.wts = o;        o += align256(rows * 4);
    L.d = o;          o += align256(rows * hidden * 4);
    L.g = o;          o += align256(rows * w->ffn * 4);
    L.u = o;          o += align256(rows * w->ffn * 4);
    L.shared_y = o;   o += w->shared_gate ? align256(static_cast<uint64_t>(T) * hidden * 4) : 0;
    L.gate_logit = o; o += w->shared_gate_logit ? align256(static_cast<uint64_t>(T) * 4) : 0;
    L.inner = o;
    uint64_t a = 0, b = 0, c = 0;
    const uint32_t kmax = hidden > w->ffn ? hidden : w->ffn;
    hf2q_cuda_qmatmul_id_scratch_bytes(w->n_experts, static_cast<uint32_t>(rows), kmax, HF2Q_DT_F32, &a);
    hf2q_cuda_moe_experts_scratch_bytes(w->n_experts, static_cast<uint32_t>(rows), hidden, w->ffn, &b);
    c = a > b ? a : b;
    o += align256(c);
    L.dense = o;
    if (w->shared_gate) o += dense_layout(T, hidden, w->shared_ffn).total;
    L.total = o;
    return L;
}

}  // namespace

HF2Q_API int32_t hf2q_cuda_dense_ffn_scratch_bytes(uint32_t m, uint32_t hidden, uint32_t ffn, uint64_t* out) {
    if (!out) return HF2Q_ERR_INVALID_ARGUMENT;
    *out = dense_layout(m, hidden, ffn).total;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_dense_ffn(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w_gate, uint32_t type_gate,
                                     const void* w_up, uint32_t type_up, const void* w_down, uint32_t type_down, const float* residual,
                                     float* y, uint32_t m, uint32_t hidden, uint32_t ffn, void* scratch, uint64_t scratch_bytes,
                                     uint32_t flags) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !w_gate || !w_up || !w_down || !y) return ctx_fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "dense_ffn: null pointer");
    if (m == 0) return HF2Q_OK;
    if (!scratch || reinterpret_cast<uintptr_t>(scratch) % 256 || scratch_bytes < dense_layout(m, hidden, ffn).total)
        return ctx_fail(ctx, HF2Q_ERR_WORKSPACE, "dense_ffn: needs a 256-byte aligned scratch of hf2q_cuda_dense_ffn_scratch_bytes()");
    return dense_ffn(ctx, stream, x, x_dtype, w_gate, type_gate, w_up, type_up, w_down, type_down, residual, y, m, hidden, ffn,
                     static_cast<uint8_t*>(scratch), flags);
}

HF2Q_API int32_t hf2q_cuda_moe_ffn_scratch_bytes(const hf2q_moe_ffn_weights* w, uint32_t n_tokens, uint32_t hidden, uint64_t* out) {
    if (!w || !out || w->top_k == 0 || w->n_experts == 0) return HF2Q_ERR_INVALID_ARGUMENT;
    *out = moe_layout(w, n_tokens, hidden).total;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_moe_ffn(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const hf2q_moe_ffn_weights* w,
                                   const float* residual, float* y, uint32_t n_tokens, uint32_t hidden, void* scratch,
                                   uint64_t scratch_bytes, uint32_t flags) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !w || !y || !w->router || !w->expert_gate || !w->expert_up || !w->expert_down)
        return ctx_fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_ffn: null pointer");
    if (w->top_k == 0 || w->n_experts == 0 || w->top_k > w->n_experts)
        return ctx_fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_ffn: top_k must be in 1..n_experts");
    if (w->shared_gate && (!w->shared_up || !w->shared_down))
        return ctx_fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_ffn: the shared expert needs gate, up and down");
    if (w->shared_gate_logit && (!w->shared_gate || x_dtype != HF2Q_DT_F32))      // the gate logit is an f32 row dot
        return ctx_fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_ffn: shared_gate_logit needs the shared expert and f32 activations");
    if (n_tokens == 0) return HF2Q_OK;
    const MoeLayout L = moe_layout(w, n_tokens, hidden);
    if (!scratch || reinterpret_cast<uintptr_t>(scratch) % 256 || scratch_bytes < L.total)
        return ctx_fail(ctx, HF2Q_ERR_WORKSPACE, "moe_ffn: needs a 256-byte aligned scratch of hf2q_cuda_moe_ffn_scratch_bytes()");
    uint8_t* sb = static_cast<uint8_t*>(scratch);
    const uint32_t T = n_tokens, E = w->n_experts, K = w->top_k, I = w->ffn, rows = T * K;
    float* logits = reinterpret_cast<float*>(sb + L.logits);
    uint32_t* ids = reinterpret_cast<uint32_t*>(sb + L.ids);
    float* wts = reinterpret_cast<float*>(sb + L.wts);
    float* d = reinterpret_cast<float*>(sb + L.d);
    float* g = reinterpret_cast<float*>(sb + L.g);
    float* u = reinterpret_cast<float*>(sb + L.u);
    void* inner = sb + L.inner;
    const uint64_t inner_bytes = L.dense - L.inner;
    const bool fuse = !(flags & HF2Q_FFN_NO_FUSION);
    // phase A: router logits, softmax, top-k, renormalisation
    int32_t rc = hf2q_cuda_router_logits(ctx, stream, x, x_dtype, w->router, logits, T, E, hidden);
    if (!rc) rc = hf2q_cuda_moe_softmax_topk(ctx, stream, logits, ids, wts, T, E, K);
    if (rc) return rc;
    // phases B-F in the opt-in form: shared expert + residual first, the routed experts add their weighted rows on top
    if (fuse && (flags & HF2Q_FFN_ATOMIC_COMBINE) && hf2q_cuda_moe_experts_supported(ctx, T, K, hidden, I, E, w->type_gate_up, w->type_down)) {
        float* shared_y = nullptr;
        float* gate_logit = nullptr;
        if (w->shared_gate) {
            shared_y = reinterpret_cast<float*>(sb + L.shared_y);
            rc = dense_ffn(ctx, stream, x, x_dtype, w->shared_gate, w->shared_type_gate, w->shared_up, w->shared_type_up, w->shared_down,
                           w->shared_type_down, nullptr, shared_y, T, hidden, w->shared_ffn, sb + L.dense, flags);
            if (!rc && w->shared_gate_logit) {
                gate_logit = reinterpret_cast<float*>(sb + L.gate_logit);
                rc = hf2q_cuda_rowdot(ctx, stream, static_cast<const float*>(x), w->shared_gate_logit, gate_logit, T, hidden);
            }
            if (rc) return rc;
        }
        rc = hf2q_cuda_moe_combine(ctx, stream, nullptr, nullptr, shared_y, gate_logit, residual, y, T, 0, hidden);
        if (rc) return rc;
        return hf2q_cuda_moe_experts_reduce(ctx, stream, x, x_dtype, w->expert_gate, w->expert_up, w->expert_down, ids, wts, y, T, K, hidden, I,
                                            E, w->stride_gate_up, w->type_gate_up, w->stride_down, w->type_down, inner, inner_bytes);
    }
    // phases B-E: the routed experts
    if (fuse && hf2q_cuda_moe_experts_supported(ctx, T, K, hidden, I, E, w->type_gate_up, w->type_down)) {
        rc = hf2q_cuda_moe_experts(ctx, stream, x, x_dtype, w->expert_gate, w->expert_up, w->expert_down, ids, d, T, K, hidden, I, E,
                                   w->stride_gate_up, w->type_gate_up, w->stride_down, w->type_down, inner, inner_bytes);
    } else {
        if (fuse && hf2q_cuda_qmatmul_id_swiglu_supported(ctx, T, K, I, hidden, w->type_gate_up, x_dtype)) {
            rc = hf2q_cuda_qmatmul_id_swiglu(ctx, stream, x, x_dtype, w->expert_gate, w->expert_up, ids, g, T, K, I, hidden, E, w->stride_gate_up,
                                             w->type_gate_up);
        } else {
            rc = hf2q_cuda_qmatmul_id_pair(ctx, stream, x, x_dtype, w->expert_gate, w->expert_up, ids, g, u, T, K, I, hidden, E,
                                           w->stride_gate_up, w->type_gate_up, inner, inner_bytes);
            if (!rc) rc = hf2q_cuda_silu_mul(ctx, stream, g, u, g, static_cast<uint64_t>(rows) * I);
        }
        if (!rc)
            rc = hf2q_cuda_qmatmul_id(ctx, stream, g, HF2Q_DT_F32, w->expert_down, ids, d, rows, 1, hidden, I, E, w->stride_down, w->type_down,
                                      inner, inner_bytes);
    }
    if (rc) return rc;
    // the shared expert and its sigmoid gate
    float* shared_y = nullptr;
    float* gate_logit = nullptr;
    if (w->shared_gate) {
        shared_y = reinterpret_cast<float*>(sb + L.shared_y);
        rc = dense_ffn(ctx, stream, x, x_dtype, w->shared_gate, w->shared_type_gate, w->shared_up, w->shared_type_up, w->shared_down,
                       w->shared_type_down, nullptr, shared_y, T, hidden, w->shared_ffn, sb + L.dense, flags);
        if (rc) return rc;
        if (w->shared_gate_logit) {
            gate_logit = reinterpret_cast<float*>(sb + L.gate_logit);
            rc = hf2q_cuda_rowdot(ctx, stream, static_cast<const float*>(x), w->shared_gate_logit, gate_logit, T, hidden);
            if (rc) return rc;
        }
    }
    // phase F: weighted sum over the slots + gated shared expert + residual
    return hf2q_cuda_moe_combine(ctx, stream, d, wts, shared_y, gate_logit, residual, y, T, K, hidden);
}
