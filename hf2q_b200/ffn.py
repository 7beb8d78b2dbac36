"""FFN builders on quantized weights -- host-side mirror of hf2q's
``build_dense_ffn_layer_gpu_q_into`` (src/inference/models/qwen35/gpu_ffn.rs:1086-1351) and
``build_moe_ffn_layer_gpu_q_into`` (gpu_ffn.rs:2313-2802).

They only compose calls of the C ABI (quantized products, router, element-wise glue) on torch's
current stream; nothing here computes on the host.  The math is that of the reference's scalar
specs ``dense_swiglu_cpu_ref`` (ffn.rs:91-112) and ``moe_ffn_cpu_ref`` (ffn.rs:179-336).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops


@dataclass
class DenseFfnWeightsGpuQ:
    """gate/up [intermediate, hidden], down [hidden, intermediate] as raw quantized blocks
    (DenseFfnWeightsGpuQ, gpu_ffn.rs:260-275)."""
    gate_q: ops.QuantWeight
    up_q: ops.QuantWeight
    down_q: ops.QuantWeight


@dataclass
class MoeFfnWeightsGpuQ:
    """Stacked expert weights + routing inputs (MoeFfnWeightsGpuQ, gpu_ffn.rs:362-398)."""
    router: torch.Tensor                 # f32 [num_experts, hidden]
    expert_gate: torch.Tensor            # uint8, E stacked [moe_intermediate, hidden] matrices
    expert_up: torch.Tensor
    expert_down: torch.Tensor            # uint8, E stacked [hidden, moe_intermediate] matrices
    ggml_type_gate_up: int
    ggml_type_down: int
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared: DenseFfnWeightsGpuQ | None = None
    shared_gate_logit: torch.Tensor | None = None      # f32 [hidden]


def _silu_mul(ctx, gate, up):
    out = torch.empty_like(gate)
    ctx._check(ctx._lib.hf2q_cuda_silu_mul(ctx._h, ctx._stream(), gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel()))
    return out


def build_dense_ffn_layer_gpu_q(ctx: ops.GpuContext, x: torch.Tensor, w: DenseFfnWeightsGpuQ,
                                residual: torch.Tensor | None = None, fused: bool = True) -> torch.Tensor:
    """y = down @ (silu(gate @ x) * (up @ x)) (+ residual); x [m, hidden] f32/bf16, y f32 [m, hidden].

    With ``fused`` (default) and a shape the fused kernels take, this is two products: gate/up with
    the SwiGLU in the epilogue, down with the residual add in the epilogue (mat-vec kernels up to 8
    rows, the tensor-core GEMM beyond).  Otherwise the
    reference's sequence: gate, up, silu_mul, down, add (gpu_ffn.rs:896-960)."""
    m = x.shape[0]
    inter, hidden = w.gate_q.rows, w.gate_q.cols
    if fused and ops.quantized_matmul_swiglu_supported(ctx, m, w.gate_q, x.dtype):
        c = torch.empty((m, inter), dtype=torch.float32, device=x.device)
        ops.quantized_matmul_swiglu(ctx, x, w.gate_q, w.up_q, c, m)
    else:
        a = torch.empty((m, inter), dtype=torch.float32, device=x.device)
        b = torch.empty_like(a)
        ops.quantized_matmul_ggml(ctx, x, w.gate_q, a, w.gate_q.matmul_params(m))
        ops.quantized_matmul_ggml(ctx, x, w.up_q, b, w.up_q.matmul_params(m))
        c = _silu_mul(ctx, a, b)
    y = torch.empty((m, hidden), dtype=torch.float32, device=x.device)
    if residual is not None and fused and ops.quantized_matmul_add_supported(ctx, w.down_q, c.dtype, m):
        ops.quantized_matmul_add(ctx, c, w.down_q, residual.contiguous().float(), y, m)
        return y
    ops.quantized_matmul_ggml(ctx, c, w.down_q, y, w.down_q.matmul_params(m))
    if residual is not None:
        r = residual.contiguous().float()
        ctx._check(ctx._lib.hf2q_cuda_add(ctx._h, ctx._stream(), y.data_ptr(), r.data_ptr(), y.numel()))
    return y


def build_moe_ffn_layer_gpu_q(ctx: ops.GpuContext, x: torch.Tensor, w: MoeFfnWeightsGpuQ,
                              residual: torch.Tensor | None = None, fused: bool = True) -> torch.Tensor:
    """Router -> softmax/top-k/renorm -> expert gate, up (mul_mat_id) -> SwiGLU -> expert down
    (mul_mat_id, one activation row per routed slot) -> weighted sum over the slots, plus the
    sigmoid-gated shared expert and the residual.  x f32 [T, hidden]; returns f32 [T, hidden]."""
    T, hidden = x.shape
    E, k, inter = w.num_experts, w.num_experts_per_tok, w.moe_intermediate_size
    x = x.contiguous()
    # the router is a small dense f32 matrix in the reference as well (gpu_ffn.rs:2347-2359 phase 1)
    logits = torch.empty((T, E), dtype=torch.float32, device=x.device)
    ctx._check(ctx._lib.hf2q_cuda_router_logits(ctx._h, ctx._stream(), x.data_ptr(), ops._act(x, "x"), w.router.data_ptr(),
                                                logits.data_ptr(), T, E, hidden))
    ids, wts = ops.moe_softmax_topk(ctx, logits, k)
    rows = T * k
    sg = ops.expert_stride(w.ggml_type_gate_up, inter, hidden)
    sd = ops.expert_stride(w.ggml_type_down, hidden, inter)
    pg = ops.GgmlQuantizedMatmulIdParams(T, k, inter, hidden, E, sg, w.ggml_type_gate_up)
    d = torch.empty((rows, hidden), dtype=torch.float32, device=x.device)
    if fused and ops.moe_experts_supported(ctx, T, k, hidden, inter, E, w.ggml_type_gate_up, w.ggml_type_down):
        # many routed rows: sort + gather, gate/up pair with the SwiGLU in its epilogue, down -- four launches
        ops.moe_experts(ctx, x, w.expert_gate.data_ptr(), w.expert_up.data_ptr(), w.expert_down.data_ptr(), ids, d,
                        T, k, hidden, inter, E, w.ggml_type_gate_up, w.ggml_type_down, sg, sd)
        return _moe_finish(ctx, x, w, d, wts, residual, T, k, hidden)
    scratch = ops.IdMmScratch.alloc(ctx, E, rows, max(hidden, inter))
    if fused and ops.quantized_matmul_id_swiglu_supported(ctx, pg, x.dtype):
        # few routed rows: gate, up and the SwiGLU in one launch
        act = torch.empty((rows, inter), dtype=torch.float32, device=x.device)
        ops.quantized_matmul_id_swiglu_ggml(ctx, x, w.expert_gate.data_ptr(), w.expert_up.data_ptr(), ids, act, pg)
    else:
        g = torch.empty((rows, inter), dtype=torch.float32, device=x.device)
        u = torch.empty_like(g)
        ops.quantized_matmul_id_pair_ggml(ctx, x, w.expert_gate.data_ptr(), w.expert_up.data_ptr(), ids, g, u, scratch, pg)
        act = _silu_mul(ctx, g, u)
    pd = ops.GgmlQuantizedMatmulIdParams(rows, 1, hidden, inter, E, sd, w.ggml_type_down)
    ops.quantized_matmul_id_ggml(ctx, act, w.expert_down.data_ptr(), ids, d, scratch, pd)
    return _moe_finish(ctx, x, w, d, wts, residual, T, k, hidden)


def _moe_finish(ctx, x, w, d, wts, residual, T, k, hidden):
    """Shared expert, its sigmoid gate, the weighted sum over the slots and the residual (gpu_ffn.rs:2762-2802)."""
    shared_y = gate_logit = None
    if w.shared is not None:
        shared_y = build_dense_ffn_layer_gpu_q(ctx, x, w.shared)
        if w.shared_gate_logit is not None:
            gate_logit = torch.empty((T,), dtype=torch.float32, device=x.device)
            xf = x if x.dtype == torch.float32 else x.float()
            ctx._check(ctx._lib.hf2q_cuda_rowdot(ctx._h, ctx._stream(), xf.data_ptr(), w.shared_gate_logit.data_ptr(),
                                                 gate_logit.data_ptr(), T, hidden))
    out = torch.empty((T, hidden), dtype=torch.float32, device=x.device)
    ctx._check(ctx._lib.hf2q_cuda_moe_combine(
        ctx._h, ctx._stream(), d.data_ptr(), wts.data_ptr(),
        shared_y.data_ptr() if shared_y is not None else None,
        gate_logit.data_ptr() if gate_logit is not None else None,
        residual.data_ptr() if residual is not None else None,
        out.data_ptr(), T, k, hidden))
    return out
