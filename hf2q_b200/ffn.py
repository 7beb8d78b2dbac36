"""FFN builders on quantized weights -- host-side mirror of hf2q's
``build_dense_ffn_layer_gpu_q_into`` (src/inference/models/qwen35/gpu_ffn.rs:1086-1351) and
``build_moe_ffn_layer_gpu_q_into`` (gpu_ffn.rs:2313-2802).

Each builder is ONE call of the C ABI (``hf2q_cuda_dense_ffn`` / ``hf2q_cuda_moe_ffn``, which compose the
quantized products, the router and the element-wise glue on torch's current stream); nothing here
computes on the host.  The math is that of the reference's scalar
specs ``dense_swiglu_cpu_ref`` (ffn.rs:91-112) and ``moe_ffn_cpu_ref`` (ffn.rs:179-336).
"""
from __future__ import annotations

import ctypes as C
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


class _MoeFfnWeights(C.Structure):            # hf2q_moe_ffn_weights in include/hf2q_cuda.h
    _fields_ = [("router", C.c_void_p), ("expert_gate", C.c_void_p), ("expert_up", C.c_void_p), ("expert_down", C.c_void_p),
                ("stride_gate_up", C.c_uint64), ("stride_down", C.c_uint64), ("type_gate_up", C.c_uint32), ("type_down", C.c_uint32),
                ("n_experts", C.c_uint32), ("top_k", C.c_uint32), ("ffn", C.c_uint32), ("shared_ffn", C.c_uint32),
                ("shared_gate", C.c_void_p), ("shared_up", C.c_void_p), ("shared_down", C.c_void_p),
                ("shared_type_gate", C.c_uint32), ("shared_type_up", C.c_uint32), ("shared_type_down", C.c_uint32), ("reserved", C.c_uint32),
                ("shared_gate_logit", C.c_void_p)]


def _pooled_scratch(ctx, nbytes: int, device) -> torch.Tensor:
    """The builders' scratch, grown on demand and kept on the context (decode_pool.rs:181-228 pools it per thread)."""
    sc = getattr(ctx, "_ffn_scratch", None)
    if sc is None or sc.numel() < nbytes:
        sc = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        ctx._ffn_scratch = sc
    return sc


def build_dense_ffn_layer_gpu_q(ctx: ops.GpuContext, x: torch.Tensor, w: DenseFfnWeightsGpuQ,
                                residual: torch.Tensor | None = None, fused: bool = True) -> torch.Tensor:
    """y = down @ (silu(gate @ x) * (up @ x)) (+ residual); x [m, hidden] f32/bf16, y f32 [m, hidden].

    One call of ``hf2q_cuda_dense_ffn``: with ``fused`` (default) and a shape the fused kernels take, two
    products -- gate/up with the SwiGLU in the epilogue, down with the residual add in the epilogue (mat-vec
    kernels up to 8 rows, the tensor-core GEMM beyond); otherwise the reference's sequence gate, up,
    silu_mul, down, add (gpu_ffn.rs:896-960)."""
    m = x.shape[0]
    inter, hidden = w.gate_q.rows, w.gate_q.cols
    x = x.contiguous()
    y = torch.empty((m, hidden), dtype=torch.float32, device=x.device)
    r = residual.contiguous().float() if residual is not None else None
    need = C.c_uint64()
    ctx._check(ctx._lib.hf2q_cuda_dense_ffn_scratch_bytes(m, hidden, inter, C.byref(need)))
    sc = _pooled_scratch(ctx, need.value, x.device)
    ctx._check(ctx._lib.hf2q_cuda_dense_ffn(ctx._h, ctx._stream(), x.data_ptr(), ops._act(x, "x"), w.gate_q.ptr, w.gate_q.ggml_type,
                                            w.up_q.ptr, w.up_q.ggml_type, w.down_q.ptr, w.down_q.ggml_type,
                                            r.data_ptr() if r is not None else None, y.data_ptr(), m, hidden, inter,
                                            sc.data_ptr(), sc.numel(), 0 if fused else 1))
    return y


def build_moe_ffn_layer_gpu_q(ctx: ops.GpuContext, x: torch.Tensor, w: MoeFfnWeightsGpuQ,
                              residual: torch.Tensor | None = None, fused: bool = True, atomic_combine: bool = False) -> torch.Tensor:
    """Router -> softmax/top-k/renorm -> expert gate, up (mul_mat_id) -> SwiGLU -> expert down
    (mul_mat_id, one activation row per routed slot) -> weighted sum over the slots, plus the
    sigmoid-gated shared expert and the residual.  x [T, hidden]; returns f32 [T, hidden].
    One call of ``hf2q_cuda_moe_ffn`` (build_moe_ffn_layer_gpu_q_into, gpu_ffn.rs:2313-2802).  ``atomic_combine``:
    the weighted sum over the slots happens inside the down product (floating-point atomics: last bits may vary)."""
    T, hidden = x.shape
    x = x.contiguous()
    if w.shared_gate_logit is not None and x.dtype != torch.float32:
        x = x.float()                                   # the shared expert's gate logit is an f32 row dot
    E, k, inter = w.num_experts, w.num_experts_per_tok, w.moe_intermediate_size
    cw = _MoeFfnWeights()
    cw.router, cw.expert_gate, cw.expert_up, cw.expert_down = (w.router.data_ptr(), w.expert_gate.data_ptr(), w.expert_up.data_ptr(),
                                                               w.expert_down.data_ptr())
    cw.stride_gate_up = ops.expert_stride(w.ggml_type_gate_up, inter, hidden)
    cw.stride_down = ops.expert_stride(w.ggml_type_down, hidden, inter)
    cw.type_gate_up, cw.type_down, cw.n_experts, cw.top_k, cw.ffn = int(w.ggml_type_gate_up), int(w.ggml_type_down), E, k, inter
    if w.shared is not None:
        s = w.shared
        cw.shared_gate, cw.shared_up, cw.shared_down = s.gate_q.ptr, s.up_q.ptr, s.down_q.ptr
        cw.shared_type_gate, cw.shared_type_up, cw.shared_type_down = s.gate_q.ggml_type, s.up_q.ggml_type, s.down_q.ggml_type
        cw.shared_ffn = s.gate_q.rows
        if w.shared_gate_logit is not None:
            cw.shared_gate_logit = w.shared_gate_logit.data_ptr()
    need = C.c_uint64()
    ctx._check(ctx._lib.hf2q_cuda_moe_ffn_scratch_bytes(C.byref(cw), T, hidden, C.byref(need)))
    sc = _pooled_scratch(ctx, need.value, x.device)
    out = torch.empty((T, hidden), dtype=torch.float32, device=x.device)
    r = residual.contiguous().float() if residual is not None else None
    ctx._check(ctx._lib.hf2q_cuda_moe_ffn(ctx._h, ctx._stream(), x.data_ptr(), ops._act(x, "x"), C.byref(cw),
                                          r.data_ptr() if r is not None else None, out.data_ptr(), T, hidden, sc.data_ptr(), sc.numel(),
                                          (0 if fused else 1) | (2 if atomic_combine else 0)))
    return out
