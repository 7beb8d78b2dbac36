"""Host-side mirror of the op surface hf2q's inference models call on the quantized-matmul path.

Names, argument meaning and error behaviour follow the reference (paths relative to the hf2q
source tree):

* ``GgmlType``                       src/quantize/ggml_quants/ggml_type.rs:18-54
* ``GgmlQuantizedMatmulParams``      built at src/inference/models/qwen35/gpu_ffn.rs:1218-1229,
                                     src/serve/forward_mlx.rs:408-415
* ``GgmlQuantizedMatmulIdParams``    built at gpu_ffn.rs:2606-2618
* ``GpuContext``                     src/serve/gpu.rs:19-38
* ``QuantWeight``/``load_quant_weight``  MlxQWeight + load_gguf_qweight, forward_mlx.rs:364-402,
                                     9356-9386; load_tensor_with_residency, weight_loader.rs:147-159
* ``quantized_matmul_ggml``          call sites gpu_ffn.rs:1236-1306, gpu_full_attn.rs:848-855
* ``quantized_matmul_id_ggml``       quantized_matmul_id_ggml_pooled, gpu_ffn.rs:188-206
* ``IdMmScratch``                    decode_pool.rs:181-228
* ``moe_softmax_topk``               dispatch_moe_softmax_topk, gpu_ffn.rs:2551

Everything here forwards to ``libhf2q_cuda.so`` through its C ABI; there is no PyTorch or CPU
implementation behind these functions.  Ops are enqueued on torch's current CUDA stream and do
not synchronise, as the reference's ops append to a command encoder and return.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib


class GgmlType(enum.IntEnum):
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    IQ4_NL = 20
    MLX_AFFINE4_GS32 = 1000        # not a GGML id: mlx-affine 4-bit / group 32 in this library's 24-byte block


DT_F32, DT_F16, DT_BF16 = 0, 1, 2
_TORCH_DT = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16}
_DT_TORCH = {v: k for k, v in _TORCH_DT.items()}


class Hf2qError(RuntimeError):
    """A non-zero status from the C ABI (the reference's MlxError)."""

    def __init__(self, status: int, detail: str):
        self.status = status
        name = _lib.load().hf2q_cuda_strerror(status).decode()
        super().__init__(f"{name}: {detail}" if detail else name)


@dataclass(frozen=True)
class GgmlQuantizedMatmulParams:
    m: int
    n: int
    k: int
    ggml_type: int


@dataclass(frozen=True)
class GgmlQuantizedMatmulIdParams:
    n_tokens: int
    top_k: int
    n: int
    k: int
    n_experts: int
    expert_stride: int
    ggml_type: int


class GpuContext:
    """One device context (serve/gpu.rs:19-38).  Not shared between threads."""

    def __init__(self, device: int = 0):
        lib = _lib.load()
        h = C.c_void_p()
        rc = lib.hf2q_cuda_ctx_create(device, C.byref(h))
        if rc:
            raise Hf2qError(rc, f"ctx_create(device={device})")
        self._h = h
        self.device = device
        self._lib = lib

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.hf2q_cuda_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- helpers --------------------------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc:
            raise Hf2qError(rc, self._lib.hf2q_cuda_last_error(self._h).decode())

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def check_status(self) -> None:
        """Synchronises the current stream and raises if a kernel flagged a problem."""
        self._check(self._lib.hf2q_cuda_check_status(self._h, self._stream()))

    def set_wait_limit(self, clock_ticks: int) -> None:
        """Upper bound (GPU clock ticks) of the device-side waits for other GPUs; a context setting."""
        self._check(self._lib.hf2q_cuda_set_wait_limit(self._h, int(clock_ticks)))

    @property
    def launch_count(self) -> int:
        return int(self._lib.hf2q_cuda_launch_count(self._h))

    @property
    def sm_count(self) -> int:
        return int(self._lib.hf2q_cuda_sm_count(self._h))


def row_bytes(ggml_type: int, k: int) -> int:
    out = C.c_uint64()
    rc = _lib.load().hf2q_cuda_row_bytes(int(ggml_type), k, C.byref(out))
    if rc:
        raise Hf2qError(rc, f"row_bytes(type={int(ggml_type)}, k={k})")
    return out.value


def expert_stride(ggml_type: int, rows: int, cols: int) -> int:
    out = C.c_uint64()
    rc = _lib.load().hf2q_cuda_expert_stride(int(ggml_type), rows, cols, C.byref(out))
    if rc:
        raise Hf2qError(rc, f"expert_stride(type={int(ggml_type)}, rows={rows}, cols={cols})")
    return out.value


class QuantWeight:
    """Raw GGUF block bytes resident on the device + (ggml_dtype, rows, cols) -- MlxQWeight."""

    def __init__(self, ctx: GpuContext, ptr: int, nbytes: int, ggml_type: int, rows: int, cols: int,
                 owner=None, abi_owned: bool = False):
        self.ctx, self.ptr, self.nbytes = ctx, ptr, nbytes
        self.ggml_type, self.rows, self.cols = int(ggml_type), rows, cols
        self._owner, self._abi_owned = owner, abi_owned

    def matmul_params(self, m: int) -> GgmlQuantizedMatmulParams:
        return GgmlQuantizedMatmulParams(m=m, n=self.rows, k=self.cols, ggml_type=self.ggml_type)

    def row_slice(self, r0: int, r1: int) -> "QuantWeight":
        """Rows [r0, r1) as a view: rows are contiguous byte ranges, so a shard is a byte slice."""
        rb = row_bytes(self.ggml_type, self.cols)
        return QuantWeight(self.ctx, self.ptr + r0 * rb, (r1 - r0) * rb, self.ggml_type, r1 - r0,
                           self.cols, owner=self)

    def free(self) -> None:
        if self._abi_owned and self.ptr:
            self.ctx._lib.hf2q_cuda_free(self.ctx._h, C.c_void_p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            if self.ctx._h:
                self.free()
        except Exception:
            pass


def load_quant_weight(ctx: GpuContext, raw, ggml_type: int, rows: int, cols: int) -> QuantWeight:
    """Uploads raw block bytes unchanged.  ``raw`` is a uint8 numpy array (host) or a uint8 CUDA
    tensor already on the device (kept alive by the returned object)."""
    want = rows * row_bytes(ggml_type, cols)
    if isinstance(raw, torch.Tensor):
        if raw.dtype != torch.uint8 or not raw.is_cuda or not raw.is_contiguous():
            raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "device weight must be a contiguous uint8 CUDA tensor")
        if raw.numel() != want:
            raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, f"byte length {raw.numel()} != rows*row_bytes {want}")
        return QuantWeight(ctx, raw.data_ptr(), want, ggml_type, rows, cols, owner=raw)
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    if raw.size != want:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, f"byte length {raw.size} != rows*row_bytes {want}")
    dev = C.c_void_p()
    ctx._check(ctx._lib.hf2q_cuda_upload_blocks(ctx._h, raw.ctypes.data, raw.size, C.byref(dev)))
    return QuantWeight(ctx, dev.value, want, ggml_type, rows, cols, abi_owned=True)


def load_mlx_affine_weight(ctx: GpuContext, codes: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                           bits: int = 4, group_size: int = 32) -> QuantWeight:
    """MlxQWeight::from_mlx_affine_linear (src/serve/forward_mlx.rs:425-520): mlx-affine codes (u32/i32 [n, k/8], eight
    nibbles per word, low nibble first) with f32 scales and biases [n, k/32] on the device -> one weight of type
    MLX_AFFINE4_GS32 that every quantized product of this package takes (the interleave runs once, here)."""
    n, k = codes.shape[0], codes.shape[1] * 8
    for t, name in ((codes, "codes"), (scales, "scales"), (biases, "biases")):
        if not t.is_cuda or not t.is_contiguous():
            raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, f"{name} must be a contiguous CUDA tensor")
    if codes.dtype not in (torch.int32, torch.uint32) or scales.dtype != torch.float32 or biases.dtype != torch.float32:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "codes must be 32-bit integers, scales and biases float32")
    if tuple(scales.shape) != (n, k // 32) or tuple(biases.shape) != (n, k // 32):
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "scales / biases must be [n, k / 32]")
    out = torch.empty(n * (k // 32) * 24, dtype=torch.uint8, device=codes.device)
    ctx._check(ctx._lib.hf2q_cuda_affine_pack(ctx._h, ctx._stream(), codes.data_ptr(), scales.data_ptr(), biases.data_ptr(), n, k, bits,
                                              group_size, out.data_ptr()))
    return QuantWeight(ctx, out.data_ptr(), out.numel(), GgmlType.MLX_AFFINE4_GS32, n, k, owner=out)


def _act(t: torch.Tensor, name: str) -> int:
    if not t.is_cuda or not t.is_contiguous():
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, f"{name} must be a contiguous CUDA tensor")
    if t.dtype not in (torch.float32, torch.bfloat16):
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, f"{name} dtype {t.dtype} (want float32 or bfloat16)")
    return _TORCH_DT[t.dtype]


def quantized_matmul_workspace_bytes(params: GgmlQuantizedMatmulParams, x_dtype=torch.bfloat16) -> int:
    out = C.c_uint64()
    rc = _lib.load().hf2q_cuda_qmatmul_workspace_bytes(params.m, params.n, params.k, int(params.ggml_type),
                                                       _TORCH_DT[x_dtype], C.byref(out))
    if rc:
        raise Hf2qError(rc, "qmatmul_workspace_bytes")
    return out.value


def quantized_matmul_ggml(ctx: GpuContext, input: torch.Tensor, weight: QuantWeight, out: torch.Tensor,
                          params: GgmlQuantizedMatmulParams, workspace: torch.Tensor | None = None) -> None:
    """out[m,n] = input[m,k] . dequant(weight[n,k])^T   (f32 out, fp32 accumulation)."""
    xdt = _act(input, "input")
    if out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous():
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "out must be a contiguous float32 CUDA tensor")
    if input.numel() < params.m * params.k or out.numel() < params.m * params.n:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "input/out smaller than [m,k] / [m,n]")
    if weight.rows != params.n or weight.cols != params.k or weight.ggml_type != int(params.ggml_type):
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "params do not match the weight's (rows, cols, type)")
    if workspace is None:
        # the reference keeps such scratch in per-thread pools (decode_pool.rs:51-76); so does this mirror
        need = quantized_matmul_workspace_bytes(params, input.dtype)
        if need:
            ws = getattr(ctx, "_ws", None)
            if ws is None or ws.numel() < need:
                ws = torch.empty(need, dtype=torch.uint8, device=input.device)
                ctx._ws = ws
            workspace = ws
    ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
    ctx._check(ctx._lib.hf2q_cuda_qmatmul(ctx._h, ctx._stream(), input.data_ptr(), xdt, weight.ptr,
                                          out.data_ptr(), params.m, params.n, params.k,
                                          int(params.ggml_type), ws_ptr, ws_bytes))


def quantized_matmul_mm_tensor_perm021(ctx: GpuContext, input: torch.Tensor, weight: QuantWeight, out: torch.Tensor,
                                       m: int, head_dim: int) -> None:
    """out[m,n] = X . dequant(weight)^T where X[t, h*head_dim + f] = input[h, t, f]: the O projection reading the
    attention output heads-outermost (GgmlQuantizedMatmulPerm021Params {m,n,k,head_dim,ggml_type},
    forward_prefill_batched.rs:2218-2258)."""
    xdt = _act(input, "input")
    if out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous() or out.numel() < m * weight.rows:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "out must be a contiguous float32 CUDA tensor of [m, n]")
    if input.numel() < m * weight.cols:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "input smaller than [k / head_dim, m, head_dim]")
    need = (m * weight.cols * 2 + 255) // 256 * 256
    ws = getattr(ctx, "_ws", None)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=input.device)
        ctx._ws = ws
    ctx._check(ctx._lib.hf2q_cuda_qmatmul_perm021(ctx._h, ctx._stream(), input.data_ptr(), xdt, weight.ptr, out.data_ptr(), m,
                                                  weight.rows, weight.cols, head_dim, weight.ggml_type, ws.data_ptr(), ws.numel()))


class _RowSegment(C.Structure):                  # hf2q_row_segment in include/hf2q_cuda.h
    _fields_ = [("w", C.c_void_p), ("rows", C.c_uint32), ("ggml_type", C.c_uint32)]


def norm_supported(ctx: GpuContext, m: int, weight: "QuantWeight") -> bool:
    """Whether a product of m f32 rows against `weight` can take the RMSNorm fused into its launch."""
    return bool(ctx._lib.hf2q_cuda_norm_supported(ctx._h, m, weight.cols, weight.ggml_type))


def quantized_matmul_segments(ctx: GpuContext, input: torch.Tensor, weights, out: torch.Tensor, m: int,
                              workspace: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None,
                              norm_eps: float = 0.0) -> None:
    """out[m, n] = input[m, k] . W^T for a matrix W whose row ranges are separate QuantWeights of possibly
    different block formats (fused QKV of a Q4_K_M model: Q/K rows Q4_K, V rows Q6_K,
    standard_policy.rs:563-567); n = sum of the ranges' rows, ranges in row order."""
    xdt = _act(input, "input")
    k = weights[0].cols
    n = sum(w.rows for w in weights)
    if any(w.cols != k for w in weights):
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "all row ranges must share k")
    if out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous() or out.numel() < m * n or input.numel() < m * k:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "out must be a contiguous float32 CUDA tensor of [m, n]; input [m, k]")
    segs = (_RowSegment * len(weights))()
    for s, w in zip(segs, weights):
        s.w, s.rows, s.ggml_type = w.ptr, w.rows, w.ggml_type
    if norm_weight is not None:      # RMSNorm(input) fused into the launches (rms_norm_rows, forward_cpu.rs:36-48)
        ctx._check(ctx._lib.hf2q_cuda_norm_qmatmul_segments(ctx._h, ctx._stream(), input.data_ptr(), norm_weight.data_ptr(), norm_eps,
                                                           segs, len(weights), out.data_ptr(), m, k))
        return
    if workspace is None and m > 8:
        need = quantized_matmul_workspace_bytes(GgmlQuantizedMatmulParams(m, n, k, weights[0].ggml_type), input.dtype)
        ws = getattr(ctx, "_ws", None)
        if ws is None or ws.numel() < need:
            ws = torch.empty(need, dtype=torch.uint8, device=input.device)
            ctx._ws = ws
        workspace = ws
    ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
    ctx._check(ctx._lib.hf2q_cuda_qmatmul_segments(ctx._h, ctx._stream(), input.data_ptr(), xdt, segs, len(weights), out.data_ptr(),
                                                  m, k, ws_ptr, ws_bytes))


def quantized_matmul_swiglu_supported(ctx: GpuContext, m: int, weight: QuantWeight, x_dtype=torch.bfloat16) -> bool:
    """Whether gate and up products of shape `weight` with m activation rows fit the one fused launch."""
    xdt = DT_BF16 if x_dtype == torch.bfloat16 else DT_F32
    return bool(ctx._lib.hf2q_cuda_qmatmul_swiglu_ws_supported(ctx._h, m, weight.rows, weight.cols, weight.ggml_type, xdt))


def _pooled_workspace(ctx: GpuContext, m: int, weight: QuantWeight, x_dtype, device):
    """(pointer, bytes) of the context's pooled GEMM workspace grown for m rows of `weight` (decode_pool.rs:51-76)."""
    need = quantized_matmul_workspace_bytes(GgmlQuantizedMatmulParams(m, weight.rows, weight.cols, weight.ggml_type), x_dtype)
    if not need:
        return None, 0
    ws = getattr(ctx, "_ws", None)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        ctx._ws = ws
    return ws.data_ptr(), ws.numel()


def quantized_matmul_swiglu(ctx: GpuContext, input: torch.Tensor, gate: QuantWeight, up: QuantWeight, out: torch.Tensor, m: int,
                            norm_weight: torch.Tensor | None = None, norm_eps: float = 0.0) -> None:
    """out[m,n] = silu(input . gate^T) * (input . up^T) in one launch (gpu_ffn.rs:896-935: gate, up, dispatch_silu_mul);
    with ``norm_weight`` the input is RMS-normalised inside the same launch (few rows only).  More than 8 rows take
    the tensor-core form, which computes the two tiles side by side."""
    xdt = _act(input, "input")
    if out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous() or out.numel() < m * gate.rows:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "out must be a contiguous float32 CUDA tensor of [m, n]")
    if (gate.rows, gate.cols, gate.ggml_type) != (up.rows, up.cols, up.ggml_type) or input.numel() < m * gate.cols:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "gate and up must share (rows, cols, type); input must hold [m, k]")
    if norm_weight is not None:
        ctx._check(ctx._lib.hf2q_cuda_norm_qmatmul_swiglu(ctx._h, ctx._stream(), input.data_ptr(), norm_weight.data_ptr(), norm_eps, gate.ptr,
                                                          up.ptr, out.data_ptr(), m, gate.rows, gate.cols, gate.ggml_type))
        return
    ws_ptr, ws_bytes = _pooled_workspace(ctx, m, gate, input.dtype, input.device)
    ctx._check(ctx._lib.hf2q_cuda_qmatmul_swiglu_ws(ctx._h, ctx._stream(), input.data_ptr(), xdt, gate.ptr, up.ptr, out.data_ptr(),
                                                    m, gate.rows, gate.cols, gate.ggml_type, ws_ptr, ws_bytes))


def quantized_matmul_add_supported(ctx: GpuContext, weight: QuantWeight, x_dtype=torch.float32, m: int = 1) -> bool:
    xdt = DT_BF16 if x_dtype == torch.bfloat16 else DT_F32
    return bool(ctx._lib.hf2q_cuda_qmatmul_add_ws_supported(ctx._h, m, weight.rows, weight.cols, weight.ggml_type, xdt))


def quantized_matmul_add(ctx: GpuContext, input: torch.Tensor, weight: QuantWeight, residual: torch.Tensor, out: torch.Tensor, m: int) -> None:
    """out[m,n] = residual + input . weight^T (gpu_ffn.rs:947-960: the optional add_residual of the dense builder)."""
    xdt = _act(input, "input")
    for t, name in ((residual, "residual"), (out, "out")):
        if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous() or t.numel() < m * weight.rows:
            raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, f"{name} must be a contiguous float32 CUDA tensor of [m, n]")
    if input.numel() < m * weight.cols:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "input smaller than [m, k]")
    ws_ptr, ws_bytes = _pooled_workspace(ctx, m, weight, input.dtype, input.device)
    ctx._check(ctx._lib.hf2q_cuda_qmatmul_add_ws(ctx._h, ctx._stream(), input.data_ptr(), xdt, weight.ptr, residual.data_ptr(),
                                                 out.data_ptr(), m, weight.rows, weight.cols, weight.ggml_type, ws_ptr, ws_bytes))


def quantized_matmul_host(ctx: GpuContext, x_host: np.ndarray, weight: QuantWeight, y_host: np.ndarray,
                          m: int, x_dtype: int = DT_F32, wait: bool = True) -> None:
    """Host-buffer form: copies x in, runs, copies y out (hf2q_cuda_qmatmul_host).  With
    ``wait=False`` the call only queues the work (hf2q_cuda_qmatmul_host_async); y_host is valid
    after ``host_sync(ctx)`` and both arrays must stay alive until then."""
    fn = ctx._lib.hf2q_cuda_qmatmul_host if wait else ctx._lib.hf2q_cuda_qmatmul_host_async
    ctx._check(fn(ctx._h, x_host.ctypes.data, x_dtype, weight.ptr, y_host.ctypes.data, m, weight.rows, weight.cols,
                  weight.ggml_type))


class _HostProduct(C.Structure):                 # hf2q_host_product in include/hf2q_cuda.h
    _fields_ = [("x_host", C.c_void_p), ("w_dev", C.c_void_p), ("y_host", C.c_void_p), ("m", C.c_uint32), ("n", C.c_uint32),
                ("k", C.c_uint32), ("ggml_type", C.c_uint32), ("x_dtype", C.c_uint32), ("reserved", C.c_uint32)]


class HostBatch:
    """A list of independent host-buffer products (x_host, weight, y_host, m, x_dtype) for ``quantized_matmul_host_batch``;
    the arrays are kept alive by the object.  ``y_host`` may be None only for ``GatherGroup.host_batch`` (a rank that
    does not take the gathered result on the host)."""

    def __init__(self, items):
        self._keep = list(items)
        self.array = (_HostProduct * len(self._keep))()
        for slot, (x, w, y, m, xdt) in zip(self.array, self._keep):
            slot.x_host, slot.w_dev, slot.y_host = x.ctypes.data, w.ptr, (y.ctypes.data if y is not None else None)
            slot.m, slot.n, slot.k, slot.ggml_type, slot.x_dtype = m, w.rows, w.cols, w.ggml_type, xdt

    def __len__(self):
        return len(self._keep)


def quantized_matmul_host_batch(ctx: GpuContext, batch: HostBatch) -> None:
    """Queues every product of the batch with one call (hf2q_cuda_qmatmul_host_batch); results are valid after ``host_sync``."""
    ctx._check(ctx._lib.hf2q_cuda_qmatmul_host_batch(ctx._h, C.cast(batch.array, C.c_void_p), len(batch)))


def host_sync(ctx: GpuContext) -> None:
    """Waits for everything queued by ``quantized_matmul_host(..., wait=False)``."""
    ctx._check(ctx._lib.hf2q_cuda_host_sync(ctx._h))


class IdMmScratch:
    """Device scratch of the expert-routed product (decode_pool.rs:181-228)."""

    def __init__(self, ctx: GpuContext, n_experts: int, max_rows: int, k: int = 0, x_dtype=torch.bfloat16):
        out = C.c_uint64()
        ctx._check(ctx._lib.hf2q_cuda_qmatmul_id_scratch_bytes(n_experts, max_rows, k, _TORCH_DT[x_dtype], C.byref(out)))
        self.nbytes = out.value
        self.buf = torch.empty(max(self.nbytes, 16), dtype=torch.uint8, device=f"cuda:{ctx.device}")

    @classmethod
    def alloc(cls, ctx: GpuContext, n_experts: int, max_rows: int, k: int = 0, x_dtype=torch.bfloat16) -> "IdMmScratch":
        return cls(ctx, n_experts, max_rows, k, x_dtype)


def quantized_matmul_id_ggml(ctx: GpuContext, input: torch.Tensor, weight_ptr: int, ids: torch.Tensor,
                             out: torch.Tensor, scratch: IdMmScratch | None,
                             params: GgmlQuantizedMatmulIdParams) -> None:
    """out[t*top_k+s, :] = input[t, :] . dequant(W[ids[t*top_k+s]])^T  -- mul_mat_id."""
    xdt = _act(input, "input")
    if ids.dtype not in (torch.int32, torch.uint32) or not ids.is_cuda or not ids.is_contiguous():
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "ids must be a contiguous 32-bit integer CUDA tensor")
    rows = params.n_tokens * params.top_k
    if ids.numel() < rows or out.numel() < rows * params.n or input.numel() < params.n_tokens * params.k:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "ids/input/out smaller than the params require")
    if out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous():
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "out must be a contiguous float32 CUDA tensor")
    sp, sb = (scratch.buf.data_ptr(), scratch.nbytes) if scratch is not None else (None, 0)
    wp = weight_ptr.ptr if isinstance(weight_ptr, QuantWeight) else int(weight_ptr)
    ctx._check(ctx._lib.hf2q_cuda_qmatmul_id(ctx._h, ctx._stream(), input.data_ptr(), xdt, wp,
                                             ids.data_ptr(), out.data_ptr(), params.n_tokens, params.top_k,
                                             params.n, params.k, params.n_experts, params.expert_stride,
                                             int(params.ggml_type), sp, sb))


def quantized_matmul_id_pair_ggml(ctx: GpuContext, input: torch.Tensor, weight_a: int, weight_b: int, ids: torch.Tensor,
                                  out_a: torch.Tensor, out_b: torch.Tensor, scratch: IdMmScratch | None,
                                  params: GgmlQuantizedMatmulIdParams) -> None:
    """mul_mat_id against two stacked expert tensors of the same geometry (gate and up) sharing input and ids."""
    xdt = _act(input, "input")
    if ids.dtype not in (torch.int32, torch.uint32) or not ids.is_cuda or not ids.is_contiguous():
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "ids must be a contiguous 32-bit integer CUDA tensor")
    rows = params.n_tokens * params.top_k
    if ids.numel() < rows or min(out_a.numel(), out_b.numel()) < rows * params.n or input.numel() < params.n_tokens * params.k:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "ids/input/out smaller than the params require")
    for out in (out_a, out_b):
        if out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous():
            raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "outputs must be contiguous float32 CUDA tensors")
    sp, sb = (scratch.buf.data_ptr(), scratch.nbytes) if scratch is not None else (None, 0)
    wa = weight_a.ptr if isinstance(weight_a, QuantWeight) else int(weight_a)
    wb = weight_b.ptr if isinstance(weight_b, QuantWeight) else int(weight_b)
    ctx._check(ctx._lib.hf2q_cuda_qmatmul_id_pair(ctx._h, ctx._stream(), input.data_ptr(), xdt, wa, wb, ids.data_ptr(),
                                                  out_a.data_ptr(), out_b.data_ptr(), params.n_tokens, params.top_k,
                                                  params.n, params.k, params.n_experts, params.expert_stride,
                                                  int(params.ggml_type), sp, sb))


def quantized_matmul_id_swiglu_supported(ctx: GpuContext, params: GgmlQuantizedMatmulIdParams, x_dtype=torch.float32) -> bool:
    xdt = DT_BF16 if x_dtype == torch.bfloat16 else DT_F32
    return bool(ctx._lib.hf2q_cuda_qmatmul_id_swiglu_supported(ctx._h, params.n_tokens, params.top_k, params.n, params.k,
                                                               int(params.ggml_type), xdt))


def quantized_matmul_id_swiglu_ggml(ctx: GpuContext, input: torch.Tensor, weight_gate: int, weight_up: int, ids: torch.Tensor,
                                    out: torch.Tensor, params: GgmlQuantizedMatmulIdParams) -> None:
    """out[row] = silu(gate_e . x) * (up_e . x) for few routed rows in one launch (gpu_ffn.rs:2606-2760)."""
    xdt = _act(input, "input")
    if ids.dtype not in (torch.int32, torch.uint32) or not ids.is_cuda or not ids.is_contiguous():
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "ids must be a contiguous 32-bit integer CUDA tensor")
    rows = params.n_tokens * params.top_k
    if ids.numel() < rows or out.numel() < rows * params.n or input.numel() < params.n_tokens * params.k:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "ids/input/out smaller than the params require")
    if out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous():
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "out must be a contiguous float32 CUDA tensor")
    wg = weight_gate.ptr if isinstance(weight_gate, QuantWeight) else int(weight_gate)
    wu = weight_up.ptr if isinstance(weight_up, QuantWeight) else int(weight_up)
    ctx._check(ctx._lib.hf2q_cuda_qmatmul_id_swiglu(ctx._h, ctx._stream(), input.data_ptr(), xdt, wg, wu, ids.data_ptr(),
                                                    out.data_ptr(), params.n_tokens, params.top_k, params.n, params.k,
                                                    params.n_experts, params.expert_stride, int(params.ggml_type)))


def moe_experts_supported(ctx: GpuContext, n_tokens: int, top_k: int, hidden: int, ffn: int, n_experts: int,
                          type_gate_up: int, type_down: int) -> bool:
    return bool(ctx._lib.hf2q_cuda_moe_experts_supported(ctx._h, n_tokens, top_k, hidden, ffn, n_experts, int(type_gate_up), int(type_down)))


def moe_experts(ctx: GpuContext, input: torch.Tensor, gate_ptr: int, up_ptr: int, down_ptr: int, ids: torch.Tensor, out: torch.Tensor,
                n_tokens: int, top_k: int, hidden: int, ffn: int, n_experts: int, type_gate_up: int, type_down: int,
                stride_gate_up: int | None = None, stride_down: int | None = None) -> None:
    """out[t*top_k+s, :] = down_e . (silu(gate_e . x_t) * (up_e . x_t)), e = ids[t*top_k+s]: the routed experts of an MoE
    layer for many routed rows in four launches (gpu_ffn.rs:2606-2760 runs mul_mat_id x2, silu_mul, mul_mat_id)."""
    xdt = _act(input, "input")
    rows = n_tokens * top_k
    if ids.dtype not in (torch.int32, torch.uint32) or not ids.is_cuda or not ids.is_contiguous() or ids.numel() < rows:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "ids must be a contiguous 32-bit integer CUDA tensor of n_tokens * top_k")
    if out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous() or out.numel() < rows * hidden:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "out must be a contiguous float32 CUDA tensor of [n_tokens * top_k, hidden]")
    if input.numel() < n_tokens * hidden:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "input smaller than [n_tokens, hidden]")
    sg = stride_gate_up if stride_gate_up is not None else expert_stride(type_gate_up, ffn, hidden)
    sd = stride_down if stride_down is not None else expert_stride(type_down, hidden, ffn)
    need = C.c_uint64()
    ctx._check(ctx._lib.hf2q_cuda_moe_experts_scratch_bytes(n_experts, rows, hidden, ffn, C.byref(need)))
    sc = getattr(ctx, "_moe_scratch", None)
    if sc is None or sc.numel() < need.value:
        sc = torch.empty(need.value, dtype=torch.uint8, device=input.device)
        ctx._moe_scratch = sc
    ctx._check(ctx._lib.hf2q_cuda_moe_experts(ctx._h, ctx._stream(), input.data_ptr(), xdt, int(gate_ptr), int(up_ptr), int(down_ptr),
                                              ids.data_ptr(), out.data_ptr(), n_tokens, top_k, hidden, ffn, n_experts, sg,
                                              int(type_gate_up), sd, int(type_down), sc.data_ptr(), sc.numel()))


def moe_experts_reduce(ctx: GpuContext, input: torch.Tensor, gate_ptr: int, up_ptr: int, down_ptr: int, ids: torch.Tensor,
                       weights: torch.Tensor, out: torch.Tensor, n_tokens: int, top_k: int, hidden: int, ffn: int, n_experts: int,
                       type_gate_up: int, type_down: int) -> None:
    """``moe_experts`` with the weighted sum over the slots folded into the down product: every slot's row times
    weights[slot] is ADDED to out[token] (f32 [n_tokens, hidden], initialised by the caller) with floating-point atomics."""
    xdt = _act(input, "input")
    rows = n_tokens * top_k
    if out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous() or out.numel() < n_tokens * hidden:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "out must be a contiguous float32 CUDA tensor of [n_tokens, hidden]")
    if weights.dtype != torch.float32 or weights.numel() < rows or ids.numel() < rows:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "ids / weights must hold n_tokens * top_k entries")
    need = C.c_uint64()
    ctx._check(ctx._lib.hf2q_cuda_moe_experts_scratch_bytes(n_experts, rows, hidden, ffn, C.byref(need)))
    sc = getattr(ctx, "_moe_scratch", None)
    if sc is None or sc.numel() < need.value:
        sc = torch.empty(need.value, dtype=torch.uint8, device=input.device)
        ctx._moe_scratch = sc
    ctx._check(ctx._lib.hf2q_cuda_moe_experts_reduce(ctx._h, ctx._stream(), input.data_ptr(), xdt, int(gate_ptr), int(up_ptr), int(down_ptr),
                                                     ids.data_ptr(), weights.data_ptr(), out.data_ptr(), n_tokens, top_k, hidden, ffn,
                                                     n_experts, expert_stride(type_gate_up, ffn, hidden), int(type_gate_up),
                                                     expert_stride(type_down, hidden, ffn), int(type_down), sc.data_ptr(), sc.numel()))


def dequantize(ctx: GpuContext, weight: QuantWeight, out_dtype=torch.float32) -> torch.Tensor:
    out = torch.empty((weight.rows, weight.cols), dtype=out_dtype, device=f"cuda:{ctx.device}")
    ctx._check(ctx._lib.hf2q_cuda_dequantize(ctx._h, ctx._stream(), weight.ptr, weight.ggml_type,
                                             weight.rows, weight.cols, out.data_ptr(), _TORCH_DT[out_dtype]))
    return out


def moe_softmax_topk(ctx: GpuContext, logits: torch.Tensor, top_k: int):
    if logits.dtype != torch.float32 or not logits.is_cuda or not logits.is_contiguous() or logits.dim() != 2:
        raise Hf2qError(_lib.ERR_INVALID_ARGUMENT, "logits must be a contiguous float32 [tokens, experts] CUDA tensor")
    t, e = logits.shape
    ids = torch.empty(t * top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(t * top_k, dtype=torch.float32, device=logits.device)
    ctx._check(ctx._lib.hf2q_cuda_moe_softmax_topk(ctx._h, ctx._stream(), logits.data_ptr(), ids.data_ptr(),
                                                   w.data_ptr(), t, e, top_k))
    return ids, w
