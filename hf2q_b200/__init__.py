"""hf2q_b200 -- B200 (sm_100a) backend for hf2q's quantized-weight matmul path.

The product is ``libhf2q_cuda.so`` (C ABI in ``include/hf2q_cuda.h``).  This package is the thin
host-side mirror of the op surface hf2q's inference models call (``quantized_matmul_ggml``,
``quantized_matmul_id_ggml``, the raw-block weight loader); PyTorch supplies device buffers,
streams and ``torch.distributed`` only.
"""
from .ops import (  # noqa: F401
    GgmlType, GgmlQuantizedMatmulParams, GgmlQuantizedMatmulIdParams, Hf2qError, GpuContext,
    QuantWeight, IdMmScratch, load_quant_weight, load_mlx_affine_weight, quantized_matmul_ggml, quantized_matmul_id_ggml, quantized_matmul_id_pair_ggml,
    dequantize, moe_softmax_topk, row_bytes, expert_stride,
)
from . import ffn, dist, gguf, decoder  # noqa: F401,E402
