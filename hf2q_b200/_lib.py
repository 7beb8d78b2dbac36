"""ctypes binding of libhf2q_cuda.so -- the same symbols a Rust ``hf2q-cuda-sys`` crate would bind.

There is no fallback: if the library is missing or a symbol is absent, import fails loudly.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libhf2q_cuda.so"
HEADER = PKG.parent / "include" / "hf2q_cuda.h"

OK = 0
ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED_TYPE, ERR_CUDA, ERR_WORKSPACE = 1, 2, 3, 4
ERR_TIMEOUT, ERR_OUT_OF_MEMORY, ERR_NO_DEVICE = 5, 6, 7

i32, u32, u64, vp = C.c_int32, C.c_uint32, C.c_uint64, C.c_void_p
pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); kept in the order of include/hf2q_cuda.h
SIGNATURES = {
    "hf2q_cuda_ctx_create": (i32, [i32, pp]),
    "hf2q_cuda_ctx_destroy": (i32, [vp]),
    "hf2q_cuda_strerror": (C.c_char_p, [i32]),
    "hf2q_cuda_last_error": (C.c_char_p, [vp]),
    "hf2q_cuda_check_status": (i32, [vp, vp]),
    "hf2q_cuda_block_geometry": (i32, [u32, C.POINTER(u32), C.POINTER(u32)]),
    "hf2q_cuda_row_bytes": (i32, [u32, u64, C.POINTER(u64)]),
    "hf2q_cuda_expert_stride": (i32, [u32, u64, u64, C.POINTER(u64)]),
    "hf2q_cuda_upload_blocks": (i32, [vp, vp, u64, pp]),
    "hf2q_cuda_free": (i32, [vp, vp]),
    "hf2q_cuda_dequantize": (i32, [vp, vp, vp, u32, u64, u64, vp, u32]),
    "hf2q_cuda_qmatmul": (i32, [vp, vp, vp, u32, vp, vp, u32, u32, u32, u32, vp, u64]),
    "hf2q_cuda_qmatmul_workspace_bytes": (i32, [u32, u32, u32, u32, u32, C.POINTER(u64)]),
    "hf2q_cuda_qmatmul_segments": (i32, [vp, vp, vp, u32, vp, u32, vp, u32, u32, vp, u64]),
    "hf2q_cuda_qmatmul_static": (i32, [vp, vp, vp, u32, vp, vp, u32, u32, u32, u32]),
    "hf2q_cuda_qmatmul_static_max_elements": (u64, []),
    "hf2q_cuda_qmatmul_id_swiglu_supported": (i32, [vp, u32, u32, u32, u32, u32, u32]),
    "hf2q_cuda_qmatmul_id_swiglu": (i32, [vp, vp, vp, u32, vp, vp, vp, vp, u32, u32, u32, u32, u32, u64, u32]),
    "hf2q_cuda_qmatmul_swiglu_supported": (i32, [vp, u32, u32, u32, u32, u32]),
    "hf2q_cuda_qmatmul_swiglu": (i32, [vp, vp, vp, u32, vp, vp, vp, u32, u32, u32, u32]),
    "hf2q_cuda_qmatmul_add_supported": (i32, [vp, u32, u32, u32, u32]),
    "hf2q_cuda_qmatmul_add": (i32, [vp, vp, vp, u32, vp, vp, vp, u32, u32, u32, u32]),
    "hf2q_cuda_affine_pack": (i32, [vp, vp, vp, vp, vp, u32, u32, u32, u32, vp]),
    "hf2q_cuda_qmatmul_perm021": (i32, [vp, vp, vp, u32, vp, vp, u32, u32, u32, u32, u32, vp, u64]),
    "hf2q_cuda_qmatmul_swiglu_ws_supported": (i32, [vp, u32, u32, u32, u32, u32]),
    "hf2q_cuda_qmatmul_swiglu_ws": (i32, [vp, vp, vp, u32, vp, vp, vp, u32, u32, u32, u32, vp, u64]),
    "hf2q_cuda_qmatmul_add_ws_supported": (i32, [vp, u32, u32, u32, u32, u32]),
    "hf2q_cuda_qmatmul_add_ws": (i32, [vp, vp, vp, u32, vp, vp, vp, u32, u32, u32, u32, vp, u64]),
    "hf2q_cuda_qmatmul_host": (i32, [vp, vp, u32, vp, vp, u32, u32, u32, u32]),
    "hf2q_cuda_qmatmul_host_async": (i32, [vp, vp, u32, vp, vp, u32, u32, u32, u32]),
    "hf2q_cuda_host_sync": (i32, [vp]),
    "hf2q_cuda_qmatmul_host_batch": (i32, [vp, vp, u32]),
    "hf2q_cuda_ipc_alloc": (i32, [vp, u64, pp, vp]),
    "hf2q_cuda_ipc_open": (i32, [vp, vp, pp]),
    "hf2q_cuda_ipc_close": (i32, [vp, vp]),
    "hf2q_cuda_qmatmul_gather": (i32, [vp, vp, vp, u32, vp, vp, u32, u32, u32, u32]),
    "hf2q_cuda_gather_wait": (i32, [vp, vp, vp]),
    "hf2q_cuda_gather_sum": (i32, [vp, vp, vp, vp, u32, u32]),
    "hf2q_cuda_qmatmul_gather_host_batch": (i32, [vp, vp, u64, u32, vp, u32]),
    "hf2q_cuda_gather_supported": (i32, [vp, vp, u32, u32, u32, u32, u32]),
    "hf2q_cuda_gather_copy": (i32, [vp, vp, vp, vp, u32]),
    "hf2q_cuda_set_wait_limit": (i32, [vp, u64]),
    "hf2q_cuda_comm_unique_id": (i32, [vp]),
    "hf2q_cuda_comm_create": (i32, [i32, vp, i32, i32, pp]),
    "hf2q_cuda_comm_destroy": (i32, [vp]),
    "hf2q_cuda_comm_last_error": (C.c_char_p, [vp]),
    "hf2q_cuda_qmatmul_rowshard_workspace_bytes": (i32, [u32, u32, u32, u32, u32, u32, C.POINTER(u64)]),
    "hf2q_cuda_qmatmul_rowshard": (i32, [vp, vp, vp, vp, u32, vp, vp, u32, u32, u32, u32, vp, u64]),
    "hf2q_cuda_qmatmul_id_ep_scratch_bytes": (i32, [u32, u32, u32, u32, u32, u32, u32, C.POINTER(u64)]),
    "hf2q_cuda_qmatmul_id_ep": (i32, [vp, vp, vp, vp, u32, vp, vp, vp, u32, u32, u32, u32, u32, u64, u32, vp, u64]),
    "hf2q_cuda_moe_experts_ep_scratch_bytes": (i32, [u32, u32, u32, u32, u32, u32, u32, C.POINTER(u64)]),
    "hf2q_cuda_moe_experts_ep": (i32, [vp, vp, vp, vp, u32, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u64, u64, u32, u32, vp, u64]),
    "hf2q_cuda_qmatmul_id": (i32, [vp, vp, vp, u32, vp, vp, vp, u32, u32, u32, u32, u32, u64, u32, vp, u64]),
    "hf2q_cuda_qmatmul_id_pair": (i32, [vp, vp, vp, u32, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u64, u32, vp, u64]),
    "hf2q_cuda_qmatmul_id_scratch_bytes": (i32, [u32, u32, u32, u32, C.POINTER(u64)]),
    "hf2q_cuda_moe_experts_scratch_bytes": (i32, [u32, u32, u32, u32, C.POINTER(u64)]),
    "hf2q_cuda_moe_experts_supported": (i32, [vp, u32, u32, u32, u32, u32, u32, u32]),
    "hf2q_cuda_moe_experts": (i32, [vp, vp, vp, u32, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u64, u32, u64, u32, vp, u64]),
    "hf2q_cuda_dense_ffn_scratch_bytes": (i32, [u32, u32, u32, C.POINTER(u64)]),
    "hf2q_cuda_dense_ffn": (i32, [vp, vp, vp, u32, vp, u32, vp, u32, vp, u32, vp, vp, u32, u32, u32, vp, u64, u32]),
    "hf2q_cuda_moe_ffn_scratch_bytes": (i32, [vp, u32, u32, C.POINTER(u64)]),
    "hf2q_cuda_moe_ffn": (i32, [vp, vp, vp, u32, vp, vp, vp, u32, u32, vp, u64, u32]),
    "hf2q_cuda_moe_experts_reduce": (i32, [vp, vp, vp, u32, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u64, u32, u64, u32, vp, u64]),
    "hf2q_cuda_moe_softmax_topk": (i32, [vp, vp, vp, vp, vp, u32, u32, u32]),
    "hf2q_cuda_silu_mul": (i32, [vp, vp, vp, vp, vp, u64]),
    "hf2q_cuda_moe_combine": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32]),
    "hf2q_cuda_router_logits": (i32, [vp, vp, vp, u32, vp, vp, u32, u32, u32]),
    "hf2q_cuda_rowdot": (i32, [vp, vp, vp, vp, vp, u32, u32]),
    "hf2q_cuda_kv_cache_bytes": (i32, [u32, u32, u32, C.POINTER(u64), C.POINTER(u64)]),
    "hf2q_cuda_get_rows": (i32, [vp, vp, vp, u32, u32, u32, vp, u32, vp]),
    "hf2q_cuda_rms_norm": (i32, [vp, vp, vp, vp, vp, C.c_float, vp, u32, u32, u32]),
    "hf2q_cuda_rope_kv_append": (i32, [vp, vp, vp, u32, u32, C.c_float, vp, vp]),
    "hf2q_cuda_attn_decode_scratch_bytes": (i32, [vp, u32, u32, C.POINTER(u64)]),
    "hf2q_cuda_attn_decode": (i32, [vp, vp, vp, u32, vp, vp, vp, u32, vp, u64]),
    "hf2q_cuda_norm_supported": (i32, [vp, u32, u32, u32]),
    "hf2q_cuda_norm_qmatmul_segments": (i32, [vp, vp, vp, vp, C.c_float, vp, u32, vp, u32, u32]),
    "hf2q_cuda_norm_qmatmul_swiglu": (i32, [vp, vp, vp, vp, C.c_float, vp, vp, vp, u32, u32, u32, u32]),
    "hf2q_cuda_attn_decode_fused": (i32, [vp, vp, vp, u32, C.c_float, vp, vp, vp, u32, vp, u64]),
    "hf2q_cuda_attn_prefill": (i32, [vp, vp, vp, u32, u32, vp, u32, vp, u32]),
    "hf2q_cuda_argmax": (i32, [vp, vp, vp, u32, vp, vp]),
    "hf2q_cuda_add": (i32, [vp, vp, vp, vp, u64]),
    "hf2q_cuda_launch_count": (u64, [vp]),
    "hf2q_cuda_sm_count": (i32, [vp]),
    "hf2q_cuda_version": (C.c_char_p, []),
}


def declared_symbols() -> list[str]:
    """Every function name the public header declares."""
    text = HEADER.read_text()
    return sorted(set(re.findall(r"HF2Q_API\s+[\w\s\*]+?\b(hf2q_cuda_\w+)\s*\(", text)))


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing -- build it with `python -m hf2q_b200.build` "
                              "(there is no CPU or PyTorch fallback for this library)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
