"""CPU oracle for the quantized-weight matmul path -- TEST INFRASTRUCTURE, not product code.

ctypes front end of ``oracle/ggml_quants_oracle.cpp`` (a C++ restatement of hf2q's
``src/quantize/ggml_quants`` quantizers, their implied dequantisers, and the scalar f32 reference
math of ``src/inference/models/qwen35/ffn.rs`` / ``gpu_ffn.rs``).  Only the tests, the smoke check
and the benchmark's CPU-baseline leg import this package; the CUDA library never does.

Pinning status: quantizer bytes are pinned by the reference's golden fixtures; dequantised values
are "parity unpinned" in the reference (no test of its own compares them) and are anchored here by
the re-encode identity plus the independent numpy restatement in ``oracle/np_dequant.py``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "liboracle.so"
_SRC = _HERE / "ggml_quants_oracle.cpp"

# GGUF numeric type ids (src/quantize/ggml_quants/ggml_type.rs:18-33)
Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = 2, 3, 6, 7, 8, 12, 13, 14, 20
TYPE_NAMES = {Q4_0: "q4_0", Q8_0: "q8_0", Q4_K: "q4_k", Q5_K: "q5_k", Q6_K: "q6_k",
              Q4_1: "q4_1", Q5_0: "q5_0", Q5_1: "q5_1", IQ4_NL: "iq4_nl"}
ALL_TYPES = tuple(TYPE_NAMES)
# the five formats the benchmark workloads name; the other four are the quantizer's fall-back targets
# for tensors whose row length is not a multiple of 256 (standard_policy.rs:128-192)
MAIN_TYPES = (Q4_0, Q8_0, Q4_K, Q5_K, Q6_K)


def build(force: bool = False) -> Path:
    """Compile the oracle with the committed Makefile when the library is missing or stale."""
    stale = (not _SO.exists()) or _SO.stat().st_mtime < _SRC.stat().st_mtime
    if force or stale:
        env = dict(os.environ)
        env.pop("CXX", None)
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_SO))
        i64, u32, u64, vp, ci = C.c_int64, C.c_uint32, C.c_uint64, C.c_void_p, C.c_int
        L.oracle_block_geometry.argtypes = [u32, C.POINTER(ci), C.POINTER(ci)]
        L.oracle_row_bytes.argtypes = [u32, i64]
        L.oracle_row_bytes.restype = i64
        L.oracle_f16_round_trip.argtypes = [vp, vp, i64]
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_nearest_int.argtypes = [C.c_float]
        L.oracle_quantize.argtypes = [u32, vp, i64, i64, vp, vp, ci]
        L.oracle_encode_q4_0_simple.argtypes = [vp, i64, vp]
        L.oracle_dequantize.argtypes = [u32, vp, i64, vp, ci]
        L.oracle_matmul_a_by_bt.argtypes = [vp, vp, i64, i64, i64, vp, ci]
        L.oracle_matmul_a_by_bt.restype = None
        L.oracle_matmul_f64.argtypes = [vp, vp, i64, i64, i64, vp, ci]
        L.oracle_matmul_f64.restype = None
        L.oracle_qmatmul.argtypes = [u32, vp, vp, i64, i64, i64, vp, vp, ci, vp]
        L.oracle_qmatmul_id.argtypes = [u32, vp, u64, vp, vp, i64, i64, i64, i64, i64, vp, ci]
        L.oracle_softmax_topk_renorm.argtypes = [vp, i64, i64, i64, vp, vp]
        L.oracle_softmax_topk_renorm.restype = None
        L.oracle_dense_swiglu.argtypes = [vp, vp, vp, vp, i64, i64, i64, vp, ci]
        L.oracle_dense_swiglu.restype = None
        L.oracle_moe_ffn.argtypes = [vp] * 9 + [i64] * 6 + [vp]
        L.oracle_moe_ffn.restype = None
        L.oracle_mulberry32_uniform.argtypes = [vp, i64, u32]
        L.oracle_mulberry32_uniform.restype = None
        L.oracle_mulberry32_imatrix.argtypes = [vp, i64, u32]
        L.oracle_mulberry32_imatrix.restype = None
        L.oracle_max_threads.restype = ci
        L.oracle_set_threads.argtypes = [ci]
        L.oracle_set_threads.restype = None
        _lib = L
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def set_threads(n: int) -> None:
    """Default thread count of the OpenMP loops from here on (overrides an inherited OMP_NUM_THREADS)."""
    lib().oracle_set_threads(int(n))


def block_geometry(t: int) -> tuple[int, int]:
    be, bb = C.c_int(), C.c_int()
    if lib().oracle_block_geometry(t, C.byref(be), C.byref(bb)):
        raise ValueError(f"unsupported ggml type {t}")
    return be.value, bb.value


def row_bytes(t: int, k: int) -> int:
    r = lib().oracle_row_bytes(t, k)
    if r < 0:
        raise ValueError(f"k={k} is not a whole number of type-{t} blocks")
    return int(r)


def f16_round_trip(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().oracle_f16_round_trip(_p(x), _p(out), x.size)
    return out


def quantize(t: int, src, n_per_row: int, imatrix=None, threads: int = 0) -> np.ndarray:
    """f32 [rows, n_per_row] -> raw block bytes (uint8), row-major, as the reference's quantizers emit."""
    src = _f32(src).reshape(-1)
    if src.size % n_per_row:
        raise ValueError("src length is not a multiple of n_per_row")
    rows = src.size // n_per_row
    out = np.empty(rows * row_bytes(t, n_per_row), dtype=np.uint8)
    im = None
    if imatrix is not None:
        im = _f32(imatrix)
        if im.size != n_per_row:
            raise ValueError("imatrix length must equal n_per_row")
    rc = lib().oracle_quantize(t, _p(src), rows, n_per_row, _p(im) if im is not None else None,
                               _p(out), threads or max_threads())
    if rc:
        raise ValueError(f"oracle_quantize failed rc={rc}")
    return out


def encode_q4_0_simple(vals) -> np.ndarray:
    vals = _f32(vals).reshape(-1)
    out = np.empty(vals.size // 32 * 18, dtype=np.uint8)
    if lib().oracle_encode_q4_0_simple(_p(vals), vals.size, _p(out)):
        raise ValueError("length must be a multiple of 32")
    return out


def dequantize(t: int, blocks, threads: int = 0) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    be, bb = block_geometry(t)
    if blocks.size % bb:
        raise ValueError("byte length is not a whole number of blocks")
    n = blocks.size // bb * be
    out = np.empty(n, dtype=np.float32)
    if lib().oracle_dequantize(t, _p(blocks), n, _p(out), threads or max_threads()):
        raise ValueError("oracle_dequantize failed")
    return out


def matmul_a_by_bt(lhs, rhs, threads: int = 0) -> np.ndarray:
    lhs, rhs = _f32(lhs), _f32(rhs)
    m, k = lhs.shape
    n, k2 = rhs.shape
    assert k == k2
    out = np.empty((m, n), dtype=np.float32)
    lib().oracle_matmul_a_by_bt(_p(lhs), _p(rhs), m, k, n, _p(out), threads or max_threads())
    return out


def matmul_f64(lhs, rhs, threads: int = 0) -> np.ndarray:
    lhs, rhs = _f32(lhs), _f32(rhs)
    m, k = lhs.shape
    n, k2 = rhs.shape
    assert k == k2
    out = np.empty((m, n), dtype=np.float64)
    lib().oracle_matmul_f64(_p(lhs), _p(rhs), m, k, n, _p(out), threads or max_threads())
    return out


def qmatmul(t: int, w_blocks, x, n: int, k: int, threads: int = 1):
    """Reference CPU path: dequantise to f32 then matmul_a_by_bt.  Returns (y, t_dequant, t_matmul)."""
    w_blocks = np.ascontiguousarray(w_blocks, dtype=np.uint8).reshape(-1)
    x = _f32(x).reshape(-1, k)
    assert w_blocks.size == n * row_bytes(t, k)
    y = np.empty((x.shape[0], n), dtype=np.float32)
    scratch = np.empty(n * k, dtype=np.float32)
    tt = (C.c_double * 2)()
    rc = lib().oracle_qmatmul(t, _p(w_blocks), _p(x), x.shape[0], n, k, _p(scratch), _p(y), threads, tt)
    if rc:
        raise ValueError("oracle_qmatmul failed")
    return y, tt[0], tt[1]


def qmatmul_id(t: int, w_stacked, expert_stride: int, x, ids, n_tokens: int, top_k: int, n: int,
               k: int, n_experts: int, threads: int = 0) -> np.ndarray:
    w_stacked = np.ascontiguousarray(w_stacked, dtype=np.uint8).reshape(-1)
    x = _f32(x).reshape(n_tokens, k)
    ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
    assert ids.size == n_tokens * top_k
    y = np.empty((n_tokens * top_k, n), dtype=np.float32)
    rc = lib().oracle_qmatmul_id(t, _p(w_stacked), expert_stride, _p(x), _p(ids), n_tokens, top_k, n,
                                 k, n_experts, _p(y), threads or max_threads())
    if rc:
        raise ValueError(f"oracle_qmatmul_id failed rc={rc}")
    return y


def softmax_topk_renorm(logits, topk: int):
    logits = _f32(logits)
    t, e = logits.shape
    ids = np.empty(t * topk, dtype=np.uint32)
    w = np.empty(t * topk, dtype=np.float32)
    lib().oracle_softmax_topk_renorm(_p(logits), t, e, topk, _p(ids), _p(w))
    return ids, w


def mulberry32_uniform(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().oracle_mulberry32_uniform(_p(out), n, seed)
    return out


def mulberry32_imatrix(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().oracle_mulberry32_imatrix(_p(out), n, seed)
    return out


def dense_swiglu(x, gate, up, down, threads: int = 0) -> np.ndarray:
    """dense_swiglu_cpu_ref (ffn.rs:91-112) on f32 (dequantised) weights."""
    x, gate, up, down = _f32(x), _f32(gate), _f32(up), _f32(down)
    seq, h = x.shape
    m = gate.shape[0]
    y = np.empty((seq, h), dtype=np.float32)
    lib().oracle_dense_swiglu(_p(x), _p(gate), _p(up), _p(down), seq, h, m, _p(y), threads or max_threads())
    return y


def moe_ffn(x, router, eg, eu, ed, topk: int, shared=None) -> np.ndarray:
    """moe_ffn_cpu_ref (ffn.rs:179-336).  eg/eu: [E, m_moe, h]; ed: [E, h, m_moe];
    shared = (gate_logit[h], gate[m_sh,h], up[m_sh,h], down[h,m_sh]) or None."""
    x, router, eg, eu, ed = _f32(x), _f32(router), _f32(eg), _f32(eu), _f32(ed)
    seq, h = x.shape
    ne, m_moe = eg.shape[0], eg.shape[1]
    out = np.empty((seq, h), dtype=np.float32)
    if shared is not None:
        sl, sg, su, sd = (_f32(a) for a in shared)
        m_sh = sg.shape[0]
        lib().oracle_moe_ffn(_p(x), _p(router), _p(eg), _p(eu), _p(ed), _p(sl), _p(sg), _p(su), _p(sd), seq, h, ne, topk, m_moe, m_sh, _p(out))
    else:
        lib().oracle_moe_ffn(_p(x), _p(router), _p(eg), _p(eu), _p(ed), None, None, None, None, seq, h, ne, topk, m_moe, 0, _p(out))
    return out
