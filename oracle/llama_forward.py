"""CPU restatement of a Llama-shaped decoder forward -- TEST INFRASTRUCTURE, not product code.

Plain numpy, float64 products on the oracle's dequantised weights (the accuracy yardstick of
this build), following the reference's scalar specs: ``rms_norm_rows`` and ``residual_add``
(src/inference/models/qwen35/forward_cpu.rs:36-56), ``matmul_a_by_bt`` (ffn.rs:38-50),
``dense_swiglu_cpu_ref`` (ffn.rs:91-112), the causal softmax attention of
``gated_full_attention_cpu_ref`` (full_attn.rs:219-360) without its output gate and with the
plain rotary embedding of the Llama architecture (pairs (2i, 2i+1), angle pos * theta^(-2i/d)),
``embed_tokens`` / ``apply_output_head`` (io_heads.rs).

The KV cache is modelled the way the CUDA path stores it: K (after the rotation) and V are
rounded to signed 8-bit codes with one f32 scale amax / 127 per (head, position) -- a stand-in
for the reference's 8-bit codebook cache (kv_cache.rs:1982-2012), whose codebook lives in the
external mlx-native crate -- and attention reads the rounded values.
"""
from __future__ import annotations

import numpy as np


def rms_norm_rows(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return x * inv * w


def rope(x: np.ndarray, pos: np.ndarray, theta: float) -> np.ndarray:
    """x [T, heads, d]; pairs (2i, 2i+1) rotated by pos * theta^(-2i/d)."""
    d = x.shape[-1]
    freq = theta ** (-np.arange(0, d, 2, dtype=np.float64) / d)
    ang = pos[:, None].astype(np.float64) * freq[None, :]
    cs, sn = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = a * cs - b * sn
    out[..., 1::2] = a * sn + b * cs
    return out


def quantize_kv(v: np.ndarray) -> np.ndarray:
    """[T, heads, d] -> the values an int8 cache with one f32 scale per (token, head) holds."""
    v32 = v.astype(np.float32)
    amax = np.abs(v32).max(axis=-1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = np.where(amax > 0, np.float32(127.0) / amax, np.float32(0.0)).astype(np.float32)
    codes = np.rint((v32 * inv).astype(np.float32))
    scale = (amax / np.float32(127.0)).astype(np.float32)
    return (codes * scale).astype(np.float64)


def forward(ids: np.ndarray, W: dict, cfg) -> np.ndarray:
    """Logits [T, vocab] of the prompt ``ids``; W maps tensor names to dequantised f32 matrices
    (token_embd, output, out_norm, blk.i.{attn_norm, attn_q, attn_k, attn_v, attn_output, ffn_norm,
    ffn_gate, ffn_up, ffn_down})."""
    T = len(ids)
    H, nh, nkv, d = cfg.hidden, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    g = nh // nkv
    pos = np.arange(T)
    x = W["token_embd"][ids].astype(np.float64)
    f64 = lambda name: W[name].astype(np.float64)
    mask = np.triu(np.ones((T, T), dtype=bool), k=1)
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        xn = rms_norm_rows(x, f64(p + "attn_norm"), cfg.rms_eps)
        q = (xn @ f64(p + "attn_q").T).reshape(T, nh, d)
        k = (xn @ f64(p + "attn_k").T).reshape(T, nkv, d)
        v = (xn @ f64(p + "attn_v").T).reshape(T, nkv, d)
        q = rope(q, pos, cfg.rope_theta) / np.sqrt(d)
        k = quantize_kv(rope(k, pos, cfg.rope_theta))
        v = quantize_kv(v)
        att = np.empty((T, nh, d))
        for h in range(nh):
            s = q[:, h, :] @ k[:, h // g, :].T
            s[mask] = -np.inf
            s = s - s.max(axis=-1, keepdims=True)
            pr = np.exp(s)
            pr /= pr.sum(axis=-1, keepdims=True)
            att[:, h, :] = pr @ v[:, h // g, :]
        x = x + att.reshape(T, nh * d) @ f64(p + "attn_output").T
        xn = rms_norm_rows(x, f64(p + "ffn_norm"), cfg.rms_eps)
        a, b = xn @ f64(p + "ffn_gate").T, xn @ f64(p + "ffn_up").T
        x = x + ((a / (1.0 + np.exp(-a))) * b) @ f64(p + "ffn_down").T
    xn = rms_norm_rows(x, f64("out_norm"), cfg.rms_eps)
    return xn @ f64("output").T
