"""Seeded synthetic inputs shared by the tests, the smoke check and the benchmark.

Weights are i.i.d. N(0, sigma=0.02) float32 from numpy's PCG64 ``default_rng(seed)``, passed
through the f16 round trip hf2q's converter applies before quantizing
(src/convert/orchestrator.rs:536-550) and then through the oracle's quantizer.  Activations are
N(0, 1); bf16 activations are rounded once on the host and every consumer sees those values.
"""
from __future__ import annotations

import numpy as np

import oracle

FIXTURES = {oracle.Q4_0: ("q4_0", 64), oracle.Q8_0: ("q8_0", 64), oracle.Q4_K: ("q4_k", 512),
            oracle.Q5_K: ("q5_k", 512), oracle.Q6_K: ("q6_k", 512), oracle.Q4_1: ("q4_1", 64),
            oracle.Q5_0: ("q5_0", 64), oracle.Q5_1: ("q5_1", 64), oracle.IQ4_NL: ("iq4_nl", 64)}


def make_weight_f32(n: int, k: int, seed: int, sigma: float = 0.02) -> np.ndarray:
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(sigma)
    return oracle.f16_round_trip(w).reshape(n, k)


def make_quant_weight(t: int, n: int, k: int, seed: int) -> np.ndarray:
    return oracle.quantize(t, make_weight_f32(n, k, seed), k)


def make_x(m: int, k: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((m, k), dtype=np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def rel_l2(a: np.ndarray, ref: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(a - ref) / (den if den > 0 else 1.0))


def random_finite_blocks(t: int, nblocks: int, seed: int) -> np.ndarray:
    """Uniformly random block bytes whose f16 scale fields are finite (exponent != 31)."""
    be, bb = oracle.block_geometry(t)
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
    offs = {oracle.Q4_0: [0], oracle.Q8_0: [0], oracle.Q4_K: [0, 2], oracle.Q5_K: [0, 2], oracle.Q6_K: [208],
            oracle.Q4_1: [0, 2], oracle.Q5_0: [0], oracle.Q5_1: [0, 2], oracle.IQ4_NL: [0]}[t]
    for o in offs:
        hi = raw[:, o + 1]
        bad = (hi & 0x7C) == 0x7C
        raw[bad, o + 1] = hi[bad] & 0xBF       # clear one exponent bit -> finite
    return raw.reshape(-1)


def _f16_field(raw2: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(raw2).view("<f2").astype(np.float32).reshape(-1)


def stored_codes(t: int, raw: np.ndarray) -> np.ndarray:
    """The integer codes L a block stores, per element in natural order, straight from the packing
    loops of hf2q's quantizers (q4_0.rs:60-64, q8_0.rs:66, q4_k.rs:204-215, q5_k.rs:137-158,
    q6_k.rs:120-143).  Shape [blocks, block elements], int32."""
    be, bb = oracle.block_geometry(t)
    b = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, bb)
    nb = b.shape[0]
    if t == oracle.Q4_0:
        qs = b[:, 2:18]
        return np.concatenate([qs & 15, qs >> 4], axis=1).astype(np.int32)
    if t == oracle.Q8_0:
        return b[:, 2:34].view(np.int8).astype(np.int32)
    if t in (oracle.Q4_1, oracle.IQ4_NL):
        qs = b[:, 4:20] if t == oracle.Q4_1 else b[:, 2:18]
        return np.concatenate([qs & 15, qs >> 4], axis=1).astype(np.int32)
    if t in (oracle.Q5_0, oracle.Q5_1):
        o = 2 if t == oracle.Q5_0 else 4
        qh = np.ascontiguousarray(b[:, o:o + 4]).view("<u4").astype(np.int64).reshape(-1, 1)
        qs = b[:, o + 4:o + 20].astype(np.int32)
        j = np.arange(16)
        lo = (qs & 15) | ((((qh >> j) & 1) << 4).astype(np.int32))
        hi = (qs >> 4) | ((((qh >> (j + 16)) & 1) << 4).astype(np.int32))
        return np.concatenate([lo, hi], axis=1).astype(np.int32)
    if t in (oracle.Q4_K, oracle.Q5_K):
        qs = (b[:, 16:144] if t == oracle.Q4_K else b[:, 48:176]).reshape(nb, 4, 32)
        lo, hi = (qs & 15).astype(np.int32), (qs >> 4).astype(np.int32)
        if t == oracle.Q5_K:
            qh = b[:, 16:48].astype(np.int32)
            for c in range(4):
                lo[:, c, :] += 16 * ((qh >> (2 * c)) & 1)
                hi[:, c, :] += 16 * ((qh >> (2 * c + 1)) & 1)
        return np.stack([lo, hi], axis=2).reshape(nb, 256)
    ql, qh = b[:, 0:128].astype(np.int32), b[:, 128:192].astype(np.int32)
    out = np.empty((nb, 256), np.int32)
    for n in range(2):
        for l in range(32):
            h = qh[:, 32 * n + l]
            out[:, 128 * n + l] = (ql[:, 64 * n + l] & 15) | ((h & 3) << 4)
            out[:, 128 * n + l + 32] = (ql[:, 64 * n + l + 32] & 15) | (((h >> 2) & 3) << 4)
            out[:, 128 * n + l + 64] = (ql[:, 64 * n + l] >> 4) | (((h >> 4) & 3) << 4)
            out[:, 128 * n + l + 96] = (ql[:, 64 * n + l + 32] >> 4) | (((h >> 6) & 3) << 4)
    return out


def reencode_codes(t: int, raw: np.ndarray, y: np.ndarray):
    """Recomputes the integer codes from dequantised values ``y`` with the STORED f16 scales and
    packed sub-block scales, by the formulas of the quantizers' second pass (q4_k.rs:183-197,
    q5_k.rs:100-123, q6_k.rs:96-110, q4_0.rs:47-64, q8_0.rs:59-67).  Returns (codes, valid): codes
    [blocks, block elements] int32 comparable with ``stored_codes``; valid marks the elements
    whose (sub-)block scale is non-zero (the quantizers skip the others and keep earlier codes).
    float32 arithmetic, one operation per numpy call."""
    be, bb = oracle.block_geometry(t)
    b = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, bb)
    nb = b.shape[0]
    y = np.ascontiguousarray(y, dtype=np.float32).reshape(nb, be)
    one = np.float32(1.0)
    if t in (oracle.Q4_0, oracle.Q8_0):
        d = _f16_field(b[:, 0:2])[:, None]
        with np.errstate(divide="ignore"):
            inv = np.where(d != 0, one / d, np.float32(0.0)).astype(np.float32)
        v = (y * inv).astype(np.float32)
        if t == oracle.Q4_0:
            codes = np.minimum(15, np.trunc((v + np.float32(8.5)).astype(np.float32))).astype(np.int32)
        else:
            codes = (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int32)    # f32::round: half away from zero
        return codes, np.broadcast_to(d != 0, codes.shape)
    if t in (oracle.Q4_K, oracle.Q5_K):
        d = _f16_field(b[:, 0:2])[:, None]
        dmin = _f16_field(b[:, 2:4])[:, None]
        s = b[:, 4:16]
        sc = np.empty((nb, 8), np.float32)
        mn = np.empty((nb, 8), np.float32)
        sc[:, :4], mn[:, :4] = s[:, 0:4] & 63, s[:, 4:8] & 63
        sc[:, 4:] = (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)
        mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
        dd = np.repeat((d * sc).astype(np.float32), 32, axis=1)
        dm = np.repeat((dmin * mn).astype(np.float32), 32, axis=1)
        with np.errstate(divide="ignore", invalid="ignore"):
            q = np.rint(((y + dm).astype(np.float32) / dd).astype(np.float32))
        hi = 15 if t == oracle.Q4_K else 31
        valid = dd != 0
        return np.clip(np.where(valid, q, 0), 0, hi).astype(np.int32), valid
    if t in (oracle.Q4_1, oracle.Q5_1):
        # make_qkx3_quants (common.rs:339-343): L = clamp(nearest_int((x - min) / scale), 0, nmax) with the stored f16 d and m
        d = _f16_field(b[:, 0:2])[:, None]
        m = _f16_field(b[:, 2:4])[:, None]
        with np.errstate(divide="ignore", invalid="ignore"):
            q = np.rint(((y - m).astype(np.float32) / d).astype(np.float32))
        valid = np.broadcast_to(d != 0, q.shape)
        return np.clip(np.where(valid, q, 0), 0, 15 if t == oracle.Q4_1 else 31).astype(np.int32), valid
    if t == oracle.Q5_0:
        # q5_0.rs:80-100: q = min(31, trunc(x / d + 16.5)) with the stored f16 d
        d = _f16_field(b[:, 0:2])[:, None]
        with np.errstate(divide="ignore"):
            inv = np.where(d != 0, one / d, np.float32(0.0)).astype(np.float32)
        v = ((y * inv).astype(np.float32) + np.float32(16.5)).astype(np.float32)
        return np.minimum(31, np.trunc(v)).astype(np.int32), np.broadcast_to(d != 0, v.shape)
    if t == oracle.IQ4_NL:
        # iq4_nl.rs final pass: L = best_index_int8(values, x / d): the nearest codebook entry
        kv = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)
        d = _f16_field(b[:, 0:2])[:, None]
        with np.errstate(divide="ignore"):
            inv = np.where(d != 0, one / d, np.float32(0.0)).astype(np.float32)
        v = (y * inv).astype(np.float32)
        codes = np.abs(v[:, :, None] - kv[None, None, :]).argmin(axis=2).astype(np.int32)
        return codes, np.broadcast_to(d != 0, codes.shape)
    sc = b[:, 192:208].view(np.int8).astype(np.float32)
    d = _f16_field(b[:, 208:210])[:, None]
    dd = np.repeat((d * sc).astype(np.float32), 16, axis=1)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.rint((y / dd).astype(np.float32))
    valid = dd != 0
    return (np.clip(np.where(valid, q, 0), -32, 31) + 32).astype(np.int32), valid
