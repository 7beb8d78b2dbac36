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
            oracle.Q5_K: ("q5_k", 512), oracle.Q6_K: ("q6_k", 512)}


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
    offs = {oracle.Q4_0: [0], oracle.Q8_0: [0], oracle.Q4_K: [0, 2], oracle.Q5_K: [0, 2], oracle.Q6_K: [208]}[t]
    for o in offs:
        hi = raw[:, o + 1]
        bad = (hi & 0x7C) == 0x7C
        raw[bad, o + 1] = hi[bad] & 0xBF       # clear one exponent bit -> finite
    return raw.reshape(-1)
