"""Second, independent restatement of the five block dequantisers in vectorised numpy.

TEST INFRASTRUCTURE.  It shares no code with ``ggml_quants_oracle.cpp`` and is written from the
block layouts and packing loops of hf2q's quantizers (q4_0.rs:47-64, q8_0.rs:59-67,
q4_k.rs:166-215, q5_k.rs:137-158, q6_k.rs:120-143), so a shared misreading of a layout would have
to be made twice.  All arithmetic is float32 with one operation per numpy call (no fusion).
"""
from __future__ import annotations

import numpy as np

Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = 2, 3, 6, 7, 8, 12, 13, 14, 20
_GEOM = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210),
         Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), IQ4_NL: (32, 18)}
_KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)


def _f16(b: np.ndarray) -> np.ndarray:
    """Two little-endian bytes per block -> float32 (exact widening)."""
    return np.ascontiguousarray(b).view("<f2").astype(np.float32).reshape(-1)


def _scale_min_k4(s: np.ndarray):
    """12 packed bytes per block -> (sc[nb,8], m[nb,8]) as float32."""
    s = s.astype(np.uint8)
    sc = np.empty((s.shape[0], 8), np.uint8)
    mn = np.empty((s.shape[0], 8), np.uint8)
    sc[:, :4] = s[:, 0:4] & 63
    mn[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0x0F) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc.astype(np.float32), mn.astype(np.float32)


def dequantize(t: int, raw) -> np.ndarray:
    be, bb = _GEOM[t]
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, bb)
    nb = raw.shape[0]
    if t == Q4_0:
        d = _f16(raw[:, 0:2])[:, None]
        qs = raw[:, 2:18]
        lo = (qs & 15).astype(np.int32) - 8
        hi = (qs >> 4).astype(np.int32) - 8
        q = np.concatenate([lo, hi], axis=1).astype(np.float32)
        return (q * d).reshape(-1)
    if t == Q8_0:
        d = _f16(raw[:, 0:2])[:, None]
        q = raw[:, 2:34].view(np.int8).astype(np.float32)
        return (q * d).reshape(-1)
    if t in (Q4_1, Q5_0, Q5_1, IQ4_NL):
        # 32-element blocks: [d][m (Q4_1, Q5_1)][qh u32 (Q5_0, Q5_1)][16 nibble bytes]; the low nibbles are
        # elements 0..15, the high nibbles 16..31; bit j / j+16 of qh is the fifth bit of element j / j+16
        # (q4_1.rs:104-110, q5_0.rs:95-110, q5_1.rs:70-85, iq4_nl.rs nibble pack)
        d = _f16(raw[:, 0:2])[:, None]
        o = 2
        m = None
        if t in (Q4_1, Q5_1):
            m = _f16(raw[:, 2:4])[:, None]
            o = 4
        hi5 = None
        if t in (Q5_0, Q5_1):
            qh = np.ascontiguousarray(raw[:, o:o + 4]).view("<u4").astype(np.uint32).reshape(-1, 1)
            hi5 = ((qh >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(np.int32)
            o += 4
        qs = raw[:, o:o + 16]
        q = np.concatenate([qs & 15, qs >> 4], axis=1).astype(np.int32)
        if hi5 is not None:
            q = q | (hi5 << 4)
        if t == IQ4_NL:
            return (d * _KVALUES_IQ4NL[q]).astype(np.float32).reshape(-1)
        if t == Q5_0:
            return ((q - 16).astype(np.float32) * d).reshape(-1)
        prod = d * q.astype(np.float32)
        return (prod + m).astype(np.float32).reshape(-1)
    if t in (Q4_K, Q5_K):
        d = _f16(raw[:, 0:2])[:, None]
        dmin = _f16(raw[:, 2:4])[:, None]
        sc, mn = _scale_min_k4(raw[:, 4:16])
        if t == Q4_K:
            qs = raw[:, 16:144].reshape(nb, 4, 32)
            lo = (qs & 15).astype(np.float32)
            hi = (qs >> 4).astype(np.float32)
        else:
            qh = raw[:, 16:48]                       # [nb, 32]
            qs = raw[:, 48:176].reshape(nb, 4, 32)
            c = np.arange(4, dtype=np.uint8)[None, :, None]
            b1 = (qh[:, None, :] >> (2 * c)) & 1
            b2 = (qh[:, None, :] >> (2 * c + 1)) & 1
            lo = ((qs & 15) + 16 * b1).astype(np.float32)
            hi = ((qs >> 4) + 16 * b2).astype(np.float32)
        q = np.stack([lo, hi], axis=2).reshape(nb, 8, 32)      # sub-block j = 2c (+1)
        d1 = (d * sc)[:, :, None]                               # f32 product, exact
        m1 = (dmin * mn)[:, :, None]
        prod = d1 * q
        return (prod - m1).astype(np.float32).reshape(-1)
    if t == Q6_K:
        ql = raw[:, 0:128].reshape(nb, 2, 2, 32)               # [half n][which 32-run][l]
        qh = raw[:, 128:192].reshape(nb, 2, 32)
        sc = raw[:, 192:208].view(np.int8).astype(np.float32)  # [nb,16]
        d = _f16(raw[:, 208:210])[:, None]
        out = np.empty((nb, 2, 4, 32), np.float32)
        for k in range(4):
            lo = (ql[:, :, k, :] & 15) if k < 2 else (ql[:, :, k - 2, :] >> 4)
            hi = (qh >> (2 * k)) & 3
            out[:, :, k, :] = ((lo | (hi << 4)).astype(np.int32) - 32).astype(np.float32)
        q = out.reshape(nb, 16, 16)
        ds = (d * sc)[:, :, None]
        return (ds * q).astype(np.float32).reshape(-1)
    raise ValueError(f"unsupported ggml type {t}")
