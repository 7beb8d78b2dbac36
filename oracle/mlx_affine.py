"""CPU restatement of hf2q's mlx-affine (DWQ) 4-bit / group-32 weight path.  TEST INFRASTRUCTURE.

The kernel itself (``dispatch_qmm_affine_t_packed_simd4_b4``) lives in the mlx-native crate, which is not part of
the hf2q tree; what hf2q holds, and what this file follows, is
  * the packing of unpacked codes into u32 words, MlxQWeight::from_mlx_affine_linear
    (src/serve/forward_mlx.rs:452-466: element j of a word in bits 4 j .., "low nibble at slot 0"),
  * the layout of the three arrays, MlxAffineExtra (forward_mlx.rs:340-360: codes u32 [N, K/8], scales and
    biases f32 [N, K/32]),
  * the scalar specification its tests check the kernel against,
    y[r, col] = sum_k x[r, k] * (q[col, k] * scale[col, g] + bias[col, g])   (forward_mlx.rs:8886-8901, f64),
    with the bar max |y - spec| < 1e-3, and the deterministic synthetic inputs of that test (:8803-8812, :8837-8839).
Parity of the values: "parity unpinned" in the sense that the reference holds no stored output vector for this
path; the spec above is its own oracle and is what the tests here evaluate.
"""
from __future__ import annotations

import numpy as np

MLX_AFFINE4_GS32 = 1000
GROUP, BLOCK_BYTES = 32, 24


def pack_codes(q_int: np.ndarray) -> np.ndarray:
    """u8 codes [n, k] (values 0..15) -> u32 [n, k / 8], element j of a word in bits 4 j .. (forward_mlx.rs:455-466)."""
    q = np.ascontiguousarray(q_int, dtype=np.uint32)
    n, k = q.shape
    q = q.reshape(n, k // 8, 8)
    return (q << (4 * np.arange(8, dtype=np.uint32))[None, None, :]).sum(axis=2, dtype=np.uint32)


def to_blocks(codes: np.ndarray, scales: np.ndarray, biases: np.ndarray) -> np.ndarray:
    """The 24-byte container hf2q_cuda_affine_pack writes: per group f32 scale, f32 bias, the group's four code words."""
    n, kp = codes.shape
    groups = kp // 4
    out = np.empty((n, groups, 6), np.uint32)
    out[:, :, 0] = np.ascontiguousarray(scales, dtype=np.float32).view(np.uint32).reshape(n, groups)
    out[:, :, 1] = np.ascontiguousarray(biases, dtype=np.float32).view(np.uint32).reshape(n, groups)
    out[:, :, 2:] = np.ascontiguousarray(codes, dtype=np.uint32).reshape(n, groups, 4)
    return out.view(np.uint8).reshape(-1)


def dequantize_blocks(blocks: np.ndarray) -> np.ndarray:
    """f32 values of the container's elements: scale * code + bias, each operation rounded to f32."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, BLOCK_BYTES)
    sc = b[:, 0:4].copy().view(np.float32)
    bi = b[:, 4:8].copy().view(np.float32)
    qs = b[:, 8:24]
    q = np.stack([qs & 15, qs >> 4], axis=2).reshape(-1, GROUP).astype(np.float32)    # element e = nibble e
    prod = (sc * q).astype(np.float32)
    return (prod + bi).astype(np.float32).reshape(-1)


def qmm_affine_f64(x: np.ndarray, q_int: np.ndarray, scales: np.ndarray, biases: np.ndarray) -> np.ndarray:
    """The reference tests' CPU oracle (forward_mlx.rs:8886-8901): f64 accumulation of x * (q * s + b)."""
    n, k = q_int.shape
    w = q_int.astype(np.float64).reshape(n, k // GROUP, GROUP) * scales.astype(np.float64).reshape(n, -1, 1) + \
        biases.astype(np.float64).reshape(n, -1, 1)
    return x.astype(np.float64) @ w.reshape(n, k).T


def reference_vector(m: int, n: int, k: int):
    """The deterministic synthetic linear and activations of from_mlx_affine_linear_roundtrips_through_packed_kernel
    (forward_mlx.rs:8803-8812, 8837-8839), evaluated in f32 as the Rust test does."""
    groups = k // GROUP
    i = np.arange(n * k, dtype=np.int64)
    q_int = ((i * 11 + 5) % 16).astype(np.uint8).reshape(n, k)
    gi = np.arange(n * groups, dtype=np.float32)
    scales = (np.float32(0.05) + gi * np.float32(0.0017)).astype(np.float32).reshape(n, groups)
    biases = (np.float32(-0.13) + gi * np.float32(0.0023)).astype(np.float32).reshape(n, groups)
    xi = np.arange(m * k, dtype=np.float32)
    x = (np.sin((xi * np.float32(0.013) - np.float32(0.4)).astype(np.float32)).astype(np.float32) * np.float32(0.6)).astype(np.float32)
    return q_int, scales, biases, x.reshape(m, k)
