"""mlx-affine 4-bit / group-32: the oracle's packing and container against the reference's own formulas (CPU)."""
import numpy as np

from oracle import mlx_affine as A


def test_packing_puts_element_j_in_nibble_j():
    q = (np.arange(2 * 16) % 16).astype(np.uint8).reshape(2, 16)
    w = A.pack_codes(q)
    assert w.shape == (2, 2) and w.dtype == np.uint32
    assert w[0, 0] == 0x76543210 and w[0, 1] == 0xFEDCBA98                  # "low nibble at slot 0"
    for j in range(8):
        assert (int(w[1, 0]) >> (4 * j)) & 15 == q[1, j]


def test_container_round_trip_and_spec():
    q, s, b, x = A.reference_vector(16, 64, 96)
    blocks = A.to_blocks(A.pack_codes(q), s, b)
    assert blocks.size == 64 * 3 * 24
    w = A.dequantize_blocks(blocks).reshape(64, 96)
    want = q.astype(np.float32).reshape(64, 3, 32) * s[:, :, None] + b[:, :, None]
    assert np.array_equal(w, want.astype(np.float32).reshape(64, 96))
    # the reference test's bar: max |y - f64 spec| < 1e-3 (forward_mlx.rs:8903-8913)
    y = (x.astype(np.float32) @ w.T).astype(np.float32)
    assert np.abs(y - A.qmm_affine_f64(x, q, s, b)).max() < 1e-3
    assert q[0, :4].tolist() == [5, 0, 11, 6] and abs(float(s[0, 1]) - 0.0517) < 1e-6       # (i * 11 + 5) % 16; 0.05 + i * 0.0017
