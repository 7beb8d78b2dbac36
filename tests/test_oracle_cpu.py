"""CPU tests of the oracle: pinned to the reference's golden fixtures, self-consistency, edge cases."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from oracle import np_dequant
from tests.util import FIXTURES, make_weight_f32, random_finite_blocks, reencode_codes, stored_codes

GOLDEN = Path(__file__).resolve().parent / "golden"
# per-format reconstruction bounds of dequant(expected) vs input on the fixtures (abs, rel-L2)
BOUNDS = {oracle.Q4_0: (0.12, 0.068), oracle.Q8_0: (0.0043, 0.0038), oracle.Q4_K: (0.107, 0.057),
          oracle.Q5_K: (0.045, 0.028), oracle.Q6_K: (0.036, 0.014), oracle.Q4_1: (0.065, 0.058),
          oracle.Q5_0: (0.058, 0.031), oracle.Q5_1: (0.033, 0.029), oracle.IQ4_NL: (0.079, 0.061)}


def _load(t, variant):
    name, n = FIXTURES[t]
    x = np.fromfile(GOLDEN / "ggml_quants" / f"{name}_{n}_{variant}_input.bin", dtype="<f4")
    e = np.fromfile(GOLDEN / "ggml_quants" / f"{name}_{n}_{variant}_expected.bin", dtype=np.uint8)
    return x, e, n


def test_manifest_matches():
    man = json.loads((GOLDEN / "MANIFEST.json").read_text())
    assert len(man) == 36
    for fn, sha in man.items():
        assert hashlib.sha256((GOLDEN / "ggml_quants" / fn).read_bytes()).hexdigest() == sha, fn


@pytest.mark.parametrize("t", oracle.ALL_TYPES)
@pytest.mark.parametrize("variant", ["noim", "im"])
def test_quantizer_bytes_equal_golden(t, variant):
    """The reference's own byte_cmp_noim / byte_cmp_im tests (q4_k.rs:386-403 and siblings)."""
    x, expected, n = _load(t, variant)
    im = oracle.mulberry32_imatrix(n, 2) if variant == "im" else None
    got = oracle.quantize(t, x, n, im)
    assert got.shape == expected.shape
    assert np.array_equal(got, expected)


@pytest.mark.parametrize("t", oracle.ALL_TYPES)
def test_fixture_inputs_are_mulberry32_seed1(t):
    x, _, n = _load(t, "noim")
    assert np.array_equal(x, oracle.mulberry32_uniform(2 * n, 1))


@pytest.mark.parametrize("t", oracle.ALL_TYPES)
@pytest.mark.parametrize("variant", ["noim", "im"])
def test_dequant_of_golden_reconstructs_input(t, variant):
    x, expected, _ = _load(t, variant)
    y = oracle.dequantize(t, expected)
    amax, rel = BOUNDS[t]
    assert np.abs(y - x).max() <= amax
    assert np.linalg.norm(y - x) / np.linalg.norm(x) <= rel


@pytest.mark.parametrize("t", oracle.ALL_TYPES)
def test_two_dequant_restatements_agree_bitwise(t):
    for variant in ("noim", "im"):
        _, expected, _ = _load(t, variant)
        a, b = oracle.dequantize(t, expected), np_dequant.dequantize(t, expected)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    raw = random_finite_blocks(t, 512, seed=7)
    a, b = oracle.dequantize(t, raw), np_dequant.dequantize(t, raw)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    w = oracle.quantize(t, make_weight_f32(16, 1024, seed=3), 1024)
    a, b = oracle.dequantize(t, w), np_dequant.dequantize(t, w)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("t", oracle.ALL_TYPES)
@pytest.mark.parametrize("variant", ["noim", "im"])
def test_reencoding_dequantized_golden_blocks_returns_the_stored_codes_exactly(t, variant):
    """The pin the reference's algebra gives for dequantised VALUES: its quantizers recompute the
    codes as nearest_int((x + dmin*m) / (d*sc)) (and the per-format equivalents) from the stored
    scales, so feeding the oracle's dequantised values of the reference's own golden blocks back
    through that step must reproduce every stored code, bit for bit."""
    _, expected, _ = _load(t, variant)
    for deq in (oracle.dequantize, np_dequant.dequantize):
        codes, valid = reencode_codes(t, expected, deq(t, expected))
        want = stored_codes(t, expected)
        assert valid.any()
        assert np.array_equal(codes[valid], want[valid])


@pytest.mark.parametrize("t", oracle.ALL_TYPES)
def test_reencode_identity_on_synthetic_weights(t):
    raw = oracle.quantize(t, make_weight_f32(32, 2048, seed=17), 2048)
    codes, valid = reencode_codes(t, raw, oracle.dequantize(t, raw))
    assert np.array_equal(codes[valid], stored_codes(t, raw)[valid])
    # and a wrong dequantiser would be caught: shifting every value by one step moves every code
    y = oracle.dequantize(t, raw)
    step = np.abs(y).max() / 31
    bad, _ = reencode_codes(t, raw, y + np.float32(step))
    assert not np.array_equal(bad[valid], stored_codes(t, raw)[valid])


def test_topk_order_is_total_with_nan_and_ties():
    """Ties keep the lower index first; a NaN probability ranks below every number (the
    reference's partial_cmp().unwrap_or(Equal) leaves that case open, gpu_ffn.rs:1903-1908)."""
    logits = np.array([[0.5, np.nan, 0.5, 2.0, np.nan, -1.0]], np.float32)
    ids, w = oracle.softmax_topk_renorm(logits, 5)
    assert ids.tolist() == [3, 0, 2, 5, 1]
    # the softmax denominator and the selected sum are NaN, so both guards take their fall-back
    # (1.0 and 1/topk, gpu_ffn.rs:1896, 1913-1917): weights = exp(x - max) / topk, NaN stays NaN
    ev = np.exp(logits[0, [3, 0, 2, 5]] - np.float32(2.0)).astype(np.float32)
    assert np.allclose(w[:4], ev / 5, rtol=1e-6) and np.isnan(w[4])
    masked = np.array([[-np.inf, 1.0, -np.inf, 1.0]], np.float32)
    ids, w = oracle.softmax_topk_renorm(masked, 3)
    assert ids.tolist() == [1, 3, 0] and w[2] == 0.0 and abs(w[0] - 0.5) < 1e-6
    allmasked = np.full((1, 4), -np.inf, np.float32)
    ids, _ = oracle.softmax_topk_renorm(allmasked, 2)
    assert ids.tolist() == [0, 1]                # all probabilities NaN: index order


@pytest.mark.parametrize("t", oracle.ALL_TYPES)
def test_requantizing_dequantized_values_returns_the_same_bytes_for_symmetric_formats(t):
    """Re-encode identity: dequantised values lie exactly on the grid the block stores."""
    w = make_weight_f32(8, 1024, seed=11)
    raw = oracle.quantize(t, w, 1024)
    y = oracle.dequantize(t, raw)
    y2 = oracle.dequantize(t, oracle.quantize(t, y, 1024))
    # the quantizer's scale search may pick another scale for already-quantised data, so compare
    # values: the round trip must not move any element by more than half a quantisation step
    step = np.abs(y).max() / {oracle.Q4_0: 7, oracle.Q8_0: 127, oracle.Q4_K: 15, oracle.Q5_K: 31, oracle.Q6_K: 31,
                              oracle.Q4_1: 7, oracle.Q5_0: 15, oracle.Q5_1: 15, oracle.IQ4_NL: 4}[t]
    assert np.abs(y2 - y).max() <= step


def test_nearest_int_is_round_half_even():
    # common.rs:525-539
    L = oracle.lib()
    for v, want in [(0.0, 0), (1.0, 1), (-1.0, -1), (1.4, 1), (1.6, 2), (-1.4, -1), (-1.6, -2),
                    (0.5, 0), (1.5, 2), (2.5, 2), (3.5, 4)]:
        assert L.oracle_nearest_int(v) == want


def test_f16_conversion_matches_numpy_everywhere():
    bits = np.arange(65536, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    L = oracle.lib()
    got = np.array([L.oracle_f16_to_f32(int(b)) for b in bits[::7]], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32)[~np.isnan(ref[::7])], ref[::7].view(np.uint32)[~np.isnan(ref[::7])])
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 1e3, 7e4)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(oracle.f16_round_trip(x).view(np.uint32), want.view(np.uint32))


def test_zero_blocks():
    for t in oracle.ALL_TYPES:
        raw = oracle.quantize(t, np.zeros(512, np.float32), 512)
        assert np.all(oracle.dequantize(t, raw) == 0.0)


def test_simple_q4_0_encoder_matches_reference_formula():
    # gpu_full_attn.rs:427-451
    rng = np.random.default_rng(5)
    v = rng.standard_normal(64).astype(np.float32)
    v[32:] = 0.0
    raw = oracle.encode_q4_0_simple(v).reshape(2, 18)
    d0 = raw[0, :2].view("<f2")[0]
    assert d0 == np.float16(np.abs(v[:32]).max() / np.float32(7.0))
    assert raw[1, :2].view("<f2")[0] == np.float16(1.0) and np.all(raw[1, 2:] == 0x88)
    y = oracle.dequantize(oracle.Q4_0, raw.reshape(-1))
    assert np.abs(y[:32] - v[:32]).max() <= float(d0) * 0.51 + 1e-3


def test_matmul_and_topk_semantics():
    rng = np.random.default_rng(2)
    a = rng.standard_normal((3, 64)).astype(np.float32)
    b = rng.standard_normal((5, 64)).astype(np.float32)
    got = oracle.matmul_a_by_bt(a, b)
    assert np.allclose(got, a @ b.T, rtol=1e-5, atol=1e-5)
    assert np.allclose(oracle.matmul_f64(a, b), a.astype(np.float64) @ b.T.astype(np.float64))
    logits = np.array([[0.0, 1.0, 1.0, -1.0, 0.5]], np.float32)
    ids, w = oracle.softmax_topk_renorm(logits, 3)
    assert ids.tolist() == [1, 2, 4]          # tie between 1 and 2 keeps the lower index first
    assert abs(w.sum() - 1.0) < 1e-6 and w[0] == w[1] > w[2]


def test_qmatmul_id_oracle_matches_dense_per_row():
    t, n, k, ne = oracle.Q5_K, 16, 512, 4
    w = np.concatenate([oracle.quantize(t, make_weight_f32(n, k, seed=20 + e), k) for e in range(ne)])
    stride = n * oracle.row_bytes(t, k)
    x = np.random.default_rng(1).standard_normal((3, k)).astype(np.float32)
    ids = np.array([0, 3, 1, 1, 2, 0], np.uint32)
    y = oracle.qmatmul_id(t, w, stride, x, ids, 3, 2, n, k, ne)
    for r, e in enumerate(ids):
        yd, _, _ = oracle.qmatmul(t, w[e * stride:(e + 1) * stride], x[r // 2:r // 2 + 1], n, k)
        assert np.array_equal(y[r], yd[0])


def test_ffn_oracles_match_numpy():
    rng = np.random.default_rng(0)
    seq, h, m, E, k = 3, 32, 64, 4, 2
    x = rng.standard_normal((seq, h)).astype(np.float32)
    g, u = (rng.standard_normal((m, h)) * 0.1).astype(np.float32), (rng.standard_normal((m, h)) * 0.1).astype(np.float32)
    d = (rng.standard_normal((h, m)) * 0.1).astype(np.float32)
    a, b = x @ g.T, x @ u.T
    want = ((a / (1 + np.exp(-a))) * b) @ d.T
    assert np.allclose(oracle.dense_swiglu(x, g, u, d), want, rtol=1e-4, atol=1e-5)
    router = rng.standard_normal((E, h)).astype(np.float32)
    eg = (rng.standard_normal((E, m, h)) * 0.1).astype(np.float32)
    eu = (rng.standard_normal((E, m, h)) * 0.1).astype(np.float32)
    ed = (rng.standard_normal((E, h, m)) * 0.1).astype(np.float32)
    got = oracle.moe_ffn(x, router, eg, eu, ed, k)
    ids, w = oracle.softmax_topk_renorm(x @ router.T, k)
    ref = np.zeros((seq, h), np.float32)
    for t in range(seq):
        for s in range(k):
            e = int(ids[t * k + s])
            ref[t] += w[t * k + s] * oracle.dense_swiglu(x[t:t + 1], eg[e], eu[e], ed[e])[0]
    assert np.allclose(got, ref, rtol=1e-4, atol=1e-5)
