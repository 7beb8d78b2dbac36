"""Sharding rules of the tensor-parallel decoder (host logic only: byte slicing of quantized tensors)."""
import numpy as np

import oracle
from hf2q_b200 import decoder as D, decoder_tp as TP


def test_column_shard_is_the_quantisation_of_the_column_slice():
    """Blocks are independent along k, so a column shard (whole blocks of every row) of a quantized tensor is
    exactly the quantized column slice; a row shard is a byte range."""
    cfg = D.LlamaConfig(n_layers=1, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=256, max_seq=16)
    rng = np.random.default_rng(0)
    for t in (oracle.Q4_K, oracle.Q6_K, oracle.Q8_0):
        n, k, world = 24, 2048, 2
        x = (rng.standard_normal((n, k)) * 0.02).astype(np.float16).astype(np.float32)
        raw = oracle.quantize(t, x, k)
        for rank in range(world):
            got, rows, cols = TP.shard_raw("blk.0.attn_output", raw, t, n, k, cfg, rank, world)
            if TP.column_shard_ok(t, k, world):
                want = oracle.quantize(t, np.ascontiguousarray(x[:, rank * k // world:(rank + 1) * k // world]), k // world)
                assert (rows, cols) == (n, k // world) and np.array_equal(got, want), (t, rank)
            else:                                              # falls back to a row shard
                rb = oracle.row_bytes(t, k)
                assert (rows, cols) == (n // world, k)
                assert np.array_equal(got, raw.reshape(n, rb)[rank * n // world:(rank + 1) * n // world].reshape(-1))
            got, rows, cols = TP.shard_raw("blk.0.ffn_gate", raw, t, n, k, cfg, rank, world)
            rb = oracle.row_bytes(t, k)
            assert (rows, cols) == (n // world, k)
            assert np.array_equal(got, raw.reshape(n, rb)[rank * n // world:(rank + 1) * n // world].reshape(-1))
    got, rows, cols = TP.shard_raw("token_embd", raw, t, n, k, cfg, 1, 2)
    assert (rows, cols) == (n, k) and np.array_equal(got, raw)


def test_alignment_rule_on_the_llama_shapes():
    """Q4_K column shards stay 16-byte aligned at 2, 4 and 8 ranks; Q6_K rows (210-byte blocks) only in multiples of
    eight blocks, which no even split of ffn = 14336 = 7 x 2048 gives: those down tensors are sharded by rows."""
    for w in (2, 4, 8):
        assert TP.column_shard_ok(oracle.Q4_K, 4096, w) and TP.column_shard_ok(oracle.Q4_K, 14336, w)
        assert not TP.column_shard_ok(oracle.Q6_K, 14336, w)
    assert TP.column_shard_ok(oracle.Q6_K, 4096, 2) and not TP.column_shard_ok(oracle.Q6_K, 4096, 4)
    assert not TP.column_shard_ok(oracle.Q4_K, 4096, 3)        # not a whole number of blocks per rank
