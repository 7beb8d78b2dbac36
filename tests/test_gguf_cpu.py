"""GGUF v3 writer/reader round trips (the reference's writer tests are of the same kind,
src/backends/gguf/writer.rs:386-639): header fields, 32-byte alignment, metadata types, payload
bytes returned unchanged, rejection of malformed files."""
import struct

import numpy as np
import pytest

import oracle
from hf2q_b200 import gguf
from tests.util import make_quant_weight


def _sample(tmp_path):
    w = gguf.GgufWriter()
    w.add_kv("general.architecture", gguf.T_STRING, "llama")
    w.add_kv("llama.block_count", gguf.T_U32, 2)
    w.add_kv("llama.rope.freq_base", gguf.T_F32, 500000.0)
    w.add_kv("tokenizer.ggml.tokens", gguf.T_ARRAY, (gguf.T_STRING, ["a", "bc", ""]))
    w.add_kv("some.ints", gguf.T_ARRAY, (gguf.T_I32, [1, -2, 3]))
    t0 = make_quant_weight(oracle.Q4_K, 8, 512, seed=1)
    t1 = make_quant_weight(oracle.Q6_K, 5, 256, seed=2)                       # 1050 bytes: needs padding
    t2 = np.concatenate([make_quant_weight(oracle.Q5_K, 4, 256, seed=10 + e) for e in range(3)])
    t3 = np.arange(7, dtype=np.float32)
    w.add_tensor("blk.0.attn_q.weight", (8, 512), oracle.Q4_K, t0)
    w.add_tensor("blk.0.ffn_down.weight", (5, 256), oracle.Q6_K, t1)
    w.add_tensor("blk.0.ffn_gate_exps.weight", (3, 4, 256), oracle.Q5_K, t2)
    w.add_tensor("output_norm.weight", (7,), 0, t3)
    path = tmp_path / "m.gguf"
    w.write(path)
    return path, (t0, t1, t2, t3)


def test_round_trip_and_layout(tmp_path):
    path, (t0, t1, t2, t3) = _sample(tmp_path)
    blob = path.read_bytes()
    assert blob[:4] == b"GGUF" and struct.unpack_from("<IQQ", blob, 4) == (3, 4, 5)
    with gguf.GgufFile(path) as g:
        assert g.metadata["general.architecture"] == "llama"
        assert g.metadata["llama.block_count"] == 2
        assert g.metadata["llama.rope.freq_base"] == pytest.approx(500000.0)
        assert g.metadata["tokenizer.ggml.tokens"] == ["a", "bc", ""]
        assert g.metadata["some.ints"] == [1, -2, 3]
        q = g.tensor_info("blk.0.attn_q.weight")
        assert q.shape == (8, 512) and q.ggml_type == oracle.Q4_K and q.nbytes == 8 * 2 * 144
        e = g.tensor_info("blk.0.ffn_gate_exps.weight")
        assert e.shape == (3, 4, 256) and e.nbytes == 3 * 4 * 176
        for ti in g.tensors.values():
            assert ti.offset % 32 == 0                                           # ALIGNMENT, types.rs:31
        assert np.array_equal(g.load_tensor("blk.0.attn_q.weight"), t0)
        assert np.array_equal(g.load_tensor("blk.0.ffn_down.weight"), t1)
        assert np.array_equal(g.load_tensor("blk.0.ffn_gate_exps.weight"), t2)
        assert np.array_equal(g.load_tensor("output_norm.weight").view(np.float32), t3)
    assert len(blob) % 32 == 0


def test_rejects_bad_files(tmp_path):
    path, _ = _sample(tmp_path)
    blob = bytearray(path.read_bytes())
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + blob[4:])
    with pytest.raises(ValueError):
        gguf.GgufFile(bad)
    bad.write_bytes(blob[:4] + struct.pack("<I", 2) + blob[8:])
    with pytest.raises(ValueError):
        gguf.GgufFile(bad)
    bad.write_bytes(blob[: len(blob) - 64])                                      # truncated payload
    with pytest.raises(ValueError):
        gguf.GgufFile(bad)
    w = gguf.GgufWriter()
    with pytest.raises(ValueError):
        w.add_tensor("x", (2, 256), oracle.Q4_K, np.zeros(10, np.uint8))          # wrong payload size
    with pytest.raises(ValueError):
        w.add_tensor("x", (2, 100), oracle.Q4_K, np.zeros(10, np.uint8))          # not a whole block
