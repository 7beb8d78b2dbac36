"""Full decoder forward on a two-layer slice: the CUDA path (embedding rows, RMSNorm, fused QKV with a
row-range type map, rotary + 8-bit KV append, attention, O, SwiGLU FFN, output head, arg-max; prefill
through the tensor-core GEMMs, decode through the mat-vec kernels from a replayed CUDA graph) against
the numpy restatement of the reference's scalar forward in oracle/llama_forward.py."""
import numpy as np
import pytest
import torch

import oracle
from oracle import llama_forward
import hf2q_b200 as hq
from hf2q_b200 import decoder as D
from tests.util import make_quant_weight, rel_l2

pytestmark = pytest.mark.gpu

# Gate on the logits: the products themselves agree with the f64 forward to ~2e-4, but K and V are
# rounded to 8-bit codes, and an element that sits next to a rounding boundary takes the neighbouring
# code when the CUDA product differs from the f64 one in its last bits; one code step is 1/127 of a
# head's range, and a few such steps per head put the logits of two layers ~5e-3 apart.
LOGIT_GATE = 2e-2

CFG = D.LlamaConfig(n_layers=2, hidden=2048, n_heads=16, n_kv_heads=4, head_dim=128, ffn=6144, vocab=4096, max_seq=512)


def build_model(ctx, cfg, seed=0):
    """Random-init weights quantized by the oracle's port of hf2q's quantizers, under the Q4_K_M type map.
    Returns (ModelWeights on the device, {name: dequantised f32 matrix} for the oracle)."""
    types = D.q4_k_m_types(cfg)
    rng = np.random.default_rng(seed)
    ref, raws = {}, {}

    def tensor(name, n, k):
        t = types[name]
        raw = make_quant_weight(t, n, k, seed=int(rng.integers(1 << 30)))
        raws[name] = (raw, t, n, k)
        ref[name] = oracle.dequantize(t, raw).reshape(n, k)

    tensor("token_embd", cfg.vocab, cfg.hidden)
    tensor("output", cfg.vocab, cfg.hidden)
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        tensor(p + "attn_q", cfg.q_rows, cfg.hidden)
        tensor(p + "attn_k", cfg.kv_rows, cfg.hidden)
        tensor(p + "attn_v", cfg.kv_rows, cfg.hidden)
        tensor(p + "attn_output", cfg.hidden, cfg.q_rows)
        tensor(p + "ffn_gate", cfg.ffn, cfg.hidden)
        tensor(p + "ffn_up", cfg.ffn, cfg.hidden)
        tensor(p + "ffn_down", cfg.hidden, cfg.ffn)
        for nm in ("attn_norm", "ffn_norm"):
            ref[p + nm] = (1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32)
    ref["out_norm"] = (1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32)

    def up(name):
        raw, t, n, k = raws[name]
        return hq.load_quant_weight(ctx, raw, t, n, k)

    def up_cat(*names):                               # row ranges of one format back to back: one tensor
        parts = [raws[nm] for nm in names]
        t, k = parts[0][1], parts[0][3]
        assert all(p[1] == t for p in parts)
        return hq.load_quant_weight(ctx, np.concatenate([p[0] for p in parts]), t, sum(p[2] for p in parts), k)

    dev = lambda name: torch.from_numpy(ref[name]).cuda()
    layers = []
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        if types[p + "attn_v"] == types[p + "attn_q"]:       # layer 0: Q, K and V share a format -> one fused tensor, one launch
            wqk, wv = up_cat(p + "attn_q", p + "attn_k", p + "attn_v"), None
        else:                                                # layer 1: the V rows are Q6_K -> a second row range
            wqk, wv = up_cat(p + "attn_q", p + "attn_k"), up(p + "attn_v")
        layers.append(D.LayerWeights(dev(p + "attn_norm"), wqk, wv, up(p + "attn_output"),
                                     dev(p + "ffn_norm"), up(p + "ffn_gate"), up(p + "ffn_up"), up(p + "ffn_down")))
    return D.ModelWeights(up("token_embd"), layers, dev("out_norm"), up("output")), ref


@pytest.fixture(scope="module")
def model(gpu_ctx):
    w, ref = build_model(gpu_ctx, CFG)
    return D.LlamaDecoder(gpu_ctx, CFG, w, prefill_chunk=32), ref


def test_type_map_follows_use_more_bits():
    full = D.LlamaConfig()
    types = D.q4_k_m_types(full)
    more = [i for i in range(32) if types[f"blk.{i}.attn_v"] == 14]
    assert more == [0, 1, 2, 3, 6, 9, 12, 15, 18, 21, 24, 27, 28, 29, 30, 31]      # 16 of 32 layers
    assert all(types[f"blk.{i}.ffn_down"] == types[f"blk.{i}.attn_v"] for i in range(32))
    assert types["output"] == 14 and types["token_embd"] == 12 and types["blk.5.attn_q"] == 12
    assert D.q4_k_m_types(CFG)["blk.0.attn_v"] == 12 and D.q4_k_m_types(CFG)["blk.1.attn_v"] == 14


def test_prompt_logits_match_the_cpu_forward(model):
    dec, ref = model
    ids = np.random.default_rng(1).integers(0, CFG.vocab, size=41).astype(np.int32)
    got = dec.forward_logits(torch.from_numpy(ids).cuda()).cpu().numpy()          # one chunk of 41 tokens (GEMM path)
    dec.ctx.check_status()
    want = llama_forward.forward(ids, ref, CFG)
    assert rel_l2(got, want) < LOGIT_GATE
    assert (got.argmax(axis=1) == want.argmax(axis=1)).mean() > 0.9


def test_chunked_prefill_and_graph_decode_match_the_cpu_forward(model):
    dec, ref = model
    rng = np.random.default_rng(2)
    ids = rng.integers(0, CFG.vocab, size=75).astype(np.int32)                    # chunks of 32, 32 and 11 tokens
    dec.prefill(torch.from_numpy(ids).cuda())
    dec.ctx.check_status()
    want = llama_forward.forward(ids, ref, CFG)
    assert rel_l2(dec.logits.cpu().numpy()[0], want[-1]) < LOGIT_GATE
    first = int(dec.tok.item())
    assert first == int(want[-1].argmax()) and int(dec.pos.item()) == 75
    # greedy continuation from the replayed graph against the oracle's greedy continuation
    n_new = 6
    toks = dec.generate(n_new, use_graph=True).cpu().numpy()
    dec.ctx.check_status()
    seq = list(ids) + [first]
    for t in range(n_new):
        lg = llama_forward.forward(np.array(seq, np.int32), ref, CFG)[-1]
        nxt = int(lg.argmax())
        top2 = np.sort(lg)[-2:]
        if toks[t] != nxt:
            assert top2[1] - top2[0] < 1e-2 * np.abs(lg).max(), (t, toks[t], nxt)   # only a near-tie may differ
            break
        seq.append(nxt)
    assert int(dec.pos.item()) == 75 + n_new
    # the same state decoded eagerly gives the same tokens as the graph
    dec.prefill(torch.from_numpy(ids).cuda())
    eager = dec.generate(n_new, use_graph=False).cpu().numpy()
    assert np.array_equal(eager, toks)
    # ... and so do the three separate attention launches (rotary + append, split attention, merge)
    dec.prefill(torch.from_numpy(ids).cuda())
    dec.fused_attention = False
    try:
        unfused = dec.generate(n_new, use_graph=False).cpu().numpy()
    finally:
        dec.fused_attention = True
    dec.ctx.check_status()
    assert np.array_equal(unfused, toks)
    # ... and the RMSNorms as launches of their own instead of inside the products
    assert dec.fused_norm
    dec.prefill(torch.from_numpy(ids).cuda())
    dec.fused_norm = False
    try:
        sep = dec.generate(n_new, use_graph=False).cpu().numpy()
    finally:
        dec.fused_norm = True
    dec.ctx.check_status()
    assert np.array_equal(sep, toks)


def test_decode_step_equals_prefill_of_the_longer_prompt(model):
    """The mat-vec / split-attention decode step and the GEMM / tiled-attention prefill see the same cache."""
    dec, _ = model
    ids = np.random.default_rng(3).integers(0, CFG.vocab, size=50).astype(np.int32)
    full = dec.forward_logits(torch.from_numpy(ids).cuda())[-1].clone()
    dec.prefill(torch.from_numpy(ids[:-1]).cuda())
    dec.tok.copy_(torch.tensor([int(ids[-1])], dtype=torch.int32))                 # force the real next token
    dec.decode_step()
    dec.ctx.check_status()
    assert rel_l2(dec.logits[0].cpu().numpy(), full.cpu().numpy()) < LOGIT_GATE
