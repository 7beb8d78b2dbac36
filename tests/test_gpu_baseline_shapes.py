"""Parity at the sizes the benchmarks time (the five workload configurations' real shapes).

The small-shape sweeps in test_gpu_parity.py cover every format and edge; these cover the code
paths that only full-size launches reach: k-phases (4096 x 14336 with 4 and 8 activation rows),
the 2-D tensor-copy staging with 13 row groups per CTA (28672 x 4096), 256-token GEMM tiles, and
the grouped expert product with 256 experts and several weight-row tiles per CTA.  The checker is
the CPU oracle: an f64 product on the oracle's dequantised weights, gate 1e-3 relative L2.  Where
the full f64 product would take minutes on the host, a fixed sample of activation rows (tokens) or
routed rows is checked against all output columns.
"""
import numpy as np
import pytest
import torch

import oracle
import hf2q_b200 as hq
from tests.util import bf16_bits_to_f32, make_quant_weight, make_x, rel_l2, to_bf16_bits

pytestmark = pytest.mark.gpu
GATE = 1e-3

DECODE_SHAPES = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]      # (n, k)


def _x_bf16(m, k, seed):
    bits = to_bf16_bits(make_x(m, k, seed=seed))
    dev = torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(m, k)
    return dev, bf16_bits_to_f32(bits).reshape(m, k)


_cache = {}


def _weight(t, n, k, seed):
    key = (t, n, k, seed)
    if key not in _cache:
        raw = make_quant_weight(t, n, k, seed=seed)
        _cache.clear()                       # one big matrix on the host at a time
        _cache[key] = (raw, oracle.dequantize(t, raw).reshape(n, k))
    return _cache[key]


@pytest.mark.parametrize("n,k", DECODE_SHAPES)
def test_q6k_decode_sweep_full_size(gpu_ctx, n, k):
    """Workload 2: Q6_K, bf16 activations, 1 / 4 / 8 tokens, every output checked."""
    raw, wref = _weight(oracle.Q6_K, n, k, seed=n + k)
    w = hq.load_quant_weight(gpu_ctx, raw, oracle.Q6_K, n, k)
    for m in (1, 4, 8):
        xd, xs = _x_bf16(m, k, seed=50 + m)
        y = torch.full((m, n), float("nan"), device="cuda")
        hq.quantized_matmul_ggml(gpu_ctx, xd, w, y, w.matmul_params(m))
        gpu_ctx.check_status()
        err = rel_l2(y.cpu().numpy(), oracle.matmul_f64(xs, wref))
        assert err < GATE, (n, k, m, err)
        assert err < 1e-4, (n, k, m, err)        # measured ~1e-5; a coarse regression bound


def test_q4k_single_matrix_f32_activations(gpu_ctx):
    """Workload 1 at the size of the sweep's other formats: Q4_K 4096 x 14336 (phased with f32 x)."""
    n, k = 4096, 14336
    raw, wref = _weight(oracle.Q4_K, n, k, seed=5)
    w = hq.load_quant_weight(gpu_ctx, raw, oracle.Q4_K, n, k)
    for m in (1, 3):
        x = make_x(m, k, seed=60 + m)
        y = torch.full((m, n), float("nan"), device="cuda")
        hq.quantized_matmul_ggml(gpu_ctx, torch.from_numpy(x).cuda(), w, y, w.matmul_params(m))
        gpu_ctx.check_status()
        assert rel_l2(y.cpu().numpy(), oracle.matmul_f64(x, wref)) < GATE


def _sample_tokens(m, count, seed):
    rng = np.random.default_rng(seed)
    pick = set(rng.choice(m, size=min(count, m), replace=False).tolist())
    pick.update({0, m - 1, 255, 256} & set(range(m)))       # tile borders
    return np.array(sorted(pick))


@pytest.mark.parametrize("t,n,k,m", [(oracle.Q4_K, 6144, 4096, 512), (oracle.Q6_K, 4096, 14336, 512),
                                     (oracle.Q4_K, 4096, 4096, 2048), (oracle.Q6_K, 4096, 14336, 2048)])
def test_prefill_gemm_full_size(gpu_ctx, t, n, k, m):
    """Workload 3: tensor-core GEMM at 512 and 2048 tokens; 40 sampled tokens x all n outputs in f64."""
    raw, wref = _weight(t, n, k, seed=n + k + 1)
    w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
    xd, xs = _x_bf16(m, k, seed=70)
    y = torch.full((m, n), float("nan"), device="cuda")
    hq.quantized_matmul_ggml(gpu_ctx, xd, w, y, w.matmul_params(m))
    gpu_ctx.check_status()
    assert not torch.isnan(y).any()
    rows = _sample_tokens(m, 40, seed=m)
    err = rel_l2(y[torch.from_numpy(rows).cuda()].cpu().numpy(), oracle.matmul_f64(xs[rows], wref))
    assert err < GATE, (t, n, k, m, err)


def _expert_layer(distinct=16):
    """Workload 4's stacked expert tensors: 256 experts, hidden 2048, intermediate 512, Q5_K.
    Quantising 805 M weights on the host would take minutes, so `distinct` experts are quantised and
    repeated 256 / distinct times; the kernels cannot tell (they index by expert)."""
    E, H, I, t = 256, 2048, 512, oracle.Q5_K
    gate = [make_quant_weight(t, I, H, seed=300 + e) for e in range(distinct)]
    up = [make_quant_weight(t, I, H, seed=400 + e) for e in range(distinct)]
    down = [make_quant_weight(t, H, I, seed=500 + e) for e in range(distinct)]
    rep = E // distinct
    stack = lambda parts: np.concatenate(parts * rep)       # expert e holds the bytes of expert e % distinct
    return E, H, I, t, gate, up, down, stack(gate), stack(up), stack(down)


@pytest.mark.parametrize("T", [1, 2048])
def test_moe_mul_mat_id_full_size(gpu_ctx, T):
    """Workload 4: top-8 of 256 experts from the device router, gate/up pair and down products."""
    E, H, I, t, gate, up, down, wg, wu, wd = _expert_layer()
    distinct = len(gate)
    topk = 8
    R = T * topk
    wgd, wud, wdd = (torch.from_numpy(a).cuda() for a in (wg, wu, wd))
    logits = np.random.default_rng(9).standard_normal((T, E)).astype(np.float32)
    ids, wts = hq.moe_softmax_topk(gpu_ctx, torch.from_numpy(logits).cuda(), topk)
    ids_h = ids.cpu().numpy().astype(np.uint32)
    want_ids, want_w = oracle.softmax_topk_renorm(logits, topk)
    assert np.array_equal(ids_h, want_ids)
    assert np.allclose(wts.cpu().numpy(), want_w, rtol=1e-5, atol=1e-7)
    xd, xs = _x_bf16(T, H, seed=80)
    sg, sd = hq.expert_stride(t, I, H), hq.expert_stride(t, H, I)
    scratch = hq.IdMmScratch.alloc(gpu_ctx, E, R, H)
    g = torch.full((R, I), float("nan"), device="cuda")
    u = torch.full((R, I), float("nan"), device="cuda")
    hq.quantized_matmul_id_pair_ggml(gpu_ctx, xd, wgd.data_ptr(), wud.data_ptr(), ids, g, u, scratch,
                                     hq.GgmlQuantizedMatmulIdParams(T, topk, I, H, E, sg, t))
    act_bits = to_bf16_bits(make_x(R, I, seed=81))
    act = torch.from_numpy(act_bits.view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(R, I)
    act_f = bf16_bits_to_f32(act_bits).reshape(R, I)
    d = torch.full((R, H), float("nan"), device="cuda")
    hq.quantized_matmul_id_ggml(gpu_ctx, act, wdd.data_ptr(), ids, d, scratch,
                                hq.GgmlQuantizedMatmulIdParams(R, 1, H, I, E, sd, t))
    gpu_ctx.check_status()
    for out in (g, u, d):
        assert not torch.isnan(out).any()
    rows = np.arange(R) if R <= 64 else np.unique(np.concatenate([np.random.default_rng(3).choice(R, 192, replace=False), [0, R - 1]]))
    gh, uh, dh = g.cpu().numpy(), u.cpu().numpy(), d.cpu().numpy()
    deq = {}

    def wmat(kind, parts, e, shape):
        key = (kind, e % distinct)
        if key not in deq:
            deq[key] = oracle.dequantize(t, parts[e % distinct]).reshape(shape)
        return deq[key]

    got_g, got_u, got_d, ref_g, ref_u, ref_d = [], [], [], [], [], []
    for r in rows:
        e = int(ids_h[r])
        tok = r // topk
        ref_g.append(oracle.matmul_f64(xs[tok:tok + 1], wmat("g", gate, e, (I, H)))[0])
        ref_u.append(oracle.matmul_f64(xs[tok:tok + 1], wmat("u", up, e, (I, H)))[0])
        ref_d.append(oracle.matmul_f64(act_f[r:r + 1], wmat("d", down, e, (H, I)))[0])
        got_g.append(gh[r]); got_u.append(uh[r]); got_d.append(dh[r])
    for got, ref, name in ((got_g, ref_g, "gate"), (got_u, ref_u, "up"), (got_d, ref_d, "down")):
        err = rel_l2(np.stack(got), np.stack(ref))
        assert err < GATE, (name, T, err)


def test_router_with_masked_experts(gpu_ctx):
    """Rows with some logits at -inf (masked experts): valid ids, masked experts last, finite weights."""
    rng = np.random.default_rng(4)
    logits = rng.standard_normal((64, 256)).astype(np.float32)
    logits[:, ::3] = -np.inf
    logits[5, :] = -np.inf
    logits[5, 17] = 0.25                        # a single live expert, top-8 asked for
    ids, w = hq.moe_softmax_topk(gpu_ctx, torch.from_numpy(logits).cuda(), 8)
    gpu_ctx.check_status()
    want_ids, want_w = oracle.softmax_topk_renorm(logits, 8)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), want_ids)
    assert ids.max().item() < 256
    assert np.allclose(w.cpu().numpy(), want_w, rtol=1e-5, atol=1e-7)
