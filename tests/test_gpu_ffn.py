"""FFN builders on quantized weights against the reference's scalar specs (dense_swiglu_cpu_ref,
moe_ffn_cpu_ref) evaluated by the oracle on the dequantised weights.  The reference's own bar for
quantized FFN parity is max-abs < 2e-2 (gpu_ffn.rs:3599-3720); relative L2 is checked as well."""
import numpy as np
import pytest
import torch

import oracle
import hf2q_b200 as hq
from hf2q_b200 import ffn
from tests.util import make_quant_weight, make_x, rel_l2

pytestmark = pytest.mark.gpu


def _qw(ctx, t, n, k, seed):
    raw = make_quant_weight(t, n, k, seed=seed)
    return hq.load_quant_weight(ctx, raw, t, n, k), oracle.dequantize(t, raw).reshape(n, k)


@pytest.mark.parametrize("t", [oracle.Q4_0, oracle.Q4_K, oracle.Q6_K])
@pytest.mark.parametrize("m", [1, 5, 40])
def test_dense_ffn_builder(gpu_ctx, t, m):
    hidden, inter = 512, 1024
    gq, gf = _qw(gpu_ctx, t, inter, hidden, 1)
    uq, uf = _qw(gpu_ctx, t, inter, hidden, 2)
    dq, df = _qw(gpu_ctx, t, hidden, inter, 3)
    x = make_x(m, hidden, seed=4)
    res = make_x(m, hidden, seed=5)
    y = ffn.build_dense_ffn_layer_gpu_q(gpu_ctx, torch.from_numpy(x).cuda(), ffn.DenseFfnWeightsGpuQ(gq, uq, dq),
                                        residual=torch.from_numpy(res).cuda())
    gpu_ctx.check_status()
    want = oracle.dense_swiglu(x, gf, uf, df) + res
    got = y.cpu().numpy()
    assert np.abs(got - want).max() < 2e-2
    assert rel_l2(got - res, want - res) < 3e-3


@pytest.mark.parametrize("t", list(oracle.MAIN_TYPES))
@pytest.mark.parametrize("bf16", [False, True])
def test_dense_ffn_fused_launches_equal_the_separate_ops(gpu_ctx, t, bf16):
    """gate/up with the SwiGLU epilogue and down with the residual epilogue: the same arithmetic in the
    same order as gate, up, silu_mul, down, add -- bit-identical outputs, and close to the oracle."""
    from hf2q_b200 import ops
    hidden, inter = 2048, 1536 + 48                   # inter: a partial last row group of the gate/up tensors
    gq, gf = _qw(gpu_ctx, t, inter, hidden, 21)
    uq, uf = _qw(gpu_ctx, t, inter, hidden, 22)
    dq, df = _qw(gpu_ctx, t, hidden, 2048, 23)
    for m in (1, 3, 4) + ((8,) if bf16 else ()):
        x = make_x(m, hidden, seed=30 + m)
        xd = torch.from_numpy(x).cuda()
        if bf16:
            xd = xd.bfloat16()
            x = xd.float().cpu().numpy()
        assert ops.quantized_matmul_swiglu_supported(gpu_ctx, m, gq, xd.dtype)
        a = torch.empty((m, inter), device="cuda")
        b = torch.empty_like(a)
        ops.quantized_matmul_ggml(gpu_ctx, xd, gq, a, gq.matmul_params(m))
        ops.quantized_matmul_ggml(gpu_ctx, xd, uq, b, uq.matmul_params(m))
        sep = ffn._silu_mul(gpu_ctx, a, b)
        fused = torch.full((m, inter), float("nan"), device="cuda")
        ops.quantized_matmul_swiglu(gpu_ctx, xd, gq, uq, fused, m)
        gpu_ctx.check_status()
        assert torch.equal(fused, sep), (t, m)
        g64, u64 = x.astype(np.float64) @ gf.T.astype(np.float64), x.astype(np.float64) @ uf.T.astype(np.float64)
        want = g64 / (1.0 + np.exp(-g64)) * u64
        assert rel_l2(fused.cpu().numpy(), want) < 1e-3
        # down + residual (in place: the residual stream is updated where it lives)
        c = torch.from_numpy(make_x(m, 2048, seed=40 + m)).cuda()
        res = torch.from_numpy(make_x(m, hidden, seed=50 + m)).cuda()
        y = torch.empty((m, hidden), device="cuda")
        ops.quantized_matmul_ggml(gpu_ctx, c, dq, y, dq.matmul_params(m))
        want_y = y + res
        got = res.clone()
        ops.quantized_matmul_add(gpu_ctx, c, dq, got, got, m)
        gpu_ctx.check_status()
        assert torch.equal(got, want_y), (t, m)


def test_swiglu_fusion_declines_what_does_not_fit_one_launch(gpu_ctx):
    from hf2q_b200 import ops
    # the 32-element fall-back formats have no fused form; the builder then issues the separate ops
    for tf in (oracle.Q4_1, oracle.Q5_0, oracle.Q5_1, oracle.IQ4_NL):
        wf = hq.load_quant_weight(gpu_ctx, make_quant_weight(tf, 32, 2048, seed=tf), tf, 32, 2048)
        assert not ops.quantized_matmul_swiglu_supported(gpu_ctx, 1, wf, torch.bfloat16)
        assert not ops.quantized_matmul_add_supported(gpu_ctx, wf, torch.float32)
    t = oracle.Q6_K
    long_rows = hq.load_quant_weight(gpu_ctx, make_quant_weight(t, 32, 14336, seed=1), t, 32, 14336)
    assert ops.quantized_matmul_swiglu_supported(gpu_ctx, 1, long_rows, torch.bfloat16)
    assert not ops.quantized_matmul_swiglu_supported(gpu_ctx, 8, long_rows, torch.bfloat16)      # k-phases
    assert not ops.quantized_matmul_swiglu_supported(gpu_ctx, 5, long_rows, torch.float32)       # more than 4 f32 rows
    short_rows = hq.load_quant_weight(gpu_ctx, make_quant_weight(t, 32, 512, seed=2), t, 32, 512)
    assert not ops.quantized_matmul_swiglu_supported(gpu_ctx, 1, short_rows, torch.bfloat16)     # stacked row groups
    x = torch.zeros((8, 14336), device="cuda", dtype=torch.bfloat16)
    y = torch.empty((8, 32), device="cuda")
    with pytest.raises(hq.Hf2qError):
        ops.quantized_matmul_swiglu(gpu_ctx, x, long_rows, long_rows, y, 8)


@pytest.mark.parametrize("t", [oracle.Q4_0, oracle.Q5_K, oracle.Q6_K])
@pytest.mark.parametrize("bf16", [False, True])
def test_routed_swiglu_launch_equals_pair_plus_silu_mul(gpu_ctx, t, bf16):
    from hf2q_b200 import ops
    hidden, inter, E, top_k = 2048, 256 + 16, 6, 3
    stride = hq.expert_stride(t, inter, hidden)
    gate = torch.from_numpy(np.concatenate([make_quant_weight(t, inter, hidden, seed=60 + e) for e in range(E)])).cuda()
    up = torch.from_numpy(np.concatenate([make_quant_weight(t, inter, hidden, seed=70 + e) for e in range(E)])).cuda()
    for T in (1, 4):
        x = torch.from_numpy(make_x(T, hidden, seed=80 + T)).cuda()
        if bf16:
            x = x.bfloat16()
        rng = np.random.default_rng(T)
        ids = torch.from_numpy(np.stack([rng.permutation(E)[:top_k] for _ in range(T)]).astype(np.int32).reshape(-1)).cuda()
        p = hq.GgmlQuantizedMatmulIdParams(T, top_k, inter, hidden, E, stride, t)
        assert ops.quantized_matmul_id_swiglu_supported(gpu_ctx, p, x.dtype)
        g = torch.empty((T * top_k, inter), device="cuda")
        u = torch.empty_like(g)
        hq.quantized_matmul_id_pair_ggml(gpu_ctx, x, gate.data_ptr(), up.data_ptr(), ids, g, u, None, p)
        sep = ffn._silu_mul(gpu_ctx, g, u)
        fused = torch.full((T * top_k, inter), float("nan"), device="cuda")
        ops.quantized_matmul_id_swiglu_ggml(gpu_ctx, x, gate.data_ptr(), up.data_ptr(), ids, fused, p)
        gpu_ctx.check_status()
        assert torch.equal(fused, sep), (t, T)
    # an expert index out of range: that row is zero-filled and the status word says so
    bad = ids.clone()
    bad[1] = E
    ops.quantized_matmul_id_swiglu_ggml(gpu_ctx, x, gate.data_ptr(), up.data_ptr(), bad, fused, p)
    with pytest.raises(hq.Hf2qError):
        gpu_ctx.check_status()
    assert torch.count_nonzero(fused[1]) == 0 and torch.equal(fused[0], sep[0])
    big = hq.GgmlQuantizedMatmulIdParams(64, top_k, inter, hidden, E, stride, t)
    assert not ops.quantized_matmul_id_swiglu_supported(gpu_ctx, big, x.dtype)       # many rows: the grouped GEMM's job


@pytest.mark.parametrize("T", [1, 3, 70])
def test_moe_ffn_builder(gpu_ctx, T):
    t, hidden, inter, E, k, m_sh = oracle.Q5_K, 512, 256, 8, 2, 256
    rng = np.random.default_rng(7)
    eg_raw = np.concatenate([make_quant_weight(t, inter, hidden, seed=100 + e) for e in range(E)])
    eu_raw = np.concatenate([make_quant_weight(t, inter, hidden, seed=200 + e) for e in range(E)])
    ed_raw = np.concatenate([make_quant_weight(t, hidden, inter, seed=300 + e) for e in range(E)])
    router = (rng.standard_normal((E, hidden)) * 0.05).astype(np.float32)
    sgq, sgf = _qw(gpu_ctx, t, m_sh, hidden, 11)
    suq, suf = _qw(gpu_ctx, t, m_sh, hidden, 12)
    sdq, sdf = _qw(gpu_ctx, t, hidden, m_sh, 13)
    sl = (rng.standard_normal(hidden) * 0.05).astype(np.float32)
    w = ffn.MoeFfnWeightsGpuQ(router=torch.from_numpy(router).cuda(), expert_gate=torch.from_numpy(eg_raw).cuda(),
                              expert_up=torch.from_numpy(eu_raw).cuda(), expert_down=torch.from_numpy(ed_raw).cuda(),
                              ggml_type_gate_up=t, ggml_type_down=t, num_experts=E, num_experts_per_tok=k,
                              moe_intermediate_size=inter, shared=ffn.DenseFfnWeightsGpuQ(sgq, suq, sdq),
                              shared_gate_logit=torch.from_numpy(sl).cuda())
    x = make_x(T, hidden, seed=21)
    y = ffn.build_moe_ffn_layer_gpu_q(gpu_ctx, torch.from_numpy(x).cuda(), w)
    gpu_ctx.check_status()
    egf = oracle.dequantize(t, eg_raw).reshape(E, inter, hidden)
    euf = oracle.dequantize(t, eu_raw).reshape(E, inter, hidden)
    edf = oracle.dequantize(t, ed_raw).reshape(E, hidden, inter)
    want = oracle.moe_ffn(x, router, egf, euf, edf, k, shared=(sl, sgf, suf, sdf))
    got = y.cpu().numpy()
    assert np.abs(got - want).max() < 2e-2
    assert rel_l2(got, want) < 3e-3


@pytest.mark.parametrize("t", list(oracle.MAIN_TYPES))
def test_dense_ffn_gemm_forms_equal_the_separate_ops(gpu_ctx, t):
    """More than 8 rows: gate and up tiles side by side in tensor memory with the SwiGLU in the epilogue, and the
    residual added in the GEMM's epilogue -- the same tensor-core accumulation as the separate products, so the
    outputs are bit-identical to gate, up, silu_mul / down, add."""
    from hf2q_b200 import ops
    hidden, inter = 2048, 1536 + 48                   # inter: a partial last 64-row tile
    gq, gf = _qw(gpu_ctx, t, inter, hidden, 21)
    uq, uf = _qw(gpu_ctx, t, inter, hidden, 22)
    dq, _ = _qw(gpu_ctx, t, hidden, 2048, 23)
    for m, bf16 in ((9, False), (70, True), (200, False), (333, True)):
        x = make_x(m, hidden, seed=30 + m)
        xd = torch.from_numpy(x).cuda()
        if bf16:
            xd = xd.bfloat16()
            x = xd.float().cpu().numpy()
        assert ops.quantized_matmul_swiglu_supported(gpu_ctx, m, gq, xd.dtype)
        a = torch.empty((m, inter), device="cuda")
        b = torch.empty_like(a)
        ops.quantized_matmul_ggml(gpu_ctx, xd, gq, a, gq.matmul_params(m))
        ops.quantized_matmul_ggml(gpu_ctx, xd, uq, b, uq.matmul_params(m))
        sep = ffn._silu_mul(gpu_ctx, a, b)
        fused = torch.full((m, inter), float("nan"), device="cuda")
        n0 = gpu_ctx.launch_count
        ops.quantized_matmul_swiglu(gpu_ctx, xd, gq, uq, fused, m)
        assert gpu_ctx.launch_count - n0 == 2              # activation conversion + the one GEMM
        gpu_ctx.check_status()
        assert torch.equal(fused, sep), (t, m)
        g64, u64 = x.astype(np.float64) @ gf.T.astype(np.float64), x.astype(np.float64) @ uf.T.astype(np.float64)
        assert rel_l2(fused.cpu().numpy(), g64 / (1.0 + np.exp(-g64)) * u64) < 2e-3
        c = torch.from_numpy(make_x(m, 2048, seed=40 + m)).cuda()
        res = torch.from_numpy(make_x(m, hidden, seed=50 + m)).cuda()
        assert ops.quantized_matmul_add_supported(gpu_ctx, dq, c.dtype, m)
        y = torch.empty((m, hidden), device="cuda")
        ops.quantized_matmul_ggml(gpu_ctx, c, dq, y, dq.matmul_params(m))
        want_y = y + res
        got = res.clone()
        ops.quantized_matmul_add(gpu_ctx, c, dq, got, got, m)         # in place on the residual stream
        gpu_ctx.check_status()
        assert torch.equal(got, want_y), (t, m)
    # the 32-element fall-back formats have the residual form but not the pair
    wf = hq.load_quant_weight(gpu_ctx, make_quant_weight(oracle.Q5_0, 64, 2048, seed=3), oracle.Q5_0, 64, 2048)
    assert not ops.quantized_matmul_swiglu_supported(gpu_ctx, 40, wf, torch.float32)
    assert ops.quantized_matmul_add_supported(gpu_ctx, wf, torch.float32, 40)
    with pytest.raises(hq.Hf2qError):
        ops.quantized_matmul_swiglu(gpu_ctx, torch.zeros((40, 2048), device="cuda"), wf, wf, torch.empty((40, 64), device="cuda"), 40)


@pytest.mark.parametrize("tg,td", [(oracle.Q4_K, oracle.Q6_K), (oracle.Q4_0, oracle.Q8_0), (oracle.Q5_K, oracle.Q5_1)])
def test_moe_experts_equals_the_separate_ops(gpu_ctx, tg, td):
    """Sort + gather, gate/up pair with the SwiGLU epilogue writing the sorted f16 panel, down reading it:
    bit-identical to mul_mat_id (gate), (up), silu_mul, mul_mat_id (down)."""
    from hf2q_b200 import ops
    hidden, inter, E, top_k = 2048, 2048, 7, 3            # Q6_K rows are 16-byte aligned from 2048 elements on
    sg, sd = hq.expert_stride(tg, inter, hidden), hq.expert_stride(td, hidden, inter)
    gate = torch.from_numpy(np.concatenate([make_quant_weight(tg, inter, hidden, seed=60 + e) for e in range(E)])).cuda()
    up = torch.from_numpy(np.concatenate([make_quant_weight(tg, inter, hidden, seed=70 + e) for e in range(E)])).cuda()
    down = torch.from_numpy(np.concatenate([make_quant_weight(td, hidden, inter, seed=80 + e) for e in range(E)])).cuda()
    for T in (12, 150, 700):
        rows = T * top_k
        x = torch.from_numpy(make_x(T, hidden, seed=90 + T)).cuda()
        rng = np.random.default_rng(T)
        # skewed routing: expert 0 is hot, expert E-1 gets nothing
        pick = np.stack([rng.choice(E - 1, size=top_k, replace=False, p=np.r_[0.4, np.full(E - 2, 0.6 / (E - 2))]) for _ in range(T)])
        ids = torch.from_numpy(pick.astype(np.int32).reshape(-1)).cuda()
        assert ops.moe_experts_supported(gpu_ctx, T, top_k, hidden, inter, E, tg, td)
        pg = hq.GgmlQuantizedMatmulIdParams(T, top_k, inter, hidden, E, sg, tg)
        pd = hq.GgmlQuantizedMatmulIdParams(rows, 1, hidden, inter, E, sd, td)
        scratch = ops.IdMmScratch.alloc(gpu_ctx, E, rows, max(hidden, inter))
        g = torch.empty((rows, inter), device="cuda")
        u = torch.empty_like(g)
        hq.quantized_matmul_id_pair_ggml(gpu_ctx, x, gate.data_ptr(), up.data_ptr(), ids, g, u, scratch, pg)
        act = ffn._silu_mul(gpu_ctx, g, u)
        want = torch.empty((rows, hidden), device="cuda")
        hq.quantized_matmul_id_ggml(gpu_ctx, act, down.data_ptr(), ids, want, scratch, pd)
        got = torch.full((rows, hidden), float("nan"), device="cuda")
        n0 = gpu_ctx.launch_count
        ops.moe_experts(gpu_ctx, x, gate.data_ptr(), up.data_ptr(), down.data_ptr(), ids, got, T, top_k, hidden, inter, E, tg, td)
        assert gpu_ctx.launch_count - n0 == 4
        gpu_ctx.check_status()
        assert torch.equal(got, want), (tg, td, T)
    # an expert index out of range: zero row, status bit
    bad = ids.clone()
    bad[5] = E + 3
    ops.moe_experts(gpu_ctx, x, gate.data_ptr(), up.data_ptr(), down.data_ptr(), bad, got, T, top_k, hidden, inter, E, tg, td)
    with pytest.raises(hq.Hf2qError):
        gpu_ctx.check_status()
    assert torch.count_nonzero(got[5]) == 0 and torch.equal(got[4], want[4]) and torch.equal(got[6], want[6])
    assert not ops.moe_experts_supported(gpu_ctx, 4, top_k, hidden, inter, E, tg, td)          # few rows: the mat-vec forms
    assert not ops.moe_experts_supported(gpu_ctx, T, top_k, hidden, inter, E, oracle.IQ4_NL, td)


def test_builder_entries_fused_equals_reference_sequence(gpu_ctx):
    """hf2q_cuda_dense_ffn / hf2q_cuda_moe_ffn: the fused forms and the reference's own op sequence
    (HF2Q_FFN_NO_FUSION) give the same bits; the dense entry works in place on the residual stream in both."""
    import ctypes as C
    lib = _lib_load()
    t, hidden, inter = oracle.Q4_K, 2048, 2048
    gq, _ = _qw(gpu_ctx, t, inter, hidden, 1)
    uq, _ = _qw(gpu_ctx, t, inter, hidden, 2)
    dq, _ = _qw(gpu_ctx, oracle.Q6_K, hidden, inter, 3)
    w = ffn.DenseFfnWeightsGpuQ(gq, uq, dq)
    for m in (3, 40):
        x = torch.from_numpy(make_x(m, hidden, seed=4 + m)).cuda()
        res = torch.from_numpy(make_x(m, hidden, seed=5 + m)).cuda()
        a = ffn.build_dense_ffn_layer_gpu_q(gpu_ctx, x, w, residual=res, fused=True)
        b = ffn.build_dense_ffn_layer_gpu_q(gpu_ctx, x, w, residual=res, fused=False)
        gpu_ctx.check_status()
        assert torch.equal(a, b), m
        need = C.c_uint64()
        assert lib.hf2q_cuda_dense_ffn_scratch_bytes(m, hidden, inter, C.byref(need)) == 0
        sc = torch.empty(need.value, dtype=torch.uint8, device="cuda")
        for flags in (0, 1):
            y = res.clone()                                 # y doubles as the residual
            rc = lib.hf2q_cuda_dense_ffn(gpu_ctx._h, None, x.data_ptr(), 0, gq.ptr, t, uq.ptr, t, dq.ptr, oracle.Q6_K, y.data_ptr(),
                                         y.data_ptr(), m, hidden, inter, sc.data_ptr(), sc.numel(), flags)
            assert rc == 0
            torch.cuda.synchronize()
            assert torch.equal(y, a), (m, flags)
        assert lib.hf2q_cuda_dense_ffn(gpu_ctx._h, None, x.data_ptr(), 0, gq.ptr, t, uq.ptr, t, dq.ptr, oracle.Q6_K, None, y.data_ptr(),
                                       m, hidden, inter, sc.data_ptr(), 16, 0) == hq._lib.ERR_WORKSPACE
    # the expert layer, few and many routed rows, with the shared expert
    E, k, mi = 6, 2, 2048
    tq = oracle.Q5_K
    eg = torch.from_numpy(np.concatenate([make_quant_weight(tq, mi, hidden, seed=100 + e) for e in range(E)])).cuda()
    eu = torch.from_numpy(np.concatenate([make_quant_weight(tq, mi, hidden, seed=200 + e) for e in range(E)])).cuda()
    ed = torch.from_numpy(np.concatenate([make_quant_weight(tq, hidden, mi, seed=300 + e) for e in range(E)])).cuda()
    rng = np.random.default_rng(3)
    router = torch.from_numpy((rng.standard_normal((E, hidden)) * 0.05).astype(np.float32)).cuda()
    sl = torch.from_numpy((rng.standard_normal(hidden) * 0.05).astype(np.float32)).cuda()
    mw = ffn.MoeFfnWeightsGpuQ(router=router, expert_gate=eg, expert_up=eu, expert_down=ed, ggml_type_gate_up=tq, ggml_type_down=tq,
                               num_experts=E, num_experts_per_tok=k, moe_intermediate_size=mi, shared=w, shared_gate_logit=sl)
    for T in (2, 90):
        x = torch.from_numpy(make_x(T, hidden, seed=31 + T)).cuda()
        res = torch.from_numpy(make_x(T, hidden, seed=32 + T)).cuda()
        a = ffn.build_moe_ffn_layer_gpu_q(gpu_ctx, x, mw, residual=res, fused=True)
        b = ffn.build_moe_ffn_layer_gpu_q(gpu_ctx, x, mw, residual=res, fused=False)
        gpu_ctx.check_status()
        assert torch.equal(a, b), T


def _lib_load():
    from hf2q_b200 import _lib
    return _lib.load()


def test_moe_weighted_reduce_inside_the_down_product(gpu_ctx):
    """HF2Q_FFN_ATOMIC_COMBINE: the slots' rows are added to their token's row by the down product's epilogue
    (f32 atomics).  Same terms as the separate combine, summed in arrival order: equal to it within a few ulps of
    the largest term, and a defined result for a row whose expert id is out of range."""
    from hf2q_b200 import ops
    t, hidden, inter, E, k = oracle.Q5_K, 2048, 512, 16, 4
    eg = torch.from_numpy(np.concatenate([make_quant_weight(t, inter, hidden, seed=100 + e) for e in range(E)])).cuda()
    eu = torch.from_numpy(np.concatenate([make_quant_weight(t, inter, hidden, seed=200 + e) for e in range(E)])).cuda()
    ed = torch.from_numpy(np.concatenate([make_quant_weight(t, hidden, inter, seed=300 + e) for e in range(E)])).cuda()
    rng = np.random.default_rng(5)
    router = torch.from_numpy((rng.standard_normal((E, hidden)) * 0.05).astype(np.float32)).cuda()
    sgq, _ = _qw(gpu_ctx, t, 512, hidden, 11)
    suq, _ = _qw(gpu_ctx, t, 512, hidden, 12)
    sdq, _ = _qw(gpu_ctx, t, hidden, 512, 13)
    sl = torch.from_numpy((rng.standard_normal(hidden) * 0.05).astype(np.float32)).cuda()
    w = ffn.MoeFfnWeightsGpuQ(router=router, expert_gate=eg, expert_up=eu, expert_down=ed, ggml_type_gate_up=t, ggml_type_down=t,
                              num_experts=E, num_experts_per_tok=k, moe_intermediate_size=inter,
                              shared=ffn.DenseFfnWeightsGpuQ(sgq, suq, sdq), shared_gate_logit=sl)
    T = 300
    x = torch.from_numpy(make_x(T, hidden, seed=9)).cuda()
    res = torch.from_numpy(make_x(T, hidden, seed=10)).cuda()
    want = ffn.build_moe_ffn_layer_gpu_q(gpu_ctx, x, w, residual=res)
    got = ffn.build_moe_ffn_layer_gpu_q(gpu_ctx, x, w, residual=res, atomic_combine=True)
    gpu_ctx.check_status()
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) < 1e-5 * scale
    assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) < 1e-6
    # the entry itself, with one expert id out of range: that slot adds nothing
    ids = torch.from_numpy(np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32).reshape(-1)).cuda()
    wts = torch.rand(T * k, device="cuda")
    rows = torch.empty((T * k, hidden), device="cuda")
    bad = ids.clone()
    bad[7] = E + 1
    ops.moe_experts(gpu_ctx, x, eg.data_ptr(), eu.data_ptr(), ed.data_ptr(), bad, rows, T, k, hidden, inter, E, t, t)
    with pytest.raises(hq.Hf2qError):
        gpu_ctx.check_status()
    ref = (rows.view(T, k, hidden) * wts.view(T, k, 1)).sum(1)
    out = torch.zeros((T, hidden), device="cuda")
    lib = _lib_load()
    import ctypes as C
    need = C.c_uint64()
    lib.hf2q_cuda_moe_experts_scratch_bytes(E, T * k, hidden, inter, C.byref(need))
    sc = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    rc = lib.hf2q_cuda_moe_experts_reduce(gpu_ctx._h, None, x.data_ptr(), 0, eg.data_ptr(), eu.data_ptr(), ed.data_ptr(), bad.data_ptr(),
                                          wts.data_ptr(), out.data_ptr(), T, k, hidden, inter, E, hq.expert_stride(t, inter, hidden), t,
                                          hq.expert_stride(t, hidden, inter), t, sc.data_ptr(), sc.numel())
    assert rc == 0
    with pytest.raises(hq.Hf2qError):
        gpu_ctx.check_status()
    assert float((out - ref).abs().max()) < 1e-5 * float(ref.abs().max())
