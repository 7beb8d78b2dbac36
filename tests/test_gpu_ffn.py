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
