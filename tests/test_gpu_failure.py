"""Failure detection on the device: a wait for another GPU that never answers.

The fused all-gather waits on arrival counters that other ranks' kernels bump.  Here nothing ever
bumps them: one process plays "rank 0 of 2", the counter block says that rank 1 still owes
arrivals, and the wait limit of the context is a few milliseconds.  The waiting kernels must give
up, record it, RETURN (no trap, no hang), the status must read back as HF2Q_ERR_TIMEOUT, and the
same context must keep working afterwards.  No second process, no peer GPU and no fault is involved.
"""
import ctypes as C
import time

import pytest
import torch

import oracle
import hf2q_b200 as hq
from hf2q_b200 import _lib
from hf2q_b200.dist import _Gather
from tests.util import make_quant_weight, make_x, rel_l2

pytestmark = pytest.mark.gpu

LIMIT_TICKS = 8_000_000          # about 4 ms at 1.9 GHz


def _group_of_two(flags, y0, y1, n, n_total, wait_previous):
    g = _Gather()
    g.y_all[0], g.y_all[1] = y0.data_ptr(), y1.data_ptr()
    g.flags[0], g.flags[1] = flags.data_ptr(), flags.data_ptr() + 128     # "rank 1" counts in the other half
    g.n_ranks, g.rank, g.n_total, g.col0, g.wait_previous = 2, 0, n_total, 0, int(wait_previous)
    g.n_rows[0], g.n_rows[1] = n, n_total - n
    return g


def test_wait_for_a_silent_rank_times_out_and_the_context_survives(gpu_ctx):
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    t, n, k, m = oracle.Q6_K, 64, 2048, 2
    raw = make_quant_weight(t, n, k, seed=77)
    w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
    wref = oracle.dequantize(t, raw).reshape(n, k)
    x = make_x(m, k, seed=78)
    xd = torch.from_numpy(x).cuda()
    want = oracle.matmul_f64(x, wref)
    n_total = 2 * n
    y0 = torch.zeros((m, n_total), device="cuda")
    y1 = torch.zeros((m, n_total), device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[8 + 1] = 5                     # rank 1 owes five arrivals that will never come
    torch.cuda.synchronize()
    gpu_ctx.set_wait_limit(LIMIT_TICKS)
    try:
        # 1. the stand-alone wait kernel
        g = _group_of_two(flags, y0, y1, n, n_total, False)
        t0 = time.perf_counter()
        assert lib.hf2q_cuda_gather_wait(gpu_ctx._h, stream, C.byref(g)) == 0
        with pytest.raises(hq.Hf2qError) as ei:
            gpu_ctx.check_status()                      # synchronises: the kernel has returned
        assert ei.value.status == _lib.ERR_TIMEOUT
        assert time.perf_counter() - t0 < 1.0           # milliseconds, not the default second
        gpu_ctx.check_status()                          # the status word was cleared by the read-back

        # 2. the wait inside a product: it gives up, computes with the activations that are there and returns
        g = _group_of_two(flags, y0, y1, n, n_total, True)
        rc = lib.hf2q_cuda_qmatmul_gather(gpu_ctx._h, stream, xd.data_ptr(), hq.ops.DT_F32, w.ptr, C.byref(g), m, n, k, t)
        assert rc == 0, lib.hf2q_cuda_last_error(gpu_ctx._h)
        with pytest.raises(hq.Hf2qError) as ei:
            gpu_ctx.check_status()
        assert ei.value.status == _lib.ERR_TIMEOUT
        # x was a complete local tensor, so the product itself is right in both "ranks'" buffers
        assert rel_l2(y0[:, :n].cpu().numpy(), want) < 1e-3
        assert torch.equal(y0[:, :n], y1[:, :n])
        # every CTA of the launch (64 rows = 4 row groups = 4 CTAs) told "rank 1" that it arrived, and the
        # launch noted that it expects as many arrivals back from rank 1's equally large shard
        f = flags.cpu().numpy()
        assert f[32 + 0] == 4
        assert f[8 + 1] == 5 + 4
    finally:
        gpu_ctx.set_wait_limit(1 << 31)

    # 3. the same context still computes, and a wait with nothing outstanding passes at once
    flags.zero_()
    torch.cuda.synchronize()
    g = _group_of_two(flags, y0, y1, n, n_total, False)
    assert lib.hf2q_cuda_gather_wait(gpu_ctx._h, stream, C.byref(g)) == 0
    y = torch.empty((m, n), device="cuda")
    hq.quantized_matmul_ggml(gpu_ctx, xd, w, y, w.matmul_params(m))
    gpu_ctx.check_status()
    assert rel_l2(y.cpu().numpy(), want) < 1e-3


def test_wait_limit_is_validated(gpu_ctx):
    lib = _lib.load()
    assert lib.hf2q_cuda_set_wait_limit(gpu_ctx._h, 0) == _lib.ERR_INVALID_ARGUMENT
    assert lib.hf2q_cuda_set_wait_limit(gpu_ctx._h, 1 << 50) == _lib.ERR_INVALID_ARGUMENT
    assert lib.hf2q_cuda_set_wait_limit(gpu_ctx._h, 1 << 31) == 0
