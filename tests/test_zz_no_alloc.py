"""The allocation-free GEMM entry point, hf2q_cuda_qmatmul_static.

It exists for callers that cannot give the library a workspace because they have no way to
allocate device memory on the op path (the application's arena owns the whole device, or the
caller is thin FFI glue that only sees one op's tensors).  Its scratch is a fixed 8 MiB array
inside the library, shared by every call, so this file checks three things through the C ABI:
the result equals the workspace-taking entry point's, a second call right after the first (which
finds the previous call's bytes in the array) is still right, and a product larger than the array
is refused with a clear error.  The file sorts last on purpose: a run that stops at the first
failure has already gone through every other test.
"""

import numpy as np
import pytest
import torch

import oracle
import hf2q_b200 as hq
from hf2q_b200 import _lib
from tests.util import make_quant_weight, make_x, rel_l2, to_bf16_bits

pytestmark = pytest.mark.gpu


def _x_bf16(m, k, seed):
    bits = to_bf16_bits(make_x(m, k, seed=seed))
    return torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch.bfloat16)


def test_static_scratch_entry_matches_workspace_entry_twice(gpu_ctx):
    lib = _lib.load()
    t, n, k = oracle.Q4_K, 384, 2048
    raw = make_quant_weight(t, n, k, seed=123)
    w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
    wref = oracle.dequantize(t, raw).reshape(n, k)
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different shapes: the second overwrites only part of what the first
    # left in the shared array
    for m, seed in ((200, 1), (40, 2)):
        x = _x_bf16(m, k, seed)
        y_static = torch.full((m, n), float("nan"), device="cuda")
        y_ws = torch.full((m, n), float("nan"), device="cuda")
        rc = lib.hf2q_cuda_qmatmul_static(gpu_ctx._h, stream, x.data_ptr(), hq.ops.DT_BF16, w.ptr,
                                          y_static.data_ptr(), m, n, k, t)
        assert rc == 0, lib.hf2q_cuda_last_error(gpu_ctx._h)
        hq.quantized_matmul_ggml(gpu_ctx, x, w, y_ws, w.matmul_params(m))
        gpu_ctx.check_status()
        assert torch.equal(y_static, y_ws)           # same kernel, same inputs: same bits
        want = oracle.matmul_f64(x.float().cpu().numpy(), wref)
        assert rel_l2(y_static.cpu().numpy(), want) < 1e-3


def test_static_scratch_entry_refuses_what_does_not_fit(gpu_ctx):
    lib = _lib.load()
    cap = lib.hf2q_cuda_qmatmul_static_max_elements()
    assert cap == 4 * 1024 * 1024
    t, n, k = oracle.Q4_K, 128, 4096
    m = cap // k + 1                                  # one row too many
    w = hq.load_quant_weight(gpu_ctx, make_quant_weight(t, n, k, seed=5), t, n, k)
    x = torch.zeros((m, k), dtype=torch.bfloat16, device="cuda")
    y = torch.empty((m, n), device="cuda")
    rc = lib.hf2q_cuda_qmatmul_static(gpu_ctx._h, None, x.data_ptr(), hq.ops.DT_BF16, w.ptr, y.data_ptr(), m, n, k, t)
    assert rc == _lib.ERR_WORKSPACE
    assert b"fixed array" in lib.hf2q_cuda_last_error(gpu_ctx._h)
    # a layout the tensor-core path cannot take is an error too, not a silent detour
    k2 = 32 * 3
    w2 = hq.load_quant_weight(gpu_ctx, make_quant_weight(oracle.Q4_0, 16, k2, seed=6), oracle.Q4_0, 16, k2)
    x2 = torch.zeros((4, k2), dtype=torch.bfloat16, device="cuda")
    y2 = torch.empty((4, 16), device="cuda")
    rc = lib.hf2q_cuda_qmatmul_static(gpu_ctx._h, None, x2.data_ptr(), hq.ops.DT_BF16, w2.ptr, y2.data_ptr(), 4, 16, k2, oracle.Q4_0)
    assert rc == _lib.ERR_INVALID_ARGUMENT


def _static_call_leaves_free_memory_alone(ctx, device):
    """What the entry point is for: between two calls the device's free memory must not move (no
    cudaMalloc / cudaFree behind the caller's back, torch's caching allocator not involved either)."""
    lib = _lib.load()
    t, n, k, m = oracle.Q6_K, 256, 2048, 64
    raw = make_quant_weight(t, n, k, seed=31)
    with torch.cuda.device(device):
        w = hq.load_quant_weight(ctx, raw, t, n, k)
        bits = to_bf16_bits(make_x(m, k, seed=32))
        x = torch.from_numpy(bits.view(np.int16).copy()).to(f"cuda:{device}").view(torch.bfloat16)
        y = torch.empty((m, n), device=f"cuda:{device}")
        stream = torch.cuda.current_stream(device).cuda_stream

        def call():
            rc = lib.hf2q_cuda_qmatmul_static(ctx._h, stream, x.data_ptr(), hq.ops.DT_BF16, w.ptr, y.data_ptr(), m, n, k, t)
            assert rc == 0, lib.hf2q_cuda_last_error(ctx._h)

        call()                                        # first call on this device: resolves the array's address
        torch.cuda.synchronize(device)
        free0, _ = torch.cuda.mem_get_info(device)
        reserved0 = torch.cuda.memory_reserved(device)
        for _ in range(3):
            call()
        torch.cuda.synchronize(device)
        free1, _ = torch.cuda.mem_get_info(device)
        assert free1 == free0 and torch.cuda.memory_reserved(device) == reserved0
        ctx.check_status()
        want = oracle.matmul_f64(x.float().cpu().numpy(), oracle.dequantize(t, raw).reshape(n, k))
        assert rel_l2(y.cpu().numpy(), want) < 1e-3


def test_static_scratch_entry_allocates_nothing(gpu_ctx):
    _static_call_leaves_free_memory_alone(gpu_ctx, 0)


def test_static_scratch_entry_on_a_second_device():
    """The array's address is resolved per device: a context on GPU 1 must get GPU 1's copy."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = hq.GpuContext(1)
    try:
        _static_call_leaves_free_memory_alone(ctx, 1)
    finally:
        ctx.close()
