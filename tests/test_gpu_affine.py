"""mlx-affine 4-bit / group-32 weights through the C ABI: pack, dequantise, mat-vec, GEMM, embedding rows.

The scalar specification is the reference tests' own CPU oracle (forward_mlx.rs:8886-8901) and their bar is
max |y - spec| < 1e-3 on their deterministic synthetic linear (m = 16, n = 64, k = 96)."""
import ctypes as C

import numpy as np
import pytest
import torch

import hf2q_b200 as hq
from hf2q_b200 import _lib, ops
from oracle import mlx_affine as A
from tests.util import make_x, rel_l2

pytestmark = pytest.mark.gpu


def _load(ctx, q, s, b):
    codes = torch.from_numpy(A.pack_codes(q).view(np.int32)).cuda()
    return ops.load_mlx_affine_weight(ctx, codes, torch.from_numpy(s).cuda(), torch.from_numpy(b).cuda())


def test_reference_round_trip_vector(gpu_ctx):
    """from_mlx_affine_linear_roundtrips_through_packed_kernel (forward_mlx.rs:8785-8913) on this library."""
    m, n, k = 16, 64, 96
    q, s, b, x = A.reference_vector(m, n, k)
    w = _load(gpu_ctx, q, s, b)
    assert (w.rows, w.cols, w.ggml_type) == (n, k, 1000) and w.nbytes == n * 3 * 24
    # the packed container is byte-identical to the oracle's
    raw = torch.as_tensor(w._owner).cpu().numpy()
    assert np.array_equal(raw, A.to_blocks(A.pack_codes(q), s, b))
    # bit-exact dequantisation
    deq = hq.dequantize(gpu_ctx, w).cpu().numpy()
    assert np.array_equal(deq.view(np.uint32), A.dequantize_blocks(raw).reshape(n, k).view(np.uint32))
    y = torch.full((m, n), float("nan"), device="cuda")
    hq.quantized_matmul_ggml(gpu_ctx, torch.from_numpy(x).cuda(), w, y, w.matmul_params(m))
    gpu_ctx.check_status()
    assert np.abs(y.cpu().numpy() - A.qmm_affine_f64(x, q, s, b)).max() < 1e-3         # the reference's bar


def test_matvec_gemm_and_rows(gpu_ctx):
    rng = np.random.default_rng(11)
    n, k = 320, 2048
    q = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    s = (rng.random((n, k // 32), dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    b = (-8.0 * s * (1.0 + 0.1 * rng.standard_normal((n, k // 32)))).astype(np.float32)
    w = _load(gpu_ctx, q, s, b)
    for m, bf16 in ((1, False), (5, True), (8, True), (40, True), (300, False)):       # mat-vec kernels up to 8 rows, tensor-core GEMM beyond
        x = make_x(m, k, seed=m)
        xd = torch.from_numpy(x).cuda()
        if bf16:
            xd = xd.bfloat16()
            x = xd.float().cpu().numpy()
        y = torch.full((m, n), float("nan"), device="cuda")
        hq.quantized_matmul_ggml(gpu_ctx, xd, w, y, w.matmul_params(m))
        gpu_ctx.check_status()
        assert rel_l2(y.cpu().numpy(), A.qmm_affine_f64(x, q, s, b)) < 1e-3, m
    # embedding rows (token_embd of a DWQ model)
    ids = torch.tensor([3, 0, 319, 17], dtype=torch.int32, device="cuda")
    rows = torch.empty((4, k), device="cuda")
    gpu_ctx._check(gpu_ctx._lib.hf2q_cuda_get_rows(gpu_ctx._h, None, w.ptr, w.ggml_type, n, k, ids.data_ptr(), 4, rows.data_ptr()))
    torch.cuda.synchronize()
    want = A.dequantize_blocks(A.to_blocks(A.pack_codes(q), s, b)).reshape(n, k)
    assert np.array_equal(rows.cpu().numpy(), want[[3, 0, 319, 17]])


def test_pack_rejects_what_the_reference_rejects(gpu_ctx):
    """from_mlx_affine_linear_rejects_unsupported_bits (forward_mlx.rs:9327): only bits = 4, group_size = 32."""
    lib = _lib.load()
    codes = torch.zeros((4, 8), dtype=torch.int32, device="cuda")
    s = torch.ones((4, 2), device="cuda")
    out = torch.empty(4 * 2 * 24, dtype=torch.uint8, device="cuda")
    args = (gpu_ctx._h, None, codes.data_ptr(), s.data_ptr(), s.data_ptr(), 4, 64)
    assert lib.hf2q_cuda_affine_pack(*args, 8, 32, out.data_ptr()) == _lib.ERR_UNSUPPORTED_TYPE
    assert lib.hf2q_cuda_affine_pack(*args, 4, 64, out.data_ptr()) == _lib.ERR_UNSUPPORTED_TYPE
    assert lib.hf2q_cuda_affine_pack(gpu_ctx._h, None, codes.data_ptr(), s.data_ptr(), s.data_ptr(), 4, 48, 4, 32, out.data_ptr()) == _lib.ERR_INVALID_ARGUMENT
    assert lib.hf2q_cuda_affine_pack(*args, 4, 32, out.data_ptr()) == 0
