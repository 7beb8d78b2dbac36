"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Dequantisation must be bit-exact.  Matmul outputs must be within 1e-3 relative L2 of an f64 matmul
on the oracle's dequantised weights (the gate the benchmark spec states)."""
import numpy as np
import pytest
import torch

import oracle
import hf2q_b200 as hq
from hf2q_b200 import _lib
from tests.util import (FIXTURES, bf16_bits_to_f32, make_quant_weight, make_x, random_finite_blocks,
                        rel_l2, to_bf16_bits)

pytestmark = pytest.mark.gpu
GATE = 1e-3      # relative L2 vs the f64 product
TYPES = list(oracle.ALL_TYPES)


def _dev_x(x_f32: np.ndarray, bf16: bool):
    """Returns (device tensor, the float32 values the kernel will see)."""
    if bf16:
        bits = to_bf16_bits(x_f32)
        t = torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch.bfloat16)
        return t, bf16_bits_to_f32(bits).reshape(x_f32.shape)
    return torch.from_numpy(x_f32.copy()).cuda(), x_f32


def _ref(t, raw, x_seen, n, k):
    w = oracle.dequantize(t, raw).reshape(n, k)
    return oracle.matmul_f64(x_seen, w)


# ---------------------------------------------------------------- K0 dequant, bit exact
@pytest.mark.parametrize("t", TYPES)
def test_dequant_bit_exact_on_reference_fixtures(gpu_ctx, golden_dir, t):
    name, n = FIXTURES[t]
    for variant in ("noim", "im"):
        raw = np.fromfile(golden_dir / f"{name}_{n}_{variant}_expected.bin", dtype=np.uint8)
        w = hq.load_quant_weight(gpu_ctx, raw, t, 2, n)
        got = hq.dequantize(gpu_ctx, w).cpu().numpy().reshape(-1)
        want = oracle.dequantize(t, raw)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("t", TYPES)
def test_dequant_bit_exact_on_random_bit_patterns(gpu_ctx, t):
    be, _ = oracle.block_geometry(t)
    rows, k = 64, be * 24
    raw = random_finite_blocks(t, rows * 24, seed=100 + t)
    w = hq.load_quant_weight(gpu_ctx, raw, t, rows, k)
    got = hq.dequantize(gpu_ctx, w).cpu().numpy().reshape(-1)
    want = oracle.dequantize(t, raw)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("t", TYPES)
def test_dequant_bit_exact_all_f16_scales(gpu_ctx, t):
    """Every finite f16 value in the scale field(s), subnormals included."""
    be, bb = oracle.block_geometry(t)
    h = np.arange(65536, dtype=np.uint32)
    h = h[(h & 0x7C00) != 0x7C00].astype(np.uint16)
    pad = (-h.size) % 8
    h = np.concatenate([h, np.zeros(pad, np.uint16)])
    raw = random_finite_blocks(t, h.size, seed=5).reshape(h.size, bb)
    off = 208 if t == oracle.Q6_K else 0
    raw[:, off] = h & 0xFF
    raw[:, off + 1] = h >> 8
    if t in (oracle.Q4_K, oracle.Q5_K, oracle.Q4_1, oracle.Q5_1):       # the second f16 field (dmin / m)
        raw[:, 2] = h[::-1] & 0xFF
        raw[:, 3] = h[::-1] >> 8
    w = hq.load_quant_weight(gpu_ctx, raw.reshape(-1), t, h.size // 8, 8 * be)
    got = hq.dequantize(gpu_ctx, w).cpu().numpy().reshape(-1)
    want = oracle.dequantize(t, raw.reshape(-1))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_dequant_to_half_types_is_the_rounded_f32(gpu_ctx, t, dt):
    raw = make_quant_weight(t, 32, 1024, seed=9)
    w = hq.load_quant_weight(gpu_ctx, raw, t, 32, 1024)
    got = hq.dequantize(gpu_ctx, w, dt)
    want = torch.from_numpy(oracle.dequantize(t, raw).reshape(32, 1024)).to(dt)
    assert torch.equal(got.cpu(), want)


# ---------------------------------------------------------------- K1 mat-vec
SHAPES = [(32, 64), (64, 32 * 7), (8, 256), (40, 512), (72, 2048), (130, 4096), (17, 6144), (24, 14336)]


def _gemv_sweep(ctx, t, bf16, bound):
    be, _ = oracle.block_geometry(t)
    for (n, k) in SHAPES:
        if k % be:
            continue
        raw = make_quant_weight(t, n, k, seed=n + k)
        w = hq.load_quant_weight(ctx, raw, t, n, k)
        for m in (1, 2, 3, 4, 5, 8):
            xd, xs = _dev_x(make_x(m, k, seed=m), bf16)
            y = torch.full((m, n), float("nan"), device="cuda")
            hq.quantized_matmul_ggml(ctx, xd, w, y, w.matmul_params(m))
            ctx.check_status()
            err = rel_l2(y.cpu().numpy(), _ref(t, raw, xs, n, k))
            assert err < GATE, (t, n, k, m, err)
            if n * m >= 64 and k >= 1024:      # few outputs or few sub-blocks per row: too noisy for the tighter bound
                assert err < bound, (t, n, k, m, err)


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("bf16", [False, True])
def test_gemv_matches_f64_reference(gpu_ctx, t, bf16):
    """Default routing: warp-MMA kernel (integer codes as f16 subnormals) or the fp32 kernel: far inside the gate."""
    _gemv_sweep(gpu_ctx, t, bf16, 2e-5)


def test_baseline_config_1_q4k_4096(gpu_ctx):
    """W 4096x4096 N(0, 0.02) seed 0 -> Q4_K, x 1x4096 N(0,1) seed 1, y within 1e-3 rel L2."""
    t, n, k = oracle.Q4_K, 4096, 4096
    raw = make_quant_weight(t, n, k, seed=0)
    assert raw.size == 9_437_184
    w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
    deq = hq.dequantize(gpu_ctx, w).cpu().numpy()
    want_w = oracle.dequantize(t, raw).reshape(n, k)
    assert np.array_equal(deq.view(np.uint32), want_w.view(np.uint32))
    x = make_x(1, k, seed=1)
    y = torch.empty((1, n), device="cuda")
    hq.quantized_matmul_ggml(gpu_ctx, torch.from_numpy(x).cuda(), w, y, w.matmul_params(1))
    assert rel_l2(y.cpu().numpy(), oracle.matmul_f64(x, want_w)) < GATE
    # and the reference's own f32 CPU path agrees to f32 reorder noise
    y_cpu, _, _ = oracle.qmatmul(t, raw, x, n, k, threads=oracle.max_threads())
    assert rel_l2(y.cpu().numpy(), y_cpu) < 1e-5


def test_qmatmul_more_than_eight_rows(gpu_ctx):
    t, n, k, m = oracle.Q6_K, 96, 2048, 37
    raw = make_quant_weight(t, n, k, seed=4)
    w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
    xd, xs = _dev_x(make_x(m, k, seed=8), True)
    ws = torch.empty(max(1, hq.ops.quantized_matmul_workspace_bytes(w.matmul_params(m))), dtype=torch.uint8, device="cuda")
    y = torch.empty((m, n), device="cuda")
    hq.quantized_matmul_ggml(gpu_ctx, xd, w, y, w.matmul_params(m), ws)
    assert rel_l2(y.cpu().numpy(), _ref(t, raw, xs, n, k)) < GATE


# ---------------------------------------------------------------- K2 tensor-core GEMM
@pytest.mark.parametrize("t", TYPES)
def test_gemm_matches_f64_reference(gpu_ctx, t):
    """m > 8 takes the tcgen05 kernel (f16 operands, fp32 accumulate): gate 1e-3 relative L2."""
    for (n, k, m, bf16) in [(128, 256, 16, True), (200, 1024, 33, True), (384, 2048, 130, False),
                            (96, 4096, 300, True), (520, 512, 64, True)]:
        raw = make_quant_weight(t, n, k, seed=3 * n + k + m)
        w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
        xd, xs = _dev_x(make_x(m, k, seed=m), bf16)
        y = torch.full((m, n), float("nan"), device="cuda")
        hq.quantized_matmul_ggml(gpu_ctx, xd, w, y, w.matmul_params(m))
        gpu_ctx.check_status()
        err = rel_l2(y.cpu().numpy(), _ref(t, raw, xs, n, k))
        assert err < GATE, (t, n, k, m, err)


@pytest.mark.parametrize("t", [oracle.Q4_0, oracle.Q6_K, oracle.Q8_0])
def test_gemm_perm021_reads_heads_outermost_activations(gpu_ctx, t):
    """The O projection reading attention output stored [n_heads, seq, head_dim]: bit-identical to the plain
    product on the token-major copy (the permute only changes where the f16 staging reads), any m."""
    from hf2q_b200 import ops
    n, k, hd = 192, 2048, 128
    raw = make_quant_weight(t, n, k, seed=77)
    w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
    for m, bf16 in ((1, True), (7, False), (40, True), (300, True)):
        xd, xs = _dev_x(make_x(m, k, seed=100 + m), bf16)
        perm = xd.view(m, k // hd, hd).permute(1, 0, 2).contiguous()           # [heads, m, head_dim]
        got = torch.full((m, n), float("nan"), device="cuda")
        ops.quantized_matmul_mm_tensor_perm021(gpu_ctx, perm, w, got, m, hd)
        gpu_ctx.check_status()
        assert rel_l2(got.cpu().numpy(), _ref(t, raw, xs, n, k)) < GATE
        if m > 8:
            want = torch.empty((m, n), device="cuda")
            hq.quantized_matmul_ggml(gpu_ctx, xd, w, want, w.matmul_params(m))
            assert torch.equal(got, want)
    lib = _lib.load()
    ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    rc = lib.hf2q_cuda_qmatmul_perm021(gpu_ctx._h, None, perm.data_ptr(), 1, w.ptr, got.data_ptr(), 4, n, k, 100, t, ws.data_ptr(), ws.numel())
    assert rc == _lib.ERR_INVALID_ARGUMENT                                     # head_dim must divide k


def test_gemm_needs_its_workspace(gpu_ctx):
    t, n, k, m = oracle.Q4_K, 128, 512, 64
    w = hq.load_quant_weight(gpu_ctx, make_quant_weight(t, n, k, seed=1), t, n, k)
    x = torch.randn(m, k, device="cuda")
    y = torch.empty(m, n, device="cuda")
    lib = _lib.load()
    rc = lib.hf2q_cuda_qmatmul(gpu_ctx._h, None, x.data_ptr(), 0, w.ptr, y.data_ptr(), m, n, k, t, None, 0)
    assert rc == _lib.ERR_WORKSPACE


def test_row_shard_is_a_byte_slice(gpu_ctx):
    t, n, k = oracle.Q6_K, 64, 4096
    raw = make_quant_weight(t, n, k, seed=6)
    w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
    xd, xs = _dev_x(make_x(2, k, seed=3), True)
    full = torch.empty((2, n), device="cuda")
    hq.quantized_matmul_ggml(gpu_ctx, xd, w, full, w.matmul_params(2))
    part = torch.empty((2, 24), device="cuda")
    ws = w.row_slice(16, 40)
    hq.quantized_matmul_ggml(gpu_ctx, xd, ws, part, ws.matmul_params(2))
    assert torch.equal(part, full[:, 16:40].contiguous())


def test_host_buffer_call(gpu_ctx):
    t, n, k, m = oracle.Q4_K, 256, 2048, 4
    raw = make_quant_weight(t, n, k, seed=12)
    w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
    x = make_x(m, k, seed=2)
    y = np.empty((m, n), np.float32)
    hq.ops.quantized_matmul_host(gpu_ctx, x, w, y, m)
    assert rel_l2(y, _ref(t, raw, x, n, k)) < GATE
    # queued form: more calls than staging slots, different shapes, one wait at the end
    outs = []
    for i in range(21):                    # 8 staging slots: every slot is reused, and grows when a larger m arrives
        mi = (1 + i % 3) if i != 13 else 12
        xi = make_x(mi, k, seed=20 + i)
        yi = np.full((mi, n), np.nan, np.float32)
        hq.ops.quantized_matmul_host(gpu_ctx, xi, w, yi, mi, wait=False)
        outs.append((xi, yi))
    hq.ops.host_sync(gpu_ctx)
    for xi, yi in outs:
        assert rel_l2(yi, _ref(t, raw, xi, n, k)) < GATE


def test_host_buffer_batch_call(gpu_ctx):
    """One call queues many independent host-buffer products (mat-vec and GEMM sized, several formats); a second
    batch issued before the first one was waited for reuses the staging buffers in order."""
    specs = [(oracle.Q4_K, 256, 2048, 4), (oracle.Q6_K, 96, 2048, 1), (oracle.Q8_0, 64, 512, 8), (oracle.Q5_K, 128, 1024, 40),
             (oracle.Q4_0, 80, 256, 3)] * 4                                   # 20 products: groups of 2, 4 | 1, 1, 2, 2, 4, 4 (from the end)
    ws, raws = [], []
    for i, (t, n, k, m) in enumerate(specs):
        raw = make_quant_weight(t, n, k, seed=300 + i)
        raws.append(raw)
        ws.append(hq.load_quant_weight(gpu_ctx, raw, t, n, k))

    def make(seed):
        xs = [make_x(m, k, seed=seed + i) for i, (t, n, k, m) in enumerate(specs)]
        ys = [np.full((m, n), np.nan, np.float32) for (t, n, k, m) in specs]
        return xs, ys, hq.ops.HostBatch([(x, w, y, m, hq.ops.DT_F32) for x, w, y, (t, n, k, m) in zip(xs, ws, ys, specs)])

    xa, ya, ba = make(1000)
    xb, yb, bb = make(2000)
    hq.ops.quantized_matmul_host_batch(gpu_ctx, ba)
    hq.ops.quantized_matmul_host_batch(gpu_ctx, bb)
    hq.ops.host_sync(gpu_ctx)
    gpu_ctx.check_status()
    for xs, ys in ((xa, ya), (xb, yb)):
        for x, y, raw, (t, n, k, m) in zip(xs, ys, raws, specs):
            assert rel_l2(y, _ref(t, raw, x, n, k)) < GATE, (t, n, k, m)
    # The same batch again and again (a decode loop): from its second arrival on it is replayed as one CUDA graph.
    # New contents in the same host buffers must come through, another batch in between must not disturb it, and the
    # launch counter must advance by the same amount per call.
    per_call = []
    for rep in range(4):
        for i, x in enumerate(xa):
            x[...] = make_x(x.shape[0], x.shape[1], seed=5000 + 100 * rep + i)
        for y in ya:
            y[...] = np.nan
        n0 = gpu_ctx.launch_count
        hq.ops.quantized_matmul_host_batch(gpu_ctx, ba)
        per_call.append(gpu_ctx.launch_count - n0)
        if rep == 2:
            hq.ops.quantized_matmul_host_batch(gpu_ctx, bb)
        hq.ops.host_sync(gpu_ctx)
        gpu_ctx.check_status()
        for x, y, raw, (t, n, k, m) in zip(xa, ya, raws, specs):
            assert rel_l2(y, _ref(t, raw, x, n, k)) < GATE, (rep, t, n, k, m)
    assert len(set(per_call)) == 1 and per_call[0] >= len(specs)
    lib = _lib.load()
    assert lib.hf2q_cuda_qmatmul_host_batch(gpu_ctx._h, None, 3) == _lib.ERR_INVALID_ARGUMENT
    assert lib.hf2q_cuda_qmatmul_host_batch(gpu_ctx._h, None, 0) == 0


# ---------------------------------------------------------------- K3 routed mat-vec
@pytest.mark.parametrize("t", TYPES)
def test_mul_mat_id_small(gpu_ctx, t):
    ne, n, k, top_k = 6, 48, 512, 2
    be, _ = oracle.block_geometry(t)
    stride = hq.expert_stride(t, n, k)
    raw = np.concatenate([make_quant_weight(t, n, k, seed=50 + e) for e in range(ne)])
    wdev = torch.from_numpy(raw).cuda()
    for n_tokens in (1, 3, 9):
        rng = np.random.default_rng(n_tokens)
        ids = rng.integers(0, ne, size=n_tokens * top_k).astype(np.uint32)
        xd, xs = _dev_x(make_x(n_tokens, k, seed=77), True)
        y = torch.full((n_tokens * top_k, n), float("nan"), device="cuda")
        p = hq.GgmlQuantizedMatmulIdParams(n_tokens, top_k, n, k, ne, stride, t)
        scratch = hq.IdMmScratch.alloc(gpu_ctx, ne, n_tokens * top_k, k)
        hq.quantized_matmul_id_ggml(gpu_ctx, xd, wdev.data_ptr(), torch.from_numpy(ids.view(np.int32)).cuda(), y, scratch, p)
        gpu_ctx.check_status()
        want = oracle.qmatmul_id(t, raw, stride, xs, ids, n_tokens, top_k, n, k, ne)
        assert rel_l2(y.cpu().numpy(), want) < 2e-5


@pytest.mark.parametrize("t", [oracle.Q5_K, oracle.Q6_K, oracle.Q8_0])
def test_mul_mat_id_pair_matches_two_single_calls(gpu_ctx, t):
    """gate + up in one call: few rows (one routed mat-vec launch for both tensors) and many rows
    (sort/gather once, two grouped products); bad ids zero the rows of both outputs."""
    ne, n, k, top_k = 8, 128, 2048 if t == oracle.Q6_K else 512, 2
    stride = hq.expert_stride(t, n, k)
    raws = [np.concatenate([make_quant_weight(t, n, k, seed=s0 + e) for e in range(ne)]) for s0 in (300, 400)]
    wa, wb = (torch.from_numpy(r).cuda() for r in raws)
    for n_tokens in (1, 5, 40):
        rows = n_tokens * top_k
        ids = np.random.default_rng(n_tokens).integers(0, ne, size=rows).astype(np.uint32)
        xd, xs = _dev_x(make_x(n_tokens, k, seed=9), True)
        p = hq.GgmlQuantizedMatmulIdParams(n_tokens, top_k, n, k, ne, stride, t)
        scratch = hq.IdMmScratch.alloc(gpu_ctx, ne, rows, k)
        idd = torch.from_numpy(ids.view(np.int32)).cuda()
        ya, yb = (torch.full((rows, n), float("nan"), device="cuda") for _ in range(2))
        hq.quantized_matmul_id_pair_ggml(gpu_ctx, xd, wa.data_ptr(), wb.data_ptr(), idd, ya, yb, scratch, p)
        gpu_ctx.check_status()
        for y, w, raw in ((ya, wa, raws[0]), (yb, wb, raws[1])):
            single = torch.full((rows, n), float("nan"), device="cuda")
            hq.quantized_matmul_id_ggml(gpu_ctx, xd, w.data_ptr(), idd, single, scratch, p)
            assert torch.equal(y, single)                                   # same kernels, same order of sums
            want = oracle.qmatmul_id(t, raw, stride, xs, ids, n_tokens, top_k, n, k, ne)
            assert rel_l2(y.cpu().numpy(), want) < GATE
        gpu_ctx.check_status()


def test_mul_mat_id_down_projection_form(gpu_ctx):
    """down: n_tokens = T*top_k, top_k = 1, one activation row per routed slot (forward_mlx.rs:5324-5375)."""
    t, ne, n, k = oracle.Q5_K, 8, 256, 512
    stride = hq.expert_stride(t, n, k)
    raw = np.concatenate([make_quant_weight(t, n, k, seed=90 + e) for e in range(ne)])
    wdev = torch.from_numpy(raw).cuda()
    rows = 16
    ids = np.random.default_rng(0).integers(0, ne, size=rows).astype(np.uint32)
    xd, xs = _dev_x(make_x(rows, k, seed=5), False)
    y = torch.empty((rows, n), device="cuda")
    p = hq.GgmlQuantizedMatmulIdParams(rows, 1, n, k, ne, stride, t)
    hq.quantized_matmul_id_ggml(gpu_ctx, xd, wdev.data_ptr(), torch.from_numpy(ids.view(np.int32)).cuda(), y, None, p)
    want = oracle.qmatmul_id(t, raw, stride, xs, ids, rows, 1, n, k, ne)
    assert rel_l2(y.cpu().numpy(), want) < 2e-5


# ---------------------------------------------------------------- K4 grouped tensor-core mul_mat_id
@pytest.mark.parametrize("t", TYPES)
def test_mul_mat_id_grouped(gpu_ctx, t):
    """More than 32 routed rows: device-side sort by expert + one grouped tcgen05 launch."""
    for (ne, n, k, n_tokens, top_k, bf16) in [(8, 256, 512, 40, 2, True), (16, 130, 1024, 300, 4, False),
                                              (32, 512, 2048, 64, 8, True), (4, 2048, 512, 200, 1, True)]:
        stride = hq.expert_stride(t, n, k)
        raw = np.concatenate([make_quant_weight(t, n, k, seed=1000 + 7 * e + n) for e in range(ne)])
        wdev = torch.from_numpy(raw).cuda()
        rng = np.random.default_rng(n_tokens + ne)
        ids = rng.integers(0, ne, size=n_tokens * top_k).astype(np.uint32)
        if ne >= 16:
            ids[ids == 3] = 5                      # an expert that receives no rows at all
        xd, xs = _dev_x(make_x(n_tokens, k, seed=11), bf16)
        rows = n_tokens * top_k
        y = torch.full((rows, n), float("nan"), device="cuda")
        p = hq.GgmlQuantizedMatmulIdParams(n_tokens, top_k, n, k, ne, stride, t)
        scratch = hq.IdMmScratch.alloc(gpu_ctx, ne, rows, k)
        assert scratch.nbytes > 0
        hq.quantized_matmul_id_ggml(gpu_ctx, xd, wdev.data_ptr(), torch.from_numpy(ids.view(np.int32)).cuda(), y, scratch, p)
        gpu_ctx.check_status()
        want = oracle.qmatmul_id(t, raw, stride, xs, ids, n_tokens, top_k, n, k, ne)
        got = y.cpu().numpy()
        assert np.isfinite(got).all()
        assert rel_l2(got, want) < GATE, (t, ne, n, k, n_tokens, top_k, rel_l2(got, want))


def test_mul_mat_id_grouped_needs_scratch_and_reports_bad_ids(gpu_ctx):
    t, ne, n, k, rows = oracle.Q4_K, 4, 128, 256, 64
    stride = hq.expert_stride(t, n, k)
    raw = np.concatenate([make_quant_weight(t, n, k, seed=e) for e in range(ne)])
    wdev = torch.from_numpy(raw).cuda()
    ids_np = np.random.default_rng(3).integers(0, ne, size=rows).astype(np.int32)
    ids_np[10] = 99                                  # out of range
    ids = torch.from_numpy(ids_np).cuda()
    xd, xs = _dev_x(make_x(rows, k, seed=4), True)
    y = torch.full((rows, n), 7.0, device="cuda")
    p = hq.GgmlQuantizedMatmulIdParams(rows, 1, n, k, ne, stride, t)
    with pytest.raises(hq.Hf2qError) as ei:
        hq.quantized_matmul_id_ggml(gpu_ctx, xd, wdev.data_ptr(), ids, y, None, p)
    assert ei.value.status == _lib.ERR_WORKSPACE
    scratch = hq.IdMmScratch.alloc(gpu_ctx, ne, rows, k)
    hq.quantized_matmul_id_ggml(gpu_ctx, xd, wdev.data_ptr(), ids, y, scratch, p)
    with pytest.raises(hq.Hf2qError):
        gpu_ctx.check_status()
    got = y.cpu().numpy()
    assert np.all(got[10] == 0)
    good = np.ones(rows, bool); good[10] = False
    ids_ok = ids_np.astype(np.uint32).copy(); ids_ok[10] = 0
    want = oracle.qmatmul_id(t, raw, stride, xs, ids_ok, rows, 1, n, k, ne)
    assert rel_l2(got[good], want[good]) < GATE


def test_bad_expert_id_is_reported_not_faulted(gpu_ctx):
    t, ne, n, k = oracle.Q4_K, 2, 16, 256
    stride = hq.expert_stride(t, n, k)
    raw = np.concatenate([make_quant_weight(t, n, k, seed=e) for e in range(ne)])
    wdev = torch.from_numpy(raw).cuda()
    ids = torch.tensor([0, 7], dtype=torch.int32, device="cuda")
    x = torch.randn(2, k, device="cuda")
    y = torch.full((2, n), 5.0, device="cuda")
    hq.quantized_matmul_id_ggml(gpu_ctx, x, wdev.data_ptr(), ids, y, None, hq.GgmlQuantizedMatmulIdParams(2, 1, n, k, ne, stride, t))
    with pytest.raises(hq.Hf2qError) as ei:
        gpu_ctx.check_status()
    assert ei.value.status == _lib.ERR_INVALID_ARGUMENT
    assert torch.all(y[1] == 0)
    gpu_ctx.check_status()          # the word was cleared; the context stays usable


# ---------------------------------------------------------------- router
def test_softmax_topk_matches_oracle(gpu_ctx):
    for (T, E, k) in [(1, 256, 8), (33, 256, 8), (5, 64, 4), (7, 128, 40)]:
        logits = np.random.default_rng(T + E).standard_normal((T, E)).astype(np.float32)
        ids, w = hq.moe_softmax_topk(gpu_ctx, torch.from_numpy(logits).cuda(), k)
        ids_o, w_o = oracle.softmax_topk_renorm(logits, k)
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ids_o)
        assert np.allclose(w.cpu().numpy(), w_o, rtol=2e-6, atol=1e-8)
    logits = np.zeros((2, 16), np.float32)       # all ties: lowest indices win, in order
    ids, w = hq.moe_softmax_topk(gpu_ctx, torch.from_numpy(logits).cuda(), 4)
    assert ids.cpu().numpy().reshape(2, 4).tolist() == [[0, 1, 2, 3]] * 2
    assert np.allclose(w.cpu().numpy(), 0.25)


# ---------------------------------------------------------------- error behaviour
def test_invalid_arguments_are_errors_not_fallbacks(gpu_ctx):
    t, n, k = oracle.Q4_K, 16, 256
    w = hq.load_quant_weight(gpu_ctx, make_quant_weight(t, n, k, seed=1), t, n, k)
    x = torch.randn(1, k, device="cuda")
    y = torch.empty(1, n, device="cuda")
    with pytest.raises(hq.Hf2qError):      # params disagree with the weight
        hq.quantized_matmul_ggml(gpu_ctx, x, w, y, hq.GgmlQuantizedMatmulParams(1, n, k, oracle.Q6_K))
    with pytest.raises(hq.Hf2qError):      # f16 activations are not part of the op surface
        hq.quantized_matmul_ggml(gpu_ctx, x.half(), w, y, w.matmul_params(1))
    lib = _lib.load()
    rc = lib.hf2q_cuda_qmatmul(gpu_ctx._h, None, x.data_ptr(), 0, w.ptr, y.data_ptr(), 1, n, k, 10, None, 0)
    assert rc == _lib.ERR_UNSUPPORTED_TYPE     # Q2_K: not on this path
    rc = lib.hf2q_cuda_qmatmul(gpu_ctx._h, None, x.data_ptr(), 0, w.ptr, y.data_ptr(), 1, n, k + 32, t, None, 0)
    assert rc == _lib.ERR_INVALID_ARGUMENT
    with pytest.raises(hq.Hf2qError):
        hq.load_quant_weight(gpu_ctx, np.zeros(100, np.uint8), t, n, k)
    # m == 0 and n_tokens == 0 are no-ops, not errors
    assert lib.hf2q_cuda_qmatmul(gpu_ctx._h, None, x.data_ptr(), 0, w.ptr, y.data_ptr(), 0, n, k, t, None, 0) == 0


def test_gguf_file_feeds_the_kernels(gpu_ctx, tmp_path):
    """GGUF file -> reader -> raw-block upload -> product: the loader contract end to end."""
    from hf2q_b200 import gguf
    t, n, k = oracle.Q6_K, 64, 2048
    raw = make_quant_weight(t, n, k, seed=77)
    wtr = gguf.GgufWriter()
    wtr.add_kv("general.architecture", gguf.T_STRING, "test")
    wtr.add_tensor("blk.0.ffn_down.weight", (n, k), t, raw)
    path = tmp_path / "w.gguf"
    wtr.write(path)
    with gguf.GgufFile(path) as g:
        w = g.load_quant_weight(gpu_ctx, "blk.0.ffn_down.weight")
        assert (w.rows, w.cols, w.ggml_type) == (n, k, t)
        xd, xs = _dev_x(make_x(2, k, seed=1), True)
        y = torch.empty((2, n), device="cuda")
        hq.quantized_matmul_ggml(gpu_ctx, xd, w, y, w.matmul_params(2))
        assert rel_l2(y.cpu().numpy(), _ref(t, raw, xs, n, k)) < 2e-5
        deq = hq.dequantize(gpu_ctx, w).cpu().numpy()
        assert np.array_equal(deq.view(np.uint32), oracle.dequantize(t, raw).reshape(n, k).view(np.uint32))


def test_gather_entry_single_rank(gpu_ctx):
    """hf2q_cuda_qmatmul_gather with one rank: columns land at col0 of a wider buffer, the wait kernel
    and the in-kernel wait pass at once, phases (long rows) accumulate in the buffer."""
    import ctypes as C
    from hf2q_b200.dist import _Gather
    lib, h = gpu_ctx._lib, gpu_ctx._h
    # (Q4_K with 1, 2 and 4 blocks per row: the stacked row groups of short rows -- the O shard of a tensor-parallel decoder)
    for (t, n, k, m) in ((oracle.Q6_K, 48, 2048, 3), (oracle.Q6_K, 32, 14336, 8), (oracle.Q4_K, 200, 512, 2), (oracle.Q4_K, 72, 256, 1),
                         (oracle.Q4_K, 130, 1024, 4)):
        raw = make_quant_weight(t, n, k, seed=n + k)
        w = hq.load_quant_weight(gpu_ctx, raw, t, n, k)
        n_total, col0 = n + 40, 24
        ybuf, fbuf = C.c_void_p(), C.c_void_p()
        hy, hf = (C.c_uint8 * 64)(), (C.c_uint8 * 64)()
        gpu_ctx._check(lib.hf2q_cuda_ipc_alloc(h, m * n_total * 4, C.byref(ybuf), hy))
        gpu_ctx._check(lib.hf2q_cuda_ipc_alloc(h, 256, C.byref(fbuf), hf))
        g = _Gather()
        g.y_all[0], g.flags[0] = ybuf.value, fbuf.value
        g.n_ranks, g.rank, g.n_total, g.col0, g.wait_previous = 1, 0, n_total, col0, 1
        g.n_rows[0] = n
        xd, xs = _dev_x(make_x(m, k, seed=3), True)
        for _ in range(2):        # the second call waits (trivially) for the first
            gpu_ctx._check(lib.hf2q_cuda_qmatmul_gather(h, gpu_ctx._stream(), xd.data_ptr(), hq.ops.DT_BF16, w.ptr, C.byref(g),
                                                        m, n, k, t))
        gpu_ctx._check(lib.hf2q_cuda_gather_wait(h, gpu_ctx._stream(), C.byref(g)))
        gpu_ctx.check_status()
        from hf2q_b200.dist import _DevView
        y = torch.as_tensor(_DevView(ybuf.value, (m, n_total), "<f4"), device="cuda").cpu().numpy()
        assert rel_l2(y[:, col0:col0 + n], _ref(t, raw, xs, n, k)) < 2e-5
        assert not y[:, :col0].any() and not y[:, col0 + n:].any()          # nothing outside the rank's columns
        if m == 1:
            # the exchange without a product, and the sum of the gathered parts into a vector
            src = torch.arange(16, dtype=torch.float32, device="cuda")
            g.col0, g.n_rows[0] = 4, 16
            gpu_ctx._check(lib.hf2q_cuda_gather_copy(h, gpu_ctx._stream(), C.byref(g), src.data_ptr(), 16))
            acc = torch.ones(8, device="cuda")
            gpu_ctx._check(lib.hf2q_cuda_gather_sum(h, gpu_ctx._stream(), C.byref(g), acc.data_ptr(), 8, 2))
            gpu_ctx.check_status()
            y2 = torch.as_tensor(_DevView(ybuf.value, (1, n_total), "<f4"), device="cuda").cpu().numpy()[0]
            assert np.array_equal(y2[4:20], np.arange(16, dtype=np.float32))
            assert np.array_equal(acc.cpu().numpy(), 1.0 + y2[0:8] + y2[8:16])
            assert lib.hf2q_cuda_gather_supported(h, w.ptr, 1, n, k, t, 0) == 1
        lib.hf2q_cuda_free(h, ybuf.value)
        lib.hf2q_cuda_free(h, fbuf.value)
    # argument checks
    g = _Gather()
    assert lib.hf2q_cuda_qmatmul_gather(h, None, xd.data_ptr(), hq.ops.DT_BF16, w.ptr, C.byref(g), 1, n, k, t) == _lib.ERR_INVALID_ARGUMENT
    odd = hq.load_quant_weight(gpu_ctx, make_quant_weight(oracle.Q6_K, 16, 1792, seed=1), oracle.Q6_K, 16, 1792)      # 1470-byte rows
    assert lib.hf2q_cuda_gather_supported(h, odd.ptr, 1, 16, 1792, oracle.Q6_K, 0) == 0


def test_gather_host_batch_single_rank(gpu_ctx):
    """hf2q_cuda_qmatmul_gather_host_batch with one rank: host activations in, the products through the gathering
    mat-vec into the group's two alternating buffers, the rows lifted out by the wait-and-take launch and copied to the
    host; an item without y_host runs but returns nothing; the buffer parity is the caller's."""
    import ctypes as C
    from hf2q_b200.dist import _Gather
    lib, h = gpu_ctx._lib, gpu_ctx._h
    specs = [(oracle.Q6_K, 48, 2048, 3), (oracle.Q4_K, 200, 512, 8), (oracle.Q5_K, 64, 1024, 1), (oracle.Q8_0, 96, 256, 4),
             (oracle.Q4_0, 40, 512, 2)]
    n_total, max_m = 256, 8
    buf_bytes = (max_m * n_total * 4 + 255) & ~255
    ybuf, fbuf = C.c_void_p(), C.c_void_p()
    hy, hf = (C.c_uint8 * 64)(), (C.c_uint8 * 64)()
    gpu_ctx._check(lib.hf2q_cuda_ipc_alloc(h, 2 * buf_bytes, C.byref(ybuf), hy))
    gpu_ctx._check(lib.hf2q_cuda_ipc_alloc(h, 256, C.byref(fbuf), hf))
    g = _Gather()
    g.y_all[0], g.flags[0] = ybuf.value, fbuf.value
    g.n_ranks, g.rank, g.n_total, g.col0, g.wait_previous = 1, 0, n_total, 0, 1
    raws = [make_quant_weight(t, n, k, seed=70 + i) for i, (t, n, k, m) in enumerate(specs)]
    ws = [hq.load_quant_weight(gpu_ctx, raw, t, n, k) for raw, (t, n, k, m) in zip(raws, specs)]
    xs_t = [torch.from_numpy(make_x(m, k, seed=80 + i)).bfloat16() for i, (t, n, k, m) in enumerate(specs)]
    xs_h = [xt.view(torch.int16).numpy() for xt in xs_t]
    ys = [np.full((m, n), np.nan, np.float32) if i != 2 else None for i, (t, n, k, m) in enumerate(specs)]
    batch = hq.ops.HostBatch([(xh, w, y, m, hq.ops.DT_BF16) for xh, w, y, (t, n, k, m) in zip(xs_h, ws, ys, specs)])
    parity = 0
    for rep in range(3):
        gpu_ctx._check(lib.hf2q_cuda_qmatmul_gather_host_batch(h, C.byref(g), buf_bytes, parity, C.cast(batch.array, C.c_void_p), len(batch)))
        parity ^= len(batch) & 1
        hq.ops.host_sync(gpu_ctx)
        gpu_ctx.check_status()
        for i, (xt, y, raw, (t, n, k, m)) in enumerate(zip(xs_t, ys, raws, specs)):
            if y is None:
                continue
            assert rel_l2(y, _ref(t, raw, xt.float().numpy(), n, k)) < GATE, (rep, t, n, k, m)
            y[...] = np.nan
    # argument checks: no group, a product wider than the group's buffer
    assert lib.hf2q_cuda_qmatmul_gather_host_batch(h, None, buf_bytes, 0, C.cast(batch.array, C.c_void_p), len(batch)) == _lib.ERR_INVALID_ARGUMENT
    g.n_total = 100
    assert lib.hf2q_cuda_qmatmul_gather_host_batch(h, C.byref(g), buf_bytes, 0, C.cast(batch.array, C.c_void_p), len(batch)) == _lib.ERR_INVALID_ARGUMENT
    lib.hf2q_cuda_free(h, ybuf.value)
    lib.hf2q_cuda_free(h, fbuf.value)


@pytest.mark.parametrize("t", TYPES)
def test_device_dequant_of_golden_blocks_reencodes_to_the_stored_codes(gpu_ctx, golden_dir, t):
    """The reference's quantizers recompute the codes from (x + dmin*m) / (d*sc) with the stored
    scales; the DEVICE dequantiser's values of the reference's golden blocks must give every
    stored code back through that step."""
    from tests.util import reencode_codes, stored_codes
    name, n = FIXTURES[t]
    for variant in ("noim", "im"):
        raw = np.fromfile(golden_dir / f"{name}_{n}_{variant}_expected.bin", dtype=np.uint8)
        w = hq.load_quant_weight(gpu_ctx, raw, t, 2, n)
        y = hq.dequantize(gpu_ctx, w).cpu().numpy().reshape(-1)
        codes, valid = reencode_codes(t, raw, y)
        assert np.array_equal(codes[valid], stored_codes(t, raw)[valid])


@pytest.mark.parametrize("m", [1, 6, 72, 300])
def test_row_range_type_map(gpu_ctx, m):
    """hf2q_cuda_qmatmul_segments: a fused-QKV-like matrix whose last rows are Q6_K and the rest Q4_K
    (plus a Q5_K middle range), one call, against the f64 product on the oracle's weights."""
    k = 2048
    segs = [(oracle.Q4_K, 320), (oracle.Q5_K, 48), (oracle.Q6_K, 136)]
    raws = [make_quant_weight(t, rows, k, seed=900 + i) for i, (t, rows) in enumerate(segs)]
    ws = [hq.load_quant_weight(gpu_ctx, raw, t, rows, k) for raw, (t, rows) in zip(raws, segs)]
    n = sum(rows for _, rows in segs)
    xd, xs = _dev_x(make_x(m, k, seed=m), True)
    y = torch.full((m, n), float("nan"), device="cuda")
    hq.ops.quantized_matmul_segments(gpu_ctx, xd, ws, y, m)
    gpu_ctx.check_status()
    want = np.concatenate([_ref(t, raw, xs, rows, k) for raw, (t, rows) in zip(raws, segs)], axis=1)
    assert rel_l2(y.cpu().numpy(), want) < GATE
    # the same ranges through separate calls give the same bits
    c0 = 0
    for w, (t, rows) in zip(ws, segs):
        yi = torch.empty((m, rows), device="cuda")
        hq.quantized_matmul_ggml(gpu_ctx, xd, w, yi, w.matmul_params(m))
        assert torch.equal(yi, y[:, c0:c0 + rows])
        c0 += rows
    # a range the selected kernel cannot take is an error, not a detour
    bad = hq.load_quant_weight(gpu_ctx, make_quant_weight(oracle.Q4_0, 16, 96, seed=1), oracle.Q4_0, 16, 96)
    with pytest.raises(hq.Hf2qError):
        hq.ops.quantized_matmul_segments(gpu_ctx, torch.zeros((2, 96), device="cuda"), [bad], torch.empty((2, 16), device="cuda"), 2)
