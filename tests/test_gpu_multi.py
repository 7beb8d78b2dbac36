"""Two-GPU tests of the sharded paths over NCCL (skipped on a single-GPU box): row-sharded dense
product + all-gather, and expert-parallel mul_mat_id + all-to-all, with the CUDA library doing the
local compute and the CPU oracle as the checker."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist

    import oracle
    import hf2q_b200 as hq
    from hf2q_b200 import dist as hd
    from tests.util import make_quant_weight, make_x, rel_l2

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = hq.GpuContext(rank)
        ok = True
        # --- dense: rows sharded, outputs all-gathered
        t, n, k, m = oracle.Q6_K, 512, 2048, 4
        raw = make_quant_weight(t, n, k, seed=3)
        rb = oracle.row_bytes(t, k)
        r0, r1 = hd.shard_rows(n, world, rank)
        w = hq.load_quant_weight(ctx, raw[r0 * rb:r1 * rb], t, r1 - r0, k)
        x = make_x(m, k, seed=4)
        xd = torch.from_numpy(x).cuda()

        def local(xx):
            y = torch.empty((m, r1 - r0), device="cuda")
            hq.quantized_matmul_ggml(ctx, xx, w, y, w.matmul_params(m))
            return y

        y = hd.rowshard_matmul(xd, local, n).cpu().numpy()
        want = oracle.matmul_f64(x, oracle.dequantize(t, raw).reshape(n, k))
        ok &= rel_l2(y, want) < 1e-3
        # --- dense again, all-gather inside the kernel (peer stores + arrival counters), a chain of
        # products where each waits for the previous one's columns from every rank
        gg = hd.GatherGroup(ctx, 8, n)
        xb = make_x(8, k, seed=5)
        for step, mm in enumerate((1, 4, 8, 3)):
            xs = torch.from_numpy(xb[:mm] * (step + 1)).cuda().bfloat16()          # bf16: up to 8 rows per launch
            gg.matmul(xs, w, mm, r0, wait_previous=step > 0)
            gg.wait()
            torch.cuda.synchronize()
            got = gg.output(mm).cpu().numpy()
            ok &= rel_l2(got, oracle.matmul_f64(xs.float().cpu().numpy(), oracle.dequantize(t, raw).reshape(n, k))) < 1e-3
            dist.barrier()                      # nobody overwrites the buffers while a peer still reads them
        # the same chain from a CUDA graph (no collective call inside): replay twice
        xs = torch.from_numpy(xb[:2]).cuda().bfloat16()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            gg.matmul(xs, w, 2, r0)
            gg.matmul(xs, w, 2, r0, wait_previous=True)
            gg.wait()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        ok &= rel_l2(gg.output(2).cpu().numpy(), oracle.matmul_f64(xs.float().cpu().numpy(), oracle.dequantize(t, raw).reshape(n, k))) < 1e-3
        dist.barrier()
        gg.close()
        # --- MoE: experts sharded, routed rows exchanged
        t, E, n, k = oracle.Q5_K, 8, 256, 512
        stride = hq.expert_stride(t, n, k)
        raw = np.concatenate([make_quant_weight(t, n, k, seed=60 + e) for e in range(E)])
        e_local = E // world
        mine = torch.from_numpy(raw[rank * e_local * stride:(rank + 1) * e_local * stride]).cuda()
        rows = 90 + 10 * rank
        rng = np.random.default_rng(rank)
        ids = rng.integers(0, E, size=rows).astype(np.int32)
        xr = make_x(rows, k, seed=70 + rank)

        def local_id(xx, lids):
            r = xx.shape[0]
            yy = torch.empty((r, n), device="cuda")
            sc = hq.IdMmScratch.alloc(ctx, e_local, r, k)
            hq.quantized_matmul_id_ggml(ctx, xx.contiguous(), mine.data_ptr(), lids.contiguous(), yy, sc,
                                        hq.GgmlQuantizedMatmulIdParams(r, 1, n, k, e_local, stride, t))
            return yy

        got = hd.ep_mul_mat_id(torch.from_numpy(xr).cuda(), torch.from_numpy(ids).cuda(), E, n, local_id).cpu().numpy()
        want = oracle.qmatmul_id(t, raw, stride, xr, ids.astype(np.uint32), rows, 1, n, k, E)
        ok &= rel_l2(got, want) < 1e-3
        ctx.check_status()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_gpu_rowshard_and_expert_parallel():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        world = 4 if torch.cuda.device_count() >= 4 else 2      # four ranks also cover the several-peers form of the fused gather
        procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
            assert p.exitcode == 0
        assert all(ret.get(r) for r in range(world))
