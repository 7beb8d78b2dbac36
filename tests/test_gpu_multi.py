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
        # --- dense again, all-gather inside the kernel (peer stores + per-source arrival counters)
        gg = hd.GatherGroup(ctx, 8, n)
        xb = make_x(8, k, seed=5)
        wfull = oracle.dequantize(t, raw).reshape(n, k)
        for step, mm in enumerate((1, 4, 8, 3)):
            xs = torch.from_numpy(xb[:mm] * (step + 1)).cuda().bfloat16()          # bf16: up to 8 rows per launch
            gg.matmul(xs, w, mm, r0, wait_previous=step > 0)
            gg.wait()
            torch.cuda.synchronize()
            got = gg.output(mm).cpu().numpy()
            ok &= rel_l2(got, oracle.matmul_f64(xs.float().cpu().numpy(), wfull)) < 1e-3
        dist.barrier()
        gg.close()
        # --- a real chain: the gathered output of every product is the next product's activations, no host
        # synchronisation in between, uneven shards (different CTA counts per rank), two alternating buffers
        nt = 768
        sizes = [400, 368] if world == 2 else [200, 184, 192, 192][:world]
        assert sum(sizes) == nt
        c0 = sum(sizes[:rank])
        raws = [make_quant_weight(oracle.Q6_K, nt, 2048, seed=11), make_quant_weight(oracle.Q4_K, nt, nt, seed=12),
                make_quant_weight(oracle.Q5_K, nt, nt, seed=13), make_quant_weight(oracle.Q8_0, nt, nt, seed=14)]
        types = [oracle.Q6_K, oracle.Q4_K, oracle.Q5_K, oracle.Q8_0]      # (Q6_K rows of 768 elements are not 16-byte aligned)
        ks = [2048, nt, nt, nt]
        shards = []
        for tt, rw, kk in zip(types, raws, ks):
            rbk = oracle.row_bytes(tt, kk)
            shards.append(hq.load_quant_weight(ctx, rw[c0 * rbk:(c0 + sizes[rank]) * rbk], tt, sizes[rank], kk))
        gg = hd.GatherGroup(ctx, 4, nt)
        mm = 3
        x0 = make_x(mm, 2048, seed=21)
        x0d = torch.from_numpy(x0).cuda()
        want = [x0.astype(np.float64)]
        for tt, rw, kk in zip(types, raws, ks):
            want.append(want[-1] @ oracle.dequantize(tt, rw).reshape(nt, kk).astype(np.float64).T * 8.0)

        def chain(snapshots):
            xin = x0d
            for i, wsh in enumerate(shards):
                gg.matmul(xin, wsh, mm, None, wait_previous=i > 0, n_rows=sizes)
                xin = gg.output(mm)
                # (a model would normalise here; a scale keeps the values away from zero)
                # the scale runs as a torch kernel on the same stream AFTER a wait, so it reads complete data
                gg.wait()
                xin.mul_(8.0)
                if snapshots is not None:
                    snapshots.append(xin.clone())
            gg.wait()

        snaps = []
        chain(snaps)
        torch.cuda.synchronize()
        for i, sn in enumerate(snaps):
            ok &= rel_l2(sn.cpu().numpy(), want[i + 1]) < 1e-3
        dist.barrier()
        # the products alone, back to back (each waits inside the kernel for the previous one's columns),
        # captured in a graph and replayed: 4 products = an even number, so buffers alternate consistently
        def bare_chain():
            xin = x0d
            for i, wsh in enumerate(shards):
                gg.matmul(xin, wsh, mm, None, wait_previous=True, n_rows=sizes)
                xin = gg.output(mm)
            gg.wait()

        want_b = [x0.astype(np.float64)]
        for tt, rw, kk in zip(types, raws, ks):
            want_b.append(want_b[-1] @ oracle.dequantize(tt, rw).reshape(nt, kk).astype(np.float64).T)
        bare_chain()
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            bare_chain()
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
        ok &= rel_l2(gg.output(mm).cpu().numpy(), want_b[-1]) < 1e-3
        ctx.check_status()
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
        # --- the same two schemes through the library's own C entries (NCCL inside the library)
        comm = hd.Comm(ctx)
        got_c = comm.qmatmul_id_ep(torch.from_numpy(xr).cuda(), torch.from_numpy(ids).cuda(), mine.data_ptr(), n, k, E, stride, t,
                                   cap_recv=world * 130).cpu().numpy()
        ok &= rel_l2(got_c, want) < 1e-3
        # dense, rows sharded, mat-vec (m = 4) and tensor-core (m = 40) sizes
        td, nd, kd = oracle.Q6_K, 512, 2048
        rawd = make_quant_weight(td, nd, kd, seed=3)
        rbd = oracle.row_bytes(td, kd)
        nl = nd // world
        wsh = hq.load_quant_weight(ctx, rawd[rank * nl * rbd:(rank + 1) * nl * rbd], td, nl, kd)
        wd_full = oracle.dequantize(td, rawd).reshape(nd, kd)
        for mm in (4, 40):
            xm = make_x(mm, kd, seed=90 + mm)
            yc = comm.qmatmul_rowshard(torch.from_numpy(xm).cuda(), wsh, mm).cpu().numpy()
            ok &= rel_l2(yc, oracle.matmul_f64(xm, wd_full)) < 1e-3
        # the whole expert FFN expert-parallel: gate, up, SwiGLU and down at the owner, one exchange each way
        H, I = 512, 256
        sg, sdn = hq.expert_stride(t, I, H), hq.expert_stride(t, H, I)
        rg = np.concatenate([make_quant_weight(t, I, H, seed=100 + e) for e in range(E)])
        ru = np.concatenate([make_quant_weight(t, I, H, seed=200 + e) for e in range(E)])
        rdn = np.concatenate([make_quant_weight(t, H, I, seed=300 + e) for e in range(E)])
        lg = torch.from_numpy(rg[rank * e_local * sg:(rank + 1) * e_local * sg]).cuda()
        lu = torch.from_numpy(ru[rank * e_local * sg:(rank + 1) * e_local * sg]).cuda()
        ldn = torch.from_numpy(rdn[rank * e_local * sdn:(rank + 1) * e_local * sdn]).cuda()
        xe = make_x(rows, H, seed=80 + rank)
        ye = comm.moe_experts_ep(torch.from_numpy(xe).cuda(), torch.from_numpy(ids).cuda(), lg.data_ptr(), lu.data_ptr(), ldn.data_ptr(),
                                 H, I, E, sg, sdn, t, t, cap_recv=world * 130).cpu().numpy()
        want_e = np.empty((rows, H))
        for r in range(rows):
            e = int(ids[r])
            gf = oracle.dequantize(t, rg[e * sg:(e + 1) * sg]).reshape(I, H).astype(np.float64)
            uf = oracle.dequantize(t, ru[e * sg:(e + 1) * sg]).reshape(I, H).astype(np.float64)
            df = oracle.dequantize(t, rdn[e * sdn:(e + 1) * sdn]).reshape(H, I).astype(np.float64)
            a, b = gf @ xe[r].astype(np.float64), uf @ xe[r].astype(np.float64)
            want_e[r] = df @ ((a / (1.0 + np.exp(-a))) * b)
        ok &= rel_l2(ye, want_e) < 2e-3
        torch.cuda.synchronize()
        comm.close()
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
        try:
            for p in procs:
                p.join(300)
        finally:
            # a rank stuck in a collective must not keep its GPU after the test
            for p in procs:
                if p.is_alive():
                    p.terminate()
                    p.join(10)
                    if p.is_alive():
                        p.kill()
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert all(ret.get(r) for r in range(world))


def _two_device_main(ret):
    import oracle
    import hf2q_b200 as hq
    from tests.util import make_quant_weight, make_x, rel_l2

    ok = True
    ctxs = [hq.GpuContext(0), hq.GpuContext(1)]
    for t, n, k in ((oracle.Q6_K, 300, 4096), (oracle.Q4_K, 256, 2048)):
        raw = make_quant_weight(t, n, k, seed=n)
        wref = oracle.dequantize(t, raw).reshape(n, k)
        for d, ctx in enumerate(ctxs):
            with torch.cuda.device(d):
                w = hq.load_quant_weight(ctx, raw, t, n, k)
                for m in (2, 72):                               # mat-vec and tensor-core GEMM: both need > 48 KB of shared memory
                    x = make_x(m, k, seed=m + d)
                    xd = torch.from_numpy(x).to(f"cuda:{d}")
                    y = torch.empty((m, n), device=f"cuda:{d}")
                    hq.quantized_matmul_ggml(ctx, xd, w, y, w.matmul_params(m))
                    ctx.check_status()
                    ok &= rel_l2(y.cpu().numpy(), oracle.matmul_f64(x, wref)) < 1e-3
    ret["ok"] = bool(ok)


def test_one_process_two_devices():
    """Contexts on two GPUs in one process: the shared-memory opt-in of every kernel is per device."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        p = ctx.Process(target=_two_device_main, args=(ret,))
        p.start()
        try:
            p.join(240)
        finally:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
        assert p.exitcode == 0 and ret.get("ok")
