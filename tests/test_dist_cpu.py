"""world_size-2 gloo tests of the multi-GPU host logic (row-sharded all-gather, expert-parallel
all-to-all).  The local compute is the CPU oracle, so these run without a GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from hf2q_b200 import dist as hd
from tests.util import make_quant_weight, make_x


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def _run(fn, world=2):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, fn, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        return dict(ret)


def test_shard_rows_covers_everything():
    for n, w in [(4096, 8), (6144, 4), (10, 3), (7, 8)]:
        spans = [hd.shard_rows(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1


T_DENSE, N_DENSE, K_DENSE = oracle.Q6_K, 52, 512       # 52 rows over 2 ranks: even; 51 would be ragged


def _dense_case(rank, world, n=N_DENSE):
    raw = make_quant_weight(T_DENSE, n, K_DENSE, seed=5)
    rb = oracle.row_bytes(T_DENSE, K_DENSE)
    r0, r1 = hd.shard_rows(n, world, rank)
    shard = raw[r0 * rb:r1 * rb]                          # a row shard is a byte slice
    x = torch.from_numpy(make_x(3, K_DENSE, seed=6))

    def local(xx):
        y, _, _ = oracle.qmatmul(T_DENSE, shard, xx.numpy(), r1 - r0, K_DENSE)
        return torch.from_numpy(y)

    return hd.rowshard_matmul(x, local, n).numpy()


def _dense_ragged(rank, world):
    return _dense_case(rank, world, n=51)


@pytest.mark.parametrize("fn,n", [(_dense_case, N_DENSE), (_dense_ragged, 51)])
def test_rowshard_allgather_matches_unsharded(fn, n):
    out = _run(fn)
    raw = make_quant_weight(T_DENSE, n, K_DENSE, seed=5)
    want, _, _ = oracle.qmatmul(T_DENSE, raw, make_x(3, K_DENSE, seed=6), n, K_DENSE)
    for r in range(2):
        assert np.array_equal(out[r], want)


T_MOE, E_MOE, N_MOE, K_MOE = oracle.Q5_K, 8, 24, 256


def _moe_case(rank, world):
    stride = N_MOE * oracle.row_bytes(T_MOE, K_MOE)
    raw = np.concatenate([make_quant_weight(T_MOE, N_MOE, K_MOE, seed=40 + e) for e in range(E_MOE)])
    e_local = E_MOE // world
    mine = raw[rank * e_local * stride:(rank + 1) * e_local * stride]      # experts sharded by expert
    rng = np.random.default_rng(100 + rank)                                # each rank routes its own rows
    rows = 11 + 3 * rank
    ids = torch.from_numpy(rng.integers(0, E_MOE, size=rows).astype(np.int32))
    if rank == 1:
        ids[:] = ids % e_local                                             # rank 1 sends nothing to itself... all to rank 0
    x = torch.from_numpy(rng.standard_normal((rows, K_MOE)).astype(np.float32))

    def local(xx, lids):
        y = oracle.qmatmul_id(T_MOE, mine, stride, xx.numpy(), lids.numpy().astype(np.uint32), xx.shape[0], 1, N_MOE, K_MOE, e_local)
        return torch.from_numpy(y)

    got = hd.ep_mul_mat_id(x, ids, E_MOE, N_MOE, local).numpy()
    want = oracle.qmatmul_id(T_MOE, raw, stride, x.numpy(), ids.numpy().astype(np.uint32), rows, 1, N_MOE, K_MOE, E_MOE)
    return bool(np.array_equal(got, want))


def test_expert_parallel_all_to_all_matches_single_rank():
    out = _run(_moe_case)
    assert out[0] and out[1]
