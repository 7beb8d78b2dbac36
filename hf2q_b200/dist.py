"""Multi-GPU wrappers of the quantized-matmul path: one process per GPU, torch.distributed plumbing.

The reference is single-device (no collective exists in hf2q), so both schemes are new:

* dense weights are sharded by OUTPUT ROWS -- a shard is a contiguous byte range of the raw block
  bytes -- and every product is followed by an all-gather of the output columns;
* MoE experts are sharded BY EXPERT (E / world per rank); routed rows travel to the rank that owns
  their expert with an all-to-all, are multiplied there by the local grouped product, and travel
  back with a second all-to-all.

The functions take the local compute as a callable, so the same host logic runs over NCCL with
the CUDA library and over gloo on CPU in the tests.  With those, remote data always lands in local
memory (the collective's receive buffer) before any kernel reads it.

``GatherGroup`` is the fused form of the dense scheme for 1..8 activation rows: the mat-vec kernel
itself stores this rank's columns into every rank's output buffer (peer memory mapped through CUDA
IPC) and bumps the peers' arrival counters, so a decode step needs no collective call at all and
can be replayed from a CUDA graph.  Plain stores only: no multicast, no TMA on peer memory.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Sequence

import torch
import torch.distributed as dist


def shard_rows(n: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [r0, r1) of an n-row weight owned by `rank`: contiguous, sizes differ by at most one."""
    base, rem = divmod(n, world)
    r0 = rank * base + min(rank, rem)
    return r0, r0 + base + (1 if rank < rem else 0)


def rowshard_matmul(x: torch.Tensor, local_matmul: Callable[[torch.Tensor], torch.Tensor], n: int,
                    group=None) -> torch.Tensor:
    """y[m, n] = x . W^T with W sharded by rows: local product, then all-gather of the columns.

    ``local_matmul(x)`` returns this rank's [m, n_local] float32 block (n_local from shard_rows)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    y_local = local_matmul(x)
    m = y_local.shape[0]
    sizes = [shard_rows(n, world, r)[1] - shard_rows(n, world, r)[0] for r in range(world)]
    assert y_local.shape[1] == sizes[rank]
    if world == 1:
        return y_local
    pad = max(sizes)
    if len(set(sizes)) == 1:
        out = torch.empty((world * m, pad), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(out, y_local.contiguous(), group=group)
        return out.view(world, m, pad).permute(1, 0, 2).reshape(m, n)
    send = torch.zeros((m, pad), dtype=y_local.dtype, device=y_local.device)
    send[:, : sizes[rank]] = y_local
    parts = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(parts, send, group=group)
    return torch.cat([p[:, :s] for p, s in zip(parts, sizes)], dim=1)


def expert_owner(ids: torch.Tensor, n_experts: int, world: int) -> torch.Tensor:
    """Rank that owns each routed row's expert (experts are split into `world` equal ranges)."""
    assert n_experts % world == 0, "experts must divide evenly over the ranks"
    return torch.div(ids.to(torch.int64), n_experts // world, rounding_mode="floor")


def ep_mul_mat_id(x_rows: torch.Tensor, ids: torch.Tensor, n_experts: int, n_out: int,
                  local_mul_mat_id: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], group=None) -> torch.Tensor:
    """Expert-parallel mul_mat_id.

    x_rows: [R, k] activations, one row per routed row held by THIS rank; ids: [R] global expert ids.
    ``local_mul_mat_id(x, local_ids)`` multiplies rows by this rank's experts (ids relative to the
    rank's first expert) and returns [rows, n_out] float32.  Returns [R, n_out] in the caller's order.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    e_local = n_experts // world
    if world == 1:
        return local_mul_mat_id(x_rows, ids)
    owner = expert_owner(ids, n_experts, world)
    order = torch.sort(owner, stable=True).indices                  # rows grouped by destination rank
    send_counts = torch.bincount(owner, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)   # how many rows each peer sends us
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    x_send = x_rows.index_select(0, order).contiguous()
    id_send = (ids.index_select(0, order).to(torch.int64) - owner.index_select(0, order) * e_local).to(torch.int32).contiguous()
    x_recv = torch.empty((sum(rc), x_rows.shape[1]), dtype=x_rows.dtype, device=x_rows.device)
    id_recv = torch.empty((sum(rc),), dtype=torch.int32, device=x_rows.device)
    dist.all_to_all_single(x_recv, x_send, output_split_sizes=rc, input_split_sizes=sc, group=group)
    dist.all_to_all_single(id_recv, id_send, output_split_sizes=rc, input_split_sizes=sc, group=group)
    y_recv = local_mul_mat_id(x_recv, id_recv) if x_recv.shape[0] else torch.empty((0, n_out), dtype=torch.float32, device=x_rows.device)
    y_back = torch.empty((x_rows.shape[0], n_out), dtype=torch.float32, device=x_rows.device)
    dist.all_to_all_single(y_back, y_recv.contiguous(), output_split_sizes=sc, input_split_sizes=rc, group=group)
    out = torch.empty_like(y_back)
    out.index_copy_(0, order, y_back)
    _ = rank
    return out


class Comm:
    """The library's own NCCL communicator (hf2q_cuda_comm_*): the 128-byte id is made on rank 0 and
    handed round with torch.distributed, then every rank joins.  Used by the C-ABI forms
    ``qmatmul_rowshard`` / ``qmatmul_id_ep`` / ``moe_experts_ep`` below, which run the pack and unpack
    kernels and the NCCL calls inside the library."""

    def __init__(self, ctx, group=None):
        self.ctx, self.lib = ctx, ctx._lib
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        ident = (C.c_uint8 * 128)()
        if self.rank == 0:
            rc = self.lib.hf2q_cuda_comm_unique_id(ident)
            if rc:
                raise RuntimeError(f"hf2q_cuda_comm_unique_id failed ({rc}): NCCL not found")
        box = [bytes(ident)]
        dist.broadcast_object_list(box, src=0, group=group)
        h = C.c_void_p()
        rc = self.lib.hf2q_cuda_comm_create(ctx.device, (C.c_uint8 * 128).from_buffer_copy(box[0]), self.rank, self.world, C.byref(h))
        if rc:
            raise RuntimeError(f"hf2q_cuda_comm_create failed ({rc})")
        self._h = h

    def _check(self, rc: int) -> None:
        if rc:
            from . import ops
            detail = self.lib.hf2q_cuda_comm_last_error(self._h).decode() or self.lib.hf2q_cuda_last_error(self.ctx._h).decode()
            raise ops.Hf2qError(rc, detail)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.lib.hf2q_cuda_comm_destroy(self._h)
            self._h = None

    def qmatmul_rowshard(self, x: torch.Tensor, w_shard, m: int) -> torch.Tensor:
        """y[m, world * n_local] = x . W^T, W sharded by rows (hf2q_cuda_qmatmul_rowshard)."""
        from . import ops
        xdt = ops._act(x, "x")
        need = C.c_uint64()
        self._check(self.lib.hf2q_cuda_qmatmul_rowshard_workspace_bytes(m, w_shard.rows, w_shard.cols, w_shard.ggml_type, xdt, self.world, C.byref(need)))
        ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device=x.device)
        y = torch.empty((m, self.world * w_shard.rows), dtype=torch.float32, device=x.device)
        self._check(self.lib.hf2q_cuda_qmatmul_rowshard(self.ctx._h, self._h, self.ctx._stream(), x.data_ptr(), xdt, w_shard.ptr, y.data_ptr(), m,
                                                        w_shard.rows, w_shard.cols, w_shard.ggml_type, ws.data_ptr(), ws.numel()))
        self._keep = ws
        return y

    def qmatmul_id_ep(self, x_rows: torch.Tensor, ids: torch.Tensor, w_local_ptr: int, n: int, k: int, n_experts: int, stride: int,
                      ggml_type: int, cap_recv: int) -> torch.Tensor:
        """Expert-parallel mul_mat_id through the C ABI (hf2q_cuda_qmatmul_id_ep)."""
        from . import ops
        xdt = ops._act(x_rows, "x_rows")
        rows = x_rows.shape[0]
        need = C.c_uint64()
        self._check(self.lib.hf2q_cuda_qmatmul_id_ep_scratch_bytes(rows, cap_recv, self.world, n, k, n_experts, xdt, C.byref(need)))
        sc = torch.empty(max(need.value, 256), dtype=torch.uint8, device=x_rows.device)
        y = torch.empty((rows, n), dtype=torch.float32, device=x_rows.device)
        self._check(self.lib.hf2q_cuda_qmatmul_id_ep(self.ctx._h, self._h, self.ctx._stream(), x_rows.data_ptr(), xdt, ids.data_ptr(), w_local_ptr,
                                                     y.data_ptr(), rows, cap_recv, n, k, n_experts, stride, ggml_type, sc.data_ptr(), sc.numel()))
        self._keep = sc
        return y

    def moe_experts_ep(self, x_rows: torch.Tensor, ids: torch.Tensor, gate_ptr: int, up_ptr: int, down_ptr: int, hidden: int, inter: int,
                       n_experts: int, stride_gu: int, stride_d: int, type_gu: int, type_d: int, cap_recv: int,
                       scratch: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """y[rows, hidden] = down_e(silu(gate_e x) * (up_e x)) with the experts spread over the ranks (hf2q_cuda_moe_experts_ep)."""
        from . import ops
        xdt = ops._act(x_rows, "x_rows")
        rows = x_rows.shape[0]
        if scratch is None:
            need = C.c_uint64()
            self._check(self.lib.hf2q_cuda_moe_experts_ep_scratch_bytes(rows, cap_recv, self.world, hidden, inter, n_experts, xdt, C.byref(need)))
            scratch = torch.empty(max(need.value, 256), dtype=torch.uint8, device=x_rows.device)
        y = out if out is not None else torch.empty((rows, hidden), dtype=torch.float32, device=x_rows.device)
        self._check(self.lib.hf2q_cuda_moe_experts_ep(self.ctx._h, self._h, self.ctx._stream(), x_rows.data_ptr(), xdt, ids.data_ptr(), gate_ptr, up_ptr,
                                                      down_ptr, y.data_ptr(), rows, cap_recv, hidden, inter, n_experts, stride_gu, stride_d, type_gu,
                                                      type_d, scratch.data_ptr(), scratch.numel()))
        self._keep = scratch
        return y


class _Gather(C.Structure):                        # hf2q_gather in include/hf2q_cuda.h
    _fields_ = [("y_all", C.c_void_p * 8), ("flags", C.c_void_p * 8), ("n_ranks", C.c_uint32), ("rank", C.c_uint32),
                ("n_total", C.c_uint32), ("col0", C.c_uint32), ("wait_previous", C.c_uint32), ("n_rows", C.c_uint32 * 8)]


class _DevView:
    """Lets torch wrap a raw device pointer (zero copy)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


class GatherGroup:
    """Output buffers [max_m][n_total] and arrival counters of all ranks, mapped into this process.

    Every rank owns TWO output buffers and products alternate between them, so that a decode chain
    (x of a product = the previous product's gathered output) never stores into a buffer that a
    rank still reads: product i+1 overwrites the buffer of product i-1, and a rank only starts
    storing product i+1 after every rank has signalled product i complete, i.e. after every rank
    has finished reading product i-1's output.  That holds when every product after the first is
    issued with ``wait_previous=True``; a product issued without it is ordered by the caller.  A
    captured graph whose first product reads the last product's output must hold an even number of
    products of this group.

    Every rank must issue the same sequence of ``matmul`` calls.  ``matmul(..., wait_previous=True)``
    makes the kernel wait, after it has started prefetching weights, until the previous products'
    columns from all ranks have arrived here.  ``wait()`` queues a tiny kernel that waits for
    everything issued so far."""

    def __init__(self, ctx, max_m: int, n_total: int, group=None):
        self.ctx, self.group = ctx, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.max_m, self.n_total = max_m, n_total
        self._buf_bytes = (max_m * n_total * 4 + 255) & ~255
        self._next = 0                 # buffer the next product writes
        lib, h = ctx._lib, ctx._h
        own_y, own_f = C.c_void_p(), C.c_void_p()
        hy, hf = (C.c_uint8 * 64)(), (C.c_uint8 * 64)()
        self.y_ptrs, self.flag_ptrs, self._opened = [], [], []
        # Every rank takes part in both exchanges even if something failed locally, so that a failure
        # (no peer access, IPC not permitted) raises on all ranks instead of leaving some of them waiting.
        err = None
        try:
            ctx._check(lib.hf2q_cuda_ipc_alloc(h, 2 * self._buf_bytes, C.byref(own_y), hy))
            ctx._check(lib.hf2q_cuda_ipc_alloc(h, 256, C.byref(own_f), hf))
        except Exception as exc:                      # noqa: BLE001
            err = exc
        handles = [None] * self.world
        dist.all_gather_object(handles, None if err else (bytes(hy), bytes(hf)), group=group)
        if err is None and all(hd is not None for hd in handles):
            try:
                for r, (by, bf) in enumerate(handles):
                    if r == self.rank:
                        self.y_ptrs.append(own_y.value)
                        self.flag_ptrs.append(own_f.value)
                        continue
                    py, pf = C.c_void_p(), C.c_void_p()
                    ctx._check(lib.hf2q_cuda_ipc_open(h, (C.c_uint8 * 64).from_buffer_copy(by), C.byref(py)))
                    self._opened.append(py.value)
                    ctx._check(lib.hf2q_cuda_ipc_open(h, (C.c_uint8 * 64).from_buffer_copy(bf), C.byref(pf)))
                    self._opened.append(pf.value)
                    self.y_ptrs.append(py.value)
                    self.flag_ptrs.append(pf.value)
            except Exception as exc:                  # noqa: BLE001
                err = exc
        oks = [None] * self.world
        dist.all_gather_object(oks, err is None, group=group)     # also: nobody launches before everyone has mapped the buffers
        if not all(oks):
            for ptr in self._opened:
                lib.hf2q_cuda_ipc_close(h, ptr)
            for own in (own_y, own_f):
                if own.value:
                    lib.hf2q_cuda_free(h, own.value)
            raise RuntimeError(f"GatherGroup: peer buffers could not be set up on every rank (this rank: {err})")

    def _struct(self, col0: int, wait_previous: bool, buf: int, n_rows: Sequence[int]) -> _Gather:
        g = _Gather()
        for r in range(self.world):
            g.y_all[r] = self.y_ptrs[r] + buf * self._buf_bytes
            g.flags[r] = self.flag_ptrs[r]
            g.n_rows[r] = n_rows[r]
        g.n_ranks, g.rank, g.n_total, g.col0, g.wait_previous = self.world, self.rank, self.n_total, col0, int(wait_previous)
        return g

    def matmul(self, x: torch.Tensor, weight, m: int, col0: int | None = None, wait_previous: bool = False,
               n_rows: Sequence[int] | None = None) -> None:
        """Columns [col0, col0 + weight.rows) of y[m, n_total] = x . dequant(weight)^T on every rank.

        ``n_rows[r]`` = rows of rank r's shard of this product (default: every rank holds as many rows
        as this one); ``col0`` defaults to the sum of the earlier ranks' rows."""
        from . import ops
        if m > self.max_m:
            raise ValueError(f"m={m} exceeds the group's {self.max_m} rows")
        if n_rows is None:
            n_rows = [weight.rows] * self.world
        if col0 is None:
            col0 = sum(n_rows[: self.rank])
        g = self._struct(col0, wait_previous and self.world > 1, self._next, n_rows)
        self.ctx._check(self.ctx._lib.hf2q_cuda_qmatmul_gather(
            self.ctx._h, self.ctx._stream(), x.data_ptr(), ops._act(x, "x"), weight.ptr, C.byref(g), m, weight.rows,
            weight.cols, weight.ggml_type))
        self._next ^= 1

    def supports(self, weight, m: int, x_dtype=torch.float32) -> bool:
        """Whether ``matmul`` takes this product (else: a plain product into a local buffer + ``copy``)."""
        from . import ops
        return bool(self.ctx._lib.hf2q_cuda_gather_supported(self.ctx._h, weight.ptr, m, weight.rows, weight.cols, weight.ggml_type,
                                                             ops._TORCH_DT[x_dtype]))

    def copy(self, src: torch.Tensor, col0: int, n_each: Sequence[int] | None = None) -> None:
        """The exchange alone: src (f32, n values) -> columns [col0, col0 + n) of row 0 on every rank; counts as one
        product of the group (buffers alternate, arrival counters advance)."""
        n = src.numel()
        g = self._struct(col0, False, self._next, list(n_each) if n_each is not None else [n] * self.world)
        self.ctx._check(self.ctx._lib.hf2q_cuda_gather_copy(self.ctx._h, self.ctx._stream(), C.byref(g), src.data_ptr(), n))
        self._next ^= 1

    def sum_into(self, x: torch.Tensor, n: int, n_parts: int | None = None) -> None:
        """x[:n] += the sum of the most recent product's n-value parts (columns r * n .. of its buffer, r < n_parts;
        default one partial per rank), after waiting for every rank's columns; rank order, so every rank gets the
        same bits.  ``n_parts=1`` adds a gathered full-length result."""
        g = self._struct(0, False, self._next ^ 1, [1] * self.world)
        self.ctx._check(self.ctx._lib.hf2q_cuda_gather_sum(self.ctx._h, self.ctx._stream(), C.byref(g), x.data_ptr(), n,
                                                           self.world if n_parts is None else n_parts))

    def host_batch(self, batch) -> None:
        """``ops.HostBatch`` through the sharded product (hf2q_cuda_qmatmul_gather_host_batch): every rank passes the
        same products with its own shard as the weight; item.y_host (where given) receives the gathered
        [m, world * rows] result.  Valid after ``ops.host_sync``; counts as len(batch) products of the group."""
        g = self._struct(0, True, 0, [1] * self.world)
        self.ctx._check(self.ctx._lib.hf2q_cuda_qmatmul_gather_host_batch(
            self.ctx._h, C.byref(g), self._buf_bytes, self._next, C.cast(batch.array, C.c_void_p), len(batch)))
        self._next ^= len(batch) & 1

    def wait(self) -> None:
        if self.world > 1:
            g = self._struct(0, False, 0, [1] * self.world)
            self.ctx._check(self.ctx._lib.hf2q_cuda_gather_wait(self.ctx._h, self.ctx._stream(), C.byref(g)))

    def output(self, m: int) -> torch.Tensor:
        """The most recent product's full-width output on this rank as a float32 [m, n_total] tensor (no copy)."""
        buf = self._next ^ 1
        ptr = self.y_ptrs[self.rank] + buf * self._buf_bytes
        return torch.as_tensor(_DevView(ptr, (m, self.n_total), "<f4"), device=f"cuda:{self.ctx.device}")

    def close(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)         # peers may still be storing into our buffers
        for p in self._opened:
            self.ctx._lib.hf2q_cuda_ipc_close(self.ctx._h, p)
        self._opened = []
        self.ctx._lib.hf2q_cuda_free(self.ctx._h, self.y_ptrs[self.rank])
        self.ctx._lib.hf2q_cuda_free(self.ctx._h, self.flag_ptrs[self.rank])
