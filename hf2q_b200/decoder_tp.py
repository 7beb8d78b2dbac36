"""Tensor-parallel decode step of the Llama-shaped decoder (one process per GPU, `world` ranks, world | n_kv_heads).

hf2q itself is single-device; this is the "rows sharded over 1/2/4/8 GPUs" reading of its decode path built on
the row-sharded mat-vec with the all-gather in its epilogue (``hf2q_cuda_qmatmul_gather``).  Sharding, Megatron
style, so that a layer needs TWO exchanges instead of four:

* QKV, gate and up are sharded by OUTPUT rows (heads / FFN rows): no exchange, their consumers (attention over
  the rank's own heads and KV cache, the SwiGLU, the next projection) only need the local slice;
* O and down are sharded by their CONTRACTION dimension (each rank holds the columns that match its slice of
  the attention output / FFN activation, repacked dense at load time: blocks are independent along k, so a
  column shard is a byte range of every row).  Every rank's product is a full-length PARTIAL sum; the gather
  epilogue places the N partials side by side in every rank's buffer and ``hf2q_cuda_gather_sum`` adds them to
  the residual stream in rank order (same bits on every rank: the stream stays replicated);
* the output head is sharded by vocabulary rows and gathered; arg-max runs replicated on the gathered logits.

All waits are inside ``gather_sum`` / ``gather_wait`` (bounded); a decode step contains no host
synchronisation and no NCCL call and is captured into one CUDA graph per rank.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib, ops
from .decoder import LlamaConfig, _KvCache
from .dist import GatherGroup


@dataclass
class TpLayerWeights:
    attn_norm: torch.Tensor            # f32 [hidden] (replicated)
    wqk: ops.QuantWeight               # this rank's q heads, then its k heads (then its v heads when V shares the format)
    wv: ops.QuantWeight | None
    wo: ops.QuantWeight                # [hidden, q_rows / world]: the columns of attn_output for this rank's heads
    ffn_norm: torch.Tensor
    gate: ops.QuantWeight              # [ffn / world, hidden]
    up: ops.QuantWeight
    down: ops.QuantWeight              # [hidden, ffn / world], or [hidden / world, ffn] where a column shard would be unaligned


@dataclass
class TpModelWeights:
    token_embd: ops.QuantWeight        # full [vocab, hidden] (one row is read per token)
    layers: list
    out_norm: torch.Tensor
    output: ops.QuantWeight            # [vocab / world, hidden]


def column_shard_ok(ggml_type: int, k: int, world: int) -> bool:
    """Whether a 1 / world column shard of a [n, k] tensor keeps 16-byte aligned rows of whole 256-element blocks
    (what the gathering mat-vec needs).  Q6_K rows (210 bytes per block) are aligned only in multiples of 8 blocks;
    a tensor that fails this is sharded by rows instead, with its input gathered first."""
    kl = k // world
    return k % world == 0 and kl % 256 == 0 and ops.row_bytes(ggml_type, kl) % 16 == 0


def shard_raw(name: str, raw: np.ndarray, ggml_type: int, n: int, k: int, cfg: LlamaConfig, rank: int, world: int):
    """Rank `rank`'s part of one GGUF tensor of the model as (bytes, rows, cols): a row range for attn_q / attn_k /
    attn_v / ffn_gate / ffn_up / output, a column range (whole blocks of every row) for attn_output / ffn_down where
    ``column_shard_ok`` (else a row range), everything for token_embd."""
    rb = ops.row_bytes(ggml_type, k)
    rows = np.ascontiguousarray(raw, dtype=np.uint8).reshape(n, rb)
    base = name.split(".")[-1]
    if base in ("attn_output", "ffn_down") and column_shard_ok(ggml_type, k, world):
        c0, c1 = rank * k // world, (rank + 1) * k // world
        b0, b1 = ops.row_bytes(ggml_type, c0) if c0 else 0, ops.row_bytes(ggml_type, c1)
        return np.ascontiguousarray(rows[:, b0:b1]).reshape(-1), n, c1 - c0
    if base == "token_embd":
        return rows.reshape(-1), n, k
    r0, r1 = rank * n // world, (rank + 1) * n // world
    return np.ascontiguousarray(rows[r0:r1]).reshape(-1), r1 - r0, k


class TensorParallelDecoder:
    """Decode-only (the prompt is fed token by token, or the caches are filled by the caller)."""

    def __init__(self, ctx: ops.GpuContext, cfg: LlamaConfig, weights: TpModelWeights, group=None):
        import torch.distributed as dist
        self.ctx, self.cfg, self.w, self.lib = ctx, cfg, weights, ctx._lib
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        c, W = cfg, self.world
        if c.n_kv_heads % W or c.ffn % W or c.vocab % W:
            raise ops.Hf2qError(_lib.ERR_INVALID_ARGUMENT, f"{W} ranks must divide n_kv_heads={c.n_kv_heads}, ffn={c.ffn} and vocab={c.vocab}")
        self.heads_l, self.kv_l = c.n_heads // W, c.n_kv_heads // W
        self.ffn_l, self.vocab_l = c.ffn // W, c.vocab // W
        dev = torch.device("cuda", ctx.device)
        self.dev = dev
        self.kv_bufs, self.kv = [], []
        for _ in range(c.n_layers):
            kc = torch.zeros((self.kv_l, c.max_seq, c.head_dim), dtype=torch.int8, device=dev)
            ks = torch.zeros((self.kv_l, c.max_seq), dtype=torch.float32, device=dev)
            vc, vs = torch.zeros_like(kc), torch.zeros_like(ks)
            self.kv_bufs.append((kc, ks, vc, vs))
            self.kv.append(_KvCache(kc.data_ptr(), ks.data_ptr(), vc.data_ptr(), vs.data_ptr(), self.kv_l, c.head_dim, c.max_seq))
        f32 = dict(dtype=torch.float32, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tok = torch.zeros(1, dtype=torch.int32, device=dev)
        self.x = torch.zeros((1, c.hidden), **f32)
        self.qkv = torch.zeros((1, (self.heads_l + 2 * self.kv_l) * c.head_dim), **f32)
        self.att = torch.zeros((1, self.heads_l * c.head_dim), **f32)
        self.act = torch.zeros((1, self.ffn_l), **f32)
        self.tmp = torch.zeros((1, c.hidden), **f32)
        self.xn = torch.zeros((1, c.hidden), **f32)
        need = C.c_uint64()
        ctx._check(self.lib.hf2q_cuda_attn_decode_scratch_bytes(ctx._h, self.heads_l, self.kv_l, C.byref(need)))
        self.att_scratch = torch.zeros(max(need.value, 16), dtype=torch.uint8, device=dev)
        # the partial sums of O and down: world x hidden values per product; the logits: vocab values
        self.partials = GatherGroup(ctx, 1, W * c.hidden, group=group)
        self.logit_group = GatherGroup(ctx, 1, c.vocab, group=group)
        self.wide = GatherGroup(ctx, 1, max(c.ffn, c.q_rows, c.hidden), group=group)      # gathered inputs / outputs of row-sharded O / down
        self._graph = None
        for lw in weights.layers:
            for w_ in (lw.wqk, lw.wv, lw.gate):
                if w_ is not None and not ops.norm_supported(ctx, 1, w_):
                    raise ops.Hf2qError(_lib.ERR_INVALID_ARGUMENT, "a sharded tensor does not take the fused RMSNorm")

    def _s(self):
        return self.ctx._stream()

    def _project_sum(self, inp: torch.Tensor, weight: ops.QuantWeight, k_full: int) -> None:
        """self.x += (full input) . W^T for a projection whose input `inp` is this rank's slice of a length-k_full vector.
        Column-sharded weight (cols == len(inp)): partial products, exchanged and summed.  Row-sharded weight
        (cols == k_full; used where a column shard would break the 16-byte row alignment): the input slices are
        gathered first, the product's own epilogue gathers its rows, and the gathered result is added."""
        c = self.cfg
        if weight.cols != k_full:
            return self._partial_sum(inp, weight)
        nl = inp.numel()
        self.wide.copy(inp, self.rank * nl)                                   # everyone's slice -> the full input on every rank
        xin = self.wide.output(1)[:, :k_full]
        self.wide.matmul(xin, weight, 1, self.rank * weight.rows, wait_previous=True, n_rows=[weight.rows] * self.world)
        self.wide.sum_into(self.x, c.hidden, n_parts=1)

    def _partial_sum(self, inp: torch.Tensor, weight: ops.QuantWeight) -> None:
        """self.x += all-reduce(inp . weight^T): the ranks' partial products side by side in every rank's buffer
        (from the product's own epilogue where the shard's rows are 16-byte aligned, else from a plain product and
        the copy kernel), then added in rank order."""
        c = self.cfg
        if self.partials.supports(weight, 1, inp.dtype):
            self.partials.matmul(inp, weight, 1, self.rank * c.hidden, n_rows=[c.hidden] * self.world)
        else:
            ops.quantized_matmul_ggml(self.ctx, inp, weight, self.tmp, weight.matmul_params(1))
            self.partials.copy(self.tmp, self.rank * c.hidden)
        self.partials.sum_into(self.x, c.hidden)

    def decode_step(self) -> None:
        c, ctx, lib = self.cfg, self.ctx, self.lib
        w = self.w.token_embd
        ctx._check(lib.hf2q_cuda_get_rows(ctx._h, self._s(), w.ptr, w.ggml_type, w.rows, w.cols, self.tok.data_ptr(), 1, self.x.data_ptr()))
        for i, lw in enumerate(self.w.layers):
            segs = [lw.wqk] if lw.wv is None else [lw.wqk, lw.wv]
            ops.quantized_matmul_segments(ctx, self.x, segs, self.qkv, 1, norm_weight=lw.attn_norm, norm_eps=c.rms_eps)
            ctx._check(lib.hf2q_cuda_attn_decode_fused(ctx._h, self._s(), self.qkv.data_ptr(), self.heads_l, c.rope_theta, C.byref(self.kv[i]),
                                                       self.pos.data_ptr(), self.att.data_ptr(), ops.DT_F32, self.att_scratch.data_ptr(),
                                                       self.att_scratch.numel()))
            self._project_sum(self.att, lw.wo, c.q_rows)                                    # x += O(att), summed over the ranks
            ops.quantized_matmul_swiglu(ctx, self.x, lw.gate, lw.up, self.act, 1, norm_weight=lw.ffn_norm, norm_eps=c.rms_eps)
            self._project_sum(self.act, lw.down, c.ffn)                                     # x += down(act)
        ctx._check(lib.hf2q_cuda_rms_norm(ctx._h, self._s(), self.x.data_ptr(), None, self.w.out_norm.data_ptr(), c.rms_eps, self.xn.data_ptr(),
                                          ops.DT_F32, 1, c.hidden))
        self.logit_group.matmul(self.xn, self.w.output, 1, self.rank * self.vocab_l, n_rows=[self.vocab_l] * self.world)
        self.logit_group.wait()
        self.logits = self.logit_group.output(1)
        ctx._check(lib.hf2q_cuda_argmax(ctx._h, self._s(), self.logits.data_ptr(), c.vocab, self.tok.data_ptr(), self.pos.data_ptr()))

    @property
    def launches_per_token(self) -> int:
        qkv = sum(1 if lw.wv is None else 2 for lw in self.w.layers)
        return 1 + qkv + 6 * self.cfg.n_layers + 4          # attention, O, sum, gate/up, down, sum per layer (+ a copy where a shard is unaligned); norm, head, wait, arg-max

    def weight_bytes_per_token(self) -> int:
        total = self.w.output.nbytes + ops.row_bytes(self.w.token_embd.ggml_type, self.w.token_embd.cols)
        for lw in self.w.layers:
            total += sum(w.nbytes for w in (lw.wqk, lw.wv, lw.wo, lw.gate, lw.up, lw.down) if w is not None)
        return total

    def capture(self) -> None:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.decode_step()
        self._graph = g

    def generate(self, n: int, use_graph: bool = True, collect: bool = True):
        """Greedy decode of n tokens from the current (tok, pos); every rank calls it with the same n."""
        out = torch.empty(n, dtype=torch.int32, device=self.dev) if collect else None
        if use_graph and self._graph is None:
            # a captured step holds an ODD number of logit products: replays always write the same one of the two
            # logit buffers, which is safe here (a rank reaches the next step's head only after every rank's
            # arg-max of this step: the partial-sum exchanges in between order them)
            saved = (self.pos.clone(), self.tok.clone())
            self.decode_step()
            self.pos.copy_(saved[0]); self.tok.copy_(saved[1])
            self.decode_step()                        # two warm-up steps leave both groups' buffer parity unchanged
            torch.cuda.synchronize(self.dev)
            self.pos.copy_(saved[0]); self.tok.copy_(saved[1])
            self.capture()
            self.pos.copy_(saved[0]); self.tok.copy_(saved[1])
        for t in range(n):
            if use_graph:
                self._graph.replay()
            else:
                self.decode_step()
            if collect:
                out[t:t + 1].copy_(self.tok)
        return out

    def close(self) -> None:
        self.partials.close()
        self.logit_group.close()
        self.wide.close()
