"""A Llama-shaped decoder forward on the quantized-matmul path: host-side mirror of the greedy
loop ``Qwen35Model::forward_gpu_greedy`` (src/inference/models/qwen35/forward_gpu.rs:4140) for plain
pre-norm layers (RMSNorm -> fused QKV -> rotary -> attention over an 8-bit KV cache -> O ->
RMSNorm -> SwiGLU FFN), with the reference's FFN call sites (forward_gpu.rs:4776 / :4807) served
by the fused products of this library.

Everything computes in ``libhf2q_cuda.so``; this module only orders the C-ABI calls on torch's
current stream and owns the buffers.  Weights arrive as raw GGUF block bytes (uploaded unchanged);
which tensor gets which block format follows the Q4_K_M policy of
``src/quantize/ggml_quants/standard_policy.rs``: Q4_K everywhere except ``attn_v`` and
``ffn_down`` of the layers ``use_more_bits`` selects (:325-329, :563-567, :646-658), which are Q6_K,
and ``output.weight`` (:440-442), Q6_K.

A decode step is pure device work -- the token id and the position live in device memory, the
arg-max kernel writes the next id and advances the position -- so it is captured into one CUDA
graph and replayed once per generated token.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib, ops


@dataclass(frozen=True)
class LlamaConfig:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_seq: int = 32768

    @property
    def q_rows(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_rows(self) -> int:
        return self.n_kv_heads * self.head_dim


def use_more_bits(i_layer: int, n_layers: int) -> bool:
    """standard_policy.rs:325-329."""
    return i_layer < n_layers // 8 or i_layer >= 7 * n_layers // 8 or (i_layer - n_layers // 8) % 3 == 2


def q4_k_m_types(cfg: LlamaConfig) -> dict:
    """Block format of every tensor under the Q4_K_M mix: {name: ggml type}."""
    q4, q6 = int(ops.GgmlType.Q4_K), int(ops.GgmlType.Q6_K)
    t = {"token_embd": q4, "output": q6}
    for i in range(cfg.n_layers):
        more = use_more_bits(i, cfg.n_layers)
        t[f"blk.{i}.attn_q"] = t[f"blk.{i}.attn_k"] = t[f"blk.{i}.attn_output"] = q4
        t[f"blk.{i}.ffn_gate"] = t[f"blk.{i}.ffn_up"] = q4
        t[f"blk.{i}.attn_v"] = t[f"blk.{i}.ffn_down"] = q6 if more else q4
    return t


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor            # f32 [hidden]
    wqk: ops.QuantWeight               # [q_rows + kv_rows, hidden]: the Q rows followed by the K rows -- or all of
                                       # Q, K and V ([q_rows + 2 kv_rows, hidden]) when V shares their block format
    wv: ops.QuantWeight | None         # [kv_rows, hidden], or None when wqk holds the V rows too
    wo: ops.QuantWeight                # [hidden, q_rows]
    ffn_norm: torch.Tensor
    gate: ops.QuantWeight              # [ffn, hidden]
    up: ops.QuantWeight
    down: ops.QuantWeight              # [hidden, ffn]


@dataclass
class ModelWeights:
    token_embd: ops.QuantWeight        # [vocab, hidden]
    layers: list
    out_norm: torch.Tensor
    output: ops.QuantWeight            # [vocab, hidden]


class _KvCache(C.Structure):           # hf2q_kv_cache in include/hf2q_cuda.h
    _fields_ = [("k_codes", C.c_void_p), ("k_scale", C.c_void_p), ("v_codes", C.c_void_p), ("v_scale", C.c_void_p),
                ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("max_seq", C.c_uint32)]


class LlamaDecoder:
    def __init__(self, ctx: ops.GpuContext, cfg: LlamaConfig, weights: ModelWeights, prefill_chunk: int = 2048):
        self.ctx, self.cfg, self.w = ctx, cfg, weights
        self.lib = ctx._lib
        dev = torch.device("cuda", ctx.device)
        self.dev = dev
        c = cfg
        self.qkv_cols = c.q_rows + 2 * c.kv_rows
        # the 8-bit KV cache: one pair of (codes, scales) for K and for V per layer
        self.kv_bufs, self.kv = [], []
        for _ in range(c.n_layers):
            kc = torch.zeros((c.n_kv_heads, c.max_seq, c.head_dim), dtype=torch.int8, device=dev)
            ks = torch.zeros((c.n_kv_heads, c.max_seq), dtype=torch.float32, device=dev)
            vc = torch.zeros_like(kc)
            vs = torch.zeros_like(ks)
            self.kv_bufs.append((kc, ks, vc, vs))
            self.kv.append(_KvCache(kc.data_ptr(), ks.data_ptr(), vc.data_ptr(), vs.data_ptr(), c.n_kv_heads, c.head_dim, c.max_seq))
        # device-resident loop state
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)          # position of the token being processed
        self.tok = torch.zeros(1, dtype=torch.int32, device=dev)          # its id (written by the arg-max kernel)
        # single-token buffers of the decode step
        f32 = dict(dtype=torch.float32, device=dev)
        self.x = torch.zeros((1, c.hidden), **f32)
        self.xn = torch.zeros((1, c.hidden), **f32)
        self.qkv = torch.zeros((1, self.qkv_cols), **f32)
        self.att = torch.zeros((1, c.q_rows), **f32)
        self.act = torch.zeros((1, c.ffn), **f32)
        self.tmp = torch.zeros((1, c.hidden), **f32)
        self.fused_attention = True
        self.fused_prefill = True          # prompt chunks: SwiGLU pair and residual adds inside the tensor-core products
        self._pf_delta = None
        # RMSNorm inside the product that consumes it, where every tensor of the model allows it
        self.fused_norm = all(ops.norm_supported(ctx, 1, w) for lw in weights.layers for w in (lw.wqk, lw.wv, lw.gate) if w is not None) and \
            ops.norm_supported(ctx, 1, weights.output)
        self.logits = torch.zeros((1, c.vocab), **f32)
        need = C.c_uint64()
        ctx._check(self.lib.hf2q_cuda_attn_decode_scratch_bytes(ctx._h, c.n_heads, c.n_kv_heads, C.byref(need)))
        self.att_scratch = torch.zeros(max(need.value, 16), dtype=torch.uint8, device=dev)
        self.prefill_chunk = prefill_chunk
        self._pf = None                 # prefill buffers, allocated on first use
        self._graph = None
        for lw in weights.layers:
            if not ops.quantized_matmul_swiglu_supported(ctx, 1, lw.gate, torch.float32):
                raise ops.Hf2qError(_lib.ERR_INVALID_ARGUMENT, "gate/up shape does not fit the fused SwiGLU launch")

    # ---- thin wrappers over the C ABI (current stream) -----------------------------------------
    def _s(self):
        return self.ctx._stream()

    def _get_rows(self, ids, m, out):
        w = self.w.token_embd
        self.ctx._check(self.lib.hf2q_cuda_get_rows(self.ctx._h, self._s(), w.ptr, w.ggml_type, w.rows, w.cols, ids.data_ptr(), m, out.data_ptr()))

    def _rms(self, x, delta, weight, out, m):
        self.ctx._check(self.lib.hf2q_cuda_rms_norm(self.ctx._h, self._s(), x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                                    weight.data_ptr(), self.cfg.rms_eps, out.data_ptr(), ops._TORCH_DT[out.dtype], m, self.cfg.hidden))

    def _rope_append(self, qkv, m, layer):
        self.ctx._check(self.lib.hf2q_cuda_rope_kv_append(self.ctx._h, self._s(), qkv.data_ptr(), m, self.cfg.n_heads, self.cfg.rope_theta,
                                                          self.pos.data_ptr(), C.byref(self.kv[layer])))

    @staticmethod
    def _qkv_segments(lw):
        return [lw.wqk] if lw.wv is None else [lw.wqk, lw.wv]

    def _matmul_add(self, inp, weight):
        """self.x += inp . weight^T: residual add in the product's epilogue where the shape allows, else two calls."""
        if ops.quantized_matmul_add_supported(self.ctx, weight, inp.dtype):
            ops.quantized_matmul_add(self.ctx, inp, weight, self.x, self.x, 1)
        else:
            ops.quantized_matmul_ggml(self.ctx, inp, weight, self.tmp, weight.matmul_params(1))
            self.ctx._check(self.lib.hf2q_cuda_add(self.ctx._h, self._s(), self.x.data_ptr(), self.tmp.data_ptr(), self.x.numel()))

    # ---- one decode step: token self.tok at position self.pos -> next token, position + 1 -------
    def decode_step(self) -> None:
        c, ctx, lib = self.cfg, self.ctx, self.lib
        self._get_rows(self.tok, 1, self.x)
        fn = self.fused_norm
        for i, lw in enumerate(self.w.layers):
            if fn:
                ops.quantized_matmul_segments(ctx, self.x, self._qkv_segments(lw), self.qkv, 1, norm_weight=lw.attn_norm, norm_eps=c.rms_eps)
            else:
                self._rms(self.x, None, lw.attn_norm, self.xn, 1)
                ops.quantized_matmul_segments(ctx, self.xn, self._qkv_segments(lw), self.qkv, 1)
            if self.fused_attention:      # rotary + KV append + split attention + merge: one launch
                ctx._check(lib.hf2q_cuda_attn_decode_fused(ctx._h, self._s(), self.qkv.data_ptr(), c.n_heads, c.rope_theta, C.byref(self.kv[i]),
                                                           self.pos.data_ptr(), self.att.data_ptr(), ops.DT_F32, self.att_scratch.data_ptr(),
                                                           self.att_scratch.numel()))
            else:
                self._rope_append(self.qkv, 1, i)
                ctx._check(lib.hf2q_cuda_attn_decode(ctx._h, self._s(), self.qkv.data_ptr(), c.n_heads, C.byref(self.kv[i]), self.pos.data_ptr(),
                                                     self.att.data_ptr(), ops.DT_F32, self.att_scratch.data_ptr(), self.att_scratch.numel()))
            self._matmul_add(self.att, lw.wo)                                               # x += O(att)
            if fn:
                ops.quantized_matmul_swiglu(ctx, self.x, lw.gate, lw.up, self.act, 1, norm_weight=lw.ffn_norm, norm_eps=c.rms_eps)
            else:
                self._rms(self.x, None, lw.ffn_norm, self.xn, 1)
                ops.quantized_matmul_swiglu(ctx, self.xn, lw.gate, lw.up, self.act, 1)      # silu(gate x) * (up x)
            self._matmul_add(self.act, lw.down)                                             # x += down(act)
        if fn:
            ops.quantized_matmul_segments(ctx, self.x, [self.w.output], self.logits, 1, norm_weight=self.w.out_norm, norm_eps=c.rms_eps)
        else:
            self._rms(self.x, None, self.w.out_norm, self.xn, 1)
            ops.quantized_matmul_ggml(ctx, self.xn, self.w.output, self.logits, self.w.output.matmul_params(1))
        ctx._check(lib.hf2q_cuda_argmax(ctx._h, self._s(), self.logits.data_ptr(), c.vocab, self.tok.data_ptr(), self.pos.data_ptr()))

    @property
    def launches_per_token(self) -> int:
        per_layer = (0 if self.fused_norm else 2) + (1 if self.fused_attention else 3) + 3        # norms, attention, O / gate+up / down
        qkv = sum(len(self._qkv_segments(lw)) for lw in self.w.layers)                            # one launch per row range of the fused QKV
        return 1 + per_layer * self.cfg.n_layers + qkv + (2 if self.fused_norm else 3)

    def capture(self) -> None:
        """Captures one decode step into a CUDA graph (after a few eager steps have warmed every kernel up)."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.decode_step()
        self._graph = g

    def generate(self, n: int, use_graph: bool = True, collect: bool = True):
        """Greedy decode of n tokens starting from the current (tok, pos) state; returns the generated ids
        (``collect=False``: nothing is copied out between the steps and None is returned)."""
        out = torch.empty(n, dtype=torch.int32, device=self.dev) if collect else None
        if use_graph and self._graph is None:
            saved = (self.pos.clone(), self.tok.clone())
            self.decode_step()                        # warm-up outside the capture; state restored below
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

    # ---- prefill: m tokens per chunk through the GEMM path ---------------------------------------
    def _prefill_buffers(self, m):
        if self._pf is None or self._pf["m"] < m:
            c = self.cfg
            f32 = dict(dtype=torch.float32, device=self.dev)
            self._pf = {"m": m, "x": torch.empty((m, c.hidden), **f32), "xn": torch.empty((m, c.hidden), **f32),
                        "qkv": torch.empty((m, self.qkv_cols), **f32), "att": torch.empty((m, c.q_rows), **f32),
                        "o": torch.empty((m, c.hidden), **f32), "g": torch.empty((m, c.ffn), **f32),
                        "u": torch.empty((m, c.ffn), **f32)}
        return self._pf

    def prefill(self, ids: torch.Tensor) -> None:
        """Runs the prompt (int32 ids on the device) from position 0, fills the KV cache, and leaves
        (tok, pos) = (greedy next token, len(ids)) for ``generate``; self.logits holds the last logits."""
        c, ctx, lib = self.cfg, self.ctx, self.lib
        T = int(ids.numel())
        if T == 0 or T >= c.max_seq:
            raise ops.Hf2qError(_lib.ERR_INVALID_ARGUMENT, f"prompt length {T} must be in 1..max_seq-1")
        ids = ids.to(self.dev, torch.int32).contiguous()
        for p0 in range(0, T, self.prefill_chunk):
            m = min(self.prefill_chunk, T - p0)
            b = self._prefill_buffers(min(self.prefill_chunk, T))
            x, xn, qkv, att, o, g, u = (b[k][:m] for k in ("x", "xn", "qkv", "att", "o", "g", "u"))
            self.pos.fill_(p0)
            self._get_rows(ids[p0:p0 + m], m, x)
            delta = None
            for i, lw in enumerate(self.w.layers):
                self._rms(x, delta, lw.attn_norm, xn, m)                                   # x += previous layer's FFN output (unfused form)
                ops.quantized_matmul_segments(ctx, xn, self._qkv_segments(lw), qkv, m)
                self._rope_append(qkv, m, i)
                ctx._check(lib.hf2q_cuda_attn_prefill(ctx._h, self._s(), qkv.data_ptr(), m, c.n_heads, C.byref(self.kv[i]), p0,
                                                      att.data_ptr(), ops.DT_F32))
                # the residual stream is updated in the epilogue of the O and down products where the shape allows
                if self.fused_prefill and ops.quantized_matmul_add_supported(ctx, lw.wo, att.dtype, m):
                    ops.quantized_matmul_add(ctx, att, lw.wo, x, x, m)
                    self._rms(x, None, lw.ffn_norm, xn, m)
                else:
                    ops.quantized_matmul_ggml(ctx, att, lw.wo, o, lw.wo.matmul_params(m))
                    self._rms(x, o, lw.ffn_norm, xn, m)                                    # x += O(att)
                if (self.fused_prefill and lw.gate.ggml_type == lw.up.ggml_type and
                        ops.quantized_matmul_swiglu_supported(ctx, m, lw.gate, xn.dtype)):
                    ops.quantized_matmul_swiglu(ctx, xn, lw.gate, lw.up, g, m)             # gate, up and the SwiGLU in one product
                else:
                    ops.quantized_matmul_ggml(ctx, xn, lw.gate, g, lw.gate.matmul_params(m))
                    ops.quantized_matmul_ggml(ctx, xn, lw.up, u, lw.up.matmul_params(m))
                    ctx._check(lib.hf2q_cuda_silu_mul(ctx._h, self._s(), g.data_ptr(), u.data_ptr(), g.data_ptr(), g.numel()))
                if self.fused_prefill and ops.quantized_matmul_add_supported(ctx, lw.down, g.dtype, m):
                    ops.quantized_matmul_add(ctx, g, lw.down, x, x, m)
                    delta = None
                else:
                    ops.quantized_matmul_ggml(ctx, g, lw.down, o, lw.down.matmul_params(m))
                    delta = o
            self._pf_delta = delta
            if p0 + m == T:
                # only the last token's logits are needed: x_last += delta_last, final norm, output head
                self.x.copy_(x[m - 1:m])
                self._rms(self.x, None if delta is None else delta[m - 1:m], self.w.out_norm, self.xn, 1)
                ops.quantized_matmul_ggml(ctx, self.xn, self.w.output, self.logits, self.w.output.matmul_params(1))
                self.pos.fill_(T - 1)
                ctx._check(lib.hf2q_cuda_argmax(ctx._h, self._s(), self.logits.data_ptr(), c.vocab, self.tok.data_ptr(), self.pos.data_ptr()))

    def forward_logits(self, ids: torch.Tensor) -> torch.Tensor:
        """Logits of every prompt position (test helper for short prompts): runs ``prefill`` on each prefix length...
        is quadratic, so instead one chunk is run and the output head is applied to all rows."""
        c, ctx = self.cfg, self.ctx
        T = int(ids.numel())
        saved = self.prefill_chunk
        self.prefill_chunk = max(saved, T)
        try:
            self.prefill(ids)
        finally:
            self.prefill_chunk = saved
        b = self._pf
        x = b["x"][:T]
        xn = torch.empty((T, c.hidden), dtype=torch.float32, device=self.dev)
        xs = x.clone()
        self._rms(xs, None if self._pf_delta is None else self._pf_delta[:T], self.w.out_norm, xn, T)
        logits = torch.empty((T, c.vocab), dtype=torch.float32, device=self.dev)
        ops.quantized_matmul_ggml(ctx, xn, self.w.output, logits, self.w.output.matmul_params(T))
        return logits

    def kv_bytes_per_position(self) -> int:
        c = self.cfg
        return c.n_layers * 2 * c.n_kv_heads * (c.head_dim + 4)

    def weight_bytes_per_token(self) -> int:
        """Weight bytes one decode step reads: every layer tensor once, the output head once, one embedding row."""
        total = self.w.output.nbytes + ops.row_bytes(self.w.token_embd.ggml_type, self.w.token_embd.cols)
        for lw in self.w.layers:
            total += sum(w.nbytes for w in (lw.wqk, lw.wv, lw.wo, lw.gate, lw.up, lw.down) if w is not None)
        return total
