#!/usr/bin/env python
"""Benchmark of the quantized-weight matmul path on B200.

Headline workload (one GPU): the Q6_K decode GEMV sweep -- weight shapes (out x in) 6144x4096,
4096x4096, 28672x4096 and 4096x14336, N(0, 0.02) weights quantized to Q6_K (210 B per 256 elements)
by the CPU oracle's port of hf2q's quantizer, bf16 N(0,1) activations, batches of 1, 4 and 8 tokens,
fp32 accumulation.  Every matrix is smaller than the 126 MB L2, so the sweep rotates over `--copies`
distinct device copies of the four matrices (>= 1 GiB in total): no launch finds its weights in L2.
One "step" is `--passes` passes over all copies x shapes x token counts (16 by default, so that the
default 20..200 steps time a region of 0.5 s and more).

  metric  = dequant-GEMV HBM GB/s = algorithmic bytes (W + 2*m*K + 4*m*N per launch) / device time
  value   = inputs resident in HBM, launches back to back on one stream, CUDA-event timed
  e2e     = the same sweep through the host-buffer C-ABI call (hf2q_cuda_qmatmul_host_batch): one call
            per pass queues, for every product, the copy of its activations from pinned host memory,
            the kernel and the copy of y back to pinned host memory; one hf2q_cuda_host_sync per pass
            waits for all of them
  secondary (one GPU) = the other kernels of the path, measured in the same run with the same
            timing rules: Q4_K 4096x4096 f32 mat-vec, the Q4_K_M prefill GEMM sweep (TFLOP/s against
            the measured bf16 peaks), and the Q5_K expert layer at 1 and 2048 tokens.

Multi-GPU (torchrun, one rank per GPU).  `value` is WEAK scaling: each rank holds the shapes above
as ITS row shard of a matrix G times taller.  The mat-vec kernel stores its columns into every
rank's full-width output buffer itself (peer memory over NVLink, per-source arrival counters), so
a step contains no collective call and is replayed from a CUDA graph like the single-GPU step.  The
line also carries `strong`: the listed shapes themselves split G ways by rows, same kernels.  Before
timing, every rank checks one gathered full-width product against the oracle and the run stops on
a mismatch.  The e2e leg goes through the same sharded call: pinned x -> device on every rank,
hf2q_cuda_qmatmul_gather, and the full-width y -> pinned host on rank 0.

`--impl reference` times the reference's CPU path for the same products (the oracle's port of
"dequantise to f32, then matmul_a_by_bt") on the host cores, one bounded sample per step.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]   # (n, k)
TOKENS = [1, 4, 8]
Q6_K = 14
METRIC = "dequant-GEMV HBM GB/s"
UNIT = "GB/s"
WORKLOAD = ("Q6_K decode GEMV sweep: shapes 6144x4096, 4096x4096, 28672x4096, 4096x14336; "
            "m in {1,4,8}; bf16 activations; fp32 accumulate")


def algo_bytes(n: int, k: int, m: int, row_bytes: int) -> int:
    return n * row_bytes + 2 * m * k + 4 * m * n


def measured_hbm_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# DRAM bytes per algorithmic byte of gemv_mma_kernel<Q6_K>: `dram__bytes_read.sum + dram__bytes_write.sum` of the ncu
# capture summarised in profiles/gemv_q6k_sweep.md (four m = 1 launches: 183.27 MB over 179.14 MB algorithmic).
NCU_DRAM_BYTES_PER_ALGORITHMIC_BYTE = 1.0231


def ncu_traffic_per_launch() -> float | None:
    """DRAM bytes per algorithmic byte of the headline kernel, from the ncu capture (a constant of that capture, not
    a measurement of this run)."""
    return NCU_DRAM_BYTES_PER_ALGORITHMIC_BYTE


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self._nv:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self) -> dict:
        if self._thr:
            self._stop.set()
            self._thr.join()
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def make_weights(seed0: int = 0):
    """One quantized copy of the four matrices (host bytes), Q6_K."""
    import oracle
    from tests.util import make_quant_weight
    return [make_quant_weight(Q6_K, n, k, seed=seed0 + i) for i, (n, k) in enumerate(SHAPES)]


def cpu_reference_pass(raws, xs, threads: int, row_frac: float = 1.0) -> tuple[float, int]:
    """One pass of the reference CPU path over (the first `row_frac` of the rows of) the four
    matrices x token counts.  Returns (seconds, algorithmic bytes)."""
    import oracle
    tot_t, tot_b = 0.0, 0
    for (n, k), raw in zip(SHAPES, raws):
        rb = oracle.row_bytes(Q6_K, k)
        nn = max(8, int(n * row_frac))
        for m in TOKENS:
            _, td, tm = oracle.qmatmul(Q6_K, raw[: nn * rb], xs[(k, m)], nn, k, threads=threads)
            tot_t += td + tm
            tot_b += algo_bytes(nn, k, m, rb)
    return tot_t, tot_b


def host_inputs():
    from tests.util import bf16_bits_to_f32, make_x, to_bf16_bits
    bits, vals = {}, {}
    for k in sorted({k for _, k in SHAPES}):
        for m in TOKENS:
            b = to_bf16_bits(make_x(m, k, seed=1000 + m))
            bits[(k, m)] = b
            vals[(k, m)] = bf16_bits_to_f32(b).reshape(m, k)
    return bits, vals


def host_threads() -> int:
    """Host threads this process may use.  torchrun exports OMP_NUM_THREADS=1 for its workers, which
    would turn the reference arm into a single-core run: take the count from the CPU affinity mask."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    threads = host_threads()
    oracle.set_threads(threads)
    raws = make_weights()
    _, xvals = host_inputs()
    # size the per-step sample so that warmup + steps end within ~2.5 minutes
    t_full, _ = cpu_reference_pass(raws, xvals, threads)
    budget = 150.0 / max(1, args.steps + args.warmup)
    row_frac = min(1.0, budget / max(t_full, 1e-6))
    for _ in range(args.warmup):
        cpu_reference_pass(raws, xvals, threads, row_frac)
    t, b = 0.0, 0
    for _ in range(args.steps):
        dt, db = cpu_reference_pass(raws, xvals, threads, row_frac)
        t += dt
        b += db
    val = b / t / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"per step: the first {row_frac:.4f} of the rows of each of the four Q6_K matrices x "
                                   "m in {1,4,8} (dequantise to f32 + sequential-k f32 matmul, OpenMP over rows)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def measured_tensor_peaks() -> tuple[float, float, str]:
    """(sustained, burst) measured bf16 TFLOP/s of this pool's B200s, else the stated fall-back."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            j = json.loads(p.read_text())
            return float(j["bf16_tflops_sustained"]), float(j["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1400.0, 1590.0, "fallback"


def _random_weight(torch, oracle, dev, t, rows, k, exp_mask=0x3B):
    """Random block bytes with finite, small scales: throughput does not depend on the values
    (parity is what the tests check on real quantizer output).  exp_mask bounds the f16 scales'
    exponent: 0x3B keeps |d| < 1, 0x0F keeps |d| < 2^-11 (weights of order one at most, for chains of
    products whose intermediate values must stay inside the f16 range)."""
    rb = oracle.row_bytes(t, k)
    raw = torch.randint(0, 256, (rows * rb,), dtype=torch.uint8, device=dev)
    _, bb = oracle.block_geometry(t)
    v = raw.view(-1, bb)
    for o in {2: [1], 8: [1], 12: [1, 3], 13: [1, 3], 14: [209]}[t]:       # high byte of each f16 scale
        v[:, o] &= exp_mask
    return raw


def _timed(torch, fn, reps, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / reps


def _graph_of(torch, fn):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


def bench_gemm(hq, oracle, torch, ctx, dev, args, toks=None) -> dict:
    """BASELINE config 3: Q4_K for 6144x4096 (rows 0-5119; the V rows 5120-6143 are Q6_K: a row-range
    type map), 4096x4096, 28672x4096 and Q6_K for the 4096x14336 down projection, bf16 activations,
    M in {512, 2048, 4096}; TFLOP/s = 2*M*N*K / CUDA-event time (activation conversion included)."""
    toks = toks or [512, 2048, 4096]
    sampler = ClockSampler(ctx.device)
    sampler.start()
    l0 = ctx.launch_count
    per, flops, secs = {}, 0.0, 0.0
    reps = max(3, min(args.steps, 10))
    for name, segs, k in (("qkv_6144x4096[Q4_K 0-5119|Q6_K 5120-6143]", [(12, 5120), (14, 1024)], 4096),
                          ("o_4096x4096[Q4_K]", [(12, 4096)], 4096),
                          ("gate_up_28672x4096[Q4_K]", [(12, 28672)], 4096),
                          ("down_4096x14336[Q6_K]", [(14, 4096)], 14336)):
        ws = [hq.load_quant_weight(ctx, _random_weight(torch, oracle, dev, t, rows, k), t, rows, k) for t, rows in segs]
        n = sum(rows for _, rows in segs)
        for m in toks:
            x = torch.randn(m, k, device=dev).bfloat16()
            y = torch.empty(m, n, device=dev)

            def run():
                hq.ops.quantized_matmul_segments(ctx, x, ws, y, m)

            dt = _timed(torch, run, reps)
            per[f"{name}_M{m}"] = round(2.0 * m * n * k / dt / 1e12, 1)
            flops += 2.0 * m * n * k
            secs += dt
        del ws
    # the same gate/up product with the two tiles side by side and the SwiGLU in the epilogue, and the down product
    # with the residual in its epilogue (reported beside the sweep, not part of its sum)
    fused = {}
    # (scales of order 2^-11 keep gate and up of order one, as real activations are: the SiLU's division then stays on
    # its fast path; with |gate| in the thousands half of the divisions take the slow path for an infinite divisor)
    gq, uq = (hq.load_quant_weight(ctx, _random_weight(torch, oracle, dev, 12, 14336, 4096, exp_mask=0x0F), 12, 14336, 4096) for _ in range(2))
    dq = hq.load_quant_weight(ctx, _random_weight(torch, oracle, dev, 14, 4096, 14336), 14, 4096, 14336)
    for m in toks:
        x = torch.randn(m, 4096, device=dev).bfloat16()
        act = torch.empty(m, 14336, device=dev)
        dt = _timed(torch, lambda: hq.ops.quantized_matmul_swiglu(ctx, x, gq, uq, act, m), reps)
        fused[f"gate_up_swiglu_2x14336x4096[Q4_K]_M{m}"] = round(2.0 * m * 28672 * 4096 / dt / 1e12, 1)
        a16 = torch.randn(m, 14336, device=dev).bfloat16()
        res = torch.zeros(m, 4096, device=dev)
        dt = _timed(torch, lambda: hq.ops.quantized_matmul_add(ctx, a16, dq, res, res, m), reps)
        fused[f"down_add_4096x14336[Q6_K]_M{m}"] = round(2.0 * m * 4096 * 14336 / dt / 1e12, 1)
    del gq, uq, dq
    sus, burst, kind = measured_tensor_peaks()
    val = flops / secs / 1e12
    ctx.check_status()
    return {"metric": "prefill dequant-GEMM TFLOP/s", "value": round(val, 1), "unit": "TFLOP/s",
            "higher_is_better": True, "dtype": "f16 operands, f32 accumulate",
            "config": {"workload": "Q4_K_M prefill GEMM sweep (fused QKV with Q6_K V rows, Q4_K o and gate/up, Q6_K down), bf16 activations",
                       "tokens": toks, "timing": f"CUDA events over {reps} calls per case, activation conversion kernel included"},
            "roofline": {"bound": "tensor", "achieved": round(val, 1), "peak": sus, "unit": "TFLOP/s",
                         "frac": round(val / sus, 4), "peak_source": f"of {kind} (sustained)", "peak_burst": burst,
                         "frac_of_burst": round(val / burst, 4), "kernel": "gemm_tc_kernel", "traffic": None},
            "per_case_TFLOPs": per, "fused_epilogue_TFLOPs": fused, "gpu_launches": int(ctx.launch_count - l0), "clocks": sampler.stop()}


def bench_config1(hq, oracle, torch, ctx, dev, args) -> dict:
    """BASELINE config 1: one Q4_K 4096x4096 matrix, x f32 [1, 4096]; graph over 8 distinct copies."""
    t, n, k, m = 12, 4096, 4096, 1
    sampler = ClockSampler(ctx.device)
    sampler.start()
    ws = [hq.load_quant_weight(ctx, _random_weight(torch, oracle, dev, t, n, k), t, n, k) for _ in range(16)]
    x = torch.randn(m, k, device=dev)
    y = torch.empty(m, n, device=dev)
    pr = hq.GgmlQuantizedMatmulParams(m, n, k, t)

    def walk():
        for w in ws:
            hq.quantized_matmul_ggml(ctx, x, w, y, pr)

    graph = _graph_of(torch, walk)
    dt = _timed(torch, graph.replay, max(20, min(args.steps * 4, 200))) / len(ws)
    b = n * oracle.row_bytes(t, k) + 4 * k + 4 * n
    peak, kind = measured_hbm_peak()
    ctx.check_status()
    return {"metric": "Q4_K 4096x4096 f32 mat-vec", "value": round(b / dt / 1e9, 1), "unit": "GB/s", "us_per_launch": round(dt * 1e6, 2),
            "config": {"workload": "Q4_K 4096x4096, x f32 [1,4096]; CUDA graph over 16 distinct copies (151 MB, larger than L2)"},
            "roofline": {"bound": "hbm", "achieved": round(b / dt / 1e9, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(b / dt / 1e9 / peak, 4), "peak_source": f"of {kind}", "kernel": "gemv_mma_kernel<Q4_K>", "traffic": None},
            "clocks": sampler.stop()}


def bench_matvec(hq, oracle, torch, ctx, dev, args) -> dict:
    """Every block format on the decode shapes: per-launch time from a CUDA graph that walks 8
    distinct copies of the matrix (so weights come from HBM), bf16 activations."""
    peak_h, kind_h = measured_hbm_peak()
    per, tot_b, tot_s = {}, 0.0, 0.0
    l0 = ctx.launch_count
    sampler = ClockSampler(ctx.device)
    sampler.start()
    for t in ([int(args.qtype)] if args.qtype else [2, 8, 12, 13, 14]):
        for n, k in SHAPES:
            ws = [hq.load_quant_weight(ctx, _random_weight(torch, oracle, dev, t, n, k), t, n, k) for _ in range(8)]
            rb = oracle.row_bytes(t, k)
            for m in (1, 4, 8):
                x = torch.randn(m, k, device=dev).bfloat16()
                y = torch.empty(m, n, device=dev)
                pr = hq.GgmlQuantizedMatmulParams(m, n, k, t)

                def walk():
                    for w in ws:
                        hq.quantized_matmul_ggml(ctx, x, w, y, pr)

                graph = _graph_of(torch, walk)
                dt = _timed(torch, graph.replay, max(3, min(args.steps, 20))) / len(ws)
                b = n * rb + 2 * m * k + 4 * m * n
                per[f"{oracle.TYPE_NAMES[t]}_{n}x{k}_m{m}"] = {"us": round(dt * 1e6, 2), "GBps": round(b / dt / 1e9, 1)}
                tot_b += b
                tot_s += dt
            del ws
    val = tot_b / tot_s / 1e9
    ctx.check_status()
    return {"metric": "dequant-GEMV HBM GB/s (all block formats)", "value": round(val, 1), "unit": "GB/s",
            "higher_is_better": True, "dtype": "f32",
            "config": {"workload": "decode mat-vec, 4 shapes x m in {1,4,8} x block formats, bf16 activations; "
                                   "CUDA graph over 8 copies of each matrix (inputs larger than L2)"},
            "roofline": {"bound": "hbm", "achieved": round(val, 1), "peak": peak_h, "unit": "GB/s", "frac": round(val / peak_h, 4),
                         "peak_source": f"of {kind_h}", "kernel": "gemv_mma_kernel", "traffic": None},
            "per_launch": per, "gpu_launches": int(ctx.launch_count - l0), "clocks": sampler.stop()}


def bench_moe(hq, oracle, torch, ctx, dev, args, toks=None) -> dict:
    """BASELINE config 4: 256 experts, hidden 2048, intermediate 512, top-8, Q5_K; the whole expert
    layer (router softmax/top-k outputs -> gate, up, SwiGLU, down, weighted combine) at T in {1, 2048}."""
    t, E, H, I, topk = 13, 256, 2048, 512, 8
    sg, sd = hq.expert_stride(t, I, H), hq.expert_stride(t, H, I)
    # scales of order 2^-11: the SwiGLU output feeds the down product as f16 and must stay inside its range
    wg, wu, wd = (_random_weight(torch, oracle, dev, t, E * I, H, exp_mask=0x0F), _random_weight(torch, oracle, dev, t, E * I, H, exp_mask=0x0F),
                  _random_weight(torch, oracle, dev, t, E * H, I, exp_mask=0x0F))
    res = {}
    l0 = ctx.launch_count
    sampler = ClockSampler(ctx.device)
    sampler.start()
    sus, burst, kind_t = measured_tensor_peaks()
    peak_h, kind_h = measured_hbm_peak()
    for T in (toks or [1, 2048]):
        # decode (few tokens) touches 8 experts = 17 MB per layer, far less than L2: rotate over
        # routings that pick different experts so that weights come from HBM; one CUDA graph
        # holds all of them (launch overhead of the Python calls stays out of the timing)
        nsets = 16 if T <= 8 else 1
        x = (torch.randn(T, H, device=dev) * 0.02).bfloat16()
        R = T * topk
        g, u = torch.empty(R, I, device=dev), torch.empty(R, I, device=dev)
        d = torch.empty(R, H, device=dev)
        out = torch.empty(T, H, device=dev)
        sc = hq.IdMmScratch.alloc(ctx, E, R, H)
        pg = hq.GgmlQuantizedMatmulIdParams(T, topk, I, H, E, sg, t)
        pd = hq.GgmlQuantizedMatmulIdParams(R, 1, H, I, E, sd, t)
        id_sets, wt_sets = [], []
        for i in range(nsets):
            if T <= 8:          # disjoint expert groups per set
                logits = torch.full((T, E), -30.0, device=dev)
                logits[:, (i * topk * T) % E:(i * topk * T) % E + topk * T] = torch.randn(T, topk * T, device=dev)
            else:
                logits = torch.randn(T, E, device=dev)
            ids, wts = hq.moe_softmax_topk(ctx, logits, topk)
            id_sets.append(ids)
            wt_sets.append(wts)

        fused = hq.ops.quantized_matmul_id_swiglu_supported(ctx, pg, x.dtype)
        experts = hq.ops.moe_experts_supported(ctx, T, topk, H, I, E, t, t)

        def layer(ids, wts):
            if experts:   # many routed rows: sort + gather, gate/up pair with the SwiGLU epilogue, down
                hq.ops.moe_experts(ctx, x, wg.data_ptr(), wu.data_ptr(), wd.data_ptr(), ids, d, T, topk, H, I, E, t, t, sg, sd)
            else:
                if fused:     # few routed rows: gate, up and the SwiGLU in one launch
                    hq.ops.quantized_matmul_id_swiglu_ggml(ctx, x, wg.data_ptr(), wu.data_ptr(), ids, g, pg)
                else:
                    hq.quantized_matmul_id_pair_ggml(ctx, x, wg.data_ptr(), wu.data_ptr(), ids, g, u, sc, pg)   # gate + up
                    ctx._check(ctx._lib.hf2q_cuda_silu_mul(ctx._h, ctx._stream(), g.data_ptr(), u.data_ptr(), g.data_ptr(), g.numel()))
                hq.quantized_matmul_id_ggml(ctx, g, wd.data_ptr(), ids, d, sc, pd)
            ctx._check(ctx._lib.hf2q_cuda_moe_combine(ctx._h, ctx._stream(), d.data_ptr(), wts.data_ptr(), None, None, None,
                                                      out.data_ptr(), T, topk, H))

        def all_sets():
            for ids, wts in zip(id_sets, wt_sets):
                layer(ids, wts)

        graph = _graph_of(torch, all_sets)
        dt = _timed(torch, graph.replay, max(3, min(args.steps, 20))) / nsets
        dt_atomic = None
        if experts:
            # the opt-in form: weighted reduce inside the down product (f32 atomics), no [rows][hidden] round trip
            def layer_atomic():
                out.zero_()
                hq.ops.moe_experts_reduce(ctx, x, wg.data_ptr(), wu.data_ptr(), wd.data_ptr(), id_sets[0], wt_sets[0], out, T, topk, H, I, E, t, t)
            dt_atomic = _timed(torch, _graph_of(torch, layer_atomic).replay, max(3, min(args.steps, 20)))
        nexp = int(torch.unique(id_sets[0]).numel())
        wbytes = nexp * (2 * sg + sd)
        fl = 2.0 * R * 3 * I * H
        t_hbm, t_tc = wbytes / (peak_h * 1e9), fl / (sus * 1e12)
        res[f"T{T}"] = {"us_per_layer": round(dt * 1e6, 1), "TFLOPs": round(fl / dt / 1e12, 2),
                        "weight_GBps": round(wbytes / dt / 1e9, 1), "experts_touched": nexp,
                        "roofline_hbm_us": round(t_hbm * 1e6, 1), "roofline_tensor_us": round(t_tc * 1e6, 1),
                        "frac_of_binding_roofline": round(max(t_hbm, t_tc) / dt, 4),
                        "us_per_layer_reduce_in_down_product": round(dt_atomic * 1e6, 1) if dt_atomic else None,
                        "swiglu_in_gate_up_launch": bool(fused or experts), "launches_per_layer": 5 if experts else (3 if fused else None),
                        "timing": f"CUDA graph of {nsets} layer(s) with different routings; gate+up, SwiGLU, down and the weighted combine"}
    ctx.check_status()
    last = res[sorted(res)[-1]]
    return {"metric": "MoE mul_mat_id layer time", "value": last["us_per_layer"], "unit": "us",
            "higher_is_better": False, "dtype": "f16 operands, f32 accumulate",
            "config": {"workload": "Qwen3-style A3B expert layer: 256 experts, hidden 2048, intermediate 512, top-8, Q5_K; "
                                   "gate + up + SwiGLU + down mul_mat_id + weighted combine (router outputs from the softmax/top-k kernel)"},
            "roofline": {"bound": "hbm", "achieved": last["weight_GBps"], "peak": peak_h, "unit": "GB/s",
                         "frac": round(last["weight_GBps"] / peak_h, 4), "peak_source": f"of {kind_h}; tensor: {kind_t} sustained",
                         "kernel": "gemm_tc_kernel<grouped> + moe_sort/gather (T=2048), gemv_mma_kernel (T=1)", "traffic": None},
            "per_case": res, "gpu_launches": int(ctx.launch_count - l0), "clocks": sampler.stop()}


def bench_attention(hq, oracle, torch, ctx, dev, args) -> dict:
    """The decode step's attention launch alone (config 5 shapes: 32 query / 8 KV heads of 128, 8-bit KV): rotary
    embedding of the query, append of the new position, split attention over `--tokens` cached positions and the
    merge, one launch per layer; 8 layers with their own caches rotate so that the cache comes from HBM."""
    import ctypes as C
    from hf2q_b200 import decoder as D
    n_ctx, layers, n_q, n_kv, hd = (args.tokens or 8192), 8, 32, 8, 128
    max_seq = n_ctx + 64
    bufs, kvs = [], []
    g = torch.Generator(device=dev).manual_seed(0)
    for _ in range(layers):
        kc = torch.randint(-127, 128, (n_kv, max_seq, hd), dtype=torch.int8, device=dev, generator=g)
        vc = torch.randint(-127, 128, (n_kv, max_seq, hd), dtype=torch.int8, device=dev, generator=g)
        ks = torch.rand((n_kv, max_seq), device=dev, generator=g) * 0.02
        vs = torch.rand((n_kv, max_seq), device=dev, generator=g) * 0.02
        bufs.append((kc, ks, vc, vs))
        kvs.append(D._KvCache(kc.data_ptr(), ks.data_ptr(), vc.data_ptr(), vs.data_ptr(), n_kv, hd, max_seq))
    qkv = torch.randn((1, (n_q + 2 * n_kv) * hd), device=dev, generator=g)
    out = torch.empty((1, n_q * hd), device=dev)
    pos = torch.full((1,), n_ctx, dtype=torch.int32, device=dev)
    need = C.c_uint64()
    ctx._check(ctx._lib.hf2q_cuda_attn_decode_scratch_bytes(ctx._h, n_q, n_kv, C.byref(need)))
    scratch = torch.zeros(max(need.value, 16), dtype=torch.uint8, device=dev)

    def all_layers():
        for kv in kvs:
            ctx._check(ctx._lib.hf2q_cuda_attn_decode_fused(ctx._h, ctx._stream(), qkv.data_ptr(), n_q, 500000.0, C.byref(kv), pos.data_ptr(),
                                                            out.data_ptr(), hq.ops.DT_F32, scratch.data_ptr(), scratch.numel()))

    sampler = ClockSampler(ctx.device)
    sampler.start()
    l0 = ctx.launch_count
    graph = _graph_of(torch, all_layers)
    dt = _timed(torch, graph.replay, max(3, min(args.steps, 20))) / layers
    ctx.check_status()
    kv_bytes = 2 * n_kv * (n_ctx + 1) * (hd + 4)
    peak, kind = measured_hbm_peak()
    return {"metric": "decode attention time per layer", "value": round(dt * 1e6, 2), "unit": "us", "higher_is_better": False,
            "dtype": "int8 KV codes, f32 scores and accumulation",
            "config": {"workload": f"decode attention, 32 query / 8 KV heads of 128, 8-bit KV cache, {n_ctx} cached positions; "
                                   f"one launch per layer (rotary, append, split attention, merge), {layers} layers rotating",
                       "timing": "CUDA events around replays of one CUDA graph of the layers"},
            "roofline": {"bound": "hbm", "achieved": round(kv_bytes / dt / 1e9, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(kv_bytes / dt / 1e9 / peak, 4), "peak_source": f"of {kind}", "kernel": "attn_decode_fused_kernel",
                         "traffic": None},
            "gpu_launches": int(ctx.launch_count - l0), "clocks": sampler.stop()}


def build_llama_weights(hq, oracle, torch, ctx, dev, cfg, distinct_rows: int = 16384):
    """Random-init Llama-shaped weights under the Q4_K_M type map, quantized by the oracle's port of
    hf2q's quantizers.  To keep the host work to seconds, ONE tensor is quantized per distinct (role,
    block format) and every layer gets its own device copy of those bytes (so a decode step streams
    every layer from HBM); the two vocabulary-sized tensors repeat a block of `distinct_rows` rows."""
    from hf2q_b200 import decoder as D
    from tests.util import make_quant_weight
    types = D.q4_k_m_types(cfg)
    cache = {}

    def raw(role, t, n, k, seed):
        key = (role, t)
        if key not in cache:
            cache[key] = torch.from_numpy(make_quant_weight(t, n, k, seed=seed)).to(dev)
        return cache[key]

    def weight(role, t, n, k, seed):
        return hq.load_quant_weight(ctx, raw(role, t, n, k, seed).clone(), t, n, k)

    def vocab_weight(role, t, seed):
        rows = min(distinct_rows, cfg.vocab)
        block = raw(role, t, rows, cfg.hidden, seed)
        reps = (cfg.vocab + rows - 1) // rows
        rb = oracle.row_bytes(t, cfg.hidden)
        full = block.repeat(reps)[: cfg.vocab * rb].contiguous()
        return hq.load_quant_weight(ctx, full, t, cfg.vocab, cfg.hidden)

    ones = lambda: torch.ones(cfg.hidden, dtype=torch.float32, device=dev)
    layers = []
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        same = types[p + "attn_v"] == types[p + "attn_q"]        # V shares the block format of Q and K: one tensor, one launch
        layers.append(D.LayerWeights(
            ones(),
            weight("qkv", types[p + "attn_q"], cfg.q_rows + 2 * cfg.kv_rows, cfg.hidden, 9) if same
            else weight("qk", types[p + "attn_q"], cfg.q_rows + cfg.kv_rows, cfg.hidden, 1),
            None if same else weight("v", types[p + "attn_v"], cfg.kv_rows, cfg.hidden, 2),
            weight("o", types[p + "attn_output"], cfg.hidden, cfg.q_rows, 3), ones(),
            weight("gate", types[p + "ffn_gate"], cfg.ffn, cfg.hidden, 4), weight("up", types[p + "ffn_up"], cfg.ffn, cfg.hidden, 5),
            weight("down", types[p + "ffn_down"], cfg.hidden, cfg.ffn, 6)))
    return D.ModelWeights(vocab_weight("embd", types["token_embd"], 7), layers, ones(), vocab_weight("out", types["output"], 8))


def bench_decode_tp(hq, oracle, torch, ctx, dev, args, rank, world, barrier) -> dict | None:
    """BASELINE config 5 on `world` GPUs: the tensor-parallel decode step (hf2q_b200/decoder_tp.py) on Llama-3-8B
    shapes.  Every rank holds its shard of every tensor (random block bytes with small scales: throughput does not
    depend on the values); the 8-bit KV caches of the rank's heads are filled with random codes for 8192
    positions instead of running a prefill; 100 greedy tokens from one captured CUDA graph per rank."""
    import torch.distributed as dist
    from hf2q_b200 import decoder as D, decoder_tp as TP
    cfg = D.LlamaConfig()
    if cfg.n_kv_heads % world or cfg.vocab % world or cfg.ffn % world:
        return None
    types = D.q4_k_m_types(cfg)
    n_ctx, n_new = 8192, 100
    hl, kl, fl, vl = cfg.n_heads // world, cfg.n_kv_heads // world, cfg.ffn // world, cfg.vocab // world

    def weight(t, n, k):
        # block scales below 2^-15: weights of a few hundredths, the size of a random-init model's, so that 32 layers
        # of random weights keep their activations inside the f16 range
        return hq.load_quant_weight(ctx, _random_weight(torch, oracle, dev, t, n, k, exp_mask=0x03), t, n, k)

    ones = lambda: torch.ones(cfg.hidden, dtype=torch.float32, device=dev)
    layers = []
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        tq, tv = types[p + "attn_q"], types[p + "attn_v"]
        same = tq == tv
        layers.append(TP.TpLayerWeights(
            ones(), weight(tq, (hl + kl + (kl if same else 0)) * cfg.head_dim, cfg.hidden), None if same else weight(tv, kl * cfg.head_dim, cfg.hidden),
            weight(types[p + "attn_output"], cfg.hidden, hl * cfg.head_dim), ones(),
            weight(types[p + "ffn_gate"], fl, cfg.hidden), weight(types[p + "ffn_up"], fl, cfg.hidden),
            weight(types[p + "ffn_down"], cfg.hidden, fl) if TP.column_shard_ok(types[p + "ffn_down"], cfg.ffn, world)
            else weight(types[p + "ffn_down"], cfg.hidden // world, cfg.ffn)))
    embd = hq.load_quant_weight(ctx, _random_weight(torch, oracle, dev, types["token_embd"], 16384, cfg.hidden, exp_mask=0x03).repeat(8)[
        : cfg.vocab * oracle.row_bytes(types["token_embd"], cfg.hidden)].contiguous(), types["token_embd"], cfg.vocab, cfg.hidden)
    w = TP.TpModelWeights(embd, layers, ones(), weight(types["output"], vl, cfg.hidden))
    dec = TP.TensorParallelDecoder(ctx, cfg, w)
    g = torch.Generator(device=dev).manual_seed(rank)
    for kc, ks, vc, vs in dec.kv_bufs:
        kc[:, :n_ctx].copy_(torch.randint(-127, 128, kc[:, :n_ctx].shape, dtype=torch.int8, device=dev, generator=g))
        vc[:, :n_ctx].copy_(torch.randint(-127, 128, vc[:, :n_ctx].shape, dtype=torch.int8, device=dev, generator=g))
        ks[:, :n_ctx].fill_(0.01)
        vs[:, :n_ctx].fill_(0.01)
    dec.pos.fill_(n_ctx)
    dec.tok.fill_(1)
    dec.generate(6, use_graph=True, collect=False)              # captures the step and warms the replay
    dec.pos.fill_(n_ctx)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    dec.generate(n_new, use_graph=True, collect=False)
    e1.record()
    barrier()
    status = "ok"
    try:                                   # every rank goes on to the collective calls below whatever its own status word says
        ctx.check_status()
    except hq.Hf2qError as exc:
        status = str(exc)
    tt = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    dt = float(tt.item()) * 1e-3
    finite = bool(torch.isfinite(dec.logits).all().item())
    wbytes = dec.weight_bytes_per_token()
    line = {"metric": "decode tok/s", "value": round(n_new / dt, 1), "unit": "tok/s", "higher_is_better": True,
            "ms_per_token": round(1e3 * dt / n_new, 4),
            "config": {"workload": f"Llama-3-8B shapes, Q4_K_M type map, tensor-parallel over {world} GPUs: QKV / gate / up sharded by rows, O / down by "
                                   f"their contraction dimension with the partial sums exchanged inside the products' gather epilogue and added in rank order "
                                   f"(Q6_K down tensors, whose column shards would lose the 16-byte row alignment, by rows with their input gathered first), "
                                   f"output head sharded by vocabulary; "
                                   f"{n_new} greedy tokens at {n_ctx} cached positions (caches filled with random codes, no prefill)",
                       "launch_mode": "one CUDA graph of the decode step per rank; no NCCL call and no host synchronisation inside a step"},
            "weight_bytes_per_token_per_rank": wbytes, "launches_per_token_per_rank": dec.launches_per_token, "logits_finite": finite,
            "status_rank0": status}
    dec.close()
    return line


def bench_decode(hq, oracle, torch, ctx, dev, args) -> dict:
    """BASELINE config 5: random-init decoder forward on Llama-3-8B shapes, Q4_K_M weights, 8-bit KV cache
    with room for 32K positions; greedy decode of 200 tokens after an 8192-token prefill of uniform-random
    ids.  One GPU; the decode loop is one captured CUDA graph replayed per token."""
    from hf2q_b200 import decoder as D
    cfg = D.LlamaConfig()
    n_prompt, n_new = (args.tokens or 8192), 200
    sampler = ClockSampler(ctx.device)
    t0 = time.perf_counter()
    w = build_llama_weights(hq, oracle, torch, ctx, dev, cfg)
    dec = D.LlamaDecoder(ctx, cfg, w)
    t_build = time.perf_counter() - t0
    ids = torch.randint(0, cfg.vocab, (n_prompt,), dtype=torch.int32, device=dev, generator=torch.Generator(device=dev).manual_seed(0))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    dec.prefill(ids)
    e1.record()
    torch.cuda.synchronize()
    ctx.check_status()
    prefill_s = e0.elapsed_time(e1) * 1e-3
    state = (dec.pos.clone(), dec.tok.clone())
    dec.generate(8, use_graph=True, collect=False)              # captures the step and warms the replay
    dec.pos.copy_(state[0]); dec.tok.copy_(state[1])
    torch.cuda.synchronize()
    l0 = ctx.launch_count
    sampler.start()
    e0.record()
    dec.generate(n_new, use_graph=True, collect=False)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ctx.check_status()
    dt = e0.elapsed_time(e1) * 1e-3
    assert int(dec.pos.item()) == n_prompt + n_new
    logits_finite = bool(torch.isfinite(dec.logits).all().item())
    tok_s = n_new / dt
    wbytes = dec.weight_bytes_per_token()
    ctx_mid = n_prompt + n_new // 2
    kvbytes = dec.kv_bytes_per_position() * ctx_mid
    peak, kind = measured_hbm_peak()
    roof_tok_s = peak * 1e9 / (wbytes + kvbytes)
    return {"metric": "decode tok/s", "value": round(tok_s, 1), "unit": "tok/s", "higher_is_better": True,
            "ms_per_token": round(1e3 * dt / n_new, 4), "dtype": "f32 activations, f32 accumulate, int8 KV",
            "config": {"workload": f"Llama-3-8B shapes (32 layers, hidden 4096, 32/8 heads, head dim 128, FFN 14336, vocab 128256, RMSNorm, RoPE theta 500000), "
                                   f"Q4_K_M type map (Q6_K attn_v / ffn_down on 16 layers, Q6_K output), 8-bit per-(head, position)-scaled KV cache sized for 32K positions; "
                                   f"greedy decode of {n_new} tokens after a {n_prompt}-token prefill of uniform-random ids",
                       "weights": "N(0, sigma=0.02) quantized by the oracle's port of hf2q's quantizers: one tensor per (role, format), a device copy per layer",
                       "launch_mode": "one CUDA graph of the whole decode step, replayed per token; token id and position stay on the device"},
            "roofline": {"bound": "hbm", "achieved": round((wbytes + kvbytes) / (dt / n_new) / 1e9, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(tok_s / roof_tok_s, 4), "peak_source": f"of {kind}", "roofline_tok_s": round(roof_tok_s, 1),
                         "weight_bytes_per_token": wbytes, "kv_bytes_per_token_at_mid_context": kvbytes,
                         "kernel": "gemv_mma_kernel (7 products per layer in 4-5 launches) + attn_decode_fused_kernel + glue", "traffic": None},
            "prefill": {"tokens": n_prompt, "seconds": round(prefill_s, 3), "tok_s": round(n_prompt / prefill_s, 1),
                        "note": "tensor-core GEMMs with fused epilogues + tensor-core causal attention over the 8-bit cache; not the timed metric"},
            "launches_per_token": dec.launches_per_token, "gpu_launches": int(dec.launches_per_token * n_new), "logits_finite": logits_finite,
            "host_seconds_building_weights": round(t_build, 1), "eager_launches_seen": int(ctx.launch_count - l0), "clocks": clocks}


def run_secondary(args) -> None:
    """One of the other workloads alone on one GPU: one JSON line."""
    import torch

    import hf2q_b200 as hq
    import oracle

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ctx = hq.GpuContext(0)
    toks = [args.tokens] if args.tokens else None
    if args.workload == "gemm":
        line = bench_gemm(hq, oracle, torch, ctx, dev, args, toks)
    elif args.workload == "matvec":
        line = bench_matvec(hq, oracle, torch, ctx, dev, args)
    elif args.workload == "config1":
        line = bench_config1(hq, oracle, torch, ctx, dev, args)
    elif args.workload == "decode":
        line = bench_decode(hq, oracle, torch, ctx, dev, args)
    elif args.workload == "attention":
        line = bench_attention(hq, oracle, torch, ctx, dev, args)
    else:
        line = bench_moe(hq, oracle, torch, ctx, dev, args, toks)
    line.update({"n_gpus": 1, "data": "synthetic"})
    print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--copies", type=int, default=8, help="distinct device copies of the four matrices")
    ap.add_argument("--passes", type=int, default=16, help="passes over all copies x shapes x token counts per step")
    ap.add_argument("--e2e-steps", type=int, default=0, help="passes of the host-buffer leg (0 = auto)")
    ap.add_argument("--no-chain-wait", action="store_true",
                    help="several GPUs: products do not wait for the previous product's columns (analysis aid)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="one GPU: skip the config 1 / GEMM / MoE measurements")
    ap.add_argument("--no-decode", action="store_true", help="one GPU: skip the full-decoder decode tok/s measurement")
    ap.add_argument("--no-strong", action="store_true", help="several GPUs: skip the strong-scaling leg")
    ap.add_argument("--no-graph", action="store_true", help="issue launches eagerly instead of replaying a CUDA graph")
    ap.add_argument("--qtype", default="", help="matvec: one ggml type number (2, 8, 12, 13, 14) instead of all five")
    ap.add_argument("--workload", default="gemv", choices=["gemv", "gemm", "moe", "matvec", "config1", "decode", "attention"],
                    help="gemv: the headline Q6_K decode sweep (default, carries the others as `secondary`); gemm: Q4_K_M prefill "
                         "GEMM sweep; moe: Qwen3-style A3B expert layer (Q5_K mul_mat_id); matvec: all block formats; config1: Q4_K 4096^2 f32")
    ap.add_argument("--tokens", type=int, default=0, help="gemm/moe: one token count instead of the sweep")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload != "gemv":
        run_secondary(args)
        return

    import torch
    import torch.distributed as dist

    import hf2q_b200 as hq
    import oracle
    from tests.util import rel_l2

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    oracle.set_threads(max(1, host_threads() // max(1, world)))      # torchrun exports OMP_NUM_THREADS=1
    ctx = hq.GpuContext(local_rank)

    # ---- inputs: every rank builds its own shard set (distinct seeds per rank) ----
    raws = make_weights(seed0=10 * rank)
    xbits, xvals = host_inputs()
    row_b = {k: oracle.row_bytes(Q6_K, k) for _, k in SHAPES}
    weights = []     # [copy][shape] -> QuantWeight
    for c in range(args.copies):
        weights.append([hq.load_quant_weight(ctx, torch.from_numpy(r).to(dev), Q6_K, n, k)
                        for r, (n, k) in zip(raws, SHAPES)])
    xdev = {key: torch.from_numpy(b.view(np.int16).copy()).to(dev).view(torch.bfloat16).reshape(key[1], key[0])
            for key, b in xbits.items()}
    ydev = {(n, m): torch.empty((m, n), dtype=torch.float32, device=dev) for n, _ in SHAPES for m in TOKENS}
    # Several GPUs: each rank's shard is rows [rank*n, (rank+1)*n) of a matrix world*n rows tall, and the
    # kernel itself stores its columns into every rank's full-width output (peer stores + arrival
    # counters, hf2q_b200.dist.GatherGroup; two alternating output buffers); each product waits for the
    # previous one's columns from all ranks before it reads its activations, as a decode chain would.
    gather = None
    if world > 1:
        from hf2q_b200.dist import GatherGroup
        try:
            gather = GatherGroup(ctx, max(TOKENS), world * max(n for n, _ in SHAPES))
        except RuntimeError as exc:          # raised on every rank or on none
            if rank == 0:
                print(f"[bench] {exc}; using NCCL all-gathers after each product (eager launches)", file=sys.stderr)
    ygath = {}
    if world > 1 and gather is None:
        ygath = {(n, m): torch.empty((world, m, n), dtype=torch.float32, device=dev) for n, _ in SHAPES for m in TOKENS}
    params = {(n, k, m): hq.GgmlQuantizedMatmulParams(m, n, k, Q6_K) for n, k in SHAPES for m in TOKENS}

    launches_per_pass = args.copies * len(SHAPES) * len(TOKENS)
    bytes_per_pass = args.copies * sum(algo_bytes(n, k, m, row_b[k]) for n, k in SHAPES for m in TOKENS)
    working_set = args.copies * sum(len(r) for r in raws)

    def one_pass(grp):
        for m in TOKENS:
            for c in range(args.copies):
                for (n, k), w in zip(SHAPES, weights[c]):
                    if grp is None:
                        hq.quantized_matmul_ggml(ctx, xdev[(k, m)], w, ydev[(n, m)], params[(n, k, m)])
                        if world > 1:
                            dist.all_gather_into_tensor(ygath[(n, m)], ydev[(n, m)])
                    else:
                        grp.matmul(xdev[(k, m)], w, m, rank * n, wait_previous=not args.no_chain_wait)
        if grp is not None:
            grp.wait()           # the pass ends when every rank's columns of the last product are here

    def step():
        for _ in range(args.passes):
            one_pass(gather)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- parity before timing (the oracle is the checker, never the timed path) ----
    # One GPU: one product against the f64 product on the oracle's weights.  Several GPUs: EVERY rank
    # checks one gathered full-width product -- all ranks' columns as they arrived in its own buffer
    # -- against the oracle; any mismatch ends the run with a non-zero exit code.
    wref = {}

    def ref_weight(r, i):
        # rank r's copy of shape i (its seed), dequantised by the oracle
        if (r, i) not in wref:
            n, k = SHAPES[i]
            raw = raws[i] if r == rank else make_weights_one(i, seed0=10 * r)
            wref[(r, i)] = oracle.dequantize(Q6_K, raw).reshape(n, k)
        return wref[(r, i)]

    def make_weights_one(i, seed0):
        from tests.util import make_quant_weight
        n, k = SHAPES[i]
        return make_quant_weight(Q6_K, n, k, seed=seed0 + i)

    verify = {"checked": None}
    n1, k1 = SHAPES[1]
    if gather is None:
        y = ydev[(n1, 4)]
        hq.quantized_matmul_ggml(ctx, xdev[(k1, 4)], weights[0][1], y, params[(n1, k1, 4)])
        ctx.check_status()
        err = rel_l2(y.cpu().numpy(), oracle.matmul_f64(xvals[(k1, 4)], ref_weight(rank, 1)))
        if not err < 1e-3:
            raise SystemExit(f"parity check failed before timing: rel L2 {err}")
        verify = {"checked": "4096x4096 m=4 on this GPU", "rel_l2": err}
    else:
        barrier()
        ok = 1.0
        errs = []
        for i, m in ((1, 4), (3, 8)):                   # a single-phase shape and the k-phase shape
            n, k = SHAPES[i]
            gather.matmul(xdev[(k, m)], weights[0][i], m, rank * n, wait_previous=True)
            gather.wait()
            torch.cuda.synchronize()
            got = gather.output(m)[:, : world * n].cpu().numpy()
            want = np.concatenate([oracle.matmul_f64(xvals[(k, m)], ref_weight(r, i)) for r in range(world)], axis=1)
            err = rel_l2(got, want)
            errs.append(err)
            if not err < 1e-3:
                ok = 0.0
            dist.barrier()
        try:
            ctx.check_status()
        except hq.Hf2qError:
            ok = 0.0
        vote = torch.tensor([ok], device=dev)
        dist.all_reduce(vote, op=dist.ReduceOp.MIN)
        if float(vote.item()) < 1.0:
            print(f"[bench] rank {rank}: gathered product differs from the oracle (rel L2 {errs}) or a wait ran out", file=sys.stderr)
            dist.destroy_process_group()
            raise SystemExit(3)
        verify = {"checked": f"gathered full-width products (4096x4096 m=4, 4096x14336 m=8) on all {world} ranks", "rel_l2_rank0": max(errs)}
        wref.clear()

    for _ in range(args.warmup):
        one_pass(gather)
    barrier()
    # One step's launches are captured into a CUDA graph and replayed (what a decode loop does); the
    # multi-GPU step contains no collective call (the all-gather is in the kernels), so it is captured
    # the same way.  (One pass holds an even number of products, so the two output buffers alternate
    # consistently across replays.)
    graph = None
    if not args.no_graph and (world == 1 or gather is not None):     # NCCL calls are not captured
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step()
            graph = g
        except Exception as exc:      # capture unsupported: fall back to eager launches, say so
            print(f"[bench] graph capture failed ({exc}); timing eager launches", file=sys.stderr)
            graph = None
    run_step = graph.replay if graph is not None else step
    graph_used = graph is not None
    for _ in range(3):
        run_step()
    barrier()
    l0 = ctx.launch_count
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        run_step()
    ev1.record()
    barrier()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1)
    per_step_launches = args.passes * (launches_per_pass + (1 if gather is not None else 0))
    gpu_launches = (ctx.launch_count - l0) if graph is None else per_step_launches * args.steps
    ctx.check_status()
    if world > 1:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    ms_per_step = ms / args.steps
    bytes_per_step = args.passes * bytes_per_pass
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    per_gpu = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # ---- per-(m) breakdown, kernel only, rank-local (explains the aggregate) ----
    breakdown = {}
    for m in TOKENS:
        def walk_m():
            for c in range(args.copies):
                for (n, k), w in zip(SHAPES, weights[c]):
                    hq.quantized_matmul_ggml(ctx, xdev[(k, m)], w, ydev[(n, m)], params[(n, k, m)])
        gm = _graph_of(torch, walk_m)
        dt = _timed(torch, gm.replay, max(5, min(20, args.steps)))
        b = args.copies * sum(algo_bytes(n, k, m, row_b[k]) for n, k in SHAPES)
        breakdown[f"m{m}_GBps"] = round(b / dt / 1e9, 1)
        del gm

    # ---- strong scaling (several GPUs): the listed shapes themselves, rows split over the ranks ----
    strong = None
    if gather is not None and not args.no_strong:
        sw = []
        for c in range(args.copies):
            row = []
            for (n, k), w in zip(SHAPES, weights[c]):
                row.append(w.row_slice(0, n // world))          # any n/world rows of the rank's bytes: same work
            sw.append(row)
        sg = GatherGroup(ctx, max(TOKENS), max(n for n, _ in SHAPES))

        def strong_pass():
            for m in TOKENS:
                for c in range(args.copies):
                    for (n, k), w in zip(SHAPES, sw[c]):
                        sg.matmul(xdev[(k, m)], w, m, rank * (n // world), wait_previous=True)
            sg.wait()

        def strong_step():
            for _ in range(args.passes):
                strong_pass()

        for _ in range(3):
            strong_pass()
        barrier()
        gs = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gs):
            strong_step()
        for _ in range(2):
            gs.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, min(args.steps, 10))
        e0.record()
        for _ in range(reps):
            gs.replay()
        e1.record()
        barrier()
        sms = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(sms, op=dist.ReduceOp.MAX)
        ctx.check_status()
        strong = {"ms_per_step": round(float(sms.item()), 4), "GBps": round(bytes_per_step / (float(sms.item()) * 1e-3) / 1e9, 1),
                  "what": f"the listed shapes split {world} ways by rows (total bytes = the one-GPU sweep's); same kernels, same chain waits; "
                          "divide by the one-GPU value of this bench for the speed-up"}
        del gs
        sg.close()

    # ---- expert-parallel MoE layer (several GPUs): BASELINE config 4 with the experts split 256 / G per GPU ----
    moe_ep = None
    if world > 1 and not args.no_strong:
        from hf2q_b200.dist import Comm
        t5, E, H, I, topk, T = 13, 256, 2048, 512, 8, 2048
        comm = Comm(ctx)
        e_local = E // world
        sg, sdn = hq.expert_stride(t5, I, H), hq.expert_stride(t5, H, I)
        wg, wu, wd = (_random_weight(torch, oracle, dev, t5, e_local * I, H, 0x0F), _random_weight(torch, oracle, dev, t5, e_local * I, H, 0x0F),
                      _random_weight(torch, oracle, dev, t5, e_local * H, I, 0x0F))
        t_local = T // world                                   # tokens are sharded over the ranks as well
        R = t_local * topk
        gen = torch.Generator(device=dev).manual_seed(100 + rank)
        logits = torch.randn(t_local, E, device=dev, generator=gen)
        ids5, wts5 = hq.moe_softmax_topk(ctx, logits, topk)
        xrows = (torch.randn(t_local, H, device=dev, generator=gen) * 0.02).bfloat16().repeat_interleave(topk, dim=0).contiguous()
        cap = T * topk                                          # every routed row of the job could land on one rank
        need = ctypes.c_uint64()
        comm._check(comm.lib.hf2q_cuda_moe_experts_ep_scratch_bytes(R, cap, world, H, I, E, hq.ops.DT_BF16, ctypes.byref(need)))
        scr = torch.empty(need.value, dtype=torch.uint8, device=dev)
        yrows = torch.empty((R, H), dtype=torch.float32, device=dev)
        outl = torch.empty((t_local, H), dtype=torch.float32, device=dev)

        def ep_layer():
            comm.moe_experts_ep(xrows, ids5, wg.data_ptr(), wu.data_ptr(), wd.data_ptr(), H, I, E, sg, sdn, t5, t5, cap, scratch=scr, out=yrows)
            ctx._check(ctx._lib.hf2q_cuda_moe_combine(ctx._h, ctx._stream(), yrows.data_ptr(), wts5.data_ptr(), None, None, None, outl.data_ptr(),
                                                      t_local, topk, H))

        for _ in range(3):
            ep_layer()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            ep_layer()
        e1.record()
        barrier()
        tt = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ctx.check_status()
        us = float(tt.item()) * 1e3
        moe_ep = {"metric": "expert-parallel MoE layer time", "value": round(us, 1), "unit": "us", "higher_is_better": False,
                  "tokens_per_s": round(T / (us * 1e-6), 1),
                  "config": {"workload": f"256 experts (Q5_K, hidden 2048, intermediate 512, top-8) split {e_local} per GPU over {world} GPUs; "
                                         f"{T} tokens sharded {t_local} per GPU; hf2q_cuda_moe_experts_ep (device pack, ncclSend/Recv all-to-all, gate+up, "
                                         "SwiGLU, down at the owner, all-to-all back, device unpack) + weighted combine; one host read-back of the row counts per call",
                             "timing": f"CUDA events over {reps} eager calls, max over ranks"}}
        comm.close()

    # ---- tensor-parallel decode (several GPUs): BASELINE config 5 with every tensor sharded ----
    decode_tp = None
    if world > 1 and not args.no_decode and not args.no_strong:
        decode_tp = bench_decode_tp(hq, oracle, torch, ctx, dev, args, rank, world, barrier)

    # ---- e2e leg: host buffers through the public call ----
    pin_x = {key: torch.from_numpy(b.view(np.int16).copy()).pin_memory() for key, b in xbits.items()}
    np_x = {key: t.numpy() for key, t in pin_x.items()}
    if gather is None:
        pin_y = {(n, m): torch.empty((m, n), dtype=torch.float32).pin_memory() for n, _ in SHAPES for m in TOKENS}
        np_y = {key: t.numpy() for key, t in pin_y.items()}

        batch = hq.ops.HostBatch([(np_x[(k, m)], w, np_y[(n, m)], m, hq.ops.DT_BF16)
                                  for m in TOKENS for c in range(args.copies) for (n, k), w in zip(SHAPES, weights[c])])

        def e2e_pass():
            hq.ops.quantized_matmul_host_batch(ctx, batch)
            hq.ops.host_sync(ctx)                    # the pass's results are in pinned host memory from here on
        e2e_api = ("hf2q_cuda_qmatmul_host_batch: one call queues the pass's products (each: pinned host x -> device, kernel, y -> pinned host; the library replays the unchanged batch as one CUDA graph), "
                   "hf2q_cuda_host_sync once per pass")
        d2h = args.copies * sum(4 * m * n for n, _ in SHAPES for m in TOKENS)
    else:
        # the sharded call: every rank copies its activations in, the product gathers, rank 0 (the
        # rank that would hand the result on) copies the full-width output to pinned host memory
        pin_y = {(n, m): torch.empty((m, world * n), dtype=torch.float32).pin_memory() for n, _ in SHAPES for m in TOKENS} if rank == 0 else {}
        np_y = {key: t.numpy() for key, t in pin_y.items()}
        batch = hq.ops.HostBatch([(np_x[(k, m)], w, np_y.get((n, m)), m, hq.ops.DT_BF16)
                                  for m in TOKENS for c in range(args.copies) for (n, k), w in zip(SHAPES, weights[c])])

        def e2e_pass():
            gather.host_batch(batch)
            hq.ops.host_sync(ctx)
        e2e_api = ("hf2q_cuda_qmatmul_gather_host_batch: one call per rank queues the pass's products (each: pinned host x -> device on every rank, "
                   "hf2q_cuda_qmatmul_gather with the all-gather in the kernel, full-width y -> pinned host on rank 0), hf2q_cuda_host_sync once per pass")
        d2h = args.copies * sum(4 * m * n * world for n, _ in SHAPES for m in TOKENS)

    e2e_passes = args.e2e_steps or max(3, min(args.steps, 20))
    for _ in range(3):
        e2e_pass()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_passes):
        e2e_pass()
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        ts = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        e2e_s = float(ts.item())
    ctx.check_status()
    e2e_val = world * bytes_per_pass * e2e_passes / e2e_s / 1e9
    h2d = args.copies * sum(2 * m * k for _, k in SHAPES for m in TOKENS)

    if rank != 0:
        if gather is not None:
            gather.close()
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_hbm_peak()
    ratio = ncu_traffic_per_launch()
    mean_launch_bytes = bytes_per_pass / launches_per_pass
    roofline = {
        "bound": "hbm", "achieved": round(per_gpu, 1), "peak": peak, "unit": "GB/s",
        "frac": round(per_gpu / peak, 4), "peak_source": f"of {peak_kind}",
        "kernel": "gemv_mma_kernel<Q6_K>, m in {1,4,8}",
        "traffic": None if ratio is None else round(ratio * mean_launch_bytes),
        "traffic_source": "dram bytes / algorithmic bytes of the ncu capture summarised in profiles/gemv_q6k_sweep.md (1.0231) x this run's mean launch",
        "algorithmic_bytes_per_launch_mean": round(mean_launch_bytes),
        "frac_of_nominal_8TBps": round(per_gpu / 8000.0, 4),
        "breakdown": breakdown,
    }

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        threads = host_threads()
        cpu_reference_pass(raws, xvals, threads)           # warm
        t, b = cpu_reference_pass(raws, xvals, threads)
        n, k = SHAPES[1]
        _, td, tm = oracle.qmatmul(Q6_K, raws[1], xvals[(k, 1)], n, k, threads=1)
        cpu_baseline = {
            "value": round(b / t / 1e9, 3), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": "one pass over one copy of the four Q6_K matrices x m in {1,4,8}: dequantise to f32 + "
                      "sequential-k f32 matmul, OpenMP over rows on all host threads",
            "single_thread_4096x4096_m1_GBps": round(algo_bytes(n, k, 1, row_b[k]) / (td + tm) / 1e9, 3),
        }

    secondary = None
    if world == 1 and not args.no_secondary:
        del weights, graph
        torch.cuda.empty_cache()
        secondary = {"config1_q4k_f32": bench_config1(hq, oracle, torch, ctx, dev, args),
                     "config3_prefill_gemm": bench_gemm(hq, oracle, torch, ctx, dev, args),
                     "config4_moe_layer": bench_moe(hq, oracle, torch, ctx, dev, args)}
        if not args.no_decode:
            torch.cuda.empty_cache()
            secondary["config5_decode"] = bench_decode(hq, oracle, torch, ctx, dev, args)

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": WORKLOAD,
            "weights": "N(0, sigma=0.02), f16 round trip, Q6_K via the oracle's port of hf2q's quantizer",
            "l2_policy": f"inputs larger than L2: {args.copies} distinct copies of the 4 matrices "
                         f"({working_set / 2**30:.2f} GiB) rotated so no launch re-reads cached weights",
            "step": f"{args.passes} passes over {args.copies} copies x 4 shapes x 3 token counts",
            "launches_per_step": per_step_launches, "bytes_per_step": bytes_per_step,
            "launch_mode": "CUDA graph replay of one captured step" if graph_used else "eager launches",
            "parallelism": "single GPU" if world == 1 else
                           (f"row-sharded x{world}, each rank's shard = the listed shapes; the all-gather of every output is "
                            "in the kernel's epilogue (stores to the peers' buffers over NVLink + per-source arrival counters, two "
                            "alternating output buffers), each product waits for the previous one's columns from all ranks") if gather is not None else
                           f"row-sharded x{world}, each rank's shard = the listed shapes; NCCL all-gather after every product",
            "parity_before_timing": verify,
        },
        "gpu_launches": int(gpu_launches),
        "e2e": {"value": round(e2e_val, 1), "unit": UNIT, "h2d_bytes_per_step": h2d * args.passes, "d2h_bytes_per_step": d2h * args.passes,
                "passes_timed": e2e_passes, "api": e2e_api},
        "roofline": roofline,
        "clocks": clocks,
    }
    if strong is not None:
        line["strong"] = strong
    if moe_ep is not None:
        line.setdefault("secondary", {})["config4_moe_expert_parallel"] = moe_ep
    if decode_tp is not None:
        line.setdefault("secondary", {})["config5_decode_tensor_parallel"] = decode_tp
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    if secondary is not None:
        line["secondary"] = secondary
    print(json.dumps(line))
    if gather is not None:
        gather.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
