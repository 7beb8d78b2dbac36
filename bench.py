#!/usr/bin/env python
"""Benchmark of the quantized-weight mat-vec path (the decode hot path) on B200.

Workload (one GPU): the Q6_K decode GEMV sweep -- weight shapes (out x in) 6144x4096, 4096x4096,
28672x4096 and 4096x14336, N(0, 0.02) weights quantized to Q6_K (210 B per 256 elements) by the
CPU oracle's port of hf2q's quantizer, bf16 N(0,1) activations, batches of 1, 4 and 8 tokens,
fp32 accumulation.  Every matrix is smaller than the 126 MB L2, so the sweep rotates over
`--copies` distinct device copies of the four matrices (>= 1 GiB in total): no launch finds its
weights in L2.  One "step" is one pass over all copies x shapes x token counts.

  metric  = dequant-GEMV HBM GB/s = algorithmic bytes (W + 2*m*K + 4*m*N per launch) / device time
  value   = inputs resident in HBM, launches back to back on one stream, CUDA-event timed
  e2e     = the same sweep through the host-buffer C-ABI call (hf2q_cuda_qmatmul_host_async): every
            call queues the copy of its activations from pinned host memory, the kernel and the copy
            of y back to pinned host memory; one hf2q_cuda_host_sync per step waits for all of them

Multi-GPU (torchrun, one rank per GPU): weak scaling.  Each rank holds the shapes above as ITS row
shard of a matrix G times taller and runs the same sweep; the mat-vec kernel stores its columns into
every rank's full-width output buffer itself (peer memory over NVLink, arrival counters), so a step
contains no collective call and is replayed from a CUDA graph like the single-GPU step.

`--impl reference` times the reference's CPU path for the same products (the oracle's port of
"dequantise to f32, then matmul_a_by_bt") on the host cores, one bounded sample per step.
"""
from __future__ import annotations

import argparse
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


def ncu_traffic_per_launch() -> float | None:
    """Mean DRAM bytes per launch scaled to this sweep, from the committed ncu summary."""
    p = ROOT / "profiles" / "gemv_q6k_traffic.json"
    if not p.exists():
        return None
    try:
        return float(json.loads(p.read_text())["dram_bytes_per_algorithmic_byte"])
    except Exception:
        return None


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


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    threads = oracle.max_threads()
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
        "config": {"workload": "Q6_K decode GEMV sweep, 4 shapes x m in {1,4,8}, bf16 activations"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"per step: the first {row_frac:.4f} of the rows of each of the four Q6_K matrices x "
                                   "m in {1,4,8} (dequantise to f32 + sequential-k f32 matmul, OpenMP over rows)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def measured_tensor_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops_sustained"]), "measured (sustained)"
        except Exception:
            pass
    return 1400.0, "fallback"


def run_secondary(args) -> None:
    """The other two kernels of the path on one GPU, same timing rules, one JSON line each run.

    gemm: BASELINE config 3 -- Q4_K for 6144x4096, 4096x4096, 28672x4096 and Q6_K for the 4096x14336
          down projection, bf16 activations, M in {512, 2048, 4096}; metric = TFLOP/s (2*M*N*K).
    moe:  BASELINE config 4 -- 256 experts, hidden 2048, intermediate 512, top-8, Q5_K; gate, up and
          down mul_mat_id at T in {1, 2048}; metric = layer time and the two rooflines.
    Weights here are random block bytes with finite scales (throughput does not depend on the values;
    parity is what the tests check)."""
    import torch

    import hf2q_b200 as hq
    import oracle

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ctx = hq.GpuContext(0)

    def random_weight(t, rows, k):
        rb = oracle.row_bytes(t, k)
        raw = torch.randint(0, 256, (rows * rb,), dtype=torch.uint8, device=dev)
        be, bb = oracle.block_geometry(t)
        v = raw.view(-1, bb)
        for o in {2: [1], 8: [1], 12: [1, 3], 13: [1, 3], 14: [209]}[t]:       # high byte of each f16 scale
            v[:, o] &= 0x3B                                                     # finite, |d| < 1
        return raw

    def timed(fn, reps):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / reps

    sampler = ClockSampler(0)
    sampler.start()
    l0 = ctx.launch_count
    if args.workload == "gemm":
        cases = [(12, 6144, 4096), (12, 4096, 4096), (12, 28672, 4096), (14, 4096, 14336)]
        toks = [args.tokens] if args.tokens else [512, 2048, 4096]
        rows, flops, secs = {}, 0.0, 0.0
        for (t, n, k) in cases:
            w = hq.load_quant_weight(ctx, random_weight(t, n, k), t, n, k)
            for m in toks:
                x = torch.randn(m, k, device=dev).bfloat16()
                y = torch.empty(m, n, device=dev)
                prm = hq.GgmlQuantizedMatmulParams(m, n, k, t)
                dt = timed(lambda: hq.quantized_matmul_ggml(ctx, x, w, y, prm), max(3, min(args.steps, 20)))
                rows[f"{oracle.TYPE_NAMES[t]}_{n}x{k}_M{m}"] = round(2.0 * m * n * k / dt / 1e12, 1)
                flops += 2.0 * m * n * k
                secs += dt
        peak, kind = measured_tensor_peak()
        val = flops / secs / 1e12
        line = {"metric": "prefill dequant-GEMM TFLOP/s", "value": round(val, 1), "unit": "TFLOP/s", "n_gpus": 1,
                "higher_is_better": True, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                "config": {"workload": "Q4_K_M prefill GEMM sweep (Q4_K x3 shapes, Q6_K 4096x14336), bf16 activations",
                           "tokens": toks, "timing": "CUDA events, activation conversion kernel included"},
                "roofline": {"bound": "tensor", "achieved": round(val, 1), "peak": peak, "unit": "TFLOP/s",
                             "frac": round(val / peak, 4), "peak_source": f"of {kind}", "kernel": "gemm_tc_kernel", "traffic": None},
                "per_case_TFLOPs": rows}
    elif args.workload == "matvec":
        # every block format on the decode shapes: per-launch time from a CUDA graph that walks 8
        # distinct copies of the matrix (so weights come from HBM), bf16 activations
        peak_h, kind_h = measured_hbm_peak()
        shapes = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]
        per, tot_b, tot_s = {}, 0.0, 0.0
        for t in ([int(args.qtype)] if args.qtype else [2, 8, 12, 13, 14]):
            for n, k in shapes:
                ws = [hq.load_quant_weight(ctx, random_weight(t, n, k), t, n, k) for _ in range(8)]
                rb = oracle.row_bytes(t, k)
                for m in (1, 4, 8):
                    x = torch.randn(m, k, device=dev).bfloat16()
                    y = torch.empty(m, n, device=dev)
                    pr = hq.GgmlQuantizedMatmulParams(m, n, k, t)

                    def walk():
                        for w in ws:
                            hq.quantized_matmul_ggml(ctx, x, w, y, pr)

                    for _ in range(3):
                        walk()
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        walk()
                    dt = timed(graph.replay, max(3, min(args.steps, 20))) / len(ws)
                    b = n * rb + 2 * m * k + 4 * m * n
                    per[f"{oracle.TYPE_NAMES[t]}_{n}x{k}_m{m}"] = {"us": round(dt * 1e6, 2), "GBps": round(b / dt / 1e9, 1)}
                    tot_b += b
                    tot_s += dt
                del ws
        val = tot_b / tot_s / 1e9
        line = {"metric": "dequant-GEMV HBM GB/s (all block formats)", "value": round(val, 1), "unit": "GB/s", "n_gpus": 1,
                "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "decode mat-vec, 4 shapes x m in {1,4,8} x block formats, bf16 activations; "
                                       "CUDA graph over 8 copies of each matrix (inputs larger than L2)"},
                "roofline": {"bound": "hbm", "achieved": round(val, 1), "peak": peak_h, "unit": "GB/s", "frac": round(val / peak_h, 4),
                             "peak_source": f"of {kind_h}", "kernel": "gemv_mma_kernel", "traffic": None},
                "per_launch": per}
    else:
        t, E, H, I, topk = 13, 256, 2048, 512, 8
        sg, sd = hq.expert_stride(t, I, H), hq.expert_stride(t, H, I)
        wg, wu, wd = random_weight(t, E * I, H), random_weight(t, E * I, H), random_weight(t, E * H, I)
        res = {}
        for T in ([args.tokens] if args.tokens else [1, 2048]):
            # decode (few tokens) touches 8 experts = 17 MB per layer, far less than L2: rotate over
            # routings that pick different experts so that weights come from HBM; one CUDA graph
            # holds all of them (launch overhead of the Python calls stays out of the timing)
            nsets = 16 if T <= 8 else 1
            x = torch.randn(T, H, device=dev).bfloat16()
            R = T * topk
            g, u = torch.empty(R, I, device=dev), torch.empty(R, I, device=dev)
            d = torch.empty(R, H, device=dev)
            act = torch.randn(R, I, device=dev).bfloat16()
            sc = hq.IdMmScratch.alloc(ctx, E, R, H)
            pg = hq.GgmlQuantizedMatmulIdParams(T, topk, I, H, E, sg, t)
            pd = hq.GgmlQuantizedMatmulIdParams(R, 1, H, I, E, sd, t)
            id_sets = []
            for i in range(nsets):
                if T <= 8:          # disjoint expert groups per set
                    logits = torch.full((T, E), -30.0, device=dev)
                    logits[:, (i * topk * T) % E:(i * topk * T) % E + topk * T] = torch.randn(T, topk * T, device=dev)
                else:
                    logits = torch.randn(T, E, device=dev)
                id_sets.append(hq.moe_softmax_topk(ctx, logits, topk)[0])

            fused = hq.ops.quantized_matmul_id_swiglu_supported(ctx, pg, x.dtype)

            def layer(ids):
                if fused:     # few routed rows: gate, up and the SwiGLU in one launch
                    hq.ops.quantized_matmul_id_swiglu_ggml(ctx, x, wg.data_ptr(), wu.data_ptr(), ids, g, pg)
                else:
                    hq.quantized_matmul_id_pair_ggml(ctx, x, wg.data_ptr(), wu.data_ptr(), ids, g, u, sc, pg)   # gate + up
                # (down reads synthetic activations: products of random block bytes leave the f16 range)
                hq.quantized_matmul_id_ggml(ctx, act, wd.data_ptr(), ids, d, sc, pd)

            def all_sets():
                for ids in id_sets:
                    layer(ids)

            for _ in range(3):
                all_sets()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                all_sets()
            dt = timed(graph.replay, max(3, min(args.steps, 20))) / nsets
            nexp = int(torch.unique(id_sets[0]).numel())
            wbytes = nexp * (2 * sg + sd)
            res[f"T{T}"] = {"us_per_layer": round(dt * 1e6, 1), "TFLOPs": round(2.0 * R * 3 * I * H / dt / 1e12, 2),
                            "weight_GBps": round(wbytes / dt / 1e9, 1), "experts_touched": nexp,
                            "swiglu_in_gate_up_launch": bool(fused),
                            "timing": f"CUDA graph of {nsets} layer(s) with different routings"}
        peak_h, kind_h = measured_hbm_peak()
        last = res[sorted(res)[-1]]
        line = {"metric": "MoE mul_mat_id layer time", "value": last["us_per_layer"], "unit": "us", "n_gpus": 1,
                "higher_is_better": False, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                "config": {"workload": "Qwen3-style A3B expert layer: 256 experts, hidden 2048, intermediate 512, top-8, Q5_K; "
                                       "gate + up + down mul_mat_id (router outputs from the softmax/top-k kernel)"},
                "roofline": {"bound": "hbm", "achieved": last["weight_GBps"], "peak": peak_h, "unit": "GB/s",
                             "frac": round(last["weight_GBps"] / peak_h, 4), "peak_source": f"of {kind_h}",
                             "kernel": "gemm_tc_kernel<grouped> + moe_sort/gather (T=2048), gemv_mma_kernel (T=1)", "traffic": None},
                "per_case": res}
    line["gpu_launches"] = int(ctx.launch_count - l0)
    line["clocks"] = sampler.stop()
    ctx.check_status()
    print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--copies", type=int, default=8, help="distinct device copies of the four matrices")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-buffer leg (0 = auto)")
    ap.add_argument("--no-chain-wait", action="store_true",
                    help="several GPUs: products do not wait for the previous product's columns (analysis aid)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="issue launches eagerly instead of replaying a CUDA graph")
    ap.add_argument("--qtype", default="", help="matvec: one ggml type number (2, 8, 12, 13, 14) instead of all five")
    ap.add_argument("--workload", default="gemv", choices=["gemv", "gemm", "moe", "matvec"],
                    help="gemv: the headline Q6_K decode sweep (default); gemm: Q4_K_M prefill GEMM sweep; "
                         "moe: Qwen3-style A3B expert layer (Q5_K mul_mat_id)")
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

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
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
    # counters, hf2q_b200.dist.GatherGroup); each product waits for the previous one's columns from
    # all ranks before it reads its activations, as a decode chain would.
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

    launches_per_step = args.copies * len(SHAPES) * len(TOKENS)
    bytes_per_step = args.copies * sum(algo_bytes(n, k, m, row_b[k]) for n, k in SHAPES for m in TOKENS)
    working_set = args.copies * sum(len(r) for r in raws)

    def step():
        for m in TOKENS:
            for c in range(args.copies):
                for (n, k), w in zip(SHAPES, weights[c]):
                    if gather is None:
                        hq.quantized_matmul_ggml(ctx, xdev[(k, m)], w, ydev[(n, m)], params[(n, k, m)])
                        if world > 1:
                            dist.all_gather_into_tensor(ygath[(n, m)], ydev[(n, m)])
                    else:
                        gather.matmul(xdev[(k, m)], w, m, rank * n, wait_previous=not args.no_chain_wait)
        if gather is not None:
            gather.wait()           # the step ends when every rank's columns of the last product are here

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- parity spot check before timing (oracle is the checker, never the timed path) ----
    if rank == 0:
        from tests.util import rel_l2
        n, k = SHAPES[1]
        y = ydev[(n, 4)]
        hq.quantized_matmul_ggml(ctx, xdev[(k, 4)], weights[0][1], y, params[(n, k, 4)])
        ctx.check_status()
        wref = oracle.dequantize(Q6_K, raws[1]).reshape(n, k)
        err = rel_l2(y.cpu().numpy(), oracle.matmul_f64(xvals[(k, 4)], wref))
        if not err < 1e-3:
            raise SystemExit(f"parity check failed before timing: rel L2 {err}")

    # Several GPUs: one trial step of the fused form.  A rank whose bounded waits ran out (a peer's
    # columns never arrived) or whose step took implausibly long votes to drop it, and then every rank
    # uses NCCL all-gathers instead: the bench must end either way.
    if gather is not None:
        barrier()
        t_trial = time.perf_counter()
        step()
        torch.cuda.synchronize()
        bad = time.perf_counter() - t_trial > 0.5
        try:
            ctx.check_status()
        except hq.Hf2qError:
            bad = True
        vote = torch.tensor([1.0 if bad else 0.0], device=dev)
        dist.all_reduce(vote, op=dist.ReduceOp.MAX)
        if float(vote.item()) > 0:
            if rank == 0:
                print("[bench] the fused gather did not complete its trial step; using NCCL all-gathers after each product (eager launches)",
                      file=sys.stderr)
            gather.close()
            gather = None
            ygath = {(n, m): torch.empty((world, m, n), dtype=torch.float32, device=dev) for n, _ in SHAPES for m in TOKENS}

    for _ in range(args.warmup):
        step()
    barrier()
    # One step's launches are captured into a CUDA graph and replayed (what a decode loop does); the
    # multi-GPU step contains no collective call (the all-gather is in the kernels), so it is captured
    # the same way.
    graph = None
    if not args.no_graph and (world == 1 or gather is not None):     # NCCL calls are not captured
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step()
            graph = g
            l_per = launches_per_step
        except Exception as exc:      # capture unsupported: fall back to eager launches, say so
            print(f"[bench] graph capture failed ({exc}); timing eager launches", file=sys.stderr)
            graph = None
    run_step = graph.replay if graph is not None else step
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
    gpu_launches = (ctx.launch_count - l0) if graph is None else (launches_per_step + (1 if gather is not None else 0)) * args.steps
    ctx.check_status()
    if world > 1:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    ms_per_step = ms / args.steps
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    per_gpu = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # ---- per-(m) breakdown, kernel only, rank-local (explains the aggregate) ----
    breakdown = {}
    for m in TOKENS:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, min(20, args.steps))
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            for c in range(args.copies):
                for (n, k), w in zip(SHAPES, weights[c]):
                    hq.quantized_matmul_ggml(ctx, xdev[(k, m)], w, ydev[(n, m)], params[(n, k, m)])
        e1.record()
        torch.cuda.synchronize()
        b = args.copies * sum(algo_bytes(n, k, m, row_b[k]) for n, k in SHAPES)
        breakdown[f"m{m}_GBps"] = round(b * reps / (e0.elapsed_time(e1) * 1e-3) / 1e9, 1)

    # ---- e2e leg: host buffers through hf2q_cuda_qmatmul_host ----
    pin_x = {key: torch.from_numpy(b.view(np.int16).copy()).pin_memory() for key, b in xbits.items()}
    pin_y = {(n, m): torch.empty((m, n), dtype=torch.float32).pin_memory() for n, _ in SHAPES for m in TOKENS}
    np_x = {key: t.numpy() for key, t in pin_x.items()}
    np_y = {key: t.numpy() for key, t in pin_y.items()}

    def e2e_step():
        for m in TOKENS:
            for c in range(args.copies):
                for (n, k), w in zip(SHAPES, weights[c]):
                    hq.ops.quantized_matmul_host(ctx, np_x[(k, m)], w, np_y[(n, m)], m, hq.ops.DT_BF16, wait=False)
        hq.ops.host_sync(ctx)                    # the step's results are in pinned host memory from here on

    e2e_steps = args.e2e_steps or max(3, min(args.steps, 30))
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        ts = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        e2e_s = float(ts.item())
    e2e_val = world * bytes_per_step * e2e_steps / e2e_s / 1e9
    h2d = args.copies * sum(2 * m * k for _, k in SHAPES for m in TOKENS)
    d2h = args.copies * sum(4 * m * n for n, _ in SHAPES for m in TOKENS)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_hbm_peak()
    ratio = ncu_traffic_per_launch()
    mean_launch_bytes = bytes_per_step / launches_per_step
    roofline = {
        "bound": "hbm", "achieved": round(per_gpu, 1), "peak": peak, "unit": "GB/s",
        "frac": round(per_gpu / peak, 4), "peak_source": f"of {peak_kind}",
        "kernel": "gemv_mma_kernel<Q6_K>, m in {1,4,8}",
        "traffic": None if ratio is None else round(ratio * mean_launch_bytes),
        "algorithmic_bytes_per_launch_mean": round(mean_launch_bytes),
        "frac_of_nominal_8TBps": round(per_gpu / 8000.0, 4),
        "breakdown": breakdown,
    }

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        threads = oracle.max_threads()
        cpu_reference_pass(raws, xvals, threads)           # warm
        t, b = cpu_reference_pass(raws, xvals, threads)
        t1, b1 = 0.0, 0
        n, k = SHAPES[1]
        _, td, tm = oracle.qmatmul(Q6_K, raws[1], xvals[(k, 1)], n, k, threads=1)
        cpu_baseline = {
            "value": round(b / t / 1e9, 3), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": "one pass over one copy of the four Q6_K matrices x m in {1,4,8}: dequantise to f32 + "
                      "sequential-k f32 matmul, OpenMP over rows on all host threads",
            "single_thread_4096x4096_m1_GBps": round(algo_bytes(n, k, 1, row_b[k]) / (td + tm) / 1e9, 3),
        }

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": "Q6_K decode GEMV sweep: shapes 6144x4096, 4096x4096, 28672x4096, 4096x14336; "
                        "m in {1,4,8}; bf16 activations; fp32 accumulate",
            "weights": "N(0, sigma=0.02), f16 round trip, Q6_K via the oracle's port of hf2q's quantizer",
            "l2_policy": f"inputs larger than L2: {args.copies} distinct copies of the 4 matrices "
                         f"({working_set / 2**30:.2f} GiB) rotated so no launch re-reads cached weights",
            "launches_per_step": launches_per_step, "bytes_per_step": bytes_per_step,
            "launch_mode": "CUDA graph replay of one captured step" if graph is not None else "eager launches",
            "parallelism": "single GPU" if world == 1 else
                           (f"row-sharded x{world}, each rank's shard = the listed shapes; the all-gather of every output is "
                            "in the kernel's epilogue (stores to the peers' buffers over NVLink + arrival counters), each "
                            "product waits for the previous one's columns from all ranks") if gather is not None else
                           f"row-sharded x{world}, each rank's shard = the listed shapes; NCCL all-gather after every product",
        },
        "gpu_launches": int(gpu_launches),
        "e2e": {"value": round(e2e_val, 1), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "api": "hf2q_cuda_qmatmul_host_async per product (pinned host x -> device, kernel, y -> pinned host), hf2q_cuda_host_sync once per step"},
        "roofline": roofline,
        "clocks": clocks,
    }
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
