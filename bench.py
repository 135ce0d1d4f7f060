#!/usr/bin/env python3
"""Benchmark of the split W4A4 + tail linear on the Qwen3-8B decoder-layer shapes at prefill.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): the four linears of one Qwen3-8B decoder layer at M = 2048 tokens per GPU and
tail ratio 0.05 -- qkv_proj 4096->6144 (one fused GEMM), o_proj 4096->4096, gate_up 4096->2x12288 (one
shared prologue, one GEMM), down_proj 12288->4096 (12 (x) 1024 Hadamard) -- each as prologue + tail
gather + tcgen05 GEMM with fused dequant.  Synthetic, seeded inputs: activations N(0,1) with 16 channels
x50, weights N(0, 0.02).  With N GPUs every rank runs the same step on its own 2048 rows (token-row
sharding, replicated weights, no collective): weak scaling.

The printed JSON line carries the whole-job throughput (`value`, TOPS = 2*M*N*K summed over the four
linears and all ranks / time), the same metric through the public API with host buffers (`e2e`), the
roofline of the dense GEMM kernel, the per-kernel breakdown and a CPU baseline (the numpy oracle timed on a
bounded sample).  `--impl reference` times only that CPU oracle.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYER = [  # name, K, N
    ("qkv_proj", 4096, 6144),
    ("o_proj", 4096, 4096),
    ("gate_up_proj", 4096, 24576),
    ("down_proj", 12288, 4096),
]
M_TOKENS = 2048
RATIO = 0.05
CPU_SAMPLE_ROWS = 256
METRIC = "split W4A4+tail linear TOPS, Qwen3-8B layer shapes, prefill M=2048/GPU, ratio 0.05"
NOMINAL_INT8_TOPS = 4500.0


def measured_dram_traffic(kernel: str):
    """dram__bytes_read.sum + dram__bytes_write.sum of one step's launches of `kernel`, from the table that is kept
    beside the profile summaries and rewritten whenever the kernel is captured again (None when it has no entry)."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            e = json.load(f).get(kernel)
        return int(e["bytes_per_step"]) if e else None
    except Exception:
        return None


def layer_ops(m: int) -> float:
    return float(sum(2.0 * m * n * k for _, k, n in LAYER))


def ops_step_of(m: int) -> float:
    return layer_ops(m)


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16": float(d["bf16_tflops"]),
                "bf16_sustained": float(d["bf16_tflops_sustained"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------- CPU oracle arm
def cpu_oracle_setup():
    from oracle import oracle as O
    ws = []
    for i, (name, K, N) in enumerate(LAYER):
        kind = O.HAD_KRON12 if K == 12288 else O.HAD_WHT
        w = O.prepare_weight(O.make_weights(N, K, seed=100 + i), kind)
        x = O.make_activations(CPU_SAMPLE_ROWS, K, seed=200 + i, n_outlier=16)
        ws.append((kind, O.ceil_ratio_count(K, RATIO), w, x))
    return O, ws


def cpu_oracle_step(O, ws):
    for kind, R, w, x in ws:
        O.split_linear_t16(x, w, kind, R)


def use_all_host_threads() -> int:
    """Gives the BLAS under numpy every core of the box and says how many it got.  A launcher (torchrun) exports
    OMP_NUM_THREADS=1 to its workers, so the count is set explicitly: in the environment when numpy is not loaded
    yet, through threadpoolctl in any case."""
    n = os.cpu_count() or 1
    if "numpy" not in sys.modules:
        for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
            os.environ[var] = str(n)
    try:
        import numpy  # noqa: F401
        from threadpoolctl import threadpool_info, threadpool_limits
        threadpool_limits(limits=n)
        got = max([int(p.get("num_threads", 1)) for p in threadpool_info()] or [1])
        return max(got, 1)
    except Exception:
        return n


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = use_all_host_threads()
    O, ws = cpu_oracle_setup()
    for _ in range(args.warmup):
        cpu_oracle_step(O, ws)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_oracle_step(O, ws)
    dt = time.perf_counter() - t0
    ms = dt * 1e3 / max(args.steps, 1)
    tops = layer_ops(CPU_SAMPLE_ROWS) / (ms * 1e-3) / 1e12
    sample = (f"numpy restatement of the path (oracle/oracle.py), online part only, all four linears of the layer on "
              f"{CPU_SAMPLE_ROWS} of the 2048 rows per step")
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4 x int4 -> int32, fp32 dequant, bf16 out",
        "data": "synthetic",
        "config": {"workload": "Qwen3-8B decoder layer linears: qkv 4096->6144, o 4096->4096, gate_up 4096->24576, "
                               "down 12288->4096 (BASELINE configs[1])",
                   "rows_per_step": CPU_SAMPLE_ROWS, "rows_of_the_gpu_arm": M_TOKENS, "tail_ratio": RATIO,
                   "same_config": CPU_SAMPLE_ROWS == M_TOKENS,
                   "note": "a bounded sample of the rows; throughput (TOPS) is per row and comparable, ms_per_step is not"},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Reads SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.power_w, self.capped = [], 0
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                self.capped += 1 if mask & getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4) else 0
                self.power_w.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._loop, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t is not None:
            self._t.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}

    def power_summary(self):
        p = sorted(self.power_w)
        return {"power_w": p[len(p) // 2] if p else None,
                "sw_power_cap_fraction": (self.capped / len(self.samples)) if self.samples else None}


# --------------------------------------------------------------------------------------- GPU arm
def run_ours(args) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist
    from tailquant_kernel_b200 import SplitLinear, ops
    from tailquant_kernel_b200._lib import TQ_HAD_KRON12, TQ_HAD_WHT

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- prepared weights (replicated) and this rank's token rows
    gen = torch.Generator(device="cpu")
    lins, xs, host_x, host_y = [], [], [], []
    for i, (name, K, N) in enumerate(LAYER):
        gen.manual_seed(100 + i)
        W = (torch.randn((N, K), generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16).to(dev)
        lin = SplitLinear(W, ratio=RATIO, had_kind=TQ_HAD_KRON12 if K == 12288 else TQ_HAD_WHT,
                          tail_engine=args.tail_engine)
        del W
        gen.manual_seed(1000 * (rank + 1) + i)
        x = torch.randn((M_TOKENS, K), generator=gen, dtype=torch.float32)
        ch = torch.randperm(K, generator=gen)[:16]
        x[:, ch] *= 50.0
        hx = x.to(torch.bfloat16).pin_memory()
        lins.append(lin)
        host_x.append(hx)
        xs.append(hx.to(dev))
        host_y.append(torch.empty((M_TOKENS, N), dtype=torch.bfloat16).pin_memory())
    dev_x = [torch.empty_like(x) for x in xs]
    torch.cuda.synchronize()

    def step():
        for lin, x in zip(lins, xs):
            lin.forward(x)

    # End to end through the public API with HOST buffers: the four linears have independent inputs, so the
    # host->device copy of linear i+1 and the device->host copy of linear i-1 run on their own streams (the two
    # copy engines work in both directions at once) while linear i computes.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in lins]
    ev_done = [torch.cuda.Event() for _ in lins]
    ev_free = [torch.cuda.Event() for _ in lins]
    dev_y = [torch.empty((M_TOKENS, lin.N), dtype=torch.bfloat16, device=dev) for lin in lins]

    def step_e2e():
        # Steps are pipelined the way a serving loop would run them: the copy-in of step n + 1 starts as soon as
        # linear i of step n has consumed its input buffer, and the copy-out of step n drains while step n + 1
        # computes.  Every step still moves all of its inputs host -> device and all of its outputs device -> host.
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(s_in):
            for i, (hx, dx) in enumerate(zip(host_x, dev_x)):
                s_in.wait_event(ev_done[i])  # the previous step's linear i has read dx
                dx.copy_(hx, non_blocking=True)
                ev_in[i].record(s_in)
        for i, (lin, dx) in enumerate(zip(lins, dev_x)):
            cur.wait_event(ev_in[i])
            cur.wait_event(ev_free[i])      # the previous step's copy-out of this buffer has finished
            dev_y[i].copy_(lin.forward(dx))  # out of the layer's workspace, which the next forward reuses
            ev_done[i].record(cur)
        with torch.cuda.stream(s_out):
            for i, hy in enumerate(host_y):
                s_out.wait_event(ev_done[i])
                hy.copy_(dev_y[i], non_blocking=True)
                ev_free[i].record(s_out)

    def drain_e2e():
        cur = torch.cuda.current_stream()
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    def timed(fn, steps, warmup, sample_clocks=False, drain=None):
        for _ in range(warmup):
            fn()
        if drain:
            drain()
        barrier()
        sampler = ClockSampler(local) if sample_clocks else None
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if drain:
            drain()  # the stop event waits for the copy streams: the last step's outputs are in host memory
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sampler else None
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, clocks

    ms_step, clocks = timed(step, args.steps, args.warmup, sample_clocks=True)
    ms_e2e, _ = timed(step_e2e, args.steps, max(args.warmup, 3), drain=drain_e2e)
    assert ops.gemm_status() == 0, "a bounded device-side wait ran out during the benchmark"

    # ---- per-kernel device time over the same four linears (CUDA events on the launching stream)
    def kernel_ms(fn, reps=10):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    wss = [lin.workspace(M_TOKENS) for lin in lins]
    mma = args.tail_engine == "mma"

    def pro_call(lin, x, ws):
        return lambda: ops.split_prologue(x, lin.w.had_kind, lin.R, lin.descending_rank, out=ws.pro)

    def tail_call(lin, ws):
        return lambda: ops.tail_gather(ws.pro.tail_idx, ws.pro.tail_val, lin.w.w_t, ws.tail, lin.R)

    def gemm_call(lin, ws):
        if mma:
            return lambda: ops.split_gemm_mma(ws.pro.a_q8, ws.pro.body_scale, lin.w.b_col, lin.w.w_scale, ws.out,
                                              w_rot=lin.w.w_rot, pro=ws.pro, R=lin.R)
        return lambda: ops.split_gemm_fused(ws.pro.a_pack, ws.pro.body_scale, lin.w.b_col, lin.w.w_scale, ws.out,
                                            tail=ws.tail)

    def run_all(calls):
        def f():
            for c in calls:
                c()
        return f

    t_pro = kernel_ms(run_all([pro_call(l, x, w) for l, x, w in zip(lins, xs, wss)]))
    t_gemm = kernel_ms(run_all([gemm_call(l, w) for l, w in zip(lins, wss)]))
    t_tail = 0.0 if mma else kernel_ms(run_all([tail_call(l, w) for l, w in zip(lins, wss)]))
    per_linear = {}
    for (name, K, N), lin, x, ws in zip(LAYER, lins, xs, wss):
        g = kernel_ms(gemm_call(lin, ws))
        pr = kernel_ms(pro_call(lin, x, ws))
        per_linear[name] = {"gemm_ms": g, "prologue_ms": pr, "gemm_tops": 2.0 * M_TOKENS * N * K / (g * 1e-3) / 1e12}
        if not mma:
            tl = kernel_ms(tail_call(lin, ws))
            per_linear[name].update({"tail_ms": tl, "tail_gflops": 2.0 * M_TOKENS * lin.R * N / (tl * 1e-3) / 1e9})

    # comparison lines on the same shapes: unfused bf16 cuBLAS linear (the baseline's GPU comparison) and
    # int8 cuBLAS (torch._int_mm), the best dense INT8 rate a library reaches on this box
    bf16_ms, int8_ms = 0.0, 0.0
    for (name, K, N), x in zip(LAYER, xs):
        Wb = torch.randn((N, K), device=dev, dtype=torch.bfloat16) * 0.02
        bf16_ms += kernel_ms(lambda: torch.nn.functional.linear(x, Wb))
        del Wb
        a8 = torch.randint(-8, 8, (M_TOKENS, K), dtype=torch.int8, device=dev)
        b8 = torch.randint(-8, 8, (N, K), dtype=torch.int8, device=dev).t()
        int8_ms += kernel_ms(lambda: torch._int_mm(a8, b8))
        del a8, b8

    # Layer latency the way the reference times its layers (CUDA graph, warm-ups, >= 30 replays; median of 5 runs):
    # tools/bench_hadamard_three_schemes_quarot_dense_sharedqkv_inplace_fusedtopr_v43.py:105-123
    def graph_median_ms(fn, replays=30, runs=5):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
        out = []
        for _ in range(runs):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(replays):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            out.append(e0.elapsed_time(e1) / replays)
        return sorted(out)[len(out) // 2]

    Wbs = [torch.randn((N, K), device=dev, dtype=torch.bfloat16) * 0.02 for (_, K, N) in LAYER]

    def step_bf16():
        for x, Wb in zip(xs, Wbs):
            torch.nn.functional.linear(x, Wb)

    graph_split_ms = graph_median_ms(step)
    graph_bf16_ms = graph_median_ms(step_bf16)

    # ---- the same layer graphs replayed for about two seconds each: what the board sustains under its power cap
    # (the timed region above is some tens of milliseconds at burst clocks)
    def sustained(fn, burst_ms, seconds=2.0):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        n = max(50, int(seconds / (burst_ms * 1e-3)))
        sampler = ClockSampler(local)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler.start()
        e0.record()
        for _ in range(n):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        clk = sampler.stop()
        out = {"layer_ms": e0.elapsed_time(e1) / n, "replays": n, "sm_mhz": clk["sm_mhz"]}
        out.update(sampler.power_summary())
        return out

    sustained_split = sustained(step, graph_split_ms, args.sustained_seconds) if args.sustained_seconds > 0 else None
    sustained_bf16 = sustained(step_bf16, graph_bf16_ms, args.sustained_seconds) if args.sustained_seconds > 0 else None
    del Wbs

    # ---- plain pinned copies of one step's inputs and outputs, no compute: the ceiling of the end-to-end figure
    def copy_only():
        with torch.cuda.stream(s_in):
            for hx, dx in zip(host_x, dev_x):
                dx.copy_(hx, non_blocking=True)
        with torch.cuda.stream(s_out):
            for hy, dy in zip(host_y, dev_y):
                hy.copy_(dy, non_blocking=True)

    ms_copy, _ = timed(copy_only, max(args.steps // 2, 3), 3, drain=drain_e2e)

    # ---- N > 1: the same 2048 rows cut over the ranks (strong scaling), and the column-parallel gate_up
    strong, colpar = None, None
    if world > 1:
        rows = M_TOKENS // world
        xs_s = [x[rank * rows:(rank + 1) * rows].contiguous() for x in xs]

        def step_strong():
            for lin, x in zip(lins, xs_s):
                lin.forward(x)

        ms_strong, _ = timed(step_strong, args.steps, args.warmup)
        strong = {"rows_per_gpu": rows, "ms_per_step": ms_strong, "tops": ops_step_of(M_TOKENS) / (ms_strong * 1e-3) / 1e12,
                  "speedup_over_one_gpu": ms_step / ms_strong, "efficiency": ms_step / ms_strong / world,
                  "note": "M = 2048 rows of the layer cut into contiguous slabs, one per GPU, no collective; one GPU's "
                          "time for all 2048 rows is this run's ms_per_step.  A 256-row slab is a single row of "
                          "256 x 256 tiles: 16 to 96 tiles for 74 CTA pairs, so most of the GPU idles at N = 8"}
        from tailquant_kernel_b200 import shard
        name, Kg, Ng = LAYER[2]
        gen.manual_seed(100 + 2)
        Wg = (torch.randn((Ng, Kg), generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16).to(dev)
        cp = shard.ColumnParallelSplitLinear(Wg, rank, world, ratio=RATIO, had_kind=TQ_HAD_WHT)
        del Wg
        xg = xs[2] if rank == 0 else torch.empty_like(xs[2])
        dist.broadcast(xg, 0)  # column parallelism works on the SAME rows on every rank
        y_cp = cp.forward(xg)
        y_full = lins[2].forward(xg)
        cp_equal = bool(torch.equal(y_cp, y_full))
        ms_cp, _ = timed(lambda: cp.forward(xg), args.steps, args.warmup)
        ms_cp_gemm, _ = timed(lambda: cp.local.forward(xg), args.steps, args.warmup)
        ms_row, _ = timed(lambda: lins[2].forward(xs_s[2]), args.steps, args.warmup)
        ms_one, _ = timed(lambda: lins[2].forward(xs[2]), args.steps, args.warmup)
        colpar = {"linear": name, "rows": M_TOKENS, "columns_per_gpu": Ng // world,
                  "ms_linear_plus_all_gather": ms_cp, "ms_linear_only": ms_cp_gemm,
                  "ms_all_gather": ms_cp - ms_cp_gemm, "gathered_bytes_per_gpu": 2 * M_TOKENS * (Ng - Ng // world),
                  "ms_row_sharded_same_work": ms_row, "ms_one_gpu": ms_one, "equals_unsplit_layer": cp_equal,
                  "note": "gate_up cut over output channels, one NCCL all_gather_into_tensor of the bf16 slabs over NVLink; "
                          "the row shard needs no exchange at all and is the default"}

    peaks = load_peaks()
    ops_step = layer_ops(M_TOKENS)
    # no INT8 peak was measured: twice the bf16 matmul figure -- the burst one, because the roofline entry times its
    # kernel in isolation (ten launches, a few milliseconds: the clocks stay at their maximum, see `clocks`)
    int8_peak = 2.0 * peaks["bf16"]
    gemm_tops = ops_step / (t_gemm * 1e-3) / 1e12
    pro_bytes = sum(M_TOKENS * (2 * K + (K if mma else K // 2) + 4 * lin.R + 4) for (_, K, _), lin in zip(LAYER, lins))
    pro_gbs = pro_bytes / (t_pro * 1e-3) / 1e9
    tail_flops = sum(2.0 * M_TOKENS * lin.R * N for (_, K, N), lin in zip(LAYER, lins))
    # tensor-pipe time the kernel's MMAs need at the measured library rates: the int8 product, plus (tensor-core
    # tail) a dense bf16 product of the same shape over the zero-filled tail matrix
    pipe_ms = ops_step / (int8_peak * 1e12) * 1e3 + (ops_step / (peaks["bf16"] * 1e12) * 1e3 if mma else 0.0)
    t_sum = t_gemm + t_tail + t_pro

    h2d = sum(int(h.numel() * h.element_size()) for h in host_x)
    d2h = sum(int(h.numel() * h.element_size()) for h in host_y)
    # The dominant kernel: with the tensor-core tail all four projections of the layer run on CTA pairs
    # (pair_gemm_kernel: each has more than 74 one-CTA tiles); the roofline entry sums its four launches of a step.
    if mma:
        dom = [n for (n, K, N) in LAYER]
        kname = ("pair_gemm_kernel (tcgen05 cta_group::2: kind::i8 dense + kind::f16 tail, fused dequant); launches: "
                 + ", ".join(dom))
    else:
        dom = [n for (n, K, N) in LAYER]
        kname = "gemm_kernel<256> (tcgen05 kind::i8, fused dequant + tail add)"
    dom_ms = sum(per_linear[n]["gemm_ms"] for n in dom)
    dom_ops = sum(2.0 * M_TOKENS * N * K for (n, K, N) in LAYER if n in dom)
    dom_tops = dom_ops / (dom_ms * 1e-3) / 1e12
    line = {
        "metric": METRIC,
        "value": ops_step * world / (ms_step * 1e-3) / 1e12,
        "unit": "TOPS",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "int4 x int4 -> int32 (tcgen05 kind::i8), bf16 tail, fp32 dequant, bf16 out",
        "data": "synthetic",
        "config": {"workload": "Qwen3-8B decoder layer linears: qkv 4096->6144, o 4096->4096, gate_up 4096->24576, "
                               "down 12288->4096 (BASELINE configs[1])",
                   "rows_per_gpu": M_TOKENS, "global_rows": M_TOKENS * world, "tail_ratio": RATIO,
                   "tail_engine": args.tail_engine,
                   "parallelism": f"token-row shard x{world}, replicated weights, no collective",
                   "l2": "per-step working set (96 MB int4 + 386 MB bf16 weights, 260 MB activations/outputs) exceeds the 126 MB L2"},
        "e2e": {"value": ops_step * world / (ms_e2e * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "copy_only_ms_per_step": ms_copy,
                "copy_only_gbs_all_gpus": (h2d + d2h) * world / (ms_copy * 1e-3) / 1e9,
                "note": "copy_only = the same pinned host<->device copies of one step with no compute between them "
                        "(both directions at once, all ranks together): the ceiling the end-to-end figure sits under"},
        "gpu_launches": (8 if mma else 12) * args.steps,
        "clocks": clocks,
        "roofline": {"kernel": kname, "bound": "tensor",
                     "achieved": dom_tops, "peak": int8_peak, "unit": "TFLOP/s", "frac": dom_tops / int8_peak,
                     "ms_per_step_in_kernel": dom_ms,
                     "traffic": measured_dram_traffic("pair_gemm_kernel") if mma else None,
                     "peak_note": f"2 x burst bf16 cuBLAS figure ({peaks['source']}; the kernel is timed alone); nominal dense INT8 {NOMINAL_INT8_TOPS}; "
                                  "achieved counts the algorithmic 2*M*N*K of the INT4 product only",
                     "frac_of_nominal_int8": dom_tops / NOMINAL_INT8_TOPS,
                     "all_gemm_launches_tops": gemm_tops,
                     "tensor_pipe_ms_at_library_rates": pipe_ms, "frac_of_library_rate_pipe_time": pipe_ms / t_gemm,
                     "int8_cublas_same_shapes_tops": ops_step / (int8_ms * 1e-3) / 1e12},
        "kernels": {
            "gemm": {"ms_per_step": t_gemm, "share": t_gemm / t_sum, "tops": gemm_tops},
            "prologue": {"ms_per_step": t_pro, "share": t_pro / t_sum, "bound": "hbm",
                         "achieved_gbs": pro_gbs, "peak_gbs": peaks["hbm_gbs"], "frac": pro_gbs / peaks["hbm_gbs"]},
            "per_linear": per_linear,
        },
        "bf16_cublas_linear_ms_per_step": bf16_ms,
        "int8_cublas_gemm_ms_per_step": int8_ms,
        "split_over_bf16": ms_step / bf16_ms,
        "sustained": None if sustained_split is None else {
            "split": sustained_split, "bf16_cublas": sustained_bf16,
            "split_over_bf16": sustained_split["layer_ms"] / sustained_bf16["layer_ms"],
            "tops": ops_step_of(M_TOKENS) / (sustained_split["layer_ms"] * 1e-3) / 1e12,
            "protocol": "the layer's CUDA graph replayed for about 2 s; clocks and power are NVML medians over that time"},
        "graph_latency": {"split_layer_ms": graph_split_ms, "bf16_cublas_layer_ms": graph_bf16_ms,
                          "split_over_bf16": graph_split_ms / graph_bf16_ms,
                          "protocol": "one CUDA graph per layer (4 linears), 5 warm-ups, 30 replays, median of 5 runs"},
    }
    if strong is not None:
        line["strong"] = strong
        line["column_parallel"] = colpar
    if not mma:
        line["kernels"]["tail_gather"] = {"ms_per_step": t_tail, "share": t_tail / t_sum,
                                          "gflops": tail_flops / (t_tail * 1e-3) / 1e9,
                                          "bound": "CUDA-core fma + shared-memory gathers"}

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = use_all_host_threads()
        O, ws = cpu_oracle_setup()
        cpu_oracle_step(O, ws)
        t0 = time.perf_counter()
        reps = 2
        for _ in range(reps):
            cpu_oracle_step(O, ws)
        dt = (time.perf_counter() - t0) / reps
        # ---- one sampled row per 1024 and 256 output channels of every linear against the oracle (as the checker)
        import numpy as np
        worst, frac = 0.0, 0.0
        for i, ((name, K, N), lin) in enumerate(zip(LAYER, lins)):
            rows_s = np.array([0, M_TOKENS // 2 - 1, M_TOKENS - 1])
            chan = np.concatenate([np.arange(0, 128), np.arange(N - 128, N)])
            gen.manual_seed(100 + i)
            Wc = (torch.randn((N, K), generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            wb = Wc[torch.from_numpy(chan)].contiguous().view(torch.int16).numpy().view(np.uint16)
            del Wc
            xb = host_x[i][torch.from_numpy(rows_s)].contiguous().view(torch.int16).numpy().view(np.uint16)
            kind = O.HAD_KRON12 if K == 12288 else O.HAD_WHT
            y_ref, y32, _, _ = O.split_linear_t16(xb, O.prepare_weight(wb, kind), kind, lin.R)
            y = lin.forward(xs[i])[torch.from_numpy(rows_s).to(dev)][:, torch.from_numpy(chan).to(dev)]
            got = O.bf16_bits_to_f32(y.contiguous().view(torch.int16).cpu().numpy().view(np.uint16))
            err = np.abs(got.astype(np.float64) - y32.astype(np.float64))
            half_ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(y32), 1e-30))) - 8)
            assert bool(np.all(err <= np.maximum(2e-2, half_ulp * (1 + 1e-6) + 1e-3))), f"parity: {name} leaves the output bounds"
            assert err.sum() / np.abs(y32).sum() <= 1e-2, f"parity: {name} mean relative error"
            worst = max(worst, float(err.max()))
            frac = max(frac, float((O.f32_to_bf16_bits(got) != y_ref).mean()))
        line["parity_checked"] = True
        line["parity"] = {"rows_per_linear": 3, "channels_per_linear": 256, "max_abs_err_vs_fp32_oracle": worst,
                          "worst_fraction_not_equal_to_bf16_of_oracle": frac,
                          "bounds": "max-abs <= max(2e-2, half an output ulp), mean-rel <= 1e-2"}
        line["cpu_baseline"] = {
            "value": layer_ops(CPU_SAMPLE_ROWS) / dt / 1e12, "unit": "TOPS", "cores": cores, "kind": "port",
            "sample": f"numpy oracle, online path of all four linears on {CPU_SAMPLE_ROWS} of the 2048 rows, mean of {reps} passes"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------- other baseline configs
def run_extra(args) -> None:
    """Secondary workloads of the baseline (one JSON line per case, device time by CUDA events):
    decode      : Qwen3-8B layer shapes at M in {1, 8, 32, 64}, split-K path, int4-weight GB/s against HBM peak
    llama_sweep : Llama-3-8B layer shapes at M = 4096, ratios 0 / 0.01 / 0.05 / 0.10 (K = 14336 uses block-128)
    prefill36   : baseline config 3 (Qwen3-8B, 36 layers, seq 4096, random init): whole-prefill latency with all linears on
                  the split path and bf16 attention
    single      : baseline config 1 (M = 512, K = N = 4096, ratio 0.05), both tail engines
    latency_table : CSV `K,N,ratio,b16,b64,b256` (ms per forward at 16 / 64 / 256 token rows, CUDA-graph replay) in
                  the format the reference's policy calibrator reads
                  (tools/calibrate_shape_latency_cegrad_ratio_v1.py:365-440), Qwen3-8B per-projection shapes
    probe       : a few untimed launches of ONE kernel of ONE linear of the layer (`--only`, `--probe prologue|gemm`,
                  `--ratio`, `--steps` launches at `--rows-per-gpu` rows): a small target for a profiler capture"""
    import torch
    from tailquant_kernel_b200 import SplitLinear

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    peaks = load_peaks()

    def ms_of(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    def graph_ms_of(fn, reps=50):
        """Device time of fn replayed from a CUDA graph (host launch cost excluded), as the reference times
        its layers (tools/bench_hadamard_three_schemes_quarot_dense_sharedqkv_inplace_fusedtopr_v43.py:105-123)."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        return ms_of(graph.replay, reps)

    def data(M, K, N, seed):
        g = torch.Generator(device="cpu")
        g.manual_seed(seed)
        W = (torch.randn((N, K), generator=g) * 0.02).to(torch.bfloat16).to(dev)
        x = torch.randn((M, K), generator=g)
        x[:, torch.randperm(K, generator=g)[: max(16, K // 100)]] *= 50.0
        return x.to(torch.bfloat16).to(dev), W

    if args.workload == "probe":
        from tailquant_kernel_b200 import ops as _ops
        from tailquant_kernel_b200._lib import TQ_HAD_KRON12, TQ_HAD_WHT
        name, K, N = next((l for l in LAYER if l[0] == (args.only or "o_proj")))
        M = args.rows_per_gpu
        _ops.set_prologue_mode(args.prologue_mode)
        x, W = data(M, K, N, 7)
        lin = SplitLinear(W, ratio=args.ratio, had_kind=TQ_HAD_KRON12 if K == 12288 else TQ_HAD_WHT)
        del W
        ws = lin.prologue(x)
        for _ in range(max(1, args.steps)):
            if args.probe == "prologue":
                lin.prologue(x)
            else:
                lin.compute(ws, M)
        torch.cuda.synchronize()
        print(json.dumps({"workload": "probe", "linear": name, "M": M, "K": K, "N": N, "R": lin.R, "kernel": args.probe,
                          "launches": max(1, args.steps)}), flush=True)
    elif args.workload == "decode":
        for name, K, N in LAYER:
            if args.only and name != args.only:
                continue
            _, W = data(1, K, N, 7)
            lin = SplitLinear(W, ratio=RATIO, tail_engine="gather")
            n_copies = max(2, int((300 * 2 ** 20) // (K * N // 2)) + 1)
            b_copies = [lin.w.b_col] + [lin.w.b_col.clone() for _ in range(n_copies - 1)]
            for M in (1, 8, 32, 64):
                x, _ = data(M, K, N, 11 + M)
                ws = lin.prologue(x)
                from tailquant_kernel_b200 import ops as _ops
                t_all = graph_ms_of(lambda: lin.forward(x))
                # the weight stream is timed with the packed weights rotating through > 300 MB of copies inside
                # one graph, so that every launch reads them from HBM and not from the 126 MB L2
                tc = lin._decode_uses_tc(M)  # the layer's dispatch of the dense part
                part = torch.empty((_ops.gemv_plan(M, N, K), M, N), dtype=torch.int32, device=dev)

                def all_copies():
                    for b in b_copies:
                        if tc:
                            _ops.matmul_splitk(ws.pro.a_pack, b, part[0], lin._pick_split_k(M))
                        else:
                            _ops.gemv_partials(ws.pro.a_pack, b, part)
                t_gemm = graph_ms_of(all_copies) / len(b_copies)
                t_pro = graph_ms_of(lambda: lin.prologue(x))
                t_tail = graph_ms_of(lambda: _ops.tail_gather_small(ws.pro.tail_idx, ws.pro.tail_val, lin.w.w_t, ws.tail, lin.R))
                wbytes = K * N / 2
                print(json.dumps({"workload": "decode", "linear": name, "M": M, "K": K, "N": N, "R": lin.R,
                                  "linear_ms": t_all, "splitk_gemm_ms": t_gemm,
                                  "dense_kernel": "tcgen05 split-K GEMM (int32 atomics)" if tc else "weight-streaming GEMV (mma.sync s8), partial sums per K range",
                                  "prologue_ms": t_pro, "tail_gather_ms": t_tail,
                                  "timing": "CUDA graph replay; splitk_gemm_ms = mean launch of the partial-sum GEMV over %d weight copies "
                                            "(HBM-resident), the other figures with L2-warm operands" % len(b_copies),
                                  "int4_weight_gbs": wbytes / (t_gemm * 1e-3) / 1e9,
                                  "frac_of_hbm_peak": wbytes / (t_gemm * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                  "tail_row_bytes": 2.0 * M * lin.R * N}), flush=True)
            del b_copies
    elif args.workload == "latency_table":
        # the seven per-projection shapes of a Qwen3-8B layer (the policy's units), ratios of the policy grid
        shapes = [(4096, 4096), (4096, 1024), (4096, 12288), (12288, 4096)]
        print("K,N,ratio,b16,b64,b256", flush=True)
        for K, N in shapes:
            _, W = data(1, K, N, 21)
            for ratio in (0.0, 0.01, 0.02, 0.05, 0.10, 0.16):
                lin = SplitLinear(W, ratio=ratio)
                cols = []
                for M in (16, 64, 256):
                    x, _ = data(M, K, N, 31 + M)
                    cols.append(graph_ms_of(lambda: lin.forward(x)))
                print(f"{K},{N},{ratio},{cols[0]:.5f},{cols[1]:.5f},{cols[2]:.5f}", flush=True)
                del lin
    elif args.workload == "prefill36":
        # Baseline config 3: Qwen3-8B, 36 decoder layers, random init, `--batch` sequences of `--seq-len` tokens, every
        # linear of a layer on the split W4A4 + tail path at ratio 0.05 (qkv and gate_up as fused projections, input /
        # post-attention RMSNorm folded into their prologues, SwiGLU folded into the gate_up epilogue), attention in
        # bf16 (torch SDPA).  Under torchrun the batch is cut into whole sequences per rank (no communication: the
        # linears are row-independent and attention stays inside a sequence), weights replicated.  Whole-prefill
        # latency by CUDA events, max over ranks; `--check` compares every linear of layer 0 with the CPU oracle.
        import torch.distributed as dist
        import torch.nn.functional as F
        from tailquant_kernel_b200 import interleave_gate_up
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if world > 1:
            dist.init_process_group("nccl", device_id=dev)
        if args.batch % world:
            raise SystemExit("--batch must be a multiple of the number of GPUs (whole sequences per rank)")
        Bl = args.batch // world
        H, NH, NKV, HD, I, L, S = 4096, 32, 8, 128, 12288, args.layers, args.seq_len
        theta, rms_eps = 1e6, 1e-6
        g = torch.Generator(device=dev)  # (the same seed gives every rank the same weights)
        g.manual_seed(5)

        def rnd(n, k):
            return (torch.randn((n, k), generator=g, device=dev) * 0.02).to(torch.bfloat16)

        def rms(x, w):
            v = x.float()
            return (w * (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + rms_eps)).to(torch.bfloat16))

        pos = torch.arange(S, device=dev, dtype=torch.float32)
        inv = 1.0 / (theta ** (torch.arange(0, HD, 2, device=dev, dtype=torch.float32) / HD))
        ang = pos[:, None] * inv[None, :]
        cos, sin = torch.cat((ang.cos(), ang.cos()), -1).to(torch.bfloat16), torch.cat((ang.sin(), ang.sin()), -1).to(torch.bfloat16)

        def rope(t):  # t [B, S, heads, HD]
            t1, t2 = t[..., : HD // 2], t[..., HD // 2:]
            return t * cos[None, :, None, :] + torch.cat((-t2, t1), -1) * sin[None, :, None, :]

        layers, host_w0 = [], None
        for li in range(L):
            wq, wk, wv, wo = rnd(NH * HD, H), rnd(NKV * HD, H), rnd(NKV * HD, H), rnd(H, NH * HD)
            wg, wu, wd = rnd(I, H), rnd(I, H), rnd(H, I)
            ones = torch.ones(H, dtype=torch.bfloat16, device=dev)
            qn, kn = torch.ones(HD, dtype=torch.bfloat16, device=dev), torch.ones(HD, dtype=torch.bfloat16, device=dev)
            wqkv = torch.cat((wq, wk, wv), 0)
            wgu_il = interleave_gate_up(wg, wu)
            if li == 0 and args.check and rank == 0:
                host_w0 = {"qkv": wqkv.cpu(), "o": wo.cpu(), "gu": wgu_il.cpu(), "d": wd.cpu()}
            lay = {"ln1": ones, "ln2": ones.clone(), "qn": qn, "kn": kn,
                   "s_qkv": SplitLinear(wqkv, ratio=RATIO, rms_weight=ones, rms_eps=rms_eps),
                   "s_o": SplitLinear(wo, ratio=RATIO),
                   "s_gu": SplitLinear(wgu_il, ratio=RATIO, rms_weight=ones, rms_eps=rms_eps, epilogue="swiglu"),
                   "s_d": SplitLinear(wd, ratio=RATIO, had_kind=None)}
            if args.with_bf16:
                lay.update({"wqkv": wqkv, "wo": wo, "wgu": torch.cat((wg, wu), 0), "wd": wd})
            layers.append(lay)
            del wq, wk, wv, wg, wu, wgu_il
        g.manual_seed(1000 + rank)  # every rank its own sequences
        x0 = torch.randn((Bl * S, H), generator=g, device=dev).to(torch.bfloat16)

        def attention(qkv, lay):
            q, k, v = qkv.view(Bl, S, -1).split((NH * HD, NKV * HD, NKV * HD), -1)
            q = rope(rms(q.reshape(Bl, S, NH, HD), lay["qn"]))
            k = rope(rms(k.reshape(Bl, S, NKV, HD), lay["kn"]))
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2),
                                               v.reshape(Bl, S, NKV, HD).transpose(1, 2), is_causal=True, enable_gqa=True)
            return o.transpose(1, 2).reshape(Bl * S, NH * HD)

        def forward_split():
            h = x0
            for lay in layers:
                a = attention(lay["s_qkv"](h), lay)          # input RMSNorm inside the prologue
                h = h + lay["s_o"](a)
                h = h + lay["s_d"](lay["s_gu"](h))           # post-attention RMSNorm in the prologue, SwiGLU in the epilogue
            return h

        def forward_bf16():
            h = x0
            for lay in layers:
                a = attention(F.linear(rms(h, lay["ln1"]), lay["wqkv"]), lay)
                h = h + F.linear(a, lay["wo"])
                gu = F.linear(rms(h, lay["ln2"]), lay["wgu"])
                h = h + F.linear(F.silu(gu[:, :I]) * gu[:, I:], lay["wd"])
            return h

        def timed_ranks(fn, reps):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms

        reps = 5 if Bl * S <= 8192 else 3
        t_split = timed_ranks(forward_split, reps)
        out = {"workload": "prefill36", "n_gpus": world, "layers": L, "batch": args.batch, "sequences_per_gpu": Bl,
               "seq_len": S, "hidden": H, "ratio": RATIO, "split_prefill_ms": t_split,
               "tokens_per_s": args.batch * S / (t_split * 1e-3),
               "parallelism": f"whole sequences per GPU x{world}, replicated weights, no collective",
               "attention": "torch SDPA bf16 (GQA 32/8, head_dim 128, RoPE theta 1e6, q/k RMSNorm)",
               "fusions": "RMSNorm in the qkv / gate_up prologues, SwiGLU in the gate_up epilogue"}
        if args.with_bf16:
            t_bf = timed_ranks(forward_bf16, reps)
            out.update({"bf16_prefill_ms": t_bf, "bf16_tokens_per_s": args.batch * S / (t_bf * 1e-3),
                        "split_over_bf16": t_split / t_bf})

        # time spent outside the linears (attention, RoPE, norms of q/k, residual adds), measured on the same stack
        def forward_rest():
            h = x0
            qkv = torch.empty((Bl * S, (NH + 2 * NKV) * HD), dtype=torch.bfloat16, device=dev).normal_()
            for lay in layers:
                a = attention(qkv, lay)
                h = h + a
            return h
        out["non_linear_part_ms"] = timed_ranks(forward_rest, reps)

        if args.check and rank == 0:
            # every linear of layer 0 on 32 sampled token rows against the CPU oracle, each stage fed with the GPU's own
            # input of that stage (the attention output and the residual stream are taken from the GPU run)
            import numpy as np
            from oracle import oracle as O
            lay = layers[0]
            rows = torch.linspace(0, Bl * S - 1, 32).long().to(dev)
            bits = lambda t: t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
            ones_b = np.full((H,), 0x3F80, np.uint16)
            h = x0
            qkv = lay["s_qkv"](h).clone()
            a = attention(qkv, lay)
            o = lay["s_o"](a).clone()
            h1 = h + o
            gu = lay["s_gu"](h1).clone()
            d = lay["s_d"](gu).clone()
            torch.cuda.synchronize()

            def bounds(name, got_bits, y32, slack=1e-3):
                got = O.bf16_bits_to_f32(got_bits)
                err = np.abs(got.astype(np.float64) - y32.astype(np.float64))
                half_ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(y32), 1e-30))) - 8)
                assert bool(np.all(err <= np.maximum(2e-2, half_ulp * (1 + 1e-6) + slack))), f"layer 0 {name}: outside the output bounds"
                assert err.sum() / np.abs(y32).sum() <= 1e-2, f"layer 0 {name}: mean relative error"
                return float(err.max())

            res = {}
            R4, R12 = O.ceil_ratio_count(H, RATIO), O.ceil_ratio_count(I, RATIO)
            w = O.prepare_weight(bits(host_w0["qkv"]), O.HAD_WHT)
            xn = O.rmsnorm_bf16(bits(h[rows]), ones_b, eps=rms_eps)
            res["qkv"] = bounds("qkv", bits(qkv[rows]), O.split_linear_t16(xn, w, O.HAD_WHT, R4)[1])
            w = O.prepare_weight(bits(host_w0["o"]), O.HAD_WHT)
            res["o"] = bounds("o", bits(o[rows]), O.split_linear_t16(bits(a[rows]), w, O.HAD_WHT, R4)[1])
            w = O.prepare_weight(bits(host_w0["gu"]), O.HAD_WHT)
            xn = O.rmsnorm_bf16(bits(h1[rows]), ones_b, eps=rms_eps)
            y_bits = O.split_linear_t16(xn, w, O.HAD_WHT, R4)[0]
            want = O.swiglu_bf16(y_bits)
            gotb = bits(gu[rows])
            frac = float((want != gotb).mean())
            wa, ga = O.bf16_bits_to_f32(want), O.bf16_bits_to_f32(gotb)
            # SwiGLU of the bf16 outputs: one step of the linear's output can move the product by a few of its steps
            assert frac < 0.02 and bool(np.all(np.abs(wa - ga) <= np.maximum(np.abs(wa), np.abs(ga)) * 2.0 ** -5 + 1e-3)), \
                f"layer 0 gate_up + SwiGLU: {frac:.4f} of the outputs differ"
            res["gate_up_swiglu_fraction_not_equal"] = frac
            w = O.prepare_weight(bits(host_w0["d"]), O.HAD_KRON12)
            res["down"] = bounds("down", bits(d[rows]), O.split_linear_t16(bits(gu[rows]), w, O.HAD_KRON12, R12)[1])
            out["layer0_check"] = {"rows": 32, "max_abs_err": res, "checked": True}
        if rank == 0:
            print(json.dumps(out), flush=True)
        if world > 1:
            dist.destroy_process_group()
    elif args.workload == "llama_sweep":
        shapes = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672), ("down", 14336, 4096)]
        M = 4096
        for name, K, N in shapes:
            x, W = data(M, K, N, 3)
            bf = ms_of(lambda: torch.nn.functional.linear(x, W))
            for ratio in (0.0, 0.01, 0.05, 0.10):
                lin = SplitLinear(W, ratio=ratio)
                t = ms_of(lambda: lin.forward(x))
                print(json.dumps({"workload": "llama_sweep", "linear": name, "M": M, "K": K, "N": N, "ratio": ratio,
                                  "R": lin.R, "split_ms": t, "bf16_ms": bf, "split_over_bf16": t / bf,
                                  "tops": 2.0 * M * N * K / (t * 1e-3) / 1e12}), flush=True)
                del lin
    else:
        M, K, N = 512, 4096, 4096
        x, W = data(M, K, N, 0)
        bf = ms_of(lambda: torch.nn.functional.linear(x, W))
        for eng in ("mma", "gather"):
            lin = SplitLinear(W, ratio=RATIO, tail_engine=eng)
            t = ms_of(lambda: lin.forward(x))
            print(json.dumps({"workload": "single", "tail_engine": eng, "M": M, "K": K, "N": N, "R": lin.R,
                              "split_ms": t, "bf16_ms": bf, "tops": 2.0 * M * N * K / (t * 1e-3) / 1e12}), flush=True)


def main() -> None:
    global M_TOKENS, METRIC, CPU_SAMPLE_ROWS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="layer workload: also replay the layer graphs this long and report what the board sustains (0 = skip)")
    ap.add_argument("--rows-per-gpu", type=int, default=M_TOKENS,
                    help="token rows per GPU (2048 = the headline config; 4096 per GPU on 8 GPUs is the M = 32768 run)")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tail-engine", default="mma", choices=["mma", "gather"],
                    help="mma: tail on the tensor cores inside the GEMM kernel; gather: exact-order CUDA-core kernel")
    ap.add_argument("--workload", default="layer",
                    choices=["layer", "decode", "llama_sweep", "single", "latency_table", "prefill36", "probe"],
                    help="layer = the benchmark proper (baseline configs[1]); the others print secondary figures")
    ap.add_argument("--reference-rows", type=int, default=CPU_SAMPLE_ROWS,
                    help="token rows of the 2048 that the CPU arm (and the cpu_baseline leg) works through per step")
    ap.add_argument("--only", default="", help="decode / probe: restrict to one linear (qkv_proj, o_proj, gate_up_proj, down_proj)")
    ap.add_argument("--probe", default="gemm", choices=["prologue", "gemm"], help="probe: which kernel of the linear to launch")
    ap.add_argument("--ratio", type=float, default=RATIO, help="probe: tail ratio (0 = pure W4A4)")
    ap.add_argument("--prologue-mode", type=int, default=-1, choices=[-1, 0],
                    help="probe: 0 = the general prologue kernel also where the specialised one is built")
    ap.add_argument("--layers", type=int, default=36, help="prefill36: decoder layers")
    ap.add_argument("--seq-len", type=int, default=4096, help="prefill36: tokens")
    ap.add_argument("--with-bf16", action="store_true", help="prefill36: also time the same stack on bf16 cuBLAS linears")
    ap.add_argument("--batch", type=int, default=1, help="prefill36: sequences in the batch (cut into whole sequences per GPU)")
    ap.add_argument("--check", action="store_true", help="prefill36: compare the linears of layer 0 with the CPU oracle on 32 token rows")
    args = ap.parse_args()
    M_TOKENS = args.rows_per_gpu
    CPU_SAMPLE_ROWS = args.reference_rows
    METRIC = METRIC.replace("M=2048/GPU", f"M={M_TOKENS}/GPU")
    if args.workload != "layer":
        run_extra(args)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
