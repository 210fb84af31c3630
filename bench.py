#!/usr/bin/env python
"""Benchmark of the B200 KernelForge hot paths.  Prints ONE JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline workload (`flash_attn`): fused attention forward, MHA fp16, B=2 H=16 N=2048 D=64, non-causal,
softmax scale 1/8 -- the configuration the reference quotes its attention TFLOPS on.  A step is one call
of the hot path on one batch.  W untimed steps, then blocks of exactly K steps: the K launches of a block are
replayed from one CUDA graph (no host work between launches), every block sits between a barrier +
synchronize on both sides and two CUDA events on the launching stream; `value` comes from the MEDIAN block
(max over ranks), `blocks`, `block_ms` and `per_rank_ms` tell how many there were and how they spread.
`e2e` is the same metric through `kernelforge.ops.flash_attn` with host buffers: pinned host -> device
copies of q, k, v, the call, and the device -> host copy of o, pipelined over three streams and three
buffer sets, all inside the timed region.

Every other part of the metric is reported under `also`, each with its own `roofline` (algorithmic bytes or
FLOPs of the reference's formulas / event time / measured peak) and `cpu_baseline` (the reference's FP32 CPU
path -- plain torch on the host cores -- on a bounded sample, all threads and one thread):
    c1_*  INT4 linear at M=1, 5632x2048 (the first-named part of the metric; repeated at top level as
          `headline_alt`), and the same kernel on stacked copies (its streaming regime)
    c2_*  the headline's causal twin and the N x D sweep
    c3_*  GQA causal prefill at N=2048 and KV-cache decode attention
    c4_*  the decoder-linear shapes of a Qwen2.5-1.5B layer x M in {1, 16, 128, 1024}
    c5_*  end-to-end greedy decode of the TinyLlama-1.1B architecture
With N > 1 (torchrun, one rank per GPU) every rank runs the same per-GPU attention workload on its own batch
(attention shards over batch x heads with no communication: weak scaling); the N-sharded INT4 linear and
the tensor-parallel decode are added under `also`.

FLOP and byte counts are the reference's formulas: 4*B*H*Nq*Nk*D (halved when causal),
kernelforge/bench_utils.py:193-196; packed + scales + x + y bytes, bench/bench_gemm.py:80,98.

`--impl reference` times the reference's FP32 CPU path on the host cores, on the headline configuration: a step
is a bounded sample of (batch, head) slices, `ms_per_step` is the time of one full step (all B*H slices).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "kernel-forge_b200"))
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
HEADLINE = (2, 16, 16, 2048, 2048, 64)   # B, H, Hk, Nq, Nk, D
QWEN_SHAPES = {"q_o_proj": (1536, 1536), "k_v_proj": (256, 1536), "gate_up_proj": (8960, 1536), "down_proj": (1536, 8960)}


# ----------------------------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------------------------

def measured_peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi from before the warm-up to after the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines, self.marks = index, None, [], []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            time.sleep(1.0)   # the sampler is up and printing before any warm-up launch
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def mark(self):
        """Start / end of the timed region (host time): samples between the first and the last mark count as 'under load'."""
        self.marks.append(time.perf_counter())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.1)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self) -> dict:
        lo, hi = (self.marks[0], self.marks[-1]) if len(self.marks) >= 2 else (0.0, float("inf"))
        sm, sm_all, mx, reasons = [], [], [], set()
        for t, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clk, cmax = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            sm_all.append(clk)
            mx.append(cmax)
            if lo - 0.05 <= t <= hi + 0.05:
                sm.append(clk)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        if not sm_all:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        use = sm or sm_all
        return {"sm_mhz": statistics.median(use), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(use), "samples_in_timed_region": len(sm)}


def dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import datetime
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))
    return world, rank, local


def barrier_sync(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def gather_ranks(value: float, world: int) -> list[float]:
    if world == 1:
        return [value]
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [float(x.item()) for x in out]


def time_blocks(step_fn, steps: int, warmup: int, world: int, min_blocks: int = 25, min_seconds: float = 0.3,
                max_blocks: int = 400, graph: bool = True, sampler: ClockSampler | None = None) -> dict:
    """W untimed eager steps, then blocks of exactly K steps, each between barrier + synchronize and two events on
    the launching stream.  With `graph` the K launches of a block are one CUDA-graph replay (same kernels, same
    arguments, no host work between them).  Returns the per-block times of this rank and the max over ranks of the
    median block."""
    for i in range(warmup):
        step_fn(i)
    torch.cuda.synchronize()
    runner = None
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(steps):
                    step_fn(warmup + i)
        torch.cuda.synchronize()
        g.replay()          # one untimed replay
        runner = g.replay
    else:
        def runner():
            for i in range(steps):
                step_fn(warmup + i)
    times = []
    t_begin = time.perf_counter()
    if sampler:
        sampler.mark()
    while True:
        barrier_sync(world)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner()
        b.record()
        barrier_sync(world)
        times.append(a.elapsed_time(b))
        if world > 1:   # every rank must run the same number of blocks: a fixed count
            if len(times) >= max(min_blocks, 40):
                break
        elif len(times) >= min_blocks and (time.perf_counter() - t_begin >= min_seconds or len(times) >= max_blocks):
            break
    if sampler:
        sampler.mark()
    med = statistics.median(times)
    per_rank = gather_ranks(med, world)
    return {"block_ms": max(per_rank), "blocks": len(times), "steps_per_block": steps,
            "this_rank_block_ms": {"min": min(times), "median": med, "max": max(times)},
            "per_rank_ms": {"min": min(per_rank), "median": statistics.median(per_rank), "max": max(per_rank)}}


def time_graph_calls(launch_all, n_calls: int, steps: int, warmup: int, world: int, device) -> float:
    """A CUDA graph holding `n_calls` launches (distinct, L2-cold operands); returns microseconds per call."""
    side = torch.cuda.Stream(device)
    with torch.cuda.stream(side):
        launch_all(side)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            launch_all(side)
    for _ in range(max(2, warmup // 2)):
        graph.replay()
    barrier_sync(world)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        graph.replay()
    b.record()
    barrier_sync(world)
    ms = max(gather_ranks(a.elapsed_time(b), world))
    return 1e3 * ms / (steps * n_calls)


def roofline(bound: str, achieved: float, peaks: dict, peak_kind: str, traffic=None, **extra) -> dict:
    peak = peaks["hbm_gbs"] if bound == "hbm" else peaks["bf16_tflops"]
    unit = "GB/s" if bound == "hbm" else "TFLOP/s"
    return dict({"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                 "traffic": traffic, "peak_source": f"{peak_kind} " + ("HBM copy" if bound == "hbm" else "dense bf16 cuBLAS burst")},
                **extra)


# ----------------------------------------------------------------------------------------------
# CPU baselines: the reference's FP32 CPU path (plain torch on the host cores), bounded samples
# ----------------------------------------------------------------------------------------------

def _time_cpu(fn, budget_s: float, min_runs: int = 2) -> tuple[float, int]:
    fn()  # warm-up
    runs, t0 = 0, time.perf_counter()
    while True:
        fn()
        runs += 1
        el = time.perf_counter() - t0
        if runs >= min_runs and el >= budget_s:
            return el / runs, runs
        if el >= 4 * budget_s:
            return el / runs, runs


def _with_threads(n: int, fn):
    old = torch.get_num_threads()
    torch.set_num_threads(n)
    try:
        return fn()
    finally:
        torch.set_num_threads(old)


def cpu_threads() -> int:
    return max(1, os.cpu_count() or 1)


def cpu_attention(cfg, causal: bool, budget_s: float, unit_flops: bool = True) -> dict:
    """One (batch, kv-head group) slice of the workload per run; slices are independent and identical in cost."""
    from oracle import kf_oracle_torch as kt
    b, h, hk, nq, nk, d = cfg
    g = h // hk
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(1, g, nq, d, generator=gen).half()
    k = torch.randn(1, 1, nk, d, generator=gen).half()
    v = torch.randn(1, 1, nk, d, generator=gen).half()
    slices = b * hk
    flops_slice = 4.0 * g * nq * nk * d / (2 if causal else 1)
    bytes_slice = (2 * nk * d + 2 * g * nq * d) * 2
    n_thr = cpu_threads()
    s_all, runs = _with_threads(n_thr, lambda: _time_cpu(lambda: kt.attention(q, k, v, causal), budget_s))
    s_one, _ = _with_threads(1, lambda: _time_cpu(lambda: kt.attention(q, k, v, causal), min(budget_s, 3.0), 1))
    if unit_flops:
        val, one, unit = flops_slice / s_all / 1e12, flops_slice / s_one / 1e12, "TFLOP/s"
    else:
        val, one, unit = bytes_slice / s_all / 1e9, bytes_slice / s_one / 1e9, "GB/s"
    return {"value": val, "unit": unit, "cores": n_thr, "value_1_thread": one, "kind": "port",
            "seconds_per_full_step": s_all * slices,
            "sample": f"{runs} runs of one (batch, kv head) slice with its {g} query head(s); the step has {slices} such slices; "
                      f"torch FP32 on CPU (oracle/kf_oracle_torch.py)"}


def cpu_int4_linear(m: int, n: int, k: int, group: int, budget_s: float) -> dict:
    from oracle import kf_oracle_torch as kt
    from kernelforge import quantize as kq
    gen = torch.Generator().manual_seed(1)
    qw = kq.quantize_weight(torch.randn(n, k, generator=gen) * 0.02, group)
    x = torch.randn(m, k, generator=gen).half()
    nbytes = n * k // 2 + 2 * n * (k // group) + 2 * m * k + 2 * m * n
    fn = lambda: kt.int4_linear(x, qw.packed, qw.scales, group)
    n_thr = cpu_threads()
    s_all, runs = _with_threads(n_thr, lambda: _time_cpu(fn, budget_s))
    s_one, _ = _with_threads(1, lambda: _time_cpu(fn, min(budget_s, 2.0), 1))
    return {"value": nbytes / s_all / 1e9, "unit": "GB/s", "tflops": 2.0 * m * n * k / s_all / 1e12, "cores": n_thr,
            "value_1_thread": nbytes / s_one / 1e9, "kind": "port", "seconds_per_call": s_all,
            "sample": f"{runs} full calls: dequantize to FP32 + FP32 matmul, torch on CPU (oracle/kf_oracle_torch.py)"}


def cpu_decode_step(shape, batch: int, kv_len: int, budget_s: float) -> dict:
    """One decode step of the FP32 model on the host: the 7 linears (dequantised weights, FP32 matmul) and the attention
    of ONE layer plus the lm_head are timed; a step is layers x (layer time) + lm_head time."""
    s = shape
    gen = torch.Generator().manual_seed(2)
    rn = lambda *sz: torch.randn(*sz, generator=gen) * 0.02
    qd, kd = s.heads * s.head_dim, s.kv_heads * s.head_dim
    w = {"qkv": rn(qd + 2 * kd, s.hidden), "o": rn(s.hidden, qd), "gu": rn(2 * s.intermediate, s.hidden), "down": rn(s.hidden, s.intermediate)}
    lm = rn(s.vocab, s.hidden)
    kc, vc = torch.randn(batch, s.kv_heads, kv_len, s.head_dim, generator=gen), torch.randn(batch, s.kv_heads, kv_len, s.head_dim, generator=gen)
    x = torch.randn(batch, s.hidden, generator=gen)
    from oracle import kf_oracle_torch as kt

    def layer():
        qkv = x @ w["qkv"].T
        q = qkv[:, :qd].view(batch, s.heads, 1, s.head_dim)
        a = kt.attention(q, kc, vc, False).reshape(batch, qd)
        h = x + a @ w["o"].T
        gu = h @ w["gu"].T
        return h + (torch.nn.functional.silu(gu[:, :s.intermediate]) * gu[:, s.intermediate:]) @ w["down"].T

    n_thr = cpu_threads()
    t_layer, runs = _with_threads(n_thr, lambda: _time_cpu(layer, budget_s))
    t_head, _ = _with_threads(n_thr, lambda: _time_cpu(lambda: x @ lm.T, min(1.0, budget_s), 1))
    t1_layer, _ = _with_threads(1, lambda: _time_cpu(layer, min(2.0, budget_s), 1))
    t1_head, _ = _with_threads(1, lambda: _time_cpu(lambda: x @ lm.T, 0.5, 1))
    step, step1 = s.layers * t_layer + t_head, s.layers * t1_layer + t1_head
    return {"value": batch / step, "unit": "tok/s", "cores": n_thr, "value_1_thread": batch / step1, "kind": "port",
            "seconds_per_step": step,
            "sample": f"{runs} runs of one decoder layer (FP32 weights, KV cache of {kv_len}) and the lm_head at batch {batch}; "
                      f"step = {s.layers} x layer + lm_head; torch FP32 on CPU"}


# ----------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------

def attn_sets(b, h, hk, nq, nk, d, n_sets, device, seed=0):
    """q, k, v ~ N(0, 1) in fp16, seeded, generated on the device (timing inputs; the parity tests use host-made bits)."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *sz: torch.randn(*sz, generator=g, device=device, dtype=torch.float32).half()
    return [(rn(b, h, nq, d), rn(b, hk, nk, d), rn(b, hk, nk, d)) for _ in range(n_sets)]


def bench_flash_attn(args, world, device, causal: bool, cfg=HEADLINE, sampler=None, e2e=False, steps=None, quick=False) -> dict:
    from kernelforge import ops
    b, h, hk, nq, nk, d = cfg
    steps = steps or args.steps
    flops = 4.0 * b * h * nq * nk * d / (2 if causal else 1)
    per_set = (2 * b * h * nq * d + 2 * b * hk * nk * d) * 2
    n_sets = max(2, math.ceil(2 * L2_BYTES / per_set))  # rotating inputs: footprint > 2x L2, every step is L2-cold
    sets = attn_sets(b, h, hk, nq, nk, d, n_sets, device)

    def step(i):
        q, k, v = sets[i % n_sets]
        ops.flash_attn(q, k, v, causal=causal)

    r = time_blocks(step, steps, args.warmup, world, sampler=sampler, min_blocks=5 if quick else 25,
                    min_seconds=0.05 if quick else 0.3)
    ms_step = r["block_ms"] / steps
    out = {"tflops": world * flops / (ms_step * 1e-3) / 1e12, "ms_per_step": ms_step, "flops_per_step": flops,
           "n_sets": n_sets, "timing": r}
    if e2e:
        out["e2e"] = bench_flash_attn_e2e(args, world, device, causal, cfg, sets[0], flops)
        out["parity"] = attn_parity_sample(sets[0], causal)
    return out


def attn_parity_sample(first_set, causal: bool, heads=2) -> dict:
    """The result of the timed kernel on the first input set against an FP32 torch formulation of the same attention on
    the GPU (softmax(q k^T / sqrt(D)) v on `heads` heads of batch item 0): maximum absolute error, the fp16 rounding floor
    of the same reference tensor, and the reference's own bound (tests/test_attention.py:17: 2e-3 for fp16)."""
    from kernelforge import ops
    q, k, v = first_set
    o = ops.flash_attn(q, k, v, causal=causal)
    g = q.shape[1] // k.shape[1]
    qs, ks, vs = q[:1, :heads].float(), k[:1, :max(1, heads // g)].float(), v[:1, :max(1, heads // g)].float()
    ks, vs = ks.repeat_interleave(g, dim=1)[:, :heads], vs.repeat_interleave(g, dim=1)[:, :heads]
    sc = qs @ ks.transpose(-1, -2) / math.sqrt(q.shape[-1])
    if causal:
        nq, nk = sc.shape[-2:]
        sc = sc.masked_fill(torch.ones(nq, nk, dtype=torch.bool, device=sc.device).triu(1 + nk - nq), float("-inf"))
    ref = torch.softmax(sc, dim=-1) @ vs
    err = (o[:1, :heads].float() - ref).abs().max().item()
    floor = (ref.half().float() - ref).abs().max().item()
    return {"max_abs_err": err, "fp16_rounding_floor": floor, "bound": 2e-3, "heads_checked": heads,
            "reference": "FP32 torch attention on the GPU, same inputs"}


def bench_flash_attn_e2e(args, world, device, causal, cfg, first_set, flops) -> dict:
    """Host buffers in, host buffer out, through ops.flash_attn: H2D, kernel and D2H of consecutive steps overlap on
    three streams with three buffer sets (one cudaMemcpyAsync per tensor)."""
    from kernelforge import ops
    depth = 3
    hq, hk_, hv = (t.cpu().pin_memory() for t in first_set)
    ho = [torch.empty_like(hq).pin_memory() for _ in range(depth)]
    dq, dk, dv = ([torch.empty_like(t) for _ in range(depth)] for t in first_set)
    s_in, s_run, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device)
    ev_in = [torch.cuda.Event() for _ in range(depth)]
    ev_run = [torch.cuda.Event() for _ in range(depth)]
    ev_out = [torch.cuda.Event() for _ in range(depth)]

    def run(n_steps):
        for i in range(n_steps):
            s = i % depth
            with torch.cuda.stream(s_in):
                if i >= depth:
                    s_in.wait_event(ev_run[s])      # the kernel that read this buffer set has finished
                dq[s].copy_(hq, non_blocking=True)
                dk[s].copy_(hk_, non_blocking=True)
                dv[s].copy_(hv, non_blocking=True)
                ev_in[s].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[s])
                o = ops.flash_attn(dq[s], dk[s], dv[s], causal=causal)
                ev_run[s].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[s])
                if i >= depth:
                    s_out.wait_event(ev_out[s])
                o.record_stream(s_out)
                ho[s].copy_(o, non_blocking=True)
                ev_out[s].record(s_out)

    e2e_steps = max(6, min(args.steps, 30))
    run(depth)
    barrier_sync(world)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(s_in)
    run(e2e_steps)
    b.record(s_out)
    barrier_sync(world)
    ms = max(gather_ranks(a.elapsed_time(b), world))
    return {"value": world * flops * e2e_steps / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": hq.numel() * 2 + hk_.numel() * 2 + hv.numel() * 2, "d2h_bytes_per_step": ho[0].numel() * 2,
            "steps": e2e_steps, "ms_per_step": ms / e2e_steps,
            "how": "pinned host -> device copies, ops.flash_attn, device -> host copy; three streams, three buffer sets"}


def bench_decode_attn(args, world, device, batch=8, nk=4096) -> dict:
    """GQA decode attention (Hq=32, Hkv=4, D=64, q_len 1).  One CUDA graph holds one call per input set (sets total
    > 2x L2, so every call reads its K/V from HBM); a step replays the graph."""
    from kernelforge import ops
    h, hk, d = 32, 4, 64
    nbytes = 2 * batch * hk * nk * d * 2 + 2 * batch * h * d * 2
    n_sets = max(2, math.ceil(2 * L2_BYTES / nbytes))
    sets = attn_sets(batch, h, hk, 1, nk, d, n_sets, device, seed=1)
    keep = []

    def launch_all(stream):
        keep.clear()
        for q, k, v in sets:
            keep.append(ops.flash_attn(q, k, v, causal=True))

    us = time_graph_calls(launch_all, n_sets, max(5, args.steps // 4), args.warmup, world, device)
    return {"gbs": nbytes / (us * 1e-6) / 1e9, "us_per_call": us, "bytes_per_call": nbytes, "batch": batch, "nk": nk, "n_sets": n_sets}


def bench_int4(args, world, device, m, n, k, group=128, stack=1, pdl=True) -> dict:
    """INT4 linear through the dispatcher's kernels on L2-cold weight copies inside a CUDA graph (what a decode step or a
    layer loop sees), microseconds per call; for M <= 8 also with programmatic dependent launch."""
    from kernelforge import _capi, ops
    from kernelforge import quantize as kq
    nbytes = n * k // 2 + 2 * n * (k // group) + 2 * m * k + 2 * m * n
    copies = max(4 if nbytes < L2_BYTES else 2, math.ceil(3 * L2_BYTES / nbytes))
    g = torch.Generator().manual_seed(0)
    # `stack` > 1: the weight is `stack` copies of an (n / stack) x k matrix stacked along N (cheap to build, same kernel work)
    qw = kq.quantize_weight((torch.randn(n // stack, k, generator=g) * 0.02).to(device), group)
    p0 = qw.packed.repeat(stack, 1) if stack > 1 else qw.packed
    s0 = qw.scales.repeat(stack, 1) if stack > 1 else qw.scales
    packed = [p0] + [p0.clone() for _ in range(copies - 1)]
    scales = [s0] + [s0.clone() for _ in range(copies - 1)]
    x = torch.randn(m, k, generator=g).half().to(device)
    lib = _capi.lib()
    out = {"bytes_per_call": nbytes, "copies": copies, "M": m, "N": n, "K": k}
    if m <= ops.GEMV_MAX_M:
        ys = [torch.empty(m, n, dtype=torch.float16, device=device) for _ in range(copies)]
        for name, flags in (("graph", 0), ("graph_pdl", 1)) if pdl else (("graph", 0),):
            def launch_all(stream, flags=flags):
                for i in range(copies):
                    _capi.check(lib.kfb_int4_gemv(x.data_ptr(), packed[i].data_ptr(), scales[i].data_ptr(), ys[i].data_ptr(),
                                                  m, n, k, group, flags, stream.cuda_stream))
            try:
                us = time_graph_calls(launch_all, copies, max(5, args.steps // 4), args.warmup, world, device)
                out[name] = {"gbs": nbytes / (us * 1e-6) / 1e9, "us_per_call": us}
            except Exception as exc:  # report, never hide
                out[name] = {"error": repr(exc)[:200]}
    else:
        keep = []

        def launch_all(stream):
            keep.clear()
            for i in range(copies):
                keep.append(ops.int4_matmul(x, packed[i], scales[i], group))
        us = time_graph_calls(launch_all, copies, max(5, args.steps // 4), args.warmup, world, device)
        out["graph"] = {"gbs": nbytes / (us * 1e-6) / 1e9, "us_per_call": us}
    if m <= ops.PREPACKED_GEMV_MAX_M and stack == 1 and n % 16 == 0 and k % 64 == 0 and k <= 12288:
        # the same product on the private fragment-order copy of the weight (kfb_int4_gemv_prepacked, what int4_linear
        # runs once ops.prepack_weight_ has been called on the packed tensor)
        pre = [ops.prepack_int4(pw) for pw in packed]
        yp = [torch.empty(m, n, dtype=torch.float16, device=device) for _ in range(copies)]
        for name, use_pdl in (("prepacked_graph", False), ("prepacked_graph_pdl", True)) if pdl else (("prepacked_graph", False),):
            def launch_pre(stream, use_pdl=use_pdl):
                with _capi.programmatic_launch(use_pdl):
                    for i in range(copies):
                        _capi.check(lib.kfb_int4_gemv_prepacked(x.data_ptr(), pre[i].data_ptr(), scales[i].data_ptr(), yp[i].data_ptr(),
                                                                m, n, k, group, None, None, stream.cuda_stream))
            try:
                us = time_graph_calls(launch_pre, copies, max(5, args.steps // 4), args.warmup, world, device)
                out[name] = {"gbs": nbytes / (us * 1e-6) / 1e9, "us_per_call": us}
            except Exception as exc:  # report, never hide
                out[name] = {"error": repr(exc)[:200]}
        del pre, yp
    best = min((v["us_per_call"] for v in out.values() if isinstance(v, dict) and "us_per_call" in v), default=None)
    out["us_per_call"] = best
    if best:
        out["gbs"] = nbytes / (best * 1e-6) / 1e9
        out["tflops"] = 2.0 * m * n * k / (best * 1e-6) / 1e12
    return out


def llama_weights(shape, seed=0, std=0.02):
    """Random-init weights of the architecture, generated once on the host and shared by every batch size."""
    g = torch.Generator().manual_seed(seed)
    s = shape
    rn = lambda *sz: (torch.randn(*sz, generator=g) * std).half()
    qd, kd = s.heads * s.head_dim, s.kv_heads * s.head_dim
    layers = [{"in_norm": torch.ones(s.hidden), "post_norm": torch.ones(s.hidden), "q": rn(qd, s.hidden),
               "k": rn(kd, s.hidden), "v": rn(kd, s.hidden), "o": rn(s.hidden, qd), "gate": rn(s.intermediate, s.hidden),
               "up": rn(s.intermediate, s.hidden), "down": rn(s.hidden, s.intermediate)} for _ in range(s.layers)]
    return {"embed": rn(s.vocab, s.hidden), "lm_head": rn(s.vocab, s.hidden), "final_norm": torch.ones(s.hidden), "layers": layers}


def bench_decode_e2e(args, device, batch: int, weights, prompt_len=512, new_tokens=256, tp_group=None) -> dict:
    """Greedy decode of a random-init TinyLlama-1.1B-architecture model (22 layers, hidden 2048, 32 heads, 4 KV heads,
    head dim 64, SiLU MLP 5632, vocab 32000; weights ~ N(0, 0.02)), all decoder linears INT4 g128, fused attention,
    static KV cache, one CUDA graph per decode step.  Prompt = uniform random token ids (stands in for the
    reference's WikiText-2 prompt, which is not available offline).  tok/s = batch * steps / device time."""
    from kernelforge.llama_decode import TINYLLAMA_1B, LlamaInt4Decoder
    dec = LlamaInt4Decoder(TINYLLAMA_1B, weights, device, batch, prompt_len + new_tokens + 48, tp_group=tp_group)
    ids = torch.randint(0, TINYLLAMA_1B.vocab, (batch, prompt_len), generator=torch.Generator().manual_seed(0))
    t0 = time.perf_counter()
    dec.prefill(ids)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    dec.capture()
    for _ in range(3):
        dec.graph.replay()  # warm-up steps (they advance the sequence like any other step)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = new_tokens - 3
    a.record()
    for _ in range(steps):
        dec.graph.replay()
    b.record()
    b.synchronize()
    ms = a.elapsed_time(b)
    persistent_ms = None
    if getattr(dec, "persistent_ok", False) and not dec.persistent:
        # the same step as ONE persistent cooperative kernel (kfb_decode_step_persistent), for comparison
        n_p = 32   # (the cache was sized with 48 spare rows)
        if True:
            dec.persistent = True
            dec.capture()
            for _ in range(3):
                dec.graph.replay()
            a.record()
            for _ in range(n_p - 3):
                dec.graph.replay()
            b.record()
            b.synchronize()
            persistent_ms = a.elapsed_time(b) / (n_p - 3)
            dec.persistent = False
    s = TINYLLAMA_1B
    weight_bytes = s.layers * (2 * s.hidden * s.heads * s.head_dim + 2 * s.hidden * s.kv_heads * s.head_dim
                               + 3 * s.hidden * s.intermediate) * (0.5 + 2 / 128) + s.vocab * s.hidden * 2
    kv_bytes = s.layers * 2 * batch * s.kv_heads * (prompt_len + new_tokens / 2) * s.head_dim * 2
    out = {"tok_per_s": batch * steps / (ms * 1e-3), "ms_per_step": ms / steps, "batch": batch, "prompt": prompt_len,
           "steps_timed": steps, "prefill_s": prefill_s, "bytes_per_step": weight_bytes + kv_bytes,
           "hbm_gbs": (weight_bytes + kv_bytes) / (ms / steps * 1e-3) / 1e9,
           "kernels_per_step": getattr(dec, "kernels_per_step", None)}
    if persistent_ms is not None:
        out["persistent_kernel_ms_per_step"] = persistent_ms
    dec.release()   # the graph holds captured NCCL work when tensor-parallel: free it before any process-group teardown
    del dec
    torch.cuda.empty_cache()
    return out


def bench_sharded_linear(args, world, device, m=128, n=8960, k=1536, group=128) -> dict:
    """int4_linear sharded over output features: local N/world rows + one NCCL all-gather of [M, N/world]."""
    from kernelforge import parallel as kp
    from kernelforge import quantize as kq
    g = torch.Generator().manual_seed(0)
    qw = kq.quantize_weight((torch.randn(n, k, generator=g) * 0.02).to(device), group)
    lin = kp.ShardedInt4Linear.from_full(qw)
    x = torch.randn(m, k, generator=g).half().to(device)
    steps = 2 * max(10, args.steps // 2)   # even: the fused path alternates two result buffers
    keep = []

    def run(mod):
        def step(i):
            keep.append(mod(x))
            if len(keep) > 4:
                keep.pop(0)
        return step

    out = {"rows_per_rank": n // world}
    for name, build, how in (
            ("nccl_all_gather", lambda: lin, "local GEMM + nccl all_gather_into_tensor"),
            ("fused_peer_store", lambda: kp.FusedShardedInt4Linear.from_full(qw, max_m=m, alias=True),
             "GEMM epilogue stores its tile into every rank's symmetric buffer; device-side rendezvous (no NCCL kernel)")):
        try:
            mod = build()
            rec = {"how": how}
            for mode, graph in (("eager", False), ("graph", True)):
                r = time_blocks(run(mod), steps, args.warmup, world, min_blocks=5, min_seconds=0.05, graph=graph)
                us = 1e3 * r["block_ms"] / steps
                rec[mode] = {"us_per_call": us, "tflops": 2.0 * m * n * k / (us * 1e-6) / 1e12}
            out[name] = rec
        except Exception as exc:  # report, never hide
            out[name] = {"error": repr(exc)[:300]}
    return out


# ----------------------------------------------------------------------------------------------
# the `also` groups
# ----------------------------------------------------------------------------------------------

def group_c1(args, world, device, peaks, kind, full: bool) -> dict:
    out = {}
    r = bench_int4(args, world, device, 1, 5632, 2048)
    r["roofline"] = roofline("hbm", r["gbs"], peaks, kind, note="5,962,752 algorithmic bytes per call; back-to-back calls on L2-cold "
                             "weight copies in a CUDA graph (what a decode step sees)")
    if full:
        r["cpu_baseline"] = cpu_int4_linear(1, 5632, 2048, 128, 2.0)
    out["c1_int4_linear_m1_5632x2048"] = r
    for mm, stack in ((1, 32), (1, 128), (8, 128)) if full else ():
        s = bench_int4(args, world, device, mm, 5632 * stack, 2048, stack=stack)
        s["roofline"] = roofline("hbm", s["gbs"], peaks, kind, traffic=194900000 if (mm, stack) == (1, 32) else None,
                                 note=f"the same GEMV kernel on {stack} stacked copies of the 5632x2048 weight: its streaming regime")
        out[f"c1_stream_m{mm}_{5632 * stack}x2048"] = s
    return out


def group_c2(args, world, device, peaks, kind, full: bool) -> dict:
    out = {}
    fc = bench_flash_attn(args, world, device, causal=True)
    out["c2_flash_attn_causal_b2_h16_n2048_d64"] = {
        "tflops": fc["tflops"], "ms_per_step": fc["ms_per_step"],
        "roofline": roofline("tensor", fc["tflops"] / world, peaks, kind),
        "cpu_baseline": cpu_attention(HEADLINE, True, 3.0) if full else None}
    if full:
        sweep = {}
        for d in (64, 128):
            for n in (512, 1024, 2048, 4096, 8192):
                for causal in (False, True):
                    if (n, d) == (2048, 64):
                        continue
                    r = bench_flash_attn(args, world, device, causal, (2, 16, 16, n, n, d), steps=max(2, min(args.steps, 10)), quick=True)
                    sweep[f"n{n}_d{d}_{'causal' if causal else 'full'}"] = {
                        "tflops": round(r["tflops"], 1), "ms_per_step": round(r["ms_per_step"], 4),
                        "frac": round(r["tflops"] / world / peaks["bf16_tflops"], 4)}
        out["c2_sweep_b2_h16"] = sweep
    return out


def group_c3(args, world, device, peaks, kind, full: bool) -> dict:
    out = {}
    cfg = (1, 32, 4, 2048, 2048, 64)
    r = bench_flash_attn(args, world, device, True, cfg)
    out["c3_gqa_prefill_b1_hq32_hkv4_n2048_d64_causal"] = {
        "tflops": r["tflops"], "ms_per_step": r["ms_per_step"], "roofline": roofline("tensor", r["tflops"] / world, peaks, kind),
        "cpu_baseline": cpu_attention(cfg, True, 2.0) if full else None}
    for batch, nk in ((1, 4096), (8, 4096), (64, 4096), (8, 16384)) if full else ((8, 4096),):
        dd = bench_decode_attn(args, world, device, batch, nk)
        dd["roofline"] = roofline("hbm", dd["gbs"], peaks, kind)
        if full and (batch, nk) in ((8, 4096), (64, 4096)):
            dd["cpu_baseline"] = cpu_attention((batch, 32, 4, 1, nk, 64), True, 1.5, unit_flops=False)
        out[f"c3_decode_attn_b{batch}_nk{nk}"] = dd
    return out


def group_c4(args, world, device, peaks, kind) -> dict:
    out = {}
    for name, (n, k) in QWEN_SHAPES.items():
        for m in (1, 16, 128, 1024):
            r = bench_int4(args, world, device, m, n, k, pdl=False)
            tensor_bound = m >= 128
            rec = {"N": n, "K": k, "M": m, "us_per_call": r["us_per_call"], "bytes": r["bytes_per_call"], "gbs": r["gbs"],
                   "pct_of_hbm_peak": 100 * r["gbs"] / peaks["hbm_gbs"], "tflops": r["tflops"],
                   "roofline": roofline("tensor", r["tflops"], peaks, kind) if tensor_bound else roofline("hbm", r["gbs"], peaks, kind)}
            if m in (1, 128):
                rec["cpu_baseline"] = cpu_int4_linear(m, n, k, 128, 0.6)
            out[f"c4_{name}_{n}x{k}_m{m}"] = rec
    return out


def group_c5(args, world, device, peaks, kind, full: bool) -> dict:
    from kernelforge.llama_decode import TINYLLAMA_1B
    out = {}
    weights = llama_weights(TINYLLAMA_1B)
    for batch in (1, 8, 32) if full else (1,):
        try:
            r = bench_decode_e2e(args, device, batch, weights)
            r["roofline"] = roofline("hbm", r["hbm_gbs"], peaks, kind, note="weights (INT4 + scales, fp16 lm_head) + KV cache read once per step")
            if batch in (1, 32):
                r["cpu_baseline"] = cpu_decode_step(TINYLLAMA_1B, batch, 640, 2.0)
            out[f"c5_decode_e2e_tinyllama_arch_b{batch}"] = r
        except Exception as exc:  # report, never hide
            out[f"c5_decode_e2e_tinyllama_arch_b{batch}"] = {"error": repr(exc)[:300]}
    return out


def group_multi_gpu(args, world, device, peaks, kind) -> dict:
    import torch.distributed as dist
    from kernelforge.llama_decode import TINYLLAMA_1B
    out = {"mg_int4_linear_n_sharded_m128_8960x1536": bench_sharded_linear(args, world, device)}
    weights = llama_weights(TINYLLAMA_1B)
    for batch in (1, 32):
        key = f"mg_decode_e2e_tinyllama_arch_tp{world}_b{batch}"
        try:
            r = bench_decode_e2e(args, device, batch, weights, tp_group=dist.group.WORLD)
            r["note"] = "ONE model sharded over the GPUs (strong scaling); tok/s is the model's, not per GPU"
            out[key] = r
        except Exception as exc:  # report, never hide
            out[key] = {"error": repr(exc)[:300]}
    return out


# ----------------------------------------------------------------------------------------------
# single-kernel modes (few launches: what profiler captures are taken from)
# ----------------------------------------------------------------------------------------------

def single_kernel_main(args):
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, kind = measured_peaks()
    if args.workload == "int4_gemv":
        dims = [int(v) for v in args.shape.split(",")] if args.shape else [5632, 2048]
        n, k, m = dims[0], dims[1], (dims[2] if len(dims) > 2 else 1)
        r = bench_int4(args, 1, device, m, n, k)
        print(json.dumps({"metric": f"int4_linear M={m} HBM GB/s (% peak)", "unit": "GB/s", "value": r["gbs"], "n_gpus": 1,
                          "config": {"workload": f"int4_gemv M={m} N={n} K={k} g128"}, "detail": r,
                          "roofline": roofline("hbm", r["gbs"], peaks, kind)}))
    elif args.workload == "int4_gemm":
        m, n, k = (int(v) for v in args.shape.split(",")) if args.shape else (1024, 8960, 1536)
        r = bench_int4(args, 1, device, m, n, k, pdl=False)
        print(json.dumps({"metric": "int4_linear TFLOPS (% peak)", "unit": "TFLOP/s", "value": r["tflops"], "n_gpus": 1,
                          "config": {"workload": f"int4_gemm M={m} N={n} K={k} g128", "l2": f"{r['copies']} rotating weight copies"},
                          "detail": r, "roofline": roofline("tensor", r["tflops"], peaks, kind)}))
    elif args.workload == "decode_attn":
        b, nk = (int(v) for v in args.shape.split(",")) if args.shape else (8, 4096)
        r = bench_decode_attn(args, 1, device, b, nk)
        print(json.dumps({"metric": "decode attention HBM GB/s (% peak)", "unit": "GB/s", "value": r["gbs"], "n_gpus": 1,
                          "config": {"workload": f"decode attn Hq=32 Hkv=4 D=64 B={b} Nk={nk}"}, "detail": r,
                          "roofline": roofline("hbm", r["gbs"], peaks, kind)}))
    elif args.workload == "decode_step":
        from kernelforge.llama_decode import TINYLLAMA_1B
        batch = int(args.shape) if args.shape else 1
        r = bench_decode_e2e(args, device, batch, llama_weights(TINYLLAMA_1B), new_tokens=3 + max(1, args.steps))
        print(json.dumps({"metric": "decode tok/s", "unit": "tok/s", "value": r["tok_per_s"], "n_gpus": 1,
                          "config": {"workload": f"greedy decode, TinyLlama-1.1B architecture, batch {batch}, prompt 512"}, "detail": r,
                          "roofline": roofline("hbm", r["hbm_gbs"], peaks, kind)}))
    else:  # flash_attn_only
        cfg = HEADLINE
        if args.shape:
            b_, h_, n_, d_ = (int(v) for v in args.shape.split(","))
            cfg = (b_, h_, h_, n_, n_, d_)
        r = bench_flash_attn(args, 1, device, args.causal, cfg, quick=True)
        print(json.dumps({"metric": "flash_attn TFLOPS (% peak)", "unit": "TFLOP/s", "value": r["tflops"], "n_gpus": 1,
                          "ms_per_step": r["ms_per_step"],
                          "config": {"workload": f"flash_attn fwd fp16 B={cfg[0]} H={cfg[1]} N={cfg[3]} D={cfg[5]} "
                                                 f"{'causal' if args.causal else 'non-causal'}"},
                          "roofline": roofline("tensor", r["tflops"], peaks, kind)}))


# ----------------------------------------------------------------------------------------------
# main
# ----------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="flash_attn", choices=["flash_attn", "flash_attn_only", "int4_gemv", "int4_gemm", "decode_attn", "decode_step"],
                    help="flash_attn = headline + every other part of the metric under `also`; the others run one kernel only "
                         "(few launches, for profiler captures)")
    ap.add_argument("--shape", default=None, help="override: B,H,N,D (flash_attn_only) / N,K[,M] (int4_gemv) / M,N,K (int4_gemm) / B,NK (decode_attn) / B (decode_step)")
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--headline-only", action="store_true", help="skip the `also` groups")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 1)
    if args.workload != "flash_attn":
        return single_kernel_main(args)

    config = {"workload": "flash_attn fwd MHA fp16 B=2 H=16 N=2048 D=64 non-causal, scale 1/sqrt(64)",
              "l2": "inputs rotate over distinct sets totalling > 2x the 126 MB L2",
              "per_gpu": "same batch shape on every GPU (batch x heads shard, no communication)",
              "timing": "blocks of K steps, each one CUDA-graph replay between barrier + synchronize, CUDA events; median block, max over ranks"}
    base = {"metric": "flash_attn TFLOPS (% peak) [headline]; int4_linear M=1 HBM GB/s [headline_alt]; decode tok/s and the rest under `also`",
            "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": config}

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        b, h = HEADLINE[0], HEADLINE[1]
        per_step = max(1.0, min(args.cpu_seconds, 100.0 / max(1, args.steps + args.warmup)))
        vals = [cpu_attention(HEADLINE, False, per_step) for _ in range(args.warmup + args.steps)][args.warmup:]
        v = statistics.mean(x["value"] for x in vals)
        cb = dict(vals[-1], value=v)
        ms_step = 1e3 * statistics.mean(x["seconds_per_full_step"] for x in vals)
        line = dict(base, impl="reference", value=v, ms_per_step=ms_step, cpu_baseline=cb, gpu_launches=0,
                    e2e={"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        line["config"] = dict(config, timing=f"each step times a bounded sample of the {b * h} (batch, head) slices of the workload; "
                                             "ms_per_step is the time of one full step at that rate")
        print(json.dumps(line))
        return

    world, rank, local = dist_setup()
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    peaks, kind = measured_peaks()
    full = world == 1 and not args.headline_only

    with ClockSampler(device.index) as clocks:
        fa = bench_flash_attn(args, world, device, causal=False, sampler=clocks, e2e=True)
    also = {}
    if not args.headline_only:
        also.update(group_c1(args, world, device, peaks, kind, full))
        also.update(group_c2(args, world, device, peaks, kind, full))
        also.update(group_c3(args, world, device, peaks, kind, full))
        if world == 1:
            also.update(group_c4(args, world, device, peaks, kind))
            also.update(group_c5(args, world, device, peaks, kind, full))
        else:
            also.update(group_multi_gpu(args, world, device, peaks, kind))

    t = fa["timing"]
    line = dict(base)
    line.update({
        "value": fa["tflops"], "ms_per_step": fa["ms_per_step"], "blocks": t["blocks"], "block_ms": t["block_ms"],
        "per_rank_ms": t["per_rank_ms"], "e2e": fa["e2e"], "parity": fa["parity"], "gpu_launches": args.steps,
        "clocks": clocks.summary(),
        "roofline": roofline("tensor", fa["tflops"] / world, peaks, kind,
                             # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload from an ncu capture
                             # (q, k, v read once = 25.2 MB; o stays in L2 until after the launch)
                             traffic=25205760, kernel="attn_prefill_pair_kernel<64,fp16>"),
    })
    c1 = also.get("c1_int4_linear_m1_5632x2048")
    if c1:
        line["headline_alt"] = {"metric": "int4_linear M=1 K=2048 N=5632 g128 HBM GB/s", "value": c1["gbs"], "unit": "GB/s",
                                "us_per_call": c1["us_per_call"], "roofline": c1["roofline"]}
    line["also"] = also
    if rank == 0:
        line["cpu_baseline"] = cpu_attention(HEADLINE, False, args.cpu_seconds) if full else None
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
