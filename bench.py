#!/usr/bin/env python
"""Benchmark of the B200 KernelForge hot paths.  Prints ONE JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline workload (`flash_attn`): fused attention forward, MHA fp16, B=2 H=16 N=2048 D=64, non-causal,
softmax scale 1/8 -- the configuration the reference quotes its attention TFLOPS on.  A step is one call
of the hot path on one batch.  `value` is whole-job TFLOP/s with inputs resident in HBM (CUDA events on
the launching stream, max over ranks); `e2e` is the same metric through `kernelforge.ops.flash_attn`
with host buffers (pinned host -> device copies of q, k, v and the device -> host copy of o inside the
timed region).  Other workloads of the metric are reported under `also` (INT4 GEMV at M=1 in GB/s,
causal prefill, GQA decode attention) and can be made the headline with --workload.

FLOP and byte counts are the reference's formulas: 4*B*H*Nq*Nk*D (halved when causal),
kernelforge/bench_utils.py:193-196; packed + scales + x + y bytes, bench/bench_gemm.py:80,98.

With N > 1 (torchrun, one rank per GPU) every rank runs the same per-GPU workload on its own batch
(attention shards over batch x heads with no communication): weak scaling, no collective in the data path.

`--impl reference` times the reference's FP32 CPU path (the numpy restatement in oracle/, all host
threads) on a bounded sample of the same workload.
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


# ----------------------------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------------------------

def measured_peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    return world, rank, local


def barrier_sync(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int) -> float:
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(step_fn, steps: int, warmup: int, world: int) -> float:
    """W untimed steps, then exactly K steps between two events on the current stream; ms, max over ranks."""
    for i in range(warmup):
        step_fn(i)
    barrier_sync(world)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        step_fn(warmup + i)
    end.record()
    barrier_sync(world)
    return max_over_ranks(start.elapsed_time(end), world)


# ----------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------

def attn_sets(b, h, hk, nq, nk, d, n_sets, device, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    sets = []
    for _ in range(n_sets):
        q = torch.randn(b, h, nq, d, generator=g).half()
        k = torch.randn(b, hk, nk, d, generator=g).half()
        v = torch.randn(b, hk, nk, d, generator=g).half()
        sets.append((q.to(device), k.to(device), v.to(device)))
    return sets


def bench_flash_attn(args, world, device, causal: bool, cfg=(2, 16, 16, 2048, 2048, 64)) -> dict:
    from kernelforge import ops
    b, h, hk, nq, nk, d = cfg
    flops = 4.0 * b * h * nq * nk * d / (2 if causal else 1)
    per_set = (2 * b * h * nq * d + 2 * b * hk * nk * d) * 2
    n_sets = max(2, math.ceil(2 * L2_BYTES / per_set))  # rotating inputs: footprint > 2x L2, every step is L2-cold
    sets = attn_sets(b, h, hk, nq, nk, d, n_sets, device)

    def step(i):
        q, k, v = sets[i % n_sets]
        ops.flash_attn(q, k, v, causal=causal)

    with ClockSampler(device.index) as clocks:
        ms = time_steps(step, args.steps, args.warmup, world)
    tflops = world * flops * args.steps / (ms * 1e-3) / 1e12

    # end to end through the public op with host buffers
    hq, hk_, hv = (t.cpu().pin_memory() for t in sets[0])
    ho = torch.empty_like(hq).pin_memory()
    dq, dk, dv = (torch.empty_like(t) for t in sets[0])

    def e2e_step(i):
        dq.copy_(hq, non_blocking=True)
        dk.copy_(hk_, non_blocking=True)
        dv.copy_(hv, non_blocking=True)
        ho.copy_(ops.flash_attn(dq, dk, dv, causal=causal), non_blocking=True)

    e2e_steps = max(3, min(args.steps, 20))
    ms_e2e = time_steps(e2e_step, e2e_steps, 3, world)
    return {
        "tflops": tflops, "ms_per_step": ms / args.steps, "flops_per_step": flops, "launches_per_step": 1,
        "clocks": clocks.summary(), "n_sets": n_sets,
        "e2e": {"value": world * flops * e2e_steps / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": hq.numel() * 2 + hk_.numel() * 2 + hv.numel() * 2,
                "d2h_bytes_per_step": ho.numel() * 2},
    }


def bench_decode_attn(args, world, device, batch=8, nk=4096) -> dict:
    """GQA decode attention (Hq=32, Hkv=4, D=64, q_len 1).  One CUDA graph holds one call per input set
    (sets total > 2x L2, so every call reads its K/V from HBM); a step replays the graph.  Launching from a
    graph removes the Python / ctypes overhead of ~50 us per call, which otherwise hides the kernel."""
    from kernelforge import ops
    h, hk, d = 32, 4, 64
    nbytes = 2 * batch * hk * nk * d * 2 + 2 * batch * h * d * 2
    n_sets = max(2, math.ceil(2 * L2_BYTES / nbytes))
    sets = attn_sets(batch, h, hk, 1, nk, d, n_sets, device, seed=1)
    side = torch.cuda.Stream(device)
    with torch.cuda.stream(side):
        for q, k, v in sets[:2]:
            ops.flash_attn(q, k, v, causal=True)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            outs = [ops.flash_attn(q, k, v, causal=True) for q, k, v in sets]
    ms = time_steps(lambda i: graph.replay(), args.steps, args.warmup, world)
    calls = args.steps * n_sets
    return {"gbs": world * nbytes * calls / (ms * 1e-3) / 1e9, "us_per_call": 1e3 * ms / calls,
            "bytes_per_call": nbytes, "batch": batch, "nk": nk, "n_sets": n_sets}


def bench_int4_gemv(args, world, device, m=1, n=5632, k=2048, group=128, stack=1) -> dict:
    """INT4 linear at M=1.  Three figures on the same algorithmic bytes: a CUDA graph of back-to-back calls
    over distinct weight copies (what a decode step sees; every call reads L2-cold weights), the same with
    programmatic dependent launch, and single event-timed calls (latency)."""
    from kernelforge import _capi, ops
    from kernelforge import quantize as kq
    nbytes = n * k // 2 + 2 * n * (k // group) + 2 * m * k + 2 * m * n
    copies = max(4 if nbytes < L2_BYTES else 2, math.ceil(3 * L2_BYTES / nbytes))
    g = torch.Generator().manual_seed(0)
    # `stack` > 1: the weight is `stack` copies of an (n / stack) x k matrix stacked along N (cheap to build, same kernel work)
    qw = kq.quantize_weight((torch.randn(n // stack, k, generator=g) * 0.02).to(device), group)
    packed = [qw.packed.repeat(stack, 1) for _ in range(copies)]
    scales = [qw.scales.repeat(stack, 1) for _ in range(copies)]
    x = torch.randn(m, k, generator=g).half().to(device)
    ys = [torch.empty(m, n, dtype=torch.float16, device=device) for _ in range(copies)]
    lib = _capi.lib()

    def launch_all(flags, stream):
        for i in range(copies):
            _capi.check(lib.kfb_int4_gemv(x.data_ptr(), packed[i].data_ptr(), scales[i].data_ptr(), ys[i].data_ptr(),
                                          m, n, k, group, flags, stream))

    out = {"bytes_per_call": nbytes, "copies": copies}
    side = torch.cuda.Stream(device)
    for name, flags in (("graph", 0), ("graph_pdl", 1)):
        try:
            with torch.cuda.stream(side):
                launch_all(flags, side.cuda_stream)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    launch_all(flags, side.cuda_stream)
            ms = time_steps(lambda i: graph.replay(), args.steps, args.warmup, world)
            out[name] = {"gbs": world * nbytes * copies * args.steps / (ms * 1e-3) / 1e9,
                         "us_per_call": 1e3 * ms / (args.steps * copies)}
        except Exception as exc:  # report, never hide
            out[name] = {"error": repr(exc)[:200]}
    # single calls, L2-cold weights (rotating copies), one event pair each
    times = []
    for i in range(args.warmup + 50):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        ops.int4_linear(x, packed[i % copies], scales[i % copies], group)
        b.record()
        b.synchronize()
        if i >= args.warmup:
            times.append(a.elapsed_time(b))
    med = statistics.median(times)
    out["single_call"] = {"gbs": nbytes / (med * 1e-3) / 1e9, "us_per_call": med * 1e3}
    return out


def bench_decode_e2e(args, device, batch: int, prompt_len=512, new_tokens=256, tp_group=None) -> dict:
    """Greedy decode of a random-init TinyLlama-1.1B-architecture model (22 layers, hidden 2048, 32 heads, 4 KV heads,
    head dim 64, SiLU MLP 5632, vocab 32000; weights ~ N(0, 0.02)), all decoder linears INT4 g128, fused attention,
    static KV cache, one CUDA graph per decode step.  Prompt = uniform random token ids (stands in for the
    reference's WikiText-2 prompt, which is not available offline).  tok/s = batch * steps / device time."""
    from kernelforge.llama_decode import TINYLLAMA_1B, LlamaInt4Decoder
    dec = LlamaInt4Decoder.random_init(TINYLLAMA_1B, device, batch, prompt_len + new_tokens + 8, seed=0, tp_group=tp_group)
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
    s = TINYLLAMA_1B
    weight_bytes = s.layers * (2 * s.hidden * s.heads * s.head_dim + 2 * s.hidden * s.kv_heads * s.head_dim
                               + 3 * s.hidden * s.intermediate) * (0.5 + 2 / 128) + s.vocab * s.hidden * 2
    kv_bytes = s.layers * 2 * batch * s.kv_heads * (prompt_len + new_tokens / 2) * s.head_dim * 2
    out = {"tok_per_s": batch * steps / (ms * 1e-3), "ms_per_step": ms / steps, "batch": batch, "prompt": prompt_len,
           "steps_timed": steps, "prefill_s": prefill_s, "bytes_per_step": weight_bytes + kv_bytes,
           "hbm_gbs": (weight_bytes + kv_bytes) / (ms / steps * 1e-3) / 1e9}
    dec.release()   # the graph holds captured NCCL work when tensor-parallel: free it before any process-group teardown
    del dec
    torch.cuda.empty_cache()
    return out


def bench_sharded_linear(args, world, device, m=128, n=8960, k=1536, group=128) -> dict:
    """int4_linear sharded over output features: local N/world rows + one NCCL all-gather of [M, N/world]."""
    import torch.distributed as dist
    from kernelforge import parallel as kp
    from kernelforge import quantize as kq
    g = torch.Generator().manual_seed(0)
    qw = kq.quantize_weight((torch.randn(n, k, generator=g) * 0.02).to(device), group)
    lin = kp.ShardedInt4Linear.from_full(qw)
    x = torch.randn(m, k, generator=g).half().to(device)
    ms = time_steps(lambda i: lin(x), args.steps, args.warmup, world)
    out = {"us_per_call": 1e3 * ms / args.steps, "tflops": 2.0 * m * n * k * args.steps / (ms * 1e-3) / 1e12,
           "rows_per_rank": n // world, "collective": "nccl all_gather_into_tensor"}
    try:
        fused = kp.FusedShardedInt4Linear.from_full(qw, max_m=m)
        ms_f = time_steps(lambda i: fused(x), args.steps, args.warmup, world)
        out["fused_peer_store"] = {"us_per_call": 1e3 * ms_f / args.steps,
                                   "tflops": 2.0 * m * n * k * args.steps / (ms_f * 1e-3) / 1e12,
                                   "how": "GEMM epilogue stores its tile into every rank's symmetric buffer"}
    except Exception as exc:  # report, never hide
        out["fused_peer_store"] = {"error": repr(exc)[:300]}
    return out


# ----------------------------------------------------------------------------------------------
# CPU baseline (the oracle = restatement of the reference's FP32 CPU path)
# ----------------------------------------------------------------------------------------------

def cpu_attention_sample(budget_s: float, causal: bool, cfg=(2, 16, 16, 2048, 2048, 64)) -> dict:
    from oracle import kf_oracle as ko
    b, h, hk, nq, nk, d = cfg
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 1, nq, d), dtype=np.float32).astype(np.float16)
    k = rng.standard_normal((1, 1, nk, d), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((1, 1, nk, d), dtype=np.float32).astype(np.float16)
    ko.attention(q, k, v, causal)  # warm-up
    heads, t0 = 0, time.perf_counter()
    while True:  # (batch, head) slices are independent and identical in cost: time as many as fit the budget
        ko.attention(q, k, v, causal)
        heads += 1
        el = time.perf_counter() - t0
        if el >= budget_s:
            break
    flops_head = 4.0 * nq * nk * d / (2 if causal else 1)
    return {"value": heads * flops_head / el / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "seconds": el,
            "sample": f"{heads} (batch, head) slices (the workload has {b * h}) in {el:.1f} s, numpy/BLAS threads"}


# ----------------------------------------------------------------------------------------------
# main
# ----------------------------------------------------------------------------------------------

def single_kernel_main(args):
    """One kernel, few launches: the command profiler captures are taken from."""
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, peak_kind = measured_peaks()
    if args.workload == "int4_gemv":
        n, k = (int(v) for v in args.shape.split(",")) if args.shape else (5632, 2048)
        r = bench_int4_gemv(args, 1, device, 1, n, k)
        best = max((r[x]["gbs"] for x in ("graph", "graph_pdl") if "gbs" in r.get(x, {})), default=0.0)
        print(json.dumps({"metric": "int4_linear M=1 HBM GB/s (% peak)", "unit": "GB/s", "value": best, "n_gpus": 1,
                          "config": {"workload": f"int4_gemv M=1 N={n} K={k} g128"}, "detail": r,
                          "roofline": {"bound": "hbm", "achieved": best, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                       "frac": best / peaks["hbm_gbs"], "traffic": None, "peak_source": peak_kind}}))
    elif args.workload == "int4_gemm":
        from kernelforge import ops
        from kernelforge import quantize as kq
        m, n, k = (int(v) for v in args.shape.split(",")) if args.shape else (1024, 8960, 1536)
        g = torch.Generator().manual_seed(0)
        copies = max(2, math.ceil(2 * L2_BYTES / (n * k // 2 + 2 * m * k + 2 * m * n)))
        qws = [kq.quantize_weight((torch.randn(n, k, generator=g) * 0.02).to(device), 128) for _ in range(copies)]
        xs = [torch.randn(m, k, generator=g).half().to(device) for _ in range(copies)]
        ms = time_steps(lambda i: ops.int4_gemm_ragged(xs[i % copies], qws[i % copies].packed, qws[i % copies].scales, 128),
                        args.steps, args.warmup, 1)
        tf = 2.0 * m * n * k * args.steps / (ms * 1e-3) / 1e12
        print(json.dumps({"metric": "int4_linear TFLOPS (% peak)", "unit": "TFLOP/s", "value": tf, "n_gpus": 1,
                          "config": {"workload": f"int4_gemm M={m} N={n} K={k} g128", "l2": f"{copies} rotating weight/activation sets"},
                          "ms_per_step": ms / args.steps,
                          "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                       "frac": tf / peaks["bf16_tflops"], "traffic": None, "peak_source": peak_kind}}))
    else:
        b, nk = (int(v) for v in args.shape.split(",")) if args.shape else (8, 4096)
        r = bench_decode_attn(args, 1, device, b, nk)
        print(json.dumps({"metric": "decode attention HBM GB/s (% peak)", "unit": "GB/s", "value": r["gbs"], "n_gpus": 1,
                          "config": {"workload": f"decode attn Hq=32 Hkv=4 D=64 B={b} Nk={nk}"}, "detail": r,
                          "roofline": {"bound": "hbm", "achieved": r["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                       "frac": r["gbs"] / peaks["hbm_gbs"], "traffic": None, "peak_source": peak_kind}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="flash_attn", choices=["flash_attn", "flash_attn_only", "int4_gemv", "int4_gemm", "decode_attn"],
                    help="flash_attn = headline + every other workload under `also`; the others run one kernel only "
                         "(small, for profiler captures)")
    ap.add_argument("--shape", default=None, help="override: B,H,N,D (attention) / N,K (int4_gemv) / M,N,K (int4_gemm) / B,NK (decode_attn)")
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload in ("int4_gemv", "int4_gemm", "decode_attn"):
        return single_kernel_main(args)

    config = {"workload": "flash_attn fwd MHA fp16 B=2 H=16 N=2048 D=64 non-causal, scale 1/sqrt(64)",
              "l2": "inputs rotate over distinct sets totalling > 2x the 126 MB L2",
              "per_gpu": "same batch shape on every GPU (batch x heads shard, no communication)"}
    base = {"metric": "flash_attn TFLOPS (% peak) [headline]; int4_linear M=1 HBM GB/s and decode tok/s under `also`", "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": config}

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        per_step = max(1.0, min(args.cpu_seconds, 120.0 / max(1, args.steps + args.warmup)))
        vals = [cpu_attention_sample(per_step, False) for _ in range(args.warmup + args.steps)][args.warmup:]
        v = statistics.mean(x["value"] for x in vals)
        cb = dict(vals[-1], value=v)
        ms_step = 1e3 * statistics.mean(x["seconds"] for x in vals)
        line = dict(base, impl="reference", value=v, ms_per_step=ms_step, cpu_baseline=cb, gpu_launches=0,
                    e2e={"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        print(json.dumps(line))
        return

    world, rank, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    peaks, peak_kind = measured_peaks()

    cfg = (2, 16, 16, 2048, 2048, 64)
    if args.shape:
        b_, h_, n_, d_ = (int(v) for v in args.shape.split(","))
        cfg = (b_, h_, h_, n_, n_, d_)
        config["workload"] = f"flash_attn fwd MHA fp16 B={b_} H={h_} N={n_} D={d_} {'causal' if args.causal else 'non-causal'} (override)"
    fa = bench_flash_attn(args, world, device, causal=args.causal, cfg=cfg)
    also = {}
    if args.workload == "flash_attn":
        fc = bench_flash_attn(args, world, device, causal=True)
        also["flash_attn_causal"] = {"tflops": fc["tflops"], "ms_per_step": fc["ms_per_step"],
                                     "frac_of_peak": fc["tflops"] / world / peaks["bf16_tflops"]}
        gv = bench_int4_gemv(args, world, device)
        best = max((gv[k]["gbs"] for k in ("graph", "graph_pdl") if "gbs" in gv.get(k, {})), default=None)
        also["int4_gemv_m1_5632x2048"] = dict(gv, roofline={
            "bound": "hbm", "achieved": None if best is None else best / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": None if best is None else best / world / peaks["hbm_gbs"], "traffic": None,
            "note": "achieved = sustained back-to-back calls on L2-cold weight copies; single_call is latency"})
        gs = bench_int4_gemv(args, world, device, 1, 5632 * 32, 2048, stack=32)
        sbest = max((gs[k]["gbs"] for k in ("graph", "graph_pdl") if "gbs" in gs.get(k, {})), default=None)
        also["int4_gemv_m1_stream_180224x2048"] = dict(gs, roofline={
            "bound": "hbm", "achieved": None if sbest is None else sbest / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": None if sbest is None else sbest / world / peaks["hbm_gbs"],
            "traffic": 194900000,  # ncu: 190.5 MB read + 4.4 MB written per launch (profiles/int4_gemv_M1_N180224_K2048.md)
            "note": "same kernel on 32 stacked copies of the 5632x2048 weight: the streaming regime of the GEMV"})
        for mm in (1, 8):
            gl = bench_int4_gemv(args, world, device, mm, 5632 * 128, 2048, stack=128)
            lbest = max((gl[k]["gbs"] for k in ("graph", "graph_pdl") if "gbs" in gl.get(k, {})), default=None)
            also[f"int4_gemv_m{mm}_stream_720896x2048"] = dict(gl, roofline={
                "bound": "hbm", "achieved": None if lbest is None else lbest / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": None if lbest is None else lbest / world / peaks["hbm_gbs"], "traffic": None,
                "note": "128 stacked copies (738 MB): long enough for launch, ramp and tail (~10 us) not to dominate"})
        if world > 1:
            also["int4_linear_n_sharded_m128_8960x1536"] = bench_sharded_linear(args, world, device)
            import torch.distributed as dist
            # tensor-parallel decode: every linear sharded over output features, 4 all-gathers per layer.  Run by default on
            # 2 GPUs (the configuration this was verified on); KFB_BENCH_TP=1 enables it for 4 and 8
            for batch in ((1, 32) if (world == 2 or os.environ.get("KFB_BENCH_TP") == "1") else ()):
                try:
                    r = bench_decode_e2e(args, device, batch, tp_group=dist.group.WORLD)
                    r["note"] = "ONE model sharded over the GPUs (strong scaling); tok/s is the model's, not per GPU"
                    also[f"decode_e2e_tinyllama_arch_tp{world}_b{batch}"] = r
                except Exception as exc:  # report, never hide
                    also[f"decode_e2e_tinyllama_arch_tp{world}_b{batch}"] = {"error": repr(exc)[:300]}
        if world == 1:
            for batch in (1, 8, 32):
                try:
                    r = bench_decode_e2e(args, device, batch)
                    r["frac_of_hbm"] = r["hbm_gbs"] / peaks["hbm_gbs"]
                    also[f"decode_e2e_tinyllama_arch_b{batch}"] = r
                except Exception as exc:  # report, never hide
                    also[f"decode_e2e_tinyllama_arch_b{batch}"] = {"error": repr(exc)[:300]}
        for batch, nk in ((1, 4096), (8, 4096), (64, 4096), (8, 16384)):
            dd = bench_decode_attn(args, world, device, batch, nk)
            dd["frac_of_hbm"] = dd["gbs"] / world / peaks["hbm_gbs"]
            also[f"decode_attn_b{batch}_nk{nk}"] = dd

    line = dict(base)
    line.update({
        "value": fa["tflops"], "ms_per_step": fa["ms_per_step"], "e2e": fa["e2e"], "gpu_launches": args.steps,
        "clocks": fa["clocks"],
        "roofline": {"bound": "tensor", "achieved": fa["tflops"] / world, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": fa["tflops"] / world / peaks["bf16_tflops"],
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload from the ncu
                     # capture summarised in profiles/attn_prefill_B2_H16_N2048_D64.md (q, k, v read once = 25.2 MB)
                     "traffic": 25205760 if (not args.shape and not args.causal) else None,
                     "peak_source": f"{peak_kind} dense bf16 cuBLAS burst", "kernel": "attn_prefill_kernel<64,fp16>"},
        "also": also,
    })
    if rank == 0:
        full = args.workload == "flash_attn" and not args.shape
        line["cpu_baseline"] = cpu_attention_sample(args.cpu_seconds, False) if (world == 1 and full) else None
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
