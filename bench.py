#!/usr/bin/env python
"""Benchmark of the HSTU jagged attention forward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg4] [--impl reference]

A step is one call of the operator (scheduler pre-pass + attention kernel) over one synthetic jagged batch.
The default workload is the long-sequence batch ("cfg4": B=256, H=8, d=128, lognormal lengths up to 8192, bf16);
with N GPUs its sequences are split over the ranks by a FLOP-balanced partition, one process per GPU, no
collective on the data path (total work fixed => "scaling": "strong").  Rank 0 prints one JSON line:

  value        useful TFLOP/s over all ranks, inputs resident in HBM, CUDA events, max over ranks
  e2e          same metric through the torch operator with HOST (pinned) inputs and a host copy of the result,
               copies inside the timed region
  roofline     the attention kernel against the measured dense-bf16 peak (MEASURED_PEAKS.json)
  cpu_baseline the CPU oracle (a port of the reference's PyTorch golden) on this box's cores, bounded sample
  clocks       SM clock and throttle reasons sampled during the timed region

`--impl reference` times that CPU port alone (rank 0 only) and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "hstu_jagged_fwd_causal_tflops"
UNIT = "TFLOP/s"

# DRAM bytes (read + write) per token of one attention-kernel launch, from one ncu capture of the first 24 sequences
# of cfg4 (412.4 MB for 51 883 tokens).  An estimate for the full launch, not a measurement of it: the compulsory part
# (q / k / v / out) scales with the tokens, K/V re-reads after L2 eviction would grow faster with the sequence length.
TRAFFIC_BYTES_PER_TOKEN = {"cfg4": 412.4e6 / 51883}

WORKLOAD_DESC = {
    "cfg2": "cfg2: B=32 H=4 d=128 bf16, L~U[256,1024], max_seq_len=1024, causal, no rab",
    "cfg3": "cfg3: cfg2 + rab [32,4,1024,1024] bf16 + num_target~U[0,32] (group 1)",
    "cfg4": "cfg4: B=256 H=8 d=128 bf16, L~lognormal(ln2048,0.6) in [64,8192], max_seq_len=8192, causal, no rab",
    "cfg5": "cfg5: B=4096 H=4 d=64 bf16, L~lognormal(ln200,0.8) in [8,2048], shared rab [4,2048,2048], "
            "num_target~U[1,64] (group 1)",
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops_burst=p["bf16_tflops"], tflops_sustained=p["bf16_tflops_sustained"], hbm=p["hbm_gbs"],
                    source="measured")
    return dict(tflops_burst=1590.0, tflops_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU through NVML (read-only) while the timed region runs."""

    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index, period=0.02):
        self.samples, self.mask, self.max_mhz = [], 0, None
        self._stop = threading.Event()
        self._thread = None
        self.period = period
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        reasons = [name for bit, name in self.REASONS.items() if self.mask & bit and name != "gpu_idle"]
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(self.samples)}


def load_workloads():
    """ops_rec_b200/workloads.py loaded by path: importing the package would load the native libraries, and the
    reference arm must run without any of the product's code in its process."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_hstu_workloads", os.path.join(ROOT, "ops_rec_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod   # (dataclasses look their module up by name)
    spec.loader.exec_module(mod)
    return mod


def cpu_forward_sample(w, W, seconds_target=15.0):
    """Time the reference's CPU implementation of the forward (torch, all host threads) on a length-stratified sample
    of the workload's sequences.  With the reference's own files present (baseline/_ref, see oracle/fetch_reference.py)
    this is `Kernel._forward_impl` of its PyTorch golden, one B = 1 call per sampled sequence with explicit
    scale = 1 / max_seq_len (its batched form pads to [B, H, maxL, maxL]: 550 GB for cfg4) and the mask built by its
    create_causal_mask - kind "reference"; otherwise the restatement in oracle/hstu_oracle.py - kind "port".
    Returns a dict(tflops, tokens_per_s, desc, cores, seconds, kind)."""
    import numpy as np
    import torch

    from oracle import fetch_reference

    torch.set_num_threads(os.cpu_count() or 1)
    order = np.argsort(w.lengths, kind="stable")
    n = min(8, len(order))
    picks = order[np.linspace(0, len(order) - 1, n).round().astype(int)]
    sub = w.subset(np.unique(picks), name=w.name + "-sample")
    kw = W.materialize(sub, "cpu")
    ref = fetch_reference.load()
    if ref is not None:
        Kernel, causal_mask = ref
        off = kw["seq_offset"].tolist()
        scale = 1.0 / kw["max_seq_len"]
        tgt = kw["num_target"].tolist() if kw["num_target"] is not None else None
        bias = kw["attn_bias"]

        def run():
            outs = []
            for b in range(len(off) - 1):
                L = off[b + 1] - off[b]
                o = torch.tensor([0, L])
                sl = slice(off[b], off[b + 1])
                rab = None
                if bias is not None:
                    blk = bias if bias.dim() == 3 else bias[b]
                    rab = blk[None, :, :L, :L].float().clone()
                t = tgt[b] if tgt else None
                mask = causal_mask(L, L, None, t if t else None, kw["target_group_size"] if t else None)[None, None]
                ker = Kernel(kw["alpha"], scale, rab is not None, L, L, o, o)
                outs.append(ker._forward_impl(kw["q"][sl].float(), kw["k"][sl].float(), kw["v"][sl].float(), rab, mask))
            return outs
        kind, what = "reference", "the reference's PyTorch golden Kernel._forward_impl (fp32, one B=1 call per sequence)"
    else:
        from oracle import hstu_oracle as O

        def run():
            return O.hstu_jagged_forward(**kw)
        kind, what = "port", "CPU restatement of the reference golden (fp32; the reference's own files are not present)"
    t0 = time.perf_counter()
    run()
    dt = time.perf_counter() - t0
    reps = 1
    # repeat the same sample to fill the time budget (bounded), keep the best rate
    while dt * (reps + 1) < seconds_target and reps < 5:
        t1 = time.perf_counter()
        run()
        dt = min(dt, time.perf_counter() - t1)
        reps += 1
    desc = (f"{sub.batch} of {w.batch} sequences of {w.name} (length-stratified, {sub.tokens} tokens, "
            f"{sub.flops() / 1e9:.1f} GFLOP), {what}, best of {reps}")
    return dict(tflops=sub.flops() / dt / 1e12, tokens_per_s=sub.tokens / dt, desc=desc,
                cores=torch.get_num_threads(), seconds=dt, kind=kind)


def run_reference(args, rank):
    """--impl reference: the reference's CPU implementation alone, on this box's host cores.  Nothing of the product
    is imported (no native library is loaded into this process)."""
    if rank != 0:
        return
    W = load_workloads()
    w = W.make_workload(args.workload)
    if args.max_batch:
        import numpy as np
        w = w.subset(np.arange(min(args.max_batch, w.batch)))
    vals = []
    r = None
    t_all = time.perf_counter()
    for i in range(args.warmup + args.steps):
        r = cpu_forward_sample(w, W, seconds_target=0.0)
        if i >= args.warmup:
            vals.append(r)
        if time.perf_counter() - t_all > 150:  # keep the whole run within minutes
            break
    if not vals:
        vals = [r]
    tf = statistics.median(v["tflops"] for v in vals)
    tk = statistics.median(v["tokens_per_s"] for v in vals)
    ms = statistics.median(v["seconds"] for v in vals) * 1e3
    desc, cores, kind = r["desc"], r["cores"], r["kind"]
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus, "steps": len(vals),
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "tokens_per_s": tk,
        "config": {"workload": WORKLOAD_DESC[args.workload], "step": "bounded sample: " + desc},
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    # this arm is the reference alone: none of the product's native code may be in the process
    with open("/proc/self/maps") as f:
        maps = f.read()
    assert "ops_rec_b200" not in sys.modules and "libhstu_b200" not in maps and "_torch_shim" not in maps
    print(json.dumps(line), flush=True)


def run_ln_mul(args, local_rank):
    """--op ln_mul: (LayerNorm(x) * gamma + beta) * u on fp32 [A, 1024], A = 262 144 rows (x, u, out: 1 GiB each, far
    beyond L2).  HBM-bound: algorithmic bytes = 12 per element; peak = the measured copy bandwidth."""
    import statistics
    import torch
    import ops_rec_b200 as ops_rec
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    a, r = 262144, 1024
    gen = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(a, r, device=dev, generator=gen)
    u = torch.randn(a, r, device=dev, generator=gen)
    gamma, beta = torch.randn(r, device=dev, generator=gen), torch.randn(r, device=dev, generator=gen)
    op = ops_rec.ascendc.activation.ln_mul
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        op(x, u, gamma, beta)
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        for i in range(args.steps):
            starts[i].record()
            op(x, u, gamma, beta)
            ends[i].record()
        torch.cuda.synchronize()
    ms = statistics.mean(s.elapsed_time(e) for s, e in zip(starts, ends))
    nbytes = 12.0 * a * r + 8.0 * r
    peaks = load_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "ln_mul_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": f"ln_mul fp32 [{a}, {r}]", "l2": "3 GiB per step: no flush"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"],
                     "traffic": None, "kernel": "ln_mul_rows_kernel<32, true>", "algorithmic_bytes_per_launch": nbytes},
        "gpu_launches": args.steps, "clocks": clocks.summary()}), flush=True)


def run_in_linear_silu(args, local_rank):
    """--op in_linear_silu: x [65536, 1024] . weight [4096, 1024]^T + bias -> linear_output and the four SiLU outputs
    (bf16).  Tensor-bound: 2 m n k = 550 GFLOP per launch; it also writes 2 x m x n x 2 bytes = 1.07 GB."""
    import statistics
    import torch
    import ops_rec_b200 as ops_rec
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    m, k, n = args.m, 1024, 4096
    gen = torch.Generator(device=dev).manual_seed(1)
    x = (torch.randn(m, k, device=dev, generator=gen)).to(torch.bfloat16)
    w = (torch.randn(n, k, device=dev, generator=gen) * (6.0 / (n + k)) ** 0.5).to(torch.bfloat16)
    bias = torch.ones(n, device=dev)
    split = [n // 4] * 4
    op = ops_rec.ascendc.activation.distance_in_linear_silu
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        op(x, w, bias, split)
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        for i in range(args.steps):
            starts[i].record()
            op(x, w, bias, split)
            ends[i].record()
        torch.cuda.synchronize()
    ms = statistics.mean(s.elapsed_time(e) for s, e in zip(starts, ends))
    flops = 2.0 * m * n * k
    peaks = load_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "in_linear_silu_tflops", "value": tf, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"in_linear_silu bf16 m={m} k={k} n={n}, even split", "l2": "1.2 GB per step: no flush"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                     "frac": tf / peaks["tflops_burst"], "traffic": None, "kernel": "in_linear_silu_kernel",
                     "algorithmic_flops_per_launch": flops},
        "gpu_launches": args.steps, "clocks": clocks.summary()}), flush=True)


def time_cold(step, flush, reps):
    """Per-launch device time of `step` with a cold L2: a buffer larger than the L2 is rewritten before every launch,
    one CUDA-event pair per launch on the launching stream (the host runs ahead while the flush executes, so the
    interval holds device work only).  Returns the median in ms."""
    import torch
    ts = []
    for _ in range(reps):
        # (twice: ~160 us of device work, so that the host has enqueued the whole call - validation, tensor maps and
        # two launches take it some tens of microseconds - before the device gets to the first event)
        flush.zero_()
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def run_also(ops_rec, W, dev, peaks, names=("cfg2", "cfg3", "cfg5"), reps=12):
    """The other named bf16 shapes, one GPU, cold L2 (their working sets - 87 MB, 149 MB - fit the 126 MB L2, so
    back-to-back launches would flatter them).  All three are HBM-bound on compulsory traffic: hbm_frac is the
    fraction that matters, tensor_frac is given beside it."""
    import torch
    hj = ops_rec.ascendc.attention.hstu_jagged
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    out = {}
    for name in names:
        w = W.make_workload(name)
        kw = W.materialize(w, dev)

        def step():
            return hj(kw["q"], kw["k"], kw["v"], None, kw["attn_bias"], 0, kw["max_seq_len"], 0.0, kw["seq_offset"],
                      None, kw["num_target"], kw["target_group_size"], kw["alpha"])
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        ms = time_cold(step, flush, reps)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            step()
        e1.record()
        torch.cuda.synchronize()
        warm_ms = e0.elapsed_time(e1) / 20
        tf = w.flops() / (ms * 1e-3) / 1e12
        gbs = w.bytes() / (ms * 1e-3) / 1e9
        out[name] = {"value": tf, "unit": UNIT, "ms_per_step": ms, "tokens_per_s": w.tokens / (ms * 1e-3),
                     "hbm_gbs_algorithmic": gbs, "hbm_frac": gbs / peaks["hbm"], "tensor_frac": tf / peaks["tflops_burst"],
                     "l2": "cold", "steps": reps, "warm_ms_per_step": warm_ms, "workload": WORKLOAD_DESC[name]}
        del kw
        torch.cuda.empty_cache()
    # what a call costs before it computes anything: one sequence of one token (pre-pass + launch + set-up + drain)
    w1 = W.Workload("one", 1, 4, 128, 128, __import__("numpy").array([1]))
    kw = W.materialize(w1, dev)
    f = lambda: hj(kw["q"], kw["k"], kw["v"], None, None, 0, 128, 0.0, kw["seq_offset"], None, None, 0, kw["alpha"])
    for _ in range(3):
        f()
    out["fixed_cost_us"] = time_cold(f, flush, reps) * 1e3
    del kw
    # the backward of the operator (hstu_jagged_backward: 2.5 x the forward's FLOPs) on cfg4, cfg3 and cfg5 (without rab), and the
    # operator that produces q / k / v (distance_in_linear_silu, m = 65536, k = 1024, n = 4096): device-resident,
    # a few back-to-back steps each, CUDA events
    hb = ops_rec.ascendc.attention.hstu_jagged_backward
    for name, steps in (("cfg4", 5), ("cfg3", 12), ("cfg5", 8)):
        w = W.make_workload(name)
        if name == "cfg5":
            w.rab = None   # cfg5's rab is shared by the batch; the backward takes a per-sequence bias only
        kw = W.materialize(w, dev)
        grad = torch.randn_like(kw["q"]) * 0.1
        ctx = None if kw["num_target"] is None else torch.zeros_like(kw["num_target"])

        def bstep():
            return hb(grad, kw["q"], kw["k"], kw["v"], None, kw["attn_bias"], 0, kw["max_seq_len"], 0.0,
                      kw["seq_offset"], ctx, kw["num_target"], kw["target_group_size"], kw["alpha"])
        for _ in range(3):
            bstep()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            bstep()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        tf = 2.5 * w.flops() / (ms * 1e-3) / 1e12
        out["backward_" + name] = {"value": tf, "unit": UNIT, "ms_per_step": ms, "steps": steps,
                                   "tensor_frac": tf / peaks["tflops_burst"], "l2": "warm (back to back)",
                                   "flops": "2.5 x forward (S, dP, dV, dK, dQ; recomputation not counted)"}
        if name == "cfg5":
            out["backward_" + name]["workload"] = "cfg5 without its rab (shared by the batch: no per-sequence gradient)"
        del kw, grad
        torch.cuda.empty_cache()
    m, k, n = 65536, 1024, 4096
    gen = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)
    wt = (torch.randn(n, k, device=dev, generator=gen) * (6.0 / (n + k)) ** 0.5).to(torch.bfloat16)
    bias = torch.ones(n, device=dev)
    op = ops_rec.ascendc.activation.distance_in_linear_silu
    for _ in range(3):
        op(x, wt, bias, [n // 4] * 4)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        op(x, wt, bias, [n // 4] * 4)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 20
    tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    out["in_linear_silu"] = {"value": tf, "unit": UNIT, "ms_per_step": ms, "steps": 20,
                             "tensor_frac": tf / peaks["tflops_burst"], "workload": f"bf16 m={m} k={k} n={n}, even split"}
    return out


def paged_workload(W):
    """A cfg5-shaped serving batch for hstu_paged: every user's history (cfg5's L - T rows) sits in a paged KV cache
    (pages of 128 rows handed out in shuffled order), the call brings the last 16 history rows (or fewer) plus the
    T targets as queries."""
    import numpy as np
    w = W.make_workload("cfg5")
    T = w.targets.astype(np.int64)
    cache_len = np.maximum(w.lengths - T, 1)
    new_hist = np.minimum(16, cache_len)
    lq = new_hist + T
    prev = cache_len - new_hist
    i = np.arange(16)[None, :]
    hist_pairs = ((i < new_hist[:, None]) * (i + prev[:, None] + 1)).sum(1)
    pairs = hist_pairs + T * (cache_len + 1)
    return dict(w=w, T=T, cache_len=cache_len, new_hist=new_hist, lq=lq, pairs=pairs, page=128)


def run_paged(args, local_rank):
    """--op paged: ops_rec::hstu_paged on the serving batch above (B=4096, H=4, d=64, bf16), inputs resident in HBM.
    HBM-bound: algorithmic bytes = q + out + the cached K/V rows + the target K/V rows, each once."""
    import numpy as np
    import torch
    import ops_rec_b200 as ops_rec
    from ops_rec_b200 import workloads as W
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    pw = paged_workload(W)
    w, page = pw["w"], pw["page"]
    B, H, D = w.batch, w.heads, w.dim
    if args.max_batch:
        B = min(B, args.max_batch)
    rng = np.random.default_rng(0)
    cache_len, lq, T = pw["cache_len"][:B], pw["lq"][:B], pw["T"][:B]
    pages_per = (cache_len + page - 1) // page
    total_pages = int(pages_per.sum())
    order = rng.permutation(total_pages)
    page_off = np.concatenate([[0], np.cumsum(pages_per)])
    last_len = np.where(cache_len % page == 0, page, cache_len % page)
    gen = torch.Generator(device=dev).manual_seed(1)
    rnd = lambda *s: (torch.randn(*s, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    tq = int(lq.sum())
    q, k, v = rnd(tq, H, D), rnd(tq, H, D), rnd(tq, H, D)
    cache = rnd(total_pages, 2, page, H, D)
    i64 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int64, device=dev)
    off_q, off_k = i64(np.concatenate([[0], np.cumsum(lq)])), i64(np.concatenate([[0], np.cumsum(cache_len + T)]))
    off_t = i64(np.concatenate([[0], np.cumsum(T)]))
    meta = (i64(page_off), i64(order), i64(last_len), i64(T))
    max_q, max_k = int(lq.max()), int((cache_len + T).max())
    op = ops_rec.ascendc.attention.hstu_paged

    def step():
        return op(q, k, v, cache, None, None, 0, max_q, max_k, 0.0, off_q, off_k, off_t, meta[0], meta[1], meta[2],
                  meta[3], 1, 1.0 / D)
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        for i in range(args.steps):
            starts[i].record()
            step()
            ends[i].record()
        torch.cuda.synchronize()
    ms = statistics.mean(s.elapsed_time(e) for s, e in zip(starts, ends))
    flops = float(H * 4 * D * pw["pairs"][:B].sum())
    nbytes = float((2 * tq + 2 * int((cache_len + T).sum())) * H * D * 2)
    peaks = load_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "hstu_paged_fwd_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "tokens_per_s": tq / (ms * 1e-3),
        "config": {"workload": f"hstu_paged: B={B} H={H} d={D} bf16, cache rows per user = cfg5's history "
                               f"(mean {cache_len.mean():.0f}), page size {page}, {int(T.sum())} targets + up to 16 new "
                               f"history rows per user as queries", "query_tokens": tq,
                   "kv_rows": int((cache_len + T).sum()), "l2": f"{nbytes / 1e6:.0f} MB per step: no flush"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"],
                     "traffic": None, "kernel": "hstu_paged_gather_kernel + hstu_tc_kernel",
                     "algorithmic_bytes_per_launch": nbytes, "note": "the gather pass moves the K/V rows a second time "
                     "(staging write + read), which the algorithmic bytes do not count"},
        "gpu_launches": 4 * args.steps, "clocks": clocks.summary()}), flush=True)


def run_backward(args, ops_rec, W, full, mine, kw, dev, rank, world, local_rank, warmup, barrier):
    """--op backward: hstu_jagged_backward on the same workload, inputs resident in HBM.  FLOPs: the five products
    of the backward (S, dP, dV, dK, dQ) = 2.5 x the forward's two; the kernels recompute S and dP in both passes,
    which is not counted."""
    import statistics
    import torch
    import torch.distributed as dist
    hb = ops_rec.ascendc.attention.hstu_jagged_backward
    grad = torch.randn_like(kw["q"]) * 0.1
    flops = 2.5 * full.flops()

    def step():
        return hb(grad, kw["q"], kw["k"], kw["v"], None, kw["attn_bias"], 0, kw["max_seq_len"], 0.0,
                  kw["seq_offset"], None if kw["num_target"] is None else torch.zeros_like(kw["num_target"]),
                  kw["num_target"], kw["target_group_size"], kw["alpha"])

    for _ in range(warmup):
        step()
    barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        barrier()
        for i in range(args.steps):
            starts[i].record()
            step()
            ends[i].record()
        barrier()
    t = torch.tensor([starts[0].elapsed_time(ends[-1])], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        peaks = load_peaks()
        ms = float(t.item()) / args.steps
        k_ms = statistics.mean(s.elapsed_time(e) for s, e in zip(starts, ends))
        achieved = 2.5 * mine.flops() / (k_ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "hstu_jagged_bwd_causal_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": full.dtype, "data": "synthetic",
            "config": {"workload": WORKLOAD_DESC[args.workload], "op": "hstu_jagged_backward"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tflops_burst"], "traffic": None,
                         "kernel": "hstu_bwd_tc_kernel (dQ pass + dK/dV pass)"},
            "gpu_launches": 3 * args.steps, "clocks": clocks.summary()}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg4", choices=sorted(WORKLOAD_DESC))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--op", default="forward", choices=["forward", "backward", "ln_mul", "in_linear_silu", "paged"],
                    help="backward: time hstu_jagged_backward (device-resident only) instead of the forward; "
                         "ln_mul: time ops_rec::ln_mul on [262144, 1024] fp32 (HBM roofline); "
                         "in_linear_silu: time ops_rec::distance_in_linear_silu, m=65536 k=1024 n=4096 bf16; "
                         "paged: time ops_rec::hstu_paged on a cfg5-shaped serving batch")
    ap.add_argument("--m", type=int, default=65536, help="--op in_linear_silu: rows of x (small cases for captures)")
    ap.add_argument("--no-also", action="store_true",
                    help="skip the cold-L2 timings of cfg2 / cfg3 / cfg5 that the default run adds to its line")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="length of the back-to-back loop behind the line's \"sustained\" figure (0 = skip)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-chunks", type=int, default=8,
                    help="the end-to-end run sends the batch through in this many chunks of whole sequences")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--max-batch", type=int, default=0,
                    help="keep only the first N sequences of the workload (small cases for profiler captures)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.op == "ln_mul":
        if rank == 0:
            run_ln_mul(args, local_rank)
        return
    if args.op == "in_linear_silu":
        if rank == 0:
            run_in_linear_silu(args, local_rank)
        return
    if args.op == "paged":
        if rank == 0:
            run_paged(args, local_rank)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    import ops_rec_b200 as ops_rec
    from ops_rec_b200 import cabi
    from ops_rec_b200 import workloads as W

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    full = W.make_workload(args.workload)
    if args.max_batch:
        full = full.subset(np.arange(min(args.max_batch, full.batch)))
    parts = W.partition_lpt(full.lengths, world)
    mine = full.subset(parts[rank])
    flop_imb, tok_imb = W.imbalance(full.lengths, parts)
    kw = W.materialize(mine, dev, seed=1 + rank)
    hj = ops_rec.ascendc.attention.hstu_jagged

    def step():
        return hj(kw["q"], kw["k"], kw["v"], None, kw["attn_bias"], 0, kw["max_seq_len"], 0.0, kw["seq_offset"],
                  None, kw["num_target"], kw["target_group_size"], kw["alpha"])

    warmup = max(args.warmup, 3)
    if args.op == "backward":
        run_backward(args, ops_rec, W, full, mine, kw, dev, rank, world, local_rank, warmup, barrier)
        return
    for _ in range(warmup):
        out = step()
    barrier()

    # ---- device-resident timing: K steps, one event pair per step on the launching stream
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        barrier()
        for i in range(args.steps):
            starts[i].record()
            out = step()
            ends[i].record()
        barrier()
    total_ms = starts[0].elapsed_time(ends[-1])
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms_max = float(t.item())

    # status word of a launch through the C ABI (0 = consistent inputs, no bounded wait gave up)
    _, status = cabi.hstu_jagged_forward(
        kw["q"], kw["k"], kw["v"], None, kw["attn_bias"], 0, kw["max_seq_len"], 0.0, kw["seq_offset"], None,
        kw["num_target"], kw["target_group_size"], kw["alpha"], return_status=True)
    assert status == 0, f"device status word {status:#x}"

    # ---- end-to-end: pinned host inputs -> device -> operator -> pinned host result, all inside the timed region.
    # The batch goes through in chunks of whole sequences (equal token counts): chunk c+1 is copied in and chunk c-1
    # copied out while chunk c is computed, on three streams; every chunk is one call of the public operator.
    host_in = {k: v.cpu().pin_memory() for k, v in kw.items() if isinstance(v, torch.Tensor)}
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host_in.values())
    d2h = host_out.numel() * host_out.element_size()
    off_h = host_in["seq_offset"]
    nseq = off_h.numel() - 1
    nchunks = max(1, min(args.e2e_chunks, nseq))
    cuts = [0]
    for c in range(1, nchunks):
        target = int(off_h[-1]) * c // nchunks
        cuts.append(max(cuts[-1], int(torch.searchsorted(off_h, target))))
    cuts.append(nseq)
    per_seq_bias = host_in.get("attn_bias") is not None and host_in["attn_bias"].dim() == 4 \
        and host_in["attn_bias"].shape[0] == nseq
    chunks = []
    for s0, s1 in zip(cuts[:-1], cuts[1:]):
        if s1 <= s0:
            continue
        t0, t1 = int(off_h[s0]), int(off_h[s1])
        hc = {"q": host_in["q"][t0:t1], "k": host_in["k"][t0:t1], "v": host_in["v"][t0:t1],
              "seq_offset": (off_h[s0:s1 + 1] - t0).pin_memory()}
        if host_in.get("num_target") is not None:
            hc["num_target"] = host_in["num_target"][s0:s1]
        if host_in.get("attn_bias") is not None and per_seq_bias:
            hc["attn_bias"] = host_in["attn_bias"][s0:s1]
        dc = {k: torch.empty(v.shape, dtype=v.dtype, device=dev) for k, v in hc.items()}
        chunks.append((t0, t1, hc, dc))
    shared_bias_h = host_in.get("attn_bias") if not per_seq_bias else None
    shared_bias_d = torch.empty_like(shared_bias_h, device=dev) if shared_bias_h is not None else None
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def e2e_step():
        cur = torch.cuda.current_stream(dev)
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            if shared_bias_h is not None:
                shared_bias_d.copy_(shared_bias_h, non_blocking=True)
        for t0, t1, hc, dc in chunks:
            with torch.cuda.stream(s_in):
                for k, v in hc.items():
                    dc[k].copy_(v, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            cur.wait_event(ready)
            o = hj(dc["q"], dc["k"], dc["v"], None, dc.get("attn_bias", shared_bias_d), 0, kw["max_seq_len"], 0.0,
                   dc["seq_offset"], None, dc.get("num_target"), kw["target_group_size"], kw["alpha"])
            done = torch.cuda.Event()
            done.record(cur)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                host_out[t0:t1].copy_(o, non_blocking=True)
            o.record_stream(s_out)
        cur.wait_stream(s_out)
        cur.wait_stream(s_in)

    e2e_step()
    torch.cuda.synchronize(dev)
    # the chunked run gives bit-for-bit what the whole-batch, device-resident run gave
    assert torch.equal(host_out, out.cpu()), "end-to-end result differs from the device-resident result"
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / args.e2e_steps

    # ---- sustained: the same step back to back for a couple of seconds (all ranks), clocks sampled
    sus = None
    if args.sustained_seconds > 0:
        n_sus = max(args.steps, int(args.sustained_seconds * 1e3 / max(total_ms_max / args.steps, 1e-3)) + 1)
        with ClockSampler(local_rank) as sus_clocks:
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n_sus):
                step()
            e1.record()
            barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sus = (n_sus, float(t.item()), sus_clocks.summary())

    if rank == 0:
        peaks = load_peaks()
        ms_per_step = total_ms_max / args.steps
        value = full.flops() / (ms_per_step * 1e-3) / 1e12
        # roofline of the attention kernel on this rank: useful FLOPs of this rank's launch / its mean duration
        # (event pairs enclose pre-pass + attention kernel of one call; the pre-pass is a few microseconds)
        k_ms = statistics.mean(step_ms)
        achieved = mine.flops() / (k_ms * 1e-3) / 1e12
        sustained = total_ms_max > 500.0
        peak = peaks["tflops_sustained"] if sustained else peaks["tflops_burst"]
        hbm_gbs = mine.bytes() / (k_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": full.dtype, "data": "synthetic",
            "config": {
                "workload": WORKLOAD_DESC[args.workload] + (f" (first {full.batch} sequences only)" if args.max_batch else ""),
                "tokens": full.tokens, "useful_flops": full.flops(),
                "partition": f"LPT by L(L+1) over {world} rank(s); max/mean FLOPs {flop_imb:.4f}, tokens {tok_imb:.4f}",
                "l2": f"inputs+output of a step are {mine.bytes() / 1e6:.0f} MB per rank "
                      + ("(larger than the 126 MB L2; no flush)" if mine.bytes() > 2 * 126e6 else "(L2-resident: warm number)"),
            },
            "tokens_per_s": full.tokens / (ms_per_step * 1e-3),
            "frac_of_bf16_peak": value / (world * peak),
            "roofline": {
                "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": (TRAFFIC_BYTES_PER_TOKEN[args.workload] * mine.tokens
                            if args.workload in TRAFFIC_BYTES_PER_TOKEN else None),
                "peak_kind": ("sustained" if sustained else "burst") + " of " + peaks["source"],
                "kernel": "hstu_tc_kernel", "kernel_ms": k_ms, "algorithmic_flops_per_launch": mine.flops(),
                "hbm_gbs_algorithmic": hbm_gbs, "hbm_frac": hbm_gbs / peaks["hbm"],
            },
            "e2e": {"value": full.flops() / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": args.e2e_steps,
                    "chunks": len(chunks)},
            "gpu_launches": 2 * args.steps,
            "clocks": clocks.summary(),
        }
        if sus is not None:
            n_sus, sus_ms, sc = sus
            sv = full.flops() * n_sus / (sus_ms * 1e-3) / 1e12
            line["sustained"] = {
                "value": sv, "unit": UNIT, "steps": n_sus, "seconds": sus_ms * 1e-3,
                "frac": sv / (world * peaks["tflops_sustained"]), "peak": peaks["tflops_sustained"],
                "peak_kind": "sustained of " + peaks["source"], "clocks": sc,
                # what the same run would give at the maximum SM clock (the kernel is clock-bound, not memory-bound)
                "value_at_max_clock": (sv * sc["sm_max_mhz"] / sc["sm_mhz"]) if sc.get("sm_mhz") else None,
            }
        if world == 1 and not args.no_also and not args.max_batch and args.workload == "cfg4":
            del kw, out, host_in, host_out, chunks
            torch.cuda.empty_cache()
            line["also"] = run_also(ops_rec, W, dev, peaks)
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_forward_sample(full, W)
            line["cpu_baseline"] = {"value": r["tflops"], "unit": UNIT, "cores": r["cores"], "kind": r["kind"],
                                    "sample": r["desc"], "tokens_per_s": r["tokens_per_s"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
