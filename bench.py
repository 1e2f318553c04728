#!/usr/bin/env python
"""Benchmark of the OmniMoE layer forward (tokens/s) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward of the layer over one batch of synthetic tokens.  The workload at any N
is the quick-start shape (hidden 1024, intermediate 4096, 4096 experts as a 64 x 64 grid, top-k 16,
bf16, 4096 tokens per GPU): the single-GPU configuration the headline metric is quoted on.
With N > 1 (launched with torch.distributed.run, one rank per GPU) every rank runs its own replica on
its own tokens - token data parallelism, no collective in the forward - so scaling is "weak".

Printed JSON keys (one line, rank 0):
  value      tokens/s, inputs resident in HBM, K CUDA-graph replays (independent steps, two in flight on two
             streams so that one step's kernel tails overlap the next step's heads), device-timed
  e2e        tokens/s through GraphedOmniMoE with HOST input and output buffers: every step copies
             its tokens from pinned host memory, runs the forward and copies the result back;
             steps are pipelined over independent slots; the leg runs untimed for --link-warmup seconds first
             (the host link needs traffic to leave its low-power state)
  roofline   of the dominant kernel (gate/up GEMM with the SwiGLU epilogue), timed live here
  cpu_baseline  the reference's own PyTorch layer (OmniMoE_Torch) on the host cores, N = 1 only
  config     static description of the workload, identical in both arms
  detail     measured extras: the same step one at a time, the sustained figure (the K-step block repeated for
             a second or more, median block, with the SM clock sampled meanwhile), layer_frac (algorithmic
             FLOP of the whole layer / step time / measured peak)
  partitioned_c5  the largest configuration (65536 tokens, hidden 4096, intermediate 11008, 1024 x 1024
             experts, top-k 64; strong scaling): on one GPU the whole layer, on N > 1 GPUs with the expert
             tables row-partitioned and dispatched / combined over NCCL; with the device time of its
             phases and a parity check of sampled tokens against the CPU oracle.  Its sub-record
             column_partitioned is the same step with the same tables cut by columns instead (all-to-all of
             token / state columns, all-reduce of the dot products, no host synchronisation), checked the
             same way; best_mode / best_ms_per_step name the faster of the two
Synthetic data: x ~ N(0,1), weights from the module's default initialisation under seed 0 (quick-start
shape) or N(0, 0.02) (largest configuration).

--impl reference times the reference project's own CPU implementation of the same workload (its
PyTorch module, staged unmodified under oracle/_ref by `python -m oracle.make_ref`; the restatement in
oracle/omni_oracle.py only if that folder is empty) on all host cores; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(hidden=1024, intermediate=4096, experts=4096, top_k=16, tokens=4096)
WORKLOAD = "quick-start layer: hidden 1024, intermediate 4096, 4096 experts (64x64), top-k 16, x bf16 [1,4096,1024]"
SLOTS = 4  # independent weight + activation sets rotated between steps (working set > L2)
RESIDENT_STREAMS = 2  # steps in flight: the tail of one step's kernels overlaps the head of the next one's
C5 = dict(T=65536, H=4096, I=11008, N=1 << 20, k=64)

# DRAM bytes (read + write) per launch of the gate/up GEMM kernel: ncu, one launch of this workload
# (25.26 MB read + 1.27 MB written)
GATE_UP_DRAM_BYTES_PER_LAUNCH = 26_528_768


def static_config(world: int) -> dict:
    """Description of the workload; the same dictionary in both arms."""
    return {"workload": WORKLOAD, "tokens_per_gpu_per_step": CFG["tokens"], "parallelism": f"token-dp{world}",
            "l2": f"GPU arm: {SLOTS} independent weight+activation sets rotated between steps (about 130 MB each, > 126 MB L2 in total)",
            "launch": f"GPU arm: one CUDA graph per step, {RESIDENT_STREAMS} independent steps in flight (round-robin over {RESIDENT_STREAMS} streams)"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tf=p["bf16_tflops"], tf_sustained=p.get("bf16_tflops_sustained"), src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, src="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25", "-i",
                 str(self.index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.file.flush()
        rows = [r.strip().split(", ") for r in open(self.file.name) if r.strip()]
        os.unlink(self.file.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for nm, v in zip(names, r[2:6]):
                if v.strip().lower() == "active":
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_slots(dev):
    from omni_moe_b200.modules.omni_moe import OmniMoE, OmniMoEConfig
    slots = []
    for s in range(SLOTS):
        torch.manual_seed(s)  # slot 0 = seed 0, the named configuration; the others only differ in values
        m = OmniMoE(OmniMoEConfig(CFG["hidden"], CFG["intermediate"], "silu", CFG["experts"], CFG["top_k"]))
        m = m.to(torch.bfloat16).to(dev).eval()
        g = m.graphed(CFG["tokens"], dev)
        x_host = torch.randn(CFG["tokens"], CFG["hidden"], generator=torch.Generator().manual_seed(100 + s))
        x_host = x_host.to(torch.bfloat16).pin_memory()
        y_host = torch.empty_like(x_host).pin_memory()
        g.x.copy_(x_host)
        slots.append(dict(module=m, graph=g, x_host=x_host, y_host=y_host, stream=torch.cuda.Stream(device=dev)))
    torch.cuda.synchronize()
    return slots


def barrier(dist_on):
    torch.cuda.synchronize()
    if dist_on:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, dist_on: bool, dev) -> float:
    if not dist_on:
        return ms
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def time_resident(slots, steps, warmup, dist_on, dev, n_streams=RESIDENT_STREAMS, sustain_s: float = 0.0):
    """K graph replays, rotating the slots, issued round-robin on n_streams streams (independent
    steps, as a server with several batches in flight runs them); CUDA events on the main stream, which
    forks to and joins the replay streams, around the lot.  Returns (ms of the first K-step block, list of
    the ms of the further identical blocks issued back to back until `sustain_s` seconds have passed)."""
    streams = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]
    for i in range(warmup):
        slots[i % SLOTS]["graph"].replay()
    barrier(dist_on)
    main = torch.cuda.current_stream()

    def block():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        for s in streams:
            s.wait_event(e0)
        for i in range(steps):
            with torch.cuda.stream(streams[i % n_streams]):
                slots[i % SLOTS]["graph"].replay()
        for s in streams:
            main.wait_stream(s)
        e1.record(main)
        return e0, e1

    first = block()
    barrier(dist_on)
    first_ms = max_over_ranks(first[0].elapsed_time(first[1]), dist_on, dev)
    later = []
    if sustain_s > 0:
        t0 = time.perf_counter()
        pending = []
        while time.perf_counter() - t0 < sustain_s or len(pending) < 3:
            pending.append(block())
            if len(pending) % 8 == 0:
                pending[-8][1].synchronize()   # keep the host at most a few blocks ahead of the device
        barrier(dist_on)
        later = [a.elapsed_time(b) for a, b in pending]
    return first_ms, later


def time_e2e(slots, steps, warmup, dist_on, dev, link_warmup_s=0.1):
    """Host buffers in and out every step; slot s runs on its own stream so that the copies of one
    step overlap the kernels of another."""
    def step(i):
        s = slots[i % SLOTS]
        with torch.cuda.stream(s["stream"]):
            s["graph"].x.copy_(s["x_host"], non_blocking=True)
            s["graph"].replay()
            s["y_host"].copy_(s["graph"].y, non_blocking=True)

    # The host link idles while the resident legs run and needs some tens of milliseconds of traffic to leave its
    # low-power state (a bare copy loop on these boxes: 36 GB/s over its first 100 copies of 8 MiB, 54 GB/s after).
    # A serving process is in that steady state, so the same steps run untimed for LINK_WARMUP_S first.
    link_steps, t0 = 0, time.perf_counter()
    while link_warmup_s > 0 and time.perf_counter() - t0 < link_warmup_s:
        for i in range(SLOTS):
            step(i)
        link_steps += SLOTS
        slots[0]["stream"].synchronize()
    for i in range(warmup):
        step(i)
    barrier(dist_on)
    main = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(main)
    for s in slots:
        s["stream"].wait_event(e0)
    for i in range(steps):
        step(i)
    for s in slots:
        main.wait_stream(s["stream"])
    e1.record(main)
    barrier(dist_on)
    return max_over_ranks(e0.elapsed_time(e1), dist_on, dev), link_steps


def time_gate_up(slots, reps):
    """Average duration of the dominant kernel alone: `SLOTS` launches (one per weight set) captured in a
    CUDA graph so that host launch cost does not count, replays timed with CUDA events on the replay
    stream."""
    from omni_moe_b200 import _lib
    lib = _lib.load()
    t, h, i = CFG["tokens"], CFG["hidden"], CFG["intermediate"]

    def launch(s, stream_ptr):
        m, b, g = s["module"], s["graph"].buffers, s["graph"]
        _lib.check(lib.omni_mlp_gate_up(g.x.data_ptr(), m.gate_proj.weight.data_ptr(), m.up_proj.weight.data_ptr(), t, h, i,
                                        b.act.data_ptr(), b.status.data_ptr(), stream_ptr))
    for s in slots:
        launch(s, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for s in slots:
                launch(s, side.cuda_stream)
    torch.cuda.synchronize()
    times = []
    for _ in range(max(reps // SLOTS, 3)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / SLOTS)
    return statistics.mean(times)


def _workload_inputs():
    """x of slot 0 of the workload, as the GPU arm draws it."""
    return torch.randn(1, CFG["tokens"], CFG["hidden"], generator=torch.Generator().manual_seed(100)).to(torch.bfloat16)


def _cpu_forward_fn(dtype=torch.bfloat16):
    """A callable running one forward of the whole workload on the CPU, and what it is.

    First choice: the reference project's own PyTorch module (OmniMoE_Torch, omni_moe/modules/omni_moe.py:109-194),
    loaded unmodified from oracle/_ref, built as the quick-start snippet builds it (default initialisation under
    seed 0, then .to(bfloat16)) and fed the bf16 tokens.  Fallback when oracle/_ref is empty: the fp32
    restatement in oracle/omni_oracle.py on bf16-rounded parameters."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = _workload_inputs()
    from oracle import ref_loader
    ref = ref_loader.load_layer()
    if ref is not None:
        ref_layer, ref_config = ref
        torch.manual_seed(0)
        m = ref_layer(ref_config(CFG["hidden"], CFG["intermediate"], "silu", CFG["experts"], CFG["top_k"]))
        m = m.to(dtype).eval()
        xd = x.to(dtype)
        name = "bf16" if dtype == torch.bfloat16 else "f32"
        return (lambda: m(xd)), "reference", name, cores, f"OmniMoE_Torch of the reference project (unmodified file), module and tokens in {name}"
    from oracle import omni_oracle as orc
    from omni_moe_b200.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(0)
    m = OmniMoE(OmniMoEConfig(CFG["hidden"], CFG["intermediate"], "silu", CFG["experts"], CFG["top_k"]))
    sd = {k: v.detach().to(torch.bfloat16).float() if v.is_floating_point() else v for k, v in m.state_dict().items()}
    prm = orc.params_from_state_dict(sd, CFG["experts"], CFG["top_k"])
    xf = x.float()
    return (lambda: orc.layer_forward(prm, xf)), "port", "f32", cores, "restatement of OmniMoE_Torch (oracle/omni_oracle.py), fp32 math on bf16-rounded parameters"


def cpu_baseline_rate(seconds_budget: float = 12.0):
    """tokens/s of the CPU path over whole-workload forwards for about `seconds_budget` seconds, all host threads."""
    fwd, kind, dtype, cores, what = _cpu_forward_fn()
    with torch.no_grad():
        fwd()  # warm-up
        n, t0 = 0, time.perf_counter()
        while True:
            fwd()
            n += 1
            el = time.perf_counter() - t0
            if el > seconds_budget or n >= 100:
                break
    out = {"value": CFG["tokens"] * n / el, "unit": "tokens/s", "cores": cores, "kind": kind, "dtype": dtype,
           "sample": f"{n} forwards of the whole workload ({CFG['tokens']} tokens each) in {el:.1f} s; {what}"}
    if kind == "reference":
        # the same module in float32 (the precision the parity oracle computes in), a few forwards for the record
        fwd32 = _cpu_forward_fn(torch.float32)[0]
        with torch.no_grad():
            fwd32()
            n32, t0 = 0, time.perf_counter()
            while n32 < 20:
                fwd32()
                n32 += 1
                el32 = time.perf_counter() - t0
                if el32 > 4.0:
                    break
        out["float32"] = {"value": CFG["tokens"] * n32 / el32, "unit": "tokens/s",
                          "sample": f"{n32} forwards in {el32:.1f} s, module and tokens in float32"}
    return out


def run_reference(args, rank):
    """The reference's CPU implementation of the path on the host cores; rank 0 only.  Every step is one
    forward over the whole workload (4096 tokens).  If the requested number of steps would take more than
    about two and a half minutes on this host, fewer steps are run and the line says so."""
    if rank != 0:
        return
    fwd, kind, dtype, cores, what = _cpu_forward_fn()
    steps, warmup, note = args.steps, args.warmup, ""
    with torch.no_grad():
        fwd()
        t0 = time.perf_counter()
        fwd()
        d = time.perf_counter() - t0
        if (steps + warmup) * d > 150.0:
            warmup = min(warmup, 3)
            steps = max(3, int(150.0 / d) - warmup)
            note = f"; {steps} steps instead of {args.steps} to stay within the time budget ({d:.2f} s per step on this host)"
        for _ in range(warmup):
            fwd()
        t0 = time.perf_counter()
        for _ in range(steps):
            fwd()
        el = time.perf_counter() - t0
    v = CFG["tokens"] * steps / el
    line = {
        "impl": "reference", "metric": "OmniMoE layer fwd tokens/s", "value": v, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": 1e3 * el / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": static_config(args.gpus),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": kind, "dtype": dtype,
                         "sample": f"each step = one forward over the whole workload ({CFG['tokens']} tokens); {what}{note}"},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# largest configuration: one GPU, or expert tables row-partitioned over the ranks
# ------------------------------------------------------------------------------------------------
def _c5_parity(inner, tables, part, x_local, y_local, indices, rank, world, dist_on, dev, samples_total=256):
    """Sampled tokens of the step against the CPU oracle.  Every rank contributes `samples_total / world`
    of its tokens (rows of x, y and the selected expert ids); rank 0 reruns the router on the CPU, asks
    every rank for the table rows the sampled tokens touch (a rank fills in the rows it owns, the rest stay
    zero, a sum-reduce assembles them), and recomputes the outputs in fp32."""
    import numpy as np
    import torch.distributed as dist
    from oracle import omni_oracle as orc
    t_local, h = x_local.shape
    k, n = inner.top_k, inner.num_expert_sqrt
    per = max(1, -(-samples_total // world))
    pick = torch.linspace(0, t_local - 1, per, device=dev).long()
    xs, ys, gi = x_local[pick].contiguous(), y_local.reshape(-1, h)[pick].contiguous(), indices[pick].contiguous()
    if dist_on:
        def gather(t):
            out = torch.empty((world * t.size(0),) + tuple(t.shape[1:]), device=dev, dtype=t.dtype)
            dist.all_gather_into_tensor(out, t)
            return out
        xs, ys, gi = gather(xs), gather(ys), gather(gi)
    s_total = xs.size(0)
    lpx = lpy = es = ei = None
    if rank == 0:
        # the launcher pins every rank to one OpenMP thread; the check below is a few dozen GFLOP on the host
        torch.set_num_threads(max(1, min(16, (os.cpu_count() or 1) // max(world, 1))))
        xf = xs.float().cpu()
        sd = {kk: v.detach().float().cpu() for kk, v in inner.state_dict().items() if "embed" not in kk}
        lpx = orc.router_log_probs(orc.router_batchnorm_eval(orc.router_logits(xf, sd["router_gate_x.weight"]),
                                                             sd["router_norm_x.running_mean"], sd["router_norm_x.running_var"]))
        lpy = orc.router_log_probs(orc.router_batchnorm_eval(orc.router_logits(xf, sd["router_gate_y.weight"]),
                                                             sd["router_norm_y.running_mean"], sd["router_norm_y.running_var"]))
        es, ei = orc.router_topk(lpx, lpy, n, k)
        need = torch.unique(torch.cat([torch.from_numpy(ei).reshape(-1), gi.reshape(-1).long().cpu()]))
        need = need[(need >= 0) & (need < inner.num_experts)].to(dev)
        count = torch.tensor([need.numel()], device=dev)
    else:
        count = torch.zeros(1, dtype=torch.long, device=dev)
    if dist_on:
        dist.broadcast(count, 0)
        if rank != 0:
            need = torch.empty(int(count.item()), dtype=torch.long, device=dev)
        dist.broadcast(need, 0)
    up_l, down_l = tables
    by_columns = part is not None and hasattr(part, "width")
    lo, hi = (part.lo, part.hi) if part is not None else (0, inner.num_experts)
    mine = (need >= lo) & (need < hi)
    rows = []
    for tab in (up_l, down_l):
        r = torch.zeros((need.numel(), h), device=dev, dtype=torch.float32)
        if by_columns:
            r[:, lo:hi] = tab[need].float()        # every rank holds its columns of every row
        else:
            r[mine] = tab[need[mine] - lo].float()
        if dist_on:
            dist.reduce(r, 0, op=dist.ReduceOp.SUM)
        rows.append(r)
    if rank != 0:
        return None
    up_rows, down_rows = (r.cpu() for r in rows)
    need_c = need.cpu()
    compact = torch.searchsorted(need_c, torch.from_numpy(ei).reshape(-1)).view(s_total, k)
    ey = orc.expert_forward(xf, up_rows, down_rows, orc.routing_weights(es), compact)
    ey += orc.mlp_forward(xf, sd["gate_proj.weight"], sd["up_proj.weight"], sd["down_proj.weight"])
    gi_c = gi.cpu()
    ndiff, gaps = orc.routing_flip_gaps(lpx, lpy, es, ei, gi_c, n)
    same = (gi_c.long().numpy() == ei).all(axis=1)
    a, e = ys.float().cpu()[same], ey[same]
    err = (a - e).abs()
    within = bool((err <= 2e-2 + 2e-2 * e.abs()).all()) if same.any() else False
    return {"tokens_checked": int(s_total), "tokens_compared": int(same.sum()),
            "routing_mismatch_frac": float(ndiff) / float(s_total * k),
            "max_flip_gap": float(gaps.max()) if ndiff else 0.0,
            "max_abs_err": float(err.max()) if same.any() else None,
            "within_rtol2e-2_atol2e-2": within,
            "oracle": "oracle/omni_oracle.py, fp32 on the bf16 operands; rows fetched from the ranks that own them"}


def run_c5(world, rank, dev, dist_on, steps=5, warmup=2):
    """One GPU: the whole layer.  N > 1: tokens sharded (65536 / N per rank), tables row-partitioned."""
    from omni_moe_b200.layer_bench import build_module, _fill_normal_
    cfg = C5
    t_local = cfg["T"] // world
    x = torch.empty(1, t_local, cfg["H"], device=dev, dtype=torch.bfloat16)
    _fill_normal_(x, 1.0, 7 + rank)
    part = None
    if dist_on:
        from omni_moe_b200.parallel import ExpertPartition, PartitionedOmniMoE
        part = ExpertPartition(cfg["N"], world, rank)
        inner = build_module(cfg, dev, table_rows=part.hi - part.lo, row_offset=part.lo)
        layer = PartitionedOmniMoE(inner, None, table_slices=(inner.up_embed.weight.data, inner.down_embed.weight.data))
        tables = (layer.up_local.data, layer.down_local.data)
        run = lambda: layer(x)
    else:
        inner = build_module(cfg, dev)
        layer = None
        tables = (inner.up_embed.weight.data, inner.down_embed.weight.data)
        run = lambda: inner(x)
    with torch.no_grad():
        for _ in range(warmup):
            y = run()
        inner.check_status()
        barrier(dist_on)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            y = run()
        e1.record()
        barrier(dist_on)
        ms = max_over_ranks(e0.elapsed_time(e1) / steps, dist_on, dev)
        phases = None
        if layer is not None:
            layer.record_phases = True
            y = run()
            phases = layer.phases_ms()
            layer.record_phases = False
        inner.check_status()
        parity = _c5_parity(inner, tables, part, x.view(t_local, cfg["H"]), y, inner.last_routing[1], rank, world, dist_on, dev)
    out = {"workload": "largest configuration: 65536 tokens, hidden 4096, intermediate 11008, 1048576 experts (1024x1024), top-k 64, bf16",
           "mode": f"expert tables row-partitioned over {world} GPUs, NCCL dispatch / combine" if dist_on else "whole layer on one GPU",
           "scaling": "strong", "ms_per_step": ms, "tokens_s": cfg["T"] / (ms * 1e-3), "steps": steps, "warmup": warmup,
           "tables_gib_per_gpu": 2 * tables[0].numel() * 2 / 2 ** 30, "phases_ms": phases, "parity": parity}
    if dist_on and cfg["H"] % world == 0:
        # the same tables cut by columns instead of rows (same memory per GPU): partial dot products all-reduced, state
        # columns returned by an all-to-all, no host synchronisation in the step
        from omni_moe_b200.parallel import ColumnPartitionedOmniMoE, columns_from_row_slices
        up_cols = columns_from_row_slices(tables[0])
        down_cols = columns_from_row_slices(tables[1])
        del layer, tables
        torch.cuda.empty_cache()
        col = ColumnPartitionedOmniMoE(inner, None, table_slices=(up_cols, down_cols))
        with torch.no_grad():
            for _ in range(warmup):
                y = col(x)
            inner.check_status()
            barrier(dist_on)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                y = col(x)
            e1.record()
            barrier(dist_on)
            ms_c = max_over_ranks(e0.elapsed_time(e1) / steps, dist_on, dev)
            col.record_phases = True
            y = col(x)
            phases_c = col.phases_ms()
            col.record_phases = False
            inner.check_status()
            parity_c = _c5_parity(inner, (col.up_cols.data, col.down_cols.data), col.part, x.view(t_local, cfg["H"]), y,
                                  inner.last_routing[1], rank, world, dist_on, dev)
        out["column_partitioned"] = {
            "mode": f"the same tables cut by columns over {world} GPUs: all-to-all of token / state columns, all-reduce of the dot products",
            "ms_per_step": ms_c, "tokens_s": cfg["T"] / (ms_c * 1e-3), "tables_gib_per_gpu": 2 * up_cols.numel() * 2 / 2 ** 30,
            "phases_ms": phases_c, "parity": parity_c}
        out["best_mode"] = "column_partitioned" if ms_c < ms else "row_partitioned"
        out["best_ms_per_step"] = min(ms, ms_c)
        out["best_tokens_s"] = cfg["T"] / (min(ms, ms_c) * 1e-3)
        del col, up_cols, down_cols
        layer = tables = None
    del layer, inner, tables, x, y
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--link-warmup", type=float, default=0.1,
                    help="seconds of untimed end-to-end steps before the e2e leg's warm-up (0 = none)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-c5", action="store_true", help="skip the largest-configuration leg")
    ap.add_argument("--sustain", type=float, default=1.0, help="seconds of back-to-back blocks for the sustained figure")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist_on = world > 1
    if dist_on:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=dev)

    cpu_line = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        # first, while the process may still run on every host core (the placement below narrows that)
        cpu_line = cpu_baseline_rate()
    from omni_moe_b200.host import bind_near_gpu
    placement = bind_near_gpu(local_rank)   # before the pinned host buffers are allocated
    slots = build_slots(dev)
    from omni_moe_b200.modules.omni_moe import OmniMoE
    ms, _ = time_resident(slots, args.steps, args.warmup, dist_on, dev)
    ms_serial, _ = time_resident(slots, args.steps, args.warmup, dist_on, dev, n_streams=1)   # one step at a time, for the record
    ms_e2e, link_steps = time_e2e(slots, args.steps, args.warmup, dist_on, dev, args.link_warmup)
    # sustained: the same K-step block back to back for a second or more, clocks sampled meanwhile
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _, later = time_resident(slots, args.steps, 3, dist_on, dev, sustain_s=args.sustain)
    clocks = sampler.stop() if rank == 0 else None
    sustained_ms = max_over_ranks(statistics.median(later), dist_on, dev)
    for s in slots:
        s["module"].check_status()
    gemm_ms = time_gate_up(slots, 40)
    del slots
    torch.cuda.empty_cache()
    c5 = None
    if not args.no_c5:
        c5 = run_c5(world, rank, dev, dist_on)

    if rank == 0:
        pk = peaks()
        tokens_total = CFG["tokens"] * args.steps * world
        flops = 4.0 * CFG["tokens"] * CFG["hidden"] * CFG["intermediate"]
        achieved = flops / (gemm_ms * 1e-3) / 1e12
        t_, h_, i_, k_ = CFG["tokens"], CFG["hidden"], CFG["intermediate"], CFG["top_k"]
        n_ = int(math.isqrt(CFG["experts"]))
        layer_flops = 6.0 * t_ * h_ * i_ + 4.0 * t_ * h_ * n_ + 4.0 * t_ * k_ * h_   # MLP + router gates + routed experts
        step_ms = ms / args.steps
        line = {
            "metric": "OmniMoE layer fwd tokens/s", "value": tokens_total / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": static_config(world),
            "detail": {
                "one_step_at_a_time_ms_per_step": ms_serial / args.steps,
                "sustained_ms_per_step": sustained_ms / args.steps,
                "sustained_tokens_s": CFG["tokens"] * world / (sustained_ms / args.steps * 1e-3),
                "sustained_blocks": len(later), "sustained_seconds": sum(later) * 1e-3,
                "sustained_sm_mhz_median": clocks["sm_mhz"] if clocks else None,
                "layer_flops_per_step": layer_flops,
                "layer_frac": layer_flops / (step_ms * 1e-3) / 1e12 / pk["tf"],
                "layer_frac_sustained": (layer_flops / (sustained_ms / args.steps * 1e-3) / 1e12 / pk["tf_sustained"]) if pk["tf_sustained"] else None,
                "layer_frac_note": "algorithmic FLOP of one step (6THI + 4TH sqrtN + 4TkH) / step time / measured bf16 peak "
                                   "(burst peak for the first block, sustained peak for the sustained blocks)",
            },
            "e2e": {"value": tokens_total / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": CFG["tokens"] * CFG["hidden"] * 2, "d2h_bytes_per_step": CFG["tokens"] * CFG["hidden"] * 2,
                    "ms_per_step": ms_e2e / args.steps, "pipeline": f"{SLOTS} slots, one stream each",
                    "link_warmup": f"{link_steps} untimed steps of the same pipeline ({args.link_warmup:.2f} s) before the {args.warmup} warm-up steps: "
                                   "the host link needs traffic to leave its low-power state",
                    "host_placement": placement["reason"]},
            "gpu_launches": OmniMoE.kernels_per_forward(CFG["experts"], CFG["hidden"], 64, CFG["top_k"]) * args.steps,
            "clocks": clocks,
            "roofline": {"kernel": "gemm_pair_kernel<EPI_SWIGLU> (gate/up projections + SwiGLU, tcgen05 cta_group::2)", "bound": "tensor",
                         "achieved": achieved, "peak": pk["tf"], "unit": "TFLOP/s", "frac": achieved / pk["tf"],
                         "traffic": GATE_UP_DRAM_BYTES_PER_LAUNCH, "peak_source": pk["src"] + " (burst: kernel timed alone)",
                         "ms_per_launch": gemm_ms, "flops_per_launch": flops},
            "partitioned_c5": c5,
        }
        if cpu_line is not None:
            line["cpu_baseline"] = cpu_line
        print(json.dumps(line), flush=True)
    if dist_on:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
