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
             steps are pipelined over independent slots
  roofline   of the dominant kernel (gate/up GEMM with the SwiGLU epilogue), timed live here
  cpu_baseline  the CPU oracle (a restatement of the reference's PyTorch path) on the host cores
Synthetic data: x ~ N(0,1), weights from the module's default initialisation under seed 0.
"""
from __future__ import annotations

import argparse
import json
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

# DRAM bytes (read + write) per launch of the gate/up GEMM kernel, from the ncu capture summarised
# in profiles/gemm_pair_gate_up_quickstart.md (25.26 MB read + 1.27 MB written)
GATE_UP_DRAM_BYTES_PER_LAUNCH = 26_528_768


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


RESIDENT_STREAMS = 2  # steps in flight: the tail of one step's kernels overlaps the head of the next one's


def time_resident(slots, steps, warmup, dist_on, dev, n_streams=RESIDENT_STREAMS):
    """K graph replays, rotating the slots, issued round-robin on n_streams streams (independent
    steps, as a server with several batches in flight runs them); CUDA events on the main stream, which
    forks to and joins the replay streams, around the lot."""
    streams = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]
    for i in range(warmup):
        slots[i % SLOTS]["graph"].replay()
    barrier(dist_on)
    main = torch.cuda.current_stream()
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
    barrier(dist_on)
    return max_over_ranks(e0.elapsed_time(e1), dist_on, dev)


def time_e2e(slots, steps, warmup, dist_on, dev):
    """Host buffers in and out every step; slot s runs on its own stream so that the copies of one
    step overlap the kernels of another."""
    def step(i):
        s = slots[i % SLOTS]
        with torch.cuda.stream(s["stream"]):
            s["graph"].x.copy_(s["x_host"], non_blocking=True)
            s["graph"].replay()
            s["y_host"].copy_(s["graph"].y, non_blocking=True)

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
    return max_over_ranks(e0.elapsed_time(e1), dist_on, dev)


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


def _oracle_setup(sample_tokens: int):
    from oracle import omni_oracle as orc
    from omni_moe_b200.modules.omni_moe import OmniMoE, OmniMoEConfig
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    torch.manual_seed(0)
    m = OmniMoE(OmniMoEConfig(CFG["hidden"], CFG["intermediate"], "silu", CFG["experts"], CFG["top_k"]))
    sd = {k: v.detach().to(torch.bfloat16).float() if v.is_floating_point() else v for k, v in m.state_dict().items()}
    p = orc.params_from_state_dict(sd, CFG["experts"], CFG["top_k"])
    x = torch.randn(1, sample_tokens, CFG["hidden"], generator=torch.Generator().manual_seed(100)).bfloat16().float()
    return orc, p, x, cores


def cpu_oracle_rate(seconds_budget: float = 15.0, sample_tokens: int = 1024):
    """tokens/s of the CPU oracle on a bounded sample of the workload, all host threads."""
    orc, p, x, cores = _oracle_setup(sample_tokens)
    with torch.no_grad():
        orc.layer_forward(p, x)  # warm-up
        n, t0 = 0, time.perf_counter()
        while True:
            orc.layer_forward(p, x)
            n += 1
            el = time.perf_counter() - t0
            if el > seconds_budget or n >= 50:
                break
    return sample_tokens * n / el, cores, (f"{n} forwards of the first {sample_tokens} tokens of the workload, "
                                           "fp32 math on bf16-rounded parameters")


def run_reference(args, rank):
    """The reference's CPU implementation of the path: its PyTorch layer, restated in oracle/ (the
    reference package itself cannot be imported without Triton and a GPU).  Rank 0 only.  A step is
    one forward over a bounded sample of the workload's tokens, sized so the run ends in ~2 minutes."""
    if rank != 0:
        return
    sample = 512
    orc, p, x, cores = _oracle_setup(sample)
    with torch.no_grad():
        orc.layer_forward(p, x)
        t0 = time.perf_counter()
        orc.layer_forward(p, x)
        d = time.perf_counter() - t0
        total = args.steps + args.warmup
        if total * d > 120.0:
            sample = int(max(32, min(512, sample * 120.0 / (total * d))))
            x = x[:, :sample].contiguous()
        for _ in range(args.warmup):
            orc.layer_forward(p, x)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            orc.layer_forward(p, x)
        el = time.perf_counter() - t0
    v = sample * args.steps / el
    note = f"each step = one forward over the first {sample} tokens of the workload, fp32 math on bf16-rounded parameters"
    line = {
        "impl": "reference", "metric": "OmniMoE layer fwd tokens/s", "value": v, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * el / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample_tokens_per_step": sample},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": note},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
        rate, cores, sample = cpu_oracle_rate()
        cpu_line = {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    from omni_moe_b200.host import bind_near_gpu
    placement = bind_near_gpu(local_rank)   # before the pinned host buffers are allocated
    slots = build_slots(dev)
    from omni_moe_b200.modules.omni_moe import OmniMoE
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = time_resident(slots, args.steps, args.warmup, dist_on, dev)
    ms_serial = time_resident(slots, args.steps, args.warmup, dist_on, dev, n_streams=1)   # one step at a time, for the record
    ms_e2e = time_e2e(slots, args.steps, args.warmup, dist_on, dev)
    clocks = sampler.stop() if rank == 0 else None
    for s in slots:
        s["module"].check_status()
    gemm_ms = time_gate_up(slots, 40)

    if rank == 0:
        pk = peaks()
        tokens_total = CFG["tokens"] * args.steps * world
        flops = 4.0 * CFG["tokens"] * CFG["hidden"] * CFG["intermediate"]
        achieved = flops / (gemm_ms * 1e-3) / 1e12
        line = {
            "metric": "OmniMoE layer fwd tokens/s", "value": tokens_total / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu_per_step": CFG["tokens"], "parallelism": f"token-dp{world}",
                       "l2": f"{SLOTS} independent weight+activation sets rotated between steps (about 130 MB each, > 126 MB L2 in total)",
                       "one_step_at_a_time_ms_per_step": ms_serial / args.steps,
                       "launch": f"one CUDA graph per step, {RESIDENT_STREAMS} independent steps in flight (round-robin over {RESIDENT_STREAMS} streams)"},
            "e2e": {"value": tokens_total / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": CFG["tokens"] * CFG["hidden"] * 2, "d2h_bytes_per_step": CFG["tokens"] * CFG["hidden"] * 2,
                    "ms_per_step": ms_e2e / args.steps, "pipeline": f"{SLOTS} slots, one stream each",
                    "host_placement": placement["reason"]},
            "gpu_launches": OmniMoE.kernels_per_forward(CFG["experts"], CFG["hidden"], 64, CFG["top_k"]) * args.steps,
            "clocks": clocks,
            "roofline": {"kernel": "gemm_pair_kernel<EPI_SWIGLU> (gate/up projections + SwiGLU, tcgen05 cta_group::2)", "bound": "tensor",
                         "achieved": achieved, "peak": pk["tf"], "unit": "TFLOP/s", "frac": achieved / pk["tf"],
                         "traffic": GATE_UP_DRAM_BYTES_PER_LAUNCH, "peak_source": pk["src"] + " (burst: kernel timed alone)",
                         "ms_per_launch": gemm_ms, "flops_per_launch": flops},
        }
        if cpu_line is not None:
            line["cpu_baseline"] = cpu_line
        print(json.dumps(line), flush=True)
    if dist_on:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
