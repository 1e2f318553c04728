"""Training-step (forward + backward) throughput of the layer on one GPU.

    python -m omni_moe_b200.train_bench [--config c2] [--steps 20] [--warmup 5] [--profile]

One step = forward of the module in training mode (batch-statistics BatchNorm) on a fixed batch and
the backward of a fixed output gradient into every parameter and the input; no optimizer.  Three
timings, CUDA events around K steps, one JSON line each:

  eager      the module called step by step (host launch cost included)
  graphed    the same step captured once in a CUDA graph and replayed
  torch      the same mathematics written with PyTorch eager ops and autograd on the same GPU
             (gather / matmul experts, torch.topk router), as the same-box bar

--profile instead prints the device time of every kernel of one eager step (torch.profiler, CUDA activity
only, averaged over five steps), largest first: the shares of the training step.

Synthetic data: x ~ N(0,1) and dy ~ N(0, 0.1) in bf16, parameters from the module's default
initialisation under seed 0.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.nn.functional as F

CONFIGS = {
    "c1": dict(T=512, H=256, I=1024, N=1024, k=8),
    "c2": dict(T=4096, H=1024, I=4096, N=4096, k=16),
}


def _time(fn, steps: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def torch_forward(m, x):
    """The layer's forward with PyTorch ops only (the structure of the reference's PyTorch module,
    omni_moe/modules/omni_moe.py:139-194): gather / matmul experts, torch.topk router."""
    t, h = x.shape[-2], x.shape[-1]
    n, k = m.num_expert_sqrt, m.top_k
    xx = x.view(t, h)
    lx = F.log_softmax(m.router_norm_x(m.router_gate_x(xx)), -1)
    ly = F.log_softmax(m.router_norm_y(m.router_gate_y(xx)), -1)
    kk = min(n, k)
    sx, ix = lx.topk(kk, -1)
    sy, iy = ly.topk(kk, -1)
    alls = (sx.unsqueeze(-1) + sy.unsqueeze(-2)).view(t, -1)
    alli = (ix.unsqueeze(-1) * n + iy.unsqueeze(-2)).view(t, -1)
    sc, pos = alls.topk(k, -1)
    ind = alli.gather(-1, pos)
    g = torch.exp(sc)
    s = torch.matmul(m.up_embed(ind), xx.unsqueeze(-1)).squeeze(-1)
    e = torch.matmul((F.silu(s) * g).unsqueeze(-2), m.down_embed(ind)).squeeze(-2)
    sh = m.down_proj(F.silu(m.gate_proj(xx)) * m.up_proj(xx))
    return sh + e


def torch_step(m, x, dy):
    """The layer's training step with PyTorch ops and autograd only."""
    torch_forward(m, x).backward(dy.view(x.shape[-2], x.shape[-1]))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", default="c2", choices=list(CONFIGS))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--profile", action="store_true", help="per-kernel device time of one eager step instead of the timings")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("train_bench needs a CUDA device")
    from .modules.omni_moe import OmniMoE, OmniMoEConfig
    c = CONFIGS[args.config]
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    m = OmniMoE(OmniMoEConfig(c["H"], c["I"], "silu", c["N"], c["k"])).to(torch.bfloat16).to(dev).train()
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(1, c["T"], c["H"], device=dev, generator=g).to(torch.bfloat16)
    dy = (torch.randn(1, c["T"], c["H"], device=dev, generator=g) * 0.1).to(torch.bfloat16)

    def report(impl, ms):
        print(json.dumps({"config": args.config, "impl": impl, "metric": "OmniMoE layer fwd+bwd tokens/s",
                          "value": round(c["T"] / (ms * 1e-3)), "unit": "tokens/s", "ms_per_step": round(ms, 4),
                          "steps": args.steps, "warmup": args.warmup, "dtype": "bf16", "data": "synthetic"}), flush=True)

    if args.profile:
        from torch.profiler import ProfilerActivity, profile

        def one_step():
            for p in m.parameters():
                p.grad = None
            m(x).backward(dy)
        for _ in range(3):
            one_step()
        torch.cuda.synchronize()
        reps = 5
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(reps):
                one_step()
            torch.cuda.synchronize()
        rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
        total = sum(e.device_time_total for e in rows) / reps
        print(f"device time per step: {total:.1f} us over {sum(e.count for e in rows) // reps} kernels / copies")
        for e in rows:
            if e.device_time_total / reps < 1.0:
                break
            print(f"{e.device_time_total / reps:8.1f} us {100 * e.device_time_total / reps / total:5.1f} %  x{e.count // reps:<3d} {e.key[:120]}")
        return

    # graphed first: whole-step capture wants gradient accumulators that were created on the capture stream
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            for p in m.parameters():
                p.grad = None
            m(x).backward(dy)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    for p in m.parameters():
        p.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        m(x).backward(dy)
    report("graphed", _time(graph.replay, args.steps, args.warmup))

    def eager():
        for p in m.parameters():
            p.grad = None
        m(x).backward(dy)
    report("eager", _time(eager, args.steps, args.warmup))

    def torch_eager():
        for p in m.parameters():
            p.grad = None
        torch_step(m, x, dy)
    report("torch", _time(torch_eager, args.steps, args.warmup))


if __name__ == "__main__":
    main()
