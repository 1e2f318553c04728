"""Whole-layer forward throughput of a named configuration, on one GPU or with the expert tables
row-partitioned over the GPUs of one node.

    python -m omni_moe_b200.layer_bench --config c5                       # one GPU, whole layer
    python -m omni_moe_b200.layer_bench --config c2 --impl torch          # same-box bar: PyTorch eager ops, same GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m omni_moe_b200.layer_bench --config c5 --partitioned            # tables split over N GPUs

Configurations: c2 (T 4096, H 1024, I 4096, 64x64 experts, k 16) and c5 (T 65536, H 4096, I 11008,
1024x1024 experts, k 64; 16 GiB of tables).  Synthetic data: x ~ N(0,1), all weights ~ N(0, 0.02) as the
large-table configuration specifies, BatchNorm with default running statistics, eval mode.
With --partitioned the T tokens are sharded evenly over the ranks (strong scaling: the job is the
same T tokens at every N) and rank g holds rows [g N/G, (g+1) N/G) of the tables (--columns: columns
[g H/G, (g+1) H/G) of every row).
Steps are timed with CUDA events between barriers; the maximum over ranks is reported by rank 0 as
one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

CONFIGS = {
    "c2": dict(T=4096, H=1024, I=4096, N=4096, k=16),
    "c5": dict(T=65536, H=4096, I=11008, N=1 << 20, k=64),
}


def _fill_normal_(t: torch.Tensor, std: float, seed: int):
    g = torch.Generator(device=t.device).manual_seed(seed)
    flat = t.view(-1)
    step = 1 << 26
    for s in range(0, flat.numel(), step):
        e = min(flat.numel(), s + step)
        flat[s:e] = (torch.randn(e - s, device=t.device, generator=g) * std).to(t.dtype)


def build_module(cfg, dev, table_rows=None, row_offset=0):
    """The layer with weights ~ N(0, 0.02), built directly on the device.  `table_rows` < N builds only a
    slice of the expert tables (rows row_offset ... row_offset + table_rows), for the partitioned run."""
    from .modules.omni_moe import OmniMoE, OmniMoEConfig
    with torch.device("meta"):
        m = OmniMoE(OmniMoEConfig(cfg["H"], cfg["I"], "silu", cfg["N"], cfg["k"]))
    m = m.to_empty(device=dev).to(torch.bfloat16)
    rows = cfg["N"] if table_rows is None else table_rows
    if rows != cfg["N"]:
        m.up_embed.weight = torch.nn.Parameter(torch.empty(rows, cfg["H"], device=dev, dtype=torch.bfloat16), requires_grad=False)
        m.down_embed.weight = torch.nn.Parameter(torch.empty(rows, cfg["H"], device=dev, dtype=torch.bfloat16), requires_grad=False)
    for i, (name, p) in enumerate(sorted(m.named_parameters())):
        # the table slices draw from a seed that depends on the slice, everything else is replicated
        seed = 1000 + i + (row_offset if "embed" in name else 0)
        _fill_normal_(p.data, 0.02, seed)
    for bn in (m.router_norm_x, m.router_norm_y):
        bn.running_mean.zero_()
        bn.running_var.fill_(1.0)
        bn.num_batches_tracked.zero_()
    return m.eval()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", default="c5", choices=list(CONFIGS))
    ap.add_argument("--partitioned", action="store_true")
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"],
                    help="torch: the same layer written with PyTorch eager ops (gather / matmul experts, torch.topk "
                         "router) on the same GPU, as a same-box bar; c2 only (it materialises [T, k, H] gathers)")
    ap.add_argument("--chunks", type=int, default=2, help="token ranges pipelined through the exchange (--partitioned)")
    ap.add_argument("--columns", action="store_true", help="with --partitioned: cut the tables by columns instead of rows")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1 or args.partitioned:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    assert cfg["T"] % world == 0
    t_local = cfg["T"] // world if args.partitioned else cfg["T"]
    x = torch.empty(1, t_local, cfg["H"], device=dev, dtype=torch.bfloat16)
    _fill_normal_(x, 1.0, 7 + rank)

    if args.partitioned:
        from .parallel import ExpertPartition, PartitionedOmniMoE
        part = ExpertPartition(cfg["N"], world, rank)
        inner = build_module(cfg, dev, table_rows=part.hi - part.lo, row_offset=part.lo)
        # the tables were built as slices in the first place: 16 GiB of rows never exist on one GPU
        if args.columns:
            from .parallel import ColumnPartitionedOmniMoE, columns_from_row_slices
            up_cols = columns_from_row_slices(inner.up_embed.weight.data)
            down_cols = columns_from_row_slices(inner.down_embed.weight.data)
            layer = ColumnPartitionedOmniMoE(inner, None, table_slices=(up_cols, down_cols))
        else:
            layer = PartitionedOmniMoE(inner, None, chunks=args.chunks,
                                       table_slices=(inner.up_embed.weight.data, inner.down_embed.weight.data))
        run = lambda: layer(x)
    elif args.impl == "torch":
        from .train_bench import torch_forward
        inner = build_module(cfg, dev)
        run = lambda: torch_forward(inner, x)
    else:
        inner = build_module(cfg, dev)
        run = lambda: inner(x)

    def sync():
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        for _ in range(max(args.warmup, 1)):
            y = run()
        inner.check_status()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            y = run()
        e1.record()
        sync()
    ms = e0.elapsed_time(e1) / args.steps
    if dist.is_initialized():
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    inner.check_status()
    assert bool(torch.isfinite(y.float()).all())
    phases = None
    if args.partitioned:
        with torch.no_grad():
            layer.record_phases = True
            run()
            phases = layer.phases_ms()
            layer.record_phases = False
    if rank == 0:
        tokens = cfg["T"] if args.partitioned else cfg["T"] * world
        print(json.dumps({
            "config": args.config, "impl": args.impl, "mode": ("tables column-partitioned" if args.columns else "tables row-partitioned") if args.partitioned else "replica",
            "n_gpus": world, "tokens_per_step": tokens, "ms_per_step": round(ms, 4),
            "tokens_per_s": round(tokens / (ms * 1e-3)), "steps": args.steps, "warmup": args.warmup,
            "scaling": "strong" if args.partitioned else "weak",
            "table_rows_per_gpu": (cfg["N"] + world - 1) // world if args.partitioned else cfg["N"],
            "max_memory_gib": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2), "phases_ms": phases}), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
