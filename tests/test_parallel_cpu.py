"""Exchange plumbing of the row-partitioned expert tables, on CPU ranks with the gloo backend.

Two (and three) processes each own a slice of the tables and a shard of the tokens; the dispatch,
the token-ordered receive lists and the combine are the real code of omni_moe_b200.parallel, the
per-rank arithmetic is the oracle's.  The result must equal the oracle's single-process answer."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import omni_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_local(recv, up_local, down_local):
    """Step 3 with the oracle's arithmetic: per received pair w * silu(x . up) * down, summed per token."""
    t_total, h = recv.x_all.shape
    out = torch.zeros(t_total, h)
    if recv.pair_tokens.numel():
        tok = recv.pair_tokens.long()
        e = recv.pair_experts.long()
        s = (recv.x_all.float()[tok] * up_local.float()[e]).sum(-1)
        c = torch.nn.functional.silu(s) * recv.pair_weights
        out.index_add_(0, tok, c[:, None] * down_local.float()[e])
        # the receive list is grouped by token and the offsets describe it
        off = recv.token_offsets.long()
        assert bool((tok[1:] >= tok[:-1]).all())
        assert off[0] == 0 and off[-1] == tok.numel()
        counts = torch.bincount(tok, minlength=t_total)
        assert torch.equal(off[1:] - off[:-1], counts)
    return out


def _worker(rank, world, port, t_local, h, n, k, seed, ret, chunks=1):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from omni_moe_b200.parallel import ExpertPartition, partitioned_expert_states, shard_tokens
        g = torch.Generator().manual_seed(seed)
        t = t_local * world
        x = torch.randn(t, h, generator=g)
        up = torch.randn(n, h, generator=g) * 0.1
        down = torch.randn(n, h, generator=g) * 0.1
        idx = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
        idx[:, 0] = idx[:, 1]          # duplicates inside a token
        idx[0, :] = n - 1              # a token whose pairs all go to the last rank
        w = torch.rand(t, k, generator=g)
        part = ExpertPartition(n, world, rank)
        sl = slice(rank * t_local, (rank + 1) * t_local)
        assert torch.equal(shard_tokens(x, rank, world), x[sl])
        got = partitioned_expert_states(x[sl], idx[sl], w[sl], part.slice_rows(up), part.slice_rows(down), part,
                                        local_fn=_oracle_local, chunks=chunks)
        expect = orc.expert_forward(x, up, down, w, idx)[sl]
        ret[rank] = float((got - expect).abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,t_local,n,chunks", [(2, 12, 64, 1), (3, 5, 50, 1), (2, 8, 3, 1), (2, 12, 64, 3), (3, 8, 50, 2),
                                                     (2, 7, 20, 2)])
def test_partitioned_dispatch_and_combine_gloo(world, t_local, n, chunks):
    """chunks > 1: the token ranges go through the exchange one after another (7 tokens in 2 chunks falls back to one)."""
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, t_local, 16, n, 6, 3, ret, chunks)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world and max(ret.values()) < 1e-4, dict(ret)


def _wrapper_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from omni_moe_b200.modules.omni_moe import OmniMoE, OmniMoEConfig
        from omni_moe_b200.parallel import PartitionedOmniMoE
        torch.manual_seed(0)
        full = OmniMoE(OmniMoEConfig(32, 64, "silu", 16, 2))
        rows = full.up_embed.weight.detach().clone()
        m = PartitionedOmniMoE(full, None)
        out = [m.up_local.shape == (8, 32), torch.equal(m.up_local.float(), rows[rank * 8:(rank + 1) * 8].bfloat16().float()),
               full.up_embed.weight.shape[0] == 0]
        try:
            full._operands()
            out.append(False)
        except RuntimeError as e:
            out.append("PartitionedOmniMoE" in str(e))
        # one expert row over two ranks: the second rank would hold nothing
        try:
            PartitionedOmniMoE(OmniMoE(OmniMoEConfig(32, 64, "silu", 1, 1)), None)
            out.append(rank == 0)
        except ValueError:
            out.append(rank == 1)
        ret[rank] = out
    finally:
        dist.destroy_process_group()


def test_partitioned_wrapper_keeps_the_slices_and_disarms_the_inner_module():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_wrapper_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(all(ret[r]) for r in range(world)), dict(ret)


def test_expert_partition_arithmetic():
    from omni_moe_b200.parallel import ExpertPartition
    parts = [ExpertPartition(10, 4, r) for r in range(4)]
    assert [(p.lo, p.hi) for p in parts] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    e = torch.arange(10)
    assert parts[0].owner(e).tolist() == [0, 0, 0, 1, 1, 1, 2, 2, 2, 3]
    t = torch.arange(20).view(10, 2)
    assert torch.equal(parts[3].slice_rows(t), t[9:10])


def _stats_worker(rank, world, port, counts, c, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from omni_moe_b200.parallel import synced_batch_statistics
        g = torch.Generator().manual_seed(5)
        z = torch.randn(sum(counts), c, generator=g) * 3.0 + 100.0     # a large common offset: cancellation would show
        lo = sum(counts[:rank])
        mean, var, total = synced_batch_statistics(z[lo:lo + counts[rank]])
        ev, em = torch.var_mean(z.double(), dim=0, unbiased=False)
        ret[rank] = (float((mean.double() - em).abs().max()), float((var.double() - ev).abs().max() / ev.max()), total)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("counts", [(7, 9), (1, 30, 5)])
def test_synced_batch_statistics_gloo(counts):
    """Batch statistics of router logits sharded unevenly over ranks = statistics of the whole batch."""
    world, port = len(counts), _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_stats_worker, args=(r, world, port, counts, 12, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for r in range(world):
        dm, dv, total = ret[r]
        assert dm < 1e-4 and dv < 1e-5 and total == sum(counts), (r, ret[r])


def test_synced_batch_statistics_without_process_group():
    from omni_moe_b200.parallel import synced_batch_statistics
    z = torch.randn(50, 6)
    mean, var, total = synced_batch_statistics(z)
    ev, em = torch.var_mean(z, dim=0, unbiased=False)
    assert torch.allclose(mean, em) and torch.allclose(var, ev) and total == 50


def _failure_worker(rank, world, port, scenario, ret):
    """Host-side failure injection: no device is involved, the failing rank simply behaves badly."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from omni_moe_b200.parallel import ExchangeError, ExpertPartition, dispatch_pairs, partitioned_expert_states
    g = torch.Generator().manual_seed(rank)
    n, k, h = 32, 4, 8
    t_local = 6
    if scenario == "shape_mismatch" and rank == 1:
        t_local = 5                                   # a misconfigured rank
    x = torch.randn(t_local, h, generator=g)
    idx = torch.randint(0, n, (t_local, k), generator=g, dtype=torch.int32)
    w = torch.rand(t_local, k, generator=g)
    part = ExpertPartition(n, world, rank)
    if scenario == "peer_leaves" and rank == 1:
        ret[rank] = "left"
        os._exit(0)                                   # leaves between steps, before joining the exchange
    try:
        dispatch_pairs(x, idx, w, part)
        ret[rank] = "no error"
    except ExchangeError as e:
        ret[rank] = f"{e.stage}|{e}"
    if scenario == "shape_mismatch":
        dist.destroy_process_group()
    else:
        os._exit(0)                                   # the group is broken: do not wait for the peer in teardown


@pytest.mark.parametrize("scenario", ["shape_mismatch", "peer_leaves"])
def test_exchange_failures_surface_on_the_host(scenario):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_failure_worker, args=(r, world, port, scenario, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
        assert p.exitcode == 0, p.exitcode
    if scenario == "shape_mismatch":
        for r in range(world):
            assert ret[r].startswith("count exchange|") and "same shard shape" in ret[r], ret[r]
    else:
        assert ret[1] == "left"
        assert "|" in ret[0] and ret[0].split("|")[0] in ("count exchange", "pair dispatch"), ret[0]


# ---- tables partitioned by columns -------------------------------------------------------------------------------
def _oracle_dots(x_cols, idx_all, up_cols):
    return (x_cols.float()[:, None, :] * up_cols.float()[idx_all.long()]).sum(-1)


def _oracle_combine(coef, idx_all, down_cols):
    return (coef[:, :, None] * down_cols.float()[idx_all.long()]).sum(1)


def _column_worker(rank, world, port, t_local, h, n, k, seed, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from omni_moe_b200.parallel import (ColumnPartition, column_expert_states, exchange_token_columns,
                                            return_state_columns)
        g = torch.Generator().manual_seed(seed)
        t = t_local * world
        x = torch.randn(t, h, generator=g)
        up = torch.randn(n, h, generator=g) * 0.1
        down = torch.randn(n, h, generator=g) * 0.1
        idx = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
        idx[:, 0] = idx[:, 1]          # duplicates inside a token
        w = torch.rand(t, k, generator=g)
        part = ColumnPartition(h, world, rank)
        sl = slice(rank * t_local, (rank + 1) * t_local)
        # the two exchanges are inverse to each other and keep the global token order
        cols = exchange_token_columns(x[sl], part)
        assert torch.equal(cols, x[:, part.lo:part.hi])
        back = return_state_columns(cols, part)
        assert torch.equal(back.transpose(0, 1).reshape(t_local, h), x[sl])
        got = column_expert_states(x[sl], idx[sl], w[sl], part.slice_columns(up), part.slice_columns(down), part,
                                   dots_fn=_oracle_dots, combine_fn=_oracle_combine)
        expect = orc.expert_forward(x, up, down, w, idx)[sl]
        ret[rank] = float((got - expect).abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,t_local,h,n", [(2, 12, 16, 64), (3, 5, 24, 50), (4, 3, 32, 7)])
def test_column_partitioned_exchange_gloo(world, t_local, h, n):
    """Token columns out, routing gathered, partial dot products all-reduced, state columns back: the real exchange code
    on gloo ranks with the oracle's arithmetic per rank equals the oracle's single-process answer."""
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_column_worker, args=(r, world, port, t_local, h, n, 6, 3, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world and max(ret.values()) < 1e-4, dict(ret)


def _column_wrapper_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from omni_moe_b200.modules.omni_moe import OmniMoE, OmniMoEConfig
        from omni_moe_b200.parallel import ColumnPartitionedOmniMoE, columns_from_row_slices
        torch.manual_seed(0)
        full = OmniMoE(OmniMoEConfig(32, 64, "silu", 16, 2))
        table = full.up_embed.weight.detach().clone()
        m = ColumnPartitionedOmniMoE(full, None)
        out = [m.up_cols.shape == (16, 16), torch.equal(m.up_cols.float(), table[:, rank * 16:(rank + 1) * 16].bfloat16().float()),
               full.up_embed.weight.shape[0] == 0]
        try:
            full._operands()
            out.append(False)
        except RuntimeError:
            out.append(True)
        # rows -> columns without holding the table whole
        cols = columns_from_row_slices(table[rank * 8:(rank + 1) * 8].contiguous())
        out.append(torch.equal(cols, table[:, rank * 16:(rank + 1) * 16]))
        # a hidden size that cannot be cut into slices of a multiple of 8 columns is refused
        try:
            ColumnPartitionedOmniMoE(OmniMoE(OmniMoEConfig(24, 64, "silu", 16, 2)), None)
            out.append(False)
        except ValueError:
            out.append(True)
        ret[rank] = out
    finally:
        dist.destroy_process_group()


def test_column_partitioned_wrapper_keeps_the_slices_and_disarms_the_inner_module():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_column_wrapper_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(all(ret[r]) for r in range(world)), dict(ret)
