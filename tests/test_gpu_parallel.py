"""Row-partitioned expert tables on the GPU: the pair-list kernels on one device (every rank's share
computed in turn, no communication), and the whole partitioned layer on two devices over NCCL when
two are present."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import omni_oracle as orc
from _util import assert_close, gen, zipf_indices

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _received_for_rank(x, idx, w, part):
    """What dispatch_pairs would deliver to part.rank if all tokens lived in one process."""
    from omni_moe_b200.parallel import ReceivedPairs
    t, k = idx.shape
    flat = idx.reshape(-1)
    mine = (part.owner(flat) == part.rank).nonzero().flatten()   # ascending pair id = ascending token id
    tok = torch.div(mine, k, rounding_mode="floor").to(torch.int32)
    off = torch.searchsorted(tok, torch.arange(t + 1, device=x.device, dtype=torch.int32)).to(torch.int32)
    return ReceivedPairs(x, tok.contiguous(), (flat[mine] - part.lo).to(torch.int32).contiguous(),
                         w.reshape(-1)[mine].float().contiguous(), off, [], [])


@pytest.mark.parametrize("t,h,n,k,world,skew", [(200, 256, 1000, 8, 4, False), (64, 4096, 300, 16, 2, False),
                                                  (512, 1024, 4096, 32, 8, True), (33, 72, 7, 4, 3, False)])
def test_pair_list_kernels_sum_to_the_full_answer(t, h, n, k, world, skew):
    from omni_moe_b200.parallel import ExpertPartition, local_partial_states
    g = gen(t + n)
    x = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    up = (torch.randn(n, h, generator=g) * 0.1).bfloat16()
    dn = (torch.randn(n, h, generator=g) * 0.1).bfloat16()
    w = torch.rand(t, k, generator=g)
    idx = zipf_indices(t, k, n, 1.1, 1) if skew else torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
    xc, uc, dc, wc, ic = x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda()
    total = torch.zeros(t, h, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    for r in range(world):
        part = ExpertPartition(n, world, r)
        recv = _received_for_rank(xc, ic, wc, part)
        total += local_partial_states(recv, part.slice_rows(uc), part.slice_rows(dc), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_close(total, orc.expert_forward(x, up, dn, w, idx), rtol=1e-3, atol=1e-4)


_CHILD = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["OMNI_ROOT"]); sys.path.insert(0, os.path.join(os.environ["OMNI_ROOT"], "tests"))
from oracle import omni_oracle as orc
from omni_moe_b200.modules.omni_moe import OmniMoE, OmniMoEConfig
from omni_moe_b200.parallel import PartitionedOmniMoE, shard_tokens
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
torch.manual_seed(0)
full = OmniMoE(OmniMoEConfig(256, 512, "silu", 1024, 8)).to(torch.bfloat16).eval()
sd = {k: v.float() for k, v in full.state_dict().items()}
x = torch.randn(1, 64 * world, 256).bfloat16()
p = orc.params_from_state_dict(sd, 1024, 8)
ey, _, _, _, ei = orc.layer_forward(p, x.float(), return_routing=True)
m = PartitionedOmniMoE(full.cuda(), None)
assert m.up_local.shape[0] == 1024 // world and m.inner.up_embed.weight.shape[0] == 0
xs = shard_tokens(x, rank, world).cuda().view(1, 64, 256)
y = m(xs)
m.inner.check_status()
sl = slice(rank * 64, (rank + 1) * 64)
same = (m.inner.last_routing[1].cpu().numpy() == ei[sl]).all(axis=1)
assert same.mean() > 0.95, same.mean()
a, e = y.float().cpu().view(64, 256)[same], ey.view(-1, 256)[sl][same]
bad = (a - e).abs() > 2e-2 + 2e-2 * e.abs()
assert not bad.any(), int(bad.sum())
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok", flush=True)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_partitioned_layer_two_gpus_nccl(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, OMNI_ROOT=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


_CHILD_BN = r"""
import os, sys, copy, torch, torch.distributed as dist
sys.path.insert(0, os.environ["OMNI_ROOT"])
from omni_moe_b200.modules.omni_moe import OmniMoE, OmniMoEConfig
from omni_moe_b200.parallel import shard_tokens
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
torch.manual_seed(0)
base = OmniMoE(OmniMoEConfig(256, 512, "silu", 1024, 8)).to(torch.bfloat16)
x = torch.randn(1, 96 * world, 256).bfloat16()
# one GPU, whole batch
whole = copy.deepcopy(base).cuda().train()
with torch.no_grad():
    y_whole = whole(x.cuda())
# token-sharded replicas with synchronised batch statistics: fused (no-grad) forward
dp = copy.deepcopy(base).cuda().train().sync_batch_statistics()
xs = shard_tokens(x, rank, world).cuda().view(1, 96, 256)
with torch.no_grad():
    y = dp(xs)
for a, b in ((dp.router_norm_x, whole.router_norm_x), (dp.router_norm_y, whole.router_norm_y)):
    # bf16 buffers: the two paths (merged per-rank moments / one-GPU kernel) may round the last bit differently
    assert torch.allclose(a.running_mean.float(), b.running_mean.float(), atol=2e-4), (a.running_mean - b.running_mean).abs().max()
    assert torch.allclose(a.running_var.float(), b.running_var.float(), rtol=1e-2, atol=1e-4), (a.running_var - b.running_var).abs().max()
sl = slice(rank * 96, (rank + 1) * 96)
same = (dp.last_routing[1] == whole.last_routing[1][sl]).all(dim=1)
assert same.float().mean() > 0.97, float(same.float().mean())
assert torch.allclose(y.view(96, 256)[same].float(), y_whole.view(-1, 256)[sl][same].float(), rtol=2e-2, atol=2e-2)
# differentiable forward: torch's SyncBatchNorm in place of the two norm layers
sdp = torch.nn.SyncBatchNorm.convert_sync_batchnorm(copy.deepcopy(base)).cuda().train()
ys = sdp(xs)
ys.float().square().mean().backward()
assert torch.allclose(sdp.router_norm_x.running_mean.float(), whole.router_norm_x.running_mean.float(), atol=2e-2)
assert all(p.grad is not None for p in sdp.parameters())
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok", flush=True)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_training_batchnorm_synchronised_over_two_gpus(tmp_path):
    """Token-sharded replicas in training mode normalise the router logits with the statistics of the whole batch."""
    script = tmp_path / "child_bn.py"
    script.write_text(_CHILD_BN)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, OMNI_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_two_devices():
    """Per-kernel settings (shared-memory limits) are per device: the second GPU of a process must work too."""
    from omni_moe_b200.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(0)
    base = OmniMoE(OmniMoEConfig(256, 512, "silu", 1024, 8)).to(torch.bfloat16).eval()
    x = torch.randn(1, 300, 256).bfloat16()
    outs = []
    for d in (0, 1):
        import copy
        m = copy.deepcopy(base).to(f"cuda:{d}")
        y = m(x.to(f"cuda:{d}"))
        m.check_status()
        outs.append(y.cpu())
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("t,k,n,world,chunks,rank", [(64, 8, 1000, 4, 2, 1), (4096, 64, 1 << 20, 8, 2, 5), (30, 3, 7, 3, 1, 2),
                                                      (96, 16, 4096, 2, 4, 0), (2048, 32, 262144, 4, 2, 3)])
def test_dispatch_records_from_the_planning_kernels_equal_the_torch_operators(t, k, n, world, chunks, rank):
    """omni_partition_keys -> radix pass -> omni_partition_records against the same plan written in torch operators
    (the path the gloo ranks of the CPU tests take): records and split sizes bit for bit."""
    from omni_moe_b200.parallel import ExpertPartition, _sorted_records
    part = ExpertPartition(n, world, rank)
    g = gen(t * k + world)
    idx = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
    w = torch.rand(t, k, generator=g)
    rec_cpu, cnt_cpu = _sorted_records(idx, w, part, chunks)
    rec_gpu, cnt_gpu = _sorted_records(idx.cuda(), w.cuda(), part, chunks)
    torch.cuda.synchronize()
    assert torch.equal(cnt_gpu.cpu(), cnt_cpu), (cnt_gpu, cnt_cpu)
    assert torch.equal(rec_gpu.cpu(), rec_cpu)
    assert int(cnt_cpu.sum()) == t * k


def test_dispatch_records_send_an_expert_outside_the_table_to_an_end_rank():
    """An id below 0 goes to rank 0, one past the table to the last rank, both with a row outside the slice (the expert
    kernels of that rank report and skip it); every other record is unchanged."""
    from omni_moe_b200.parallel import ExpertPartition, _sorted_records
    t, k, n, world = 32, 4, 100, 4
    part = ExpertPartition(n, world, 0)
    idx = torch.randint(0, n, (t, k), generator=gen(3), dtype=torch.int32)
    w = torch.rand(t, k, generator=gen(4))
    good, cnt_good = _sorted_records(idx.cuda(), w.cuda(), part, 1)
    bad = idx.clone()
    bad[3, 1], bad[7, 2] = -5, n + 50
    rec, cnt = _sorted_records(bad.cuda(), w.cuda(), part, 1)
    torch.cuda.synchronize()
    assert int(cnt.sum()) == t * k
    rows = part.rows_per_rank
    rec = rec.cpu()
    starts = torch.cumsum(torch.cat([torch.zeros(1, dtype=torch.long), cnt.cpu().view(-1)]), 0)
    owner_of_record = torch.bucketize(torch.arange(t * k), starts[1:], right=True)
    outside = (rec[:, 1] < 0) | (rec[:, 1] >= rows)
    assert int(outside.sum()) == 2
    assert sorted(owner_of_record[outside].tolist()) == [0, world - 1]


@pytest.mark.parametrize("t,h,n,k,world", [(200, 256, 1000, 8, 4), (64, 4096, 300, 16, 2), (512, 1024, 4096, 32, 8),
                                            (33, 96, 7, 4, 3)])
def test_column_slices_sum_to_the_full_answer(t, h, n, k, world):
    """Tables cut by columns, all ranks' shares computed in turn on one GPU: the partial dot products of the slices
    (omni_expert_dots) add up to the full dot products, and the combine over a slice gives that slice of the output."""
    from omni_moe_b200.parallel import ColumnPartition, column_combine, column_partial_dots
    g = gen(t + n)
    x = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    up = (torch.randn(n, h, generator=g) * 0.1).bfloat16()
    dn = (torch.randn(n, h, generator=g) * 0.1).bfloat16()
    w = torch.rand(t, k, generator=g)
    idx = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
    idx[:, 0] = idx[:, 1]
    parts = [ColumnPartition(h, world, r) for r in range(world)]
    xc, idxc, wc = x.cuda(), idx.cuda(), w.cuda()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    dots = sum(column_partial_dots(p.slice_columns(xc), idxc, p.slice_columns(up.cuda()), st) for p in parts)
    e_dots = (x.float()[:, None, :] * up.float()[idx.long()]).sum(-1)
    assert_close(dots, e_dots, rtol=1e-4, atol=1e-4, what="summed partial dot products")
    coef = torch.nn.functional.silu(dots) * wc
    y = torch.cat([column_combine(coef, idxc, p.slice_columns(dn.cuda()), torch.float32, st) for p in parts], dim=1)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_close(y, orc.expert_forward(x.float(), up.float(), dn.float(), w, idx), rtol=1e-3, atol=1e-4, what="column slices")


_CHILD_COLUMNS = _CHILD.replace("import PartitionedOmniMoE, shard_tokens", "import ColumnPartitionedOmniMoE as PartitionedOmniMoE, shard_tokens") \
                       .replace("assert m.up_local.shape[0] == 1024 // world and m.inner.up_embed.weight.shape[0] == 0",
                                "assert m.up_cols.shape == (1024, 256 // world) and m.inner.up_embed.weight.shape[0] == 0")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_column_partitioned_layer_two_gpus_nccl(tmp_path):
    assert "ColumnPartitionedOmniMoE" in _CHILD_COLUMNS and "up_cols" in _CHILD_COLUMNS
    script = tmp_path / "child_columns.py"
    script.write_text(_CHILD_COLUMNS)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, OMNI_ROOT=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
