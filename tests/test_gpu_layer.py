"""Whole layer (OmniMoE.forward) against the fp32 oracle on bf16-rounded parameters."""
import os

import numpy as np
import pytest
import torch

from oracle import omni_oracle as orc
from _util import assert_close, bf16_round, gen

pytestmark = pytest.mark.gpu


def _oracle_params(module):
    sd = {k: (bf16_round(v) if v.is_floating_point() and "running" not in k else v.float() if v.is_floating_point() else v)
          for k, v in module.state_dict().items()}
    sd = {k: v.cpu() for k, v in sd.items()}
    return orc.params_from_state_dict(sd, module.num_experts, module.top_k)


FLIP_GAP = 1e-4   # the log-prob tolerance of tests/test_gpu_router.py: a legitimate flip is a near-tie at that scale


def _check_flips(lpx, lpy, es, ei, indices, n, budget, what=""):
    """Routing slots may differ from the oracle's only where the two candidates are a near-tie in the
    oracle's own fp32 scores (the GEMM sums in another order than the CPU); a flip with a larger gap fails."""
    ndiff, gaps = orc.routing_flip_gaps(lpx, lpy, es, ei, indices, n)
    worst = float(gaps.max()) if ndiff else 0.0
    print(f"{what}routing slots that differ from the oracle: {ndiff} of {ei.size}, largest score gap {worst:.3g}")
    assert ndiff <= budget * ei.size, f"{ndiff} routing slots differ"
    assert worst < FLIP_GAP, f"a routing slot differs from the oracle by a score gap of {worst:.3g} (not a near-tie)"
    return ndiff


def _compare(module, x, near_tie_budget=0.002):
    """Runs the CUDA layer and the oracle; returns the fraction of routing slots that differ."""
    module = module.cuda().eval()
    with torch.no_grad():
        y = module(x.cuda())
    module.check_status()
    p = _oracle_params(module)
    ey, lpx, lpy, es, ei = orc.layer_forward(p, bf16_round(x), return_routing=True)
    scores, indices, weights = (t.cpu() for t in module.last_routing)
    # routing: the GEMM accumulates in a different order than the CPU, so a token whose k-th and
    # (k+1)-th scores are closer than that rounding may swap; everything else must agree exactly
    ndiff = _check_flips(lpx, lpy, es, ei, indices, module.num_expert_sqrt, near_tie_budget)
    rows_ok = ~(indices.numpy() != ei).any(axis=1)
    assert_close(y.reshape(-1, y.shape[-1])[torch.from_numpy(rows_ok).cuda()], ey.reshape(-1, ey.shape[-1])[rows_ok],
                 what="layer output")
    return ndiff / ei.size


def test_layer_tiny_golden(golden_dir):
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    g = np.load(os.path.join(golden_dir, "layer_tiny.npz"))
    m = OmniMoE(OmniMoEConfig(64, 128, "silu", int(g["num_experts"]), int(g["top_k"])))
    sd = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("sd.")}
    missing = m.load_state_dict(sd, strict=False)
    assert not missing.unexpected_keys
    m = m.cuda().eval()
    x = torch.from_numpy(g["x"])
    y = m(x.cuda())
    m.check_status()
    assert y.shape == x.shape and y.dtype == torch.float32
    # reference output was computed in fp32 on unrounded parameters: loose check here, the
    # rounded-parameter oracle comparison below is the tight one
    close = ((y.cpu() - torch.from_numpy(g["y"])).abs() <= 5e-2 + 5e-2 * torch.from_numpy(g["y"]).abs()).float().mean()
    assert close > 0.9
    _compare(m, x, near_tie_budget=0.02)


@pytest.mark.parametrize("expert_path", ["fused", "scheduled"])
def test_layer_config1_cpu_reference_shape(expert_path, monkeypatch):
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    monkeypatch.setenv("OMNI_MOE_B200_EXPERT", expert_path)  # both routed-expert implementations
    torch.manual_seed(0)
    m = OmniMoE(OmniMoEConfig(256, 1024, "silu", 1024, 8))
    x = torch.randn(2, 256, 256)
    _compare(m, x)


def test_layer_quick_start_shape_bf16():
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(0)
    m = OmniMoE(OmniMoEConfig(1024, 4096, "silu", 4096, 16)).to(torch.bfloat16)
    x = torch.randn(1, 4096, 1024).bfloat16()
    m = m.cuda().eval()
    y = m(x.cuda())
    m.check_status()
    assert y.dtype == torch.bfloat16 and y.shape == (1, 4096, 1024)
    y2 = m(x.cuda())
    assert torch.equal(y, y2)  # deterministic
    _compare(m, x)


def test_layer_training_mode_batch_statistics():
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(1)
    m = OmniMoE(OmniMoEConfig(128, 256, "silu", 256, 4)).cuda()
    ref = torch.nn.BatchNorm1d(16, affine=False).cuda()
    x = torch.randn(2, 64, 128).cuda()
    m.train()
    with torch.no_grad():
        m(x)
        z = x.view(-1, 128).bfloat16().float() @ m.router_gate_x.weight.bfloat16().float().t()
        ref(z)
    torch.testing.assert_close(m.router_norm_x.running_mean, ref.running_mean, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(m.router_norm_x.running_var, ref.running_var, rtol=1e-3, atol=1e-4)
    assert int(m.router_norm_x.num_batches_tracked) == 1


@pytest.mark.parametrize("momentum,dtype,tokens", [(0.1, torch.float32, 300), (None, torch.float32, 129), (0.3, torch.bfloat16, 1000),
                                                    (0.1, torch.float32, 1)])
def test_training_mode_batchnorm_kernel_matches_torch(momentum, dtype, tokens):
    """Three training-mode forwards: running statistics and batch counter follow nn.BatchNorm1d, and the
    selection uses the batch statistics (same routing as the oracle fed with the batch-normalised logits)."""
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(2)
    n = 16
    m = OmniMoE(OmniMoEConfig(128, 256, "silu", n * n, 4))
    for bn in (m.router_norm_x, m.router_norm_y):
        bn.momentum = momentum
    m = m.to(dtype).cuda().train()
    refs = [torch.nn.BatchNorm1d(n, affine=False, momentum=momentum).cuda() for _ in range(2)]
    with torch.no_grad():
        for step in range(3):
            x = torch.randn(1, tokens, 128, generator=torch.Generator().manual_seed(step)).to(dtype).cuda()
            m(x)
            m.check_status()
            xb = x.view(-1, 128).bfloat16().float()
            for ref, gate in zip(refs, (m.router_gate_x, m.router_gate_y)):
                z = xb @ gate.weight.bfloat16().float().t()
                if tokens > 1:
                    ref(z)
    if tokens > 1:
        tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-3, atol=1e-4)
        for bn, ref in zip((m.router_norm_x, m.router_norm_y), refs):
            torch.testing.assert_close(bn.running_mean.float(), ref.running_mean, **tol)
            torch.testing.assert_close(bn.running_var.float(), ref.running_var, **tol)
            assert int(bn.num_batches_tracked) == 3 and bn.running_mean.dtype == dtype
    else:
        assert int(m.router_norm_x.num_batches_tracked) == 3 and bool(torch.isfinite(m.router_norm_x.running_var).all())
    # eval after training uses the updated running statistics (no stale fold)
    m.eval()
    with torch.no_grad():
        x = torch.randn(1, 64, 128, generator=torch.Generator().manual_seed(9)).to(dtype).cuda()
        y = m(x)
    mean = torch.cat([m.router_norm_x.running_mean, m.router_norm_y.running_mean]).float()
    scale, shift = m._bn_fold_eval()
    torch.testing.assert_close(shift, -mean * scale, rtol=1e-5, atol=1e-6)
    assert bool(torch.isfinite(y.float()).all())


def test_training_mode_forward_in_a_cuda_graph():
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(3)
    m = OmniMoE(OmniMoEConfig(256, 512, "silu", 1024, 8)).to(torch.bfloat16).cuda().train()
    x = torch.randn(1, 512, 256).bfloat16().cuda()
    g = m.graphed(512)
    assert int(m.router_norm_x.num_batches_tracked) == 0, "building the graph must not count as a batch"
    with torch.no_grad():
        y_graph = g(x).clone()
        mean_after_graph = m.router_norm_x.running_mean.clone()
        assert int(m.router_norm_x.num_batches_tracked) == 1
        # the same step eagerly on a fresh copy of the statistics
        m.router_norm_x.reset_running_stats()
        m.router_norm_y.reset_running_stats()
        y_eager = m(x)
    torch.cuda.synchronize()
    assert torch.equal(y_graph.view(-1), y_eager.view(-1))
    assert torch.equal(mean_after_graph, m.router_norm_x.running_mean)


def _default_module(seed, h, i, n, k):
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(seed)
    return OmniMoE(OmniMoEConfig(h, i, "silu", n, k))


def _checksum(t):
    t = t.detach().double().cpu()
    return np.array([t.sum().item(), t.abs().sum().item()])


def test_layer_quick_start_shape_against_the_reference_fixture(golden_dir):
    """Configuration 2 of the benchmark list against what the reference module itself produced (fp32 math on
    the bf16-rounded parameters and tokens; every 64th output row, all routing decisions)."""
    g = np.load(os.path.join(golden_dir, "layer_c2.npz"))
    m = _default_module(int(g["seed"]), 1024, 4096, 4096, 16)
    x = torch.randn(1, 4096, 1024).to(torch.bfloat16)
    if not (np.allclose(_checksum(x.float()), g["x_checksum"])
            and np.allclose(_checksum(m.gate_proj.weight.to(torch.bfloat16).float()), g["gate_proj_checksum"])
            and np.allclose(_checksum(m.up_embed.weight.to(torch.bfloat16).float()), g["up_embed_checksum"])):
        pytest.skip("this torch build draws a different random stream than the one that made the fixture")
    m = m.to(torch.bfloat16).cuda().eval()
    y = m(x.cuda())
    m.check_status()
    indices = m.last_routing[1].cpu().numpy().astype(np.int64)
    ref_idx = g["indices"].astype(np.int64)
    diff = indices != ref_idx
    assert diff.mean() <= 0.002, f"{diff.sum()} routing slots differ from the reference's"
    # the flipped slots are near-ties: checked against the oracle's scores (the fixture keeps scores of every 64th token)
    p = _oracle_params(m)
    _, lpx, lpy, es, ei = orc.layer_forward(p, x.float(), return_routing=True)
    _check_flips(lpx, lpy, es, ei, indices, 64, 0.002, what="quick-start shape: ")
    rows = ~diff.any(axis=1)[::64]
    a = y.float().cpu().view(4096, 1024)[::64][torch.from_numpy(rows)]
    assert_close(a, torch.from_numpy(g["y_every64"])[torch.from_numpy(rows)], what="layer output vs reference fixture")
    sc = m.last_routing[0].cpu()[::64][torch.from_numpy(rows)]
    torch.testing.assert_close(sc, torch.from_numpy(g["scores_every64"])[torch.from_numpy(rows)], rtol=0, atol=2e-4)


@pytest.mark.parametrize("grad", [False, True])
def test_layer_training_mode_against_the_reference_fixtures(golden_dir, grad):
    """The module as constructed (training mode: BatchNorm over the batch, running statistics updated), against
    the reference module's own training-mode output: the tiny layer with everything stored, and configuration 1."""
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    g = np.load(os.path.join(golden_dir, "layer_tiny_train.npz"))
    m = OmniMoE(OmniMoEConfig(64, 128, "silu", int(g["num_experts"]), int(g["top_k"])))
    sd = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("sd.")}
    assert not m.load_state_dict(sd, strict=False).unexpected_keys
    m = m.cuda().train()
    x = torch.from_numpy(g["x"]).cuda()
    with torch.set_grad_enabled(grad):
        y = m(x)
    m.check_status()
    for axis, bn in (("x", m.router_norm_x), ("y", m.router_norm_y)):
        torch.testing.assert_close(bn.running_mean.cpu(), torch.from_numpy(g[f"run_mean_{axis}"]), rtol=2e-2, atol=2e-3)
        torch.testing.assert_close(bn.running_var.cpu(), torch.from_numpy(g[f"run_var_{axis}"]), rtol=2e-2, atol=2e-3)
    # fp32 module: the operands are rounded to bf16 for the kernels, so the reference (unrounded fp32) is
    # matched loosely here; the tight check is against the oracle on the rounded operands
    ok = ((y.detach().cpu() - torch.from_numpy(g["y"])).abs() <= 5e-2 + 5e-2 * torch.from_numpy(g["y"]).abs()).float().mean()
    assert ok > 0.9, float(ok)
    p = _oracle_params(m)
    ey, lpx, lpy, es, ei = orc.layer_forward(p, bf16_round(torch.from_numpy(g["x"])), return_routing=True, training=True)
    indices = m.last_routing[1].cpu()
    _check_flips(lpx, lpy, es, ei, indices, m.num_expert_sqrt, 0.02, what="tiny training-mode layer: ")
    rows = ~(indices.numpy() != ei).any(axis=1)
    assert_close(y.detach().reshape(-1, 64)[torch.from_numpy(rows).cuda()], ey.reshape(-1, 64)[rows], what="training-mode output")
    # configuration 1 in training mode
    g1 = np.load(os.path.join(golden_dir, "layer_c1_train.npz"))
    m1 = _default_module(int(g1["seed"]), 256, 1024, 1024, 8)
    x1 = torch.randn(2, 256, 256)
    if not (np.allclose(_checksum(x1), g1["x_checksum"]) and np.allclose(_checksum(m1.gate_proj.weight), g1["gate_proj_checksum"])):
        pytest.skip("this torch build draws a different random stream than the one that made the fixture")
    m1 = m1.cuda().train()
    with torch.set_grad_enabled(grad):
        y1 = m1(x1.cuda())
    m1.check_status()
    p1 = _oracle_params(m1)
    # the running statistics moved during the forward; the oracle's training mode does not read them
    ey1, lpx, lpy, es, ei = orc.layer_forward(p1, bf16_round(x1), return_routing=True, training=True)
    idx1 = m1.last_routing[1].cpu()
    _check_flips(lpx, lpy, es, ei, idx1, 32, 0.002, what="configuration 1, training mode: ")
    rows = ~(idx1.numpy() != ei).any(axis=1)
    assert_close(y1.detach().reshape(-1, 256)[torch.from_numpy(rows).cuda()], ey1.reshape(-1, 256)[rows], what="c1 training-mode output")
    # and the reference's own numbers (fp32 on unrounded parameters): loose, every 8th row
    ref_rows = torch.from_numpy(g1["y_every8"])
    got_rows = y1.detach().float().cpu().view(512, 256)[::8]
    frac = ((got_rows - ref_rows).abs() <= 5e-2 + 5e-2 * ref_rows.abs()).float().mean()
    assert frac > 0.9, float(frac)
    for axis, bn in (("x", m1.router_norm_x), ("y", m1.router_norm_y)):
        torch.testing.assert_close(bn.running_mean.cpu(), torch.from_numpy(g1[f"run_mean_{axis}"]), rtol=2e-2, atol=2e-3)
        torch.testing.assert_close(bn.running_var.cpu(), torch.from_numpy(g1[f"run_var_{axis}"]), rtol=2e-2, atol=2e-3)
