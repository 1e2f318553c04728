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


def _compare(module, x, near_tie_budget=0.002):
    """Runs the CUDA layer and the oracle; returns the fraction of routing slots that differ."""
    module = module.cuda().eval()
    y = module(x.cuda())
    module.check_status()
    p = _oracle_params(module)
    ey, lpx, lpy, es, ei = orc.layer_forward(p, bf16_round(x), return_routing=True)
    scores, indices, weights = (t.cpu() for t in module.last_routing)
    # routing: the GEMM accumulates in a different order than the CPU, so a token whose k-th and
    # (k+1)-th scores are closer than that rounding may swap; everything else must agree exactly
    diff = (indices.numpy() != ei)
    frac = diff.mean()
    assert frac <= near_tie_budget, f"{diff.sum()} routing slots differ"
    rows_ok = ~diff.any(axis=1)
    assert_close(y.reshape(-1, y.shape[-1])[torch.from_numpy(rows_ok).cuda()], ey.reshape(-1, ey.shape[-1])[rows_ok],
                 what="layer output")
    return frac


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
