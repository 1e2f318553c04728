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
