"""Hidden / intermediate sizes that are not multiples of 8.

The reference masks the tails of its tiles (e.g. omni_moe/ops/triton/omni_expert.py:67,123), so any size
works there; the kernels here move rows in 16-byte pieces and the operator wrappers zero-pad other sizes.
Same bars as everywhere: bf16 results within rtol / atol 2e-2 of the fp32 oracle on the same bf16-rounded
operands, gradients within 2e-2 of the gradient's scale.
"""
import pytest
import torch

from oracle import omni_oracle as orc
from _util import assert_close, bf16_round, gen

pytestmark = pytest.mark.gpu


def _scaled_close(actual, expected, what, rtol=3e-2, atol_frac=2e-2):
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} != {tuple(e.shape)}"
    scale = float(e.abs().max()) or 1.0
    bad = (a - e).abs() > atol_frac * scale + rtol * e.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())}/{bad.numel()} outside tolerance"


@pytest.mark.parametrize("t,h,n,k", [(50, 36, 64, 4), (129, 100, 256, 8), (7, 1, 16, 2), (33, 1031, 64, 6)])
def test_expert_op_any_hidden_size(t, h, n, k):
    from omni_moe.ops.triton import triton_omni_expert_func
    g = gen(t + h)
    x = torch.randn(t, h, generator=g).bfloat16()
    up = (torch.randn(n, h, generator=g) / h ** 0.5).bfloat16()
    down = (torch.randn(n, h, generator=g) * 0.2).bfloat16()
    w = torch.rand(t, k, generator=g).bfloat16()
    idx = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
    y = triton_omni_expert_func(x.cuda(), up.cuda(), down.cuda(), w.cuda(), idx.cuda())
    assert y.shape == (t, h) and y.dtype == torch.bfloat16 and y.is_contiguous()
    assert_close(y, orc.expert_forward(x, up, down, w.float(), idx), what="experts, odd hidden size")
    # gradients through the padding
    dy = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    cx, cu, cd, cw = (v.cuda().requires_grad_(True) for v in (x, up, down, w))
    triton_omni_expert_func(cx, cu, cd, cw, idx.cuda()).backward(dy.cuda())
    ex, eu, ed, ew = orc.expert_backward(x.float(), up.float(), down.float(), w.float(), idx, dy.float())
    for got, want, name in ((cx.grad, ex, "dx"), (cu.grad, eu, "d_up"), (cd.grad, ed, "d_down"), (cw.grad, ew, "d_weights")):
        assert got.shape == want.shape
        _scaled_close(got, want, f"{name} (H={h})")


@pytest.mark.parametrize("t,h,i,limit", [(50, 36, 100, None), (129, 100, 52, None), (64, 64, 20, None), (40, 20, 64, 0.5), (9, 3, 5, None)])
def test_mlp_op_any_sizes(t, h, i, limit):
    from omni_moe_b200.ops import omni_mlp_func
    g = gen(t + h + i)
    x = torch.randn(t, h, generator=g).bfloat16()
    wg = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wu = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wd = (torch.randn(h, i, generator=g) / i ** 0.5).bfloat16()
    y = omni_mlp_func(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda(), limit)
    assert y.shape == (t, h) and y.dtype == torch.bfloat16 and y.is_contiguous()
    assert_close(y, orc.mlp_forward(x, wg, wu, wd, limit=limit), what="mlp, odd sizes")
    dy = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    cx, cg, cu, cd = (v.cuda().requires_grad_(True) for v in (x, wg, wu, wd))
    omni_mlp_func(cx, cg, cu, cd, limit).backward(dy.cuda())
    exp = orc.mlp_backward(x.float(), wg.float(), wu.float(), wd.float(), dy.float(), limit=limit,
                           preact_dtype=torch.bfloat16 if limit else None)
    for got, want, name in zip((cx.grad, cg.grad, cu.grad, cd.grad), exp, ("dx", "d_gate", "d_up", "d_down")):
        _scaled_close(got, want, f"{name} (H={h}, I={i})")


@pytest.mark.parametrize("training", [False, True])
def test_layer_any_sizes(training):
    """The module with hidden 100 / intermediate 52: operator by operator (no fused launch sequence)."""
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(3)
    h, i, n_exp, k, t = 100, 52, 64, 4, 96
    m = OmniMoE(OmniMoEConfig(h, i, "silu", n_exp, k)).to(torch.bfloat16)
    with torch.no_grad():
        m.up_embed.weight.mul_(0.2)
        m.down_embed.weight.mul_(0.2)
    m = m.cuda().train(training)
    x = torch.randn(2, t // 2, h, generator=gen(4)).bfloat16()
    with torch.no_grad():
        y = m(x.cuda())
    m.check_status()
    assert y.shape == x.shape and y.dtype == torch.bfloat16
    scores, indices, weights = (v.cpu() for v in m.last_routing)
    assert indices.shape == (t, k) and int(indices.min()) >= 0 and int(indices.max()) < n_exp
    assert all(len(set(r.tolist())) == k for r in indices), "a token's experts are distinct"
    sd = {kk: bf16_round(v.float().cpu()) for kk, v in m.state_dict().items() if v.is_floating_point()}
    x2 = bf16_round(x).reshape(t, h)
    # with the module's own routing the rest of the layer must match the oracle
    want = (orc.mlp_forward(x2, sd["gate_proj.weight"], sd["up_proj.weight"], sd["down_proj.weight"])
            + orc.expert_forward(x2, sd["up_embed.weight"], sd["down_embed.weight"], weights.float(), indices))
    assert_close(y.reshape(t, h), want, what="layer with odd sizes", rtol=3e-2, atol=3e-2)
    if not training:
        # and the routing is the oracle's up to near-ties of the bf16 gate products
        st = {kk: (bf16_round(v) if v.is_floating_point() and "running" not in kk else v.float() if v.is_floating_point() else v).cpu()
              for kk, v in m.state_dict().items()}
        _, _, _, _, ei = orc.layer_forward(orc.params_from_state_dict(st, n_exp, k), x2.reshape(1, t, h), return_routing=True)
        agree = float((indices.numpy() == ei).mean())
        assert agree > 0.9, f"only {agree:.2%} of the routing slots agree with the oracle"
    # gradients flow to every parameter and the input
    xg = x.cuda().requires_grad_(True)
    m.train(True)
    m(xg).float().square().mean().backward()
    assert xg.grad is not None and xg.grad.shape == x.shape and bool(torch.isfinite(xg.grad).all())
    for name, p in m.named_parameters():
        assert p.grad is not None and p.grad.shape == p.shape and bool(torch.isfinite(p.grad).all()), name


def test_graph_capture_refuses_odd_sizes():
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    m = OmniMoE(OmniMoEConfig(100, 52, "silu", 64, 4)).to(torch.bfloat16).cuda().eval()
    with pytest.raises(RuntimeError, match="multiple of 8"):
        m.graphed(32)
