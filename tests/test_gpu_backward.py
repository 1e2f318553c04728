"""Backward of the three operators against fp32 autograd through the oracle's restatement of the
reference's PyTorch mirrors (the way the reference's own tests obtain reference gradients).

Bars: router gradients are sums of the given fp32 score gradients in a fixed order -> compared at
1e-6 relative; gradients of bf16 operands are compared at rtol/atol 2e-2 of the gradient's scale
against the fp32 oracle run on the same bf16-rounded operands.
"""
import numpy as np
import pytest
import torch

from oracle import omni_oracle as orc
from _util import assert_close, gen

pytestmark = pytest.mark.gpu


def _scaled_close(actual, expected, what, rtol=2e-2, atol_frac=2e-2):
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    scale = float(e.abs().max()) or 1.0
    bad = (a - e).abs() > atol_frac * scale + rtol * e.abs()
    assert not bad.any(), (f"{what}: {int(bad.sum())}/{bad.numel()} outside tolerance; max abs err "
                           f"{float((a - e).abs().max()):.4g} at scale {scale:.4g}")


@pytest.mark.parametrize("t,n,k,idt", [(64, 16, 4, torch.int32), (300, 64, 16, torch.int32), (129, 256, 32, torch.int64),
                                         (40, 1024, 64, torch.int32), (7, 5, 25, torch.int64), (0, 8, 2, torch.int32)])
def test_router_backward_matches_oracle(t, n, k, idt):
    from omni_moe_b200.ops.autograd import router_backward
    g = gen(t + n)
    # duplicates inside a token are legal for the scatter (they cannot come out of a top-k, the kernel does not care)
    idx = torch.randint(0, n * n, (t, k), generator=g).to(idt)
    ds = torch.randn(t, k, generator=g)
    dlx, dly = router_backward(ds.cuda(), idx.cuda(), n)
    ex, ey = orc.router_backward(ds, idx, n)
    torch.testing.assert_close(dlx.cpu(), ex, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(dly.cpu(), ey, rtol=1e-6, atol=1e-6)
    if t:
        again = router_backward(ds.cuda(), idx.cuda(), n)
        assert torch.equal(again[0], dlx) and torch.equal(again[1], dly), "the scatter must be deterministic"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_router_op_autograd(dtype):
    from omni_moe.ops.triton import triton_omni_router_func
    t, n, k = 200, 64, 16
    g = gen(3)
    lx = torch.log_softmax(torch.randn(t, n, generator=g), -1).to(dtype)
    ly = torch.log_softmax(torch.randn(t, n, generator=g), -1).to(dtype)
    cx, cy = lx.cuda().requires_grad_(True), ly.cuda().requires_grad_(True)
    scores, idx = triton_omni_router_func(cx, cy, n, k)
    assert scores.dtype == dtype and not idx.requires_grad
    wgt = torch.randn(t, k, generator=g)
    (scores.float() * wgt.cuda()).sum().backward()
    ex, ey = orc.router_backward(wgt.to(dtype).float(), idx.cpu(), n)
    assert cx.grad.dtype == dtype
    torch.testing.assert_close(cx.grad.float().cpu(), ex.to(dtype).float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(cy.grad.float().cpu(), ey.to(dtype).float(), rtol=1e-2, atol=1e-2)


def _expert_inputs(t, h, n, k, seed):
    g = gen(seed)
    x = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    up = (torch.randn(n, h, generator=g) * (2.0 / h ** 0.5)).bfloat16()
    dn = (torch.randn(n, h, generator=g) * 0.1).bfloat16()
    w = torch.rand(t, k, generator=g) * 0.2
    idx = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
    dy = (torch.randn(t, h, generator=g) * 0.3).bfloat16()
    return x, up, dn, w, idx, dy


@pytest.mark.parametrize("t,h,n,k", [(32, 64, 16, 4), (300, 256, 512, 8), (257, 1024, 4096, 16), (64, 2048, 128, 32),
                                       (40, 4096, 300, 64), (50, 72, 64, 6), (20, 8192, 64, 2), (1, 8, 1, 1)])
@pytest.mark.parametrize("grad_dtype", [torch.float32, torch.bfloat16])
def test_expert_backward_matches_oracle(t, h, n, k, grad_dtype):
    from omni_moe_b200.ops.autograd import expert_backward
    x, up, dn, w, idx, dy = _expert_inputs(t, h, n, k, t + h)
    dx, d_up, d_dn, dg, _ = expert_backward(dy.cuda(), x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), grad_dtype=grad_dtype)
    ex, eu, ed, eg = orc.expert_backward(x.float(), up.float(), dn.float(), w, idx, dy.float())
    tol = dict(rtol=2e-3, atol_frac=2e-3) if grad_dtype == torch.float32 else {}
    _scaled_close(dx, ex, "dx", **tol)
    _scaled_close(d_up, eu, "d_up", **tol)
    _scaled_close(d_dn, ed, "d_down", **tol)
    _scaled_close(dg, eg, "dg", rtol=2e-3, atol_frac=2e-3)
    untouched = torch.ones(n, dtype=torch.bool)
    untouched[idx.long().unique()] = False
    assert not d_up.cpu()[untouched].any() and not d_dn.cpu()[untouched].any()
    # compact rows = the touched rows of the dense tables, in ascending expert order
    dx2, cu, cd, dg2, ids = expert_backward(dy.cuda(), x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(),
                                            grad_dtype=grad_dtype, compact=True)
    assert torch.equal(ids.cpu().long(), idx.long().unique())
    assert torch.equal(cu, d_up[ids.long()]) and torch.equal(cd, d_dn[ids.long()])
    assert torch.equal(dx2, dx) and torch.equal(dg2, dg), "two runs must agree bit for bit"


def test_expert_op_autograd_skewed():
    """Through the drop-in op with autograd, on a routing table where one expert owns most pairs."""
    from omni_moe.ops.triton import triton_omni_expert_func
    t, h, n, k = 512, 256, 64, 8
    x, up, dn, w, idx, dy = _expert_inputs(t, h, n, k, 11)
    idx[:, :6] = 3
    cx, cu, cd = (v.cuda().requires_grad_(True) for v in (x, up, dn))
    cw = w.bfloat16().cuda().requires_grad_(True)
    y = triton_omni_expert_func(cx, cu, cd, cw, idx.cuda())
    y.backward(dy.cuda())
    ex, eu, ed, eg = orc.expert_backward(x.float(), up.float(), dn.float(), w.bfloat16().float(), idx, dy.float())
    _scaled_close(cx.grad, ex, "dx")
    _scaled_close(cu.grad, eu, "d_up")
    _scaled_close(cd.grad, ed, "d_down")
    _scaled_close(cw.grad, eg, "dg")
    assert cu.grad.dtype == torch.bfloat16 and cw.grad.dtype == torch.bfloat16


@pytest.mark.parametrize("r,c", [(64, 64), (257, 72), (1, 8), (300, 1026), (4096, 1024)])
def test_transpose_padded(r, c):
    from omni_moe_b200.ops.autograd import transpose_padded
    src = torch.randn(r, c, generator=gen(r + c)).bfloat16()
    out = transpose_padded(src.cuda()).cpu()
    rp = (r + 7) // 8 * 8
    assert out.shape == (c, rp)
    assert torch.equal(out[:, :r], src.t()) and not out[:, r:].any()
    wide = torch.full((c, 2 * rp + 8), 7.0, dtype=torch.bfloat16, device="cuda")
    transpose_padded(src.cuda(), wide[:, 8:8 + rp])
    assert torch.equal(wide[:, 8:8 + r].cpu(), src.t()) and bool((wide[:, :8] == 7).all()) and bool((wide[:, 8 + rp:] == 7).all())


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 200, 72), (1, 8, 8), (4096, 1024, 4096), (1000, 8192, 264), (513, 24, 1032)])
def test_gemm_nt_matches_fp32(m, n, k):
    from omni_moe_b200.ops.autograd import gemm_nt
    g = gen(m + n + k)
    a = (torch.randn(m, k, generator=g) * 0.5).bfloat16()
    b = (torch.randn(n, k, generator=g) * (1.0 / k ** 0.5)).bfloat16()
    out = gemm_nt(a.cuda(), b.cuda())
    ref = a.float() @ b.float().t()
    _scaled_close(out, ref, "gemm_nt", rtol=1e-2, atol_frac=4e-3)


@pytest.mark.parametrize("t,h,i", [(64, 64, 128), (300, 256, 1024), (257, 1024, 4096), (1000, 72, 264), (1, 8, 8)])
def test_mlp_backward_matches_oracle(t, h, i):
    from omni_moe_b200.ops.autograd import mlp_backward
    g = gen(t + h + i)
    x = (torch.randn(t, h, generator=g)).bfloat16()
    wg = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wu = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wd = (torch.randn(h, i, generator=g) / i ** 0.5).bfloat16()
    dy = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    dx, dwg, dwu, dwd = mlp_backward(dy.cuda(), x.cuda(), wg.cuda(), wu.cuda(), wd.cuda())
    ex, eg, eu, ed = orc.mlp_backward(x.float(), wg.float(), wu.float(), wd.float(), dy.float())
    # the training forward saves gate | up from its epilogue: same values as x Wg^T, x Wu^T rounded to bf16
    from omni_moe_b200.ops import mlp_forward
    gu = torch.empty(t, 2 * i, dtype=torch.bfloat16, device="cuda")
    y = mlp_forward(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda(), gate_up=gu)
    _scaled_close(gu[:, :i], x.float() @ wg.float().t(), "saved gate", rtol=1e-2, atol_frac=4e-3)
    _scaled_close(gu[:, i:], x.float() @ wu.float().t(), "saved up", rtol=1e-2, atol_frac=4e-3)
    assert torch.equal(y, mlp_forward(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda())), "saving must not change the output"
    dx2, _, _, dwd2 = mlp_backward(dy.cuda(), x.cuda(), wg.cuda(), wu.cuda(), wd.cuda(), gate_up=gu)
    _scaled_close(dx2, ex, "dx (saved gate/up)", rtol=3e-2, atol_frac=2e-2)
    _scaled_close(dwd2, ed, "d_down_weight (saved gate/up)", rtol=3e-2, atol_frac=2e-2)
    # intermediates (gate, up, dact, dgate, dup) are rounded to bf16 between the GEMMs, as in the reference's bf16 path
    _scaled_close(dx, ex, "dx", rtol=3e-2, atol_frac=2e-2)
    _scaled_close(dwg, eg, "d_gate_weight", rtol=3e-2, atol_frac=2e-2)
    _scaled_close(dwu, eu, "d_up_weight", rtol=3e-2, atol_frac=2e-2)
    _scaled_close(dwd, ed, "d_down_weight", rtol=3e-2, atol_frac=2e-2)


@pytest.mark.parametrize("t,h,i,limit", [(300, 256, 1024, 0.75), (257, 1024, 4096, 1.5), (77, 72, 200, 0.3), (64, 64, 128, 7.0)])
def test_mlp_limit_forward_and_backward(t, h, i, limit):
    """The clamp of the reference's fused activation (omni_moe/ops/triton/omni_mlp.py:54-61): gate and up limited
    to [-limit, limit] in the forward, no gradient through clamped entries in the backward."""
    from omni_moe_b200.ops import mlp_forward, omni_mlp_func
    from omni_moe_b200.ops.autograd import mlp_backward
    g = gen(t + i)
    x = torch.randn(t, h, generator=g).bfloat16()
    wg = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wu = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wd = (torch.randn(h, i, generator=g) / i ** 0.5).bfloat16()
    dy = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    gate = x.float() @ wg.float().t()
    clamped = float((gate.abs() > limit).float().mean())
    assert (clamped > 0.04) == (limit < 2.0), "the case must exercise the clamp (or, for the wide limit, not)"
    cx, cg, cu, cd = x.cuda(), wg.cuda(), wu.cuda(), wd.cuda()
    exp = orc.mlp_forward(x, wg, wu, wd, limit=limit)
    gu = torch.empty(t, 2 * i, dtype=torch.bfloat16, device="cuda")
    y = mlp_forward(cx, cg, cu, cd, gate_up=gu, limit=limit)
    assert_close(y, exp, what="mlp with limit")
    assert torch.equal(y, mlp_forward(cx, cg, cu, cd, limit=limit)), "saving must not change the output"
    assert torch.equal(y, omni_mlp_func(cx, cg, cu, cd, limit=limit))
    if clamped > 0.04:
        assert not torch.allclose(y.float().cpu(), orc.mlp_forward(x, wg, wu, wd), rtol=2e-2, atol=2e-2), "the clamp must matter here"
    # the saved pre-activations are the unclamped ones
    _scaled_close(gu[:, :i], gate, "saved gate", rtol=1e-2, atol_frac=4e-3)
    # which entries are clamped (a jump of the gradient) is decided on the bf16 pre-activations, as in the reference
    ex, eg, eu, ed = orc.mlp_backward(x.float(), wg.float(), wu.float(), wd.float(), dy.float(), limit=limit,
                                      preact_dtype=torch.bfloat16)
    for gate_up in (gu, None):
        dx, dwg, dwu, dwd = mlp_backward(dy.cuda(), cx, cg, cu, cd, gate_up=gate_up, limit=limit)
        for got, want, name in ((dx, ex, "dx"), (dwg, eg, "d_gate_weight"), (dwu, eu, "d_up_weight"), (dwd, ed, "d_down_weight")):
            _scaled_close(got, want, f"{name} (limit {limit})", rtol=3e-2, atol_frac=2e-2)
    # through autograd, limit passed positionally like the other arguments
    ax, ag, au, ad = (v.clone().requires_grad_(True) for v in (cx, cg, cu, cd))
    omni_mlp_func(ax, ag, au, ad, limit).backward(dy.cuda())
    for got, want, name in ((ax.grad, ex, "dx"), (ag.grad, eg, "dwg"), (au.grad, eu, "dwu"), (ad.grad, ed, "dwd")):
        _scaled_close(got, want, f"autograd {name} (limit {limit})", rtol=3e-2, atol_frac=2e-2)


def test_mlp_limit_arguments_are_checked():
    from omni_moe_b200 import _lib
    lib = _lib.load()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    rc = lib.omni_mlp_gate_up_limit(a.data_ptr(), a.data_ptr(), a.data_ptr(), 8, 8, 8, -1.0, a.data_ptr(), None, st.data_ptr(), None)
    assert rc < 0 and b"limit" in lib.omni_last_error()
    rc = lib.omni_mlp_gate_up_limit(a.data_ptr(), a.data_ptr(), a.data_ptr(), 8, 8, 8, float("nan"), a.data_ptr(), None, st.data_ptr(), None)
    assert rc < 0
    with pytest.raises(AssertionError):
        from omni_moe_b200.ops import mlp_forward
        mlp_forward(a, a, a, a, limit=0.0)


@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (300, 200, 72), (8, 8, 8), (1000, 1032, 264), (4096, 1024, 4096), (129, 520, 1000)])
def test_gemm_with_transposed_operands(m, n, k, a_t, b_t):
    """Operands given as [k, m] / [k, n] are fed to the tensor cores as MN-major tiles: same product."""
    from omni_moe_b200.ops.autograd import gemm
    if (a_t and m % 8) or (b_t and n % 8):
        pytest.skip("a transposed operand's rows (m or n elements) must be whole 16-byte pieces")
    g = gen(m + n + k)
    a = torch.randn(m, k, generator=g).bfloat16()
    b = torch.randn(n, k, generator=g).bfloat16()
    want = a.float() @ b.float().t()
    ca = (a.t().contiguous() if a_t else a).cuda()
    cb = (b.t().contiguous() if b_t else b).cuda()
    out = gemm(ca, cb, a_t, b_t)
    _lib_status_ok()
    _scaled_close(out, want, f"gemm a_t={a_t} b_t={b_t}", rtol=1e-2, atol_frac=4e-3)
    # operands that are column slices of wider matrices (row stride > row length), output likewise
    wide_a = torch.zeros(ca.size(0), ca.size(1) + 16, dtype=torch.bfloat16, device="cuda")
    wide_a[:, 8:8 + ca.size(1)] = ca
    wide_b = torch.zeros(cb.size(0), cb.size(1) + 24, dtype=torch.bfloat16, device="cuda")   # row strides stay multiples of 8
    wide_b[:, 16:16 + cb.size(1)] = cb
    wide_o = torch.full((m, n + 8), 7.0, dtype=torch.bfloat16, device="cuda")
    gemm(wide_a[:, 8:8 + ca.size(1)], wide_b[:, 16:16 + cb.size(1)], a_t, b_t, out=wide_o[:, :n])
    assert torch.equal(wide_o[:, :n], out) and bool((wide_o[:, n:] == 7.0).all())


def _lib_status_ok():
    from omni_moe_b200 import _lib
    _lib.check_device_status()


def test_gemm_transposed_any_k():
    from omni_moe_b200.ops.autograd import gemm
    g = gen(77)
    for k in (1, 5, 63, 65, 1001):
        a = torch.randn(k, 136, generator=g).bfloat16()
        b = torch.randn(k, 72, generator=g).bfloat16()
        out = gemm(a.cuda(), b.cuda(), True, True)
        _scaled_close(out, a.float().t() @ b.float(), f"k={k}", rtol=1e-2, atol_frac=4e-3)


@pytest.mark.parametrize("m,n,k0,k1", [(256, 256, 64, 64), (300, 1024, 4096, 4096), (129, 72, 128, 40), (64, 520, 192, 1000)])
def test_gemm_with_b_stacked_along_k(m, n, k0, k1):
    """out = A (b0 ; b1) with the two transposed B matrices read in place."""
    from omni_moe_b200 import _lib
    g = gen(m + n + k0 + k1)
    k = k0 + k1
    a = torch.randn(m, k, generator=g).bfloat16()
    b0 = torch.randn(k0, n, generator=g).bfloat16()
    b1 = torch.randn(k1, n, generator=g).bfloat16()
    want = a.float() @ torch.cat((b0, b1), 0).float()
    ca, c0, c1 = a.cuda(), b0.cuda(), b1.cuda()
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    st = _lib.device_status(out.device)
    _lib.check(_lib.load().omni_gemm_bf16_stacked_b(ca.data_ptr(), 0, k, c0.data_ptr(), c1.data_ptr(), k0, n, m, n, k, out.data_ptr(), n,
                                                    st.data_ptr(), _lib.stream_ptr()))
    _lib.check_device_status()
    _scaled_close(out, want, "stacked B", rtol=1e-2, atol_frac=4e-3)


@pytest.mark.parametrize("t,h,i", [(300, 256, 1024), (77, 72, 264)])
def test_mlp_backward_routes_agree(t, h, i, monkeypatch):
    """Operands read in place (default) and the route through transposed copies give the same gradients up to
    the bf16 rounding of the intermediates."""
    from omni_moe_b200.ops.autograd import mlp_backward
    g = gen(t * 3 + i)
    x = torch.randn(t, h, generator=g).bfloat16().cuda()
    wg = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16().cuda()
    wu = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16().cuda()
    wd = (torch.randn(h, i, generator=g) / i ** 0.5).bfloat16().cuda()
    dy = (torch.randn(t, h, generator=g) * 0.5).bfloat16().cuda()
    monkeypatch.delenv("OMNI_MOE_B200_MLP_BWD", raising=False)
    in_place = mlp_backward(dy, x, wg, wu, wd)
    monkeypatch.setenv("OMNI_MOE_B200_MLP_BWD", "copies")
    copies = mlp_backward(dy, x, wg, wu, wd)
    for a, b, name in zip(in_place, copies, ("dx", "d_gate", "d_up", "d_down")):
        _scaled_close(a, b, name, rtol=1e-2, atol_frac=4e-3)


def test_gemm_first_call_on_a_fresh_thread():
    """The tensor-map encode is a driver call: it must also work on a thread that has not touched CUDA yet
    (the autograd engine runs the backward on such a thread)."""
    import threading
    from omni_moe_b200.ops.autograd import gemm
    g = gen(3)
    a = torch.randn(64, 136, generator=g).bfloat16().cuda()
    b = torch.randn(64, 72, generator=g).bfloat16().cuda()
    torch.cuda.synchronize()
    box = {}

    def work():
        try:
            box["out"] = gemm(a, b, True, True)
            torch.cuda.synchronize()
        except Exception as e:  # noqa: BLE001
            box["err"] = e
    th = threading.Thread(target=work)
    th.start()
    th.join()
    assert "err" not in box, box.get("err")
    _scaled_close(box["out"], a.float().t() @ b.float(), "gemm on a fresh thread", rtol=1e-2, atol_frac=4e-3)


def test_mlp_op_autograd():
    from omni_moe.ops.triton import triton_omni_mlp_func
    t, h, i = 200, 128, 512
    g = gen(5)
    x = torch.randn(t, h, generator=g).bfloat16()
    wg = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wu = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wd = (torch.randn(h, i, generator=g) / i ** 0.5).bfloat16()
    dy = torch.randn(t, h, generator=g).bfloat16()
    cx, cg, cu, cd = (v.cuda().requires_grad_(True) for v in (x, wg, wu, wd))
    y = triton_omni_mlp_func(cx, cg, cu, cd)
    y.backward(dy.cuda())
    ex, eg, eu, ed = orc.mlp_backward(x.float(), wg.float(), wu.float(), wd.float(), dy.float())
    for got, exp, name in ((cx.grad, ex, "dx"), (cg.grad, eg, "dwg"), (cu.grad, eu, "dwu"), (cd.grad, ed, "dwd")):
        assert got.dtype == torch.bfloat16
        _scaled_close(got, exp, name, rtol=3e-2, atol_frac=2e-2)


@pytest.mark.parametrize("training", [True, False])
def test_layer_gradients_match_oracle(training):
    """The module's differentiable forward + backward against fp32 autograd with the same routing."""
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(0)
    h, i, n_exp, k, t = 128, 256, 256, 8, 384
    m = OmniMoE(OmniMoEConfig(h, i, "silu", n_exp, k)).to(torch.bfloat16)
    with torch.no_grad():
        m.up_embed.weight.mul_(0.2)     # N(0,1) rows would saturate the SiLU of a 128-wide dot product
        m.down_embed.weight.mul_(0.2)
    sd = {kk: (v.float().clone() if v.is_floating_point() else v.clone()) for kk, v in m.state_dict().items()}
    p = orc.params_from_state_dict(sd, n_exp, k)
    m = m.cuda()
    m.train(training)
    x = torch.randn(1, t, h, generator=gen(1)).bfloat16()
    dy = (torch.randn(1, t, h, generator=gen(2)) * 0.1).bfloat16()
    cx = x.cuda().requires_grad_(True)
    y = m(cx)
    assert y.requires_grad and y.dtype == torch.bfloat16
    y.backward(dy.cuda())
    scores, indices, weights = m.last_routing
    ey, eg = orc.layer_gradients(p, x.float(), indices.cpu(), dy.float(), training)
    _scaled_close(y.reshape(-1, h), ey, "y", rtol=3e-2, atol_frac=2e-2)
    got = {name: prm.grad for name, prm in m.named_parameters()}
    got["x"] = cx.grad.reshape(-1, h)
    for name, exp in eg.items():
        # router-gate gradients pass through bf16 log-probs, scores and BatchNorm: looser
        loose = name.startswith("router_gate")
        _scaled_close(got[name], exp, name, rtol=1e-1 if loose else 4e-2, atol_frac=6e-2 if loose else 3e-2)


@pytest.mark.parametrize("split", [True, 64, 128, 256, 512])
@pytest.mark.parametrize("layout", ["one_giant", "aligned_512", "mixed"])
def test_expert_backward_long_segments(layout, split):
    """Experts with more pairs than one block of sorted positions take the two-level path; it must agree
    with the single-warp path (same products, another summation order) and with the oracle, and be
    reproducible, for every block size."""
    from omni_moe_b200.ops.autograd import expert_backward
    t, h, n, k = 640, 264, 40, 4
    x, up, dn, w, idx, dy = _expert_inputs(t, h, n, k, 21)
    flat = idx.view(-1)
    if layout == "one_giant":
        flat[: 2300] = 7                       # 2300+ pairs on expert 7, crossing four 512-blocks
    elif layout == "aligned_512":
        flat[:] = torch.arange(t * k, dtype=torch.int32) // 512      # five experts, exactly 512 pairs each: none is "long"
        flat[: 1024] = 0                       # ... except expert 0 with 1024 = blocks 0 and 1 exactly
    else:
        flat[: 600] = 3
        flat[600: 1300] = 5
        flat[1300: 1813] = 9                   # 513 pairs: just over the threshold
    got = expert_backward(dy.cuda(), x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), grad_dtype=torch.float32,
                          long_segments=split)
    slow = expert_backward(dy.cuda(), x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), grad_dtype=torch.float32,
                           long_segments=False)
    ex, eu, ed, eg = orc.expert_backward(x.float(), up.float(), dn.float(), w, idx, dy.float())
    for name, a, b, e in (("d_up", got[1], slow[1], eu), ("d_down", got[2], slow[2], ed)):
        _scaled_close(a, e, name, rtol=2e-3, atol_frac=2e-3)
        _scaled_close(a, b, name + " vs single-warp path", rtol=1e-4, atol_frac=1e-5)
    again = expert_backward(dy.cuda(), x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), grad_dtype=torch.float32,
                            long_segments=split)
    assert torch.equal(again[1], got[1]) and torch.equal(again[2], got[2])
    cu = expert_backward(dy.cuda(), x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), grad_dtype=torch.bfloat16, compact=True,
                         long_segments=split)
    assert torch.equal(cu[1].float(), got[1][cu[4].long()].bfloat16().float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_layer_trains_in_other_dtypes(dtype):
    """fp32 / fp16 modules: operands are rounded to bf16 for the kernels, gradients come back in the
    parameter dtype and match fp32 autograd on the bf16-rounded operands."""
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    torch.manual_seed(1)
    h, i, n_exp, k, t = 64, 128, 64, 4, 96
    m = OmniMoE(OmniMoEConfig(h, i, "silu", n_exp, k))
    with torch.no_grad():
        m.up_embed.weight.mul_(0.3)
        m.down_embed.weight.mul_(0.3)
    m = m.to(dtype)
    sd = {kk: (v.to(torch.bfloat16).float().clone() if v.is_floating_point() and "running" not in kk else v.clone())
          for kk, v in m.state_dict().items()}
    p = orc.params_from_state_dict({kk: (v.float() if v.is_floating_point() else v) for kk, v in sd.items()}, n_exp, k)
    m = m.cuda().train()
    x = torch.randn(1, t, h, generator=gen(3)).to(dtype)
    dy = (torch.randn(1, t, h, generator=gen(4)) * 0.1).to(dtype)
    cx = x.cuda().requires_grad_(True)
    y = m(cx)
    assert y.dtype == dtype
    y.backward(dy.cuda())
    _, eg = orc.layer_gradients(p, x.to(torch.bfloat16).float(), m.last_routing[1].cpu(), dy.float(), True)
    for name, prm in m.named_parameters():
        assert prm.grad is not None and prm.grad.dtype == dtype, name
        if not name.startswith("router_gate"):   # the gates see the unrounded fp32 / fp16 x through nn.Linear
            _scaled_close(prm.grad, eg[name], name, rtol=5e-2, atol_frac=4e-2)
    assert cx.grad.dtype == dtype


def test_backward_faults_surface_through_the_device_status():
    """An out-of-range expert index in the backward is skipped by the kernels and reported (no trap):
    the shared per-device status word collects it and check_device_status() raises once."""
    from omni_moe_b200 import _lib
    from omni_moe_b200.ops.autograd import expert_backward
    _lib.check_device_status()        # start clean
    x, up, dn, w, idx, dy = _expert_inputs(16, 64, 32, 4, 5)
    idx[2, 1] = 999
    dx, d_up, d_dn, dg, _ = expert_backward(dy.cuda(), x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), grad_dtype=torch.float32)
    with pytest.raises(RuntimeError, match="expert index"):
        _lib.check_device_status()
    _lib.check_device_status()        # cleared by the report
    assert bool(torch.isfinite(dx).all()) and float(dg[2, 1]) == 0.0


@pytest.mark.parametrize("t,h,n,k,training", [(300, 64, 16, 4, True), (300, 64, 16, 4, False), (1000, 128, 64, 16, True),
                                                (257, 256, 256, 32, True), (129, 256, 256, 16, False), (5, 64, 40, 6, True)])
def test_router_front_operator_matches_fp32_autograd(t, h, n, k, training):
    """gates -> BatchNorm -> log-softmax -> selection as one operator: forward scores / indices and the
    gradients of x and both gate matrices against fp32 torch autograd fed with the same selection."""
    import torch.nn.functional as F
    from omni_moe_b200.ops.autograd import RouterFrontFunction
    g = gen(t + n + k)
    x = torch.randn(t, h, generator=g).bfloat16()
    kx = (torch.randn(n, h, generator=g) / h ** 0.5).bfloat16()
    ky = (torch.randn(n, h, generator=g) / h ** 0.5).bfloat16()
    run_mean = torch.randn(2 * n, generator=g) * 0.1
    run_var = torch.rand(2 * n, generator=g) + 0.5
    ds = torch.randn(t, k, generator=g)
    eps = 1e-5
    state = {}

    def fold(logits):
        if training:
            var, mean = torch.var_mean(logits, dim=0, unbiased=False)
        else:
            mean, var = run_mean.cuda(), run_var.cuda()
        scale = torch.rsqrt(var + eps)
        state["fold"] = (scale, -mean * scale)
        return scale.contiguous(), (-mean * scale).contiguous()

    cx, ckx, cky = (v.cuda().requires_grad_(True) for v in (x, kx, ky))
    scores, indices = RouterFrontFunction.apply(cx, ckx, cky, k, fold, training)
    (scores * ds.cuda()).sum().backward()
    # fp32 reference with the same indices
    rx, rkx, rky = (v.float().requires_grad_(True) for v in (x, kx, ky))
    z = torch.cat([rx @ rkx.t(), rx @ rky.t()], dim=1)
    if training:
        var, mean = torch.var_mean(z, dim=0, unbiased=False)
    else:
        mean, var = run_mean, run_var
    zh = (z - mean) / torch.sqrt(var + eps)
    lp = torch.cat([F.log_softmax(zh[:, :n], -1), F.log_softmax(zh[:, n:], -1)], dim=1)
    idx = indices.cpu().long()
    ref_scores = lp.gather(1, idx // n) + lp.gather(1, n + idx % n)
    (ref_scores * ds).sum().backward()
    torch.testing.assert_close(scores.cpu(), ref_scores.detach(), rtol=2e-3, atol=2e-3)
    assert bool((scores[:, :-1] >= scores[:, 1:]).all())
    for got, ref, name in ((cx.grad, rx.grad, "dx"), (ckx.grad, rkx.grad, "dKx"), (cky.grad, rky.grad, "dKy")):
        assert got.dtype == torch.bfloat16
        _scaled_close(got, ref, name, rtol=5e-2, atol_frac=3e-2)
    # reproducible
    cx2, ckx2, cky2 = (v.cuda().requires_grad_(True) for v in (x, kx, ky))
    s2, i2 = RouterFrontFunction.apply(cx2, ckx2, cky2, k, fold, training)
    (s2 * ds.cuda()).sum().backward()
    assert torch.equal(i2, indices) and torch.equal(cx2.grad, cx.grad) and torch.equal(ckx2.grad, ckx.grad)
