"""Routed-expert kernels against the fp32 oracle (bf16 operands, rtol/atol 2e-2)."""
import os

import numpy as np
import pytest
import torch

from oracle import omni_oracle as orc
from _util import assert_close, bf16_round, gen, zipf_indices

pytestmark = pytest.mark.gpu


def _inputs(t, h, n, k, seed, idx=None):
    g = gen(seed)
    x = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    up = (torch.randn(n, h, generator=g) * 0.1).bfloat16()
    dn = (torch.randn(n, h, generator=g) * 0.1).bfloat16()
    w = torch.randn(t, k, generator=g) * 0.1
    if idx is None:
        idx = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)  # duplicates allowed
    return x, up, dn, w, idx


@pytest.mark.parametrize("t,h,n,k", [(32, 64, 128, 8), (300, 256, 1024, 8), (257, 1024, 4096, 16), (64, 2048, 512, 32),
                                       (40, 4096, 300, 64), (50, 72, 64, 6), (33, 1536, 200, 4), (20, 8192, 64, 2),
                                       (1, 8, 1, 1)])
@pytest.mark.parametrize("mode", ["scheduled", "fused"])
def test_expert_matches_oracle(t, h, n, k, mode):
    from omni_moe_b200.ops import expert_forward
    if mode == "fused" and h > 2048:
        with pytest.raises(RuntimeError, match="hidden <= 2048"):
            x, up, dn, w, idx = _inputs(4, h, 8, 2, 0)
            expert_forward(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), mode="fused")
        return
    x, up, dn, w, idx = _inputs(t, h, n, k, t + h)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    for out_dtype in (torch.float32, torch.bfloat16):
        y, coef = expert_forward(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), out_dtype=out_dtype,
                                 status=st, return_coef=True, mode=mode)
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        ey = orc.expert_forward(x, up, dn, w, idx)
        ec = orc.expert_coefficients(x, up, w, idx)
        assert_close(coef, ec, rtol=1e-3, atol=1e-4, what="coefficients")
        if out_dtype == torch.float32:
            assert_close(y, ey, rtol=1e-3, atol=1e-4, what="fp32 output")
        else:
            assert_close(y, ey, what="bf16 output")


@pytest.mark.parametrize("mode", ["scheduled", "fused"])
def test_expert_residual_and_determinism(mode):
    from functools import partial
    from omni_moe_b200 import ops
    expert_forward = partial(ops.expert_forward, mode=mode)
    x, up, dn, w, idx = _inputs(100, 512, 256, 8, 3)
    res = torch.randn(100, 512, generator=gen(4))
    a = expert_forward(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), out_dtype=torch.float32, residual=res.cuda())
    b = expert_forward(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), out_dtype=torch.float32, residual=res.cuda())
    assert torch.equal(a, b)  # no atomics: bit-identical from run to run
    assert_close(a, orc.expert_forward(x, up, dn, w, idx) + res, rtol=1e-3, atol=1e-4)
    rb = res.bfloat16()
    inplace = rb.cuda().clone()   # residual and output may be one buffer
    from omni_moe_b200 import _lib
    lib, st = _lib.load(), torch.zeros(1, dtype=torch.int32, device="cuda")
    xc, uc, dc, wc, ic = x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda()
    if mode == "fused":
        _lib.check(lib.omni_expert_fused(xc.data_ptr(), uc.data_ptr(), dc.data_ptr(), wc.data_ptr(), ic.data_ptr(), 100, 8,
                                         512, 256, inplace.data_ptr(), inplace.data_ptr(), 1, None, st.data_ptr(),
                                         _lib.stream_ptr()))
        assert_close(inplace, orc.expert_forward(x, up, dn, w, idx) + rb.float())
    c = expert_forward(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), out_dtype=torch.bfloat16, residual=rb.cuda())
    assert_close(c, orc.expert_forward(x, up, dn, w, idx) + rb.float())


@pytest.mark.parametrize("mode", ["scheduled", "fused"])
def test_expert_skewed_routing(mode):
    # hot experts: thousands of pairs on one expert, duplicates inside tokens
    t, h, n, k = 2048, 256, 4096, 32
    idx = zipf_indices(t, k, n, 1.1, 5)
    x, up, dn, w, _ = _inputs(t, h, n, k, 6)
    w = torch.distributions.Dirichlet(torch.ones(k)).sample((t,))
    from omni_moe_b200.ops import expert_forward
    y = expert_forward(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), out_dtype=torch.bfloat16, mode=mode)
    assert_close(y, orc.expert_forward(x, up, dn, w, idx))


def test_expert_golden_mirror_and_drop_in(golden_dir):
    g = np.load(os.path.join(golden_dir, "expert_mirror.npz"))
    from omni_moe.ops.triton import triton_omni_expert_func
    args = [torch.from_numpy(g[k]) for k in ("x", "up", "down", "w", "indices")]
    # fp32 call: float32 arithmetic end to end, so the reference's own fp32 output is matched tightly
    y = triton_omni_expert_func(*[a.cuda() for a in args])
    assert y.dtype == torch.float32
    assert_close(y, torch.from_numpy(g["y"]), rtol=1e-4, atol=1e-5, what="fp32 operator vs the reference mirror's output")
    x, up, dn, w, idx = args
    # the bf16 kernels on the rounded operands, against the oracle evaluated on the same rounded operands
    from omni_moe_b200.ops import expert_forward
    y32 = expert_forward(x.bfloat16().cuda(), up.bfloat16().cuda(), dn.bfloat16().cuda(), w.cuda(), idx.cuda(), out_dtype=torch.float32)
    assert_close(y32, orc.expert_forward(bf16_round(x), bf16_round(up), bf16_round(dn), w, idx), rtol=1e-3, atol=1e-4)
    yb = triton_omni_expert_func(x.bfloat16().cuda(), up.bfloat16().cuda(), dn.bfloat16().cuda(), w.bfloat16().cuda(), idx.cuda())
    assert yb.dtype == torch.bfloat16


@pytest.mark.parametrize("mode", ["scheduled", "fused"])
def test_expert_bad_index_is_reported_not_faulting(mode):
    from omni_moe_b200.ops import expert_forward
    x, up, dn, w, idx = _inputs(16, 64, 32, 4, 8)
    idx[3, 2] = 1000
    idx[5, 0] = -7
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = expert_forward(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), out_dtype=torch.float32, status=st, mode=mode)
    torch.cuda.synchronize()
    assert int(st.item()) & 1
    good = torch.ones(16, dtype=torch.bool)
    good[3] = good[5] = False
    ey = orc.expert_forward(x, up, dn, w, idx.clamp(0, 31))
    assert_close(y[good.cuda()], ey[good], rtol=1e-3, atol=1e-4)


def test_expert_stress_shape_properties():
    # a slice of the skewed stress configuration (hidden 2048, 262144 experts, k = 32, Zipf 1.1):
    # linearity in the routing weights and agreement with the oracle on sampled tokens
    t, h, n, k = 4096, 2048, 262144, 32
    g = gen(0)
    x = torch.randn(t, h, generator=g).bfloat16()
    up = (torch.randn(n, h, generator=g) * 0.02).bfloat16()
    dn = (torch.randn(n, h, generator=g) * 0.02).bfloat16()
    idx = zipf_indices(t, k, n, 1.1, 0)
    w = torch.distributions.Dirichlet(torch.ones(k)).sample((t,))
    from omni_moe_b200.ops import expert_forward
    xc, uc, dc, ic = x.cuda(), up.cuda(), dn.cuda(), idx.cuda()
    y1 = expert_forward(xc, uc, dc, w.cuda(), ic, out_dtype=torch.float32)
    y2 = expert_forward(xc, uc, dc, (2 * w).cuda(), ic, out_dtype=torch.float32)
    assert_close(y2, 2 * y1, rtol=1e-5, atol=1e-7, what="linearity in the weights")
    sel = torch.arange(0, t, 64)
    ey = orc.expert_forward(x[sel], up, dn, w[sel], idx[sel])
    assert_close(y1[sel.cuda()], ey, rtol=1e-3, atol=1e-4)


def _mma_shape(h, n, k):
    """Shapes whose dot products the routed kernel runs on the tensor cores (the others stay on the CUDA cores)."""
    return h in (256, 512, 1024) and os.environ.get("OMNI_MOE_B200_ROUTED", "")[:1] != "l"


@pytest.mark.parametrize("t,h,n,k", [(300, 256, 32, 8), (257, 1024, 64, 16), (100, 512, 100, 24), (64, 2048, 16, 32),
                                       (130, 72, 200, 2), (50, 128, 8, 30), (4103, 1024, 64, 16), (1, 128, 8, 2), (33, 640, 16, 5),
                                       (1000, 384, 64, 12), (5000, 512, 32, 16), (2, 1024, 4, 16), (95, 896, 64, 1), (77, 1024, 128, 32),
                                       (64, 256, 200, 30), (40, 512, 16, 17)])
def test_routed_kernel_equals_separate_router_and_expert_kernels(t, h, n, k):
    """omni_route_expert_fused = omni_router_logits_topk followed by omni_expert_fused: the routing bit for bit;
    the output bit for bit from the one-warp-per-token kernel, and within bf16 rounding of it (and within the
    bf16 bar of the fp32 oracle) from the tensor-core kernel, whose sums run in another order."""
    from omni_moe_b200 import _lib
    from omni_moe_b200.ops import expert_forward, route_expert_fused
    g = gen(t + n + k)
    N = n * n
    x = (torch.randn(t, h, generator=g) * 0.5).bfloat16().cuda()
    up = (torch.randn(N, h, generator=g) * 0.1).bfloat16().cuda()
    dn = (torch.randn(N, h, generator=g) * 0.1).bfloat16().cuda()
    logits = torch.randn(t, 2 * n, generator=g).cuda()
    logits[::7] = 0.0  # some tokens where every score ties: exercises the exact re-scan inside the fused kernel
    scale = (torch.rand(2 * n, generator=g) + 0.5).cuda()
    shift = (torch.randn(2 * n, generator=g) * 0.1).cuda()
    res = torch.randn(t, h, generator=g).bfloat16().cuda()
    lib = _lib.load()
    sc = torch.empty(t, k, device="cuda")
    idx = torch.empty(t, k, device="cuda", dtype=torch.int32)
    w = torch.empty(t, k, device="cuda")
    lp = torch.empty(t, 2 * n, device="cuda")
    _lib.check(lib.omni_router_logits_topk(logits.data_ptr(), 2 * n, scale.data_ptr(), shift.data_ptr(), t, n, k,
                                           sc.data_ptr(), idx.data_ptr(), 0, w.data_ptr(), lp.data_ptr(), _lib.stream_ptr()))
    y_ref = expert_forward(x, up, dn, w, idx, out_dtype=torch.bfloat16, residual=res, mode="fused")
    y, sc2, idx2, w2 = route_expert_fused(logits, x, up, dn, k, scale, shift, residual=res)
    torch.cuda.synchronize()
    _lib.check_device_status()
    assert torch.equal(idx2, idx) and torch.equal(sc2, sc) and torch.equal(w2, w)
    mma = _mma_shape(h, n, k)

    def same_output(got):
        if not mma:
            assert torch.equal(got, y_ref)
            return
        # both round the same fp32 sum (up to its last bits) to bf16: at most one bf16 step apart
        assert_close(got, y_ref, rtol=2 ** -7, atol=1e-3, what="tensor-core routed kernel vs one-warp-per-token kernel")
        ey = orc.expert_forward(x.cpu(), up.cpu(), dn.cpu(), w.cpu(), idx.cpu()) + res.float().cpu()
        assert_close(got, ey, what="tensor-core routed kernel vs oracle")
        y_again, _, _, _ = route_expert_fused(logits, x, up, dn, k, scale, shift, residual=res)
        assert torch.equal(y_again, got), "the output must be identical run to run"

    same_output(y)
    # and the selection is the oracle's, given the log-probs the kernel computed
    es, ei = orc.router_topk(lp[:, :n].cpu().contiguous(), lp[:, n:].cpu().contiguous(), n, k)
    np.testing.assert_array_equal(idx2.cpu().numpy(), ei)
    # in place
    y_in = res.clone()
    _lib.check(lib.omni_route_expert_fused(logits.data_ptr(), 2 * n, scale.data_ptr(), shift.data_ptr(), x.data_ptr(),
                                           up.data_ptr(), dn.data_ptr(), t, n, k, h, N, y_in.data_ptr(), y_in.data_ptr(),
                                           None, None, None, None, _lib.stream_ptr()))
    torch.cuda.synchronize()
    same_output(y_in)


def test_routed_tensor_core_kernel_keeps_fp32_coefficients():
    """Only the operands of the dot products pass through the tensor cores; the coefficient w * silu(dot) stays in
    fp32.  With one expert per token, no residual and Down rows that are all 0.75 the output is
    bf16(coefficient x 0.75): a coefficient cut to bf16 would round differently on a large share of the tokens."""
    from omni_moe_b200.ops import route_expert_fused
    t, h, n, k = 256, 256, 16, 1
    g = gen(5)
    x = (torch.randn(t, h, generator=g) * 0.5).bfloat16().cuda()
    up = (torch.randn(n * n, h, generator=g) * 0.1).bfloat16().cuda()
    dn = torch.full((n * n, h), 0.75).bfloat16().cuda()
    logits = torch.randn(t, 2 * n, generator=g).cuda()
    y, sc, idx, w = route_expert_fused(logits, x, up, dn, k)
    torch.cuda.synchronize()
    coef = orc.expert_coefficients(x.cpu(), up.cpu(), w.cpu(), idx.cpu())[:, 0]
    expect = (coef * 0.75).bfloat16().float()       # one rounding: of the exact product
    got = y.float().cpu()[:, 0]
    cut = (coef.bfloat16().float() * 0.75).bfloat16().float()
    assert (cut != expect).float().mean() > 0.1, "the inputs do not tell a truncated coefficient from a full one"
    assert (got == expect).float().mean() > 0.97, float((got == expect).float().mean())


def _sampled_oracle(x, up, dn, w, idx, sel):
    """fp32 oracle output for the tokens `sel` of device-resident inputs: only the table rows those tokens
    touch are copied to the host (the oracle indexes a compact table through remapped ids)."""
    isel = idx[sel].long()
    need = torch.unique(isel)
    compact = torch.searchsorted(need, isel.reshape(-1)).view(isel.shape)
    return orc.expert_forward(x[sel].float().cpu(), up[need].float().cpu(), dn[need].float().cpu(), w[sel].float().cpu(),
                              compact.cpu())


def _normal_on_device(shape, std, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = torch.empty(shape, device="cuda", dtype=torch.bfloat16)
    flat = out.view(-1)
    for s in range(0, flat.numel(), 1 << 27):
        e = min(flat.numel(), s + (1 << 27))
        flat[s:e] = (torch.randn(e - s, device="cuda", generator=g) * std).to(torch.bfloat16)
    return out


def test_expert_stress_shape_full_size_against_sampled_oracle():
    """The whole skewed stress configuration (32768 tokens, hidden 2048, 512 x 512 experts, k = 32, Zipf(1.1) with
    replacement, Dirichlet(1) weights, tables ~ N(0, 0.02)) through the scheduled path; every 128th token is
    recomputed by the oracle.  Also: the schedule puts the head expert's ~136 k pairs in one segment."""
    from omni_moe_b200.ops import expert_forward
    t, h, n, k = 32768, 2048, 262144, 32
    x = _normal_on_device((t, h), 1.0, 1)
    up = _normal_on_device((n, h), 0.02, 2)
    dn = _normal_on_device((n, h), 0.02, 3)
    idx = zipf_indices(t, k, n, 1.1, 0).cuda()
    w = torch.distributions.Dirichlet(torch.ones(k)).sample((t,)).to(torch.bfloat16).float().cuda()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    y, coef = expert_forward(x, up, dn, w, idx, out_dtype=torch.float32, status=st, return_coef=True, mode="scheduled")
    yb = expert_forward(x, up, dn, w, idx, out_dtype=torch.bfloat16, status=st, mode="scheduled")
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert int((idx == 0).sum()) > t, "the head expert owns more pairs than there are tokens (duplicates inside a token)"
    sel = torch.arange(0, t, 128, device="cuda")
    ey = _sampled_oracle(x, up, dn, w, idx, sel)
    assert_close(y[sel], ey, rtol=1e-3, atol=1e-4, what="stress shape, fp32 output")
    assert_close(yb[sel], ey, what="stress shape, bf16 output")
    ec = orc.expert_coefficients(x[sel].float().cpu(), up[torch.unique(idx[sel].long())].float().cpu(), w[sel].cpu(),
                                 torch.searchsorted(torch.unique(idx[sel].long()), idx[sel].long().reshape(-1)).view(-1, k).cpu())
    assert_close(coef[sel], ec, rtol=1e-3, atol=1e-4, what="stress shape, coefficients")


def test_expert_largest_configuration_dimensions_against_sampled_oracle():
    """Expert path at the dimensions of the largest configuration (hidden 4096, k = 64, 2^20 experts: 8 GiB per
    table) on 4096 tokens: the 16-vector coefficient kernel and the two-slab combine at their real size; 64
    tokens are recomputed by the oracle from the rows they touch."""
    from omni_moe_b200.ops import expert_forward
    t, h, n, k = 4096, 4096, 1 << 20, 64
    free, _ = torch.cuda.mem_get_info()
    if free < 24 << 30:
        pytest.skip("needs 24 GiB of free device memory")
    x = _normal_on_device((t, h), 1.0, 4)
    up = _normal_on_device((n, h), 0.02, 5)
    dn = _normal_on_device((n, h), 0.02, 6)
    g = torch.Generator(device="cuda").manual_seed(7)
    idx = torch.randint(0, n, (t, k), device="cuda", dtype=torch.int32, generator=g)
    idx[:, 1] = idx[:, 0]                      # a duplicate inside every token
    idx[5, :] = n - 1                          # one token entirely on the last row
    w = torch.rand(t, k, device="cuda", generator=g) * 0.1
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = expert_forward(x, up, dn, w, idx, out_dtype=torch.float32, status=st, mode="scheduled")
    yb = expert_forward(x, up, dn, w, idx, out_dtype=torch.bfloat16, status=st, mode="scheduled")
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    sel = torch.cat([torch.arange(0, t, 65, device="cuda"), torch.tensor([5], device="cuda")])
    ey = _sampled_oracle(x, up, dn, w, idx, sel)
    assert_close(y[sel], ey, rtol=1e-3, atol=1e-4, what="largest configuration, fp32 output")
    assert_close(yb[sel], ey, what="largest configuration, bf16 output")
    del up, dn
    torch.cuda.empty_cache()


@pytest.mark.parametrize("t,h,n,k", [(300, 256, 1024, 8), (257, 1024, 4096, 16), (65, 512, 100, 32), (9, 1024, 40, 17), (1, 256, 1, 1)])
def test_fused_tensor_core_gather_matches_oracle(t, h, n, k):
    """omni_expert_fused with a bf16 output and no coefficient output, hidden 256 / 512 / 1024: the kernel whose dot
    products run on the tensor cores.  Against the oracle, with a residual, run to run identical, bad indices
    reported and skipped."""
    from omni_moe_b200.ops import expert_forward
    x, up, dn, w, idx = _inputs(t, h, n, k, t + h + 1)
    res = torch.randn(t, h, generator=gen(t)).bfloat16()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = (x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda())
    y = expert_forward(*args, out_dtype=torch.bfloat16, residual=res.cuda(), status=st, mode="fused")
    y2 = expert_forward(*args, out_dtype=torch.bfloat16, residual=res.cuda(), status=st, mode="fused")
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and torch.equal(y, y2)
    assert_close(y, orc.expert_forward(x, up, dn, w, idx) + res.float(), what="tensor-core gather, bf16 output")
    # the fp32 / coefficient-returning form is the CUDA-core kernel: the two agree to bf16 rounding
    y32 = expert_forward(*args, out_dtype=torch.float32, status=st, mode="fused")
    y16 = expert_forward(*args, out_dtype=torch.bfloat16, status=st, mode="fused")
    assert_close(y16, y32, rtol=2 ** -7, atol=1e-3, what="tensor-core vs CUDA-core gather")
    if t >= 9 and k >= 2:
        bad = idx.clone()
        bad[3, 1] = n + 5
        bad[5, 0] = -2
        yb = expert_forward(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), bad.cuda(), out_dtype=torch.bfloat16, status=st, mode="fused")
        torch.cuda.synchronize()
        assert int(st.item()) & 1
        wz = w.clone()
        wz[3, 1] = 0.0
        wz[5, 0] = 0.0
        assert_close(yb, orc.expert_forward(x, up, dn, wz, bad.clamp(0, n - 1)), what="bad indices are skipped")


@pytest.mark.parametrize("t,h,n,k", [(100, 256, 500, 8), (33, 1024, 4096, 32), (7, 4100, 64, 5), (64, 2048, 300, 128), (1, 4, 1, 1)])
def test_expert_float32_operands_are_computed_in_float32(t, h, n, k):
    """float32 tensors through the drop-in operator: float32 arithmetic end to end (omni_expert_fused_f32), checked
    against the fp32 oracle on the unrounded operands at rtol 1e-4 / atol 1e-5 - two orders below what bf16 operands
    give - with duplicates, a residual through the C ABI, and bad indices reported and skipped."""
    from omni_moe.ops.triton import triton_omni_expert_func
    from omni_moe_b200.ops.expert import expert_forward_f32
    g = gen(t + h + n)
    x = torch.randn(t, h, generator=g) * 0.5
    up = torch.randn(n, h, generator=g) * 0.1
    dn = torch.randn(n, h, generator=g) * 0.1
    w = torch.randn(t, k, generator=g) * 0.1
    idx = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
    if k > 1:
        idx[:, 1] = idx[:, 0]
    y = triton_omni_expert_func(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda())
    assert y.dtype == torch.float32
    ey = orc.expert_forward(x, up, dn, w, idx)
    assert_close(y, ey, rtol=1e-4, atol=1e-5, what="float32 expert operator")
    res = torch.randn(t, h, generator=g)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    y2 = expert_forward_f32(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), idx.cuda(), residual=res.cuda(), status=st)
    assert_close(y2, ey + res, rtol=1e-4, atol=1e-5, what="float32 expert kernel with residual")
    assert int(st.item()) == 0
    if t > 3:
        bad = idx.clone()
        bad[2, 0] = n
        yb = expert_forward_f32(x.cuda(), up.cuda(), dn.cuda(), w.cuda(), bad.cuda(), status=st)
        torch.cuda.synchronize()
        assert int(st.item()) & 1
        wz = w.clone()
        wz[2, 0] = 0.0
        assert_close(yb, orc.expert_forward(x, up, dn, wz, bad.clamp(0, n - 1)), rtol=1e-4, atol=1e-5)


def _hot_run(x, up, w, idx, n, min_run):
    """omni_expert_coef_hot through the C ABI; returns the coefficients and the ids it treated densely."""
    from omni_moe_b200 import _lib
    from omni_moe_b200.ops.scheduler import schedule
    lib = _lib.load()
    t, h = x.shape
    k = idx.size(1)
    sch = schedule(idx, n, segments=False)
    ws = torch.zeros(int(lib.omni_expert_coef_hot_workspace(t, h)), dtype=torch.uint8, device="cuda")
    coef = torch.full((t, k), float("nan"), device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(lib.omni_expert_coef_hot(x.data_ptr(), up.data_ptr(), w.data_ptr(), sch.sorted_pair_ids.data_ptr(),
                                        sch.sorted_experts.data_ptr(), t, k, h, n, min_run, coef.data_ptr(),
                                        ws.data_ptr(), ws.numel(), st.data_ptr(), _lib.stream_ptr()))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ids = ws[:65 * 4].view(torch.int32).cpu()
    count = int(ids[64])
    assert (ids[count:64] == 0x7fffffff).all()
    return coef, ids[:count].tolist()


def _plain_coef(x, up, w, idx, n):
    from omni_moe_b200 import _lib
    from omni_moe_b200.ops.scheduler import schedule
    lib = _lib.load()
    t, h = x.shape
    k = idx.size(1)
    sch = schedule(idx, n, segments=False)
    coef = torch.full((t, k), float("nan"), device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(lib.omni_expert_coef(x.data_ptr(), up.data_ptr(), w.data_ptr(), sch.sorted_pair_ids.data_ptr(),
                                    sch.sorted_experts.data_ptr(), t, k, h, n, coef.data_ptr(), st.data_ptr(),
                                    _lib.stream_ptr()))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return coef


@pytest.mark.parametrize("t,h,n,k,min_run", [(4096, 512, 4096, 8, 512), (1000, 264, 300, 6, 64), (2048, 4096, 512, 4, 128),
                                             (4099, 1024, 70000, 16, 0), (33, 264, 7, 4, 8), (129, 8, 3, 1, 16)])
def test_hot_experts_take_the_dense_products_and_agree_with_the_gathered_ones(t, h, n, k, min_run):
    """Skewed routing: the experts that fill a whole window of min_run sorted positions are found (every expert with
    2 * min_run - 1 pairs must be among them unless 64 others come first, none with fewer than min_run pairs may be),
    their pairs read the GEMM's products, and all coefficients agree with the gather-only kernel and the oracle."""
    x = (torch.randn((t, h), generator=gen(1)) * 1.0).cuda().to(torch.bfloat16)
    up = (torch.randn((n, h), generator=gen(2)) * 0.05).cuda().to(torch.bfloat16)
    idx = zipf_indices(t, k, n, 1.3, 7).cuda()
    w = (torch.randn((t, k), generator=gen(3)) * 1.0).abs().cuda()
    coef_hot, hot = _hot_run(x, up, w, idx, n, min_run)
    coef_plain = _plain_coef(x, up, w, idx, n)
    tau = min_run if min_run > 0 else max(512, t // 32)
    counts = torch.bincount(idx.reshape(-1).long().cpu(), minlength=n)
    assert hot == sorted(set(hot)), hot
    assert all(int(counts[e]) >= tau for e in hot), [(e, int(counts[e])) for e in hot]
    must = [e for e in range(n) if int(counts[e]) >= 2 * tau - 1]
    assert len(hot) > 0 and (len(hot) == 64 or set(must) <= set(hot)), (hot, must)
    assert_close(coef_hot, coef_plain, rtol=1e-4, atol=1e-5 * float(coef_plain.abs().max()) + 1e-6, what="hot vs gathered")
    is_hot = torch.isin(idx.cpu(), torch.tensor(hot, dtype=torch.int32))
    assert torch.equal(coef_hot.cpu()[~is_hot], coef_plain.cpu()[~is_hot]), "pairs on other experts take the same path as before"
    sel = torch.arange(0, t, max(1, t // 64))
    e_coef = orc.expert_coefficients(x[sel].float().cpu(), up.float().cpu(), w[sel].cpu(), idx[sel].cpu())
    assert_close(coef_hot[sel], e_coef, rtol=1e-3, atol=1e-4, what="hot vs oracle")


def test_hot_experts_none_found_is_the_plain_kernel_bit_for_bit():
    """Uniform routing: no expert fills a window; the dense GEMM launch returns at once and nothing reads its output."""
    t, h, n, k = 4096, 512, 65536, 8
    x = (torch.randn((t, h), generator=gen(1)) * 1.0).cuda().to(torch.bfloat16)
    up = (torch.randn((n, h), generator=gen(2)) * 0.05).cuda().to(torch.bfloat16)
    idx = torch.randint(0, n, (t, k), generator=torch.Generator().manual_seed(5), dtype=torch.int32).cuda()
    w = (torch.randn((t, k), generator=gen(3)) * 1.0).abs().cuda()
    coef_hot, hot = _hot_run(x, up, w, idx, n, 0)
    assert hot == []
    assert torch.equal(coef_hot, _plain_coef(x, up, w, idx, n))


def test_hot_experts_through_the_op_and_bad_indices_are_still_reported():
    from omni_moe_b200.ops import expert_forward
    t, h, n, k = 4096, 512, 4096, 8
    x = (torch.randn((t, h), generator=gen(1)) * 1.0).cuda().to(torch.bfloat16)
    up = (torch.randn((n, h), generator=gen(2)) * 0.05).cuda().to(torch.bfloat16)
    dn = (torch.randn((n, h), generator=gen(4)) * 0.05).cuda().to(torch.bfloat16)
    idx = zipf_indices(t, k, n, 1.3, 7).cuda()
    w = (torch.randn((t, k), generator=gen(3)) * 1.0).abs().cuda()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    y_hot = expert_forward(x, up, dn, w, idx, out_dtype=torch.float32, status=st, mode="scheduled", hot=True, hot_min_run=256)
    y_plain = expert_forward(x, up, dn, w, idx, out_dtype=torch.float32, status=st, mode="scheduled", hot=False)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_close(y_hot, y_plain, rtol=1e-4, atol=1e-5 * float(y_plain.abs().max()), what="hot vs gathered, output")
    ey = orc.expert_forward(x[:64].float().cpu(), up.float().cpu(), dn.float().cpu(), w[:64].cpu(), idx[:64].cpu())
    assert_close(y_hot[:64], ey, rtol=1e-3, atol=1e-4, what="hot path vs oracle")
    bad = idx.clone()
    bad[5, 1] = n + 3
    expert_forward(x, up, dn, w, bad, out_dtype=torch.float32, status=st, mode="scheduled", hot=True, hot_min_run=256)
    torch.cuda.synchronize()
    assert int(st.item()) & 1  # OMNI_ST_BAD_EXPERT_INDEX: reported, nothing faults
