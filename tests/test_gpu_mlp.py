"""tcgen05 GEMM paths (router gate logits, shared SwiGLU MLP) against the fp32 oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import omni_oracle as orc
from _util import assert_close, bf16_round, gen

pytestmark = pytest.mark.gpu


def _status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("t,h,n", [(128, 64, 64), (300, 256, 32), (1000, 1024, 64), (129, 72, 100), (4096, 1024, 64),
                                     (513, 2048, 256), (64, 512, 1024), (1, 8, 1)])
def test_router_gate_logits(t, h, n):
    from omni_moe_b200 import _lib
    g = gen(t + h)
    x = torch.randn(t, h, generator=g).bfloat16()
    kx = (torch.randn(n, h, generator=g) / h ** 0.5).bfloat16()
    ky = (torch.randn(n, h, generator=g) / h ** 0.5).bfloat16()
    xc, kxc, kyc = x.cuda(), kx.cuda(), ky.cuda()
    z = torch.full((t, 2 * n), float("nan"), device="cuda")
    st = _status()
    _lib.check(_lib.load().omni_router_gate(xc.data_ptr(), kxc.data_ptr(), kyc.data_ptr(), t, h, n, z.data_ptr(),
                                            st.data_ptr(), _lib.stream_ptr()))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ez = torch.cat([orc.router_logits(x, kx), orc.router_logits(x, ky)], 1)
    assert_close(z, ez, rtol=1e-4, atol=1e-4, what="router logits")


@pytest.mark.parametrize("t,h,i", [(128, 64, 128), (48, 64, 96), (300, 256, 1024), (1000, 1024, 4096), (77, 72, 200),
                                     (4096, 1024, 4096), (130, 4096, 1408)])
def test_mlp_matches_oracle(t, h, i):
    from omni_moe_b200.ops import mlp_forward
    g = gen(t + i)
    x = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    wg = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wu = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wd = (torch.randn(h, i, generator=g) / i ** 0.5).bfloat16()
    st = _status()
    y = mlp_forward(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda(), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_close(y, orc.mlp_forward(x, wg, wu, wd), what="mlp")
    res = torch.randn(t, h, generator=g)
    y2 = mlp_forward(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda(), residual=res.cuda(), status=st)
    assert_close(y2, orc.mlp_forward(x, wg, wu, wd) + res, what="mlp + residual")
    assert int(st.item()) == 0


def test_mlp_golden_mirror_and_drop_in(golden_dir):
    g = np.load(os.path.join(golden_dir, "mlp_mirror.npz"))
    from omni_moe.ops.triton import triton_omni_mlp_func
    x, wg, wu, wd = (torch.from_numpy(g[k]) for k in ("x", "gate", "up", "down"))
    y = triton_omni_mlp_func(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda())
    assert y.dtype == torch.float32 and y.shape == (48, 64)
    # float32 tensors are computed in float32: the reference's own fp32 tolerance against its mirror's output
    assert_close(y, torch.from_numpy(g["y"]), rtol=1e-4, atol=1e-5 * float(np.abs(g["y"]).max()) + 1e-6, what="fp32 drop-in vs golden")
    assert_close(y, orc.mlp_forward(x, wg, wu, wd), rtol=1e-4, atol=1e-5 * float(np.abs(g["y"]).max()) + 1e-6, what="fp32 drop-in vs oracle")
    # and with gradients, through autograd
    xs = [t.cuda().requires_grad_() for t in (x, wg, wu, wd)]
    triton_omni_mlp_func(*xs).square().sum().backward()
    assert all(t.grad is not None and torch.isfinite(t.grad).all() for t in xs)
    yb = triton_omni_mlp_func(x.bfloat16().cuda(), wg.bfloat16().cuda(), wu.bfloat16().cuda(), wd.bfloat16().cuda())
    assert yb.dtype == torch.bfloat16


def test_mlp_repeatable():
    from omni_moe_b200.ops import mlp_forward
    g = gen(1)
    x = torch.randn(512, 256, generator=g).bfloat16().cuda()
    wg = (torch.randn(512, 256, generator=g) / 16).bfloat16().cuda()
    wu = (torch.randn(512, 256, generator=g) / 16).bfloat16().cuda()
    wd = (torch.randn(256, 512, generator=g) / 22).bfloat16().cuda()
    a = mlp_forward(x, wg, wu, wd)
    for _ in range(5):
        assert torch.equal(a, mlp_forward(x, wg, wu, wd))


@pytest.mark.parametrize("t,h,i,n", [(300, 256, 512, 32), (4096, 1024, 4096, 64), (129, 72, 200, 100), (64, 512, 256, 300)])
def test_gate_up_with_router_tiles(t, h, i, n):
    """The fused launch gives the activation of omni_mlp_gate_up and the logits of omni_router_gate."""
    import torch.nn.functional as F
    from omni_moe_b200 import _lib
    g = gen(t + n)
    x = (torch.randn(t, h, generator=g) * 0.5).bfloat16()
    wg = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    wu = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
    kx = (torch.randn(n, h, generator=g) / h ** 0.5).bfloat16()
    ky = (torch.randn(n, h, generator=g) / h ** 0.5).bfloat16()
    dev = [v.cuda() for v in (x, wg, wu, kx, ky)]
    act = torch.full((t, i), float("nan"), device="cuda", dtype=torch.bfloat16)
    logits = torch.full((t, 2 * n), float("nan"), device="cuda")
    st = _status()
    _lib.check(_lib.load().omni_mlp_gate_up_router(*[v.data_ptr() for v in dev], t, h, i, n, act.data_ptr(),
                                                   logits.data_ptr(), st.data_ptr(), _lib.stream_ptr()))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    xf = x.float()
    assert_close(act, F.silu(xf @ wg.float().t()) * (xf @ wu.float().t()), what="activation")
    ez = torch.cat([orc.router_logits(x, kx), orc.router_logits(x, ky)], 1)
    assert_close(logits, ez, rtol=1e-4, atol=1e-4, what="router logits")


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 200, 72), (1, 8, 8), (33, 1032, 136), (4096, 1024, 1024), (513, 24, 1032)])
def test_tma_store_epilogue_equals_direct_stores(m, n, k):
    """The pair kernels' output leaves either through shared memory + TMA stores or through direct
    256-bit / 128-bit / scalar stores; both must write the same bits, including clipped edge tiles and an
    output that is a column slice of a wider matrix."""
    from omni_moe_b200 import _lib
    from omni_moe_b200.ops.autograd import gemm_nt
    lib = _lib.load()
    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) * 0.5).bfloat16().cuda()
    b = (torch.randn(n, k, generator=g) / k ** 0.5).bfloat16().cuda()
    outs = []
    try:
        for mode in (1, 0):
            os.environ["OMNI_MOE_B200_TMA_STORE"] = str(mode)   # read by the library at every call
            wide = torch.full((m, 2 * n + 16), 3.0, dtype=torch.bfloat16, device="cuda")
            dense = gemm_nt(a, b)
            gemm_nt(a, b, out=wide[:, 8:8 + n])
            torch.cuda.synchronize()
            assert bool((wide[:, :8] == 3).all()) and bool((wide[:, 8 + n:] == 3).all()), "wrote outside the slice"
            assert torch.equal(wide[:, 8:8 + n], dense)
            outs.append(dense)
    finally:
        os.environ.pop("OMNI_MOE_B200_TMA_STORE", None)
    assert torch.equal(outs[0], outs[1])
    ref = a.float() @ b.float().t()
    assert float((outs[0].float() - ref).abs().max()) <= 2e-2 * float(ref.abs().max()) + 1e-3


def test_tma_store_swiglu_and_saved_preactivations():
    from omni_moe_b200 import _lib
    from omni_moe_b200.ops import mlp_forward
    lib = _lib.load()
    t, h, i = 777, 264, 1096
    g = torch.Generator().manual_seed(9)
    x = torch.randn(t, h, generator=g).bfloat16().cuda()
    wg = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16().cuda()
    wu = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16().cuda()
    wd = (torch.randn(h, i, generator=g) / i ** 0.5).bfloat16().cuda()
    res = torch.randn(t, h, generator=g).cuda()
    got = []
    try:
        for mode in (1, 0):
            os.environ["OMNI_MOE_B200_TMA_STORE"] = str(mode)   # read by the library at every call
            gu = torch.empty(t, 2 * i, dtype=torch.bfloat16, device="cuda")
            act = torch.empty(t, i, dtype=torch.bfloat16, device="cuda")
            y = mlp_forward(x, wg, wu, wd, residual=res, act=act, gate_up=gu)
            torch.cuda.synchronize()
            got.append((y, act, gu))
    finally:
        os.environ.pop("OMNI_MOE_B200_TMA_STORE", None)
    for a_, b_ in zip(got[0], got[1]):
        assert torch.equal(a_, b_)


def test_single_cta_gemm_path_in_a_subprocess():
    """OMNI_MOE_B200_GEMM=1cta selects the single-CTA kernels for the MLP GEMMs (read once per process)."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r"""
import sys, torch
sys.path.insert(0, %r)
from oracle import omni_oracle as orc
from omni_moe_b200.ops import mlp_forward
g = torch.Generator().manual_seed(0)
t, h, i = 300, 264, 520
x = torch.randn(t, h, generator=g).bfloat16()
wg = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
wu = (torch.randn(i, h, generator=g) / h ** 0.5).bfloat16()
wd = (torch.randn(h, i, generator=g) / i ** 0.5).bfloat16()
res = torch.randn(t, h, generator=g)
y = mlp_forward(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda(), residual=res.cuda())
e = orc.mlp_forward(x.float(), wg.float(), wu.float(), wd.float()) + res
bad = (y.float().cpu() - e).abs() > 2e-2 + 2e-2 * e.abs()
assert not bad.any(), int(bad.sum())
print("single-cta ok")
""" % root
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, OMNI_MOE_B200_GEMM="1cta"), capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and "single-cta ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_bounded_wait_gives_up_and_leaves_the_context_usable():
    """The wait primitive of the GEMM kernels on a barrier nobody arrives on: it returns after its probe limit with
    the time-out bit in the status word and the abort flag up, and the next ordinary call is bit-correct."""
    from omni_moe_b200 import _lib
    from omni_moe_b200.ops.autograd import gemm_nt
    lib = _lib.load()
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(200, 256, generator=g) * 0.5).bfloat16().cuda()
    b = (torch.randn(136, 256, generator=g) / 16).bfloat16().cuda()
    before = gemm_nt(a, b)
    out = torch.full((4,), 7, dtype=torch.int32, device="cuda")
    _lib.check(lib.omni_selftest_wait_timeout(out.data_ptr(), 2000, _lib.stream_ptr()))
    torch.cuda.synchronize()
    assert out.tolist() == [_lib.OMNI_ST_WAIT_TIMEOUT if hasattr(_lib, "OMNI_ST_WAIT_TIMEOUT") else 2, 0, 0, 1], out.tolist()
    after = gemm_nt(a, b)
    torch.cuda.synchronize()
    assert torch.equal(before, after)
    with pytest.raises(RuntimeError):
        _lib.check(lib.omni_selftest_wait_timeout(out.data_ptr(), 0, _lib.stream_ptr()))
