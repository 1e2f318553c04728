"""Router selection kernel against the oracle: indices and scores bit-exact."""
import numpy as np
import pytest
import torch

from oracle import omni_oracle as orc
from _util import gen

pytestmark = pytest.mark.gpu


def _run(lx, ly, n, k, index_dtype=torch.int32):
    from omni_moe_b200.ops import router_topk
    s, i, w = router_topk(lx.cuda(), ly.cuda(), n, k, index_dtype=index_dtype, with_weights=True)
    torch.cuda.synchronize()
    return s.cpu().numpy(), i.cpu().numpy(), w.cpu().numpy()


def _check(lx, ly, n, k, **kw):
    s, i, w = _run(lx, ly, n, k, **kw)
    es, ei = orc.router_topk(lx, ly, n, k)
    np.testing.assert_array_equal(i.astype(np.int64), ei)
    np.testing.assert_array_equal(s, es)
    np.testing.assert_allclose(w, np.exp(es), rtol=1e-6)


@pytest.mark.parametrize("t,n,k", [(257, 32, 8), (1024, 64, 16), (333, 256, 32), (70, 512, 32), (64, 1024, 64),
                                     (40, 128, 128), (5, 8, 64), (3, 4, 16), (9, 16, 2), (17, 100, 12), (1, 1, 1),
                                     (90, 300, 16), (65, 400, 6), (129, 200, 10), (77, 130, 3), (50, 513, 33), (31, 72, 127)])
def test_topk_matches_oracle_fp32(t, n, k):
    g = gen(t * 131 + n)
    lx = torch.log_softmax(torch.randn(t, n, generator=g), -1)
    ly = torch.log_softmax(torch.randn(t, n, generator=g), -1)
    _check(lx, ly, n, k)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("t,n,k", [(512, 64, 16), (200, 256, 32), (100, 128, 64)])
def test_topk_low_precision_inputs_tie_heavy(dtype, t, n, k):
    # 16-bit log-probs collide often: exercises the tie rule and the exact re-scan
    g = gen(7)
    lx = torch.log_softmax(torch.randn(t, n, generator=g), -1).to(dtype)
    ly = torch.log_softmax(torch.randn(t, n, generator=g), -1).to(dtype)
    _check(lx, ly, n, k)


def test_topk_explicit_ties():
    n, k = 16, 8
    z = torch.zeros(4, n)
    _check(z, z, n, k)                       # every sum ties: lowest flat indices win
    q = torch.randint(-3, 1, (300, n), generator=gen(3)).float()   # few distinct values
    _check(q, q.flip(1).contiguous(), n, k)
    _check(q, q.flip(1).contiguous(), n, 16)
    q64 = torch.randint(-2, 1, (100, 64), generator=gen(4)).float()
    _check(q64, q64.roll(5, 1).contiguous(), 64, 32)
    neg0 = torch.tensor([[0.0, -0.0, -1.0, -1.0]])
    _check(neg0, neg0, 4, 4)


def test_topk_rounding_tie_outside_pruned_region():
    # Near 2^24 the fp32 spacing is 2, so adding 1.0 or 0.5 rounds to the same sum.  Sub-key 5 ranks
    # first on x and sub-key 3 second, yet their sums tie and the cell of sub-key 3 has the lower flat
    # index.  For k = 3 the third winner (rank 1 on x, rank 1 on y) lies outside the
    # (i+1)(j+1) <= k region, which only the exact re-scan can find.
    n = 8
    lx = torch.full((1, n), -50.0)
    ly = torch.full((1, n), -60.0)
    lx[0, 5], lx[0, 3] = 1.0, 0.5
    ly[0, 0], ly[0, 1] = 16777220.0, 16777216.0
    es, ei = orc.router_topk(lx, ly, n, 3)
    assert ei.tolist() == [[24, 40, 25]]
    for k in (2, 3, 4, 6):
        _check(lx, ly, n, k)


def test_topk_int64_indices_and_minus_inf():
    g = gen(11)
    lx = torch.log_softmax(torch.randn(50, 64, generator=g) * 30, -1)
    ly = torch.log_softmax(torch.randn(50, 64, generator=g) * 30, -1)
    lx[:, 3] = -float("inf")
    _check(lx, ly, 64, 16, index_dtype=torch.int64)


def test_drop_in_signature_and_dtypes():
    from omni_moe.ops.triton import triton_omni_router_func
    g = gen(5)
    lx = torch.log_softmax(torch.randn(128, 64, generator=g), -1).bfloat16()
    ly = torch.log_softmax(torch.randn(128, 64, generator=g), -1).bfloat16()
    s, i = triton_omni_router_func(lx.cuda(), ly.cuda(), 64, 16)
    assert s.dtype == torch.bfloat16 and i.dtype == torch.int32 and s.shape == i.shape == (128, 16)
    es, ei = orc.router_topk(lx, ly, 64, 16)
    np.testing.assert_array_equal(i.cpu().numpy(), ei)
    np.testing.assert_array_equal(s.float().cpu().numpy(), torch.from_numpy(es).bfloat16().float().numpy())
    s0, i0 = triton_omni_router_func(lx.cuda(), ly.cuda(), 64, 0)
    assert s0.shape == (128, 0)
    se, ie = triton_omni_router_func(lx[:0].cuda(), ly[:0].cuda(), 64, 16)
    assert se.shape == (0, 16)


def test_router_microbench_shape_properties():
    # 16384 tokens, 256 x 256 grid, k = 16: full size, checked through properties and a sampled oracle run
    t, n, k = 16384, 256, 16
    g = gen(0)
    lx = torch.log_softmax(torch.randn(t, n, generator=g), -1)
    ly = torch.log_softmax(torch.randn(t, n, generator=g), -1)
    s, i, w = _run(lx, ly, n, k, index_dtype=torch.int64)
    assert (np.diff(s, axis=1) <= 0).all()
    ix, iy = i // n, i % n
    np.testing.assert_array_equal(np.take_along_axis(lx.numpy(), ix, 1) + np.take_along_axis(ly.numpy(), iy, 1), s)
    assert all(len(set(r)) == k for r in i[::97])
    sel = slice(0, t, 31)
    es, ei = orc.router_topk(lx[sel], ly[sel], n, k)
    np.testing.assert_array_equal(i[sel], ei)


def test_fused_logits_topk_matches_oracle_on_its_own_log_probs():
    from omni_moe_b200.ops import router_gate_topk
    t, h, n, k = 300, 256, 64, 16
    g = gen(2)
    x = torch.randn(t, h, generator=g).bfloat16()
    kx = (torch.randn(n, h, generator=g) / h ** 0.5).bfloat16()
    ky = (torch.randn(n, h, generator=g) / h ** 0.5).bfloat16()
    mean = torch.randn(2 * n, generator=g) * 0.2
    var = torch.rand(2 * n, generator=g) + 0.5
    scale = torch.rsqrt(var + 1e-5)
    shift = -mean * scale
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    s, i, w, lp = router_gate_topk(x.cuda(), kx.cuda(), ky.cuda(), k, scale.cuda(), shift.cuda(),
                                   return_log_probs=True, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    lp = lp.cpu()
    # (a) given the log-probs the kernel produced, the selection is bit-exact
    es, ei = orc.router_topk(lp[:, :n].contiguous(), lp[:, n:].contiguous(), n, k)
    np.testing.assert_array_equal(i.cpu().numpy(), ei)
    np.testing.assert_array_equal(s.cpu().numpy(), es)
    # (b) the log-probs themselves agree with the fp32 oracle to GEMM rounding
    zx = orc.router_batchnorm_eval(orc.router_logits(x, kx), mean[:n], var[:n])
    zy = orc.router_batchnorm_eval(orc.router_logits(x, ky), mean[n:], var[n:])
    np.testing.assert_allclose(lp[:, :n].numpy(), orc.router_log_probs(zx).numpy(), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(lp[:, n:].numpy(), orc.router_log_probs(zy).numpy(), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("t,n,momentum,dt", [(1000, 64, 0.1, torch.float32), (65, 1024, None, torch.float32), (4097, 256, 0.25, torch.bfloat16),
                                              (1, 8, 0.1, torch.float32)])
def test_batchnorm_statistics_kernel(t, n, momentum, dt):
    """omni_router_bn_train against torch: fold (scale, shift) from biased batch variance, running
    statistics with the unbiased one, batch counter; a large common offset shows any cancellation."""
    from omni_moe_b200 import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(t + n)
    z = (torch.randn(t, 2 * n, generator=g) * 2.0 + 50.0).cuda()
    rm = [(torch.randn(n, generator=g) * 0.1).to(dt).cuda() for _ in range(2)]
    rv = [(torch.rand(n, generator=g) + 0.5).to(dt).cuda() for _ in range(2)]
    nbt = [torch.full((), 4, dtype=torch.int64, device="cuda") for _ in range(2)]
    rm0, rv0 = [v.clone() for v in rm], [v.clone() for v in rv]
    scale = torch.empty(2 * n, device="cuda")
    shift = torch.empty(2 * n, device="cuda")
    scratch = torch.empty(int(lib.omni_router_bn_train_scratch_bytes(t, n)), dtype=torch.uint8, device="cuda")
    mom = -1.0 if momentum is None else momentum
    _lib.check(lib.omni_router_bn_train(z.data_ptr(), 2 * n, t, n, 1e-5, 1e-3, mom, mom, rm[0].data_ptr(), rv[0].data_ptr(),
                                        rm[1].data_ptr(), rv[1].data_ptr(), _lib.dtype_code(dt), nbt[0].data_ptr(), nbt[1].data_ptr(),
                                        scale.data_ptr(), shift.data_ptr(), scratch.data_ptr(), scratch.numel(), _lib.stream_ptr()))
    torch.cuda.synchronize()
    var, mean = torch.var_mean(z.double(), dim=0, unbiased=False)
    eps = torch.cat([torch.full((n,), 1e-5), torch.full((n,), 1e-3)]).double().cuda()
    e_scale = torch.rsqrt(var + eps)
    torch.testing.assert_close(scale.double(), e_scale, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(shift.double(), -mean * e_scale, rtol=1e-4, atol=1e-3)
    assert int(nbt[0]) == 5 and int(nbt[1]) == 5
    m_eff = 1.0 / 5 if momentum is None else momentum
    unb = var * (t / max(t - 1, 1))
    tol = dict(rtol=2e-2, atol=2e-2) if dt == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    for a in range(2):
        sl = slice(a * n, (a + 1) * n)
        torch.testing.assert_close(rm[a].double(), (1 - m_eff) * rm0[a].double() + m_eff * mean[sl], **tol)
        torch.testing.assert_close(rv[a].double(), (1 - m_eff) * rv0[a].double() + m_eff * unb[sl], **tol)
