"""omni_schedule_static: the scheduling entry point for hosts that cannot allocate device memory
(a plugin that only sees the tensors handed to it, a memory-planned region, a service whose
allocator belongs to someone else).  Its radix-sort scratch is a fixed array inside the library,
so the call takes inputs and outputs only.

Checked here, through the C ABI: two calls in a row (the second one meets the scratch as the first
left it) give exactly what omni_schedule gives with a caller-provided workspace; a problem beyond
the stated limit is refused with a clear message.  This file sorts last on purpose, so a run that
stops at the first failure has already been through every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _outputs(p, cap, dev, wdtype):
    i32 = dict(device=dev, dtype=torch.int32)
    return dict(perm=torch.full((p,), -1, **i32), sorted_e=torch.full((p,), -1, **i32),
                token_ids=torch.full((p,), -1, **i32), sorted_w=torch.zeros(p, device=dev, dtype=wdtype),
                expert_ids=torch.full((cap,), -1, **i32), offsets=torch.full((cap + 1,), -1, **i32),
                meta=torch.full((4,), -1, **i32))


def _call(lib, static, ind, w, n, out, ws=None):
    from omni_moe_b200 import _lib
    t, k = ind.shape
    head = (ind.data_ptr(), 0, w.data_ptr(), w.element_size(), t, k, n, out["perm"].data_ptr(),
            out["sorted_e"].data_ptr(), out["token_ids"].data_ptr(), out["sorted_w"].data_ptr(),
            out["expert_ids"].data_ptr(), out["offsets"].data_ptr(), out["meta"].data_ptr())
    st = torch.cuda.current_stream().cuda_stream
    if static:
        _lib.check(lib.omni_schedule_static(*head, st))
    else:
        _lib.check(lib.omni_schedule(*head, ws.data_ptr(), ws.numel(), st))


@pytest.mark.parametrize("t,k,n", [(4096, 16, 4096), (1000, 32, 1 << 20)])
def test_static_scratch_matches_workspace_entry_point_twice(t, k, n):
    from omni_moe_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    assert t * k <= lib.omni_schedule_static_max_pairs()
    for call in range(2):  # different data each time: stale scratch contents must not leak through
        g = torch.Generator().manual_seed(10 * call + k)
        ind = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32).to(dev)
        w = torch.rand(t, k, generator=g).to(dev)
        p, cap = t * k, min(t * k, n)
        ref, got = _outputs(p, cap, dev, w.dtype), _outputs(p, cap, dev, w.dtype)
        ws = torch.empty(lib.omni_schedule_workspace_bytes(p, n), device=dev, dtype=torch.uint8)
        _call(lib, False, ind, w, n, ref, ws)
        _call(lib, True, ind, w, n, got)
        torch.cuda.synchronize()
        u = int(ref["meta"][0])
        assert got["meta"].tolist() == ref["meta"].tolist() and ref["meta"][2].item() == 0
        for name in ("perm", "sorted_e", "token_ids", "sorted_w"):
            assert torch.equal(got[name], ref[name]), name          # integer / copied data: bit-exact
        assert torch.equal(got["expert_ids"][:u], ref["expert_ids"][:u])
        assert torch.equal(got["offsets"][:u + 1], ref["offsets"][:u + 1])
        # and it is a sort: experts ascending, pair ids ascending inside an expert
        se, perm = got["sorted_e"].long(), got["perm"].long()
        assert bool((se[1:] >= se[:-1]).all())
        same = se[1:] == se[:-1]
        assert bool((perm[1:][same] > perm[:-1][same]).all())


def test_static_scratch_refuses_problems_beyond_its_limit():
    from omni_moe_b200 import _lib
    lib = _lib.load()
    limit = lib.omni_schedule_static_max_pairs()
    t, k = limit // 16 + 1, 16
    dev = torch.device("cuda:0")
    ind = torch.zeros((t, k), dtype=torch.int32, device=dev)
    out = _outputs(t * k, 16, dev, torch.float32)
    rc = lib.omni_schedule_static(ind.data_ptr(), 0, None, 0, t, k, 16, out["perm"].data_ptr(),
                                  out["sorted_e"].data_ptr(), None, None, None, None, out["meta"].data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    assert rc < 0
    msg = lib.omni_last_error().decode()
    assert "at most" in msg and str(limit) in msg
    torch.cuda.synchronize()
    assert out["perm"].eq(-1).all()  # nothing was enqueued
