"""Generate the golden fixtures in this directory from the reference project.

Run where a checkout of the reference project (HKUSTDial/omni-moe) is available, with its path in
``OMNI_MOE_REFERENCE``::

    OMNI_MOE_REFERENCE=<checkout> python tests/golden/make_golden.py

The reference package cannot be imported as shipped on a CPU-only host (its
``omni_moe.ops.triton`` package needs Triton, a GPU and an un-vendored
``triton_kernels`` dependency at import time), so that one sub-package is
replaced by an empty stand-in before the *unmodified* reference files are
imported:

* ``omni_moe/modules/omni_moe.py``  -> ``OmniMoE_Torch`` (the PyTorch layer)
* ``omni_moe/ops/triton/omni_scheduler.py`` -> ``get_scheduling_info`` (torch only)
* ``tests/test_router.py``, ``tests/test_expert.py``, ``tests/test_mlp.py``
  -> the ``pytorch_*_forward`` mirrors

The fixtures are small ``.npz`` files; each stores the inputs (or the seed that
regenerates them plus a checksum of the regenerated tensors) and the outputs
the reference produced.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np
import torch

REF = os.environ.get("OMNI_MOE_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set OMNI_MOE_REFERENCE to a checkout of the reference project (HKUSTDial/omni-moe)")
HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference():
    stub = types.ModuleType("omni_moe.ops.triton")
    for name in ("triton_omni_mlp_func", "triton_omni_router_func", "triton_omni_expert_func"):
        setattr(stub, name, None)
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.join(REF, "tests"))
    for k in [k for k in sys.modules if k == "omni_moe" or k.startswith("omni_moe.")]:
        del sys.modules[k]
    import omni_moe  # noqa: F401  (reference package root)
    sys.modules["omni_moe.ops.triton"] = stub
    from omni_moe.modules.omni_moe import OmniMoE_Torch, OmniMoEConfig

    def by_path(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    sched = by_path("ref_omni_scheduler", "omni_moe/ops/triton/omni_scheduler.py")
    t_router = by_path("ref_test_router", "tests/test_router.py")
    t_expert = by_path("ref_test_expert", "tests/test_expert.py")
    t_mlp = by_path("ref_test_mlp", "tests/test_mlp.py")
    return OmniMoE_Torch, OmniMoEConfig, sched, t_router, t_expert, t_mlp


def checksum(t: torch.Tensor) -> np.ndarray:
    t = t.detach().double()
    return np.array([t.sum().item(), t.abs().sum().item()], dtype=np.float64)


def state_arrays(module) -> dict:
    return {"sd." + k: v.detach().numpy() for k, v in module.state_dict().items()
            if not k.endswith("num_batches_tracked")}


def main():
    OmniMoE_Torch, OmniMoEConfig, sched, t_router, t_expert, t_mlp = load_reference()
    torch.set_num_threads(1)  # one thread: reduction order fixed

    # ---- tiny layer, everything stored (RNG independent) ------------------------------
    torch.manual_seed(1234)
    cfg = dict(hidden_size=64, intermediate_size=128, hidden_act="silu", num_experts=256,
               num_experts_per_token=4)
    m = OmniMoE_Torch(OmniMoEConfig(**cfg)).eval()
    with torch.no_grad():  # non-trivial BatchNorm running statistics
        m.router_norm_x.running_mean.normal_(0, 0.3)
        m.router_norm_y.running_mean.normal_(0, 0.3)
        m.router_norm_x.running_var.uniform_(0.5, 2.0)
        m.router_norm_y.running_var.uniform_(0.5, 2.0)
    x = torch.randn(2, 16, 64)
    with torch.no_grad():
        y = m(x)
    np.savez_compressed(os.path.join(HERE, "layer_tiny.npz"), x=x.numpy(), y=y.numpy(),
                        num_experts=256, top_k=4, **state_arrays(m))

    # ---- configuration 1 of the benchmark list: seeds + outputs ---------------------------
    torch.manual_seed(0)
    m = OmniMoE_Torch(OmniMoEConfig(256, 1024, "silu", 1024, 8)).eval()
    x = torch.randn(2, 256, 256)
    with torch.no_grad():
        y = m(x)
        # routing decisions, recomputed with the module's own statements
        h = x.view(-1, 256)
        lpx = torch.log_softmax(m.router_norm_x(m.router_gate_x(h)), -1)
        lpy = torch.log_softmax(m.router_norm_y(m.router_gate_y(h)), -1)
        sx, ix = lpx.topk(8, -1)
        sy, iy = lpy.topk(8, -1)
        alls = (sx.unsqueeze(-1) + sy.unsqueeze(-2)).view(512, -1)
        alli = (ix.unsqueeze(-1) * 32 + iy.unsqueeze(-2)).view(512, -1)
        sc, pos = alls.topk(8, -1)
        idx = alli.gather(-1, pos)
    np.savez_compressed(
        os.path.join(HERE, "layer_c1.npz"),
        seed=0, x_checksum=checksum(x), up_embed_checksum=checksum(m.up_embed.weight),
        gate_proj_checksum=checksum(m.gate_proj.weight),
        y_every8=y.view(512, 256)[::8].numpy(), y_checksum=checksum(y),
        scores=sc.numpy(), indices=idx.numpy().astype(np.int16))

    # ---- training mode (the module as constructed, omni_moe/modules/omni_moe.py:53-54): batch statistics -----
    torch.manual_seed(4321)
    m = OmniMoE_Torch(OmniMoEConfig(**cfg)).train()
    x = torch.randn(2, 16, 64)
    sd_before = {k: v.copy() for k, v in state_arrays(m).items()}   # copies: the forward updates the running statistics in place
    with torch.no_grad():
        y = m(x)
    np.savez_compressed(os.path.join(HERE, "layer_tiny_train.npz"), x=x.numpy(), y=y.numpy(), num_experts=256, top_k=4,
                        run_mean_x=m.router_norm_x.running_mean.numpy(), run_var_x=m.router_norm_x.running_var.numpy(),
                        run_mean_y=m.router_norm_y.running_mean.numpy(), run_var_y=m.router_norm_y.running_var.numpy(),
                        **sd_before)
    torch.manual_seed(0)
    m = OmniMoE_Torch(OmniMoEConfig(256, 1024, "silu", 1024, 8)).train()
    x = torch.randn(2, 256, 256)
    with torch.no_grad():
        y = m(x)
    np.savez_compressed(
        os.path.join(HERE, "layer_c1_train.npz"), seed=0, x_checksum=checksum(x), gate_proj_checksum=checksum(m.gate_proj.weight),
        y_every8=y.view(512, 256)[::8].numpy(), y_checksum=checksum(y),
        run_mean_x=m.router_norm_x.running_mean.numpy(), run_var_x=m.router_norm_x.running_var.numpy(),
        run_mean_y=m.router_norm_y.running_mean.numpy(), run_var_y=m.router_norm_y.running_var.numpy())

    # ---- configuration 2 (quick-start shape): fp32 run on bf16-rounded parameters and tokens -----------------
    # what the bf16 kernels are compared with: the reference module computing in fp32 on exactly the bf16 operands
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // 2))
    torch.manual_seed(0)
    m = OmniMoE_Torch(OmniMoEConfig(1024, 4096, "silu", 4096, 16)).eval()
    with torch.no_grad():
        for prm in m.parameters():
            prm.copy_(prm.to(torch.bfloat16).float())
        x = torch.randn(1, 4096, 1024).to(torch.bfloat16).float()
        y = m(x)
        h = x.view(-1, 1024)
        lpx = torch.log_softmax(m.router_norm_x(m.router_gate_x(h)), -1)
        lpy = torch.log_softmax(m.router_norm_y(m.router_gate_y(h)), -1)
        sx, ix = lpx.topk(16, -1)
        sy, iy = lpy.topk(16, -1)
        alls = (sx.unsqueeze(-1) + sy.unsqueeze(-2)).view(4096, -1)
        alli = (ix.unsqueeze(-1) * 64 + iy.unsqueeze(-2)).view(4096, -1)
        sc, pos = alls.topk(16, -1)
        idx = alli.gather(-1, pos)
    np.savez_compressed(
        os.path.join(HERE, "layer_c2.npz"), seed=0, x_checksum=checksum(x), gate_proj_checksum=checksum(m.gate_proj.weight),
        up_embed_checksum=checksum(m.up_embed.weight), y_every64=y.view(4096, 1024)[::64].numpy(), y_checksum=checksum(y),
        scores_every64=sc[::64].numpy(), indices=idx.numpy().astype(np.int16))
    torch.set_num_threads(1)

    # ---- router mirror (tests/test_router.py:8-22) --------------------------------------
    g = torch.Generator().manual_seed(0)
    lx = torch.log_softmax(torch.randn(64, 32, generator=g), -1)
    ly = torch.log_softmax(torch.randn(64, 32, generator=g), -1)
    # the mirror keeps all num_keys sub-keys per axis, i.e. it searches the full grid
    sc8 = t_router.pytorch_router_forward(lx, ly, 32, 8)
    sc16 = t_router.pytorch_router_forward(lx[:, :16].contiguous(), ly[:, :16].contiguous(), 16, 16)
    np.savez_compressed(os.path.join(HERE, "router_mirror.npz"), lx=lx.numpy(), ly=ly.numpy(),
                        scores_n32_k8=sc8.numpy(), scores_n16_k16=sc16.numpy())

    # ---- expert mirror (tests/test_expert.py:8-25), duplicate experts allowed --------
    g = torch.Generator().manual_seed(0)
    hs = torch.randn(32, 64, generator=g) * 0.5
    up = torch.randn(128, 64, generator=g) * 0.1
    dn = torch.randn(128, 64, generator=g) * 0.1
    rw = torch.randn(32, 8, generator=g) * 0.1
    ind = torch.randint(0, 128, (32, 8), generator=g, dtype=torch.int32)
    ind[0, 1] = ind[0, 0]                                       # a duplicate inside one token
    ye = t_expert.pytorch_expert_forward(hs, up, dn, rw, ind.long())
    np.savez_compressed(os.path.join(HERE, "expert_mirror.npz"), x=hs.numpy(), up=up.numpy(),
                        down=dn.numpy(), w=rw.numpy(), indices=ind.numpy(), y=ye.numpy())

    # ---- MLP mirror (tests/test_mlp.py:8-21) ----------------------------------------
    g = torch.Generator().manual_seed(42)
    hs = torch.randn(48, 64, generator=g) * 0.5
    wg = torch.randn(96, 64, generator=g) * 0.1
    wu = torch.randn(96, 64, generator=g) * 0.1
    wd = torch.randn(64, 96, generator=g) * 0.1
    ym = t_mlp.pytorch_mlp_forward(hs, wg, wu, wd)
    np.savez_compressed(os.path.join(HERE, "mlp_mirror.npz"), x=hs.numpy(), gate=wg.numpy(),
                        up=wu.numpy(), down=wd.numpy(), y=ym.numpy())

    # ---- scheduler (omni_moe/ops/triton/omni_scheduler.py:48-101) -------------------------
    out = {}
    for tag, (t, k, n, seed) in {"a": (64, 8, 128, 0), "b": (33, 6, 16, 1), "c": (16, 4, 4096, 2)}.items():
        g = torch.Generator().manual_seed(seed)
        w = torch.rand(t, k, generator=g)
        ind = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
        s = sched.get_scheduling_info(w, ind, n, 16)
        assert s.num_groups == 0
        out.update({
            f"{tag}.w": w.numpy(), f"{tag}.indices": ind.numpy(), f"{tag}.num_experts": n,
            f"{tag}.tail_token_ids": s.tail_token_ids.numpy(),
            f"{tag}.tail_expert_ids": s.tail_expert_ids.numpy(),
            f"{tag}.tail_routing_weights": s.tail_routing_weights.numpy(),
            f"{tag}.tail_offsets": s.tail_offsets.numpy(),
            f"{tag}.tail_sorted_pair_ids": s.tail_sorted_pair_ids.numpy(),
            f"{tag}.num_tail_experts": s.num_tail_experts,
            f"{tag}.max_tail_pairs_per_expert": s.max_tail_pairs_per_expert,
        })
    np.savez_compressed(os.path.join(HERE, "schedule_ref.npz"), **out)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
