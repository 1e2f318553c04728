"""The C-ABI library loads and exports everything the header declares; argument checks that need
no device are exercised.  No kernel is launched here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from omni_moe_b200 import _lib
    from omni_moe_b200.build import build
    build()
    return _lib.load()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "omni_moe_b200.h")).read()
    return sorted(set(re.findall(r"OMNI_API[^;(]*?\b(omni_\w+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = header_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"


def test_bindings_cover_header():
    from omni_moe_b200 import _lib
    assert sorted(_lib.SIGNATURES) == header_symbols()


def test_version_and_rejections(lib):
    assert lib.omni_version() == 100
    # k out of range is refused before anything touches the device
    rc = lib.omni_router_topk(None, None, 0, 4, 8, 0, None, None, 0, None, None)
    assert rc < 0 and b"k must be" in lib.omni_last_error()
    rc = lib.omni_router_topk(None, None, 0, 4, 2000, 4, None, None, 0, None, None)
    assert rc < 0 and b"sqrt_n" in lib.omni_last_error()
    rc = lib.omni_expert_coef(None, None, None, None, None, 4, 2, 12, 16, None, None, None)
    assert rc < 0 and b"multiple of 8" in lib.omni_last_error()
    rc = lib.omni_mlp_fwd(None, None, None, None, 4, 64, 100, None, None, None, None, None)
    assert rc < 0 and b"intermediate" in lib.omni_last_error()
    # entries of the backward and of the clamp: argument errors come back as codes with a message
    rc = lib.omni_mlp_gate_up_limit(None, None, None, 4, 64, 64, -0.5, None, None, None, None)
    assert rc < 0 and b"limit" in lib.omni_last_error()
    rc = lib.omni_swiglu_bwd_limit(None, None, 4, 64, float("nan"), None, None, None, 0, None, None)
    assert rc < 0 and b"limit" in lib.omni_last_error()
    rc = lib.omni_swiglu_bwd(None, None, 4, 12, None, None, None, 0, None)
    assert rc < 0 and b"multiple of 8" in lib.omni_last_error()
    rc = lib.omni_mlp_gate_up_save(None, None, None, 4, 64, 64, None, None, None, None)
    assert rc < 0 and b"NULL" in lib.omni_last_error()
    assert lib.omni_schedule_workspace_bytes(65536, 4096) > 4 * 65536 * 4
    assert lib.omni_schedule_workspace_bytes(-1, 4096) == 0


def test_no_fallback_when_library_missing(monkeypatch):
    from omni_moe_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libomni_moe_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_ops_refuse_cpu_tensors():
    import torch
    from omni_moe_b200.ops import omni_router_func
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        omni_router_func(torch.zeros(4, 8), torch.zeros(4, 8), 8, 2)


def test_reference_assert_messages():
    import torch
    from omni_moe_b200.ops import omni_router_func
    with pytest.raises(AssertionError, match="multiple of 2"):
        omni_router_func(torch.zeros(4, 8), torch.zeros(4, 8), 8, 3)
    with pytest.raises(AssertionError, match="less than or equal to 128"):
        omni_router_func(torch.zeros(4, 16), torch.zeros(4, 16), 16, 130)


def test_module_state_dict_matches_reference_names():
    from omni_moe.modules.omni_moe import OmniMoE, OmniMoEConfig
    m = OmniMoE(OmniMoEConfig(64, 128, "silu", 256, 4))
    keys = set(m.state_dict().keys())
    assert keys == {
        "gate_proj.weight", "up_proj.weight", "down_proj.weight", "router_gate_x.weight", "router_gate_y.weight",
        "router_norm_x.running_mean", "router_norm_x.running_var", "router_norm_x.num_batches_tracked",
        "router_norm_y.running_mean", "router_norm_y.running_var", "router_norm_y.num_batches_tracked",
        "up_embed.weight", "down_embed.weight"}
    assert m.up_embed.weight.shape == (256, 64) and m.router_gate_x.weight.shape == (16, 64)
    with pytest.raises(ValueError):
        OmniMoE(OmniMoEConfig(64, 128, "gelu", 256, 4))
