"""Loads the reference project's own PyTorch layer from ``oracle/_ref/`` (test infrastructure).

``oracle/_ref/`` is filled by ``python -m oracle.make_ref`` with unmodified files of the reference
project.  Its module file (omni_moe/modules/omni_moe.py) imports the three Triton operator entry
points at the top (lines 7-11), and that sub-package needs Triton, a GPU and an un-vendored
dependency at import time; only ``OmniMoE_Torch`` (lines 109-194), which never calls them, is wanted
here, so an empty stand-in is put in ``sys.modules`` for the duration of the import and removed
again.  Nothing of this library is imported on the way: what is timed is the reference's code alone.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_MODULE_FILE = os.path.join(REF_DIR, "omni_moe", "modules", "omni_moe.py")
_SCHED_FILE = os.path.join(REF_DIR, "omni_moe", "ops", "triton", "omni_scheduler.py")
_cache = {}


def available() -> bool:
    return os.path.isfile(_MODULE_FILE)


def _exec(name: str, path: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_layer():
    """``(OmniMoE_Torch, OmniMoEConfig)`` of the reference, or ``None`` if ``oracle/_ref`` is empty."""
    if not available():
        return None
    if "layer" not in _cache:
        names = ("omni_moe", "omni_moe.ops", "omni_moe.ops.triton")
        saved = {n: sys.modules.get(n) for n in names}
        try:
            for n in names:
                stub = types.ModuleType(n)
                stub.__path__ = []  # a package, so that the dotted import resolves through sys.modules
                sys.modules[n] = stub
            for fn in ("triton_omni_mlp_func", "triton_omni_router_func", "triton_omni_expert_func"):
                setattr(sys.modules["omni_moe.ops.triton"], fn, None)
            mod = _exec("_omni_moe_reference_layer", _MODULE_FILE)
        finally:
            for n, m in saved.items():
                if m is None:
                    sys.modules.pop(n, None)
                else:
                    sys.modules[n] = m
        _cache["layer"] = (mod.OmniMoE_Torch, mod.OmniMoEConfig)
    return _cache["layer"]


def load_scheduler():
    """The reference's ``omni_scheduler`` module (``get_scheduling_info``), or ``None``."""
    if not os.path.isfile(_SCHED_FILE):
        return None
    if "sched" not in _cache:
        _cache["sched"] = _exec("_omni_moe_reference_scheduler", _SCHED_FILE)
    return _cache["sched"]
