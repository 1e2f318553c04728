"""omni_moe_b200: the OmniMoE layer-forward hot path as hand-written sm_100a CUDA kernels.

Same Python surface as the reference project for this path:
``omni_moe_b200.modules.omni_moe.{OmniMoE, OmniMoEConfig}`` and the three op functions in
``omni_moe_b200.ops`` (also importable under their reference names from ``omni_moe.ops.triton``).
"""
from . import _lib  # noqa: F401
from ._lib import check_status  # noqa: F401

__version__ = "0.1.0"
