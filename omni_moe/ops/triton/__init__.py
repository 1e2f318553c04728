# The reference exposes its operators under ``omni_moe.ops.triton``; the names are kept, the
# implementation behind them is the CUDA library (nothing here uses Triton).
from omni_moe_b200.ops import (  # noqa: F401
    triton_omni_expert_func,
    triton_omni_mlp_func,
    triton_omni_router_func,
)
from omni_moe_b200.ops import scheduler as omni_scheduler  # noqa: F401
