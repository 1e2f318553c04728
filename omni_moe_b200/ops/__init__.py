"""Operator interface of the hot path: same call signatures as the reference's
``omni_moe.ops.triton`` (omni_moe/ops/triton/interface.py:7-72)."""
from .router import omni_router_func, router_topk, router_gate_topk
from .scheduler import SchedulingInfo, get_scheduling_info, schedule
from .expert import omni_expert_func, expert_forward, route_expert_fused
from .mlp import omni_mlp_func, mlp_forward

# reference names
triton_omni_router_func = omni_router_func
triton_omni_expert_func = omni_expert_func
triton_omni_mlp_func = omni_mlp_func

__all__ = [
    "omni_router_func", "omni_expert_func", "omni_mlp_func",
    "triton_omni_router_func", "triton_omni_expert_func", "triton_omni_mlp_func",
    "router_topk", "router_gate_topk", "SchedulingInfo", "get_scheduling_info", "schedule",
    "expert_forward", "route_expert_fused", "mlp_forward",
]
