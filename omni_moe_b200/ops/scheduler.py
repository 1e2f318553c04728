"""Expert-centric scheduling (reference: omni_moe/ops/triton/omni_scheduler.py:5-101, tail path)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib


@dataclass(frozen=True)
class SchedulingInfo:
    """Same tail fields as the reference ``SchedulingInfo`` (omni_moe/ops/triton/omni_scheduler.py:5-43).
    The grouped path of the reference never triggers for T*k/N <= 256 and is not provided:
    ``num_groups`` is always 0."""
    tail_token_ids: torch.Tensor = None
    tail_expert_ids: torch.Tensor = None
    tail_routing_weights: torch.Tensor = None
    tail_offsets: torch.Tensor = None
    tail_sorted_pair_ids: torch.Tensor = None
    num_tail_experts: int = 0
    max_tail_pairs_per_expert: int = 0
    num_groups: int = 0
    max_group_tokens: int = 0


@dataclass
class RawSchedule:
    """Device-side result of :func:`schedule`; nothing here forces a host synchronisation.
    ``expert_ids`` / ``offsets`` are allocated at capacity; ``meta[0]`` holds the number of valid segments."""
    sorted_pair_ids: torch.Tensor
    sorted_experts: torch.Tensor
    token_ids: torch.Tensor | None
    sorted_weights: torch.Tensor | None
    expert_ids: torch.Tensor | None
    offsets: torch.Tensor | None
    meta: torch.Tensor          # int32 [4]: U, max pairs per expert, status word, reserved
    workspace: torch.Tensor


def workspace_bytes(num_pairs: int, num_experts: int) -> int:
    return int(_lib.load().omni_schedule_workspace_bytes(num_pairs, num_experts))


def schedule(indices: torch.Tensor, num_experts: int, weights: torch.Tensor | None = None,
             segments: bool = True, workspace: torch.Tensor | None = None) -> RawSchedule:
    """Stable sort of the (token, expert) pairs by expert on the current stream; no host sync."""
    _lib.require_cuda(indices, weights)
    assert indices.dim() == 2 and indices.dtype in (torch.int32, torch.int64)
    indices = indices.contiguous()
    t, k = indices.shape
    p = t * k
    dev = indices.device
    if weights is not None:
        assert weights.shape == indices.shape and weights.element_size() in (2, 4)
        weights = weights.detach().contiguous()
    need = workspace_bytes(p, num_experts)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, device=dev, dtype=torch.uint8)
    i32 = dict(device=dev, dtype=torch.int32)
    perm = torch.empty(p, **i32)
    sorted_e = torch.empty(p, **i32)
    token_ids = torch.empty(p, **i32) if segments else None
    sorted_w = torch.empty(p, device=dev, dtype=weights.dtype) if (weights is not None and segments) else None
    cap = min(p, num_experts)
    expert_ids = torch.empty(cap, **i32) if segments else None
    offsets = torch.empty(cap + 1, **i32) if segments else None
    meta = torch.empty(4, **i32)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().omni_schedule(
            indices.data_ptr(), int(indices.dtype == torch.int64), _lib.ptr(weights),
            weights.element_size() if weights is not None else 0, t, max(k, 1), num_experts,
            perm.data_ptr(), sorted_e.data_ptr(), _lib.ptr(token_ids), _lib.ptr(sorted_w),
            _lib.ptr(expert_ids), _lib.ptr(offsets), meta.data_ptr(), workspace.data_ptr(), workspace.numel(),
            _lib.stream_ptr()))
    return RawSchedule(perm, sorted_e, token_ids, sorted_w, expert_ids, offsets, meta, workspace)


def get_scheduling_info(G: torch.Tensor, Indices: torch.Tensor, num_experts: int, group_size: int = 16) -> SchedulingInfo:
    """Drop-in for the reference ``get_scheduling_info`` (tail path).  Like the reference it reads
    two scalars back to the host (number of distinct experts, longest segment)."""
    raw = schedule(Indices, num_experts, weights=G, segments=True)
    u, mx, st, _ = raw.meta.tolist()
    if st:
        raise RuntimeError("omni_schedule: " + _lib.status_message(st))
    return SchedulingInfo(
        tail_token_ids=raw.token_ids, tail_expert_ids=raw.expert_ids[:u], tail_routing_weights=raw.sorted_weights,
        tail_offsets=raw.offsets[:u + 1], tail_sorted_pair_ids=raw.sorted_pair_ids,
        num_tail_experts=u, max_tail_pairs_per_expert=mx)
