"""Routed-expert op (reference: omni_moe/ops/triton/omni_expert.py:920-992, interface.py:54-72)."""
from __future__ import annotations

import os

import torch

from .. import _lib
from ._common import as_bf16, pad_last
from .scheduler import schedule

L2_RESIDENT_TABLE_BYTES = 48 << 20  # both tables together; above this the expert-ordered path reads less HBM


def use_fused_path(num_experts: int, hidden: int) -> bool:
    """True when the token-centric single kernel is the better choice: the Up and Down tables
    (2 * N * H bf16) stay resident in the 126 MB L2 next to the activations, and a row fits in
    registers.  ``OMNI_MOE_B200_EXPERT=fused|scheduled`` overrides."""
    import os
    forced = os.environ.get("OMNI_MOE_B200_EXPERT", "")
    if forced == "scheduled":
        return False
    if hidden > 2048:
        return False
    if forced == "fused":
        return True
    return 2 * num_experts * hidden * 2 <= L2_RESIDENT_TABLE_BYTES


def region_cells(sqrt_n: int, k: int) -> int:
    """Cells of the pruned candidate region of the router search: (i+1)(j+1) <= k in rank space."""
    kk = min(sqrt_n, k)
    return sum(min(kk, k // (i + 1)) for i in range(kk))


def use_routed_kernel(num_experts: int, hidden: int, sqrt_n: int, k: int) -> bool:
    """True when router selection and routed experts can run as the single fused kernel
    (``omni_route_expert_fused``): the fused-expert regime plus its limits on the router shape."""
    return (use_fused_path(num_experts, hidden) and sqrt_n <= 256 and 1 <= k <= min(32, sqrt_n * sqrt_n)
            and sqrt_n * sqrt_n <= num_experts and region_cells(sqrt_n, k) <= 128)


def route_expert_fused(logits: torch.Tensor, x: torch.Tensor, up_weight: torch.Tensor, down_weight: torch.Tensor, k: int,
                       bn_scale: torch.Tensor | None = None, bn_shift: torch.Tensor | None = None,
                       residual: torch.Tensor | None = None, return_routing: bool = True):
    """Router selection from ``logits [T, 2*sqrt_n]`` (fp32) and the routed-expert sum in one kernel.

    Returns ``y [T, H]`` bf16 (``residual`` added if given) and, if ``return_routing``,
    ``(scores, indices, weights)`` as :func:`omni_moe_b200.ops.router_gate_topk` would give them.
    """
    _lib.require_cuda(logits, x, up_weight, down_weight)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    assert x.dtype == up_weight.dtype == down_weight.dtype == torch.bfloat16
    x, up_weight, down_weight = x.contiguous(), up_weight.contiguous(), down_weight.contiguous()
    t, h = x.shape
    n = logits.size(1) // 2
    dev = x.device
    y = torch.empty((t, h), device=dev, dtype=torch.bfloat16)
    if residual is not None:
        assert residual.shape == y.shape and residual.dtype == torch.bfloat16 and residual.is_contiguous()
    scores = torch.empty((t, k), device=dev, dtype=torch.float32) if return_routing else None
    indices = torch.empty((t, k), device=dev, dtype=torch.int32) if return_routing else None
    weights = torch.empty((t, k), device=dev, dtype=torch.float32) if return_routing else None
    with torch.cuda.device(dev):
        _lib.check(_lib.load().omni_route_expert_fused(
            logits.data_ptr(), logits.size(1), _lib.ptr(bn_scale), _lib.ptr(bn_shift), x.data_ptr(),
            up_weight.data_ptr(), down_weight.data_ptr(), t, n, k, h, up_weight.size(0), _lib.ptr(residual),
            y.data_ptr(), _lib.ptr(scores), _lib.ptr(indices), _lib.ptr(weights), _lib.device_status(dev).data_ptr(),
            _lib.stream_ptr()))
    return (y, scores, indices, weights) if return_routing else y


def use_hot_experts(num_tokens: int) -> bool:
    """Whether the scheduled path looks for hot experts (``omni_expert_coef_hot``): on by default from 4096 tokens,
    where the one extra 64-column GEMM is noise beside the gathers; ``OMNI_MOE_B200_HOT=0`` turns it off."""
    return num_tokens >= 4096 and os.environ.get("OMNI_MOE_B200_HOT", "1") != "0"


def hot_workspace(num_tokens: int, hidden: int, dev: torch.device) -> torch.Tensor:
    return torch.empty(int(_lib.load().omni_expert_coef_hot_workspace(num_tokens, hidden)), device=dev, dtype=torch.uint8)


def expert_forward(x: torch.Tensor, up_weight: torch.Tensor, down_weight: torch.Tensor, weights: torch.Tensor,
                   indices: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                   residual: torch.Tensor | None = None, status: torch.Tensor | None = None,
                   workspace: torch.Tensor | None = None, return_coef: bool = False, mode: str = "auto",
                   hot: bool | None = None, hot_min_run: int = 0):
    """``y[t] = sum_j w[t,j] * silu(x[t] . Up[e[t,j]]) * Down[e[t,j]]`` (+ residual).

    ``x [T, H]``, ``up/down [N, H]`` bf16; ``weights [T, k]`` fp32; ``indices [T, k]`` int32.
    ``mode="scheduled"``: schedules the pairs by expert, computes the per-pair coefficients in expert
    order, then combines per token.  ``mode="fused"``: one token-centric kernel (tables resident in
    L2, hidden <= 2048).  ``mode="auto"`` picks by table size (:func:`use_fused_path`).
    ``hot`` (scheduled path): experts that own at least ``hot_min_run`` pairs (0 = max(512, T / 32)) get their
    dot products from one dense GEMM instead of a gather per pair; None = :func:`use_hot_experts`.
    ``out_dtype`` float32 or bfloat16; ``residual`` (same dtype as the output) is added in.
    """
    assert mode in ("auto", "fused", "scheduled")
    _lib.require_cuda(x, up_weight, down_weight, weights, indices)
    assert x.dtype == up_weight.dtype == down_weight.dtype == torch.bfloat16
    assert weights.dtype == torch.float32 and indices.dtype == torch.int32
    assert out_dtype in (torch.float32, torch.bfloat16)
    x, up_weight, down_weight = x.contiguous(), up_weight.contiguous(), down_weight.contiguous()
    weights, indices = weights.contiguous(), indices.contiguous()
    t, h = x.shape
    n = up_weight.size(0)
    k = indices.size(1)
    dev = x.device
    if status is None:
        status = _lib.device_status(dev)  # shared per-device word: see _lib.check_device_status
    y = torch.empty((t, h), device=dev, dtype=out_dtype)
    if residual is not None:
        assert residual.shape == y.shape and residual.dtype == out_dtype and residual.is_contiguous()
    coef = torch.empty((t, k), device=dev, dtype=torch.float32)
    if t == 0:
        return (y, coef) if return_coef else y
    if k == 0:
        y.zero_() if residual is None else y.copy_(residual)
        return (y, coef) if return_coef else y
    lib = _lib.load()
    fused = use_fused_path(n, h) if mode == "auto" else mode == "fused"
    if fused:
        with torch.cuda.device(dev):
            _lib.check(lib.omni_expert_fused(x.data_ptr(), up_weight.data_ptr(), down_weight.data_ptr(),
                                             weights.data_ptr(), indices.data_ptr(), t, k, h, n, _lib.ptr(residual),
                                             y.data_ptr(), _lib.dtype_code(out_dtype),
                                             coef.data_ptr() if return_coef else None, status.data_ptr(),
                                             _lib.stream_ptr()))
        return (y, coef) if return_coef else y
    sch = schedule(indices, n, segments=False, workspace=workspace)
    with torch.cuda.device(dev):
        st = _lib.stream_ptr()
        if use_hot_experts(t) if hot is None else hot:
            ws = hot_workspace(t, h, dev)
            _lib.check(lib.omni_expert_coef_hot(x.data_ptr(), up_weight.data_ptr(), weights.data_ptr(),
                                                sch.sorted_pair_ids.data_ptr(), sch.sorted_experts.data_ptr(), t, k, h, n,
                                                hot_min_run, coef.data_ptr(), ws.data_ptr(), ws.numel(),
                                                status.data_ptr(), st))
        else:
            _lib.check(lib.omni_expert_coef(x.data_ptr(), up_weight.data_ptr(), weights.data_ptr(),
                                            sch.sorted_pair_ids.data_ptr(), sch.sorted_experts.data_ptr(), t, k, h, n,
                                            coef.data_ptr(), status.data_ptr(), st))
        _lib.check(lib.omni_expert_combine(down_weight.data_ptr(), coef.data_ptr(), indices.data_ptr(), t, k, h, n,
                                           _lib.ptr(residual), y.data_ptr(), _lib.dtype_code(out_dtype),
                                           status.data_ptr(), st))
    return (y, coef) if return_coef else y


def expert_forward_f32(x: torch.Tensor, up_weight: torch.Tensor, down_weight: torch.Tensor, weights: torch.Tensor,
                       indices: torch.Tensor, residual: torch.Tensor | None = None, status: torch.Tensor | None = None):
    """The routed-expert sum with float32 operands and float32 arithmetic throughout (CUDA cores, one warp per token)."""
    _lib.require_cuda(x, up_weight, down_weight, weights, indices)
    assert x.dtype == up_weight.dtype == down_weight.dtype == weights.dtype == torch.float32 and indices.dtype == torch.int32
    x, up_weight, down_weight = x.contiguous(), up_weight.contiguous(), down_weight.contiguous()
    weights, indices = weights.contiguous(), indices.contiguous()
    t, h = x.shape
    k = indices.size(1)
    y = torch.empty((t, h), device=x.device, dtype=torch.float32)
    if residual is not None:
        assert residual.shape == y.shape and residual.dtype == torch.float32 and residual.is_contiguous()
    if t == 0:
        return y
    if k == 0:
        return y.zero_() if residual is None else y.copy_(residual)
    if status is None:
        status = _lib.device_status(x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().omni_expert_fused_f32(x.data_ptr(), up_weight.data_ptr(), down_weight.data_ptr(), weights.data_ptr(),
                                                     indices.data_ptr(), t, k, h, up_weight.size(0), _lib.ptr(residual),
                                                     y.data_ptr(), status.data_ptr(), _lib.stream_ptr()))
    return y


def omni_expert_func(x: torch.Tensor, up_weight: torch.Tensor, down_weight: torch.Tensor,
                     routing_weights: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Drop-in for ``triton_omni_expert_func`` (omni_moe/ops/triton/interface.py:54-72).

    :param x: (num_tokens, hidden_size)
    :param up_weight, down_weight: (num_experts, hidden_size)
    :param routing_weights: (num_tokens, num_experts_per_token)
    :param indices: (num_tokens, num_experts_per_token) integer expert ids (duplicates allowed)
    :return y: (num_tokens, hidden_size), dtype of ``x``

    bf16 (and fp16, rounded to bf16) operands go to the bf16 kernels: dot products, activation and accumulation in
    fp32.  float32 ``x`` with float32 tables is computed in float32 throughout (``omni_expert_fused_f32``) when no
    gradient is asked for; with gradients the operands are rounded to bf16 (the backward kernels are bf16).
    """
    assert x.dim() == 2 and up_weight.dim() == 2 and down_weight.shape == up_weight.shape
    assert routing_weights.shape == indices.shape and indices.size(0) == x.size(0)
    if x.size(1) % 8:
        # rows that are not whole 16-byte pieces: zero-padded columns add nothing to the dot products and
        # produce output columns that are cut off again
        y = omni_expert_func(pad_last(x), pad_last(up_weight), pad_last(down_weight), routing_weights, indices)
        return y[:, :x.size(1)].contiguous()
    if torch.is_grad_enabled() and any(t.requires_grad for t in (x, up_weight, down_weight, routing_weights)):
        from .autograd import ExpertFunction
        return ExpertFunction.apply(x, up_weight, down_weight, routing_weights, indices)
    if x.dtype == up_weight.dtype == down_weight.dtype == torch.float32 and x.size(1) % 4 == 0 and indices.size(1) <= 128:
        return expert_forward_f32(x.detach(), up_weight.detach(), down_weight.detach(), routing_weights.detach().float(),
                                  indices.to(torch.int32))
    y = expert_forward(as_bf16(x), as_bf16(up_weight), as_bf16(down_weight), routing_weights.detach().float(),
                       indices.to(torch.int32), out_dtype=torch.float32 if x.dtype == torch.float32 else torch.bfloat16)
    return y.to(x.dtype)
