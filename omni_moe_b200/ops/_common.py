"""Helpers shared by the op wrappers."""
from __future__ import annotations

import torch


def guard_no_grad(name: str, inputs, outputs):
    """If any input requires grad (and grad mode is on), tie the outputs to a node whose backward raises."""
    if torch.is_grad_enabled() and any(isinstance(t, torch.Tensor) and t.requires_grad for t in inputs):
        anchor = next(t for t in inputs if isinstance(t, torch.Tensor) and t.requires_grad)
        float_outs = [o for o in outputs if o.is_floating_point()]
        if float_outs:
            wrapped = _ForwardOnlyAnchor.apply(name, anchor, *float_outs)
            it = iter(wrapped)
            return tuple(next(it) if o.is_floating_point() else o for o in outputs)
    return tuple(outputs)


class _ForwardOnlyAnchor(torch.autograd.Function):
    @staticmethod
    def forward(ctx, name, anchor, *tensors):
        ctx.name = name
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError(f"{ctx.name}: backward is not implemented in omni_moe_b200 (forward-only build)")


def as_bf16(t: torch.Tensor) -> torch.Tensor:
    """Contiguous bf16 view or copy (the kernels compute on bf16 operands with fp32 accumulation)."""
    t = t.detach()
    if t.dtype != torch.bfloat16:
        t = t.to(torch.bfloat16)
    return t.contiguous()
