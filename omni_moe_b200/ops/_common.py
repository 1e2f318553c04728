"""Helpers shared by the op wrappers."""
from __future__ import annotations

import torch


def as_bf16(t: torch.Tensor) -> torch.Tensor:
    """Contiguous bf16 view or copy (the kernels compute on bf16 operands with fp32 accumulation)."""
    t = t.detach()
    if t.dtype != torch.bfloat16:
        t = t.to(torch.bfloat16)
    return t.contiguous()


def pad_last(t: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """``t`` with its last dimension zero-padded up to a multiple (differentiable).  The kernels move
    rows in 16-byte pieces, i.e. want row lengths that are multiples of 8 bf16 elements; other lengths
    (the reference masks its tails instead, e.g. omni_moe/ops/triton/omni_expert.py:67,123) take this
    slower way round: pad with zeros, compute, cut the result back."""
    pad = (-t.size(-1)) % multiple
    return torch.nn.functional.pad(t, (0, pad)) if pad else t


def pad_both(t: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """2-D ``t`` zero-padded in both dimensions up to multiples (differentiable)."""
    pr, pc = (-t.size(0)) % multiple, (-t.size(1)) % multiple
    return torch.nn.functional.pad(t, (0, pc, 0, pr)) if (pr or pc) else t
