"""Helpers shared by the op wrappers."""
from __future__ import annotations

import torch


def as_bf16(t: torch.Tensor) -> torch.Tensor:
    """Contiguous bf16 view or copy (the kernels compute on bf16 operands with fp32 accumulation)."""
    t = t.detach()
    if t.dtype != torch.bfloat16:
        t = t.to(torch.bfloat16)
    return t.contiguous()
