"""Shared SwiGLU MLP op (reference: omni_moe/ops/triton/interface.py:7-29, omni_mlp.py:252-303)."""
from __future__ import annotations

import torch

from .. import _lib
from ._common import as_bf16, pad_both, pad_last


def mlp_forward(x: torch.Tensor, gate_weight: torch.Tensor, up_weight: torch.Tensor, down_weight: torch.Tensor,
                residual: torch.Tensor | None = None, status: torch.Tensor | None = None,
                act: torch.Tensor | None = None, gate_up: torch.Tensor | None = None,
                limit: float | None = None) -> torch.Tensor:
    """``(silu(x Wg^T) * (x Wu^T)) Wd^T (+ residual)`` on bf16 operands with two tcgen05 GEMMs.

    ``residual``: optional fp32 ``[T, H]`` added before the result is rounded to bf16.
    ``act``: optional bf16 ``[T, I]`` scratch for the activation.
    ``gate_up``: optional bf16 ``[T, 2I]`` that receives the pre-activations ``(x Wg^T | x Wu^T)`` (kept
    for the backward in training).
    ``limit``: optional clamp of the reference's fused activation (``compute_silu_mul``,
    omni_moe/ops/triton/omni_mlp.py:54-61): gate and up are limited to ``[-limit, limit]`` before
    ``silu(gate) * up``; ``gate_up`` still receives the unclamped values.
    """
    assert limit is None or limit > 0, "limit must be positive"
    _lib.require_cuda(x, gate_weight, up_weight, down_weight)
    assert x.dtype == gate_weight.dtype == up_weight.dtype == down_weight.dtype == torch.bfloat16
    x, gate_weight, up_weight, down_weight = (v.contiguous() for v in (x, gate_weight, up_weight, down_weight))
    t, h = x.shape
    i = gate_weight.size(0)
    assert gate_weight.shape == up_weight.shape == (i, h) and down_weight.shape == (h, i)
    dev = x.device
    if status is None:
        status = _lib.device_status(dev)  # shared per-device word: see _lib.check_device_status
    if act is None:
        act = torch.empty((t, i), device=dev, dtype=torch.bfloat16)
    if residual is not None:
        assert residual.shape == (t, h) and residual.dtype == torch.float32 and residual.is_contiguous()
    y = torch.empty((t, h), device=dev, dtype=torch.bfloat16)
    if gate_up is not None:
        assert gate_up.shape == (t, 2 * i) and gate_up.dtype == torch.bfloat16 and gate_up.is_contiguous()
    if t > 0:
        lib = _lib.load()
        with torch.cuda.device(dev):
            st = _lib.stream_ptr()
            if limit is not None:
                _lib.check(lib.omni_mlp_gate_up_limit(x.data_ptr(), gate_weight.data_ptr(), up_weight.data_ptr(), t, h, i,
                                                      float(limit), act.data_ptr(), _lib.ptr(gate_up), status.data_ptr(), st))
            elif gate_up is None:
                _lib.check(lib.omni_mlp_gate_up(x.data_ptr(), gate_weight.data_ptr(), up_weight.data_ptr(), t, h, i,
                                                act.data_ptr(), status.data_ptr(), st))
            else:
                _lib.check(lib.omni_mlp_gate_up_save(x.data_ptr(), gate_weight.data_ptr(), up_weight.data_ptr(), t, h, i,
                                                     act.data_ptr(), gate_up.data_ptr(), status.data_ptr(), st))
            _lib.check(lib.omni_mlp_down(act.data_ptr(), down_weight.data_ptr(), t, h, i, _lib.ptr(residual), y.data_ptr(),
                                         status.data_ptr(), st))
    return y


def omni_mlp_func(x: torch.Tensor, gate_weight: torch.Tensor, up_weight: torch.Tensor,
                  down_weight: torch.Tensor, limit: float | None = None) -> torch.Tensor:
    """Drop-in for ``triton_omni_mlp_func`` (omni_moe/ops/triton/interface.py:7-29).

    :param x: (num_tokens, hidden_size)
    :param gate_weight, up_weight: (intermediate_size, hidden_size)
    :param down_weight: (hidden_size, intermediate_size)
    :param limit: optional clamp of gate and up before the activation (the ``limit`` of the reference's
        ``PrecisionConfig``, omni_moe/ops/triton/omni_mlp.py:27,54-61, which its public entry leaves unset)
    :return y: (num_tokens, hidden_size), dtype of ``x``

    bf16 tensors (and fp16, rounded to bf16) run the two tcgen05 GEMMs of this library with fp32 accumulation; all-float32
    tensors are computed in float32 by torch's matmuls (see below).
    """
    assert x.dim() == 2
    if all(t.dtype == torch.float32 for t in (x, gate_weight, up_weight, down_weight)):
        # float32 tensors get float32 arithmetic, as the reference gives them (its three projections are library GEMMs,
        # omni_moe/ops/triton/interface.py:23-29): this one case does not run the kernels of this library but torch's
        # float32 matmuls and elementwise operators, differentiable through autograd.  bf16 / fp16 tensors, and every
        # path of the module's fused forward, use the tcgen05 kernels below.
        _lib.require_cuda(x, gate_weight, up_weight, down_weight)
        g = torch.nn.functional.linear(x, gate_weight)
        u = torch.nn.functional.linear(x, up_weight)
        if limit is not None:
            assert limit > 0, "limit must be positive"
            g, u = g.clamp(-limit, limit), u.clamp(-limit, limit)
        return torch.nn.functional.linear(torch.nn.functional.silu(g) * u, down_weight)
    if x.size(1) % 8 or gate_weight.size(0) % 8:
        # hidden or intermediate size not a multiple of 8: zero padding leaves the result unchanged
        # (padded gate / up rows give silu(0) * 0 = 0 against zero columns of the down projection)
        y = omni_mlp_func(pad_last(x), pad_both(gate_weight), pad_both(up_weight), pad_both(down_weight), limit)
        return y[:, :x.size(1)].contiguous()
    if torch.is_grad_enabled() and any(t.requires_grad for t in (x, gate_weight, up_weight, down_weight)):
        from .autograd import MlpFunction
        return MlpFunction.apply(x, gate_weight, up_weight, down_weight, limit)
    return mlp_forward(as_bf16(x), as_bf16(gate_weight), as_bf16(up_weight), as_bf16(down_weight), limit=limit).to(x.dtype)
