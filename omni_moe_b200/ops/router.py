"""Product-key router ops (reference: omni_moe/ops/triton/omni_router.py, interface.py:32-51)."""
from __future__ import annotations

import torch

from .. import _lib


def _assert_router_inputs(lx, ly, num_expert_sqrt, k):
    # same checks and messages as the reference (omni_moe/ops/triton/utils.py:81-104)
    assert lx.dim() == 2, "router_logits_x must be a 2D tensor of shape (batch_size * seq_len, num_expert_sqrt)"
    assert ly.dim() == 2, "router_logits_y must be a 2D tensor of shape (batch_size * seq_len, num_expert_sqrt)"
    assert lx.size(0) == ly.size(0), "router_logits_x and router_logits_y must have the same first dimension"
    assert 0 <= k <= num_expert_sqrt * num_expert_sqrt, (
        f"num_experts_per_token should be in [0, {num_expert_sqrt * num_expert_sqrt}], but got {k}")
    assert k <= 128, "num_experts_per_token should be less than or equal to 128 for efficiency"
    assert k % 2 == 0, "num_experts_per_token should be a multiple of 2 for efficiency"


def router_topk(log_probs_x: torch.Tensor, log_probs_y: torch.Tensor, num_expert_sqrt: int, k: int,
                index_dtype: torch.dtype = torch.int32, with_weights: bool = False):
    """Top-k over the sqrt(N) x sqrt(N) grid of ``lpx[i] + lpy[j]`` (fp32 sums, ties to the lower index).

    Returns ``(scores float32 [T, k] sorted descending, indices [T, k])`` and, if ``with_weights``,
    ``exp(scores)`` as a third tensor.
    """
    _lib.require_cuda(log_probs_x, log_probs_y)
    assert log_probs_x.shape == log_probs_y.shape and log_probs_x.dim() == 2
    assert log_probs_x.size(1) == num_expert_sqrt, "last dimension must equal num_expert_sqrt"
    assert log_probs_x.dtype == log_probs_y.dtype
    assert index_dtype in (torch.int32, torch.int64)
    lx, ly = log_probs_x.detach().contiguous(), log_probs_y.detach().contiguous()
    t = lx.size(0)
    dev = lx.device
    scores = torch.empty((t, k), device=dev, dtype=torch.float32)
    indices = torch.empty((t, k), device=dev, dtype=index_dtype)
    weights = torch.empty((t, k), device=dev, dtype=torch.float32) if with_weights else None
    if t > 0 and k > 0:
        with torch.cuda.device(dev):
            _lib.check(_lib.load().omni_router_topk(
                lx.data_ptr(), ly.data_ptr(), _lib.dtype_code(lx.dtype), t, num_expert_sqrt, k,
                scores.data_ptr(), indices.data_ptr(), int(index_dtype == torch.int64), _lib.ptr(weights),
                _lib.stream_ptr()))
    return (scores, indices, weights) if with_weights else (scores, indices)


def router_gate_topk(x: torch.Tensor, gate_x: torch.Tensor, gate_y: torch.Tensor, k: int,
                     bn_scale: torch.Tensor | None = None, bn_shift: torch.Tensor | None = None,
                     index_dtype: torch.dtype = torch.int32, return_log_probs: bool = False,
                     status: torch.Tensor | None = None, logits: torch.Tensor | None = None):
    """Router from hidden states: the two gate GEMMs (tcgen05) followed by the fused
    BatchNorm(eval) / log-softmax / top-k kernel.

    ``x [T, H]``, ``gate_x, gate_y [sqrt_n, H]`` bf16; ``bn_scale, bn_shift [2*sqrt_n]`` fp32 fold the
    eval-mode BatchNorm of both axes (None = identity).
    Returns ``(scores fp32, indices, weights fp32 = exp(scores))`` (+ ``log_probs [T, 2*sqrt_n]``).
    """
    _lib.require_cuda(x, gate_x, gate_y)
    assert x.dim() == 2 and gate_x.shape == gate_y.shape and gate_x.size(1) == x.size(1)
    assert x.dtype == gate_x.dtype == gate_y.dtype == torch.bfloat16, "router_gate_topk takes bf16 operands"
    x, gate_x, gate_y = x.contiguous(), gate_x.contiguous(), gate_y.contiguous()
    t, h = x.shape
    n = gate_x.size(0)
    dev = x.device
    if status is None:
        status = _lib.device_status(dev)  # shared per-device word: see _lib.check_device_status
    if logits is None:
        logits = torch.empty((t, 2 * n), device=dev, dtype=torch.float32)
    scores = torch.empty((t, k), device=dev, dtype=torch.float32)
    indices = torch.empty((t, k), device=dev, dtype=index_dtype)
    weights = torch.empty((t, k), device=dev, dtype=torch.float32)
    lp = torch.empty((t, 2 * n), device=dev, dtype=torch.float32) if return_log_probs else None
    if t > 0:
        lib = _lib.load()
        with torch.cuda.device(dev):
            st = _lib.stream_ptr()
            _lib.check(lib.omni_router_gate(x.data_ptr(), gate_x.data_ptr(), gate_y.data_ptr(), t, h, n,
                                            logits.data_ptr(), status.data_ptr(), st))
            _lib.check(lib.omni_router_logits_topk(logits.data_ptr(), 2 * n, _lib.ptr(bn_scale), _lib.ptr(bn_shift),
                                                   t, n, k, scores.data_ptr(), indices.data_ptr(),
                                                   int(index_dtype == torch.int64), weights.data_ptr(),
                                                   _lib.ptr(lp), st))
    out = (scores, indices, weights)
    return out + (lp,) if return_log_probs else out


def omni_router_func(router_logits_x: torch.Tensor, router_logits_y: torch.Tensor, num_expert_sqrt: int,
                     num_experts_per_token: int):
    """Drop-in for ``triton_omni_router_func`` (omni_moe/ops/triton/interface.py:32-51).

    :return scores: (num_tokens, num_experts_per_token), dtype of the inputs, sorted descending
    :return indices: (num_tokens, num_experts_per_token) int32, ``ix * num_expert_sqrt + iy``
    """
    _assert_router_inputs(router_logits_x, router_logits_y, num_expert_sqrt, num_experts_per_token)
    if torch.is_grad_enabled() and (router_logits_x.requires_grad or router_logits_y.requires_grad):
        from .autograd import RouterFunction
        return RouterFunction.apply(router_logits_x, router_logits_y, num_expert_sqrt, num_experts_per_token)
    scores, indices = router_topk(router_logits_x, router_logits_y, num_expert_sqrt, num_experts_per_token)
    return scores.to(router_logits_x.dtype), indices
