"""CPU oracle for the OmniMoE layer-forward hot path.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain numpy / fp32 CPU
PyTorch, the algorithm of the reference project's own PyTorch path so the CUDA
kernels can be checked against it.  It is imported by the test-suite, by the
smoke check and by the benchmark's CPU-baseline leg, and by nothing else: the
shipped package never falls back to it.

Parity is pinned: ``tests/golden/`` holds outputs produced by importing the
reference project's ``OmniMoE_Torch`` module, its ``get_scheduling_info`` and
the ``pytorch_*_forward`` mirrors of its test files, and
``tests/test_oracle_golden.py`` checks every function below against them.

Every function cites the reference file (path inside the reference project)
and lines whose behaviour it follows.

Two rules are stated more sharply here than in the reference, because the
reference leaves them to the sort implementation it happens to call:

* router ties: a candidate with the higher fp32 score wins; on an exact score
  tie the lower index wins (per-axis pruning: lower sub-key index; final
  selection: lower flat expert index ``ix * sqrt_n + iy``).  ``torch.topk``
  leaves tie order unspecified (omni_moe/modules/omni_moe.py:162-175).
* scheduling ties: pairs of one expert keep ascending pair-id order
  (``p = token * k + slot``), i.e. a stable sort.  ``torch.sort`` without
  ``stable=True`` (omni_moe/ops/triton/omni_scheduler.py:71) does not promise
  this, so the reference is compared segment-by-segment as sets.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F

BN_EPS = 1e-5  # nn.BatchNorm1d default, omni_moe/modules/omni_moe.py:53-54


# --------------------------------------------------------------------------- #
# router
# --------------------------------------------------------------------------- #
def router_logits(x: torch.Tensor, gate_w: torch.Tensor) -> torch.Tensor:
    """``nn.Linear(bias=False)`` router gate in fp32: ``x @ gate_w.T``.

    Follows omni_moe/modules/omni_moe.py:70-71 (``router_gate_x/y``).
    """
    return x.float() @ gate_w.float().t()


def router_batchnorm_eval(z: torch.Tensor, running_mean: torch.Tensor,
                          running_var: torch.Tensor, eps: float = BN_EPS) -> torch.Tensor:
    """``BatchNorm1d(affine=False)`` in eval mode: ``(z - mean) / sqrt(var + eps)``.

    Follows omni_moe/modules/omni_moe.py:53-54,70-71.
    """
    return (z.float() - running_mean.float()) / torch.sqrt(running_var.float() + eps)


def router_log_probs(z: torch.Tensor) -> torch.Tensor:
    """Per-token log-softmax over one sub-key axis (omni_moe/modules/omni_moe.py:77-78)."""
    return F.log_softmax(z.float(), dim=-1)


def _topk_desc_stable(values: np.ndarray, k: int):
    """Top-k along the last axis ordered (value descending, index ascending)."""
    # A stable ascending argsort of -v keeps equal values in ascending index order.
    order = np.argsort(-values, axis=-1, kind="stable")[..., :k]
    return np.take_along_axis(values, order, axis=-1), order


def router_topk(log_probs_x, log_probs_y, num_expert_sqrt: int, num_experts_per_token: int):
    """Product-key top-k over the sqrt(N) x sqrt(N) grid of ``lpx[i] + lpy[j]``.

    Algorithm of omni_moe/modules/omni_moe.py:162-175 and
    omni_moe/ops/triton/omni_router.py:181-230 (mirror: tests/test_router.py:8-22):
    prune each axis to its ``kk = min(sqrt_n, k)`` best sub-keys, form the
    ``kk x kk`` candidate sums in fp32, take the top k; the expert index is
    ``ix * sqrt_n + iy``.  Scores come back sorted descending.

    Returns ``(scores float32 [T, k], indices int64 [T, k])``.
    """
    lpx = np.asarray(torch.as_tensor(log_probs_x).float().cpu().numpy(), dtype=np.float32)
    lpy = np.asarray(torch.as_tensor(log_probs_y).float().cpu().numpy(), dtype=np.float32)
    n, k = int(num_expert_sqrt), int(num_experts_per_token)
    assert lpx.ndim == 2 and lpy.ndim == 2 and lpx.shape == lpy.shape
    assert lpx.shape[1] == n
    t = lpx.shape[0]
    if k == 0 or t == 0:
        return np.zeros((t, k), np.float32), np.zeros((t, k), np.int64)
    # +0.0 canonicalises -0.0 so it ties with +0.0, as a float comparison would.
    lpx = lpx + np.float32(0.0)
    lpy = lpy + np.float32(0.0)
    kk = min(n, k)
    sx, ix = _topk_desc_stable(lpx, kk)
    sy, iy = _topk_desc_stable(lpy, kk)
    sums = (sx[:, :, None] + sy[:, None, :]).astype(np.float32).reshape(t, kk * kk)
    flat = (ix[:, :, None].astype(np.int64) * n + iy[:, None, :].astype(np.int64)).reshape(t, kk * kk)
    # order: sum descending, flat expert index ascending
    order = np.lexsort((flat, -sums), axis=-1)[:, :k]
    return (np.take_along_axis(sums, order, axis=-1),
            np.take_along_axis(flat, order, axis=-1))


def router_topk_full_grid(log_probs_x, log_probs_y, num_expert_sqrt: int, num_experts_per_token: int):
    """Unpruned restatement: top-k over all N sums.  Used to show pruning is exact
    whenever no two distinct sums tie after fp32 rounding."""
    lpx = torch.as_tensor(log_probs_x).float().numpy() + np.float32(0.0)
    lpy = torch.as_tensor(log_probs_y).float().numpy() + np.float32(0.0)
    n, k = int(num_expert_sqrt), int(num_experts_per_token)
    t = lpx.shape[0]
    sums = (lpx[:, :, None] + lpy[:, None, :]).astype(np.float32).reshape(t, n * n)
    flat = np.broadcast_to(np.arange(n * n, dtype=np.int64), sums.shape)
    order = np.lexsort((flat, -sums), axis=-1)[:, :k]
    return np.take_along_axis(sums, order, axis=-1), order.astype(np.int64)


def routing_weights(scores) -> np.ndarray:
    """``exp(scores)``: product of the two softmax probabilities, not renormalised
    (omni_moe/modules/omni_moe.py:86)."""
    return np.exp(np.asarray(scores, dtype=np.float32)).astype(np.float32)


def routing_flip_gaps(log_probs_x, log_probs_y, oracle_scores, oracle_indices, got_indices, num_expert_sqrt: int):
    """How far from a tie the routing slots are in which another implementation disagrees with :func:`router_topk`.

    An implementation that forms the router logits with a different summation order sees log-probs that
    differ in the last bits, so two candidates whose fp32 scores are closer than that may swap ranks or swap
    in and out of the top k.  For every slot ``[t, j]`` with ``got_indices != oracle_indices`` this returns
    ``|oracle_scores[t, j] - (lpx[t, ix] + lpy[t, iy])|`` where ``(ix, iy)`` is the expert the other
    implementation put there: the distance, in the oracle's own fp32 scores, between the candidate the oracle
    ranks ``j``-th and the one found in its place.  A legitimate flip has a gap of the order of the log-prob
    rounding (1e-5 .. 1e-4); a selection bug shows as a large gap.

    Returns ``(number of differing slots, gaps float32 [that many])``.
    """
    lpx = torch.as_tensor(log_probs_x).float().numpy()
    lpy = torch.as_tensor(log_probs_y).float().numpy()
    es = np.asarray(oracle_scores, dtype=np.float32)
    ei = np.asarray(oracle_indices).astype(np.int64)
    gi = np.asarray(torch.as_tensor(got_indices).cpu().numpy()).astype(np.int64)
    n = int(num_expert_sqrt)
    tt, jj = np.nonzero(gi != ei)
    if tt.size == 0:
        return 0, np.zeros(0, np.float32)
    e = gi[tt, jj]
    ok = (e >= 0) & (e < n * n)
    sc = np.full(tt.shape, -np.inf, np.float32)
    sc[ok] = (lpx[tt[ok], e[ok] // n] + lpy[tt[ok], e[ok] % n]).astype(np.float32)
    return int(tt.size), np.abs(es[tt, jj] - sc).astype(np.float32)


# --------------------------------------------------------------------------- #
# expert-centric scheduling
# --------------------------------------------------------------------------- #
@dataclass
class Schedule:
    """Tail fields of the reference ``SchedulingInfo`` (omni_moe/ops/triton/omni_scheduler.py:5-43)."""
    tail_token_ids: np.ndarray          # int32 [P]
    tail_expert_ids: np.ndarray         # int32 [U] ascending unique experts
    tail_routing_weights: np.ndarray    # [P] weights in sorted order
    tail_offsets: np.ndarray            # int32 [U+1] CSR offsets
    tail_sorted_pair_ids: np.ndarray    # int32 [P] stable permutation
    num_tail_experts: int
    max_tail_pairs_per_expert: int


def schedule(routing_w, indices, num_experts: int) -> Schedule:
    """Sort the T*k (token, expert) pairs by expert and build CSR offsets.

    Follows the tail path of ``get_scheduling_info``
    (omni_moe/ops/triton/omni_scheduler.py:61-101) with the sort made stable.
    """
    idx = np.asarray(torch.as_tensor(indices).cpu().numpy())
    g = np.asarray(torch.as_tensor(routing_w).float().cpu().numpy())
    t, k = idx.shape
    p = t * k
    expert = idx.reshape(-1).astype(np.int64)
    if p:
        assert expert.min() >= 0 and expert.max() < num_experts, "expert index out of range"
    perm = np.argsort(expert, kind="stable").astype(np.int32)
    sorted_e = expert[perm]
    token_ids = (perm // max(k, 1)).astype(np.int32)
    uniq, counts = np.unique(sorted_e, return_counts=True)
    offsets = np.zeros(len(uniq) + 1, np.int32)
    offsets[1:] = np.cumsum(counts)
    return Schedule(
        tail_token_ids=token_ids,
        tail_expert_ids=uniq.astype(np.int32),
        tail_routing_weights=g.reshape(-1)[perm],
        tail_offsets=offsets,
        tail_sorted_pair_ids=perm,
        num_tail_experts=int(len(uniq)),
        max_tail_pairs_per_expert=int(counts.max()) if p else 0,
    )


# --------------------------------------------------------------------------- #
# routed experts
# --------------------------------------------------------------------------- #
def expert_forward(x, up_w, down_w, routing_w, indices, chunk: int = 1024) -> torch.Tensor:
    """``y[t] = sum_j g[t,j] * silu(x[t] . Up[e[t,j]]) * Down[e[t,j]]`` in fp32.

    Follows omni_moe/modules/omni_moe.py:181-189 and tests/test_expert.py:8-25.
    The reference materialises ``[T, k, H]`` gathers; tokens are independent, so
    this runs in token chunks to bound memory.
    """
    x = torch.as_tensor(x).float()
    up_w = torch.as_tensor(up_w)
    down_w = torch.as_tensor(down_w)
    g = torch.as_tensor(routing_w).float()
    idx = torch.as_tensor(indices).long()
    t, h = x.shape
    out = torch.empty(t, h, dtype=torch.float32)
    for s in range(0, t, chunk):
        e = min(t, s + chunk)
        up = up_w[idx[s:e]].float()                       # [c, k, H]
        dn = down_w[idx[s:e]].float()
        sc = torch.matmul(up, x[s:e].unsqueeze(-1)).squeeze(-1)   # [c, k]
        co = F.silu(sc) * g[s:e]
        out[s:e] = torch.matmul(co.unsqueeze(-2), dn).squeeze(-2)
    return out


def expert_coefficients(x, up_w, routing_w, indices) -> torch.Tensor:
    """Per-pair coefficient ``g * silu(x . Up[e])`` (omni_moe/modules/omni_moe.py:183-186)."""
    x = torch.as_tensor(x).float()
    idx = torch.as_tensor(indices).long()
    up = torch.as_tensor(up_w)[idx].float()
    sc = torch.matmul(up, x.unsqueeze(-1)).squeeze(-1)
    return F.silu(sc) * torch.as_tensor(routing_w).float()


# --------------------------------------------------------------------------- #
# shared SwiGLU MLP
# --------------------------------------------------------------------------- #
def mlp_forward(x, gate_w, up_w, down_w, limit=None) -> torch.Tensor:
    """``(silu(x Wg^T) * (x Wu^T)) Wd^T`` in fp32.

    Follows omni_moe/modules/omni_moe.py:190-192, omni_moe/ops/triton/interface.py:23-29
    and tests/test_mlp.py:8-21.  ``limit`` is the clamp of the reference's fused activation
    (``compute_silu_mul``, omni_moe/ops/triton/omni_mlp.py:54-61, ``PrecisionConfig.limit`` :27):
    gate and up are limited to ``[-limit, limit]`` before ``silu(gate) * up``; the reference's public
    entry never sets it, so ``None`` is the layer's behaviour.
    """
    x = torch.as_tensor(x).float()
    g, u = x @ torch.as_tensor(gate_w).float().t(), x @ torch.as_tensor(up_w).float().t()
    if limit is not None:
        g, u = g.clamp(-limit, limit), u.clamp(-limit, limit)
    return (F.silu(g) * u) @ torch.as_tensor(down_w).float().t()


# --------------------------------------------------------------------------- #
# whole layer
# --------------------------------------------------------------------------- #
@dataclass
class LayerParams:
    """Parameter / buffer set of the reference module, same names and shapes
    (omni_moe/modules/omni_moe.py:42-58)."""
    gate_proj: torch.Tensor       # [I, H]
    up_proj: torch.Tensor         # [I, H]
    down_proj: torch.Tensor       # [H, I]
    router_gate_x: torch.Tensor   # [sqrtN, H]
    router_gate_y: torch.Tensor   # [sqrtN, H]
    norm_x_mean: torch.Tensor     # [sqrtN]
    norm_x_var: torch.Tensor
    norm_y_mean: torch.Tensor
    norm_y_var: torch.Tensor
    up_embed: torch.Tensor        # [N, H]
    down_embed: torch.Tensor      # [N, H]
    num_experts: int
    top_k: int

    @property
    def sqrt_n(self) -> int:
        return math.floor(math.sqrt(self.num_experts))  # omni_moe/modules/omni_moe.py:38


def router_batchnorm_train(z: torch.Tensor, eps: float = BN_EPS):
    """``BatchNorm1d(affine=False)`` in training mode: every column is normalised with the mean and the
    biased variance of the batch (all tokens of the call), omni_moe/modules/omni_moe.py:53-54,70-71.
    Returns ``(normalised, batch mean, unbiased batch variance)``; the last two are what the running
    statistics are updated with (momentum 0.1 by default)."""
    z = z.float()
    var_b, mean_b = torch.var_mean(z, dim=0, unbiased=False)
    t = z.size(0)
    return (z - mean_b) / torch.sqrt(var_b + eps), mean_b, var_b * (t / max(t - 1, 1))


def layer_forward(p: LayerParams, hidden_states, return_routing: bool = False, chunk: int = 1024,
                  training: bool = False):
    """``OmniMoE_Torch.forward`` in fp32 (omni_moe/modules/omni_moe.py:139-194): eval mode (running
    statistics) by default, batch statistics with ``training=True`` (the module as constructed)."""
    hs = torch.as_tensor(hidden_states)
    shape = hs.shape
    x = hs.reshape(-1, shape[-1]).float()
    n = p.sqrt_n
    zx, zy = router_logits(x, p.router_gate_x), router_logits(x, p.router_gate_y)
    if training:
        zx, zy = router_batchnorm_train(zx)[0], router_batchnorm_train(zy)[0]
    else:
        zx = router_batchnorm_eval(zx, p.norm_x_mean, p.norm_x_var)
        zy = router_batchnorm_eval(zy, p.norm_y_mean, p.norm_y_var)
    lpx, lpy = router_log_probs(zx), router_log_probs(zy)
    scores, idx = router_topk(lpx, lpy, n, p.top_k)
    w = routing_weights(scores)
    y = expert_forward(x, p.up_embed, p.down_embed, w, idx, chunk=chunk)
    y += mlp_forward(x, p.gate_proj, p.up_proj, p.down_proj)
    y = y.reshape(shape)
    if return_routing:
        return y, lpx, lpy, scores, idx
    return y


def params_from_state_dict(sd: dict, num_experts: int, top_k: int) -> LayerParams:
    """Build :class:`LayerParams` from a reference-style ``state_dict``."""
    return LayerParams(
        gate_proj=sd["gate_proj.weight"], up_proj=sd["up_proj.weight"], down_proj=sd["down_proj.weight"],
        router_gate_x=sd["router_gate_x.weight"], router_gate_y=sd["router_gate_y.weight"],
        norm_x_mean=sd["router_norm_x.running_mean"], norm_x_var=sd["router_norm_x.running_var"],
        norm_y_mean=sd["router_norm_y.running_mean"], norm_y_var=sd["router_norm_y.running_var"],
        up_embed=sd["up_embed.weight"], down_embed=sd["down_embed.weight"],
        num_experts=num_experts, top_k=top_k,
    )


# ------------------------------------------------------------------------------------------------
# Backward references.  The reference's tests obtain gradients by running torch autograd through the
# PyTorch mirrors of the three operators (tests/test_router.py:36-50,73-95,
# tests/test_expert.py and tests/test_mlp.py backward factories); these functions do the same in
# fp32 on the CPU.
# ------------------------------------------------------------------------------------------------
def router_backward(dscores, indices, num_expert_sqrt: int):
    """Gradients of ``scores[t,j] = lpx[t, ix] + lpy[t, iy]`` with respect to both log-prob tables:
    every score gradient is added to column ``ix`` of the x axis and ``iy`` of the y axis
    (what autograd yields for the topk / gather chain of tests/test_router.py:8-22; the reference's
    kernel: omni_moe/ops/triton/omni_router.py:104-164)."""
    ds = torch.as_tensor(dscores).double()
    idx = torch.as_tensor(indices).long()
    t = idx.size(0)
    dlx = torch.zeros(t, num_expert_sqrt, dtype=torch.float64)
    dly = torch.zeros(t, num_expert_sqrt, dtype=torch.float64)
    dlx.scatter_add_(1, idx // num_expert_sqrt, ds)
    dly.scatter_add_(1, idx % num_expert_sqrt, ds)
    return dlx.float(), dly.float()


def expert_backward(x, up_w, down_w, routing_w, indices, dy):
    """``(dx, d_up, d_down, dg)`` of :func:`expert_forward` by autograd in fp32 (small cases only:
    the dense table gradients are materialised)."""
    x = torch.as_tensor(x).float().clone().requires_grad_(True)
    up = torch.as_tensor(up_w).float().clone().requires_grad_(True)
    dn = torch.as_tensor(down_w).float().clone().requires_grad_(True)
    g = torch.as_tensor(routing_w).float().clone().requires_grad_(True)
    idx = torch.as_tensor(indices).long()
    sc = torch.matmul(up[idx], x.unsqueeze(-1)).squeeze(-1)
    y = torch.matmul((F.silu(sc) * g).unsqueeze(-2), dn[idx]).squeeze(-2)
    y.backward(torch.as_tensor(dy).float())
    return x.grad, up.grad, dn.grad, g.grad


def mlp_backward(x, gate_w, up_w, down_w, dy, limit=None, preact_dtype=None):
    """``(dx, d_gate_w, d_up_w, d_down_w)`` of :func:`mlp_forward` by autograd in fp32.

    ``preact_dtype`` (e.g. ``torch.bfloat16``): round the gate / up pre-activations to that dtype before
    the clamp and the activation, with the gradient passed straight through the rounding.  The
    reference keeps gate and up in the input dtype between its GEMMs and its activation kernels
    (omni_moe/ops/triton/omni_mlp.py:359-375), so with ``limit`` the set of clamped entries (a
    discontinuity of the gradient) is decided on the rounded values."""
    x = torch.as_tensor(x).float().clone().requires_grad_(True)
    wg = torch.as_tensor(gate_w).float().clone().requires_grad_(True)
    wu = torch.as_tensor(up_w).float().clone().requires_grad_(True)
    wd = torch.as_tensor(down_w).float().clone().requires_grad_(True)
    g, u = F.linear(x, wg), F.linear(x, wu)
    if preact_dtype is not None:
        g = g + (g.detach().to(preact_dtype).float() - g.detach())
        u = u + (u.detach().to(preact_dtype).float() - u.detach())
    if limit is not None:
        g, u = g.clamp(-limit, limit), u.clamp(-limit, limit)
    y = F.linear(F.silu(g) * u, wd)
    y.backward(torch.as_tensor(dy).float())
    return x.grad, wg.grad, wu.grad, wd.grad


def layer_gradients(p: "LayerParams", hidden_states, indices, dy, training: bool):
    """Gradients of the whole layer (omni_moe/modules/omni_moe.py:60-106) for FIXED routing indices,
    by fp32 autograd: returns ``(y, dict name -> gradient)`` with the reference's parameter names plus
    ``"x"``.  The selection itself is not differentiable, so the indices are an input here; BatchNorm
    uses batch statistics when ``training`` (biased variance, as nn.BatchNorm1d normalises) and the
    running statistics otherwise."""
    x = torch.as_tensor(hidden_states).float().reshape(-1, p.gate_proj.shape[1]).clone().requires_grad_(True)
    names = ["gate_proj.weight", "up_proj.weight", "down_proj.weight", "router_gate_x.weight", "router_gate_y.weight",
             "up_embed.weight", "down_embed.weight"]
    vals = [p.gate_proj, p.up_proj, p.down_proj, p.router_gate_x, p.router_gate_y, p.up_embed, p.down_embed]
    w = {n: torch.as_tensor(v).float().clone().requires_grad_(True) for n, v in zip(names, vals)}
    idx = torch.as_tensor(indices).long()
    n = p.sqrt_n
    eps = 1e-5  # nn.BatchNorm1d default, omni_moe/modules/omni_moe.py:53-54

    def norm(z, mean, var):
        if training:
            var_b, mean_b = torch.var_mean(z, dim=0, unbiased=False)
            return (z - mean_b) / torch.sqrt(var_b + eps)
        return (z - torch.as_tensor(mean).float()) / torch.sqrt(torch.as_tensor(var).float() + eps)

    lpx = F.log_softmax(norm(F.linear(x, w["router_gate_x.weight"]), p.norm_x_mean, p.norm_x_var), dim=-1)
    lpy = F.log_softmax(norm(F.linear(x, w["router_gate_y.weight"]), p.norm_y_mean, p.norm_y_var), dim=-1)
    scores = lpx.gather(1, idx // n) + lpy.gather(1, idx % n)
    g = torch.exp(scores)
    sc = torch.matmul(w["up_embed.weight"][idx], x.unsqueeze(-1)).squeeze(-1)
    experts = torch.matmul((F.silu(sc) * g).unsqueeze(-2), w["down_embed.weight"][idx]).squeeze(-2)
    shared = F.linear(F.silu(F.linear(x, w["gate_proj.weight"])) * F.linear(x, w["up_proj.weight"]), w["down_proj.weight"])
    y = shared + experts
    y.backward(torch.as_tensor(dy).float().reshape(y.shape))
    grads = {k: v.grad for k, v in w.items()}
    grads["x"] = x.grad
    return y.detach(), grads
