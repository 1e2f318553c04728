"""Autograd functions of the three operators: forward through the forward kernels, backward through
the kernels of ``csrc/backward.cu`` and the GEMMs of ``csrc/gemm_tcgen05.cu``.

Reference counterparts: ``OmniRouterFunc`` (omni_moe/ops/triton/omni_router.py:277-305),
``OmniExpertFunc`` (omni_moe/ops/triton/omni_expert.py:1280-1360) and ``TritonSwiGLUFunc`` with the
three ``nn.functional.linear`` calls around it (omni_moe/ops/triton/omni_mlp.py:359-375,
interface.py:7-29).  Gradients come back in the dtype of the corresponding input.
"""
from __future__ import annotations

import torch

from .. import _lib
from ._common import as_bf16
from .scheduler import schedule


def _status(dev) -> torch.Tensor:
    """The per-device status word (see _lib.device_status): faults of the backward kernels surface in
    _lib.check_device_status() / OmniMoE.check_status()."""
    return _lib.device_status(dev)


# ------------------------------------------------------------------------------------------------
# router
# ------------------------------------------------------------------------------------------------
def router_backward(dscores: torch.Tensor, indices: torch.Tensor, num_expert_sqrt: int):
    """``(dlog_probs_x, dlog_probs_y)`` fp32 ``[T, sqrt_n]`` from ``dscores [T, k]`` and the selected indices."""
    _lib.require_cuda(dscores, indices)
    assert dscores.shape == indices.shape and indices.dtype in (torch.int32, torch.int64)
    t, k = indices.shape
    dev = indices.device
    ds = dscores.detach().float().contiguous()
    indices = indices.contiguous()
    dlx = torch.empty((t, num_expert_sqrt), device=dev, dtype=torch.float32)
    dly = torch.empty((t, num_expert_sqrt), device=dev, dtype=torch.float32)
    status = _status(dev)
    if t > 0:
        with torch.cuda.device(dev):
            _lib.check(_lib.load().omni_router_bwd(ds.data_ptr(), indices.data_ptr(), int(indices.dtype == torch.int64), t,
                                                   num_expert_sqrt, k, dlx.data_ptr(), dly.data_ptr(), status.data_ptr(),
                                                   _lib.stream_ptr()))
    return dlx, dly


class RouterFunction(torch.autograd.Function):
    """scores, indices = top-k of lpx[i] + lpy[j]; d/dlpx[ix] += dscore, d/dlpy[iy] += dscore."""

    @staticmethod
    def forward(ctx, log_probs_x, log_probs_y, num_expert_sqrt, k):
        from .router import router_topk
        scores, indices = router_topk(log_probs_x, log_probs_y, num_expert_sqrt, k)
        ctx.save_for_backward(indices)
        ctx.n = num_expert_sqrt
        ctx.dtypes = (log_probs_x.dtype, log_probs_y.dtype)
        ctx.mark_non_differentiable(indices)
        return scores.to(log_probs_x.dtype), indices

    @staticmethod
    def backward(ctx, dscores, _dindices):
        (indices,) = ctx.saved_tensors
        dlx, dly = router_backward(dscores, indices, ctx.n)
        return dlx.to(ctx.dtypes[0]), dly.to(ctx.dtypes[1]), None, None


# ------------------------------------------------------------------------------------------------
# routed experts
# ------------------------------------------------------------------------------------------------
def expert_backward(dy: torch.Tensor, x: torch.Tensor, up_weight: torch.Tensor, down_weight: torch.Tensor,
                    weights: torch.Tensor, indices: torch.Tensor, grad_dtype: torch.dtype = torch.bfloat16,
                    compact: bool = False, need_tables: bool = True, long_segments: bool | int = True):
    """Backward of ``y[t] = sum_j g[t,j] * silu(x[t].Up[e]) * Down[e]`` for bf16 operands.

    Returns ``(dx [T,H] grad_dtype, d_up, d_down, dg [T,k] fp32, expert_ids)``.  With ``compact=False``
    ``d_up / d_down`` are dense ``[N, H]`` tables (zero rows for untouched experts) and ``expert_ids`` is
    None; with ``compact=True`` they hold one row per touched expert, ``expert_ids[s]`` names the
    expert of row ``s`` and rows beyond the number of touched experts are unspecified
    (``expert_ids`` is cut to the valid length, which costs one host read).
    ``long_segments``: give the row kernel its scratch so that experts with many pairs are summed by many
    blocks in two levels instead of by one warp (True: the library's choice of split, at most 256 MiB unless
    even the coarsest split needs more; 64 / 128 / 256 / 512: that many sorted positions per block).
    """
    _lib.require_cuda(dy, x, up_weight, down_weight, weights, indices)
    assert x.dtype == up_weight.dtype == down_weight.dtype == dy.dtype == torch.bfloat16
    assert weights.dtype == torch.float32 and indices.dtype == torch.int32
    assert grad_dtype in (torch.float32, torch.bfloat16)
    x, up_weight, down_weight, dy = x.contiguous(), up_weight.contiguous(), down_weight.contiguous(), dy.contiguous()
    weights, indices = weights.contiguous(), indices.contiguous()
    t, h = x.shape
    n = up_weight.size(0)
    k = indices.size(1)
    dev = x.device
    f32 = dict(device=dev, dtype=torch.float32)
    ds, cdown, dg = torch.empty((t, k), **f32), torch.empty((t, k), **f32), torch.empty((t, k), **f32)
    dx = torch.empty((t, h), device=dev, dtype=grad_dtype)
    status = _status(dev)
    lib = _lib.load()
    d_up = d_down = expert_ids = None
    if t == 0 or k == 0:
        dx.zero_()
        if need_tables and not compact:
            d_up = torch.zeros((n, h), device=dev, dtype=grad_dtype)
            d_down = torch.zeros((n, h), device=dev, dtype=grad_dtype)
        return dx, d_up, d_down, dg, expert_ids
    fuse_dx = bool(lib.omni_expert_bwd_dots_fuses_dx(h))
    with torch.cuda.device(dev):
        st = _lib.stream_ptr()
        _lib.check(lib.omni_expert_bwd_dots(x.data_ptr(), up_weight.data_ptr(), down_weight.data_ptr(), dy.data_ptr(),
                                            weights.data_ptr(), indices.data_ptr(), t, k, h, n, ds.data_ptr(),
                                            cdown.data_ptr(), dg.data_ptr(), dx.data_ptr() if fuse_dx else None,
                                            _lib.dtype_code(grad_dtype), status.data_ptr(), st))
        if not fuse_dx:
            # dx[t] = sum_j ds[t,j] * Up[e[t,j]]: the forward's token-centric combine with the Up table
            _lib.check(lib.omni_expert_combine(up_weight.data_ptr(), ds.data_ptr(), indices.data_ptr(), t, k, h, n, None,
                                               dx.data_ptr(), _lib.dtype_code(grad_dtype), status.data_ptr(), st))
    if need_tables:
        sch = schedule(indices, n, segments=True)
        cap = sch.expert_ids.numel()
        rows = cap if compact else n
        alloc = torch.empty if compact else torch.zeros
        d_up = alloc((rows, h), device=dev, dtype=grad_dtype)
        d_down = alloc((rows, h), device=dev, dtype=grad_dtype)
        scratch = None
        if long_segments is True:
            scratch = torch.empty(int(lib.omni_expert_bwd_rows_scratch_bytes(t * k, h)), device=dev, dtype=torch.uint8)
        elif long_segments:
            # an explicit split: room for partial rows of blocks of `long_segments` sorted positions
            blocks = -(-(t * k) // int(long_segments))
            header = ((blocks + 1) * 4 + 255) // 256 * 256
            scratch = torch.empty(header + 2 * blocks * 2 * h * 4, device=dev, dtype=torch.uint8)
        with torch.cuda.device(dev):
            _lib.check(lib.omni_expert_bwd_rows(x.data_ptr(), dy.data_ptr(), ds.data_ptr(), cdown.data_ptr(),
                                                sch.sorted_pair_ids.data_ptr(), sch.expert_ids.data_ptr(),
                                                sch.offsets.data_ptr(), sch.meta.data_ptr(), sch.meta[1:].data_ptr(), cap, t, k, h,
                                                int(compact),
                                                d_up.data_ptr(), d_down.data_ptr(), _lib.dtype_code(grad_dtype),
                                                _lib.ptr(scratch), scratch.numel() if scratch is not None else 0,
                                                status.data_ptr(), _lib.stream_ptr()))
        if compact:
            u = int(sch.meta[0].item())
            d_up, d_down, expert_ids = d_up[:u], d_down[:u], sch.expert_ids[:u]
    return dx, d_up, d_down, dg, expert_ids


class ExpertFunction(torch.autograd.Function):
    """Routed-expert sum with gradients for x, both tables and the routing weights."""

    @staticmethod
    def forward(ctx, x, up_weight, down_weight, routing_weights, indices):
        from .expert import expert_forward
        xb, ub, db = as_bf16(x), as_bf16(up_weight), as_bf16(down_weight)
        g = routing_weights.detach().float().contiguous()
        idx = indices.to(torch.int32).contiguous()
        y = expert_forward(xb, ub, db, g, idx, out_dtype=torch.float32 if x.dtype == torch.float32 else torch.bfloat16)
        ctx.save_for_backward(xb, ub, db, g, idx)
        ctx.dtypes = (x.dtype, up_weight.dtype, down_weight.dtype, routing_weights.dtype)
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        xb, ub, db, g, idx = ctx.saved_tensors
        need_tables = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        all_f32 = all(d == torch.float32 for d in ctx.dtypes[:3])
        dx, d_up, d_down, dg, _ = expert_backward(as_bf16(dy), xb, ub, db, g, idx,
                                                  grad_dtype=torch.float32 if all_f32 else torch.bfloat16,
                                                  need_tables=need_tables)
        return (dx.to(ctx.dtypes[0]) if ctx.needs_input_grad[0] else None,
                d_up.to(ctx.dtypes[1]) if ctx.needs_input_grad[1] else None,
                d_down.to(ctx.dtypes[2]) if ctx.needs_input_grad[2] else None,
                dg.to(ctx.dtypes[3]) if ctx.needs_input_grad[3] else None, None)


# ------------------------------------------------------------------------------------------------
# shared SwiGLU MLP
# ------------------------------------------------------------------------------------------------
def _pad8(v: int) -> int:
    return (v + 7) // 8 * 8


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, status: torch.Tensor | None = None):
    """``a [m, k] @ b [n, k]^T`` for bf16 row-major operands (fp32 accumulation, bf16 result).
    ``out`` may be a column slice of a wider row-major matrix (its row stride is honoured)."""
    _lib.require_cuda(a, b)
    assert a.dtype == b.dtype == torch.bfloat16 and a.dim() == b.dim() == 2 and a.size(1) == b.size(1)
    assert a.is_contiguous() and b.is_contiguous()
    m, k = a.shape
    n = b.size(0)
    if out is None:
        out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    if status is None:
        status = _status(a.device)
    if m and n:
        with torch.cuda.device(a.device):
            _lib.check(_lib.load().omni_gemm_bf16_nt(a.data_ptr(), b.data_ptr(), m, n, k, out.data_ptr(), out.stride(0),
                                                     status.data_ptr(), _lib.stream_ptr()))
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, a_transposed: bool = False, b_transposed: bool = False,
         out: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """``out [m, n] = A @ B^T`` with ``A = a`` (``[m, k]``) or ``a^T`` (``a`` is ``[k, m]``, ``a_transposed``) and
    ``B = b`` (``[n, k]``) or ``b^T`` (``b`` is ``[k, n]``, ``b_transposed``): bf16 operands read where they lie
    (row strides honoured, so column slices of wider matrices work), fp32 accumulation, bf16 result."""
    _lib.require_cuda(a, b)
    assert a.dtype == b.dtype == torch.bfloat16 and a.dim() == b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    k, m = a.shape if a_transposed else a.shape[::-1]
    kb, n = b.shape if b_transposed else b.shape[::-1]
    assert k == kb, f"contraction sizes differ: {k} vs {kb}"
    if out is None:
        out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    if status is None:
        status = _status(a.device)
    if m and n:
        with torch.cuda.device(a.device):
            _lib.check(_lib.load().omni_gemm_bf16(a.data_ptr(), int(a_transposed), a.stride(0), b.data_ptr(), int(b_transposed),
                                                  b.stride(0), m, n, k, out.data_ptr(), out.stride(0), status.data_ptr(),
                                                  _lib.stream_ptr()))
    return out


def transpose_padded(src: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``src [r, c]`` bf16 (row stride honoured) -> ``[c, pad8(r)]`` with zero padding columns, or into
    ``out``, a ``[c, >= r]`` column slice of a wider row-major matrix."""
    assert src.dtype == torch.bfloat16 and src.dim() == 2 and src.stride(1) == 1
    r, c = src.shape
    if out is None:
        out = torch.empty((c, _pad8(r)), device=src.device, dtype=torch.bfloat16)
    assert out.dtype == torch.bfloat16 and out.size(0) == c and out.size(1) >= r and out.stride(1) == 1
    if c:
        with torch.cuda.device(src.device):
            _lib.check(_lib.load().omni_transpose_bf16(src.data_ptr(), r, c, src.stride(0), out.data_ptr(), out.size(1),
                                                       out.stride(0), _lib.stream_ptr()))
    return out


def _operands_in_place() -> bool:
    """The gradient GEMMs read transposed operands in place on the CTA-pair kernels; with the single-CTA
    kernels forced (``OMNI_MOE_B200_GEMM=1cta``) or ``OMNI_MOE_B200_MLP_BWD=copies`` they go through
    transposed copies and the K-contiguous GEMM."""
    import os
    return os.environ.get("OMNI_MOE_B200_GEMM", "")[:1] != "1" and os.environ.get("OMNI_MOE_B200_MLP_BWD", "") != "copies"


def mlp_backward(dy: torch.Tensor, x: torch.Tensor, gate_weight: torch.Tensor, up_weight: torch.Tensor,
                 down_weight: torch.Tensor, need_weight_grads: bool = True, gate_up: torch.Tensor | None = None,
                 limit: float | None = None):
    """Backward of ``y = (silu(x Wg^T) * (x Wu^T)) Wd^T`` on bf16 operands.

    ``gate_up [T, 2I]`` bf16 are the pre-activations saved by the training forward
    (``mlp_forward(..., gate_up=...)``); without them they are recomputed here with two more GEMMs.
    ``limit``: the clamp the forward ran with (``mlp_forward(..., limit=...)``), if any.
    GEMMs on the tensor cores: dact = dy Wd, dx = (dgate | dup) (Wg ; Wu), dWd = dy^T act,
    (dWg ; dWu) = (dgate | dup)^T x.
    Returns ``(dx, d_gate_weight, d_up_weight, d_down_weight)`` in bf16.
    """
    _lib.require_cuda(dy, x, gate_weight, up_weight, down_weight)
    for v in (dy, x, gate_weight, up_weight, down_weight):
        assert v.dtype == torch.bfloat16
    dy, x = dy.contiguous(), x.contiguous()
    wg, wu, wd = gate_weight.contiguous(), up_weight.contiguous(), down_weight.contiguous()
    t, h = x.shape
    i = wg.size(0)
    dev = x.device
    bf = dict(device=dev, dtype=torch.bfloat16)
    status = _status(dev)
    if t == 0:
        z = torch.zeros
        return (torch.empty((0, h), **bf), z((i, h), **bf), z((i, h), **bf), z((h, i), **bf))
    lib = _lib.load()
    # gate | up pre-activations
    if gate_up is not None:
        assert gate_up.shape == (t, 2 * i) and gate_up.dtype == torch.bfloat16 and gate_up.is_contiguous()
        gu = gate_up
    else:
        gu = torch.empty((t, 2 * i), **bf)
        gemm_nt(x, wg, gu[:, :i], status)
        gemm_nt(x, wu, gu[:, i:], status)
    if _operands_in_place():
        # every GEMM reads its operands where they lie: a matrix whose contraction index is not the
        # contiguous one is fed to the tensor cores as an MN-major tile (omni_gemm_bf16)
        dact = gemm(dy, wd, False, True, status=status)                       # dy [T,H] @ Wd [H,I]
        dgu = torch.empty((t, 2 * i), **bf)
        act = torch.empty((t, i), **bf) if need_weight_grads else None
        with torch.cuda.device(dev):
            _lib.check(lib.omni_swiglu_bwd_limit(gu.data_ptr(), dact.data_ptr(), t, i, float(limit or 0.0), dgu.data_ptr(),
                                                 None, None, 0, _lib.ptr(act), _lib.stream_ptr()))
        # order: the product that reads act runs right after the kernel that wrote it, and the two that read
        # (dgate | dup) run back to back, so the second finds it in L2
        d_wg = d_wu = d_wd = None
        if need_weight_grads:
            d_wd = gemm(dy, act, True, True, status=status)                   # dy^T [H,T] @ act [T,I]
        # dx = dgate @ Wg + dup @ Wu = (dgate | dup) @ (Wg ; Wu)
        if i % 64 == 0:
            # the two weight matrices are read in place as one B operand stacked along K
            dx = torch.empty((t, h), **bf)
            with torch.cuda.device(dev):
                _lib.check(lib.omni_gemm_bf16_stacked_b(dgu.data_ptr(), 0, 2 * i, wg.data_ptr(), wu.data_ptr(), i, h, t, h, 2 * i,
                                                        dx.data_ptr(), h, status.data_ptr(), _lib.stream_ptr()))
        else:
            dx = gemm(dgu, torch.cat((wg, wu), 0), False, True, status=status)
        if need_weight_grads:
            d_wgu = gemm(dgu, x, True, True, status=status)                   # (dgate | dup)^T [2I,T] @ x [T,H]
            d_wg, d_wu = d_wgu[:i], d_wgu[i:]
        return dx, d_wg, d_wu, d_wd
    # dact = dy @ Wd   (Wd is [H, I]: its transpose has the contraction dimension contiguous)
    dact = gemm_nt(dy, transpose_padded(wd), None, status)
    dgu = torch.empty((t, 2 * i), **bf)
    tp = _pad8(t)
    dgu_t = torch.empty((2 * i, tp), **bf) if need_weight_grads else None
    act_t = torch.empty((i, tp), **bf) if need_weight_grads else None
    with torch.cuda.device(dev):
        _lib.check(lib.omni_swiglu_bwd_limit(gu.data_ptr(), dact.data_ptr(), t, i, float(limit or 0.0), dgu.data_ptr(),
                                             _lib.ptr(dgu_t), _lib.ptr(act_t), tp, None, _lib.stream_ptr()))
    # dx = dgate @ Wg + dup @ Wu = dgu @ (Wg ; Wu): B operand [H, 2I] = (Wg^T | Wu^T)
    wgu_t = torch.empty((h, 2 * i), **bf)
    transpose_padded(wg, wgu_t[:, :i])
    transpose_padded(wu, wgu_t[:, i:])
    dx = gemm_nt(dgu, wgu_t, None, status)
    d_wg = d_wu = d_wd = None
    if need_weight_grads:
        dy_t, x_t = transpose_padded(dy), transpose_padded(x)   # [H, pad8(T)]
        d_wd = gemm_nt(dy_t, act_t, None, status)              # [H, I]
        d_wgu = gemm_nt(dgu_t, x_t, None, status)              # [2I, H]
        d_wg, d_wu = d_wgu[:i], d_wgu[i:]
    return dx, d_wg, d_wu, d_wd


class MlpFunction(torch.autograd.Function):
    """Shared SwiGLU MLP with gradients for x and the three weight matrices."""

    @staticmethod
    def forward(ctx, x, gate_weight, up_weight, down_weight, limit=None):
        from .mlp import mlp_forward
        xb, wg, wu, wd = as_bf16(x), as_bf16(gate_weight), as_bf16(up_weight), as_bf16(down_weight)
        gu = torch.empty((xb.size(0), 2 * wg.size(0)), device=xb.device, dtype=torch.bfloat16)
        y = mlp_forward(xb, wg, wu, wd, gate_up=gu, limit=limit)
        ctx.save_for_backward(xb, wg, wu, wd, gu)
        ctx.limit = limit
        ctx.dtypes = (x.dtype, gate_weight.dtype, up_weight.dtype, down_weight.dtype)
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        xb, wg, wu, wd, gu = ctx.saved_tensors
        need_w = any(ctx.needs_input_grad[1:4])
        dx, d_wg, d_wu, d_wd = mlp_backward(as_bf16(dy), xb, wg, wu, wd, need_weight_grads=need_w, gate_up=gu,
                                            limit=ctx.limit)
        cast = lambda g, j: g.to(ctx.dtypes[j]) if (g is not None and ctx.needs_input_grad[j]) else None
        return cast(dx, 0), cast(d_wg, 1), cast(d_wu, 2), cast(d_wd, 3), None


# ------------------------------------------------------------------------------------------------
# router front: gate GEMMs -> BatchNorm -> log-softmax -> product-key top-k, as one differentiable op
# ------------------------------------------------------------------------------------------------
ROUTER_FRONT_MAX_SQRT_N = 256


class RouterFrontFunction(torch.autograd.Function):
    """``scores, indices = topk(log_softmax(BN(x Kx^T)) (+) log_softmax(BN(x Ky^T)))`` with the forward
    kernels of the fused inference path (tcgen05 gate GEMM with fp32 logits, fused BatchNorm fold /
    log-softmax / selection) and a backward that goes from ``dscores`` to ``dlogits`` in one call
    (``omni_router_norm_bwd``); the two small gate-weight products that remain are torch matmuls.

    ``fold`` is a callable ``logits -> (scale, shift)`` supplied by the module: the eval-mode fold of the
    running statistics, or the training-mode kernel that also updates them.
    """

    @staticmethod
    def forward(ctx, x, gate_x, gate_y, k, fold, training):
        xb, kx, ky = as_bf16(x), as_bf16(gate_x), as_bf16(gate_y)
        t, h = xb.shape
        n = kx.size(0)
        dev = xb.device
        lib = _lib.load()
        status = _status(dev)
        f32 = dict(device=dev, dtype=torch.float32)
        logits = torch.empty((t, 2 * n), **f32)
        lp = torch.empty((t, 2 * n), **f32)
        scores = torch.empty((t, k), **f32)
        indices = torch.empty((t, k), device=dev, dtype=torch.int32)
        with torch.cuda.device(dev):
            st = _lib.stream_ptr()
            if t > 0:
                _lib.check(lib.omni_router_gate(xb.data_ptr(), kx.data_ptr(), ky.data_ptr(), t, h, n, logits.data_ptr(),
                                                status.data_ptr(), st))
            scale, shift = fold(logits)
            if t > 0 and k > 0:
                _lib.check(lib.omni_router_logits_topk(logits.data_ptr(), 2 * n, scale.data_ptr(), shift.data_ptr(), t, n, k,
                                                       scores.data_ptr(), indices.data_ptr(), 0, None, lp.data_ptr(), st))
        ctx.save_for_backward(xb, kx, ky, logits, lp, scale.clone(), shift.clone(), indices)
        ctx.training = bool(training)
        ctx.dtypes = (x.dtype, gate_x.dtype, gate_y.dtype)
        ctx.mark_non_differentiable(indices)
        return scores, indices

    @staticmethod
    def backward(ctx, dscores, _dindices):
        xb, kx, ky, logits, lp, scale, shift, indices = ctx.saved_tensors
        t, k = indices.shape
        n = kx.size(0)
        dev = xb.device
        lib = _lib.load()
        status = _status(dev)
        dz = torch.empty((t, 2 * n), device=dev, dtype=torch.bfloat16)
        ds = dscores.detach().float().contiguous()
        scratch = None
        if ctx.training:
            scratch = torch.empty(int(lib.omni_router_norm_bwd_scratch_bytes(t, n)), device=dev, dtype=torch.uint8)
        if t > 0:
            with torch.cuda.device(dev):
                _lib.check(lib.omni_router_norm_bwd(ds.data_ptr(), indices.data_ptr(), lp.data_ptr(), logits.data_ptr(), 2 * n,
                                                    scale.data_ptr(), shift.data_ptr(), t, n, k, int(ctx.training), dz.data_ptr(),
                                                    _lib.ptr(scratch), scratch.numel() if scratch is not None else 0,
                                                    status.data_ptr(), _lib.stream_ptr()))
        dx = dkx = dky = None
        if ctx.needs_input_grad[0]:
            dx = (dz @ torch.cat([kx, ky], dim=0)).to(ctx.dtypes[0])
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            dk = dz.t() @ xb
            dkx, dky = dk[:n].to(ctx.dtypes[1]), dk[n:].to(ctx.dtypes[2])
        return dx, dkx, dky, None, None, None
