"""``OmniMoE`` layer backed by the sm_100a kernels.

Constructor, parameter / buffer names and shapes, and ``forward(hidden_states)`` follow the
reference module (omni_moe/modules/omni_moe.py:14-106), so a reference ``state_dict`` loads
unchanged.  Under ``torch.no_grad()`` (or with nothing requiring gradients) the forward is the fused
launch sequence below; when gradients are needed it is composed from the three differentiable
operators, like the reference's own forward.

One eval forward is four kernels (five when the router shape exceeds the fused kernel's limits, eight to ten when the expert tables are too large for L2 and the
pairs are scheduled by expert first), enqueued without a host synchronisation:

    main stream   gate/up GEMM + SwiGLU -> down GEMM ........................ -> routed experts (+= y)
    side stream                            router gate GEMM                        (selection happens inside the expert kernel)

The gate/up GEMM and the expert kernel fill the GPU on their own.  The down projection of the
quick-start shape occupies 128 of the 148 SMs, so the two small router kernels run beside it.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import _lib
from ..ops.expert import hot_workspace, use_fused_path, use_hot_experts, use_routed_kernel
from ..ops.scheduler import workspace_bytes


class OmniMoEConfig:
    """Same five fields as the reference configuration (omni_moe/modules/omni_moe.py:14-27)."""

    def __init__(self, hidden_size: int, intermediate_size: int, hidden_act: str, num_experts: int,
                 num_experts_per_token: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.hidden_act = hidden_act
        self.num_experts = num_experts
        self.num_experts_per_token = num_experts_per_token


class _Buffers:
    """Per-(token count, device) scratch of a forward; allocated once and reused."""

    def __init__(self, t, h, i, n_sqrt, n, k, dev):
        f32 = dict(device=dev, dtype=torch.float32)
        i32 = dict(device=dev, dtype=torch.int32)
        p = t * k
        self.logits = torch.empty((t, 2 * n_sqrt), **f32)
        self.scores = torch.empty((t, k), **f32)
        self.weights = torch.empty((t, k), **f32)
        self.indices = torch.empty((t, k), **i32)
        self.perm = torch.empty(max(p, 1), **i32)
        self.sorted_experts = torch.empty(max(p, 1), **i32)
        self.meta = torch.zeros(4, **i32)
        self.coef = torch.empty((t, k), **f32)
        self.act = torch.empty((t, i), device=dev, dtype=torch.bfloat16)
        self.workspace = torch.empty(workspace_bytes(p, n), device=dev, dtype=torch.uint8)
        # dense products of the hot experts (large-table path only)
        self.hot = hot_workspace(t, h, dev) if (use_hot_experts(t) and not use_fused_path(n, h)) else None
        self.status = torch.zeros(1, **i32)
        self.bn_scale = torch.empty(2 * n_sqrt, **f32)      # training-mode BatchNorm fold of this forward
        self.bn_shift = torch.empty(2 * n_sqrt, **f32)
        self.bn_scratch = torch.empty(max(int(_lib.load().omni_router_bn_train_scratch_bytes(max(t, 1), n_sqrt)), 16),
                                      device=dev, dtype=torch.uint8)
        self.side = torch.cuda.Stream(device=dev)
        self.ev_fork = torch.cuda.Event()
        self.ev_join = torch.cuda.Event()


class OmniMoE(nn.Module):
    def __init__(self, config: OmniMoEConfig):
        super().__init__()
        if config.hidden_act not in ("silu", "swish"):
            # the reference's kernels hard-code SiLU whatever hidden_act says; other names are refused here
            raise ValueError(f"hidden_act={config.hidden_act!r} is not supported: the fused kernels implement SiLU")
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.intermediate_size
        self.num_experts = config.num_experts
        self.num_expert_sqrt = math.floor(math.sqrt(self.num_experts))
        self.top_k = config.num_experts_per_token

        # shared expert
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False)
        # router gates and their (non-affine) normalisation
        self.router_gate_x = nn.Linear(self.hidden_size, self.num_expert_sqrt, bias=False)
        self.router_gate_y = nn.Linear(self.hidden_size, self.num_expert_sqrt, bias=False)
        self.router_norm_x = nn.BatchNorm1d(self.num_expert_sqrt, affine=False)
        self.router_norm_y = nn.BatchNorm1d(self.num_expert_sqrt, affine=False)
        # routed experts: one up row and one down row per expert
        self.up_embed = nn.Embedding(self.num_experts, self.hidden_size)
        self.down_embed = nn.Embedding(self.num_experts, self.hidden_size)

        self._buffers_cache: dict = {}
        self._bn_cache = None
        self.last_routing = None  # (scores, indices, weights) of the latest forward, for inspection

    # ------------------------------------------------------------------------------------------
    def _bf16_weight(self, p: torch.Tensor) -> torch.Tensor:
        w = p.detach()
        if w.dtype != torch.bfloat16:
            w = w.to(torch.bfloat16)  # fp32 / fp16 modules: operands are rounded to bf16 per call
        return w.contiguous()

    def _bn_fold_eval(self):
        """Eval-mode BatchNorm of both axes as one scale / shift pair per logit column."""
        bx, by = self.router_norm_x, self.router_norm_y
        key = (bx.running_mean._version, bx.running_var._version, by.running_mean._version, by.running_var._version,
               bx.running_mean.data_ptr(), by.running_mean.data_ptr())
        if self._bn_cache is None or self._bn_cache[0] != key:
            mean = torch.cat([bx.running_mean, by.running_mean]).float()
            var = torch.cat([bx.running_var, by.running_var]).float()
            eps = torch.cat([torch.full_like(bx.running_var, bx.eps, dtype=torch.float32),
                             torch.full_like(by.running_var, by.eps, dtype=torch.float32)])
            scale = torch.rsqrt(var + eps)
            self._bn_cache = (key, scale.contiguous(), (-mean * scale).contiguous())
        return self._bn_cache[1], self._bn_cache[2]

    def sync_batch_statistics(self, group=None, enabled: bool = True) -> "OmniMoE":
        """Training-mode BatchNorm over the tokens of every rank of ``group`` (default: all ranks), for
        data-parallel training where a batch is sharded over GPUs.  Covers the fused (no-grad) forward;
        for the differentiable forward convert the two norm layers with
        ``torch.nn.SyncBatchNorm.convert_sync_batchnorm`` - the fused forward then follows their group."""
        self._bn_sync = (group,) if enabled else None
        return self

    def _bn_group(self):
        """None = local statistics; otherwise a 1-tuple holding the process group (None inside = world)."""
        if getattr(self, "_bn_sync", None) is not None:
            return self._bn_sync
        if isinstance(self.router_norm_x, nn.SyncBatchNorm):
            return (self.router_norm_x.process_group,)
        return None

    def _bn_fold_train(self, logits: torch.Tensor, b: "_Buffers | None" = None):
        """Training-mode BatchNorm: batch statistics over all tokens (of all ranks, when synchronised),
        running statistics updated as nn.BatchNorm1d does (momentum average, unbiased variance).
        On one rank this is the library's kernel pair (no allocation, no host read: capturable); with
        synchronised statistics the per-rank moments are merged through torch.distributed."""
        n = self.num_expert_sqrt
        grp = self._bn_group()
        bx, by = self.router_norm_x, self.router_norm_y
        run_dt = bx.running_mean.dtype if bx.running_mean is not None else torch.float32
        same_layout = (bx.running_mean is None) == (by.running_mean is None) and bx.track_running_stats == by.track_running_stats
        if (grp is None and b is not None and logits.dtype == torch.float32 and logits.is_contiguous() and same_layout
                and run_dt in (torch.float32, torch.bfloat16)):
            track = bx.track_running_stats and bx.running_mean is not None
            mom = lambda bn: -1.0 if bn.momentum is None else float(bn.momentum)
            ptr = lambda t_: t_.data_ptr() if (track and t_ is not None) else None
            _lib.check(_lib.load().omni_router_bn_train(
                logits.data_ptr(), logits.size(1), logits.size(0), n, float(bx.eps), float(by.eps), mom(bx), mom(by),
                ptr(bx.running_mean), ptr(bx.running_var), ptr(by.running_mean), ptr(by.running_var), _lib.dtype_code(run_dt),
                ptr(bx.num_batches_tracked), ptr(by.num_batches_tracked), b.bn_scale.data_ptr(), b.bn_shift.data_ptr(),
                b.bn_scratch.data_ptr(), b.bn_scratch.numel(), _lib.stream_ptr()))
            self._bn_cache = None  # the running statistics changed behind torch's version counters
            return b.bn_scale, b.bn_shift
        if grp is None:
            t = logits.size(0)
            var, mean = torch.var_mean(logits, dim=0, unbiased=False)
        else:
            from ..parallel import synced_batch_statistics
            mean, var, t = synced_batch_statistics(logits, grp[0])
        with torch.no_grad():
            for bn, sl in ((bx, slice(0, n)), (by, slice(n, 2 * n))):
                if bn.track_running_stats and bn.running_mean is not None:
                    bn.num_batches_tracked += 1
                    mom = bn.momentum if bn.momentum is not None else 1.0 / float(bn.num_batches_tracked)
                    unbiased = var[sl] * (t / max(t - 1, 1))
                    bn.running_mean.mul_(1 - mom).add_(mean[sl].to(bn.running_mean.dtype), alpha=mom)
                    bn.running_var.mul_(1 - mom).add_(unbiased.to(bn.running_var.dtype), alpha=mom)
        eps = torch.cat([torch.full((n,), bx.eps), torch.full((n,), by.eps)]).to(var)
        scale = torch.rsqrt(var + eps)
        if b is not None:
            # into the forward's own buffers: they outlive the side stream this runs on, a temporary would belong to
            # that stream's allocator pool while the main stream still reads it
            b.bn_scale.copy_(scale)
            b.bn_shift.copy_(-mean * scale)
            return b.bn_scale, b.bn_shift
        return scale.contiguous(), (-mean * scale).contiguous()

    def _get_buffers(self, t: int, dev: torch.device) -> _Buffers:
        """Scratch of an eager forward, one set per (token count, device, stream): forwards of one module issued
        on different streams may overlap on the GPU, so they must not share logits / activation / status buffers
        (two forwards on the same stream are ordered by the stream).  The few most recent sets are kept."""
        key = (t, dev.index, torch.cuda.current_stream(dev).cuda_stream)
        b = self._buffers_cache.get(key)
        if b is None:
            b = _Buffers(t, self.hidden_size, self.intermediate_size, self.num_expert_sqrt, self.num_experts,
                         self.top_k, dev)
            while len(self._buffers_cache) >= 4:  # shapes and streams rarely alternate: keep a handful
                self._buffers_cache.pop(next(iter(self._buffers_cache)))
            self._buffers_cache[key] = b
        return b

    # ------------------------------------------------------------------------------------------
    def _operands(self):
        """bf16 views (or per-call bf16 copies, for fp32 / fp16 modules) of all weights."""
        if getattr(self, "_tables_partitioned", False):
            raise RuntimeError("this module's expert tables were handed to a PartitionedOmniMoE: call that wrapper, "
                               "the module alone no longer holds the rows its router selects")
        return tuple(self._bf16_weight(p.weight) for p in (
            self.gate_proj, self.up_proj, self.down_proj, self.router_gate_x, self.router_gate_y,
            self.up_embed, self.down_embed))

    def _launch(self, x: torch.Tensor, y: torch.Tensor, b: _Buffers, record_streams: bool = False) -> None:
        """Enqueue one forward on the current stream: ``x [T, H]`` bf16 contiguous -> ``y [T, H]`` bf16.
        Allocates nothing in eval mode, so it can be captured in a CUDA graph."""
        t, h, i, n, k = x.size(0), self.hidden_size, self.intermediate_size, self.num_expert_sqrt, self.top_k
        wg, wu, wd, kx, ky, up_t, down_t = self._operands()
        lib = _lib.load()
        chk = _lib.check
        main = torch.cuda.current_stream()
        st = main.cuda_stream
        status = b.status.data_ptr()
        # 1. gate/up projections + SwiGLU: fills every SM
        chk(lib.omni_mlp_gate_up(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), t, h, i, b.act.data_ptr(), status, st))
        b.ev_fork.record(main)
        # 2. side stream: router gate GEMM.  It runs on the SMs the down projection leaves free.
        routed = use_routed_kernel(self.num_experts, h, n, k)
        with torch.cuda.stream(b.side):
            b.side.wait_event(b.ev_fork)
            ss = b.side.cuda_stream
            chk(lib.omni_router_gate(x.data_ptr(), kx.data_ptr(), ky.data_ptr(), t, h, n, b.logits.data_ptr(), status, ss))
            scale, shift = self._bn_fold_train(b.logits, b) if self.training else self._bn_fold_eval()
            if not routed:
                chk(lib.omni_router_logits_topk(b.logits.data_ptr(), 2 * n, scale.data_ptr(), shift.data_ptr(), t, n, k,
                                                b.scores.data_ptr(), b.indices.data_ptr(), 0, b.weights.data_ptr(),
                                                None, ss))
            b.ev_join.record(b.side)
            if record_streams:
                for tns in (x, kx, ky, scale, shift):
                    tns.record_stream(b.side)
        # 3. main stream, meanwhile: down projection -> y
        chk(lib.omni_mlp_down(b.act.data_ptr(), wd.data_ptr(), t, h, i, None, y.data_ptr(), status, st))
        main.wait_event(b.ev_join)
        # 4. routed experts, added onto y in place
        if routed:
            # tables resident in L2: BatchNorm / log-softmax / top-k and the row gathers in one
            # token-centric kernel
            chk(lib.omni_route_expert_fused(b.logits.data_ptr(), 2 * n, scale.data_ptr(), shift.data_ptr(), x.data_ptr(),
                                            up_t.data_ptr(), down_t.data_ptr(), t, n, k, h, self.num_experts,
                                            y.data_ptr(), y.data_ptr(), b.scores.data_ptr(), b.indices.data_ptr(),
                                            b.weights.data_ptr(), status, st))
        elif use_fused_path(self.num_experts, h):
            chk(lib.omni_expert_fused(x.data_ptr(), up_t.data_ptr(), down_t.data_ptr(), b.weights.data_ptr(),
                                      b.indices.data_ptr(), t, k, h, self.num_experts, y.data_ptr(), y.data_ptr(),
                                      _lib.OMNI_BF16, None, status, st))
        else:
            # large tables: expert-centric schedule, each Up row leaves HBM once
            chk(lib.omni_schedule(b.indices.data_ptr(), 0, None, 0, t, k, self.num_experts, b.perm.data_ptr(),
                                  b.sorted_experts.data_ptr(), None, None, None, None, b.meta.data_ptr(),
                                  b.workspace.data_ptr(), b.workspace.numel(), st))
            if b.hot is not None:
                chk(lib.omni_expert_coef_hot(x.data_ptr(), up_t.data_ptr(), b.weights.data_ptr(), b.perm.data_ptr(),
                                             b.sorted_experts.data_ptr(), t, k, h, self.num_experts, 0,
                                             b.coef.data_ptr(), b.hot.data_ptr(), b.hot.numel(), status, st))
            else:
                chk(lib.omni_expert_coef(x.data_ptr(), up_t.data_ptr(), b.weights.data_ptr(), b.perm.data_ptr(),
                                         b.sorted_experts.data_ptr(), t, k, h, self.num_experts, b.coef.data_ptr(),
                                         status, st))
            chk(lib.omni_expert_combine(down_t.data_ptr(), b.coef.data_ptr(), b.indices.data_ptr(), t, k, h,
                                        self.num_experts, y.data_ptr(), y.data_ptr(), _lib.OMNI_BF16, status, st))
        self.last_routing = (b.scores, b.indices, b.weights)
        self.last_status = b.status

    @staticmethod
    def kernels_per_forward(num_experts: int, hidden: int, sqrt_n: int = 0, k: int = 0, num_tokens: int = 0) -> int:
        """Kernels of this library launched by one eval forward."""
        if sqrt_n and use_routed_kernel(num_experts, hidden, sqrt_n, k):
            return 4  # gate/up, router gates, down projection, router selection + experts
        if use_fused_path(num_experts, hidden):
            return 5  # gate/up, router gates, top-k, down projection, fused experts
        bits = max(1, (num_experts - 1).bit_length())
        passes = -(-bits // 11)
        # gate/up, router gates, top-k, down projection, 2 per radix pass, coefficients, combine;
        # from 4096 tokens also the hot-expert search and its dense GEMM
        return 4 + 2 * passes + 2 + (2 if use_hot_experts(num_tokens) else 0)

    def _needs_grad(self, hidden_states: torch.Tensor) -> bool:
        """The differentiable composition is used when gradients can be asked for: the input carries a
        graph, or the module is in training mode with trainable parameters.  An eval-mode module called
        on a plain tensor takes the fused inference path even outside ``torch.no_grad()``."""
        if not torch.is_grad_enabled():
            return False
        return hidden_states.requires_grad or (self.training and any(p.requires_grad for p in self.parameters()))

    def _fused_router_front_ok(self) -> bool:
        """The one-op router front (ops.autograd.RouterFrontFunction) covers plain BatchNorm1d layers with
        local statistics, sqrt(N) <= 256 and an even top-k in the reference's range."""
        from ..ops.autograd import ROUTER_FRONT_MAX_SQRT_N
        bx, by = self.router_norm_x, self.router_norm_y
        plain = type(bx) is nn.BatchNorm1d and type(by) is nn.BatchNorm1d and bx.track_running_stats and by.track_running_stats
        return (plain and self._bn_group() is None and self.num_expert_sqrt <= ROUTER_FRONT_MAX_SQRT_N
                and 0 < self.top_k <= 128 and self.hidden_size % 8 == 0)

    def _forward_autograd(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """Differentiable forward, composed like the reference module (omni_moe/modules/omni_moe.py:60-106) from
        operators that run the kernels of this library and carry their own backward.  The router front
        (gates, BatchNorm, log-softmax, selection) is one such operator where its limits allow, otherwise
        torch modules / functions followed by the router op, as in the reference."""
        from ..ops import omni_expert_func, omni_mlp_func, omni_router_func
        bsz, seq_len, _ = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_size)
        if self._fused_router_front_ok():
            # gate GEMMs (fp32 logits), BatchNorm fold, log-softmax and selection by the kernels of the fused
            # path; the backward goes from dscores to dlogits in one call
            import types
            from ..ops.autograd import RouterFrontFunction
            n = self.num_expert_sqrt
            if self.training:
                def fold(logits):
                    dev = logits.device
                    tmp = types.SimpleNamespace(
                        bn_scale=torch.empty(2 * n, device=dev, dtype=torch.float32),
                        bn_shift=torch.empty(2 * n, device=dev, dtype=torch.float32),
                        bn_scratch=torch.empty(max(int(_lib.load().omni_router_bn_train_scratch_bytes(max(logits.size(0), 1), n)), 16),
                                               device=dev, dtype=torch.uint8))
                    return self._bn_fold_train(logits, tmp)
            else:
                fold = lambda logits: self._bn_fold_eval()
            scores, indices = RouterFrontFunction.apply(x, self.router_gate_x.weight, self.router_gate_y.weight, self.top_k,
                                                        fold, self.training)
        else:
            logits_x = self.router_norm_x(self.router_gate_x(x))
            logits_y = self.router_norm_y(self.router_gate_y(x))
            # log-probabilities, scores and routing weights stay in fp32 (the reference keeps the module dtype):
            # bf16 log-probs tie massively, and ties are what makes a selection irreproducible
            log_probs_x = torch.nn.functional.log_softmax(logits_x, dim=-1, dtype=torch.float32)
            log_probs_y = torch.nn.functional.log_softmax(logits_y, dim=-1, dtype=torch.float32)
            scores, indices = omni_router_func(log_probs_x, log_probs_y, self.num_expert_sqrt, self.top_k)
        routing_weights = torch.exp(scores)
        experts_states = omni_expert_func(x, self.up_embed.weight, self.down_embed.weight, routing_weights, indices)
        shared = omni_mlp_func(x, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight)
        self.last_routing = (scores.detach(), indices, routing_weights.detach())
        return (shared + experts_states).view(bsz, seq_len, -1)

    def forward(self, hidden_states: torch.Tensor, **kwargs) -> torch.Tensor:
        _lib.require_cuda(hidden_states)
        if getattr(self, "_tables_partitioned", False):
            self._operands()  # raises: the tables live in the PartitionedOmniMoE wrapper
        if self._needs_grad(hidden_states) or self.hidden_size % 8 or self.intermediate_size % 8:
            # sizes that are not multiples of 8 go through the operators one by one (they pad): the fused
            # launch sequence moves rows in 16-byte pieces
            return self._forward_autograd(hidden_states)
        bsz, seq_len, _ = hidden_states.shape
        in_dtype = hidden_states.dtype
        x = hidden_states.detach().reshape(-1, self.hidden_size)
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        x = x.contiguous()
        t, h = x.size(0), self.hidden_size
        dev = x.device
        y = torch.empty((t, h), device=dev, dtype=torch.bfloat16)
        if t == 0:
            return y.view(bsz, seq_len, h).to(in_dtype)
        with torch.cuda.device(dev):
            self._launch(x, y, self._get_buffers(t, dev), record_streams=True)
        out = y.view(bsz, seq_len, h)
        return out if in_dtype == torch.bfloat16 else out.to(in_dtype)

    def graphed(self, num_tokens: int, device=None) -> "GraphedOmniMoE":
        """Capture one eval-mode forward for ``num_tokens`` tokens in a CUDA graph."""
        return GraphedOmniMoE(self, num_tokens, device)

    def check_status(self) -> None:
        """Synchronise and raise if any kernel of the latest forward reported a device-side fault."""
        st = getattr(self, "last_status", None)
        if st is not None:
            _lib.check_status(st)
        _lib.check_device_status()   # the operators of the differentiable forward / backward report here


class GraphedOmniMoE:
    """One captured forward with static input / output buffers: ``x`` (bf16 ``[T, H]``) is the input
    to fill, ``y`` the output of the latest ``replay()``.  The ~12 kernel launches and the two-stream
    fork/join become one graph launch."""

    def __init__(self, module: OmniMoE, num_tokens: int, device=None):
        if module.training and module._bn_group() is not None:
            raise RuntimeError("graph capture of a training-mode forward needs local batch statistics "
                               "(synchronised statistics go through torch.distributed on the host)")
        dev = torch.device(device) if device is not None else module.gate_proj.weight.device
        if module.gate_proj.weight.dtype != torch.bfloat16:
            raise RuntimeError("graph capture needs a bf16 module (module.to(torch.bfloat16)): "
                               "other dtypes are converted per call, which a graph would freeze")
        if module.hidden_size % 8 or module.intermediate_size % 8:
            raise RuntimeError("graph capture needs hidden and intermediate sizes that are a multiple of 8 "
                               "(other sizes run operator by operator with padded copies)")
        self.module = module
        self.x = torch.zeros((num_tokens, module.hidden_size), device=dev, dtype=torch.bfloat16)
        self.y = torch.zeros((num_tokens, module.hidden_size), device=dev, dtype=torch.bfloat16)
        self.buffers = _Buffers(num_tokens, module.hidden_size, module.intermediate_size, module.num_expert_sqrt,
                                module.num_experts, module.top_k, dev)
        with torch.cuda.device(dev):
            if not module.training:
                module._bn_fold_eval()
            # the warm-up launch of a training-mode module would count as a batch: keep the statistics as they were
            stats = [(buf, buf.clone()) for bn in (module.router_norm_x, module.router_norm_y)
                     for buf in (bn.running_mean, bn.running_var, bn.num_batches_tracked) if module.training and buf is not None]
            warm = torch.cuda.Stream()
            warm.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(warm):
                module._launch(self.x, self.y, self.buffers)
            torch.cuda.current_stream().wait_stream(warm)
            torch.cuda.synchronize()
            for buf, saved in stats:
                buf.copy_(saved)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                module._launch(self.x, self.y, self.buffers)

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.y

    def __call__(self, hidden_states: torch.Tensor) -> torch.Tensor:
        self.x.copy_(hidden_states.reshape(self.x.shape), non_blocking=True)
        self.graph.replay()
        return self.y.view(hidden_states.shape)
