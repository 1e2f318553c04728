"""Multi-GPU forms of the layer forward (one process per GPU, torch.distributed).

The reference project has no distributed code; this module is the multi-GPU design of this
implementation for the two regimes its benchmark configurations fall into:

* **Replicas, tokens sharded** (tables that fit one GPU): every rank holds all weights and runs
  ``OmniMoE.forward`` on its own tokens.  Eval-mode forward needs no collective at all, so there is
  nothing to do here beyond giving each rank its slice (:func:`shard_tokens`).

* **Expert tables row-partitioned** (the largest configuration: 2 x 8 GiB tables): rank ``g`` holds
  rows ``[g * rows_per_rank, (g + 1) * rows_per_rank)`` of ``up_embed`` / ``down_embed``; router and
  shared MLP stay replicated and token-parallel.  Per forward:

    1. route the local tokens (router GEMM + selection)                         local
    2. dispatch: every (token, expert, weight) pair goes to the rank that owns the expert row
       (``all_to_all_single`` of 12-byte records after a count exchange); the token rows themselves
       are all-gathered, because with k experts per token spread over the table nearly every rank
       needs nearly every token and one row per (token, rank) is far less than one per pair
    3. each rank computes, for all tokens, the partial sum over the pairs it received
       (``omni_schedule`` on the local expert ids -> ``omni_expert_coef_pairs`` ->
       ``omni_expert_combine_segments``)                                        local
    4. combine: ``reduce_scatter`` of the partial ``[T_total, H]`` sums back to the token owners
    5. shared MLP with the reduced expert states added in the down-projection epilogue   local

  Pairs are sent grouped by destination and, inside a destination, in ascending pair order, so what a
  rank receives is already ordered by global token id: the token segments for step 3 come from one
  ``searchsorted``.  Remote data always lands in local memory through NCCL before a kernel of this
  library reads it.

The exchange plumbing works on CPU tensors with the gloo backend as well (that is how it is tested
without GPUs); the expert arithmetic of step 3 is injected, and on CUDA it is always the kernels of
this library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist

from . import _lib


def synced_batch_statistics(z: torch.Tensor, group=None):
    """Mean and biased variance of every column of ``z [T_local, C]`` over the tokens of ALL ranks of
    ``group``, plus the global token count: what training-mode BatchNorm of the router logits needs
    when the tokens of a batch are sharded over GPUs (the reference normalises over the whole batch
    on one GPU, omni_moe/modules/omni_moe.py:53-54,70-71).

    Each rank sends ``2C + 1`` floats (its column means, its sums of squared deviations, its count);
    the per-rank moments are merged with the pairwise formula for combining variances, so nothing is
    lost to cancellation as it would be in a global sum of squares.  Without an initialised process
    group (or with a group of one) these are the local statistics.
    """
    t = z.size(0)
    zf = z.float()
    var_l, mean_l = torch.var_mean(zf, dim=0, unbiased=False) if t > 0 else (torch.zeros_like(zf[0:0].sum(0)),) * 2
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return mean_l, var_l, t
    c = z.size(1)
    packed = torch.cat([mean_l, var_l * t, torch.tensor([float(t)], device=z.device)])
    world = dist.get_world_size(group)
    gathered = torch.empty(world * (2 * c + 1), device=z.device, dtype=torch.float32)
    dist.all_gather_into_tensor(gathered, packed.contiguous(), group=group)
    gathered = gathered.view(world, 2 * c + 1)
    means, m2s, counts = gathered[:, :c], gathered[:, c:2 * c], gathered[:, 2 * c:]
    total = counts.sum()
    mean = (means * counts).sum(0) / total
    m2 = m2s.sum(0) + (counts * (means - mean) ** 2).sum(0)
    return mean, m2 / total, int(total.item())


def shard_tokens(hidden_states: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Contiguous token shard of ``[T, H]`` (or ``[B, S, H]`` flattened) for ``rank``; T must divide evenly."""
    x = hidden_states.reshape(-1, hidden_states.shape[-1])
    assert x.size(0) % world == 0, "the token count must be a multiple of the world size"
    per = x.size(0) // world
    return x[rank * per:(rank + 1) * per]


@dataclass(frozen=True)
class ExpertPartition:
    """Contiguous row partition of an expert table with ``num_experts`` rows over ``world`` ranks."""
    num_experts: int
    world: int
    rank: int

    @property
    def rows_per_rank(self) -> int:
        return -(-self.num_experts // self.world)

    @property
    def lo(self) -> int:
        return min(self.num_experts, self.rank * self.rows_per_rank)

    @property
    def hi(self) -> int:
        return min(self.num_experts, (self.rank + 1) * self.rows_per_rank)

    def owner(self, expert_ids: torch.Tensor) -> torch.Tensor:
        return torch.div(expert_ids, self.rows_per_rank, rounding_mode="floor")

    def slice_rows(self, table: torch.Tensor) -> torch.Tensor:
        """This rank's rows of a full ``[N, H]`` table (a contiguous copy)."""
        return table[self.lo:self.hi].contiguous()


@dataclass
class ReceivedPairs:
    """What a rank holds after the dispatch: all tokens' rows and the pairs routed to its table slice."""
    x_all: torch.Tensor           # [T_total, H]
    pair_tokens: torch.Tensor     # int32 [P_recv] global token id, non-decreasing
    pair_experts: torch.Tensor    # int32 [P_recv] expert row inside this rank's slice
    pair_weights: torch.Tensor    # float32 [P_recv]
    token_offsets: torch.Tensor   # int32 [T_total + 1] CSR of the pair list by token
    send_counts: list
    recv_counts: list


class ExchangeError(RuntimeError):
    """A step of the inter-rank exchange failed: a peer left or never joined (the backend's timeout or
    abort surfaces here), or the ranks disagree about the shape of the exchange.  ``stage`` names the
    step.  Raised on the host before any kernel of this library reads a buffer the failed collective
    should have filled."""

    def __init__(self, stage: str, detail: str):
        super().__init__(f"expert exchange failed at '{stage}': {detail}")
        self.stage = stage


def _collective(stage: str, fn, *args, **kwargs):
    """Runs one torch.distributed call and turns a backend failure into :class:`ExchangeError`."""
    try:
        return fn(*args, **kwargs)
    except ExchangeError:
        raise
    except RuntimeError as e:  # DistBackendError, gloo / NCCL timeouts and aborts derive from RuntimeError
        raise ExchangeError(stage, str(e).splitlines()[0] if str(e) else type(e).__name__) from e


def _stable_order_by_owner(owner: torch.Tensor, world: int) -> torch.Tensor:
    """Permutation that groups the flat pairs by owning rank, ascending pair id inside a group."""
    if owner.is_cuda:
        from .ops.scheduler import schedule
        raw = schedule(owner.view(-1, 1), world)  # the radix scheduler, one pass over `world` bins
        return raw.sorted_pair_ids.long()
    return torch.sort(owner.view(-1).long(), stable=True).indices


def dispatch_pairs(x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, part: ExpertPartition,
                   group=None) -> ReceivedPairs:
    """Step 2: send every routed pair of this rank's tokens to the rank that owns the expert row.

    ``x [T_local, H]``, ``indices [T_local, k]`` global expert ids, ``weights [T_local, k]`` float32.
    Every rank must pass the same ``T_local``.
    """
    world, rank = part.world, part.rank
    t_local, k = indices.shape
    dev = x.device
    flat_e = indices.reshape(-1).to(torch.int32)
    owner = part.owner(flat_e).to(torch.int32)
    order = _stable_order_by_owner(owner, world)
    send_counts = torch.bincount(owner.long(), minlength=world)
    # the count exchange doubles as a handshake: every rank also states its shard shape, so a peer that
    # left, or one configured with another token count or k, is noticed here, on the host, before any
    # payload moves
    hello = torch.stack([send_counts, torch.full_like(send_counts, t_local), torch.full_like(send_counts, k)], dim=1).contiguous()
    got = torch.empty_like(hello)
    _collective("count exchange", dist.all_to_all_single, got, hello, group=group)
    got_host = got.tolist()  # one host sync: the split sizes
    send_list, recv_list = send_counts.tolist(), [r[0] for r in got_host]
    for peer, (cnt, t_peer, k_peer) in enumerate(got_host):
        if t_peer != t_local or k_peer != k:
            raise ExchangeError("count exchange", f"rank {peer} shards {t_peer} tokens x {k_peer} experts, this rank "
                                                  f"{t_local} x {k}: every rank must pass the same shard shape")
        if cnt < 0 or cnt > t_peer * k_peer:
            raise ExchangeError("count exchange", f"rank {peer} announces {cnt} pairs, more than its {t_peer * k_peer}")
    # 12-byte records: global token id, expert row inside the owner's slice, weight bits
    tok = (torch.div(order, k, rounding_mode="floor") + rank * t_local).to(torch.int32)
    e_sorted = flat_e[order]
    local_e = e_sorted - owner[order] * part.rows_per_rank
    w_bits = weights.reshape(-1).float()[order].view(torch.int32)
    send = torch.stack([tok, local_e, w_bits], dim=1).contiguous()
    recv = torch.empty((sum(recv_list), 3), device=dev, dtype=torch.int32)
    _collective("pair dispatch", dist.all_to_all_single, recv, send, output_split_sizes=recv_list,
                input_split_sizes=send_list, group=group)
    x_all = torch.empty((world * t_local, x.size(1)), device=dev, dtype=x.dtype)
    _collective("token all-gather", dist.all_gather_into_tensor, x_all, x.contiguous(), group=group)
    pair_tokens = recv[:, 0].contiguous()
    bounds = torch.arange(world * t_local + 1, device=dev, dtype=torch.int32)
    token_offsets = torch.searchsorted(pair_tokens, bounds, right=False).to(torch.int32)
    return ReceivedPairs(x_all, pair_tokens, recv[:, 1].contiguous(), recv[:, 2].contiguous().view(torch.float32),
                         token_offsets, send_list, recv_list)


def local_partial_states(recv: ReceivedPairs, up_local: torch.Tensor, down_local: torch.Tensor,
                         out_dtype: torch.dtype = torch.float32, status: torch.Tensor | None = None) -> torch.Tensor:
    """Step 3 on the GPU: ``partial[t] = sum over received pairs of token t of w * silu(x[t] . Up[e]) * Down[e]``
    for all ``T_total`` tokens, over this rank's table slice.  CUDA only."""
    from .ops.scheduler import schedule
    _lib.require_cuda(recv.x_all, up_local, down_local)
    assert recv.x_all.dtype == up_local.dtype == down_local.dtype == torch.bfloat16
    x_all = recv.x_all.contiguous()
    t_total, h = x_all.shape
    n_local = up_local.size(0)
    p = recv.pair_tokens.numel()
    dev = x_all.device
    if status is None:
        status = torch.zeros(1, device=dev, dtype=torch.int32)
    partial = torch.empty((t_total, h), device=dev, dtype=out_dtype)
    coef = torch.empty(max(p, 1), device=dev, dtype=torch.float32)
    lib = _lib.load()
    with torch.cuda.device(dev):
        st = _lib.stream_ptr()
        if p:
            sch = schedule(recv.pair_experts.view(-1, 1), n_local)  # expert order over the received pairs
            _lib.check(lib.omni_expert_coef_pairs(x_all.data_ptr(), up_local.data_ptr(), recv.pair_tokens.data_ptr(),
                                                  recv.pair_weights.data_ptr(), sch.sorted_pair_ids.data_ptr(),
                                                  sch.sorted_experts.data_ptr(), p, t_total, h, n_local, coef.data_ptr(),
                                                  status.data_ptr(), st))
        _lib.check(lib.omni_expert_combine_segments(down_local.data_ptr(), coef.data_ptr(), recv.pair_experts.data_ptr(),
                                                    recv.token_offsets.data_ptr(), t_total, h, n_local, None,
                                                    partial.data_ptr(), _lib.dtype_code(out_dtype), status.data_ptr(), st))
    return partial


def combine_partials(partial: torch.Tensor, part: ExpertPartition, group=None) -> torch.Tensor:
    """Step 4: sum the per-rank partial ``[T_total, H]`` states and return this rank's token rows."""
    t_local = partial.size(0) // part.world
    if dist.get_backend(group) == "nccl":
        out = torch.empty((t_local, partial.size(1)), device=partial.device, dtype=partial.dtype)
        _collective("combine", dist.reduce_scatter_tensor, out, partial.contiguous(), op=dist.ReduceOp.SUM, group=group)
        return out
    # backends without reduce-scatter (gloo, used by the CPU tests): all-reduce, then keep the own rows
    full = partial.clone()
    _collective("combine", dist.all_reduce, full, op=dist.ReduceOp.SUM, group=group)
    return full[part.rank * t_local:(part.rank + 1) * t_local].contiguous()


def partitioned_expert_states(x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, up_local: torch.Tensor,
                              down_local: torch.Tensor, part: ExpertPartition, group=None,
                              local_fn: Callable[[ReceivedPairs, torch.Tensor, torch.Tensor], torch.Tensor] | None = None
                              ) -> torch.Tensor:
    """Steps 2-4: routed-expert states ``[T_local, H]`` (fp32) of this rank's tokens with the tables
    partitioned by rows.  ``local_fn`` replaces step 3 (the CPU tests pass the oracle's arithmetic there);
    by default it is :func:`local_partial_states`, the CUDA kernels."""
    recv = dispatch_pairs(x, indices, weights, part, group)
    partial = (local_fn or local_partial_states)(recv, up_local, down_local)
    return combine_partials(partial, part, group)


class PartitionedOmniMoE(torch.nn.Module):
    """``OmniMoE`` with the expert tables row-partitioned over the ranks of a process group.

    Build it from a full module on every rank (``PartitionedOmniMoE(full_module, group)``): the
    router and the shared MLP are kept whole, ``up_embed`` / ``down_embed`` are cut down to this
    rank's rows.  ``forward(hidden_states)`` takes this rank's tokens ``[B, S, H]`` (the same count on
    every rank) and returns their outputs.  Eval mode, bf16."""

    def __init__(self, module, group=None):
        super().__init__()
        from .modules.omni_moe import OmniMoE
        assert isinstance(module, OmniMoE)
        self.group = group
        self.part = ExpertPartition(module.num_experts, dist.get_world_size(group), dist.get_rank(group))
        self.inner = module
        with torch.no_grad():
            up = self.part.slice_rows(module.up_embed.weight.detach())
            down = self.part.slice_rows(module.down_embed.weight.detach())
        # the full tables are dropped: this rank keeps only its rows
        module.up_embed.weight = torch.nn.Parameter(up, requires_grad=False)
        module.down_embed.weight = torch.nn.Parameter(down, requires_grad=False)
        self._side = None
        #: dtype of the per-rank partial sums that are reduce-scattered: bfloat16 halves the bytes on
        #: NVLink at the cost of one rounding per rank; float32 keeps the single-GPU accuracy
        self.partial_dtype = torch.bfloat16

    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """Streams: the gate/up GEMM of the shared MLP (which needs only x) runs on a side stream while
        the main stream routes, exchanges pairs and token rows, computes this rank's partial expert
        states and reduce-scatters them; the down projection then adds the reduced states."""
        from .ops.router import router_gate_topk
        m = self.inner
        if m.training:
            raise RuntimeError("PartitionedOmniMoE runs in eval mode (batch statistics would need a cross-rank reduction)")
        _lib.require_cuda(hidden_states)
        shape = hidden_states.shape
        x = hidden_states.detach().reshape(-1, m.hidden_size).to(torch.bfloat16).contiguous()
        t, h, i = x.size(0), m.hidden_size, m.intermediate_size
        dev = x.device
        wg, wu, wd, kx, ky, up_l, down_l = m._operands()
        scale, shift = m._bn_fold_eval()
        status = torch.zeros(1, device=dev, dtype=torch.int32)
        lib = _lib.load()
        if self._side is None:
            self._side = torch.cuda.Stream(device=dev)
        act = torch.empty((t, i), device=dev, dtype=torch.bfloat16)
        y = torch.empty((t, h), device=dev, dtype=torch.bfloat16)
        with torch.cuda.device(dev):
            main = torch.cuda.current_stream()
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                _lib.check(lib.omni_mlp_gate_up(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), t, h, i, act.data_ptr(),
                                                status.data_ptr(), self._side.cuda_stream))
                for tns in (x, wg, wu, act):
                    tns.record_stream(self._side)
            scores, indices, weights = router_gate_topk(x, kx, ky, m.top_k, scale, shift, status=status)
            states = partitioned_expert_states(
                x, indices, weights, up_l, down_l, self.part, self.group,
                local_fn=lambda r, u, d: local_partial_states(r, u, d, out_dtype=self.partial_dtype, status=status))
            states = states.float()  # [T_local, H]: the down-projection epilogue adds fp32
            main.wait_stream(self._side)
            _lib.check(lib.omni_mlp_down(act.data_ptr(), wd.data_ptr(), t, h, i, states.data_ptr(), y.data_ptr(),
                                         status.data_ptr(), main.cuda_stream))
        m.last_routing = (scores, indices, weights)
        m.last_status = status
        return y.view(shape).to(hidden_states.dtype)
