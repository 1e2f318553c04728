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


def _stable_order_by_key(key: torch.Tensor, bins: int) -> torch.Tensor:
    """Permutation that groups the flat pairs by ``key`` (in ``[0, bins)``), ascending pair id inside a group."""
    if key.is_cuda:
        from .ops.scheduler import schedule
        raw = schedule(key.view(-1, 1), bins, segments=False)  # the radix scheduler, one pass over `bins` bins
        return raw.sorted_pair_ids.long()
    return torch.sort(key.view(-1).long(), stable=True).indices


@dataclass
class ExchangePlan:
    """Everything the dispatch of one step needs, after the count exchange (the one host synchronisation).

    The local tokens are cut into ``chunks`` equal ranges; a chunk is exchanged, computed and combined on
    its own, so that one chunk's transfers overlap another chunk's kernels.  ``send[c]`` holds the records of
    chunk ``c`` grouped by destination rank (ascending pair id inside a destination)."""
    chunks: int
    tokens_per_chunk: int
    send: list              # per chunk: int32 [n_c, 3] records (token id inside the chunk's all-gathered rows, local expert row, weight bits)
    send_counts: list       # per chunk: list of `world` ints
    recv_counts: list       # per chunk: list of `world` ints


def _sorted_records(indices: torch.Tensor, weights: torch.Tensor, part: ExpertPartition, chunks: int):
    """This rank's pairs as 12-byte records (token id among the chunk's all-gathered rows, expert row inside the
    owner's slice, weight bits), grouped by key = chunk * world + owner in ascending pair order, and the number of
    pairs per key as a ``[chunks, world]`` int64 tensor.  On CUDA: two kernels of the library around its radix
    pass; elsewhere the same in torch operators."""
    world, rank = part.world, part.rank
    t_local, k = indices.shape
    tc = t_local // chunks
    if indices.is_cuda and k > 0:
        from .ops.scheduler import schedule
        dev = indices.device
        idx = indices.to(torch.int32).contiguous()
        w = weights.float().contiguous()
        keys = torch.empty(t_local * k, device=dev, dtype=torch.int32)
        counts = torch.empty(chunks * world, device=dev, dtype=torch.int32)
        records = torch.empty((t_local * k, 3), device=dev, dtype=torch.int32)
        lib = _lib.load()
        with torch.cuda.device(dev):
            st = _lib.stream_ptr()
            _lib.check(lib.omni_partition_keys(idx.data_ptr(), t_local, k, part.rows_per_rank, world, chunks,
                                               keys.data_ptr(), counts.data_ptr(), st))
            order = schedule(keys.view(-1, 1), chunks * world, segments=False).sorted_pair_ids
            _lib.check(lib.omni_partition_records(idx.data_ptr(), w.data_ptr(), order.data_ptr(), t_local, k,
                                                  part.rows_per_rank, world, chunks, rank * tc, records.data_ptr(), st))
        return records, counts.view(chunks, world).long()
    flat_e = indices.reshape(-1).to(torch.int32)
    owner = part.owner(flat_e).to(torch.int32)
    pair = torch.arange(flat_e.numel(), device=flat_e.device, dtype=torch.int32)
    token = torch.div(pair, max(k, 1), rounding_mode="floor")
    chunk_of = torch.div(token, max(tc, 1), rounding_mode="floor") if chunks > 1 else torch.zeros_like(token)
    key = chunk_of * world + owner
    order = _stable_order_by_key(key, chunks * world)
    counts = torch.bincount(key.long(), minlength=chunks * world).view(chunks, world)
    tok_rec = (token[order] - chunk_of[order] * tc + rank * tc).to(torch.int32)
    local_e = flat_e[order] - owner[order] * part.rows_per_rank
    w_bits = weights.reshape(-1).float()[order].view(torch.int32)
    return torch.stack([tok_rec, local_e, w_bits], dim=1).contiguous(), counts


def plan_exchange(indices: torch.Tensor, weights: torch.Tensor, part: ExpertPartition, group=None,
                  chunks: int = 1, comm_stream=None) -> ExchangePlan:
    """Sorts this rank's pairs by (chunk, owning rank) and exchanges the counts.

    ``indices [T_local, k]`` global expert ids, ``weights [T_local, k]``.  The count exchange doubles as a
    handshake: every rank also states its shard shape, so a peer that left, or one configured with another
    token count, k or chunk count, is noticed here, on the host, before any payload moves.  On CUDA with a
    ``comm_stream`` the collective is issued on that stream (after the sort, which runs on the current one)."""
    world, rank = part.world, part.rank
    t_local, k = indices.shape
    if chunks < 1 or t_local % chunks:
        chunks = 1
    tc = t_local // chunks
    records, counts = _sorted_records(indices, weights, part, chunks)
    shape_cols = [torch.full((world, 1), v, dtype=counts.dtype, device=counts.device) for v in (t_local, k, chunks)]
    hello = torch.cat([counts.t()] + shape_cols, dim=1).contiguous()
    got = torch.empty_like(hello)
    if comm_stream is not None and hello.is_cuda:
        main = torch.cuda.current_stream()
        ready, done = torch.cuda.Event(), torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(comm_stream):
            comm_stream.wait_event(ready)
            _collective("count exchange", dist.all_to_all_single, got, hello, group=group)
            done.record(comm_stream)
        main.wait_event(done)
        hello.record_stream(comm_stream)
        got.record_stream(comm_stream)
    else:
        _collective("count exchange", dist.all_to_all_single, got, hello, group=group)
    got_host = got.tolist()  # the one host synchronisation of a step: the split sizes
    send_host = counts.tolist()
    for peer, row in enumerate(got_host):
        t_peer, k_peer, c_peer = row[-3:]
        if t_peer != t_local or k_peer != k or c_peer != chunks or len(row) != chunks + 3:
            raise ExchangeError("count exchange", f"rank {peer} shards {t_peer} tokens x {k_peer} experts in {c_peer} chunks, this "
                                                  f"rank {t_local} x {k} in {chunks}: every rank must pass the same shard shape")
        for cnt in row[:chunks]:
            if cnt < 0 or cnt > tc * k:
                raise ExchangeError("count exchange", f"rank {peer} announces {cnt} pairs, more than its {tc * k} per chunk")
    starts = [0]
    for c in range(chunks):
        starts.append(starts[-1] + sum(send_host[c]))
    send = [records[starts[c]:starts[c + 1]] for c in range(chunks)]
    recv_counts = [[got_host[p][c] for p in range(world)] for c in range(chunks)]
    return ExchangePlan(chunks, tc, send, send_host, recv_counts)


def send_pairs(plan: ExchangePlan, c: int, recv: torch.Tensor, group=None) -> None:
    """The payload collective of chunk ``c``: its 12-byte records into ``recv [sum(recv_counts[c]), 3]`` int32."""
    _collective("pair dispatch", dist.all_to_all_single, recv, plan.send[c], output_split_sizes=plan.recv_counts[c],
                input_split_sizes=plan.send_counts[c], group=group)


def received_pairs(plan: ExchangePlan, c: int, recv: torch.Tensor, x_all: torch.Tensor) -> ReceivedPairs:
    """Splits the received records of chunk ``c`` and builds the CSR of pairs by token.  What a rank receives is
    grouped by source rank and, inside a source, in ascending pair order, i.e. already ordered by token id."""
    pair_tokens = recv[:, 0].contiguous()
    bounds = torch.arange(x_all.size(0) + 1, device=recv.device, dtype=torch.int32)
    token_offsets = torch.searchsorted(pair_tokens, bounds, right=False).to(torch.int32)
    return ReceivedPairs(x_all, pair_tokens, recv[:, 1].contiguous(), recv[:, 2].contiguous().view(torch.float32),
                         token_offsets, plan.send_counts[c], plan.recv_counts[c])


def gather_token_rows(x_chunk: torch.Tensor, part: ExpertPartition, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather of a token range: ``[T, H]`` per rank -> ``[world * T, H]`` ordered by rank."""
    if out is None:
        out = torch.empty((part.world * x_chunk.size(0), x_chunk.size(1)), device=x_chunk.device, dtype=x_chunk.dtype)
    _collective("token all-gather", dist.all_gather_into_tensor, out, x_chunk.contiguous(), group=group)
    return out


def exchange_chunk(plan: ExchangePlan, c: int, x_chunk: torch.Tensor, part: ExpertPartition, group=None) -> ReceivedPairs:
    """Moves chunk ``c`` on the current stream: its pair records to the owners of the expert rows and its token
    rows ``x_chunk [T_local / chunks, H]`` to every rank."""
    recv = torch.empty((sum(plan.recv_counts[c]), 3), device=x_chunk.device, dtype=torch.int32)
    send_pairs(plan, c, recv, group)
    return received_pairs(plan, c, recv, gather_token_rows(x_chunk, part, group))


def dispatch_pairs(x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, part: ExpertPartition,
                   group=None) -> ReceivedPairs:
    """Step 2 in one piece: send every routed pair of this rank's tokens to the rank that owns the expert row.

    ``x [T_local, H]``, ``indices [T_local, k]`` global expert ids, ``weights [T_local, k]`` float32.
    Every rank must pass the same ``T_local``.
    """
    plan = plan_exchange(indices, weights, part, group, chunks=1)
    return exchange_chunk(plan, 0, x, part, group)


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
            sch = schedule(recv.pair_experts.view(-1, 1), n_local, segments=False)  # expert order over the received pairs
            _lib.check(lib.omni_expert_coef_pairs(x_all.data_ptr(), up_local.data_ptr(), recv.pair_tokens.data_ptr(),
                                                  recv.pair_weights.data_ptr(), sch.sorted_pair_ids.data_ptr(),
                                                  sch.sorted_experts.data_ptr(), p, t_total, h, n_local, coef.data_ptr(),
                                                  status.data_ptr(), st))
        _lib.check(lib.omni_expert_combine_segments(down_local.data_ptr(), coef.data_ptr(), recv.pair_experts.data_ptr(),
                                                    recv.token_offsets.data_ptr(), t_total, h, n_local, None,
                                                    partial.data_ptr(), _lib.dtype_code(out_dtype), status.data_ptr(), st))
    return partial


def combine_partials(partial: torch.Tensor, part: ExpertPartition, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Step 4: sum the per-rank partial ``[T_total, H]`` states and return this rank's token rows."""
    t_local = partial.size(0) // part.world
    if dist.get_backend(group) == "nccl":
        if out is None:
            out = torch.empty((t_local, partial.size(1)), device=partial.device, dtype=partial.dtype)
        _collective("combine", dist.reduce_scatter_tensor, out, partial.contiguous(), op=dist.ReduceOp.SUM, group=group)
        return out
    # backends without reduce-scatter (gloo, used by the CPU tests): all-reduce, then keep the own rows
    full = partial.clone()
    _collective("combine", dist.all_reduce, full, op=dist.ReduceOp.SUM, group=group)
    return full[part.rank * t_local:(part.rank + 1) * t_local].contiguous()


class _PhaseClock:
    """CUDA-event stopwatch for the phases of a partitioned step.  A phase may run in several pieces and on
    several streams; its time is the sum of its pieces, each measured on the stream it runs on."""

    def __init__(self, enabled: bool):
        self.enabled = enabled
        self.pieces = []

    def start(self, name: str):
        if not self.enabled:
            return None
        a = torch.cuda.Event(enable_timing=True)
        a.record()
        return (name, a)

    def stop(self, tok):
        if tok is None:
            return
        b = torch.cuda.Event(enable_timing=True)
        b.record()
        self.pieces.append((tok[0], tok[1], b))

    def totals(self) -> dict:
        """Milliseconds per phase; call after a synchronisation."""
        out = {}
        for name, a, b in self.pieces:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out


def partitioned_expert_states(x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, up_local: torch.Tensor,
                              down_local: torch.Tensor, part: ExpertPartition, group=None,
                              local_fn: Callable[[ReceivedPairs, torch.Tensor, torch.Tensor], torch.Tensor] | None = None,
                              chunks: int = 1, comm_stream=None, x_ready=None, clock: "_PhaseClock | None" = None,
                              between_chunks: Callable[[int], None] | None = None,
                              local_partial_dtype: torch.dtype | None = None,
                              x_all_buffers: list | None = None) -> torch.Tensor:
    """Steps 2-4: routed-expert states ``[T_local, H]`` of this rank's tokens with the tables partitioned by
    rows.  ``local_fn`` replaces step 3 (the CPU tests pass the oracle's arithmetic there); by default it is
    :func:`local_partial_states`, the CUDA kernels.

    With ``chunks > 1`` the local tokens are cut into that many equal ranges which go through dispatch,
    local kernels and combine one after another; on CUDA with a ``comm_stream`` every collective is issued
    on that stream, so the transfers of one chunk run beside the kernels of another.  ``x_ready`` is an event
    after which ``x`` may be read and ``x_all_buffers`` (one ``[world * T_local / chunks, H]`` buffer per chunk,
    allocated by the caller BEFORE that event was recorded) may be written; without them the all-gathers start
    now, on the current stream's position.  ``between_chunks(c)`` is called on
    the compute stream after chunk ``c``'s kernels were enqueued (the caller's own work, e.g. a GEMM that
    needs no exchange); ``local_partial_dtype`` is the dtype ``local_fn`` returns (default float32) - the
    pipelined form allocates the reduce-scatter outputs before the kernels run.  Returns float32 in the
    pipelined form, the dtype of ``local_fn``'s result otherwise."""
    local_fn = local_fn or local_partial_states
    clock = clock or _PhaseClock(False)
    t_local = x.size(0)
    if chunks < 1 or t_local % chunks:
        chunks = 1
    tc = t_local // chunks
    piped = x.is_cuda and comm_stream is not None
    if not piped:
        plan = plan_exchange(indices, weights, part, group, chunks)
        outs = []
        for c in range(chunks):
            recv = exchange_chunk(plan, c, x[c * tc:(c + 1) * tc], part, group)
            outs.append(combine_partials(local_fn(recv, up_local, down_local), part, group))
            if between_chunks is not None:
                between_chunks(c)
        return outs[0] if chunks == 1 else torch.cat(outs, dim=0)

    main = torch.cuda.current_stream()
    dev, h, world = x.device, x.size(1), part.world
    if x_ready is None or x_all_buffers is None:
        x_ready, x_all_buffers = None, None
    # Every buffer is allocated while the compute stream is current and reaches the communication stream through
    # an event recorded AFTER its allocation (the caching allocator may hand out a block that earlier work of the
    # compute stream still reads: the other stream has to be behind that work before it writes the block);
    # record_stream() at the end tells the allocator about the second user.
    if x_all_buffers is None:
        x_all_buffers = [torch.empty((world * tc, h), device=dev, dtype=x.dtype) for _ in range(chunks)]
        x_ready = torch.cuda.Event()
        x_ready.record(main)
    x_alls = x_all_buffers
    assert len(x_alls) == chunks and all(b.shape == (world * tc, h) for b in x_alls)
    # token rows first: they need no routing, so their all-gathers start while the router still runs
    with torch.cuda.stream(comm_stream):
        comm_stream.wait_event(x_ready)
        tk = clock.start("dispatch")
        for c in range(chunks):
            gather_token_rows(x[c * tc:(c + 1) * tc], part, group, out=x_alls[c])
        clock.stop(tk)
    tk = clock.start("plan")
    plan = plan_exchange(indices, weights, part, group, chunks, comm_stream=comm_stream)
    clock.stop(tk)
    raw = [torch.empty((sum(plan.recv_counts[c]), 3), device=dev, dtype=torch.int32) for c in range(chunks)]
    probe = local_partial_dtype if local_partial_dtype is not None else torch.float32
    reduced = [torch.empty((tc, h), device=dev, dtype=probe) for _ in range(chunks)]
    states = torch.empty((t_local, h), device=dev, dtype=torch.float32)
    ev_send = torch.cuda.Event()
    ev_send.record(main)   # the records were built on the compute stream
    ev_disp = [torch.cuda.Event() for _ in range(chunks)]
    ev_local = [torch.cuda.Event() for _ in range(chunks)]
    ev_comb = [torch.cuda.Event() for _ in range(chunks)]
    partials = [None] * chunks

    def issue_dispatch(c):
        with torch.cuda.stream(comm_stream):
            if c == 0:
                comm_stream.wait_event(ev_send)
            tk_ = clock.start("dispatch")
            send_pairs(plan, c, raw[c], group)
            clock.stop(tk_)
            ev_disp[c].record(comm_stream)

    issue_dispatch(0)
    for c in range(chunks):
        if c + 1 < chunks:
            issue_dispatch(c + 1)
        main.wait_event(ev_disp[c])
        tk = clock.start("local")
        partials[c] = local_fn(received_pairs(plan, c, raw[c], x_alls[c]), up_local, down_local)
        clock.stop(tk)
        assert partials[c].dtype == probe, "local_fn must return local_partial_dtype"
        ev_local[c].record(main)
        with torch.cuda.stream(comm_stream):
            comm_stream.wait_event(ev_local[c])
            tk_ = clock.start("combine")
            combine_partials(partials[c], part, group, out=reduced[c])
            clock.stop(tk_)
            ev_comb[c].record(comm_stream)
        if between_chunks is not None:
            between_chunks(c)
    for c in range(chunks):
        main.wait_event(ev_comb[c])
        states[c * tc:(c + 1) * tc].copy_(reduced[c])
    for tns in x_alls + raw + partials + reduced + plan.send + [x]:
        tns.record_stream(comm_stream)
    return states


class PartitionedOmniMoE(torch.nn.Module):
    """``OmniMoE`` with the expert tables row-partitioned over the ranks of a process group.

    Build it from a full module on every rank (``PartitionedOmniMoE(full_module, group)``): the router and
    the shared MLP are kept whole, and this wrapper keeps rows ``[lo, hi)`` of ``up_embed`` / ``down_embed``
    as ``up_local`` / ``down_local``.  The wrapped module is left without tables and refuses to run on its
    own (its kernels would index a slice with global expert ids).  ``forward(hidden_states)`` takes this
    rank's tokens ``[B, S, H]`` (the same count on every rank) and returns their outputs.  Eval mode, bf16.

    ``chunks`` token ranges go through the exchange one after another with the collectives on a second
    stream (see :func:`partitioned_expert_states`); ``record_phases = True`` makes every forward leave the
    device time of its phases in ``last_phases_ms`` (after a synchronisation, via :meth:`phases_ms`)."""

    def __init__(self, module, group=None, chunks: int = 2, table_slices=None):
        super().__init__()
        from .modules.omni_moe import OmniMoE
        assert isinstance(module, OmniMoE)
        self.group = group
        self.part = ExpertPartition(module.num_experts, dist.get_world_size(group), dist.get_rank(group))
        if self.part.hi - self.part.lo < 1:
            raise ValueError(f"{module.num_experts} expert rows over {self.part.world} ranks leave rank {self.part.rank} "
                             "without rows: use fewer ranks")
        self.inner = module
        if table_slices is None:
            with torch.no_grad():
                up = self.part.slice_rows(module.up_embed.weight.detach())
                down = self.part.slice_rows(module.down_embed.weight.detach())
        else:
            up, down = table_slices  # built as slices in the first place (tables too large to exist whole)
        assert up.shape == down.shape == (self.part.hi - self.part.lo, module.hidden_size)
        self.up_local = torch.nn.Parameter(up.to(torch.bfloat16).contiguous(), requires_grad=False)
        self.down_local = torch.nn.Parameter(down.to(torch.bfloat16).contiguous(), requires_grad=False)
        # the full tables are dropped; the wrapped module can no longer run by itself
        empty = lambda: torch.nn.Parameter(torch.empty(0, module.hidden_size, dtype=up.dtype, device=up.device), requires_grad=False)
        module.up_embed.weight, module.down_embed.weight = empty(), empty()
        module._tables_partitioned = True
        self.chunks = chunks
        #: the gate/up GEMM of the shared MLP is enqueued after this chunk's expert kernels (default: the last one,
        #: so that it runs while the last reduce-scatter is on the wire)
        self.mlp_after_chunk = None
        self._comm = None
        self.record_phases = False
        self._clock = None
        #: dtype of the per-rank partial sums that are reduce-scattered: bfloat16 halves the bytes on
        #: NVLink at the cost of one rounding per rank; float32 keeps the single-GPU accuracy
        self.partial_dtype = torch.bfloat16

    def phases_ms(self) -> dict:
        """Device time of the phases of the latest forward (``record_phases`` must be on): route, dispatch
        (count exchange, pair records, token rows), local (schedule + expert kernels), combine
        (reduce-scatter), mlp.  Phases on different streams overlap, so they can add up to more than the step."""
        if self._clock is None:
            return {}
        torch.cuda.synchronize()
        t = self._clock.totals()
        t["dispatch"] = t.get("dispatch", 0.0) + t.pop("plan", 0.0)
        return {k: round(v, 4) for k, v in t.items()}

    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """Compute stream: router, then per chunk the local expert kernels, the gate/up GEMM after the first
        chunk, the down projection (which adds the reduced expert states) at the end.  Communication stream:
        token all-gathers (from the start), count exchange, pair records, reduce-scatters."""
        from .ops.router import router_gate_topk
        m = self.inner
        if m.training:
            raise RuntimeError("PartitionedOmniMoE runs in eval mode (batch statistics would need a cross-rank reduction)")
        _lib.require_cuda(hidden_states)
        shape = hidden_states.shape
        x = hidden_states.detach().reshape(-1, m.hidden_size).to(torch.bfloat16).contiguous()
        t, h, i = x.size(0), m.hidden_size, m.intermediate_size
        dev = x.device
        wg, wu, wd, kx, ky = (m._bf16_weight(q.weight) for q in (m.gate_proj, m.up_proj, m.down_proj, m.router_gate_x, m.router_gate_y))
        scale, shift = m._bn_fold_eval()
        status = torch.zeros(1, device=dev, dtype=torch.int32)
        lib = _lib.load()
        clock = self._clock = _PhaseClock(self.record_phases)
        act = torch.empty((t, i), device=dev, dtype=torch.bfloat16)
        y = torch.empty((t, h), device=dev, dtype=torch.bfloat16)
        with torch.cuda.device(dev):
            if self._comm is None:
                self._comm = torch.cuda.Stream(device=dev)
            main = torch.cuda.current_stream()
            n_chunks = self.chunks if (self.chunks >= 1 and t % max(self.chunks, 1) == 0) else 1
            # the all-gathered token rows: allocated before the event the communication stream waits for
            x_alls = [torch.empty((self.part.world * (t // n_chunks), h), device=dev, dtype=torch.bfloat16) for _ in range(n_chunks)]
            x_ready = torch.cuda.Event()
            x_ready.record(main)
            tk = clock.start("route")
            scores, indices, weights = router_gate_topk(x, kx, ky, m.top_k, scale, shift, status=status)
            clock.stop(tk)

            mlp_at = n_chunks - 1 if self.mlp_after_chunk is None else min(self.mlp_after_chunk, n_chunks - 1)

            def gate_up(c):
                if c == mlp_at:
                    tk_ = clock.start("mlp")
                    _lib.check(lib.omni_mlp_gate_up(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), t, h, i, act.data_ptr(),
                                                    status.data_ptr(), main.cuda_stream))
                    clock.stop(tk_)

            states = partitioned_expert_states(
                x, indices, weights, self.up_local, self.down_local, self.part, self.group,
                local_fn=lambda r, u, d: local_partial_states(r, u, d, out_dtype=self.partial_dtype, status=status),
                chunks=n_chunks, comm_stream=self._comm, x_ready=x_ready, clock=clock, between_chunks=gate_up,
                local_partial_dtype=self.partial_dtype, x_all_buffers=x_alls)
            tk = clock.start("mlp")
            _lib.check(lib.omni_mlp_down(act.data_ptr(), wd.data_ptr(), t, h, i, states.data_ptr(), y.data_ptr(),
                                         status.data_ptr(), main.cuda_stream))
            clock.stop(tk)
        m.last_routing = (scores, indices, weights)
        m.last_status = status
        return y.view(shape).to(hidden_states.dtype)


# ---------------------------------------------------------------------------------------------------------------------
# Expert tables partitioned by COLUMNS
# ---------------------------------------------------------------------------------------------------------------------
# An expert of this layer is one Up row and one Down row, so the tables can just as well be cut along the hidden
# dimension: rank g keeps columns [g * H / G, (g + 1) * H / G) of every row (the same memory per rank as a row
# partition).  Then
#   * x[t] . Up[e] is the sum of G partial dot products, one per rank: an all-reduce of [T_total, k] floats
#     (4 bytes per pair instead of a hidden-sized partial state per token and rank);
#   * sum_j c * Down[e] over a rank's columns gives those columns of the output for ALL tokens; an all-to-all returns
#     them to the ranks that own the tokens (T_total * H / G values per rank, against T_total * H for a reduce-scatter
#     of partial states), and the token rows reach the ranks the same way (instead of an all-gather);
#   * every size is known in advance: no count exchange, no host synchronisation inside the step.
# Every rank walks all pairs, but over H / G columns each, so the bytes it gathers are the same as with a row partition.


@dataclass(frozen=True)
class ColumnPartition:
    """Contiguous column partition of ``[*, hidden]`` tables over ``world`` ranks (``hidden % world == 0``)."""
    hidden: int
    world: int
    rank: int

    @property
    def width(self) -> int:
        return self.hidden // self.world

    @property
    def lo(self) -> int:
        return self.rank * self.width

    @property
    def hi(self) -> int:
        return (self.rank + 1) * self.width

    def slice_columns(self, table: torch.Tensor) -> torch.Tensor:
        return table[:, self.lo:self.hi].contiguous()


def exchange_token_columns(x: torch.Tensor, part: ColumnPartition, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``[T_local, H]`` per rank -> ``[world * T_local, H / world]``: this rank's columns of every rank's tokens,
    ordered by source rank (= global token order when the tokens are sharded contiguously)."""
    t, h = x.shape
    send = x.view(t, part.world, part.width).transpose(0, 1).contiguous().view(part.world * t, part.width)
    if out is None:
        out = torch.empty_like(send)
    _collective("token columns", dist.all_to_all_single, out, send, group=group)
    return out


def return_state_columns(y_cols: torch.Tensor, part: ColumnPartition, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Inverse of :func:`exchange_token_columns` for the results: ``[world * T_local, H / world]`` (this rank's
    columns of all tokens) -> ``[world, T_local, H / world]`` (all column slices of this rank's tokens)."""
    if out is None:
        out = torch.empty_like(y_cols)
    _collective("state columns", dist.all_to_all_single, out, y_cols.contiguous(), group=group)
    return out.view(part.world, y_cols.size(0) // part.world, part.width)


def gather_routing(indices: torch.Tensor, weights: torch.Tensor, group=None, out=None):
    """The routing of all tokens on every rank: ``[T_local, k]`` -> ``[T_total, k]`` (expert ids int32, weights float32)."""
    world = dist.get_world_size(group)
    idx, w = indices.to(torch.int32).contiguous(), weights.float().contiguous()
    idx_all, w_all = out if out is not None else (torch.empty((world * idx.size(0), idx.size(1)), device=idx.device, dtype=torch.int32),
                                                  torch.empty((world * w.size(0), w.size(1)), device=w.device, dtype=torch.float32))
    _collective("routing all-gather", dist.all_gather_into_tensor, idx_all, idx, group=group)
    _collective("routing all-gather", dist.all_gather_into_tensor, w_all, w, group=group)
    return idx_all, w_all


def column_partial_dots(x_cols: torch.Tensor, idx_all: torch.Tensor, up_cols: torch.Tensor, status: torch.Tensor | None = None):
    """This rank's part of ``x[t] . Up[e[t, j]]`` for all tokens, ``[T_total, k]`` float32 (CUDA kernels)."""
    from .ops.scheduler import schedule
    _lib.require_cuda(x_cols, idx_all, up_cols)
    t, hs = x_cols.shape
    k, n = idx_all.size(1), up_cols.size(0)
    dots = torch.empty((t, k), device=x_cols.device, dtype=torch.float32)
    if status is None:
        status = _lib.device_status(x_cols.device)
    with torch.cuda.device(x_cols.device):
        sch = schedule(idx_all, n, segments=False)
        _lib.check(_lib.load().omni_expert_dots(x_cols.data_ptr(), up_cols.data_ptr(), sch.sorted_pair_ids.data_ptr(),
                                                sch.sorted_experts.data_ptr(), t, k, hs, n, dots.data_ptr(), status.data_ptr(),
                                                _lib.stream_ptr()))
    return dots


def column_combine(coef: torch.Tensor, idx_all: torch.Tensor, down_cols: torch.Tensor, out_dtype=torch.bfloat16,
                   status: torch.Tensor | None = None) -> torch.Tensor:
    """This rank's columns of ``sum_j coef[t, j] * Down[e[t, j]]`` for all tokens (CUDA kernel)."""
    _lib.require_cuda(coef, idx_all, down_cols)
    t, k = idx_all.shape
    n, hs = down_cols.shape
    y = torch.empty((t, hs), device=coef.device, dtype=out_dtype)
    if status is None:
        status = _lib.device_status(coef.device)
    with torch.cuda.device(coef.device):
        _lib.check(_lib.load().omni_expert_combine(down_cols.data_ptr(), coef.data_ptr(), idx_all.data_ptr(), t, k, hs, n, None,
                                                   y.data_ptr(), _lib.dtype_code(out_dtype), status.data_ptr(), _lib.stream_ptr()))
    return y


def column_expert_states(x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, up_cols: torch.Tensor,
                         down_cols: torch.Tensor, part: ColumnPartition, group=None,
                         dots_fn: Callable | None = None, combine_fn: Callable | None = None) -> torch.Tensor:
    """Routed-expert states ``[T_local, H]`` of this rank's tokens with the tables partitioned by columns, one
    collective after the other on the current stream (the plain form; :class:`ColumnPartitionedOmniMoE` overlaps
    them with the kernels).  ``dots_fn(x_cols, idx_all, up_cols)`` and ``combine_fn(coef, idx_all, down_cols)``
    replace the CUDA kernels (the CPU tests pass the oracle's arithmetic)."""
    dots_fn = dots_fn or column_partial_dots
    combine_fn = combine_fn or column_combine
    x_cols = exchange_token_columns(x, part, group)
    idx_all, w_all = gather_routing(indices, weights, group)
    dots = dots_fn(x_cols, idx_all, up_cols).float().contiguous()
    _collective("dot products", dist.all_reduce, dots, op=dist.ReduceOp.SUM, group=group)
    coef = torch.nn.functional.silu(dots) * w_all
    y_cols = combine_fn(coef, idx_all, down_cols)
    mine = return_state_columns(y_cols, part, group)
    return mine.transpose(0, 1).reshape(x.size(0), part.hidden)


class ColumnPartitionedOmniMoE(torch.nn.Module):
    """``OmniMoE`` with the expert tables partitioned by columns over the ranks of a process group.

    Build it from a full module on every rank, or pass ``table_slices = (up_cols, down_cols)``, each ``[N, H / world]``,
    when the tables are too large to exist whole.  Router and shared MLP are kept whole; the wrapped module is left
    without tables and refuses to run on its own.  ``forward(hidden_states)`` takes this rank's tokens ``[B, S, H]``
    (the same count on every rank, sharded contiguously in rank order) and returns their outputs.  Eval mode, bf16.

    Compute stream: router, schedule of all pairs, partial dot products, their all-reduce, activation, combine over the
    rank's columns, gate/up GEMM, down projection with the returned states added in its epilogue.  Communication
    stream: the token columns (from the start, beside the router), the routing all-gather, the return of the state
    columns (beside the gate/up GEMM).  Nothing on the host depends on device data: the whole step is enqueued ahead."""

    def __init__(self, module, group=None, table_slices=None):
        super().__init__()
        from .modules.omni_moe import OmniMoE
        assert isinstance(module, OmniMoE)
        self.group = group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if module.hidden_size % world or (module.hidden_size // world) % 8:
            raise ValueError(f"hidden size {module.hidden_size} cannot be cut into {world} column slices of a multiple of 8")
        self.part = ColumnPartition(module.hidden_size, world, rank)
        self.inner = module
        if table_slices is None:
            with torch.no_grad():
                up = self.part.slice_columns(module.up_embed.weight.detach())
                down = self.part.slice_columns(module.down_embed.weight.detach())
        else:
            up, down = table_slices
        assert up.shape == down.shape == (module.num_experts, self.part.width)
        self.up_cols = torch.nn.Parameter(up.to(torch.bfloat16).contiguous(), requires_grad=False)
        self.down_cols = torch.nn.Parameter(down.to(torch.bfloat16).contiguous(), requires_grad=False)
        empty = lambda: torch.nn.Parameter(torch.empty(0, module.hidden_size, dtype=up.dtype, device=up.device), requires_grad=False)
        module.up_embed.weight, module.down_embed.weight = empty(), empty()
        module._tables_partitioned = True
        self.record_phases = False
        self._clock = None
        self._comm = None

    def phases_ms(self) -> dict:
        """Device time of the phases of the latest forward (``record_phases`` must be on): route, exchange (token
        columns, routing, state columns; on the communication stream), local (schedule, dot products, combine),
        reduce (the all-reduce of the dot products), mlp."""
        if self._clock is None:
            return {}
        torch.cuda.synchronize()
        return {k: round(v, 4) for k, v in self._clock.totals().items()}

    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        from .ops.router import router_gate_topk
        m, part = self.inner, self.part
        if m.training:
            raise RuntimeError("ColumnPartitionedOmniMoE runs in eval mode (batch statistics would need a cross-rank reduction)")
        _lib.require_cuda(hidden_states)
        shape = hidden_states.shape
        x = hidden_states.detach().reshape(-1, m.hidden_size).to(torch.bfloat16).contiguous()
        t, h, i, k = x.size(0), m.hidden_size, m.intermediate_size, m.top_k
        world, hs = part.world, part.width
        dev = x.device
        wg, wu, wd, kx, ky = (m._bf16_weight(q.weight) for q in (m.gate_proj, m.up_proj, m.down_proj, m.router_gate_x, m.router_gate_y))
        scale, shift = m._bn_fold_eval()
        status = torch.zeros(1, device=dev, dtype=torch.int32)
        lib = _lib.load()
        clock = self._clock = _PhaseClock(self.record_phases)
        with torch.cuda.device(dev):
            if self._comm is None:
                self._comm = torch.cuda.Stream(device=dev)
            comm, main = self._comm, torch.cuda.current_stream()
            # every buffer that the communication stream writes is allocated here, before the events it waits for
            act = torch.empty((t, i), device=dev, dtype=torch.bfloat16)
            y = torch.empty((t, h), device=dev, dtype=torch.bfloat16)
            x_cols = torch.empty((world * t, hs), device=dev, dtype=torch.bfloat16)
            idx_all = torch.empty((world * t, k), device=dev, dtype=torch.int32)
            w_all = torch.empty((world * t, k), device=dev, dtype=torch.float32)
            y_back = torch.empty((world * t, hs), device=dev, dtype=torch.bfloat16)
            x_ready = torch.cuda.Event()
            x_ready.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(x_ready)
                tk = clock.start("exchange")
                exchange_token_columns(x, part, self.group, out=x_cols)
                clock.stop(tk)
                ev_x = torch.cuda.Event()
                ev_x.record(comm)
            tk = clock.start("route")
            scores, indices, weights = router_gate_topk(x, kx, ky, k, scale, shift, status=status)
            clock.stop(tk)
            ev_route = torch.cuda.Event()
            ev_route.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(ev_route)
                tk = clock.start("exchange")
                gather_routing(indices, weights, self.group, out=(idx_all, w_all))
                clock.stop(tk)
                ev_r = torch.cuda.Event()
                ev_r.record(comm)
            main.wait_event(ev_r)
            main.wait_event(ev_x)
            tk = clock.start("local")
            dots = column_partial_dots(x_cols, idx_all, self.up_cols, status)
            clock.stop(tk)
            tk = clock.start("reduce")
            _collective("dot products", dist.all_reduce, dots, op=dist.ReduceOp.SUM, group=self.group)
            clock.stop(tk)
            tk = clock.start("local")
            coef = torch.nn.functional.silu(dots).mul_(w_all)
            y_cols = column_combine(coef, idx_all, self.down_cols, torch.bfloat16, status)
            clock.stop(tk)
            ev_comb = torch.cuda.Event()
            ev_comb.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(ev_comb)
                tk = clock.start("exchange")
                mine = return_state_columns(y_cols, part, self.group, out=y_back)
                clock.stop(tk)
                ev_y = torch.cuda.Event()
                ev_y.record(comm)
            tk = clock.start("mlp")
            _lib.check(lib.omni_mlp_gate_up(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), t, h, i, act.data_ptr(),
                                            status.data_ptr(), main.cuda_stream))
            clock.stop(tk)
            main.wait_event(ev_y)
            states = torch.empty((t, h), device=dev, dtype=torch.float32)   # [world, t, hs] bf16 -> [t, world * hs] fp32, one pass
            states.view(t, world, hs).copy_(mine.transpose(0, 1))
            tk = clock.start("mlp")
            _lib.check(lib.omni_mlp_down(act.data_ptr(), wd.data_ptr(), t, h, i, states.data_ptr(), y.data_ptr(),
                                         status.data_ptr(), main.cuda_stream))
            clock.stop(tk)
            for tns in (x, x_cols, indices, weights, idx_all, w_all, y_cols, y_back):
                tns.record_stream(comm)
        m.last_routing = (scores, indices, weights)
        m.last_status = status
        return y.view(shape).to(hidden_states.dtype)


def columns_from_row_slices(rows_local: torch.Tensor, group=None) -> torch.Tensor:
    """Re-partitions a table from rows to columns without ever holding it whole: every rank passes its contiguous
    block of rows ``[N / world, H]`` (equal blocks, in rank order) and gets its column slice ``[N, H / world]``."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    r, h = rows_local.shape
    assert h % world == 0, "the hidden size must be a multiple of the world size"
    hs = h // world
    send = rows_local.view(r, world, hs).transpose(0, 1).contiguous().view(world * r, hs)
    out = torch.empty_like(send)
    _collective("table columns", dist.all_to_all_single, out, send, group=group)
    return out
