"""Expert-parallel 256-expert MoE layer: one process per GPU, ``torch.distributed``.

The reference has no multi-rank code; its operator is one rank's 32-expert shard
of an expert-parallel layer, selected by ``local_expert_offset``
(full-agent-pipeline/references/moe.py:165-171, moe/solution/cuda/moe.cu:180-183).
This module adds the one exchange pair that turns eight shards into the layer:

* the 256 global experts are eight shards of 32 (= the eight routing groups);
  rank ``r`` of ``R`` (R in 1, 2, 4, 8) owns shards ``[8r/R, 8(r+1)/R)``;
* tokens are data parallel: every rank holds its own ``T_local`` tokens;
* **dispatch** (all-to-all-v): each rank routes its tokens (the operator's own routing
  kernel through ``moe_fp8_block_scale_route``), and sends one record per
  (token, selected shard): the fp8 row (7168 B), its 56 block scales and its 256
  routing logits, so that the *unchanged* shard operator re-derives the routing on
  the owner and the drop-in signature is kept;
* the owner runs the shard operator once per owned shard on the records it received;
* **combine** (all-to-all-v back): one bf16 row per record; the source rank adds the
  rows of a token in ascending shard order in fp32 and casts to bf16 -- the order in
  which the layer reference sums the eight shard outputs.

Counts are exchanged with one small all-gather and read on the host (the split
sizes of ``all_to_all_single`` are host integers).  No collective other than these.

Two transports.  ``"nccl"``: the exchange is ``all_to_all_single`` and the gather / pack /
accumulate steps are torch index operations.  ``"p2p"``: every rank owns a symmetric buffer
(torch symmetric memory: the same allocation mapped into every peer over NVLink); the
dispatch is ONE kernel that gathers, packs and stores each record straight into the owner's
receive area (``moe_ep_dispatch_push``), and the combine happens inside the shard operator's
last kernel, which writes every result row directly into the source rank's receive area
(``moe_fp8_block_scale_run_rows`` with peer destinations).  Between the phases the ranks meet
at the symmetric-memory barrier (torch's barrier kernel, which waits for its peers' signals; every
rank reaches it, see ``_forward_p2p``).  The operator's own kernels use plain peer stores only: no
multicast (torch is told not to bind the buffer to a multicast object either), no TMA on peer
memory, and none of them waits on a peer.

``local_op`` and ``route_fn`` are injectable so that the host-side logic can be
tested with gloo on CPU ranks; the defaults are the CUDA operator and fail loudly
without the compiled library.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

N_SHARDS = 8
E_LOCAL = 32
H = 7168
KB = 56


def shards_of_rank(rank: int, world: int) -> List[int]:
    if N_SHARDS % world != 0:
        raise ValueError("world size must divide 8")
    per = N_SHARDS // world
    return list(range(rank * per, (rank + 1) * per))


def owner_of_shard(shard: int, world: int) -> int:
    return shard // (N_SHARDS // world)


@dataclass
class DispatchPlan:
    """Who sends what: built on every rank from its own routing result and the gathered counts."""
    token_lists: List[torch.Tensor]        # per shard: local token indices (ascending) that selected it
    send_counts: List[int]                 # rows sent to each rank
    recv_counts: List[int]                 # rows received from each rank
    counts: torch.Tensor                   # [world, 8] host int64: counts[src, shard]
    send_order: torch.Tensor               # local token index of every sent row, in send-buffer order
    send_shard: torch.Tensor               # shard of every sent row (same order)
    tokens_per_rank: List[int]             # T_local of every rank (same table on every rank)
    row_of: Optional[torch.Tensor] = None  # [T, 8] int32: position of (token, shard) in send order, -1 if absent


def build_plan(topk_idx: torch.Tensor, world: int, rank: int, group=None) -> DispatchPlan:
    """``topk_idx`` [T_local, 8] global expert ids of this rank's tokens.  One host synchronisation:
    the gathered [world, 9] table of per-shard counts and token counts."""
    dev = topk_idx.device
    T = topk_idx.shape[0]
    if dev.type == "cuda" and topk_idx.dtype == torch.int32 and topk_idx.is_contiguous():
        return _build_plan_device(topk_idx, world, rank, group)
    shard_of = (topk_idx.long() // E_LOCAL)                                   # [T, 8]
    hit = torch.zeros((T, N_SHARDS), dtype=torch.bool, device=dev)
    hit.scatter_(1, shard_of, True)
    # nonzero over the transposed mask gives (shard, token) pairs shard-major with ascending tokens
    pairs = torch.nonzero(hit.t().contiguous(), as_tuple=False)              # [n, 2]
    mine = torch.cat([hit.sum(dim=0, dtype=torch.int64), torch.tensor([T], dtype=torch.int64, device=dev)])
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(gathered, mine, group=group)
    else:
        gathered = [mine]
    table = torch.stack(gathered).cpu()                                       # [world, 9]
    counts = table[:, :N_SHARDS].contiguous()
    bounds = [0] + torch.cumsum(counts[rank], 0).tolist()
    token_lists = [pairs[bounds[s]:bounds[s + 1], 1] for s in range(N_SHARDS)]
    per = N_SHARDS // world
    send_counts = [int(counts[rank, d * per:(d + 1) * per].sum()) for d in range(world)]
    recv_counts = [int(counts[src, rank * per:(rank + 1) * per].sum()) for src in range(world)]
    return DispatchPlan(token_lists, send_counts, recv_counts, counts, pairs[:, 1].contiguous(),
                        pairs[:, 0].contiguous(), [int(x) for x in table[:, N_SHARDS]])


def _build_plan_device(topk_idx: torch.Tensor, world: int, rank: int, group=None) -> DispatchPlan:
    """``build_plan`` for a routing result on the GPU: one kernel (``moe_ep_plan``) makes the record order, the
    counts and the (token, shard) -> record table; the counts are gathered on the device and cross to the host
    once.  Same plan, element for element, as the tensor-operation path (compared in tests/test_gpu_ep.py)."""
    from . import loader
    dev = topk_idx.device
    T = topk_idx.shape[0]
    mine = torch.empty(N_SHARDS + 1, dtype=torch.int64, device=dev)
    order = torch.empty(max(1, N_SHARDS * T), dtype=torch.int64, device=dev)
    shard = torch.empty(max(1, N_SHARDS * T), dtype=torch.int64, device=dev)
    row_of = torch.empty((T, N_SHARDS), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        loader.check(loader.lib.moe_ep_plan(topk_idx.data_ptr(), int(T), mine.data_ptr(), order.data_ptr(),
                                            shard.data_ptr(), row_of.data_ptr(),
                                            torch.cuda.current_stream(dev).cuda_stream))
    if world > 1:
        table_dev = torch.empty((world, N_SHARDS + 1), dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(table_dev, mine, group=group)
    else:
        table_dev = mine.view(1, -1)
    table = table_dev.cpu()                                                   # the call's one host synchronisation
    counts = table[:, :N_SHARDS].contiguous()
    rows = table.tolist()
    own = rows[rank][:N_SHARDS]
    bounds = [0]
    for c in own:
        bounds.append(bounds[-1] + c)
    send_order, send_shard = order[:bounds[-1]], shard[:bounds[-1]]
    token_lists = [send_order[bounds[s]:bounds[s + 1]] for s in range(N_SHARDS)]
    per = N_SHARDS // world
    send_counts = [sum(own[d * per:(d + 1) * per]) for d in range(world)]
    recv_counts = [sum(rows[src][rank * per:(rank + 1) * per]) for src in range(world)]
    return DispatchPlan(token_lists, send_counts, recv_counts, counts, send_order, send_shard,
                        [rows[r][N_SHARDS] for r in range(world)], row_of)


def sum_shards(plan: DispatchPlan, back: torch.Tensor, T: int) -> torch.Tensor:
    """Layer output of this rank's tokens from the returned rows (send order: shard-major, ascending token):
    fp32 sum in ascending shard order, one bf16 rounding.  On a GPU this is one kernel
    (``moe_ep_sum_shards``); CPU tensors (the gloo tests of the host logic) take the same sum with torch."""
    dev = back.device
    if dev.type == "cuda":
        from . import loader
        row_of = plan.row_of
        if row_of is None:
            row_of = torch.full((T, N_SHARDS), -1, dtype=torch.int32, device=dev)
            n = int(plan.send_order.numel())
            if n:   # send order is shard-major: row i of `back` belongs to (send_order[i], send_shard[i])
                row_of[plan.send_order, plan.send_shard] = torch.arange(n, dtype=torch.int32, device=dev)
        out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        back = back.contiguous()
        with torch.cuda.device(dev):
            loader.check(loader.lib.moe_ep_sum_shards(back.data_ptr(), row_of.data_ptr(), int(T), out.data_ptr(),
                                                      torch.cuda.current_stream(dev).cuda_stream))
        return out
    acc = torch.zeros((T, H), dtype=torch.float32, device=dev)
    pos = 0
    for s in range(N_SHARDS):
        toks = plan.token_lists[s]
        n = int(toks.numel())
        if n:
            acc.index_add_(0, toks, back[pos:pos + n].to(torch.float32))
        pos += n
    return acc.to(torch.bfloat16)


def _all_to_all(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits, world: int, group=None):
    if world == 1:
        out.copy_(inp)
    else:
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)
    return out


class PeerExchange:
    """Symmetric receive areas of the p2p transport and their peer addresses.

    Layout (same on every rank): fp8 rows | block scales | logits for the records this rank
    receives, then the bf16 result rows that come back for the records it sent."""

    def __init__(self, rank: int, world: int, group, device, max_recv_rows: int, max_send_rows: int, n_logits: int):
        self.rank, self.world = rank, world
        al = lambda x: (x + 255) // 256 * 256
        self.off_h = 0
        self.off_s = al(max_recv_rows * H)
        self.off_l = self.off_s + al(max_recv_rows * KB * 4)
        self.off_back = self.off_l + al(max_recv_rows * n_logits * 4)
        total = self.off_back + al(max_send_rows * H * 2)
        self.max_recv_rows, self.max_send_rows, self.n_logits = max_recv_rows, max_send_rows, n_logits
        if world > 1:
            # plain peer stores only: keep torch from binding the buffer to an NVLink multicast object
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            self.buf = symm.empty(total, dtype=torch.uint8, device=device)
            grp = group if group is not None else dist.group.WORLD
            self.handle = symm.rendezvous(self.buf, group=grp.group_name)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        else:
            self.buf = torch.empty(total, dtype=torch.uint8, device=device)
            self.handle = None
            self.ptrs = [self.buf.data_ptr()]

    def barrier(self):
        if self.handle is not None:
            self.handle.barrier()

    def recv_views(self, n: int):
        h = self.buf[self.off_h:self.off_h + n * H].view(n, H)
        s = self.buf[self.off_s:self.off_s + n * KB * 4].view(torch.float32).view(n, KB)
        l = self.buf[self.off_l:self.off_l + n * self.n_logits * 4].view(torch.float32).view(n, self.n_logits)
        return h, s, l

    def back_view(self, n: int):
        return self.buf[self.off_back:self.off_back + n * H * 2].view(torch.bfloat16).view(n, H)


class ExpertParallelMoE:
    """The layer.  ``shard_weights[i]`` are the four weight tensors of the i-th shard this
    rank owns (``shards_of_rank(rank, world)`` order)."""

    def __init__(self, shard_weights: Sequence, rank: int = 0, world: int = 1, group=None,
                 local_op: Optional[Callable] = None, route_fn: Optional[Callable] = None, transport: str = "nccl"):
        if transport not in ("nccl", "p2p"):
            raise ValueError("transport must be 'nccl' or 'p2p'")
        self.transport = transport
        self._px: Optional[PeerExchange] = None
        self.rank, self.world, self.group = rank, world, group
        self.shards = shards_of_rank(rank, world)
        if len(shard_weights) != len(self.shards):
            raise ValueError(f"rank {rank} of {world} owns {len(self.shards)} shards, got {len(shard_weights)}")
        self.shard_weights = list(shard_weights)
        if local_op is None or route_fn is None:
            from . import op          # needs the compiled CUDA library; no fallback
            local_op = local_op or op.run
            route_fn = route_fn or (lambda lg, b, rsf: op.route(lg, b, 0, rsf)[0])
        self.local_op, self.route_fn = local_op, route_fn
        self.last_plan: Optional[DispatchPlan] = None
        self.last_shard_rows: List[int] = []       # records each owned shard processed in the last call

    def forward(self, routing_logits, routing_bias, hidden_states, hidden_states_scale,
                routed_scaling_factor: float) -> torch.Tensor:
        """Token-side tensors of THIS rank's tokens (definition layout, scales ``[56, T_local]``).
        Returns this rank's bf16 ``[T_local, 7168]`` output of the full 256-expert layer."""
        world, rank = self.world, self.rank
        T = routing_logits.shape[0]
        dev = hidden_states.device
        topk_idx = self.route_fn(routing_logits, routing_bias, routed_scaling_factor)
        plan = build_plan(topk_idx, world, rank, self.group)
        self.last_plan = plan
        if self.transport == "p2p":
            return self._forward_p2p(plan, routing_logits, routing_bias, hidden_states, hidden_states_scale,
                                     routed_scaling_factor)
        order = plan.send_order
        n_send, n_recv = int(order.numel()), sum(plan.recv_counts)

        # ---- dispatch: rows are grouped by destination rank, then shard, then ascending token
        hs_u8 = hidden_states.view(torch.uint8)
        send_h = hs_u8.index_select(0, order)
        send_s = hidden_states_scale.t().index_select(0, order).contiguous()          # [n, 56]
        send_l = routing_logits.index_select(0, order)
        recv_h = torch.empty((n_recv, H), dtype=torch.uint8, device=dev)
        recv_s = torch.empty((n_recv, KB), dtype=torch.float32, device=dev)
        recv_l = torch.empty((n_recv, routing_logits.shape[1]), dtype=torch.float32, device=dev)
        for out, inp in ((recv_h, send_h), (recv_s, send_s), (recv_l, send_l)):
            _all_to_all(out, inp, plan.recv_counts, plan.send_counts, world, self.group)

        # ---- local shard operator, once per owned shard, on the records of that shard
        per = N_SHARDS // world
        recv_out = torch.empty((n_recv, H), dtype=torch.bfloat16, device=dev)
        # received rows are ordered by source rank, then shard; segment (src, j) holds counts[src, shard_j] rows
        seg_start = {}
        pos = 0
        for src in range(world):
            for j, s in enumerate(self.shards):
                seg_start[(src, j)] = pos
                pos += int(plan.counts[src, s])
        self.last_shard_rows = []
        for j, s in enumerate(self.shards):
            segs = [(seg_start[(src, j)], int(plan.counts[src, s])) for src in range(world)]
            n_s = sum(n for _, n in segs)
            self.last_shard_rows.append(n_s)
            if n_s == 0:
                continue
            if per == 1:
                rows = slice(0, n_recv)
                h_s, sc_s, l_s = recv_h, recv_s, recv_l
            else:
                idx = torch.cat([torch.arange(a, a + n, device=dev) for a, n in segs])
                h_s, sc_s, l_s = recv_h.index_select(0, idx), recv_s.index_select(0, idx), recv_l.index_select(0, idx)
            out_s = torch.empty((n_s, H), dtype=torch.bfloat16, device=dev)
            w = self.shard_weights[j]
            self.local_op(l_s, routing_bias, h_s.view(torch.float8_e4m3fn), sc_s.t().contiguous(),
                          w.gemm1_weights, w.gemm1_weights_scale, w.gemm2_weights, w.gemm2_weights_scale,
                          E_LOCAL * s, routed_scaling_factor, out_s)
            if per == 1:
                recv_out = out_s
            else:
                recv_out.index_copy_(0, idx, out_s)

        # ---- combine: rows travel back along the same splits; ascending-shard fp32 accumulation
        back = torch.empty((n_send, H), dtype=torch.bfloat16, device=dev)
        _all_to_all(back, recv_out, plan.send_counts, plan.recv_counts, world, self.group)
        return sum_shards(plan, back, T)


def _forward_bf16(self, routing_logits, routing_bias, hidden_bf16, routed_scaling_factor: float) -> torch.Tensor:
    """The layer for activations that are still bf16 ``[T_local, 7168]``.  The p2p transport quantises every token
    inside the dispatch kernel (quantise + pack + send in one pass, ``moe_ep_quantize_push``); the nccl transport
    quantises first.  Bit-identical to ``forward`` on ``op.quantize_activations(hidden_bf16)``."""
    if hidden_bf16.dtype != torch.bfloat16 or hidden_bf16.dim() != 2 or hidden_bf16.shape[1] != H or \
            not hidden_bf16.is_contiguous():
        raise ValueError("hidden_bf16 must be a contiguous bfloat16 [T, 7168]")
    if self.transport != "p2p":
        from . import op
        q, sc = op.quantize_activations(hidden_bf16)
        return self.forward(routing_logits, routing_bias, q, sc, routed_scaling_factor)
    topk_idx = self.route_fn(routing_logits, routing_bias, routed_scaling_factor)
    plan = build_plan(topk_idx, self.world, self.rank, self.group)
    self.last_plan = plan
    return self._forward_p2p(plan, routing_logits, routing_bias, None, None, routed_scaling_factor,
                             hidden_bf16=hidden_bf16)


ExpertParallelMoE.forward_bf16 = _forward_bf16


def _forward_p2p(self, plan: DispatchPlan, routing_logits, routing_bias, hidden_states, hidden_states_scale,
                 routed_scaling_factor: float, hidden_bf16: Optional[torch.Tensor] = None) -> torch.Tensor:
    """p2p transport: dispatch by one push kernel, combine inside the shard operator (see module docstring).
    With ``hidden_bf16`` (and no fp8 tensors) the dispatch kernel quantises each token on its way out."""
    import ctypes

    from . import loader, op
    world, rank = self.world, self.rank
    T = routing_logits.shape[0]
    dev = routing_logits.device
    n_logits = routing_logits.shape[1]
    per = N_SHARDS // world
    # The count table as plain integers: the arithmetic below runs between the call's host synchronisation and
    # the launches that wait for it, where every tensor operation on a nine-element tensor costs microseconds.
    counts = plan.counts.tolist()                            # [world][8], identical on every rank
    totals = [sum(counts[r][s] for r in range(world)) for s in range(N_SHARDS)]   # records per shard
    # Capacity of the symmetric areas.  Every rank evaluates the SAME condition from the shared table (largest
    # receive and send count over all ranks), so either all ranks (re)allocate together -- the rendezvous is
    # collective -- or none does: no rank can fail alone in front of a barrier its peers are already waiting in.
    need_recv = max(sum(totals[d * per:(d + 1) * per]) for d in range(world))
    need_send = max(sum(counts[r]) for r in range(world))
    if self._px is None or need_recv > self._px.max_recv_rows or need_send > self._px.max_send_rows:
        t_max = max(plan.tokens_per_rank)
        cap_recv = max(1, need_recv, t_max * world * per if self._px is None else 2 * need_recv)
        cap_send = max(1, need_send, t_max * N_SHARDS if self._px is None else 2 * need_send)
        self._px = None                                     # release the old areas first
        self._px = PeerExchange(rank, world, self.group, dev, cap_recv, cap_send, n_logits)
    px = self._px
    n_send = sum(counts[rank])
    n_recv = sum(totals[s] for s in self.shards)

    def recv_row_base(d: int, s: int, src: int) -> int:
        """First row, in rank d's receive area, of the records that `src` sends for shard s (shard-major)."""
        first = d * per
        return sum(totals[first:s]) + sum(counts[r][s] for r in range(src))

    # No barrier is needed before the push.  The receive areas it overwrites were last read by the owners' shard
    # operators of the previous call, and every rank passed that call's exit barrier only after its own shard
    # operators (stream order); the back areas the shard operators of this call overwrite are read by the sources'
    # final sums of the previous call, which precede this call's entry barrier below in each source's stream.
    segs = (loader.EpSegment * N_SHARDS)()                   # the non-empty segments, packed
    by_shard = (loader.EpSegment * N_SHARDS)()               # the same, indexed by shard (count 0: none)
    nseg, first = 0, 0
    for s in range(N_SHARDS):
        n = counts[rank][s]
        if n:
            d = owner_of_shard(s, world)
            row = recv_row_base(d, s, rank)
            segs[nseg] = loader.EpSegment(first, n, px.ptrs[d] + px.off_h + row * H,
                                          px.ptrs[d] + px.off_s + row * KB * 4,
                                          px.ptrs[d] + px.off_l + row * n_logits * 4)
            by_shard[s] = segs[nseg]
            nseg += 1
        first += n
    if n_send:
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            if hidden_bf16 is not None:
                if plan.row_of is None:
                    raise ValueError("the bf16 dispatch needs the device-side plan (int32 routing result on the GPU)")
                loader.check(loader.lib.moe_ep_quantize_push(hidden_bf16.data_ptr(), routing_logits.data_ptr(), int(T),
                                                             plan.row_of.data_ptr(), by_shard, stream))
            else:
                loader.check(loader.lib.moe_ep_dispatch_push(
                    hidden_states.data_ptr(), hidden_states_scale.data_ptr(), routing_logits.data_ptr(), int(T),
                    plan.send_order.data_ptr(), n_send, segs, nseg, stream))
    # Destination of every result row, for all of this rank's shards at once (receive-area order: shard-major,
    # then source rank): the position of the row's record in the source rank's send order.  One small kernel
    # (moe_ep_row_pointers) from the eight (owned shard, source rank) runs.
    ptr_table = None
    if n_recv:
        seg_base, seg_cnt = [], []
        for s in self.shards:
            for src in range(world):
                seg_base.append(px.ptrs[src] + px.off_back + sum(counts[src][:s]) * H * 2)
                seg_cnt.append(counts[src][s])
        nseg = len(seg_base)
        base_arr = (ctypes.c_int64 * nseg)(*seg_base)
        cnt_arr = (ctypes.c_int64 * nseg)(*seg_cnt)
        ptr_table = torch.empty(n_recv, dtype=torch.int64, device=dev)
        with torch.cuda.device(dev):
            loader.check(loader.lib.moe_ep_row_pointers(base_arr, cnt_arr, nseg, H * 2, ptr_table.data_ptr(), n_recv,
                                                        torch.cuda.current_stream(dev).cuda_stream))
    px.barrier()                                            # every record has landed

    recv_h, recv_s, recv_l = px.recv_views(n_recv)
    row0 = 0
    self.last_shard_rows = []
    for j, s in enumerate(self.shards):
        n_s = totals[s]
        self.last_shard_rows.append(n_s)
        if n_s:
            rows = slice(row0, row0 + n_s)
            w = self.shard_weights[j]
            op.run_rows(recv_l[rows], routing_bias, recv_h[rows].view(torch.float8_e4m3fn),
                        recv_s[rows].t().contiguous(), w.gemm1_weights, w.gemm1_weights_scale, w.gemm2_weights,
                        w.gemm2_weights_scale, E_LOCAL * s, routed_scaling_factor, ptr_table[rows])
        row0 += n_s
    px.barrier()                                            # every result row has landed at its source

    back = px.back_view(n_send)
    return sum_shards(plan, back, T)


ExpertParallelMoE._forward_p2p = _forward_p2p


def layer_reference(shard_run: Callable[[int], torch.Tensor]) -> torch.Tensor:
    """The layer result the combine reproduces: the eight shard outputs (bf16, each from
    ``run`` with ``local_expert_offset = 32 s`` on ALL tokens) summed in fp32 in ascending shard order."""
    acc = None
    for s in range(N_SHARDS):
        o = shard_run(s).to(torch.float32)
        acc = o if acc is None else acc + o
    return acc.to(torch.bfloat16)
