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
at the symmetric-memory barrier.  Plain peer stores only: no multicast, no TMA on peer memory,
and no kernel ever waits on a peer.

``local_op`` and ``route_fn`` are injectable so that the host-side logic can be
tested with gloo on CPU ranks; the defaults are the CUDA operator and fail loudly
without the compiled library.
"""
from __future__ import annotations

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


def build_plan(topk_idx: torch.Tensor, world: int, rank: int, group=None) -> DispatchPlan:
    """``topk_idx`` [T_local, 8] global expert ids of this rank's tokens."""
    dev = topk_idx.device
    shard_of = (topk_idx.long() // E_LOCAL)                                   # [T, 8]
    hit = torch.zeros((topk_idx.shape[0], N_SHARDS), dtype=torch.bool, device=dev)
    hit.scatter_(1, shard_of, True)
    # one nonzero over the transposed mask gives (shard, token) pairs shard-major with ascending tokens:
    # a single host synchronisation instead of one per shard
    pairs = torch.nonzero(hit.t().contiguous(), as_tuple=False)              # [n, 2]
    my_counts = hit.sum(dim=0, dtype=torch.int64)
    bounds = [0] + torch.cumsum(my_counts, 0).tolist()
    token_lists = [pairs[bounds[s]:bounds[s + 1], 1] for s in range(N_SHARDS)]
    gathered = [torch.zeros_like(my_counts) for _ in range(world)]
    if world > 1:
        dist.all_gather(gathered, my_counts, group=group)
    else:
        gathered = [my_counts]
    counts = torch.stack(gathered).cpu()                                      # [world, 8]
    per = N_SHARDS // world
    send_counts = [int(counts[rank, d * per:(d + 1) * per].sum()) for d in range(world)]
    recv_counts = [int(counts[src, rank * per:(rank + 1) * per].sum()) for src in range(world)]
    send_order = pairs[:, 1].contiguous()
    return DispatchPlan(token_lists, send_counts, recv_counts, counts, send_order)


def sum_shards(plan: DispatchPlan, back: torch.Tensor, T: int) -> torch.Tensor:
    """Layer output of this rank's tokens from the returned rows (send order: shard-major, ascending token):
    fp32 sum in ascending shard order, one bf16 rounding.  On a GPU this is one kernel
    (``moe_ep_sum_shards``); CPU tensors (the gloo tests of the host logic) take the same sum with torch."""
    dev = back.device
    if dev.type == "cuda":
        from . import loader
        row_of = torch.full((T, N_SHARDS), -1, dtype=torch.int32, device=dev)
        pos = 0
        for s in range(N_SHARDS):
            toks = plan.token_lists[s]
            n = int(toks.numel())
            if n:
                row_of[toks, s] = torch.arange(pos, pos + n, dtype=torch.int32, device=dev)
            pos += n
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
        for j, s in enumerate(self.shards):
            segs = [(seg_start[(src, j)], int(plan.counts[src, s])) for src in range(world)]
            n_s = sum(n for _, n in segs)
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


def _forward_p2p(self, plan: DispatchPlan, routing_logits, routing_bias, hidden_states, hidden_states_scale,
                 routed_scaling_factor: float) -> torch.Tensor:
    """p2p transport: dispatch by one push kernel, combine inside the shard operator (see module docstring)."""
    import ctypes

    from . import loader, op
    world, rank = self.world, self.rank
    T = routing_logits.shape[0]
    dev = hidden_states.device
    n_logits = routing_logits.shape[1]
    per = N_SHARDS // world
    if self._px is None:
        # capacities for equal token counts per rank: every token of every rank may select each of my shards
        self._px = PeerExchange(rank, world, self.group, dev, max(1, T * world * per), max(1, T * N_SHARDS), n_logits)
    px = self._px
    counts = plan.counts                                    # [world, 8] host
    totals = counts.sum(dim=0)                              # records per shard over all sources
    n_send = int(counts[rank].sum())
    n_recv = int(sum(int(totals[s]) for s in self.shards))
    if n_recv > px.max_recv_rows or n_send > px.max_send_rows:
        raise RuntimeError("symmetric receive area too small for this batch")

    def recv_row_base(d: int, s: int, src: int) -> int:
        """First row, in rank d's receive area, of the records that `src` sends for shard s (shard-major)."""
        first = d * per
        return int(totals[first:s].sum()) + int(counts[:src, s].sum())

    px.barrier()                                            # peers have finished reading the previous call's areas
    segs = (loader.EpSegment * N_SHARDS)()
    nseg, first = 0, 0
    for s in range(N_SHARDS):
        n = int(counts[rank, s])
        if n:
            d = owner_of_shard(s, world)
            row = recv_row_base(d, s, rank)
            segs[nseg] = loader.EpSegment(first, n, px.ptrs[d] + px.off_h + row * H,
                                          px.ptrs[d] + px.off_s + row * KB * 4,
                                          px.ptrs[d] + px.off_l + row * n_logits * 4)
            nseg += 1
        first += n
    if n_send:
        with torch.cuda.device(dev):
            loader.check(loader.lib.moe_ep_dispatch_push(
                hidden_states.data_ptr(), hidden_states_scale.data_ptr(), routing_logits.data_ptr(), int(T),
                plan.send_order.data_ptr(), n_send, segs, nseg, torch.cuda.current_stream(dev).cuda_stream))
    px.barrier()                                            # every record has landed

    recv_h, recv_s, recv_l = px.recv_views(n_recv)
    row0 = 0
    for j, s in enumerate(self.shards):
        n_s = int(totals[s])
        if n_s:
            rows = slice(row0, row0 + n_s)
            # destination of every result row: the position of its record in the source rank's send order
            ptrs = []
            for src in range(world):
                n = int(counts[src, s])
                if n:
                    base = px.ptrs[src] + px.off_back + int(counts[src, :s].sum()) * H * 2
                    ptrs.append(base + torch.arange(n, device=dev, dtype=torch.int64) * (H * 2))
            w = self.shard_weights[j]
            op.run_rows(recv_l[rows], routing_bias, recv_h[rows].view(torch.float8_e4m3fn),
                        recv_s[rows].t().contiguous(), w.gemm1_weights, w.gemm1_weights_scale, w.gemm2_weights,
                        w.gemm2_weights_scale, E_LOCAL * s, routed_scaling_factor, torch.cat(ptrs))
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


# ---------------------------------------------------------------------------------------------
# bench.py --gpus N (N > 1), one rank per GPU under torchrun
# ---------------------------------------------------------------------------------------------
def bench_main(args):
    import json
    import os

    from . import gen, loader, op

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    T_total = 16384
    T = T_total // world
    rsf = gen.ROUTED_SCALING_FACTOR
    shards = shards_of_rank(rank, world)
    weights = [gen.make_shard_weights(1000 + s, dev) for s in shards]
    tok_all = gen.make_tokens(T_total, 0, dev)
    sl = slice(rank * T, (rank + 1) * T)
    logits = tok_all.routing_logits[sl].contiguous()
    hidden = tok_all.hidden_states[sl].contiguous()
    hscale = tok_all.hidden_states_scale[:, sl].contiguous()
    bias = tok_all.routing_bias
    del tok_all
    transports = [os.environ.get("MOE_B200_EP_TRANSPORT", "p2p")]
    if transports[0] == "p2p":
        transports.append("nccl")          # also timed, reported beside the headline

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    results = {}
    for tr in transports:
        layer = ExpertParallelMoE(weights, rank, world, transport=tr)

        def step():
            return layer.forward(logits, bias, hidden, hscale, rsf)

        for _ in range(max(args.warmup, 3)):
            step()
        sync()
        l0 = loader.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out = step()
        e1.record()
        sync()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        n_rows = torch.tensor([float(sum(layer.last_plan.recv_counts))], device=dev)
        rows_max = n_rows.clone()
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.all_reduce(rows_max, op=dist.ReduceOp.MAX)
            dist.all_reduce(n_rows, op=dist.ReduceOp.SUM)
        results[tr] = dict(ms_step=float(ms) / args.steps, launches=loader.launch_count() - l0,
                           rows=float(n_rows), rows_max=float(rows_max), digest=gen.digest(out))
        del layer
    # ---- the same layer call from host buffers: this rank's token tensors come from pinned host memory
    # and its output rows go back to pinned host memory inside the timed region
    layer = ExpertParallelMoE(weights, rank, world, transport=transports[0])
    pin = lambda t: t.cpu().pin_memory()
    h_in = [pin(logits), pin(bias), pin(hidden.view(torch.uint8)), pin(hscale)]
    d_in = [torch.empty_like(logits), torch.empty_like(bias), torch.empty_like(hidden.view(torch.uint8)),
            torch.empty_like(hscale)]
    h_out = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()

    def step_host():
        for d, h in zip(d_in, h_in):
            d.copy_(h, non_blocking=True)
        o = layer.forward(d_in[0], d_in[1], d_in[2].view(torch.float8_e4m3fn), d_in[3], rsf)
        h_out.copy_(o, non_blocking=True)

    for _ in range(3):
        step_host()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_host()
    e1.record()
    sync()
    ms_host = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms_host, op=dist.ReduceOp.MAX)
    ms_host = float(ms_host) / args.steps
    h2d = sum(t.numel() * t.element_size() for t in h_in)
    d2h = h_out.numel() * h_out.element_size()
    del layer
    assert op.kernel_status(device=dev) == 0
    if len(results) == 2:
        assert results["p2p"]["digest"] == results["nccl"]["digest"], "transports disagree"
    if rank == 0:
        head = results[transports[0]]
        ms_step, total_rows, rows_max = head["ms_step"], head["rows"], head["rows_max"]
        print(json.dumps({
            "metric": "moe_tokens_per_second", "value": T_total / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3",
            "data": "synthetic",
            "config": {"workload": "ep_layer_t16384", "T": T_total, "tokens_per_rank": T, "experts": 256,
                       "shards_per_rank": len(shards), "token_seed": 0, "weight_seeds": "1000 + shard",
                       "transport": transports[0],
                       "dispatch": "one push kernel into the owner's symmetric receive area over NVLink "
                                   "(fp8 row + scales + logits per (token, shard))" if transports[0] == "p2p"
                                   else "NCCL all_to_all_single",
                       "combine": "written by the shard operator's last kernel into the source rank's receive area "
                                  "(bf16 row per (token, shard))" if transports[0] == "p2p" else "NCCL all_to_all_single",
                       "l2": "per-rank weights (>= 1.4 GB) exceed L2", "records_total": total_rows,
                       "load_balance_bound": total_rows / world / rows_max},
            "gpu_launches": int(head["launches"]),
            "nccl_transport": ({"ms_per_step": results["nccl"]["ms_step"],
                                "tokens_per_s": T_total / (results["nccl"]["ms_step"] * 1e-3)}
                               if "nccl" in results and transports[0] != "nccl" else None),
            "fp8_tflops_per_gpu": total_rows and (T_total * 8 * 88080384 / world) / (ms_step * 1e-3) / 1e12,
            "e2e": {"value": T_total / (ms_host * 1e-3), "unit": "tokens/s", "ms_per_step": ms_host,
                    "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                    "note": "every rank copies its token tensors from pinned host memory and its output rows back"},
            "roofline": None, "cpu_baseline": None,
        }))
    if world > 1:
        dist.destroy_process_group()
