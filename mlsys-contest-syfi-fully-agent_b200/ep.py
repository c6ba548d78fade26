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
    token_lists = [torch.nonzero(hit[:, s], as_tuple=False).squeeze(1) for s in range(N_SHARDS)]
    my_counts = torch.tensor([t.numel() for t in token_lists], dtype=torch.int64, device=dev)
    gathered = [torch.zeros_like(my_counts) for _ in range(world)]
    if world > 1:
        dist.all_gather(gathered, my_counts, group=group)
    else:
        gathered = [my_counts]
    counts = torch.stack(gathered).cpu()                                      # [world, 8]
    per = N_SHARDS // world
    send_counts = [int(counts[rank, d * per:(d + 1) * per].sum()) for d in range(world)]
    recv_counts = [int(counts[src, rank * per:(rank + 1) * per].sum()) for src in range(world)]
    send_order = torch.cat(token_lists) if token_lists else torch.zeros(0, dtype=torch.int64, device=dev)
    return DispatchPlan(token_lists, send_counts, recv_counts, counts, send_order)


def _all_to_all(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits, world: int, group=None):
    if world == 1:
        out.copy_(inp)
    else:
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)
    return out


class ExpertParallelMoE:
    """The layer.  ``shard_weights[i]`` are the four weight tensors of the i-th shard this
    rank owns (``shards_of_rank(rank, world)`` order)."""

    def __init__(self, shard_weights: Sequence, rank: int = 0, world: int = 1, group=None,
                 local_op: Optional[Callable] = None, route_fn: Optional[Callable] = None):
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
        acc = torch.zeros((T, H), dtype=torch.float32, device=dev)
        pos = 0
        for s in range(N_SHARDS):
            toks = plan.token_lists[s]
            n = int(toks.numel())
            if n:
                acc.index_add_(0, toks, back[pos:pos + n].to(torch.float32))
            pos += n
        return acc.to(torch.bfloat16)


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
    layer = ExpertParallelMoE(weights, rank, world)

    def step():
        return layer.forward(logits, bias, hidden, hscale, rsf)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

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
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        rows_max = n_rows.clone()
        dist.all_reduce(rows_max, op=dist.ReduceOp.MAX)
        dist.all_reduce(n_rows, op=dist.ReduceOp.SUM)
    else:
        rows_max = n_rows
    launches = loader.launch_count() - l0
    assert op.kernel_status(device=dev) == 0
    if rank == 0:
        ms_step = float(ms) / args.steps
        total_rows = float(n_rows)
        print(json.dumps({
            "metric": "moe_tokens_per_second", "value": T_total / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3",
            "data": "synthetic",
            "config": {"workload": "ep_layer_t16384", "T": T_total, "tokens_per_rank": T, "experts": 256,
                       "shards_per_rank": len(shards), "token_seed": 0, "weight_seeds": "1000 + shard",
                       "dispatch": "NCCL all_to_all_single (fp8 row + scales + logits per (token, shard))",
                       "combine": "NCCL all_to_all_single (bf16 row per (token, shard))",
                       "l2": "per-rank weights (>= 1.4 GB) exceed L2", "records_total": total_rows,
                       "load_balance_bound": total_rows / world / float(rows_max)},
            "gpu_launches": int(launches),
            "e2e": None, "roofline": None, "cpu_baseline": None,
            "fp8_tflops_per_gpu": None,
        }))
    if world > 1:
        dist.destroy_process_group()
