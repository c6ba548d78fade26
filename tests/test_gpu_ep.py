"""GPU tests of the expert-parallel layer with the real CUDA shard operator.

World size 1 (eight shards on one GPU) against the layer reference built from the
oracle: the eight shard outputs summed in fp32 in ascending shard order.  With two
or more GPUs the same comparison runs as NCCL ranks in child processes."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import moe_oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RSF = 2.5
T_TOTAL = 64


def _layer_case(pkg, rank, world, dev, transport="nccl"):
    ep, gen = pkg.ep, pkg.gen
    torch.backends.cuda.matmul.allow_tf32 = False
    tok = gen.make_tokens(T_TOTAL, 0, dev)
    shards = ep.shards_of_rank(rank, world)
    weights = {s: gen.make_shard_weights(1000 + s, dev) for s in shards}
    layer = ep.ExpertParallelMoE([weights[s] for s in shards], rank, world, transport=transport)
    T = T_TOTAL // world
    sl = slice(rank * T, (rank + 1) * T)
    out = layer.forward(tok.routing_logits[sl].contiguous(), tok.routing_bias, tok.hidden_states[sl].contiguous(),
                        tok.hidden_states_scale[:, sl].contiguous(), RSF)
    assert pkg.op.kernel_status(device=dev) == 0
    # layer reference for THIS rank's tokens needs every shard's output: ranks exchange nothing here, each
    # builds the shards it owns on all tokens and the partial sums are reduced in fp64 for the check
    part = torch.zeros(T_TOTAL, 7168, dtype=torch.float64, device=dev)
    for s in shards:
        w = weights[s]
        r = moe_oracle.run_full(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                                w.gemm1_weights, w.gemm1_weights_scale, w.gemm2_weights, w.gemm2_weights_scale,
                                32 * s, RSF)
        part += r.output.to(torch.float64)          # bf16 shard outputs, as the layer reference sums them
    if world > 1:
        dist.all_reduce(part)
    ref = part[sl].to(torch.float32)
    m = moe_oracle.output_metrics(out, ref.to(torch.bfloat16), ref)
    # routing plan: records == number of (token, shard) pairs
    idx, _ = moe_oracle.routing(tok.routing_logits[sl], tok.routing_bias, RSF)
    want = sum(len(set((r // 32).tolist())) for r in idx.cpu())
    assert sum(layer.last_plan.send_counts) == want
    m["digest"] = pkg.gen.digest(out)
    return m


@pytest.mark.parametrize("T", [1, 7, 64, 1000, 2048, 5000])
def test_plan_kernel_matches_tensor_operation_plan(pkg, T):
    """moe_ep_plan (one kernel, no host stop before the count table) against the torch.nonzero construction:
    the same records in the same order, the same counts, and row_of consistent with them."""
    ep, gen, op = pkg.ep, pkg.gen, pkg.op
    dev = torch.device("cuda", 0)
    tok = gen.make_tokens(T, 40 + T, dev, skew=(T % 2 == 0))
    topk = op.route(tok.routing_logits, tok.routing_bias, 0, RSF)[0]
    assert topk.dtype == torch.int32
    fast = ep.build_plan(topk, 1, 0)
    slow = ep.build_plan(topk.long(), 1, 0)          # int64 indices take the tensor-operation path
    assert fast.row_of is not None and slow.row_of is None
    assert torch.equal(fast.counts, slow.counts) and fast.tokens_per_rank == slow.tokens_per_rank == [T]
    assert fast.send_counts == slow.send_counts and fast.recv_counts == slow.recv_counts
    assert torch.equal(fast.send_order, slow.send_order) and torch.equal(fast.send_shard, slow.send_shard)
    for a, b in zip(fast.token_lists, slow.token_lists):
        assert torch.equal(a, b)
    n = int(fast.send_order.numel())
    want = torch.full((T, 8), -1, dtype=torch.int32, device=dev)
    want[slow.send_order, slow.send_shard] = torch.arange(n, dtype=torch.int32, device=dev)
    assert torch.equal(fast.row_of, want)


def test_bf16_dispatch_quantises_on_the_way_out(pkg):
    """forward_bf16 (quantise + pack + send in one kernel) against forward on separately quantised activations:
    the same bits, on batches where tokens go to between one and several shards and some shards get nothing."""
    ep, gen, op = pkg.ep, pkg.gen, pkg.op
    dev = torch.device("cuda", 0)
    weights = [gen.make_shard_weights(1000 + s, dev, experts=range(0, 32, 5)) for s in range(8)]
    layer = ep.ExpertParallelMoE(weights, 0, 1, transport="p2p")
    for T, seed, skew in ((1, 3, False), (33, 4, True), (700, 5, False)):
        tok = gen.make_tokens(T, seed, dev, skew)
        x = (gen.normal(seed, 77, 0, T * 7168, dev).view(T, 7168) * 3.0).to(torch.bfloat16).contiguous()
        q, sc = op.quantize_activations(x)
        want = layer.forward(tok.routing_logits, tok.routing_bias, q, sc, RSF)
        got = layer.forward_bf16(tok.routing_logits, tok.routing_bias, x, RSF)
        assert op.kernel_status(device=dev) == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), T
        assert float(want.float().abs().max()) > 0.0
    with pytest.raises(ValueError):
        layer.forward_bf16(tok.routing_logits, tok.routing_bias, x.float(), RSF)


def _check(m):
    assert m["cosine"] >= 0.9999, m
    # each shard output is already within the operator's bar; the layer adds <= 4 of them
    assert m["max_abs_vs_f32_over_rms"] <= 4e-2, m


def test_layer_on_one_gpu(pkg):
    dev = torch.device("cuda", 0)
    a = _layer_case(pkg, 0, 1, dev)
    _check(a)
    b = _layer_case(pkg, 0, 1, dev, transport="p2p")      # world size 1: the push / row-pointer kernels, local memory
    assert a["digest"] == b["digest"], "p2p transport differs from the NCCL transport"


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from __graft_entry__ import load_package
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    try:
        a = _layer_case(load_package(), rank, world, dev)
        b = _layer_case(load_package(), rank, world, dev, transport="p2p")
        a["p2p_same_bits"] = a["digest"] == b["digest"]
        ret[rank] = a
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_layer_on_two_gpus():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    for r in range(2):
        _check(ret[r])
        assert ret[r]["p2p_same_bits"], "peer-memory transport differs from the NCCL transport"
