"""CPU tests of the expert-parallel layer's host logic with gloo ranks (world size 2, 4 and 8):
dispatch lists, count exchange, all-to-all plumbing and the ascending-shard combine.
The shard operator is replaced by a cheap per-token stand-in with the operator's
signature (the real one needs a GPU); routing is the oracle's."""
import os
import socket
import sys
import types

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RSF = 2.5


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def fake_shard_op(logits, bias, hidden, hscale, w1, s1, w2, s2, offset, rsf, out):
    """out[t] = (sum over the token's experts in [offset, offset+32) of weight * (expert + 1)) * dequant(hidden[t])."""
    import moe_oracle
    idx, w = moe_oracle.routing(logits, bias, rsf)
    T = logits.shape[0]
    e = torch.arange(256, dtype=torch.float32)
    local = ((e >= offset) & (e < offset + 32)).float()
    coef = (w * local * (e + 1.0)).sum(dim=1)                                  # [T]
    x = hidden.to(torch.float32).view(T, 56, 128) * hscale.t().unsqueeze(2)
    out.copy_((coef[:, None] * x.view(T, 7168) * w1.tag).to(torch.bfloat16))
    return out


def _worker(rank, world, port, T_total, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import moe_oracle
    from __graft_entry__ import load_package
    pkg = load_package()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        tok = pkg.gen.make_tokens(T_total, 5, "cpu")
        mk = lambda s: types.SimpleNamespace(gemm1_weights=types.SimpleNamespace(tag=1.0 + s),
                                             gemm1_weights_scale=None, gemm2_weights=None, gemm2_weights_scale=None)
        ep = pkg.ep
        shards = ep.shards_of_rank(rank, world)
        layer = ep.ExpertParallelMoE([mk(s) for s in shards], rank, world, local_op=fake_shard_op,
                                     route_fn=lambda lg, b, rsf: moe_oracle.routing(lg, b, rsf)[0].to(torch.int32))
        T = T_total // world
        sl = slice(rank * T, (rank + 1) * T)
        out = layer.forward(tok.routing_logits[sl].contiguous(), tok.routing_bias, tok.hidden_states[sl].contiguous(),
                            tok.hidden_states_scale[:, sl].contiguous(), RSF)

        def shard_run(s):
            o = torch.empty(T_total, 7168, dtype=torch.bfloat16)
            w = mk(s)
            return fake_shard_op(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                                 w.gemm1_weights, None, None, None, 32 * s, RSF, o)
        ref = ep.layer_reference(shard_run)[sl]
        plan = layer.last_plan
        ok = torch.equal(out.view(torch.int16), ref.view(torch.int16))
        # every token reaches exactly the shards its eight experts live in
        idx, _ = moe_oracle.routing(tok.routing_logits[sl], tok.routing_bias, RSF)
        want_rows = sum(len(set((r // 32).tolist())) for r in idx)
        ok = ok and sum(plan.send_counts) == want_rows
        ok = ok and int(plan.counts[rank].sum()) == want_rows
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_layer_matches_single_process_reference(world):
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, 32, ret), nprocs=world, join=True)
    assert all(ret.get(r, False) for r in range(world)), dict(ret)


def test_shard_ownership():
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    ep = load_package().ep
    for world in (1, 2, 4, 8):
        owned = [s for r in range(world) for s in ep.shards_of_rank(r, world)]
        assert owned == list(range(8))
        assert all(ep.owner_of_shard(s, world) == s // (8 // world) for s in range(8))
    with pytest.raises(ValueError):
        ep.shards_of_rank(0, 3)
