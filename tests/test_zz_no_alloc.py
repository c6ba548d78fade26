"""GPU test of the allocation-free routing entry point
(moe_fp8_block_scale_route_static).

It is for callers that cannot get device memory when they need the routing
result, so the library keeps that stage's scratch in a fixed device array.  The
test calls it through the C ABI twice in a row on different batches (the array
is shared and keeps the previous call's contents) and checks every output
against what the regular entry point leaves in its caller-owned workspace for
the same inputs: integer results bit for bit, weights exactly (same kernel code).
The file name makes pytest collect it last."""
import pytest
import torch

import ws_readers

pytestmark = pytest.mark.gpu


def call_static(pkg, tok, T, offset, rsf, dev):
    topk_idx = torch.full((T, 8), -7, dtype=torch.int32, device=dev)
    topk_w = torch.full((T, 8), -7.0, dtype=torch.float32, device=dev)
    offs = torch.full((33,), -7, dtype=torch.int32, device=dev)
    perm_token = torch.full((8 * T,), -7, dtype=torch.int32, device=dev)
    perm_weight = torch.full((8 * T,), -7.0, dtype=torch.float32, device=dev)
    rc = pkg.loader.lib.moe_fp8_block_scale_route_static(
        tok.routing_logits.data_ptr(), tok.routing_bias.data_ptr(), T, offset, rsf, topk_idx.data_ptr(),
        topk_w.data_ptr(), offs.data_ptr(), perm_token.data_ptr(), perm_weight.data_ptr(),
        torch.cuda.current_stream().cuda_stream)
    assert rc == pkg.loader.OK
    torch.cuda.synchronize()
    return topk_idx.cpu(), topk_w.cpu(), offs.cpu(), perm_token.cpu(), perm_weight.cpu()


def test_static_routing_matches_workspace_entry_point(pkg):
    dev = torch.device("cuda", 0)
    W = pkg.gen.make_shard_weights(0, dev, experts=[])       # routing does not read the weights
    rsf = 2.5
    # big first: later calls see leftovers.  4096 is the entry point's limit (the whole fixed array), 32 and 1
    # take the single-CTA routing + permutation launch.
    batches = [(4096, 2, False, 0), (2500, 1, False, 32), (300, 0, True, 0), (37, 3, False, 64), (32, 6, True, 0),
               (1, 3, False, 0)]
    tokens = [pkg.gen.make_tokens(T, seed, dev, skew) for T, seed, skew, _ in batches]
    got = [call_static(pkg, tok, T, off, rsf, dev) for tok, (T, _, _, off) in zip(tokens, batches)]
    for tok, (T, _, _, off), (idx, w, offs, ptok, pw) in zip(tokens, batches, got):
        pkg.op.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                   W.gemm1_weights, W.gemm1_weights_scale, W.gemm2_weights, W.gemm2_weights_scale, off, rsf)
        assert pkg.op.kernel_status() == 0
        im = ws_readers.intermediates(pkg, T, stages=False)
        n = im["n_sel"]
        assert torch.equal(idx, im["topk_idx"])
        assert torch.equal(w, im["topk_w"])
        assert torch.equal(offs.long(), im["offs"].long()) and int(offs[32]) == n
        assert torch.equal(ptok[:n], im["perm_token"])
        assert torch.equal(pw[:n], im["perm_weight"])


def test_static_routing_rejects_oversized_batches(pkg):
    dev = torch.device("cuda", 0)
    lib = pkg.loader.lib
    T = pkg.loader.STATIC_MAX_TOKENS + 1
    buf = torch.zeros(16, device=dev)
    p = buf.data_ptr()
    assert lib.moe_fp8_block_scale_route_static(p, p, T, 0, 2.5, p, p, p, p, p, None) == pkg.loader.EINVAL
    assert lib.moe_fp8_block_scale_route_static(p, p, -1, 0, 2.5, p, p, p, p, p, None) == pkg.loader.EINVAL
