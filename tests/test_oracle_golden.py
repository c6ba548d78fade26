"""CPU tests: the restated oracle and the seeded generators against the golden
fixtures produced from the unmodified reference definition
(tests/golden/make_golden.py).  No GPU, no compiled library needed."""
import json
import os

import numpy as np
import pytest
import torch

import moe_oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = ["cpu_ref_t8", "decode_t1", "skew_t64", "offset64_t8", "ragged_t37", "prefill_t4096"]


def load_case(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    return meta, z


@pytest.fixture(scope="module")
def lazy_weights(pkg):
    return pkg.gen.LazyShardWeights(0, "cpu")


@pytest.mark.parametrize("name", CASES)
def test_generator_reproduces_token_inputs(pkg, name):
    """The counter-based generator gives the bytes the fixtures were made from."""
    meta, _ = load_case(name)
    tok = pkg.gen.make_tokens(meta["T"], meta["token_seed"], "cpu", meta["skew"])
    assert pkg.gen.digest(tok.routing_logits, tok.routing_bias, tok.hidden_states,
                          tok.hidden_states_scale) == meta["tokens_digest"]
    assert tok.hidden_states_scale.shape == (56, meta["T"])


def test_generator_reproduces_expert_weights(pkg, lazy_weights):
    meta, _ = load_case("cpu_ref_t8")
    assert pkg.gen.digest(*lazy_weights.expert(0)) == meta["weights_digest"]["w_expert0"]


@pytest.mark.parametrize("name", CASES)
def test_oracle_routing_and_permutation_match_reference(pkg, name):
    """Selection sets, histogram, offsets and the canonical permutation, bit for bit."""
    meta, z = load_case(name)
    tok = pkg.gen.make_tokens(meta["T"], meta["token_seed"], "cpu", meta["skew"])
    idx, weights = moe_oracle.routing(tok.routing_logits, tok.routing_bias, meta["routed_scaling_factor"])
    assert np.array_equal(torch.sort(idx, dim=1).values.numpy().astype(np.int16), z["topk_sorted"])
    off = meta["local_expert_offset"]
    counts = np.zeros(32, dtype=np.int32)
    perm_token, perm_weight = [], []
    for le in range(32):
        sel = (idx == off + le).any(dim=1)
        toks = torch.nonzero(sel).squeeze(1)
        counts[le] = toks.numel()
        perm_token.append(toks)
        perm_weight.append(weights[toks, off + le])
    assert np.array_equal(counts, z["counts"])
    assert np.array_equal(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32), z["offsets"])
    assert np.array_equal(torch.cat(perm_token).numpy().astype(np.int32), z["perm_token"])
    assert np.array_equal(torch.cat(perm_weight).numpy(), z["perm_weight"])
    assert int(counts.sum()) == meta["n_sel"]


@pytest.mark.parametrize("name", ["cpu_ref_t8", "decode_t1"])
def test_oracle_output_bit_identical_to_reference(pkg, lazy_weights, name):
    """Full operator on the experts the batch uses: the bf16 output equals the
    reference definition's, bit for bit."""
    meta, z = load_case(name)
    tok = pkg.gen.make_tokens(meta["T"], meta["token_seed"], "cpu", meta["skew"])
    res = moe_oracle.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                         lazy_weights.expert, meta["local_expert_offset"], meta["routed_scaling_factor"])
    got = res.output.view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got[z["rows"]], z["out_bf16"])
    assert pkg.gen.digest(res.output) == meta["out_digest"]
    assert np.array_equal(res.output_f32.numpy()[z["rows"]], z["out_f32"])


def test_oracle_empty_and_degenerate_inputs(pkg, lazy_weights):
    """T = 0 and a token with no local expert (seed 0, T = 1) give empty / zero outputs."""
    tok = pkg.gen.make_tokens(1, 0, "cpu")
    res = moe_oracle.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                         lazy_weights.expert, 0, 2.5)
    assert int(res.counts.sum()) == 0 and float(res.output_f32.abs().max()) == 0.0
    tok0 = pkg.gen.make_tokens(0, 0, "cpu")
    res0 = moe_oracle.run(tok0.routing_logits, tok0.routing_bias, tok0.hidden_states, tok0.hidden_states_scale,
                          lazy_weights.expert, 0, 2.5)
    assert res0.output.shape == (0, 7168)


def test_routing_invariants(pkg):
    """Properties of the definition's routing that hold for any input: 8 distinct
    experts from exactly 4 groups, weights sum to the scaling factor."""
    tok = pkg.gen.make_tokens(257, 11, "cpu")
    idx, w = moe_oracle.routing(tok.routing_logits, tok.routing_bias, 2.5)
    assert all(len(set(r.tolist())) == 8 for r in idx)
    assert all(len(set((r // 32).tolist())) <= 4 for r in idx)
    assert torch.allclose(w.sum(dim=1), torch.full((257,), 2.5), rtol=1e-5)
    assert int((w > 0).sum()) == 257 * 8


def test_metrics_census():
    a = torch.tensor([1.0, 2.0, -3.0, 0.0], dtype=torch.bfloat16)
    b = a.clone()
    b[0] = torch.tensor(1.0078125, dtype=torch.bfloat16)      # one bf16 step above 1.0
    m = moe_oracle.output_metrics(b, a)
    assert m["n_diff"] == 1 and m["n_one_step"] == 1 and m["n_multi_step"] == 0
    assert abs(m["max_abs"] - 0.0078125) < 1e-9
