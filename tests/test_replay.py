"""Trace-set replay adapter: reading the flashinfer-trace layout, building a workload's inputs,
the aggregate the reference's pipeline computes (full-agent-pipeline/run_pipeline.py:364-399), and, on a
GPU, a replay of a small stand-in set with the oracle as the checker."""
import json
import os

import pytest
import torch


def _no_weights(pkg):
    return pkg.gen.make_shard_weights(0, "cpu", experts=[])


def test_written_set_reads_back(pkg, tmp_path):
    rp = pkg.replay
    written = rp.write_synthetic_trace(str(tmp_path), [1, 7, 0, 130], seed=3)
    d = rp.read_definition(str(tmp_path))
    assert d["name"] == rp.DEFINITION and list(d["inputs"]) == list(rp.INPUT_ORDER)
    assert d["inputs"]["hidden_states_scale"]["shape"] == ["num_hidden_blocks", "seq_len"]
    got = rp.read_workloads(str(tmp_path))
    assert [w.uuid for w in got] == [w.uuid for w in written] and [w.seq_len for w in got] == [1, 7, 0, 130]
    assert len({w.uuid for w in got}) == 4
    # the same arguments give the same uuids; another seed gives others
    again = rp.write_synthetic_trace(str(tmp_path / "again"), [1, 7, 0, 130], seed=3)
    other = rp.write_synthetic_trace(str(tmp_path / "other"), [1, 7, 0, 130], seed=4)
    assert [w.uuid for w in again] == [w.uuid for w in written]
    assert not {w.uuid for w in other} & {w.uuid for w in written}
    # one trace object per line with the harness's four keys
    path = tmp_path / "workloads" / rp.OP_TYPE / (rp.DEFINITION + ".jsonl")
    for line in open(path):
        obj = json.loads(line)
        assert set(obj) == {"definition", "solution", "workload", "evaluation"}
        assert obj["workload"]["inputs"]["routing_logits"]["type"] == "safetensors"
        assert obj["workload"]["inputs"]["hidden_states"] == {"type": "random"}
        assert obj["workload"]["inputs"]["local_expert_offset"] == {"type": "scalar", "value": 0}


def test_materialise_shapes_sources_and_determinism(pkg, tmp_path):
    rp = pkg.replay
    wls = rp.write_synthetic_trace(str(tmp_path), [7, 0], routed_scaling_factor=1.5)
    W = _no_weights(pkg)
    a = rp.materialise(wls[0], str(tmp_path), "cpu", weights=W)
    b = rp.materialise(wls[0], str(tmp_path), "cpu", weights=W)
    assert list(a) == list(rp.INPUT_ORDER)
    for name in rp.TOKEN_INPUTS + rp.WEIGHT_INPUTS:
        assert tuple(a[name].shape) == rp.expected_shape(name, 7), name
        assert torch.equal(a[name].view(torch.uint8), b[name].view(torch.uint8)), name
    assert a["local_expert_offset"] == 0 and a["routed_scaling_factor"] == 1.5
    assert a["gemm1_weights"] is W.gemm1_weights
    # stored tensors come from the file, generated ones from the uuid-seeded generator
    from safetensors.torch import load_file
    stored = load_file(str(tmp_path / wls[0].inputs["routing_logits"]["path"]))
    assert torch.equal(a["routing_logits"], stored["routing_logits"])
    tok = pkg.gen.make_tokens(7, rp.uuid_seed(wls[0].uuid), "cpu")
    assert torch.equal(a["hidden_states"].view(torch.uint8), tok.hidden_states.view(torch.uint8))
    assert not torch.equal(a["routing_logits"], tok.routing_logits)
    empty = rp.materialise(wls[1], str(tmp_path), "cpu", weights=W)
    assert empty["routing_logits"].shape == (0, 256) and empty["hidden_states_scale"].shape == (56, 0)


def _write_lines(root, lines, pkg):
    d = os.path.join(root, "workloads", pkg.replay.OP_TYPE)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "w.jsonl"), "w") as f:
        for obj in lines:
            f.write((obj if isinstance(obj, str) else json.dumps(obj)) + "\n")


def test_malformed_sets_are_refused(pkg, tmp_path):
    rp = pkg.replay
    wl = lambda **kw: {"definition": rp.DEFINITION, "workload": dict({"uuid": "u1", "axes": {"seq_len": 4}, "inputs": {}}, **kw)}
    cases = {
        "unknown_input": [wl(inputs={"gate": {"type": "random"}})],
        "unknown_type": [wl(inputs={"routing_logits": {"type": "zeros"}})],
        "scalar_without_value": [wl(inputs={"local_expert_offset": {"type": "scalar"}})],
        "safetensors_without_key": [wl(inputs={"routing_logits": {"type": "safetensors", "path": "x"}})],
        "no_seq_len": [wl(axes={"batch": 4})],
        "duplicate_uuid": [wl(), wl()],
        "not_json": ["{not json"],
    }
    for name, lines in cases.items():
        root = str(tmp_path / name)
        _write_lines(root, lines, pkg)
        with pytest.raises(rp.TraceError):
            rp.read_workloads(root)
    with pytest.raises(rp.TraceError):
        rp.read_workloads(str(tmp_path / "absent"))
    # other definitions' workloads in the same set are skipped, not refused
    root = str(tmp_path / "mixed")
    _write_lines(root, [{"definition": "gdn_decode", "workload": {"uuid": "x", "axes": {"batch": 1}}}, wl()], pkg)
    assert [w.uuid for w in rp.read_workloads(root)] == ["u1"]


def test_materialise_refuses_what_the_operator_cannot_take(pkg, tmp_path):
    rp = pkg.replay
    from safetensors.torch import save_file
    W = _no_weights(pkg)
    save_file({"routing_logits": torch.zeros(4, 128), "bias32": torch.zeros(256)}, str(tmp_path / "t.safetensors"))
    st = lambda key: {"type": "safetensors", "path": "./t.safetensors", "tensor_key": key}
    bad = [
        rp.Workload("a", {"seq_len": 4}, {"routing_logits": st("routing_logits")}),                 # wrong shape
        rp.Workload("b", {"seq_len": 4}, {"routing_bias": st("bias32")}),                           # wrong dtype
        rp.Workload("c", {"seq_len": 4}, {"routing_logits": st("absent")}),                         # no such tensor
        rp.Workload("d", {"seq_len": 4}, {"routing_logits": {"type": "safetensors", "path": "./no.safetensors",
                                                                "tensor_key": "x"}}),              # no such file
        rp.Workload("e", {"seq_len": 4}, {"local_expert_offset": {"type": "scalar", "value": 40}}),  # not a shard boundary
        rp.Workload("f", {"seq_len": 4}, {"local_expert_offset": {"type": "random"}}),
        rp.Workload("g", {"seq_len": 4}, {"hidden_states": {"type": "scalar", "value": 1}}),
    ]
    for wl in bad:
        with pytest.raises(rp.TraceError):
            rp.materialise(wl, str(tmp_path), "cpu", weights=W)
    ok = rp.materialise(rp.Workload("h", {"seq_len": 4}, {"local_expert_offset": {"type": "scalar", "value": 224}}),
                        str(tmp_path), "cpu", weights=W)
    assert ok["local_expert_offset"] == 224


def test_aggregate_and_reference_cache(pkg, tmp_path):
    rp = pkg.replay
    per = [
        {"status": "PASSED", "speedup": 4.0, "max_abs_err": 0.5, "max_rel_err": 0.1},
        {"status": "PASSED", "speedup": 1.0, "max_abs_err": 0.25, "max_rel_err": 0.3},
        {"status": "PASSED", "speedup": 2.0, "max_abs_err": 0.0, "max_rel_err": 0.0},
        {"status": "PASSED"},
    ]
    a = rp.aggregate(per)
    assert a["correct"] and a["num_workloads"] == 4 and a["num_passed"] == 4
    assert a["mean_speedup"] == pytest.approx(7.0 / 3) and a["median_speedup"] == 2.0 and a["min_speedup"] == 1.0
    assert a["max_abs_err"] == 0.5 and a["max_rel_err"] == 0.3
    b = rp.aggregate(per + [{"status": "INCORRECT_NUMERICAL", "speedup": 9.0}])
    assert not b["correct"] and b["num_passed"] == 4 and b["median_speedup"] == 3.0
    assert rp.aggregate([], "no workloads")["correct"] is False
    cache = tmp_path / "ref.json"
    cache.write_text(json.dumps({"u1": {"ref_latency_ms": 3.5, "iters": 5}, "u2": {"ref_latency_ms": 0}, "u3": 7}))
    assert rp.load_ref_cache(str(cache)) == {"u1": 3.5}
    assert rp.load_ref_cache(str(tmp_path / "absent.json")) == {}
    (tmp_path / "broken.json").write_text("{")
    assert rp.load_ref_cache(str(tmp_path / "broken.json")) == {}


@pytest.mark.gpu
def test_replay_of_a_stand_in_set_against_the_oracle(pkg, tmp_path):
    import moe_oracle
    rp = pkg.replay
    seq_lens = [1, 7, 16, 0, 53, 130]
    wls = rp.write_synthetic_trace(str(tmp_path), seq_lens, seed=11)
    cache = tmp_path / "ref.json"
    cache.write_text(json.dumps({wls[0].uuid: {"ref_latency_ms": 1.0}}))
    res = rp.replay(str(tmp_path), device="cuda:0", warmup_runs=1, iterations=5, num_trials=2,
                    checker=moe_oracle.harness_check, ref_latency_ms=rp.load_ref_cache(str(cache)))
    assert res["num_workloads"] == len(seq_lens) and res["error"] is None
    assert res["correct"], [(p["axes"], p["status"], p.get("log")) for p in res["per_workload"]]
    for p, T in zip(res["per_workload"], seq_lens):
        assert p["axes"] == {"seq_len": T} and p["status"] == "PASSED"
        assert p["match_ratio"] >= 0.999 and p["max_abs_err"] >= 0.0
        if T:
            assert len(p["trial_latency_ms"]) == 2 and 0.0 < p["latency_ms"] < 50.0
    first = res["per_workload"][0]
    assert first["ref_latency_ms"] == 1.0 and first["speedup"] == pytest.approx(1.0 / first["latency_ms"])
    assert res["median_speedup"] == first["speedup"]
    # a workload that cannot be built is reported and the replay goes on
    with open(tmp_path / "workloads" / rp.OP_TYPE / (rp.DEFINITION + ".jsonl"), "a") as f:
        f.write(json.dumps({"definition": rp.DEFINITION,
                            "workload": {"uuid": "broken", "axes": {"seq_len": 4},
                                         "inputs": {"routing_logits": {"type": "safetensors", "path": "./no.safetensors",
                                                                       "tensor_key": "x"}}}}) + "\n")
    res2 = rp.replay(str(tmp_path), device="cuda:0", warmup_runs=1, iterations=2, num_trials=1, limit=0,
                     checker=moe_oracle.harness_check)
    assert not res2["correct"] and res2["num_passed"] == len(seq_lens)
    assert res2["per_workload"][-1]["status"] == "RUNTIME_ERROR" and "no.safetensors" in res2["per_workload"][-1]["log"]
