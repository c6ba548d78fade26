"""Replay of a flashinfer-trace workload set through the operator.

The reference measures its solution on the contest's trace set with the third-party package
flashinfer-bench (pinned at 0.1.2 in full-agent-pipeline/uv.lock; absent here): it loads the set with
``TraceSet.from_path``, builds every workload's inputs with ``gen_inputs`` / ``load_safetensors`` and
times the runnable (full-agent-pipeline/scripts/seed_ref_cache.py:44-81), or hands the set to
``Benchmark.run_all`` with warmup_runs = 3, iterations = 50, num_trials = 3, rtol = atol = 1e-2 and
reads per-workload status, latency, speed-up and errors back (full-agent-pipeline/run_pipeline.py:300-307,
401-450), aggregated by ``_aggregate`` (run_pipeline.py:364-399).

This module restates the part of that published layout the operator's path needs and drives
``op.run`` with it:

    <root>/definitions/<op_type>/<definition>.json     axes, inputs, outputs of the operator
    <root>/workloads/<op_type>/<definition>.jsonl      one trace object per line:
        {"definition": name, "workload": {"uuid": u, "axes": {"seq_len": T}, "inputs": {name: spec}},
         "solution": null, "evaluation": null}
    input specs: {"type": "random"} | {"type": "scalar", "value": v}
                 | {"type": "safetensors", "path": <relative to root>, "tensor_key": k}

Inputs of type "random" are drawn from this package's seeded generators (``gen``), keyed by the
workload's uuid, so that a replay is reproducible; the weights (1.4 GB of e4m3) are generated once and
shared by all workloads of a replay.  Correctness is judged by a checker the caller passes in (the
benchmark and the tests pass the oracle); without one a workload's status is "UNCHECKED".

``write_synthetic_trace`` writes a stand-in set in the same layout for machines without the data set.
"""
from __future__ import annotations

import glob
import hashlib
import json
import os
import uuid as uuid_mod
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional

import torch

from . import gen

DEFINITION = "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048"
OP_TYPE = "moe"
# positional order of the reference entry point (moe/solution/cuda/moe.cu:2650-2662)
INPUT_ORDER = ("routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
               "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset",
               "routed_scaling_factor")
TOKEN_INPUTS = INPUT_ORDER[:4]
WEIGHT_INPUTS = INPUT_ORDER[4:8]
SCALAR_DEFAULTS = {"local_expert_offset": 0, "routed_scaling_factor": 2.5}
# the harness's settings (run_pipeline.py:300-307)
BENCH_DEFAULTS = dict(warmup_runs=3, iterations=50, num_trials=3, rtol=1e-2, atol=1e-2)

H, I, E_GLOBAL, E_LOCAL, BLOCK = gen.H, gen.I, gen.E_GLOBAL, gen.E_LOCAL, gen.BLOCK


class TraceError(ValueError):
    """A trace file that does not describe a workload of this operator."""


@dataclass
class Workload:
    uuid: str
    axes: Dict[str, int]
    inputs: Dict[str, dict] = field(default_factory=dict)

    @property
    def seq_len(self) -> int:
        return int(self.axes["seq_len"])


def definition_dict() -> dict:
    """The operator's definition in the trace schema: axes, inputs, outputs (shapes by axis name)."""
    const = lambda v: {"type": "const", "value": v}
    t = lambda shape, dtype: {"shape": shape, "dtype": dtype}
    return {
        "name": DEFINITION,
        "op_type": OP_TYPE,
        "description": "FP8 block-scale MoE shard with DeepSeek-V3 routing (top-8 of 256 experts, 8 groups, "
                       "4 groups kept, 32 local experts, hidden 7168, intermediate 2048)",
        "axes": {"seq_len": {"type": "var"}, "num_experts": const(E_GLOBAL), "num_local_experts": const(E_LOCAL),
                 "hidden_size": const(H), "intermediate_size": const(I), "gemm1_out_size": const(2 * I),
                 "num_hidden_blocks": const(H // BLOCK), "num_intermediate_blocks": const(I // BLOCK),
                 "num_gemm1_out_blocks": const(2 * I // BLOCK)},
        "inputs": {
            "routing_logits": t(["seq_len", "num_experts"], "float32"),
            "routing_bias": t(["num_experts"], "bfloat16"),
            "hidden_states": t(["seq_len", "hidden_size"], "float8_e4m3fn"),
            "hidden_states_scale": t(["num_hidden_blocks", "seq_len"], "float32"),
            "gemm1_weights": t(["num_local_experts", "gemm1_out_size", "hidden_size"], "float8_e4m3fn"),
            "gemm1_weights_scale": t(["num_local_experts", "num_gemm1_out_blocks", "num_hidden_blocks"], "float32"),
            "gemm2_weights": t(["num_local_experts", "hidden_size", "intermediate_size"], "float8_e4m3fn"),
            "gemm2_weights_scale": t(["num_local_experts", "num_hidden_blocks", "num_intermediate_blocks"], "float32"),
            "local_expert_offset": t(None, "int32"),
            "routed_scaling_factor": t(None, "float32"),
        },
        "outputs": {"output": t(["seq_len", "hidden_size"], "bfloat16")},
        "reference": "full-agent-pipeline/references/moe.py (not embedded)",
    }


# ----------------------------------------------------------------------------- reading a trace set
def _workload_from(obj: dict, where: str) -> Workload:
    w = obj.get("workload", obj)
    if not isinstance(w, dict) or "uuid" not in w or "axes" not in w:
        raise TraceError(f"{where}: no workload with 'uuid' and 'axes'")
    axes = {k: int(v) for k, v in w["axes"].items()}
    if "seq_len" not in axes or axes["seq_len"] < 0:
        raise TraceError(f"{where}: workload {w['uuid']} has no usable 'seq_len' axis")
    inputs = w.get("inputs") or {}
    for name, spec in inputs.items():
        if name not in INPUT_ORDER:
            raise TraceError(f"{where}: workload {w['uuid']} names an unknown input '{name}'")
        kind = spec.get("type")
        if kind not in ("random", "scalar", "safetensors"):
            raise TraceError(f"{where}: input '{name}' has unknown type {kind!r}")
        if kind == "scalar" and "value" not in spec:
            raise TraceError(f"{where}: scalar input '{name}' has no value")
        if kind == "safetensors" and not ("path" in spec and "tensor_key" in spec):
            raise TraceError(f"{where}: safetensors input '{name}' needs 'path' and 'tensor_key'")
    return Workload(str(w["uuid"]), axes, dict(inputs))


def read_definition(root: str, definition: str = DEFINITION) -> Optional[dict]:
    """The definition file of the set, or None when the set carries none for this operator."""
    for path in sorted(glob.glob(os.path.join(root, "definitions", "**", definition + ".json"), recursive=True)):
        with open(path) as f:
            return json.load(f)
    return None


def read_workloads(root: str, definition: str = DEFINITION) -> List[Workload]:
    """Every workload of ``definition`` in the set, in file order (the order the harness runs them in)."""
    if not os.path.isdir(root):
        raise TraceError(f"trace set root does not exist: {root}")
    out: List[Workload] = []
    seen = set()
    for path in sorted(glob.glob(os.path.join(root, "workloads", "**", "*.jsonl"), recursive=True)):
        with open(path) as f:
            for n, line in enumerate(f, 1):
                line = line.strip()
                if not line:
                    continue
                try:
                    obj = json.loads(line)
                except json.JSONDecodeError as e:
                    raise TraceError(f"{path}:{n}: {e}") from None
                if obj.get("definition", definition) != definition:
                    continue
                wl = _workload_from(obj, f"{path}:{n}")
                if wl.uuid in seen:
                    raise TraceError(f"{path}:{n}: duplicate workload uuid {wl.uuid}")
                seen.add(wl.uuid)
                out.append(wl)
    return out


def load_ref_cache(path: str) -> Dict[str, float]:
    """{workload uuid: reference latency in ms} from a cache file in the layout of
    run_pipeline.py:319-330 ({uuid: {"ref_latency_ms": ms, ...}}); {} if the file is absent or unreadable."""
    if not path or not os.path.isfile(path):
        return {}
    try:
        with open(path) as f:
            raw = json.load(f)
    except json.JSONDecodeError:
        return {}
    return {k: float(v["ref_latency_ms"]) for k, v in raw.items() if isinstance(v, dict) and v.get("ref_latency_ms")}


# ----------------------------------------------------------------------------- building a workload's inputs
def uuid_seed(uuid: str) -> int:
    """Generator seed of a workload: 31 bits of the sha256 of its uuid."""
    return int.from_bytes(hashlib.sha256(uuid.encode()).digest()[:4], "little") & 0x7FFFFFFF


_DTYPES = {"routing_logits": torch.float32, "routing_bias": torch.bfloat16, "hidden_states": torch.float8_e4m3fn,
           "hidden_states_scale": torch.float32, "gemm1_weights": torch.float8_e4m3fn,
           "gemm1_weights_scale": torch.float32, "gemm2_weights": torch.float8_e4m3fn,
           "gemm2_weights_scale": torch.float32}


def expected_shape(name: str, T: int):
    return {"routing_logits": (T, E_GLOBAL), "routing_bias": (E_GLOBAL,), "hidden_states": (T, H),
            "hidden_states_scale": (H // BLOCK, T), "gemm1_weights": (E_LOCAL, 2 * I, H),
            "gemm1_weights_scale": (E_LOCAL, 2 * I // BLOCK, H // BLOCK), "gemm2_weights": (E_LOCAL, H, I),
            "gemm2_weights_scale": (E_LOCAL, H // BLOCK, I // BLOCK)}[name]


def _load_safetensors(root: str, spec: dict, cache: dict) -> torch.Tensor:
    path = os.path.normpath(os.path.join(root, spec["path"]))
    if path not in cache:
        try:
            from safetensors.torch import load_file
        except ImportError as e:      # the set needs a package this machine lacks: say so, do not guess values
            raise TraceError(f"workload input {spec['path']} needs the 'safetensors' package: {e}") from None
        if not os.path.isfile(path):
            raise TraceError(f"safetensors file missing: {path}")
        cache[path] = load_file(path)
    if spec["tensor_key"] not in cache[path]:
        raise TraceError(f"{path}: no tensor '{spec['tensor_key']}'")
    return cache[path][spec["tensor_key"]]


def materialise(wl: Workload, root: str, device, weights: Optional[gen.ShardWeights] = None,
                weight_seed: int = 0, _files: Optional[dict] = None) -> dict:
    """The ten inputs of the operator for one workload, by name, on ``device``.

    Token-side tensors the workload marks "random" (or leaves out) come from ``gen.make_tokens`` with the
    workload's uuid as seed; weights marked "random" are ``weights`` (generated with ``weight_seed`` when
    not given: pass them in to share one set across workloads).  Tensors stored in safetensors files are
    checked against the operator's shapes and dtypes, not converted."""
    files = {} if _files is None else _files
    T = wl.seq_len
    kind = lambda name: wl.inputs.get(name, {"type": "random"})["type"]
    out: dict = {}
    tok = None
    for name in TOKEN_INPUTS + WEIGHT_INPUTS:
        spec = wl.inputs.get(name, {"type": "random"})
        if spec["type"] == "safetensors":
            t = _load_safetensors(root, spec, files)
            if tuple(t.shape) != expected_shape(name, T) or t.dtype != _DTYPES[name]:
                raise TraceError(f"workload {wl.uuid}: '{name}' is {tuple(t.shape)} {t.dtype}, the operator takes "
                                 f"{expected_shape(name, T)} {_DTYPES[name]}")
            out[name] = t.to(device).contiguous()
        elif spec["type"] == "scalar":
            raise TraceError(f"workload {wl.uuid}: tensor input '{name}' given as a scalar")
        elif name in TOKEN_INPUTS:
            if tok is None:
                tok = gen.make_tokens(T, uuid_seed(wl.uuid), device)
            out[name] = getattr(tok, name)
        else:
            if weights is None:
                weights = gen.make_shard_weights(weight_seed, device)
            out[name] = getattr(weights, name)
    if kind("hidden_states") != kind("hidden_states_scale"):
        raise TraceError(f"workload {wl.uuid}: hidden_states and hidden_states_scale must come from the same source")
    for name, default in SCALAR_DEFAULTS.items():
        spec = wl.inputs.get(name)
        if spec is None:
            out[name] = default
        elif spec["type"] != "scalar":
            raise TraceError(f"workload {wl.uuid}: '{name}' must be a scalar input")
        else:
            out[name] = type(default)(spec["value"])
    if out["local_expert_offset"] % E_LOCAL != 0 or not 0 <= out["local_expert_offset"] <= E_GLOBAL - E_LOCAL:
        raise TraceError(f"workload {wl.uuid}: local_expert_offset {out['local_expert_offset']} is not a shard boundary")
    return out


# ----------------------------------------------------------------------------- running a set
def _median(xs):
    xs = sorted(xs)
    if not xs:
        return None
    n = len(xs)
    return xs[n // 2] if n % 2 else 0.5 * (xs[n // 2 - 1] + xs[n // 2])


def aggregate(per: List[dict], error: Optional[str] = None) -> dict:
    """Summary of a per-workload list with the fields of the reference's EvalResult
    (run_pipeline.py:364-399): the set is correct when every workload passed."""
    speedups = [p["speedup"] for p in per if p.get("speedup")]
    abs_errs = [p["max_abs_err"] for p in per if p.get("max_abs_err") is not None]
    rel_errs = [p["max_rel_err"] for p in per if p.get("max_rel_err") is not None]
    passed = sum(1 for p in per if p.get("status") == "PASSED")
    return {
        "correct": passed == len(per) and len(per) > 0,
        "num_workloads": len(per),
        "num_passed": passed,
        "mean_speedup": sum(speedups) / len(speedups) if speedups else None,
        "median_speedup": _median(speedups),
        "min_speedup": min(speedups) if speedups else None,
        "max_abs_err": max(abs_errs) if abs_errs else None,
        "max_rel_err": max(rel_errs) if rel_errs else None,
        "per_workload": per,
        "error": error,
    }


def time_workload(fn: Callable[[], None], device, warmup_runs: int, iterations: int, num_trials: int) -> List[float]:
    """Per-trial mean latency in ms of ``fn`` on the current stream of ``device``: ``warmup_runs`` untimed
    calls, then ``iterations`` calls between two CUDA events, ``num_trials`` times."""
    trials = []
    for _ in range(num_trials):
        for _ in range(warmup_runs):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        e0.record()
        for _ in range(iterations):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        trials.append(e0.elapsed_time(e1) / iterations)
    return trials


def replay(root: str, definition: str = DEFINITION, device="cuda:0", warmup_runs: int = BENCH_DEFAULTS["warmup_runs"],
           iterations: int = BENCH_DEFAULTS["iterations"], num_trials: int = BENCH_DEFAULTS["num_trials"],
           limit: int = 0, checker: Optional[Callable[[dict, torch.Tensor], dict]] = None,
           ref_latency_ms: Optional[Dict[str, float]] = None, weight_seed: int = 0,
           weights: Optional[gen.ShardWeights] = None) -> dict:
    """Run every workload of the set through ``op.run``; returns ``aggregate(...)`` of per-workload entries
    with the keys of run_pipeline.py:427-441 (workload, workload_uuid, status, latency_ms, ref_latency_ms,
    speedup, max_abs_err, max_rel_err) plus ``axes`` and the latency of every trial.

    ``checker(inputs, output)`` returns {"passed": bool, "max_abs_err": x, "max_rel_err": y, ...}; its other
    keys are copied into the entry.  ``ref_latency_ms`` maps workload uuids to the reference's latency
    (``load_ref_cache``); the speed-up is reference / ours, as the harness defines it.  A workload whose
    inputs cannot be built, or whose call fails, gets status "RUNTIME_ERROR" and the message, and the replay
    goes on with the next one."""
    from . import op      # needs the compiled library: fails loudly without it
    dev = torch.device(device)
    workloads = read_workloads(root, definition)
    if not workloads:
        return aggregate([], f"no workloads for {definition}")
    if limit:
        workloads = workloads[:limit]
    ref_latency_ms = ref_latency_ms or {}
    needs_weights = any(wl.inputs.get(n, {"type": "random"})["type"] == "random" for wl in workloads
                        for n in WEIGHT_INPUTS)
    if weights is None and needs_weights:
        weights = gen.make_shard_weights(weight_seed, dev)
    files: dict = {}
    per = []
    for wl in workloads:
        entry = {"workload": wl.uuid[:8], "workload_uuid": wl.uuid, "axes": dict(wl.axes), "status": None}
        try:
            inp = materialise(wl, root, dev, weights=weights, _files=files)
            args = [inp[n] for n in INPUT_ORDER]
            out = torch.empty((wl.seq_len, H), dtype=torch.bfloat16, device=dev)
            op.run(*args, out)
            torch.cuda.synchronize(dev)
            status = op.kernel_status(device=dev)
            if status != 0:
                raise RuntimeError(f"kernel status {status:#x}")
            if checker is None:
                entry["status"] = "UNCHECKED"
            else:
                verdict = dict(checker(inp, out))
                entry["status"] = "PASSED" if verdict.pop("passed") else "INCORRECT_NUMERICAL"
                entry.update(verdict)
            if wl.seq_len > 0:
                trials = time_workload(lambda: op.run(*args, out), dev, warmup_runs, iterations, num_trials)
                entry["trial_latency_ms"] = trials
                entry["latency_ms"] = sum(trials) / len(trials)
                ref_ms = ref_latency_ms.get(wl.uuid)
                if ref_ms:
                    entry["ref_latency_ms"] = ref_ms
                    entry["speedup"] = ref_ms / entry["latency_ms"]
        except (TraceError, RuntimeError, ValueError) as e:
            entry["status"] = "RUNTIME_ERROR"
            entry["log"] = f"{type(e).__name__}: {e}"[:400]
        per.append(entry)
    return aggregate(per)


# ----------------------------------------------------------------------------- a stand-in set
def write_synthetic_trace(root: str, seq_lens: Iterable[int], seed: int = 0, stored_routing: bool = True,
                          local_expert_offset: int = 0, routed_scaling_factor: float = 2.5) -> List[Workload]:
    """Write a trace set for this operator under ``root`` in the layout this module reads: the definition
    file, one workload per entry of ``seq_lens`` and, with ``stored_routing``, the routing logits and bias
    of every workload in a safetensors file (the way a recorded set carries the tensors whose values
    matter); everything else is left "random".  Uuids derive from (seed, position, seq_len)."""
    os.makedirs(os.path.join(root, "definitions", OP_TYPE), exist_ok=True)
    os.makedirs(os.path.join(root, "workloads", OP_TYPE), exist_ok=True)
    with open(os.path.join(root, "definitions", OP_TYPE, DEFINITION + ".json"), "w") as f:
        json.dump(definition_dict(), f, indent=2)
    if stored_routing:
        from safetensors.torch import save_file
        blob_dir = os.path.join(root, "blob", "workloads", OP_TYPE, DEFINITION)
        os.makedirs(blob_dir, exist_ok=True)
    out = []
    with open(os.path.join(root, "workloads", OP_TYPE, DEFINITION + ".jsonl"), "w") as f:
        for i, T in enumerate(seq_lens):
            u = str(uuid_mod.uuid5(uuid_mod.NAMESPACE_OID, f"{DEFINITION}/{seed}/{i}/{int(T)}"))
            inputs = {n: {"type": "random"} for n in TOKEN_INPUTS + WEIGHT_INPUTS}
            inputs["local_expert_offset"] = {"type": "scalar", "value": int(local_expert_offset)}
            inputs["routed_scaling_factor"] = {"type": "scalar", "value": float(routed_scaling_factor)}
            if stored_routing:
                tok = gen.make_tokens(int(T), uuid_seed(u) ^ 0x5A5A5A5, "cpu")
                rel = os.path.join("blob", "workloads", OP_TYPE, DEFINITION, u + ".safetensors")
                save_file({"routing_logits": tok.routing_logits, "routing_bias": tok.routing_bias},
                          os.path.join(root, rel))
                for n in ("routing_logits", "routing_bias"):
                    inputs[n] = {"type": "safetensors", "path": "./" + rel, "tensor_key": n}
            wl = Workload(u, {"seq_len": int(T)}, inputs)
            f.write(json.dumps({"definition": DEFINITION, "solution": None,
                                "workload": {"uuid": wl.uuid, "axes": wl.axes, "inputs": wl.inputs},
                                "evaluation": None}) + "\n")
            out.append(wl)
    return out
