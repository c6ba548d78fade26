#!/usr/bin/env python
"""Benchmark of the FP8 block-scale DeepSeek-V3 MoE shard on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one call of the operator on one batch of seeded synthetic tokens.
N = 1 measures the decode workload (T = 1, the configuration the headline metric
is quoted on); N > 1 (under torchrun) measures the 256-expert layer with expert
parallelism over N GPUs (T = 16384 tokens, NCCL all-to-all dispatch and combine).
Rank 0 prints ONE JSON line.

Timing: CUDA events on the launching stream around the K timed steps (W warm-up
steps before), max over ranks.  A decode step touches < 126 MB of weights, so
consecutive steps rotate through R replicas of the shard's weights (different
addresses, same values) chosen so that a replica is reused only after more
than 3x the L2 capacity has been streamed: every step reads its weights from HBM
("inputs larger than L2"), without a flush kernel leaving dirty lines behind.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from __graft_entry__ import load_package  # noqa: E402

METRIC = "moe_tokens_per_second"
UNIT = "tokens/s"
RSF = 2.5

# single-GPU workloads (BASELINE.json configs 1, 0, 2, 3 and two sizes in between)
WORKLOADS = {
    "decode_t1":     dict(T=1, token_seed=3, skew=False),    # seed 3: first seed whose token has a local expert
    "cpu_ref_t8":    dict(T=8, token_seed=0, skew=False),
    "small_t16":     dict(T=16, token_seed=0, skew=False),
    "skew_t64":      dict(T=64, token_seed=0, skew=True),
    "mid_t512":      dict(T=512, token_seed=0, skew=False),
    "prefill_t4096": dict(T=4096, token_seed=0, skew=False),
}

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu capture
# summarised in profiles/ (None until a capture of that workload exists).
NCU_TRAFFIC_BYTES = {"decode_t1": 88_237_568 + 2_996_224,     # profiles/decode_kernel_t1.md
                     "skew_t64": 473_900_000 + 12_800_000,     # profiles/launch_shares_skew_t64_prefill_t4096.md
                     "prefill_t4096": 807_600_000 + 67_100_000}

W13_BYTES = 4096 * 7168 + 32 * 56 * 4          # one expert's GEMM1 weights + scales
W2_BYTES = 7168 * 2048 + 56 * 16 * 4
ROW_BYTES = 7168 + 56 * 4                      # one activation row + its scales


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def algorithmic_bytes(T, n_sel, n_active, n_tokens_with_local):
    """Bytes the operator must move: active experts' weights and scales, the
    activation rows it reads once, the routing logits and the bf16 output."""
    return (n_active * (W13_BYTES + W2_BYTES) + n_tokens_with_local * ROW_BYTES + T * 1024 + T * 7168 * 2)


def time_steps(fn, steps, warmup):
    """W warm-up calls, then exactly K calls between two events; returns ms per step."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


L2_BYTES = 126 << 20


def weight_replicas(W, touched_bytes):
    """Enough copies of the shard's weights that a copy is reused after > 3 x L2 of other traffic."""
    n = 1
    while n < 8 and touched_bytes * (n - 1) < 3 * L2_BYTES:
        n += 1
    reps = [W]
    for _ in range(n - 1):
        reps.append(type(W)(W.gemm1_weights.clone(), W.gemm1_weights_scale.clone(), W.gemm2_weights.clone(),
                            W.gemm2_weights_scale.clone()))
    return reps


def wtuple(w):
    return (w.gemm1_weights, w.gemm1_weights_scale, w.gemm2_weights, w.gemm2_weights_scale)


def bench_single(args):
    pkg = load_package()
    gen, op, loader = pkg.gen, pkg.op, pkg.loader
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    name = args.workload or "decode_t1"
    wl = WORKLOADS[name]
    T = wl["T"]
    W = gen.make_shard_weights(0, dev)
    tok = gen.make_tokens(T, wl["token_seed"], dev, wl["skew"])
    out = torch.empty(T, 7168, dtype=torch.bfloat16, device=dev)
    wargs = wtuple(W)
    # one untimed call tells how many experts the batch touches, which sizes the replica ring
    op.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale, *wargs, 0, RSF, out)
    sched = op.intermediates(T)["sched"]
    reps = weight_replicas(W, max(1, sched.n_active) * (W13_BYTES + W2_BYTES))
    R = len(reps)

    def step(i=0):
        op.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
               *wtuple(reps[i % R]), 0, RSF, out)

    # ---- device-resident inputs: `value`
    launches0 = loader.launch_count()
    with ClockSampler(0) as clocks:
        ms_step = time_steps(step, args.steps, args.warmup)
    launches = (loader.launch_count() - launches0) * args.steps // (args.steps + args.warmup)
    assert op.kernel_status() == 0
    im = op.intermediates(T)
    sched = im["sched"]
    value = T / (ms_step * 1e-3)

    # ---- host buffers through the host entry point: `e2e`
    pin = lambda t: t.cpu().pin_memory()
    h = [pin(tok.routing_logits), pin(tok.routing_bias), pin(tok.hidden_states), pin(tok.hidden_states_scale)]
    out_h = torch.empty(T, 7168, dtype=torch.bfloat16).pin_memory()

    def step_host(i=0):
        op.run_host(*h, *wtuple(reps[i % R]), 0, RSF, out_h)

    ms_host = time_steps(step_host, args.steps, args.warmup)
    e2e_value = T / (ms_host * 1e-3)
    h2d = sum(t.numel() * t.element_size() for t in h)
    d2h = out_h.numel() * out_h.element_size()

    # ---- per-kernel durations (events between the stages) for the roofline of the dominant kernel
    loader.set_profiling(True)
    acc = {}
    nprof = max(10, min(args.steps, 100))
    for i in range(nprof + 3):
        step(i)
        st = loader.stage_times_ms()
        if i >= 3:
            for k, v in st.items():
                acc[k] = acc.get(k, 0.0) + v
    loader.set_profiling(False)
    stage_us = {k: v / nprof * 1e3 for k, v in acc.items()}
    fused = T <= 16
    n_local_tokens = int((im["local_mask"] != 0).sum())
    op_bytes = algorithmic_bytes(T, sched.n_sel, sched.n_active, n_local_tokens)
    peak, peak_kind = measured_peaks()
    if fused:
        # one launch per step: the kernel's average launch duration is the timed region / K
        dominant, kernel_bytes, launch_us = "decode", op_bytes, ms_step * 1e3
        kernel_name = "decode_kernel: routing + GEMM1 + SwiGLU + GEMM2 + combine in one launch"
    else:
        dominant = max(("gemm1", "gemm2"), key=lambda k: stage_us[k])
        wbytes = W13_BYTES if dominant == "gemm1" else W2_BYTES
        rbytes = ROW_BYTES if dominant == "gemm1" else 0
        kernel_bytes, launch_us = sched.n_active * wbytes + sched.n_sel * rbytes, stage_us[dominant]
        kernel_name = f"grouped_gemm_kernel<{1 if dominant == 'gemm1' else 2},{sched.n_tile}>"
    achieved = kernel_bytes / (launch_us * 1e-6) / 1e9
    step(0)       # leave `out` holding replica 0's result for the self-check below
    torch.cuda.synchronize()

    # ---- self-check against the oracle and the CPU baseline (bounded sample of the same workload)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import moe_oracle
    cpu_tok = [t.cpu() for t in (tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale)]
    active = [le for le in range(32) if sched.counts[le] > 0]
    cpu_w = {le: tuple(x[le].cpu() for x in wargs) for le in active}
    t0 = time.time()
    calls = 0
    while True:
        ref = moe_oracle.run(*cpu_tok, lambda le: cpu_w[le], 0, RSF)
        calls += 1
        if time.time() - t0 > 10.0 or calls >= 50:
            break
    cpu_s = time.time() - t0
    m = moe_oracle.output_metrics(out, ref.output, ref.output_f32)
    assert m["cosine"] >= 0.9999, m

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": name, "T": T, "token_seed": wl["token_seed"], "weight_seed": 0,
                   "routing_skew": wl["skew"], "local_expert_offset": 0, "n_sel": sched.n_sel,
                   "active_experts": sched.n_active,
                   "l2": f"{R} weight replicas rotated: {R * sched.n_active * (W13_BYTES + W2_BYTES) >> 20} MiB "
                         "streamed per cycle > 3 x 126 MB L2",
                   "split_k": [sched.split1, sched.split2], "token_tile": sched.n_tile},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_host,
                "note": "token tensors from pinned host memory, bf16 output read back; weights stay resident"},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm",
                     "kernel": kernel_name,
                     "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(name),
                     "algorithmic_bytes_per_launch": kernel_bytes, "launch_us": launch_us,
                     "whole_op": {"algorithmic_bytes": op_bytes, "achieved": op_bytes / (ms_step * 1e-3) / 1e9,
                                  "frac": op_bytes / (ms_step * 1e-3) / 1e9 / peak}},
        "stage_us": stage_us,
        "cpu_baseline": {"value": calls * T / cpu_s, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{calls} calls of the oracle port on the same T={T} batch ({cpu_s:.1f} s); "
                                   "only the experts the batch uses are dequantised"},
        "parity": {k: m[k] for k in ("max_abs_over_rms", "cosine", "n_diff", "n_one_step")},
    }
    if args.sweep:
        line["sweep"] = sweep(pkg, W, [n for n in WORKLOADS if n != name], peak)
        del W, reps
        torch.cuda.empty_cache()
        line["ep_layer_single_gpu"] = ep_single_gpu(pkg, dev)
    print(json.dumps(line))


def sweep(pkg, W, names, peak):
    """Tokens/s and per-kernel roofline fractions of the other single-GPU workloads."""
    gen, op, loader = pkg.gen, pkg.op, pkg.loader
    dev = W.gemm1_weights.device
    rows = []
    for name in names:
        wl = WORKLOADS[name]
        T = wl["T"]
        tok = gen.make_tokens(T, wl["token_seed"], dev, wl["skew"])
        out = torch.empty(T, 7168, dtype=torch.bfloat16, device=dev)
        op.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale, *wtuple(W), 0, RSF, out)
        s = op.intermediates(T)["sched"]
        reps = weight_replicas(W, max(1, s.n_active) * (W13_BYTES + W2_BYTES))
        R = len(reps)

        def step(i=0):
            op.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                   *wtuple(reps[i % R]), 0, RSF, out)
        ms = time_steps(step, 30, 5)
        loader.set_profiling(True)
        acc = {}
        for i in range(10):
            step(i)
            for k, v in loader.stage_times_ms().items():
                acc[k] = acc.get(k, 0.0) + v * 100.0
        loader.set_profiling(False)
        us = ms * 1e3
        rows.append({"workload": name, "T": T, "n_sel": s.n_sel, "active_experts": s.n_active, "replicas": R,
                     "us_per_step": us, "tokens_per_s": T / us * 1e6,
                     # T <= 16 is one launch: no per-GEMM split
                     "gemm1_gbs": None if T <= 16 else (s.n_active * W13_BYTES + s.n_sel * ROW_BYTES) / acc["gemm1"] / 1e3,
                     "gemm2_gbs": None if T <= 16 else s.n_active * W2_BYTES / acc["gemm2"] / 1e3,
                     "whole_op_hbm_frac": s.n_active * (W13_BYTES + W2_BYTES) / us / 1e3 / peak,
                     "fp8_tflops": s.n_sel * 88080384 / us / 1e6,
                     "stage_us": acc})
        del reps
    return rows


def ep_single_gpu(pkg, dev, steps=3):
    """The 256-expert layer of the multi-GPU workload (T = 16384) on ONE GPU: eight shard calls
    per layer call, no communication.  The N = 1 point of the expert-parallel scaling curve."""
    gen, ep = pkg.gen, pkg.ep
    T = 16384
    weights = [gen.make_shard_weights(1000 + s, dev) for s in range(8)]
    tok = gen.make_tokens(T, 0, dev)
    layer = ep.ExpertParallelMoE(weights, 0, 1)

    def step(i=0):
        return layer.forward(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale, RSF)
    ms = time_steps(step, steps, 2)
    return {"workload": "ep_layer_t16384", "n_gpus": 1, "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3),
            "records": int(sum(layer.last_plan.recv_counts))}


def bench_reference(args):
    """The definition's CPU path on the host cores, same metric and config: the oracle
    port (the reference itself is a Python file that is not present on the GPU box).
    Inputs are generated on the CPU for the experts the batch uses; no GPU is touched."""
    pkg = load_package()
    gen = pkg.gen
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import moe_oracle
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload or "decode_t1"
    wl = WORKLOADS[name]
    T = wl["T"]
    tok = gen.make_tokens(T, wl["token_seed"], "cpu", wl["skew"])
    lazy = gen.LazyShardWeights(0, "cpu")
    cpu_tok = (tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale)
    steps, warmup = min(args.steps, 20), min(args.warmup, 3)
    for _ in range(max(1, warmup)):          # also generates the active experts' weights
        moe_oracle.run(*cpu_tok, lazy.expert, 0, RSF)
    t0 = time.time()
    for _ in range(steps):
        ref = moe_oracle.run(*cpu_tok, lazy.expert, 0, RSF)
    dt = time.time() - t0
    value = steps * T / dt
    base = {"kind": "port", "cores": torch.get_num_threads(), "value": value, "unit": UNIT,
            "sample": f"{steps} calls of the oracle port on the T={T} batch ({dt:.1f} s)"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "T": T, "token_seed": wl["token_seed"], "weight_seed": 0,
                   "routing_skew": wl["skew"], "local_expert_offset": 0, "n_sel": int(ref.counts.sum()),
                   "active_experts": int((ref.counts > 0).sum())},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-sweep", dest="sweep", action="store_false")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return bench_reference(args)
    if args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        pkg = load_package()
        return pkg.ep.bench_main(args)
    return bench_single(args)


if __name__ == "__main__":
    main()
